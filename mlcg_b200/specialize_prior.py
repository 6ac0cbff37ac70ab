"""Priors specialised to one set of structures (src/mlcg/simulation/specialize_prior.py:37-206).

A simulation usually carries several priors of one functional form (bonds between different bead groups, several
angle or dihedral families).  ``condense_all_priors_for_simulation`` merges all priors of one class into a single
``Static…`` prior: the per-term parameters are gathered once from the type tables into flat buffers, in the order of the
concatenated index mappings, and the structures' neighbour lists are rewritten to hold one entry per class.  The flat
buffers are exactly the ``[P, M]`` parameter rows the prior kernel (``mlcgb_prior_terms``) reads, so a merged class costs one
launch per evaluation however many priors went into it.
"""
from collections import defaultdict
from copy import deepcopy
from typing import Dict, List, Tuple, Type

import torch

from .data import AtomicData
from .neighbor_list import make_neighbor_list
from .nn.gradients import GradientsOut, SumOut
from .nn.prior import Dihedral, GeneralAngles, GeneralBonds, HarmonicAngles, HarmonicBonds, _Prior

#: prior classes that can be merged, in the reference's order (it also lists its improper variant, which this package does
#: not define)
to_reduce: Dict[str, Type[_Prior]] = {"Dihedral": Dihedral, "GeneralAngles": GeneralAngles, "GeneralBonds": GeneralBonds,
                                      "HarmonicBonds": HarmonicBonds, "HarmonicAngles": HarmonicAngles}


class StaticPrior(torch.nn.Module):
    """Holds the gathered per-term parameters as buffers; ``data2parameters`` hands them back for any data
    (specialize_prior.py:49-59)."""

    def __init__(self, **params):
        torch.nn.Module.__init__(self)
        self.param_names = []
        for k, v in params.items():
            self.register_buffer(k, v)
            self.param_names.append(k)

    def data2parameters(self, data):
        return {k: getattr(self, k) for k in self.param_names}


def _make_static(cls_name: str, CLS: Type[_Prior]):
    def constructor(self, **params):
        StaticPrior.__init__(self, **params)
        self.order = CLS._order
        if issubclass(CLS, Dihedral):
            self.n_degs = int(params["k1s"].shape[1])

    return type(f"Static{cls_name}", (StaticPrior, CLS), {"__init__": constructor, "name": CLS.name})


for _name, _CLS in to_reduce.items():
    globals()[f"Static{_name}"] = _make_static(_name, _CLS)


def condense_all_priors_for_simulation(priors: SumOut, data_list: List[AtomicData]) -> Tuple[SumOut, List[AtomicData]]:
    """specialize_prior.py:75-109: merge, class by class, every prior whose class is in :data:`to_reduce`.  The result is
    valid for a collated batch of the returned structures (same order)."""
    for TargetPrior in to_reduce.values():
        priors, data_list = condense_prior_for_simulation(TargetPrior, priors, data_list)
    return priors, data_list


def condense_prior_for_simulation(TargetPrior: Type[_Prior], priors: SumOut, data_list: List[AtomicData]) -> Tuple[SumOut, List[AtomicData]]:
    """specialize_prior.py:112-206."""
    static_name = None
    for k, CLS in to_reduce.items():
        if CLS is TargetPrior:
            static_name = f"Static{k}"
    if static_name is None:
        raise RuntimeError(f"The condense target {TargetPrior} has not been registered in {to_reduce}")
    StaticCLS = globals()[static_name]

    def is_target(wrapped) -> bool:
        return isinstance(wrapped.model, TargetPrior) and not isinstance(wrapped.model, StaticPrior)

    targets = [k for k, wrapped in priors.models.items() if is_target(wrapped)]
    condensed_priors = deepcopy(priors)
    condensed_data_list = deepcopy(data_list)
    if not targets:
        return condensed_priors, condensed_data_list
    for k in targets:
        condensed_priors.models.pop(k)
    n_degs = max([priors.models[k].model.n_degs for k in targets] if TargetPrior is Dihedral else [1])

    params = defaultdict(list)
    for ii, data in enumerate(data_list):
        index_mapping = []
        for k in targets:
            pp = priors.models[k].model.data2parameters(data)
            for kv, v in pp.items():
                if v.ndim == 1:
                    v = v.unsqueeze(-1)
                padded = torch.zeros((v.shape[0], n_degs), dtype=v.dtype, device=v.device)   # shorter Fourier series: zero coefficients
                padded[:, : v.shape[1]] = v
                params[kv].append(padded)
            index_mapping.append(data.neighbor_list[k]["index_mapping"])
            condensed_data_list[ii].neighbor_list.pop(k)
        condensed_data_list[ii].neighbor_list[StaticCLS.name] = make_neighbor_list(
            tag=static_name, order=TargetPrior._order, index_mapping=torch.cat(index_mapping, dim=-1))

    merged = {k: (torch.vstack(v) if TargetPrior is Dihedral else torch.cat(v).flatten()) for k, v in params.items()}
    condensed_priors.models[StaticCLS.name] = GradientsOut(StaticCLS(**merged))
    return condensed_priors, condensed_data_list
