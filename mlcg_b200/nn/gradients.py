"""Energy -> force wrappers with mlcg's names and output layout (src/mlcg/nn/gradients.py)."""
from typing import Any, List, Sequence

import torch

from ..data import ENERGY_KEY, FORCE_KEY


class GradientsOut(torch.nn.Module):
    """forces = -d(sum of energies)/d(pos); the graph of that derivative is kept in training mode so the
    force loss can be differentiated again (gradients.py:191-230)."""

    _targets = {FORCE_KEY: ENERGY_KEY}

    def __init__(self, model: torch.nn.Module, targets: str = FORCE_KEY):
        super().__init__()
        self.model = model
        self.name = self.model.name
        self.targets = [targets] if isinstance(targets, str) else list(targets) if isinstance(targets, Sequence) else []
        assert any(k in GradientsOut._targets for k in self.targets), f"targets={self.targets} should be any of {GradientsOut._targets}"

    def forward(self, data):
        # eval mode: models that can hand out the energy together with its position gradient are evaluated without an
        # autograd graph (same numbers; create_graph is False in eval mode anyway, gradients.py:191-230)
        direct = getattr(self.model, "energy_and_gradient", None)
        if direct is not None and not self.training and FORCE_KEY in self.targets and self.name != "SumOut":
            res = direct(data)
            if res is not None:
                energy, dy_dr = res
                data.out[self.name] = {ENERGY_KEY: energy, FORCE_KEY: -dy_dr}
                data.pos = data.pos.detach()
                return data
        data.pos.requires_grad_(True)
        data = self.model(data)
        if FORCE_KEY in self.targets:
            y = data.out[ENERGY_KEY] if self.name == "SumOut" else data.out[self.name][ENERGY_KEY]
            dy_dr = torch.autograd.grad(y.sum(), data.pos, create_graph=self.training)[0]
            if self.name == "SumOut":
                data.out[FORCE_KEY] = -dy_dr
            else:
                data.out[self.name][FORCE_KEY] = -dy_dr
        data.pos = data.pos.detach()
        return data

    def neighbor_list(self, **kwargs: Any):
        return self.model.neighbor_list(**kwargs)


class SumOut(torch.nn.Module):
    """Runs each component model and adds up the targets (gradients.py:59-117)."""

    name: str = "SumOut"

    def __init__(self, models: torch.nn.ModuleDict, targets: List[str] = None):
        super().__init__()
        self.targets = [ENERGY_KEY, FORCE_KEY] if targets is None else targets
        self.models = models

    def forward(self, data):
        for target in self.targets:
            data.out[target] = 0.00
        together = self._priors_together(data)
        for name in self.models.keys():
            if name in together:
                energy, dy_dr = together[name]
                data.out[self.models[name].name] = {ENERGY_KEY: energy, FORCE_KEY: -dy_dr}
            else:
                data = self.models[name](data)
            for target in self.targets:
                data.out[target] += data.out[name][target]
        return data

    def _priors_together(self, data):
        """Eval mode: every prior component that is wrapped for forces is evaluated in one launch with the others
        (:func:`mlcg_b200.nn.prior.evaluate_priors`); the results are handed out component by component in ``forward``."""
        from .prior import _Prior, evaluate_priors
        if self.training:
            return {}
        picked = {name: m.model for name, m in self.models.items()
                  if isinstance(m, GradientsOut) and isinstance(m.model, _Prior) and not m.training and FORCE_KEY in m.targets and m.name == name}
        if len(picked) < 2:
            return {}
        res = evaluate_priors(picked.values(), data)
        if res is None:
            return {}
        data.pos = data.pos.detach()
        return {name: res[p.name] for name, p in picked.items()}

    def neighbor_list(self, **kwargs):
        nl = {}
        for _, model in self.models.items():
            nl.update(**model.neighbor_list(**kwargs))
        return nl


class EnergyOut(torch.nn.Module):
    """Copies a model's energy to the top level of ``data.out`` (gradients.py:126-156)."""

    name: str = "EnergyOut"

    def __init__(self, model: torch.nn.Module, targets: List[str] = None):
        super().__init__()
        self.targets = [ENERGY_KEY] if targets is None else targets
        self.model = model
        self.name = self.model.name

    def forward(self, data):
        data = self.model(data)
        for target in self.targets:
            data.out[target] = data.out[self.name][target]
        return data
