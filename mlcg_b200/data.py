"""Minimal stand-in for ``mlcg.data.AtomicData`` (src/mlcg/data/atomic_data.py:21-103).

mlcg's container derives from ``torch_geometric.data.Data``; the hot path only reads attributes
(``pos``, ``atom_types``, ``batch``, ``n_atoms``, ``neighbor_list``) and writes ``out``.  The modules of
this package accept either mlcg's ``AtomicData`` or this class; it exists so that the package can be
exercised where torch_geometric is not installed.
"""
from typing import Any, Dict

import torch

ENERGY_KEY = "energy"
FORCE_KEY = "forces"


class AtomicData:
    def __init__(self, pos: torch.Tensor, atom_types: torch.Tensor, batch: torch.Tensor = None, n_atoms: torch.Tensor = None,
                 neighbor_list: Dict[str, Dict[str, Any]] = None, **extra):
        assert pos.dim() == 2 and pos.shape[1] == 3
        if n_atoms is not None and not n_atoms.is_cuda:      # (no device->host read for a count that lives on the device)
            assert int(torch.sum(n_atoms)) == pos.shape[0]
        self.pos = pos
        self.atom_types = atom_types
        self.batch = batch if batch is not None else torch.zeros(pos.shape[0], dtype=torch.long, device=pos.device)
        self.n_atoms = n_atoms
        self.neighbor_list = {} if neighbor_list is None else neighbor_list
        self.out = {}
        for k, v in extra.items():
            setattr(self, k, v)

    def __contains__(self, key):
        return getattr(self, key, None) is not None

    def __getitem__(self, key):
        return getattr(self, key)

    def __setitem__(self, key, value):
        setattr(self, key, value)

    def to(self, device):
        def mv(v):
            if torch.is_tensor(v):
                return v.to(device)
            if isinstance(v, dict):
                return {k: mv(x) for k, x in v.items()}
            return v

        for k, v in list(self.__dict__.items()):
            setattr(self, k, mv(v))
        return self

    @property
    def num_structures(self):
        return None if self.n_atoms is None else int(self.n_atoms.numel())


def collate(data_list):
    """Structures -> one batch, the way torch_geometric collates mlcg's ``AtomicData`` (src/mlcg/data/atomic_data.py,
    src/mlcg/simulation/base.py:621-626): positions and types concatenated, ``batch`` numbered in list order, every
    neighbour list's ``index_mapping`` shifted by the structure's first node and concatenated, ``mapping_batch`` filled in."""
    pos = torch.cat([d.pos for d in data_list])
    types = torch.cat([d.atom_types for d in data_list])
    sizes = [d.pos.shape[0] for d in data_list]
    dev = pos.device
    batch = torch.repeat_interleave(torch.arange(len(data_list), device=dev), torch.tensor(sizes, device=dev))
    first = [0]
    for n in sizes[:-1]:
        first.append(first[-1] + n)
    nls = {}
    for tag in data_list[0].neighbor_list:
        parts = [d.neighbor_list[tag] for d in data_list]
        im = torch.cat([p["index_mapping"] + off for p, off in zip(parts, first)], dim=1)
        mb = torch.cat([torch.full((p["index_mapping"].shape[1],), b, dtype=torch.long, device=dev) for b, p in enumerate(parts)])
        shifts = None if parts[0].get("cell_shifts") is None else torch.cat([p["cell_shifts"] for p in parts])
        nls[tag] = dict(tag=parts[0]["tag"], order=parts[0]["order"], index_mapping=im, cell_shifts=shifts, rcut=parts[0].get("rcut"),
                        self_interaction=parts[0].get("self_interaction"), mapping_batch=mb)
    return AtomicData(pos=pos, atom_types=types, batch=batch, n_atoms=torch.tensor(sizes, device=dev), neighbor_list=nls)
