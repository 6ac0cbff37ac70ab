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
        if n_atoms is not None:
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
