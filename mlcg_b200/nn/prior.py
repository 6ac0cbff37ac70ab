"""Prior energy terms with mlcg's class names, constructor arguments and buffers
(src/mlcg/nn/prior/harmonic.py, repulsion.py, fourier_series.py, base.py).

``forward(data)`` evaluates one fused kernel per prior that returns the per-structure energies and keeps
dE/dpos for the backward pass, so ``GradientsOut`` gets forces from a single multiply.  In training
mode (``create_graph=True`` upstream) the same terms are evaluated with differentiable torch
operations, because the analytic-gradient kernel carries no second derivative.
"""
from typing import Dict, Final

import torch

from ..backend import get_backend

KIND_BOND, KIND_ANGLE, KIND_DIHEDRAL, KIND_REPULSION = 0, 1, 2, 3

#: Energies and forces of the priors evaluated together (:func:`evaluate_priors`) are summed as 64-bit fixed-point integers, so they
#: are bit-identical from run to run; ``set_prior_determinism(False)`` sums with floating-point atomics instead.
_DETERMINISTIC = True


def set_prior_determinism(on: bool) -> None:
    global _DETERMINISTIC
    _DETERMINISTIC = bool(on)


class _PriorEnergy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pos, kind, mapping, mapping_batch, params, batch, B):
        energy, grad = get_backend().prior_terms(kind, pos, mapping, mapping_batch, params, B, want_grad=True)
        ctx.save_for_backward(grad, batch)
        return energy

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        grad, batch = ctx.saved_tensors
        return g.index_select(0, batch).unsqueeze(-1) * grad, None, None, None, None, None, None


def _batch_or_zeros(data):
    batch = getattr(data, "batch", None)
    return torch.zeros(data.pos.shape[0], dtype=torch.long, device=data.pos.device) if batch is None else batch


def _num_structures(data) -> int:
    n_atoms = getattr(data, "n_atoms", None)
    if n_atoms is not None and torch.is_tensor(n_atoms) and n_atoms.dim() == 1:
        return int(n_atoms.numel())
    batch = getattr(data, "batch", None)
    return 1 if batch is None else int(batch[-1]) + 1


def _table_from_statistics(statistics: Dict, order: int, field: str) -> torch.Tensor:
    keys = torch.tensor(list(statistics.keys()), dtype=torch.long)
    types = torch.unique(keys.flatten())
    assert types.min() >= 0
    table = torch.zeros(tuple([int(types.max()) + 1] * order))
    for key, val in statistics.items():
        table[key] = val[field]
    return table


def compute_cell_shifts(pos, mapping, pbc, cell, batch):
    """Minimum-image shifts of the points 1.. of every term relative to its point 0, ``[M, 3, order-1]`` in length units
    (base.py:5-62, restated with its conventions: the fractional displacement is ``inv(cell) @ (pos[m0] - pos[mk])``, the
    shift ``cell @ floor(frac + 0.5)``, zeroed along non-periodic directions; constants with respect to differentiation)."""
    with torch.no_grad():
        M, order = mapping.shape[1], mapping.shape[0]
        shifts = torch.zeros(M, 3, order - 1, dtype=pos.dtype, device=pos.device)
        if batch is None:
            batch = torch.zeros(pos.shape[0], dtype=torch.long, device=pos.device)
        ids = batch[mapping[0]]
        cells = cell.view(-1, 3, 3)[ids].to(pos.dtype)
        cell_inv = torch.linalg.inv(cells)
        periodic = pbc.view(-1, 3)[ids].to(pos.dtype)
        for k in range(order - 1):
            drs = pos[mapping[0]] - pos[mapping[k + 1]]
            n = torch.floor(torch.einsum("bij,bj->bi", cell_inv, drs) + 0.5)
            shifts[:, :, k] = periodic * torch.einsum("bij,bj->bi", cells, n)
    return shifts


def _data_cell_shifts(data, mapping):
    """The shifts of a prior's terms when the data carry ``pbc`` and ``cell`` (harmonic.py:214-242), else None."""
    pbc, cell = getattr(data, "pbc", None), getattr(data, "cell", None)
    if pbc is None or cell is None:
        return None
    return compute_cell_shifts(data.pos.detach(), mapping, pbc.to(data.pos.device), cell.to(data.pos.device), getattr(data, "batch", None))


def _feature_shifts(pos, mapping, pbc, cell, batch):
    return None if pbc is None or cell is None else compute_cell_shifts(pos.detach(), mapping, pbc, cell, batch)


def _shifted(pos, m, shifts):
    """Positions of the points of every term, point k >= 1 moved by its shift (internal_coordinates.py:95-99, 168-177, 233-244)."""
    pts = [pos[m[k]] for k in range(m.shape[0])]
    if shifts is not None:
        pts = [pts[0]] + [pts[k] + shifts[:, :, k - 1] for k in range(1, len(pts))]
    return pts


# differentiable torch restatements of the features: used when second derivatives are needed and for periodic data
def _distances(pos, m, shifts=None):
    p = _shifted(pos, m, shifts)
    return (p[1] - p[0]).norm(p=2, dim=1)


def _angles_cos(pos, m, shifts=None):
    p = _shifted(pos, m, shifts)
    a, b = p[0] - p[1], p[2] - p[1]
    return (a * b).sum(dim=1) / a.norm(p=2, dim=1) / b.norm(p=2, dim=1)


def _torsions(pos, m, shifts=None):
    p = _shifted(pos, m, shifts)
    b1, b2, b3 = p[1] - p[0], p[2] - p[1], p[3] - p[2]
    b1, b2, b3 = (v / v.norm(p=2, dim=1)[:, None] for v in (b1, b2, b3))
    n1, n2 = torch.cross(b1, b2, dim=1), torch.cross(b2, b3, dim=1)
    m1 = torch.cross(n1, b2, dim=1)
    return torch.atan2(-(m1 * n2).sum(-1), (n1 * n2).sum(-1))


class _Prior(torch.nn.Module):
    """base.py:66-141: a prior reads ``data.neighbor_list[self.name]`` and writes ``data.out[self.name]["energy"]``."""

    kind = None

    def _params(self, data) -> torch.Tensor:
        raise NotImplementedError

    def _energy_terms(self, pos, mapping, params, shifts=None) -> torch.Tensor:
        raise NotImplementedError

    def _interaction_types(self, data):
        mapping = data.neighbor_list[self.name]["index_mapping"]
        return tuple(data.atom_types[mapping[i]] for i in range(self.order))

    def _cached_params(self, data) -> torch.Tensor:
        """[P, M] per-term parameters.  The index lists and bead types of a simulation are static, so the gathered rows are
        kept on the module (what mlcg's StaticPrior specialisation does, src/mlcg/simulation/specialize_prior.py:49-59) and
        reused while nothing they were gathered from has changed: the key holds the identity and the in-place version counter
        of the index list, the bead types and every parameter table of this prior, and the dtype and device asked for."""
        mapping, types_ = data.neighbor_list[self.name]["index_mapping"], data.atom_types
        tables = tuple(self.buffers())
        key = tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in (mapping, types_) + tables) + (data.pos.dtype, data.pos.device)
        cached = self.__dict__.get("_param_cache")
        if cached is None or cached[0] != key:
            # (the tensors of the key are held too, so that their storage cannot be freed and handed to another tensor)
            cached = (key, self._params(data).to(data.pos.dtype).contiguous(), (mapping, types_) + tables)
            self.__dict__["_param_cache"] = cached
        return cached[1]

    def _cached_list(self, data):
        """``(kind, idx32 [order, M], params [P, M], symmetric, run_ptr | None)`` for :func:`evaluate_priors`: the index list as 32-bit integers and,
        for pair priors, whether it holds (j, i) for every (i, j) with the same parameters (then forces need no scatter to the second
        bead).  Both are worked out once per index list and parameter set (identity and version of the tensors) and kept on the
        module."""
        mapping = data.neighbor_list[self.name]["index_mapping"]
        params = self._cached_params(data)
        key = (mapping.data_ptr(), mapping._version, tuple(mapping.shape), mapping.device, id(params))
        cached = self.__dict__.get("_list_cache")
        if cached is None or cached[0] != key:
            idx32 = mapping.to(torch.int32).contiguous()
            symmetric = False
            if self.kind in (KIND_BOND, KIND_REPULSION) and mapping.shape[1] > 0 and mapping.shape[1] % 2 == 0:
                # (i, j) and (j, i) both listed, with the same parameters: the two sorted key lists agree, and so do the
                # parameters taken along in the two orders
                n = int(data.pos.shape[0])
                fwd, pf = torch.sort(mapping[0] * n + mapping[1])
                rev, pr = torch.sort(mapping[1] * n + mapping[0])
                symmetric = bool(torch.equal(fwd, rev)) and bool(torch.equal(params[:, pf], params[:, pr]))
                del fwd, rev, pf, pr
            run_ptr = None
            if symmetric:
                # runs of equal first bead (lists built from a topology are grouped by it): a warp then takes a bead's whole run
                first = idx32[0]
                starts = torch.nonzero(first[1:] != first[:-1]).flatten() + 1
                if mapping.shape[1] >= 8 * (starts.numel() + 1):
                    run_ptr = torch.cat([starts.new_zeros(1), starts, starts.new_full((1,), mapping.shape[1])]).to(torch.int64)
            cached = (key, idx32, symmetric, mapping, params, run_ptr)
            self.__dict__["_list_cache"] = cached
        return self.kind, cached[1], params, cached[2], cached[5]

    def energy_and_gradient(self, data):
        """(energy [B], d(sum of energies)/d(pos) [N,3]) straight from the prior kernel, without an autograd graph; None where
        that route does not apply (training mode, tensors off the device, periodic data)."""
        if self.training or not data.pos.is_cuda:
            return None
        nl = data.neighbor_list[self.name]
        if _data_cell_shifts(data, nl["index_mapping"]) is not None:
            return None
        return get_backend().prior_terms(self.kind, data.pos.detach(), nl["index_mapping"], nl["mapping_batch"], self._cached_params(data),
                                         _num_structures(data), want_grad=True)

    def forward(self, data):
        nl = data.neighbor_list[self.name]
        mapping, mapping_batch = nl["index_mapping"], nl["mapping_batch"]
        B = _num_structures(data)
        params = self._cached_params(data)
        shifts = _data_cell_shifts(data, mapping)
        if shifts is not None or (self.training and torch.is_grad_enabled()):
            y = self._energy_terms(data.pos, mapping, params, shifts)
            energy = torch.zeros(B, dtype=y.dtype, device=y.device).index_add_(0, mapping_batch, y)
        else:
            energy = _PriorEnergy.apply(data.pos, self.kind, mapping, mapping_batch, params, _batch_or_zeros(data), B)
        data.out[self.name] = {"energy": energy}
        return data


class Harmonic(_Prior):
    """k (x - x0)^2 + V0, no factor one half (harmonic.py:22-120)."""

    def __init__(self, statistics: Dict, name: str, order: int) -> None:
        super().__init__()
        self.allowed_interaction_keys = list(statistics.keys())
        self.name, self.order = name, order
        self.register_buffer("x_0", _table_from_statistics(statistics, order, "x_0"))
        self.register_buffer("k", _table_from_statistics(statistics, order, "k"))

    def data2parameters(self, data):
        t = self._interaction_types(data)
        params = {"x0": self.x_0[t].flatten(), "k": self.k[t].flatten()}
        params["V0"] = torch.zeros_like(params["x0"])
        return params

    def _params(self, data):
        p = self.data2parameters(data)
        return torch.stack([p["x0"], p["k"]])

    @staticmethod
    def compute(x, x0, k, V0=0):
        return k * (x - x0) ** 2 + V0


class HarmonicBonds(Harmonic):
    name: Final[str] = "bonds"
    _order = 2
    kind = KIND_BOND

    def __init__(self, statistics) -> None:
        super().__init__(statistics, HarmonicBonds.name, order=2)

    def _energy_terms(self, pos, mapping, params, shifts=None):
        return Harmonic.compute(_distances(pos, mapping, shifts), params[0], params[1])

    @staticmethod
    def compute_features(pos, mapping, pbc=None, cell=None, batch=None):
        return _distances(pos, mapping, _feature_shifts(pos, mapping, pbc, cell, batch))


class HarmonicAngles(Harmonic):
    """k (cos(theta) - x0)^2: x0 is a cosine (harmonic.py:245-297)."""

    name: Final[str] = "angles"
    _order = 3
    kind = KIND_ANGLE

    def __init__(self, statistics) -> None:
        super().__init__(statistics, HarmonicAngles.name, order=3)

    def _energy_terms(self, pos, mapping, params, shifts=None):
        return Harmonic.compute(_angles_cos(pos, mapping, shifts), params[0], params[1])

    @staticmethod
    def compute_features(pos, mapping, pbc=None, cell=None, batch=None):
        return _angles_cos(pos, mapping, _feature_shifts(pos, mapping, pbc, cell, batch))


class GeneralBonds(Harmonic):
    """Harmonic bonds under a name of the caller's choosing, so that a model can hold several bond priors over different
    index lists (harmonic.py:487-525)."""

    name: Final[str] = "bonds"
    _order = 2
    kind = KIND_BOND

    def __init__(self, statistics, name) -> None:
        super().__init__(statistics, name, order=GeneralBonds._order)

    _energy_terms = HarmonicBonds._energy_terms
    compute_features = staticmethod(HarmonicBonds.compute_features)


class GeneralAngles(Harmonic):
    """Harmonic angles (in the cosine) under a name of the caller's choosing (harmonic.py:528-566)."""

    name: Final[str] = "angles"
    _order = 3
    kind = KIND_ANGLE

    def __init__(self, statistics, name) -> None:
        super().__init__(statistics, name, order=GeneralAngles._order)

    _energy_terms = HarmonicAngles._energy_terms
    compute_features = staticmethod(HarmonicAngles.compute_features)


class Repulsion(_Prior):
    """(sigma / d)^6 over the pair list as given (repulsion.py:14-140)."""

    name: Final[str] = "repulsion"
    _neighbor_list_name = "fully connected"
    kind = KIND_REPULSION

    def __init__(self, statistics: Dict) -> None:
        super().__init__()
        self.allowed_interaction_keys = list(statistics.keys())
        self.order = 2
        self.register_buffer("sigma", _table_from_statistics(statistics, 2, "sigma"))

    def _params(self, data):
        return self.sigma[self._interaction_types(data)].flatten().unsqueeze(0)

    def _energy_terms(self, pos, mapping, params, shifts=None):
        return Repulsion.compute(_distances(pos, mapping, shifts), params[0])

    @staticmethod
    def compute_features(pos, mapping, pbc=None, cell=None, batch=None):
        return _distances(pos, mapping, _feature_shifts(pos, mapping, pbc, cell, batch))

    @staticmethod
    def compute(x, sigma):
        rr = (sigma / x) * (sigma / x)
        return rr * rr * rr


class FourierSeries(_Prior):
    """v0 + sum_n k1_n sin(n theta) + k2_n cos(n theta) (fourier_series.py:16-198)."""

    kind = KIND_DIHEDRAL

    def __init__(self, statistics: Dict, name: str = "", n_degs: int = 6, order: int = 4) -> None:
        super().__init__()
        self.allowed_interaction_keys = list(statistics.keys())
        self.order, self.name, self.n_degs = order, name, n_degs
        self.k1_names = ["k1_" + str(i) for i in range(1, n_degs + 1)]
        self.k2_names = ["k2_" + str(i) for i in range(1, n_degs + 1)]
        keys = torch.tensor(list(statistics.keys()), dtype=torch.long)
        sizes = tuple([int(torch.unique(keys.flatten()).max()) + 1] * order)
        k1, k2, v_0 = torch.zeros(n_degs, *sizes), torch.zeros(n_degs, *sizes), torch.zeros(*sizes)
        for key, val in statistics.items():
            for i in range(n_degs):
                k1[i][key] = val["k1s"][self.k1_names[i]]
                k2[i][key] = val["k2s"][self.k2_names[i]]
            v_0[key] = val["v_0"]
        self.register_buffer("k1s", k1)
        self.register_buffer("k2s", k2)
        self.register_buffer("v_0", v_0)

    def data2parameters(self, data):
        t = self._interaction_types(data)
        k1s = torch.vstack([self.k1s[i][t] for i in range(self.n_degs)]).t()
        k2s = torch.vstack([self.k2s[i][t] for i in range(self.n_degs)]).t()
        return {"k1s": k1s, "k2s": k2s, "v_0": self.v_0[t].view(-1, 1)}

    def _params(self, data):
        p = self.data2parameters(data)
        v_0 = p["v_0"][:, :1]            # (a merged prior pads v_0 to the width of the series; only column 0 counts)
        return torch.cat([v_0.t(), p["k1s"].t(), p["k2s"].t()], dim=0)   # rows: v0, k1_1..k1_n, k2_1..k2_n

    def _energy_terms(self, pos, mapping, params, shifts=None):
        n = self.n_degs
        return FourierSeries.compute(_torsions(pos, mapping, shifts), params[0], params[1:1 + n].t(), params[1 + n:1 + 2 * n].t())

    @staticmethod
    def compute(theta, v_0, k1s, k2s):
        n_degs = torch.arange(1, k1s.shape[1] + 1, dtype=theta.dtype, device=theta.device)
        angles = theta.view(-1, 1) * n_degs.view(1, -1)
        V = k1s * torch.sin(angles) + k2s * torch.cos(angles)
        if v_0.ndim > 1:
            v_0 = v_0[:, 0]
        return V.sum(dim=1) + v_0


class Dihedral(FourierSeries):
    name: Final[str] = "dihedrals"
    _order: Final[int] = 4

    def __init__(self, statistics: Dict, n_degs: int = 3, name: str = "dihedrals") -> None:
        super().__init__(statistics, name=name, n_degs=n_degs, order=self._order)

    @staticmethod
    def compute_features(pos, mapping, pbc=None, cell=None, batch=None):
        return _torsions(pos, mapping, _feature_shifts(pos, mapping, pbc, cell, batch))


def evaluate_priors(priors, data):
    """Energies and position gradients of several priors on ``data`` from one kernel launch (per eight priors): ``{name: (energy
    [B], dE/dpos [N,3])}``, or None where that route does not apply (training mode, tensors off the device, periodic data).  What
    ``SumOut`` calls for its prior components in eval mode, instead of one launch and one pass over the positions per prior."""
    priors = list(priors)
    if not priors or not data.pos.is_cuda or any(p.training for p in priors):
        return None
    if getattr(data, "pbc", None) is not None and getattr(data, "cell", None) is not None:
        return None
    from .._lib import MAX_PRIOR_SEGMENTS
    B = _num_structures(data)
    struct_of = _batch_or_zeros(data).to(torch.int32)
    out = {}
    be = get_backend()
    for lo in range(0, len(priors), MAX_PRIOR_SEGMENTS):
        chunk = priors[lo:lo + MAX_PRIOR_SEGMENTS]
        energy, grad = be.prior_eval([p._cached_list(data) for p in chunk], data.pos, struct_of, B, deterministic=_DETERMINISTIC)
        for k, p in enumerate(chunk):
            out[p.name] = (energy[k], grad[k])
    return out
