"""Radial bases with mlcg's class names, constructor arguments and parameter names
(src/mlcg/nn/radial_basis/gaussian.py, exp_normal.py, base.py)."""
from typing import Union

import torch
from torch import nn

from ..autograd import RbfExpand
from ..backend import RbfSpec
from .cutoff import CosineCutoff, IdentityCutoff, _Cutoff, cutoff_kind


class _RadialBasis(nn.Module):
    def __init__(self):
        super().__init__()
        self.cutoff = None

    def check_cutoff(self):
        if self.cutoff.cutoff_upper < self.cutoff.cutoff_lower:
            raise ValueError("Upper cutoff {} is less than lower cutoff {}".format(self.cutoff.cutoff_upper, self.cutoff.cutoff_lower))

    def _resolve_cutoff(self, cutoff, default_cls):
        if isinstance(cutoff, (float, int)):
            return default_cls(0, cutoff)
        if isinstance(cutoff, _Cutoff) or cutoff_kind(cutoff) is not None:
            return cutoff
        raise TypeError("Supplied cutoff {} is neither a number nor a _Cutoff instance.".format(cutoff))

    def _kernel_ok(self, dist: torch.Tensor) -> bool:
        """The kernels know two envelopes and take distances as a vector."""
        return cutoff_kind(self.cutoff) is not None and dist.dim() == 1 and self.num_rbf <= 256

    def _trained(self, p0: torch.Tensor, p1: torch.Tensor):
        """The parameter tensors to hand to the kernels' autograd node: those that are being trained (training mode, gradients
        on); their gradients then come from ``mlcgb_rbf_param_contract``.  In eval mode only position gradients are taken, as
        in GradientsOut with create_graph=False."""
        if not self.training or not torch.is_grad_enabled():
            return None, None
        return (p0 if p0.requires_grad else None), (p1 if p1.requires_grad else None)


class GaussianBasis(_RadialBasis):
    """exp(coeff (d - offset_k)^2) * envelope(d), gaussian.py:9-102."""

    def __init__(self, cutoff: Union[int, float, _Cutoff], num_rbf: int = 50, trainable: bool = False):
        super().__init__()
        self.cutoff = self._resolve_cutoff(cutoff, IdentityCutoff)
        self.check_cutoff()
        self.num_rbf, self.trainable = num_rbf, trainable
        offset, coeff = self._initial_params()
        if trainable:
            self.register_parameter("coeff", nn.Parameter(coeff))
            self.register_parameter("offset", nn.Parameter(offset))
        else:
            self.register_buffer("coeff", coeff)
            self.register_buffer("offset", offset)

    def _initial_params(self):
        offset = torch.linspace(self.cutoff.cutoff_lower, self.cutoff.cutoff_upper, self.num_rbf)
        return offset, -0.5 / (offset[1] - offset[0]) ** 2

    def reset_parameters(self):
        offset, coeff = self._initial_params()
        self.offset.data.copy_(offset)
        self.coeff.data.copy_(coeff)

    def spec(self) -> RbfSpec:
        c = self.cutoff
        return RbfSpec(0, self.num_rbf, cutoff_kind(c), float(c.cutoff_lower), float(c.cutoff_upper), 0.0, self.offset, self.coeff)

    def forward(self, dist: torch.Tensor) -> torch.Tensor:
        if self._kernel_ok(dist):
            return RbfExpand.apply(dist, self.spec(), 0, *self._trained(self.offset, self.coeff))
        dist = dist.unsqueeze(-1)
        return torch.exp(self.coeff * torch.pow(dist - self.offset, 2)) * self.cutoff(dist)


class ExpNormalBasis(_RadialBasis):
    """envelope(d) * exp(-beta_k (exp(alpha (lower - d)) - mean_k)^2), exp_normal.py:9-124."""

    def __init__(self, cutoff: Union[int, float, _Cutoff], num_rbf: int = 50, trainable: bool = True):
        super().__init__()
        self.cutoff = self._resolve_cutoff(cutoff, CosineCutoff)
        self.check_cutoff()
        self.num_rbf, self.trainable = num_rbf, trainable
        self.alpha = 5.0 / (self.cutoff.cutoff_upper - self.cutoff.cutoff_lower)
        means, betas = self._initial_params()
        if trainable:
            self.register_parameter("means", nn.Parameter(means))
            self.register_parameter("betas", nn.Parameter(betas))
        else:
            self.register_buffer("means", means)
            self.register_buffer("betas", betas)

    def _initial_params(self):
        start = torch.exp(torch.scalar_tensor(-self.cutoff.cutoff_upper + self.cutoff.cutoff_lower))
        means = torch.linspace(start, 1, self.num_rbf)
        betas = torch.tensor([(2 / self.num_rbf * (1 - start)) ** -2] * self.num_rbf)
        return means, betas

    def reset_parameters(self):
        means, betas = self._initial_params()
        self.means.data.copy_(means)
        self.betas.data.copy_(betas)

    def spec(self) -> RbfSpec:
        c = self.cutoff
        return RbfSpec(1, self.num_rbf, cutoff_kind(c), float(c.cutoff_lower), float(c.cutoff_upper), float(self.alpha), self.means, self.betas)

    def forward(self, dist: torch.Tensor) -> torch.Tensor:
        if self._kernel_ok(dist):
            return RbfExpand.apply(dist, self.spec(), 0, *self._trained(self.means, self.betas))
        dist = dist.unsqueeze(-1)
        inner = torch.exp(self.alpha * (-dist + self.cutoff.cutoff_lower)) - self.means
        return self.cutoff(dist) * torch.exp(-self.betas * inner ** 2)


class SymmetricTensor(nn.Module):
    """One learnable vector of length ``size`` per unordered pair of indices below ``N``, stored as the rows of the upper
    triangle (regularized_basis.py:7-61); every entry starts at ``init_val``."""

    def __init__(self, N: int, size: int, init_val: float = 1.0):
        super().__init__()
        self.N, self.size = N, size
        self.w = nn.Parameter(torch.full((N * (N + 1) // 2, size), float(init_val)))
        self.check_bounds = False

    def enable_input_bound_check(self, enable: bool = True):
        self.check_bounds = enable
        return self

    def forward(self, i: torch.Tensor, j: torch.Tensor) -> torch.Tensor:
        if self.check_bounds and bool(((i >= self.N) | (j >= self.N) | (i < 0) | (j < 0)).any()):
            raise IndexError(f"SymmetricTensor indices out of bounds [0, {self.N}): ")
        lo, hi = torch.minimum(i, j), torch.maximum(i, j)
        row = ((2 * self.N - lo + 1) * lo) // 2 + (hi - lo)      # rows of the upper triangle, row-major
        return self.w[row]


class RegularizedBasis(nn.Module):
    """A radial basis whose functions are scaled, per pair of bead types, by learnable factors clamped to [0, 1]
    (regularized_basis.py:63-235): ``forward(d, type_i, type_j)`` gives ``[n_basis_set, E, num_rbf]``, one scaled copy per
    interaction block — all from one factor table, or one table per block with ``independent_regularizations``."""

    def __init__(self, basis_function: _RadialBasis, types: int, n_basis_set: int, independent_regularizations: bool = False,
                 init_val=1.0):
        super().__init__()
        self.basis_function = basis_function
        self.types, self.n_basis_set = types, n_basis_set
        self.independent_regularizations = independent_regularizations
        self.num_rbf, self.cutoff = basis_function.num_rbf, basis_function.cutoff
        if independent_regularizations:
            vals = init_val if isinstance(init_val, list) else [init_val] * n_basis_set
            self.regularization = nn.ModuleList([SymmetricTensor(types, self.num_rbf, vals[k]) for k in range(n_basis_set)])
        else:
            if isinstance(init_val, list):
                if len(init_val) != 1:
                    raise ValueError("When using shared regularization parameters, init_val should be a single float value.")
                init_val = init_val[0]
            self.regularization = SymmetricTensor(types, self.num_rbf, init_val)

    def factors(self, type_i: torch.Tensor, type_j: torch.Tensor) -> torch.Tensor:
        """[n_basis_set, E, num_rbf], clamped to [0, 1]."""
        if self.independent_regularizations:
            f = torch.stack([r(type_i, type_j) for r in self.regularization], dim=0)
        else:
            f = self.regularization(type_i, type_j).unsqueeze(0).expand(self.n_basis_set, -1, -1)
        return torch.clamp(f, min=0.0, max=1.0)

    def forward(self, distances: torch.Tensor, type_i: torch.Tensor, type_j: torch.Tensor) -> torch.Tensor:
        return self.basis_function(distances).unsqueeze(0) * self.factors(type_i, type_j)

    def get_regularization_parameters(self) -> torch.Tensor:
        if self.independent_regularizations:
            return torch.stack([r.w for r in self.regularization])
        return self.regularization.w

    def reset_parameters(self):
        pass        # (the factors are set at construction, as in the reference)
