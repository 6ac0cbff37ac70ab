"""Non-local (attention) update of the bead features for ``AttentiveSchNet`` (src/mlcg/nn/attention.py, after SpookyNet,
Unke et al., Nat. Commun. 12, 2021): residual MLPs produce queries, keys and values from the features, and every bead
attends to the beads of its own structure — with the softmax kernel (``ExactAttention``) or its positive random-feature
approximation (``FavorAttention``, FAVOR+).  Class names, constructor arguments and ``state_dict`` keys are mlcg's; the
dense algebra runs as torch matrix products (these blocks sit next to the CFConv path, which keeps its own kernels)."""
import math
from typing import List, Optional

import torch

from .mlp import init_xavier_uniform


def _widths(layer_widths):
    return [128, 128] if layer_widths is None else layer_widths


class Residual(torch.nn.Module):
    """``x + f(x)`` with ``f`` a chain of (Linear, activation) pairs, or (activation, Linear) with ``activation_first``
    (attention.py:20-66)."""

    def __init__(self, layer_widths: List[int] = None, activation_func: torch.nn.Module = torch.nn.Tanh(), activation_first: bool = False) -> None:
        super().__init__()
        layers = []
        widths = _widths(layer_widths)
        for w_in, w_out in zip(widths[:-1], widths[1:]):
            linear = torch.nn.Linear(w_in, w_out, bias=True)
            layers += [activation_func, linear] if activation_first else [linear, activation_func]
        self.layers = torch.nn.Sequential(*layers)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for layer in self.layers:
            init_xavier_uniform(layer)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.layers(x)


class ResidualStack(torch.nn.Module):
    """``num_residual`` residual blocks in sequence (attention.py:69-111)."""

    def __init__(self, num_residual: int, layer_widths: List[int] = None, activation_func: torch.nn.Module = torch.nn.Tanh(),
                 activation_first: bool = False) -> None:
        super().__init__()
        self.stack = torch.nn.ModuleList([Residual(_widths(layer_widths), activation_func, activation_first) for _ in range(num_residual)])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for block in self.stack:
            x = block(x)
        return x


class Residual_MLP(torch.nn.Module):
    """Residual stack, then one Linear layer and the activation — or activation, then Linear, with ``activation_first``
    (attention.py:114-176)."""

    def __init__(self, num_features_in: int, num_features_out: int, num_residual: int, layer_widths: List[int] = None,
                 activation_func: torch.nn.Module = torch.nn.Tanh(), activation_first: bool = False) -> None:
        super().__init__()
        self.linear = torch.nn.Linear(num_features_in, num_features_out, bias=True)
        self.activation_func = activation_func
        self.residual = ResidualStack(num_residual, _widths(layer_widths), activation_func, activation_first)
        self.activation_first = activation_first
        self.reset_parameters()

    def reset_parameters(self) -> None:
        init_xavier_uniform(self.linear)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.residual(x)
        if self.activation_first:
            return self.linear(self.activation_func(y))
        return self.activation_func(self.linear(y))


def _same_structure(batch_seg: torch.Tensor, dtype) -> torch.Tensor:
    """[N, N] matrix of ones where two beads belong to the same structure."""
    return (batch_seg.view(-1, 1) == batch_seg.view(1, -1)).to(dtype)


class ExactAttention(torch.nn.Module):
    """Softmax attention inside each structure (attention.py:179-218): weights ``exp((q.k - max) / sqrt(d))`` with the
    maximum over the whole batch, pairs of different structures removed, rows normalised with ``eps`` in the denominator.
    The last attention weights are kept (``attention_matrix`` gives them as a numpy array, as the reference stores them)."""

    def __init__(self) -> None:
        super().__init__()
        self._weights = None

    @property
    def attention_matrix(self):
        return None if self._weights is None else self._weights.cpu().numpy()

    def forward(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, num_batch: int, batch_seg: torch.Tensor,
                mask: Optional[torch.Tensor] = None, eps: float = 1e-8) -> torch.Tensor:
        scores = Q @ K.T
        A = torch.exp((scores - torch.max(scores)) / Q.shape[-1] ** 0.5)
        if num_batch > 1:
            A = A * _same_structure(batch_seg, A.dtype)
        weights = A / (torch.sum(A, dim=-1, keepdim=True) + eps)
        self._weights = weights.detach()
        return weights @ V


class FavorAttention(torch.nn.Module):
    """FAVOR+ attention (attention.py:221-353): queries and keys are mapped to ``dimqk`` positive random features
    ``exp(omega.x / d^(1/4) - |x|^2 / (2 sqrt(d)) - max) + eps``, with which attention becomes two thin matrix products.
    ``omega`` (a buffer, part of the ``state_dict``) holds random directions, orthogonal within groups of ``dimqk``, each
    scaled by the norm of a random vector of uniform samples, as the reference draws them."""

    def __init__(self, dimv: int = 128, dimqk: int = 128) -> None:
        super().__init__()
        self.register_buffer("omega", self._omega(dimv, dimqk))

    @staticmethod
    def _omega(nrows: int, ncols: int) -> torch.Tensor:
        """``[ncols, nrows]``: ``nrows`` directions in ``ncols`` dimensions, orthogonal within every group of ``ncols``
        (QR of a random square matrix), each rescaled by the norm of a fresh random row."""
        rows = []
        remaining = nrows
        while remaining > 0:
            q, _ = torch.linalg.qr(torch.rand(size=(ncols, ncols)))
            take = min(ncols, remaining)
            rows.append(q.T[:take])
            remaining -= take
        lengths = torch.linalg.norm(torch.rand(size=(nrows, ncols)), dim=1, keepdim=True)
        return (lengths * torch.vstack(rows)).T

    def phi(self, x: torch.Tensor, is_query: bool, num_batch: int, batch_seg: torch.Tensor, eps: float = 1e-4) -> torch.Tensor:
        d, m = x.shape[-1], self.omega.shape[-1]
        U = torch.matmul(x.float() / d ** 0.25, self.omega.float())
        h = torch.sum(x ** 2, dim=-1, keepdim=True) / (2 * d ** 0.5)
        if is_query:
            maximum = torch.max(U, dim=-1, keepdim=True)[0]
        elif num_batch > 1:
            # one maximum per structure over its beads and all features; beads of other structures enter as zeros, so the
            # result is never below zero (as in the reference, which takes the maximum of the masked matrix)
            per_bead = torch.max(U, dim=-1)[0]
            floor = torch.zeros(num_batch, dtype=U.dtype, device=U.device)
            per_structure = floor.scatter_reduce(0, batch_seg, per_bead, reduce="amax", include_self=True)
            maximum = per_structure[batch_seg].unsqueeze(-1)
        else:
            maximum = torch.max(U)
        return (torch.exp(U - h - maximum) + eps) / math.sqrt(m)

    def forward(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, num_batch: int, batch_seg: torch.Tensor,
                mask: Optional[torch.Tensor] = None, eps: float = 1e-8) -> torch.Tensor:
        Q = self.phi(Q, True, num_batch, batch_seg)
        K = self.phi(K, False, num_batch, batch_seg)
        if num_batch > 1:
            d = Q.shape[-1]
            key_sums = K.new_zeros(num_batch, d).index_add_(0, batch_seg, K)
            norm = torch.sum(Q * key_sums[batch_seg], dim=-1, keepdim=True) + eps
            if mask is None:
                mask = _same_structure(batch_seg, V.dtype)
            return ((mask * (K @ Q.transpose(-1, -2))).transpose(-1, -2) @ V) / norm
        norm = Q @ torch.sum(K, 0, keepdim=True).T + eps
        return (Q @ (K.T @ V)) / norm


class Nonlocalinteractionblock(torch.nn.Module):
    """Queries, keys and values from three residual MLPs, combined by the attention block (attention.py:356-441)."""

    def __init__(self, num_features_in: int, num_features_out: int, num_residual_q: int, num_residual_k: int, num_residual_v: int,
                 attention_block: torch.nn.Module, layer_widths: List[int] = None, activation_func: torch.nn.Module = torch.nn.Tanh(),
                 activation_first: bool = False):
        super().__init__()
        make = lambda n: Residual_MLP(num_features_in, num_features_out, n, _widths(layer_widths), activation_func, activation_first)
        self.resmlp_q, self.resmlp_k, self.resmlp_v = make(num_residual_q), make(num_residual_k), make(num_residual_v)
        self.attention_block = attention_block

    def forward(self, x: torch.Tensor, num_batch: int, batch_seg: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.attention_block(self.resmlp_q(x), self.resmlp_k(x), self.resmlp_v(x), num_batch, batch_seg, mask)


class AttentiveInteractionBlock(torch.nn.Module):
    """``lin(a + attention(a))`` with ``a = activation(CFConv(x))`` (attention.py:444-524)."""

    def __init__(self, cfconv_layer: torch.nn.Module, attention_block: torch.nn.Module, hidden_channels: int = 128,
                 activation_func: torch.nn.Module = torch.nn.Tanh()):
        super().__init__()
        self.conv = cfconv_layer
        self.activation = activation_func
        self.lin = torch.nn.Linear(hidden_channels, hidden_channels)
        self.attention_block = attention_block
        self.reset_parameters()

    def reset_parameters(self):
        self.conv.reset_parameters()
        init_xavier_uniform(self.lin)

    def forward(self, x, edge_index, edge_weight, edge_attr, num_batch, batch_seg, mask: Optional[torch.Tensor] = None):
        a = self.activation(self.conv(x, edge_index, edge_weight, edge_attr))
        return self.lin(a + self.attention_block(a, num_batch, batch_seg, mask))


class AttentiveInteractionBlock2(torch.nn.Module):
    """Convolution branch ``lin(activation(CFConv(x)))`` and attention branch ``lin_a(activation(attention(x)))`` on the
    block's input, summed and passed through ``lin_o`` (attention.py:527-612)."""

    def __init__(self, cfconv_layer: torch.nn.Module, attention_block: torch.nn.Module, hidden_channels: int = 128,
                 activation_func: torch.nn.Module = torch.nn.Tanh()):
        super().__init__()
        self.conv = cfconv_layer
        self.activation = activation_func
        self.lin = torch.nn.Linear(hidden_channels, hidden_channels)
        self.lin_a = torch.nn.Linear(hidden_channels, hidden_channels)
        self.lin_o = torch.nn.Linear(hidden_channels, hidden_channels)
        self.attention_block = attention_block
        self.reset_parameters()

    def reset_parameters(self):
        self.conv.reset_parameters()
        init_xavier_uniform(self.lin)

    def forward(self, x, edge_index, edge_weight, edge_attr, num_batch, batch_seg, mask: Optional[torch.Tensor] = None):
        x_l = self.lin(self.activation(self.conv(x, edge_index, edge_weight, edge_attr)))
        x_a = self.lin_a(self.activation(self.attention_block(x, num_batch, batch_seg, mask)))
        return self.lin_o(x_a + x_l)
