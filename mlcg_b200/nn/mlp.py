"""MLP with mlcg's constructor and ``layers.{i}`` parameter names (src/mlcg/nn/mlp.py:7-58)."""
from typing import List

import torch

from ..autograd import MatmulNT, tanh as tanh_op


def init_xavier_uniform(module: torch.nn.Module, zero_bias: bool = True) -> None:
    """Xavier-uniform weights, zero bias, Linear layers only (src/mlcg/nn/_module_init.py:4-28)."""
    if isinstance(module, torch.nn.Linear):
        torch.nn.init.xavier_uniform_(module.weight)
        if module.bias is not None and zero_bias:
            torch.nn.init.constant_(module.bias, 0.0)


def linear(layer: torch.nn.Linear, x: torch.Tensor, frozen: bool) -> torch.Tensor:
    """``layer(x)`` through this package's GEMM kernels; ``frozen`` takes weight and bias out of the autograd graph."""
    w, b = layer.weight, layer.bias
    if frozen:
        w, b = w.detach(), (None if b is None else b.detach())
    return MatmulNT.apply(x, w, b)


def node_linear(layer: torch.nn.Linear, x: torch.Tensor, training: bool) -> torch.Tensor:
    """Node-sized Linear layers on the tensor-core GEMMs when the widths allow, else torch.  In eval mode (forces only) the
    weights are constants; in training mode they stay in the graph (the operators are differentiable to any order)."""
    if x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and layer.in_features <= 128 and layer.out_features <= 128:
        return linear(layer, x, frozen=not training)
    return layer(x)


class MLP(torch.nn.Module):
    def __init__(self, layer_widths: List[int] = None, activation_func: torch.nn.Module = torch.nn.Tanh(), last_bias: bool = True):
        super().__init__()
        if layer_widths is None:
            layer_widths = [10, 10, 1]
        layers = []
        for w_in, w_out in zip(layer_widths[:-2], layer_widths[1:-1]):
            layers += [torch.nn.Linear(w_in, w_out, bias=True), activation_func]
        layers.append(torch.nn.Linear(layer_widths[-2], layer_widths[-1], bias=last_bias))
        self.layers = torch.nn.Sequential(*layers)
        self.reset_parameters()

    def reset_parameters(self):
        for layer in self.layers:
            init_xavier_uniform(layer)

    def forward(self, x, data=None):
        if x.is_cuda and x.dtype == torch.float32 and x.dim() == 2:
            # fp32-equivalent tensor-core GEMMs; in eval mode the weights are constants, in training they stay in the graph
            return self.forward_edges(x, frozen=not self.training)
        return self.layers(x)

    def forward_edges(self, x: torch.Tensor, frozen: bool = False) -> torch.Tensor:
        """Same function as :meth:`forward`, with every Linear layer run by this package's GEMM kernels
        (used for the edge-sized filter network, where the row count is the number of edges).

        ``frozen=True`` takes the weights out of the autograd graph.  A custom autograd function is told
        which of its inputs *require* a gradient, not which gradients the caller asked for, so with live
        weights the edge-sized weight-gradient GEMMs would run even when only forces are wanted."""
        for layer in self.layers:
            if isinstance(layer, torch.nn.Linear):
                x = linear(layer, x, frozen)
            elif type(layer) is torch.nn.Tanh:
                x = tanh_op(x)
            else:
                x = layer(x)
        return x
