"""SchNet with mlcg's classes, constructor arguments, attribute names and ``state_dict`` keys
(src/mlcg/nn/schnet.py), computing through this package's sm_100a kernels.

``SchNet`` :32-192, ``InteractionBlock`` :195-262, ``CFConv`` :265-368, ``StandardSchNet`` :371-475.
"""
import warnings
from typing import Final, List

import torch

from .. import _lib
from ..autograd import (EdgeDiff, EdgeDistanceOnce, FusedFilterConv, FusedInteraction, PairSelect, RowScale, SchNetEval, SegIn, SegmentSum, SegPair,
                        edge_distances, plan_of)
from ..autograd import tanh as tanh_op
from ..backend import get_backend
from ..data import ENERGY_KEY
from ..neighbor_list import atomic_data2neighbor_list, edge_plan_for, validate_neighborlist
from .cutoff import cutoff_kind
from .mlp import MLP, init_xavier_uniform, node_linear

FILTER_PRECISIONS = {"fp32": 0, "bf16": 1}


class LazyRadialBasis:
    """Stands for ``rbf_layer(distances)`` without computing it.  In eval mode the fused tensor-core kernel
    evaluates the basis inside its GEMM prologue, so the ``[E, R]`` expansion never has to exist; a consumer
    that does need it calls :meth:`materialize`."""

    def __init__(self, distances: torch.Tensor, rbf_layer: torch.nn.Module, symmetric: bool):
        self.distances, self.rbf_layer, self.symmetric = distances, rbf_layer, symmetric

    def materialize(self) -> torch.Tensor:
        return _tag_symmetric(self.rbf_layer(self.distances), self.symmetric)

_SYM = "_mlcgb_symmetric"   # tag on edge tensors that are functions of the (symmetric) distance only
_PAIRS = "_mlcgb_per_pair"  # tag on tensors that hold one row per unordered pair of the edge list instead of one per edge


def _tag_symmetric(t: torch.Tensor, flag: bool) -> torch.Tensor:
    setattr(t, _SYM, flag)
    return t


def _tag_pairs(t: torch.Tensor) -> torch.Tensor:
    setattr(t, _PAIRS, True)
    return t


def _batch_of(data, ptr):
    """Structure index per bead; built from the structure pointer for data that carry no ``batch`` (a single structure)."""
    batch = getattr(data, "batch", None)
    if batch is None:
        batch = torch.repeat_interleave(torch.arange(ptr.numel() - 1, device=ptr.device), ptr[1:] - ptr[:-1], output_size=data.pos.shape[0])
    return batch


_FROZEN_WARNED = False


def _warn_frozen_weights(model):
    """Eval-mode evaluations run on kernels that treat every weight as a constant: energies and forces are exact, but the energy
    carries no graph to the parameters.  Say so, once, when someone may be relying on such a graph (gradients enabled and a
    parameter that requires them); ``model.train()`` keeps every parameter differentiable."""
    global _FROZEN_WARNED
    if _FROZEN_WARNED or not torch.is_grad_enabled() or not any(p.requires_grad for p in model.parameters()):
        return
    _FROZEN_WARNED = True
    warnings.warn("mlcg_b200: in eval mode SchNet is evaluated with its weights as constants (energies and position gradients only); "
                  "a backward pass will not reach the parameters. Use model.train() to differentiate with respect to parameters, or "
                  "p.requires_grad_(False) / torch.no_grad() to silence this message.", stacklevel=3)


class CFConv(torch.nn.Module):
    """Continuous-filter convolution (schnet.py:265-368): ``lin2( sum_j lin1(x)_j * W_ij )`` with
    ``W = filter_network(rbf) * cutoff(d)``.  Same constructor and sub-module names as the reference,
    which derives from PyG's ``MessagePassing``; the aggregation here is an ordered segmented sum."""

    def __init__(self, filter_network: torch.nn.Module, cutoff: torch.nn.Module, in_channels: int = 128, out_channels: int = 128,
                 num_filters: int = 128, aggr: str = "add"):
        super().__init__()
        if aggr != "add":
            raise NotImplementedError("mlcg_b200.CFConv implements aggr='add' (the only scheme mlcg's SchNet uses)")
        self.aggr = aggr
        self.lin1 = torch.nn.Linear(in_channels, num_filters, bias=False)
        self.lin2 = torch.nn.Linear(num_filters, out_channels)
        self.filter_network = filter_network
        self.cutoff = cutoff
        self.filter_precision = "fp32"   # "bf16": filter GEMMs with bf16 operands (eval mode only)
        self.reset_parameters()

    def reset_parameters(self):
        self.filter_network.reset_parameters()
        init_xavier_uniform(self.lin1)
        init_xavier_uniform(self.lin2)

    def fused_spec(self, rbf_layer):
        """The tensor-core kernel covers: eval mode, tanh filter MLP [R, 128, 128] with a bias on the first
        layer only, R <= 128, Gaussian / exp-normal basis with cosine or identity envelopes, float32."""
        net = self.filter_network
        if self.training or not isinstance(net, MLP) or len(net.layers) != 3 or not hasattr(rbf_layer, "spec"):
            return None
        if not getattr(get_backend(), "tensor_core_gemm", False):     # the switch that sends every GEMM to the CUDA cores
            return None
        # the answer depends on module structure, device and dtype only: kept until one of them changes
        rc = rbf_layer.cutoff
        key = (id(rbf_layer), net.layers[0].weight.device, net.layers[0].weight.dtype, id(self.cutoff), id(rc),
               getattr(self.cutoff, "cutoff_lower", None), getattr(self.cutoff, "cutoff_upper", None),
               getattr(rc, "cutoff_lower", None), getattr(rc, "cutoff_upper", None),
               tuple(map(id, net.layers)), tuple(map(id, rbf_layer._parameters.values())), tuple(map(id, rbf_layer._buffers.values())))
        cached = self.__dict__.get("_fused_spec_cache")
        if cached is not None and cached[0] == key:
            return cached[1]
        result = self._fused_spec_uncached(rbf_layer)
        self.__dict__["_fused_spec_cache"] = (key, result)
        return result

    def _fused_spec_uncached(self, rbf_layer):
        net = self.filter_network
        l0, act, l2 = net.layers
        if not (isinstance(l0, torch.nn.Linear) and isinstance(l2, torch.nn.Linear) and isinstance(act, torch.nn.Tanh)):
            return None
        if l0.bias is None or l2.bias is not None or l0.out_features != 128 or l2.out_features != 128 or l0.in_features > 128:
            return None
        if l0.weight.dtype != torch.float32 or not l0.weight.is_cuda:
            return None
        ck, rk = cutoff_kind(self.cutoff), cutoff_kind(rbf_layer.cutoff)
        if ck is None or rk is None or (ck == 1 and self.cutoff.cutoff_lower < 0):
            return None
        return rbf_layer.spec(), (ck, float(self.cutoff.cutoff_lower), float(self.cutoff.cutoff_upper) if ck == 1 else 1.0)

    def filters(self, edge_weight: torch.Tensor, edge_attr: torch.Tensor) -> torch.Tensor:
        """W[E, F] (schnet.py:340-341)."""
        C = self.cutoff(edge_weight)
        net = self.filter_network
        # eval mode evaluates energies and forces only (GradientsOut uses create_graph=False there), so the
        # filter weights are constants; training mode keeps them differentiable to second order
        h = net.forward_edges(edge_attr, frozen=not self.training) if isinstance(net, MLP) else net(edge_attr)
        return RowScale.apply(h, C.reshape(-1)) if h.dim() == 2 and C.numel() == h.shape[0] else h * C.view(-1, 1)

    def forward(self, x: torch.Tensor, edge_index: torch.Tensor, edge_weight: torch.Tensor, edge_attr: torch.Tensor) -> torch.Tensor:
        plan = plan_of(edge_index, x.shape[0])
        if isinstance(edge_attr, LazyRadialBasis):
            fused = self.fused_spec(edge_attr.rbf_layer) if x.dtype == torch.float32 and edge_attr.symmetric == plan.symmetric else None
            if fused is not None:
                net = self.filter_network.layers
                xl = node_linear(self.lin1, x, self.training)
                agg = FusedFilterConv.apply(xl, edge_weight, net[0].weight.detach(), net[0].bias.detach(), net[2].weight.detach(), plan,
                                            fused[0], fused[1], FILTER_PRECISIONS[self.filter_precision])
                return node_linear(self.lin2, agg, self.training)
            edge_attr = edge_attr.materialize()
        symmetric = bool(getattr(edge_weight, _SYM, False) and getattr(edge_attr, _SYM, False))
        W = self.filters(edge_weight, edge_attr)
        x = node_linear(self.lin1, x, self.training)
        if getattr(edge_weight, _PAIRS, False) and getattr(edge_attr, _PAIRS, False) and W.shape[0] * 2 == plan.E:
            x = SegPair.apply(x, W, plan)           # one filter row per unordered pair, read from both of its ends
        else:
            x = SegIn.apply(x, W, plan, symmetric)  # x_j = x[edge_index[0]], summed at edge_index[1]
        return node_linear(self.lin2, x, self.training)

    def message(self, x_j: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
        return x_j * W


class InteractionBlock(torch.nn.Module):
    """CFConv -> activation -> Linear (schnet.py:195-262)."""

    def __init__(self, cfconv_layer: torch.nn.Module, hidden_channels: int = 128, activation: torch.nn.Module = torch.nn.Tanh()):
        super().__init__()
        self.conv = cfconv_layer
        self.activation = activation
        self.lin = torch.nn.Linear(hidden_channels, hidden_channels)
        self.reset_parameters()

    def reset_parameters(self):
        self.conv.reset_parameters()
        init_xavier_uniform(self.lin)

    def forward(self, x, edge_index, edge_weight, edge_attr, *args):
        y = self.conv(x, edge_index, edge_weight, edge_attr)
        y = tanh_op(y) if type(self.activation) is torch.nn.Tanh else self.activation(y)
        return node_linear(self.lin, y, self.training)

    def forward_residual(self, x, edge_index, edge_weight, edge_attr, *args, fused=None):
        """``x + self(x, ...)`` (the sum at schnet.py:150).  In eval mode, when the block has the standard layout — a CFConv the
        fused filter kernel covers, tanh, 128-wide Linear layers — the whole expression runs as one autograd node whose GEMMs
        carry the activation and the sums as epilogues."""
        conv = self.conv
        if (not self.training and type(conv) is CFConv and isinstance(edge_attr, LazyRadialBasis) and isinstance(self.activation, torch.nn.Tanh)
                and x.dtype == torch.float32 and x.is_cuda and conv.lin1.bias is None and conv.lin2.bias is not None and self.lin.bias is not None):
            plan = plan_of(edge_index, x.shape[0])
            if edge_attr.symmetric != plan.symmetric:
                fused = None
            elif fused is None:          # (SchNet.forward hands over what it already worked out)
                fused = conv.fused_spec(edge_attr.rbf_layer)
            be = get_backend()
            if (fused is not None and be.gemm_fused_ok(0, x, conv.lin1.weight) and conv.lin1.out_features == 128
                    and be.gemm_fused_ok(0, x, self.lin.weight) and conv.lin2.in_features == 128 and conv.lin2.out_features == self.lin.in_features
                    and self.lin.out_features == x.shape[1] and conv.lin2.out_features % 4 == 0 and conv.lin2.out_features <= 128):
                net = conv.filter_network.layers
                return FusedInteraction.apply(x, edge_weight, conv.lin1.weight.detach(), net[0].weight.detach(), net[0].bias.detach(),
                                              net[2].weight.detach(), conv.lin2.weight.detach(), conv.lin2.bias.detach(),
                                              self.lin.weight.detach(), self.lin.bias.detach(), plan, fused[0], fused[1],
                                              FILTER_PRECISIONS[conv.filter_precision])
        return x + self(x, edge_index, edge_weight, edge_attr, *args)


class SchNet(torch.nn.Module):
    """schnet.py:32-192.  ``forward(data)`` fills ``data.out["SchNet"]["energy"]`` with one energy per structure."""

    name: Final[str] = "SchNet"

    def __init__(self, embedding_layer: torch.nn.Module, interaction_blocks: List[torch.nn.Module], rbf_layer: torch.nn.Module,
                 output_network: torch.nn.Module, self_interaction: bool = False, max_num_neighbors: int = 1000,
                 nls_distance_method: str = "custom_kernel"):
        super().__init__()
        self.embedding_layer = embedding_layer
        self.rbf_layer = rbf_layer
        self.max_num_neighbors = max_num_neighbors
        if self_interaction:
            raise NotImplementedError("The option `self_interaction` did not have function due to a bug. It only exists for compatibility and should stay `False`.")
        self.self_interaction = self_interaction
        if isinstance(interaction_blocks, list):
            self.interaction_blocks = torch.nn.Sequential(*interaction_blocks)
        elif isinstance(interaction_blocks, InteractionBlock):
            self.interaction_blocks = torch.nn.Sequential(interaction_blocks)
        else:
            raise RuntimeError("interaction_blocks must be a single InteractionBlock or a list of InteractionBlocks.")
        self.nls_distance_method = nls_distance_method
        self.output_network = output_network
        self.reset_parameters()

    def reset_parameters(self):
        self.embedding_layer.reset_parameters()
        self.rbf_layer.reset_parameters()
        for block in self.interaction_blocks:
            block.reset_parameters()
        self.output_network.reset_parameters()

    def is_nl_compatible(self, nl) -> bool:
        # (the reference reads ``self.cutoff`` here, which SchNet never sets, schnet.py:164-173; the
        #  intended comparison is with the radial basis' upper cutoff)
        return bool(validate_neighborlist(nl) and nl["order"] == 2 and nl["self_interaction"] is False
                    and nl["rcut"] == self.rbf_layer.cutoff.cutoff_upper)

    def neighbor_list(self, data, rcut: float, max_num_neighbors: int = 1000) -> dict:
        if not hasattr(self, "nls_distance_method"):
            self.nls_distance_method = "custom_kernel"
        return {SchNet.name: atomic_data2neighbor_list(data, rcut, self_interaction=False, max_num_neighbors=max_num_neighbors,
                                                       nls_distance_method=self.nls_distance_method)}

    def _structure_ptr(self, data):
        n_atoms = getattr(data, "n_atoms", None)
        if n_atoms is not None and torch.is_tensor(n_atoms) and n_atoms.dim() == 1:
            ptr = torch.zeros(n_atoms.numel() + 1, dtype=torch.int64, device=data.pos.device)
            torch.cumsum(n_atoms.to(device=data.pos.device, dtype=torch.int64), 0, out=ptr[1:])
            return ptr
        if getattr(data, "batch", None) is None:       # a single structure
            return torch.tensor([0, data.pos.shape[0]], dtype=torch.int64, device=data.pos.device)
        return get_backend().batch_to_ptr(data.batch, int(data.batch[-1]) + 1)

    # ---- whole-model evaluation in one library call (eval mode, standard layout)
    def _whole_model_slots(self):
        """(module, parameter name) of every tensor ``mlcgb_schnet_eval`` reads, or None if the layout is not the standard
        one: nn.Embedding, InteractionBlock(CFConv) blocks with tanh, output network MLP([H, w, 1]) with tanh."""
        emb, head = self.embedding_layer, self.output_network
        if type(emb) is not torch.nn.Embedding or not isinstance(head, MLP) or len(head.layers) != 3:
            return None
        h0, hact, h1 = head.layers
        if not (isinstance(h0, torch.nn.Linear) and isinstance(hact, torch.nn.Tanh) and isinstance(h1, torch.nn.Linear)):
            return None
        if h0.bias is None or h1.out_features != 1 or h0.in_features != emb.embedding_dim:
            return None
        slots = [(emb, "weight"), (h0, "weight"), (h0, "bias"), (h1, "weight"), (h1, "bias")]
        for b in self.interaction_blocks:
            if type(b) is not InteractionBlock or type(b.conv) is not CFConv or not isinstance(b.activation, torch.nn.Tanh):
                return None
            c, net = b.conv, b.conv.filter_network
            if not isinstance(net, MLP) or len(net.layers) != 3 or c.lin1.bias is not None or c.lin2.bias is None or b.lin.bias is None:
                return None
            slots += [(c.lin1, "weight"), (net.layers[0], "weight"), (net.layers[0], "bias"), (net.layers[2], "weight"), (c.lin2, "weight"),
                      (c.lin2, "bias"), (b.lin, "weight"), (b.lin, "bias")]
        return slots

    def packed_weights(self):
        """``mlcgb_schnet_weights`` over the current parameters (rebuilt whenever a parameter's storage has moved), or None."""
        slots = self.__dict__.get("_mlcgb_slots", False)
        if slots is False:
            slots = self.__dict__["_mlcgb_slots"] = self._whole_model_slots()
        if slots is None:
            return None
        tensors = [m._parameters[n] for m, n in slots]
        key = tuple(0 if t is None else t.data_ptr() for t in tensors)
        packed = self.__dict__.get("_mlcgb_packed")
        if packed is not None and packed[0] == key:
            return packed[1]
        ok = all(t is None or (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()) for t in tensors)
        H = self.embedding_layer.embedding_dim
        blocks = list(self.interaction_blocks)
        F, H2, Wh = blocks[0].conv.lin1.out_features, blocks[0].conv.lin2.out_features, self.output_network.layers[0].out_features
        ok = ok and F == 128 and all(b.conv.lin1.out_features == F and b.conv.lin2.out_features == H2 and b.conv.lin2.in_features == F
                                     and b.lin.in_features == H2 and b.lin.out_features == H and b.conv.lin1.in_features == H for b in blocks)
        ok = ok and all(v % 4 == 0 and v <= 128 for v in (H, H2, Wh))
        result = None
        if ok:
            ptr = lambda t: None if t is None else t.data_ptr()
            arr = (_lib.SchnetBlockStruct * len(blocks))()
            for i in range(len(blocks)):
                for f, t in zip(("lin1_w", "filter_w1", "filter_b1", "filter_w2", "lin2_w", "lin2_b", "lin_w", "lin_b"), tensors[5 + 8 * i: 13 + 8 * i]):
                    setattr(arr[i], f, ptr(t))
            ws = _lib.SchnetWeightsStruct(H, F, H2, Wh, len(blocks), self.embedding_layer.num_embeddings, arr, ptr(tensors[0]), ptr(tensors[1]),
                                          ptr(tensors[2]), ptr(tensors[3]), ptr(tensors[4]))
            result = (ws, (arr, tensors))
        self.__dict__["_mlcgb_packed"] = (key, result)
        return result

    def forward(self, data):
        neighbor_list = data.neighbor_list.get(self.name)
        if not self.is_nl_compatible(neighbor_list):
            neighbor_list = self.neighbor_list(data, self.rbf_layer.cutoff.cutoff_upper, self.max_num_neighbors)[self.name]
        fast = self._forward_whole_model(data, neighbor_list)
        if fast is not None:
            return fast
        x = self.embedding_layer(data.atom_types)
        edge_index = neighbor_list["index_mapping"]
        cell_shifts = neighbor_list["cell_shifts"]
        # (a host read; lists built by this package for non-periodic data are known to be shift-free)
        shifted = (not neighbor_list.get("_mlcgb_zero_shifts", False) and cell_shifts is not None and cell_shifts.numel() > 0
                   and bool(torch.any(cell_shifts != 0)))
        plan = plan_of(edge_index, data.pos.shape[0])
        if shifted:             # periodic copies: |pos[j] + shift - pos[i]| (internal_coordinates.py:72-100)
            distances = (EdgeDiff.apply(data.pos, plan) + cell_shifts.view(-1, 3).to(data.pos.dtype)).norm(p=2, dim=1)
        elif self.training:
            distances = edge_distances(data.pos, plan)          # differentiable to any order
        else:
            distances = EdgeDistanceOnce.apply(data.pos, plan)  # one kernel forward, one backward
        distances = _tag_symmetric(distances, plan.symmetric)
        specs = [b.conv.fused_spec(self.rbf_layer) if (not self.training and type(b) is InteractionBlock and type(b.conv) is CFConv) else None
                 for b in self.interaction_blocks]
        lazy_ok = not self.training and distances.dtype == torch.float32 and all(s is not None for s in specs)
        # Training on a symmetric, loop-free list: the filters depend on the pair's distance only, so the basis, the filter network
        # and all their derivatives run on one row per unordered pair (half the rows); the aggregation reads a pair's row from
        # both of its ends (autograd.SegPair).  Only for blocks known to pass these tensors straight to their CFConv.
        per_pair = (self.training and not shifted and plan.half_selection() is not None
                    and all(type(b) is InteractionBlock and type(b.conv) is CFConv for b in self.interaction_blocks))
        if lazy_ok:
            _warn_frozen_weights(self)
            rbf_expansion = LazyRadialBasis(distances, self.rbf_layer, plan.symmetric)
        elif per_pair:
            distances = _tag_pairs(PairSelect.apply(distances, plan))
            rbf_expansion = _tag_pairs(self.rbf_layer(distances))
        else:
            rbf_expansion = _tag_symmetric(self.rbf_layer(distances), plan.symmetric)
        # (number of structures for blocks that ask for it, taken from n_atoms where that avoids reading batch[-1] on the host)
        num_batch = None if all(type(b) is InteractionBlock for b in self.interaction_blocks) else self._num_structures(data)
        for block, spec in zip(self.interaction_blocks, specs):
            if type(block) is InteractionBlock:
                x = block.forward_residual(x, edge_index, distances, rbf_expansion, num_batch, data.batch, fused=spec if lazy_ok else None)
            else:
                x = x + block(x, edge_index, distances, rbf_expansion, num_batch, data.batch)
        energy = self.output_network(x, data)
        ptr = neighbor_list.get("_mlcgb_ptr")
        if ptr is None or ptr.device != x.device or ptr[-1:].numel() == 0:
            ptr = self._structure_ptr(data)
        energy = SegmentSum.apply(energy, ptr, _batch_of(data, ptr)).flatten()
        data.out[self.name] = {ENERGY_KEY: energy}
        return data

    def energy_and_gradient(self, data):
        """(energy [B], d(sum of energies)/d(pos) [N,3]) from one library call, without an autograd graph; None where the
        whole-model route does not apply (see :meth:`_whole_model_setup`)."""
        setup = self._whole_model_setup(data.pos)
        if setup is None:
            return None
        neighbor_list = data.neighbor_list.get(self.name)
        if self.is_nl_compatible(neighbor_list):
            if not neighbor_list.get("_mlcgb_zero_shifts", False):
                return None
            plan, ptr = plan_of(neighbor_list["index_mapping"], data.pos.shape[0]), neighbor_list.get("_mlcgb_ptr")
        elif self.edge_capacity:
            return self._fixed_capacity_evaluation(data, setup)
        elif getattr(data, "pbc", None) is not None and bool(torch.any(data.pbc)):
            return None         # periodic structures: distances carry cell shifts, which the one-call route does not take
        else:       # the graph alone: no neighbour-list dictionary, mapping_batch or cell shifts are needed on this route
            plan, ptr, _ = edge_plan_for(data, self.rbf_layer.cutoff.cutoff_upper, self.max_num_neighbors)
        if plan.half_selection() is None:
            return None
        if ptr is None or ptr.device != data.pos.device:
            ptr = self._structure_ptr(data)
        spec, conv_cut, weights, precision = setup
        return get_backend().schnet_eval(data.pos.detach().contiguous(), self._types(data), ptr, plan, spec, conv_cut, weights, precision,
                                         want_grad=True)

    #: Fixed edge capacity (an even number of directed edges) for evaluations that must not read the edge count on the host,
    #: e.g. a molecular-dynamics step recorded into a CUDA graph; None: buffers are sized by the count read in every call.
    edge_capacity = None

    def _fixed_capacity_evaluation(self, data, setup):
        """Radius graph, pair plan and evaluation into buffers of ``edge_capacity`` edges: no device->host read anywhere.  More
        edges than the capacity, or a list cut short by ``max_num_neighbors``, are reported by the backend's deferred status
        check (``get_backend().check_pending()``)."""
        from ..autograd import EdgePlan
        from ..neighbor_list import structure_pointer, _as_3d
        be = get_backend()
        pos = data.pos.detach().contiguous()
        N, cap = pos.shape[0], int(self.edge_capacity)
        key = (N, cap, pos.device)
        cached = self.__dict__.get("_mlcgb_rows")
        if cached is None or cached[0] != key:       # stale entries of earlier graphs stay valid point indices for the same N
            cached = self.__dict__["_mlcgb_rows"] = (key, torch.zeros((2, cap), dtype=torch.int32, device=pos.device))
        ptr = structure_pointer(data)
        res = be.radius_graph_capacity(_as_3d(pos), ptr, float(self.rbf_layer.cutoff.cutoff_upper), self.max_num_neighbors, cap, rows=cached[1])
        twin, sel, pair_of, _ = be.pair_plan(res["row0"], res["row1"], res["offsets"], N)
        plan = EdgePlan(N, cap, res["row0"], res["row1"], res["offsets"], None, res["row1"], res["offsets"], twin, res["row1"], True, False)
        plan._half, plan._pair_of = sel, pair_of
        spec, conv_cut, weights, precision = setup
        return be.schnet_eval(pos, self._types(data), ptr, plan, spec, conv_cut, weights, precision, want_grad=True, counts=res["counts"])

    @staticmethod
    def _num_structures(data) -> int:
        n_atoms = getattr(data, "n_atoms", None)
        if n_atoms is not None and torch.is_tensor(n_atoms) and n_atoms.dim() == 1:
            return int(n_atoms.numel())
        return 1 if getattr(data, "batch", None) is None else int(data.batch[-1]) + 1

    def _forward_whole_model(self, data, neighbor_list):
        setup = self._whole_model_setup(data.pos)
        if setup is None or not neighbor_list.get("_mlcgb_zero_shifts", False):
            return None
        plan = plan_of(neighbor_list["index_mapping"], data.pos.shape[0])
        if plan.half_selection() is None:
            return None
        ptr = neighbor_list.get("_mlcgb_ptr")
        if ptr is None or ptr.device != data.pos.device:
            ptr = self._structure_ptr(data)
        spec, conv_cut, weights, precision = setup
        _warn_frozen_weights(self)
        data.out[self.name] = {ENERGY_KEY: SchNetEval.apply(data.pos, self._types(data), ptr, _batch_of(data, ptr), plan, spec, conv_cut, weights, precision)}
        return data

    @staticmethod
    def _types(data):
        types = data.atom_types
        if types.dtype != torch.int64 or not types.is_contiguous():
            types = types.to(torch.int64).contiguous()
        return types

    def _whole_model_setup(self, pos):
        """(basis spec, CFConv cutoff, packed weights, filter precision) for ``mlcgb_schnet_eval``, or None: eval mode, no kernel
        profiler attached, float32 positions on CUDA, at least 128 beads, standard layout with every block on the fused filter
        kernel, one cutoff and one filter precision for all blocks.  The model-dependent part is worked out once per set of
        parameter storages and cutoff values."""
        be = get_backend()
        if (self.training or getattr(be, "profiler", True) is not None or not getattr(be, "tensor_core_gemm", False) or not pos.is_cuda
                or pos.dtype != torch.float32 or pos.shape[0] < 128):
            return None
        weights = self.packed_weights()
        if weights is None or weights[1][1][0].device != pos.device:
            return None
        blocks = self.interaction_blocks
        rc = self.rbf_layer.cutoff
        rbf = self.rbf_layer
        key = (id(weights), id(rbf), tuple(map(id, rbf._parameters.values())), tuple(map(id, rbf._buffers.values())),
               getattr(rc, "cutoff_lower", None), getattr(rc, "cutoff_upper", None),
               tuple((getattr(b.conv.cutoff, "cutoff_lower", None), getattr(b.conv.cutoff, "cutoff_upper", None), b.conv.filter_precision)
                     for b in blocks))
        cached = self.__dict__.get("_mlcgb_setup")
        if cached is not None and cached[0] == key:
            return cached[1]
        specs = [b.conv.fused_spec(self.rbf_layer) for b in blocks]
        precisions = {FILTER_PRECISIONS[b.conv.filter_precision] for b in blocks}
        result = None
        if all(s is not None for s in specs) and all(s[1] == specs[0][1] for s in specs[1:]) and len(precisions) == 1:
            result = (specs[0][0], specs[0][1], weights, precisions.pop())
        self.__dict__["_mlcgb_setup"] = (key, result, weights)      # (keeps `weights` alive, so its id stays unique)
        return result


class StandardSchNet(SchNet):
    """Convenience constructor (schnet.py:371-475): same arguments, same defaults."""

    def __init__(self, rbf_layer: torch.nn.Module, cutoff: torch.nn.Module, output_hidden_layer_widths: List[int],
                 hidden_channels: int = 128, embedding_size: int = 100, num_filters: int = 128, num_interactions: int = 3,
                 activation: torch.nn.Module = torch.nn.Tanh(), max_num_neighbors: int = 1000, aggr: str = "add",
                 nls_distance_method: str = "custom_kernel"):
        if num_interactions < 1:
            raise ValueError("At least one interaction block must be specified")
        if cutoff.cutoff_lower != rbf_layer.cutoff.cutoff_lower:
            warnings.warn("Cutoff function lower cutoff, {}, and radial basis function  lower cutoff, {}, do not match.".format(
                cutoff.cutoff_lower, rbf_layer.cutoff.cutoff_lower))
        if cutoff.cutoff_upper != rbf_layer.cutoff.cutoff_upper:
            warnings.warn("Cutoff function upper cutoff, {}, and radial basis function  upper cutoff, {}, do not match.".format(
                cutoff.cutoff_upper, rbf_layer.cutoff.cutoff_upper))
        embedding_layer = torch.nn.Embedding(embedding_size, hidden_channels)
        blocks = []
        for _ in range(num_interactions):
            filter_network = MLP(layer_widths=[rbf_layer.num_rbf, num_filters, num_filters], activation_func=activation, last_bias=False)
            cfconv = CFConv(filter_network, cutoff=cutoff, num_filters=num_filters, in_channels=hidden_channels,
                            out_channels=hidden_channels, aggr=aggr)
            blocks.append(InteractionBlock(cfconv, hidden_channels, activation))
        output_network = MLP([hidden_channels] + output_hidden_layer_widths + [1], activation_func=activation, last_bias=False)
        super().__init__(embedding_layer, blocks, rbf_layer, output_network, max_num_neighbors=max_num_neighbors,
                         nls_distance_method=nls_distance_method)


class AttentiveSchNet(SchNet):
    """SchNet whose interaction blocks add attention over the beads of each structure (schnet.py:478-674): same arguments and
    sub-module names.  ``attention_version`` "normal" (`AttentiveInteractionBlock`) or "2" (`AttentiveInteractionBlock2`); the
    attention arguments are given all together or all ``None`` (a block without the non-local part cannot be evaluated in the
    reference either)."""

    def __init__(self, rbf_layer: torch.nn.Module, cutoff: torch.nn.Module, output_hidden_layer_widths: List[int], num_features_in: int,
                 num_features_out: int, num_residual_q: int, num_residual_k: int, num_residual_v: int, attention_block: torch.nn.Module,
                 hidden_channels: int = 128, embedding_size: int = 100, num_filters: int = 128, num_interactions: int = 3,
                 activation_func: torch.nn.Module = torch.nn.Tanh(), max_num_neighbors: int = 1000, layer_widths: List[int] = None,
                 activation_first: bool = False, aggr: str = "add", attention_version: str = "normal",
                 nls_distance_method: str = "custom_kernel"):
        from .attention import AttentiveInteractionBlock, AttentiveInteractionBlock2, Nonlocalinteractionblock
        layer_widths = [128, 128] if layer_widths is None else layer_widths
        if num_interactions < 1:
            raise ValueError("At least one interaction block must be specified")
        if cutoff.cutoff_lower != rbf_layer.cutoff.cutoff_lower:
            warnings.warn("Cutoff function lower cutoff, {}, and radial basis function  lower cutoff, {}, do not match.".format(
                cutoff.cutoff_lower, rbf_layer.cutoff.cutoff_lower))
        if cutoff.cutoff_upper != rbf_layer.cutoff.cutoff_upper:
            warnings.warn("Cutoff function upper cutoff, {}, and radial basis function  upper cutoff, {}, do not match.".format(
                cutoff.cutoff_upper, rbf_layer.cutoff.cutoff_upper))
        if attention_version not in ("normal", "2"):
            raise RuntimeError("attention_version not recognized")
        block_cls = AttentiveInteractionBlock if attention_version == "normal" else AttentiveInteractionBlock2
        attention_args = [num_features_in, num_features_out, num_residual_q, num_residual_k, num_residual_v, attention_block]
        given = [a is not None for a in attention_args]
        if any(given) and not all(given):
            raise ValueError("To use Attention, you must specify 'num_features_in','num_features_out','num_residual_q','num_residual_k', "
                             "'num_residual_v' and 'attention_block'")
        embedding_layer = torch.nn.Embedding(embedding_size, hidden_channels)
        blocks = []
        for _ in range(num_interactions):
            filter_network = MLP(layer_widths=[rbf_layer.num_rbf, num_filters, num_filters], activation_func=activation_func)
            cfconv = CFConv(filter_network, cutoff=cutoff, num_filters=num_filters, in_channels=hidden_channels,
                            out_channels=hidden_channels, aggr=aggr)
            nonlocal_part = None
            if all(given):
                # (as in the reference, `layer_widths`, `activation_func` and `activation_first` do not reach the non-local part:
                # its residual blocks are 128 wide with tanh, so the features have to be 128 wide as well)
                nonlocal_part = Nonlocalinteractionblock(num_features_in, num_features_out, num_residual_q, num_residual_k, num_residual_v,
                                                         attention_block)
            blocks.append(block_cls(cfconv_layer=cfconv, hidden_channels=hidden_channels, activation_func=activation_func,
                                    attention_block=nonlocal_part))
        output_network = MLP([hidden_channels] + output_hidden_layer_widths + [1], activation_func=activation_func, last_bias=False)
        super().__init__(interaction_blocks=blocks, rbf_layer=rbf_layer, embedding_layer=embedding_layer, output_network=output_network,
                         max_num_neighbors=max_num_neighbors, nls_distance_method=nls_distance_method)

    def energy_and_gradient(self, data):
        return None         # attention mixes all beads of a structure: no one-call route


class RBFRegularizedSchNet(StandardSchNet):
    """StandardSchNet whose radial basis is scaled per pair of bead types, with one set of factors for all interaction blocks or
    one per block (schnet.py:676-803).  Also puts the factors into ``data.out["SchNet"]["radial_filters"]``.  The scaled basis is
    an explicit ``[blocks, E, R]`` tensor here (the fused filter kernel evaluates the unscaled bases only), so this model runs on
    the per-operator kernels."""

    def __init__(self, rbf_layer: torch.nn.Module, cutoff: torch.nn.Module, output_hidden_layer_widths: List[int],
                 hidden_channels: int = 128, embedding_size: int = 100, num_filters: int = 128, num_interactions: int = 3,
                 activation: torch.nn.Module = torch.nn.Tanh(), max_num_neighbors: int = 1000, aggr: str = "add",
                 nls_distance_method: str = "custom_kernel", independent_regularizations: bool = False):
        from .radial_basis import RegularizedBasis
        rbf_layer = RegularizedBasis(basis_function=rbf_layer, types=embedding_size, n_basis_set=num_interactions,
                                     independent_regularizations=independent_regularizations)
        super().__init__(rbf_layer=rbf_layer, cutoff=cutoff, output_hidden_layer_widths=output_hidden_layer_widths,
                         hidden_channels=hidden_channels, embedding_size=embedding_size, num_filters=num_filters,
                         num_interactions=num_interactions, activation=activation, max_num_neighbors=max_num_neighbors, aggr=aggr,
                         nls_distance_method=nls_distance_method)

    def energy_and_gradient(self, data):
        return None         # no one-call route: the filters depend on the bead types of each pair

    def forward(self, data):
        neighbor_list = data.neighbor_list.get(self.name)
        if not self.is_nl_compatible(neighbor_list):
            neighbor_list = self.neighbor_list(data, self.rbf_layer.cutoff.cutoff_upper, self.max_num_neighbors)[self.name]
        x = self.embedding_layer(data.atom_types)
        edge_index = neighbor_list["index_mapping"]
        if not neighbor_list.get("_mlcgb_zero_shifts", False):
            cell_shifts = neighbor_list["cell_shifts"]
            if cell_shifts is not None and cell_shifts.numel() > 0 and bool(torch.any(cell_shifts != 0)):
                raise NotImplementedError("periodic cell shifts are outside the scope of mlcg_b200")
        plan = plan_of(edge_index, data.pos.shape[0])
        distances = edge_distances(data.pos, plan) if self.training else EdgeDistanceOnce.apply(data.pos, plan)
        rbf_expansion = self.rbf_layer(distances, data.atom_types[edge_index[0]], data.atom_types[edge_index[1]])
        for block_id, block in enumerate(self.interaction_blocks):
            x = x + block(x, edge_index, distances, rbf_expansion[block_id], None, data.batch)
        energy = self.output_network(x, data)
        ptr = neighbor_list.get("_mlcgb_ptr")
        if ptr is None or ptr.device != x.device:
            ptr = self._structure_ptr(data)
        energy = SegmentSum.apply(energy, ptr, data.batch).flatten()
        data.out[self.name] = {ENERGY_KEY: energy, "radial_filters": self.rbf_layer.get_regularization_parameters()}
        return data


def set_edge_capacity(model: torch.nn.Module, capacity) -> torch.nn.Module:
    """Fixed edge capacity (directed edges, rounded up to an even number; None: off) for every SchNet of ``model``."""
    capacity = None if capacity is None else (int(capacity) + 1) // 2 * 2
    for m in model.modules():
        if isinstance(m, SchNet):
            m.edge_capacity = capacity
    return model


def set_filter_precision(model: torch.nn.Module, precision: str) -> torch.nn.Module:
    """``"fp32"`` (default: fp32-equivalent tensor-core products) or ``"bf16"`` for every CFConv of ``model``."""
    if precision not in FILTER_PRECISIONS:
        raise ValueError(f"precision must be one of {sorted(FILTER_PRECISIONS)}")
    for m in model.modules():
        if isinstance(m, CFConv):
            m.filter_precision = precision
    return model
