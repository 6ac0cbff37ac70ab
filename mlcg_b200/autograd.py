"""Differentiable operators built on the kernel primitives.

Force matching differentiates the forces (themselves a gradient) with respect to the weights, so
every operator's backward must again be differentiable (``create_graph=self.training`` at
``src/mlcg/nn/gradients.py:216-222``).  The operators below are closed under differentiation: the
backward of each one is written with operators of the same family, the same way the reference's
native distance op chains ``RadiusDistanceAGF`` -> ``RadiusDistanceAGB``
(``src/opt_radius/mlcg_opt_radius/radius.py:91-158``), so derivatives of any order come out of
autograd without further code.

Bilinear family on a fixed edge list (row 0 = centre, row 1 = neighbour)::

    SegIn (a, V)[n] = sum_{e: row1(e)=n} a[row0(e)] * V[e]      CFConv aggregation, schnet.py:346,350-368
    SegOut(a, V)[m] = sum_{e: row0(e)=m} a[row1(e)] * V[e]      its transpose
    EdgeMul(a, b)[e] = a[row0(e)] * b[row1(e)]
"""
from dataclasses import dataclass
from typing import Optional

import torch

from .backend import RbfSpec, get_backend


@dataclass
class EdgePlan:
    """Index structures derived once per edge list and shared by every operator and derivative order."""

    N: int
    E: int
    row0: torch.Tensor                 # int32 [E]
    row1: torch.Tensor                 # int32 [E]
    ptr_out: torch.Tensor              # int64 [N+1]  edges grouped by row0
    perm_out: Optional[torch.Tensor]   # int32 [E] edge ids in that grouping; None = edges already in this order
    nbr_out: torch.Tensor              # int32 [E]  row1 in that grouping
    ptr_in: torch.Tensor               # int64 [N+1]  edges grouped by row1
    perm_in: torch.Tensor              # int32 [E]
    nbr_in: torch.Tensor               # int32 [E]  row0 in that grouping
    symmetric: bool = False            # every edge has its reverse, and perm_in maps an edge to it
    loops: bool = False                # the list may hold edges (i, i)
    _half: Optional[torch.Tensor] = None
    _pair_of: Optional[torch.Tensor] = None
    _pair_rows: Optional[tuple] = None

    def half_selection(self) -> Optional[torch.Tensor]:
        """One edge per unordered pair (row0 < row1) of a symmetric, loop-free list; None if that does not apply."""
        if not self.symmetric or self.loops or self.E % 2:
            return None
        if self._half is None:
            # exactly E/2 edges have row0 < row1, so the size is known without reading the device
            self._half = torch.nonzero_static(self.row0 < self.row1, size=self.E // 2).flatten().to(torch.int32)
        return self._half

    def pair_index(self) -> Optional[torch.Tensor]:
        """For every edge the position of its unordered pair in :meth:`half_selection`; None if that does not apply."""
        sel = self.half_selection()
        if sel is None:
            return None
        if self._pair_of is None:
            self._pair_of = get_backend().pair_index(sel, self.perm_in)
        return self._pair_of

    def pair_rows(self):
        """(row0, row1) of the selected edge of every unordered pair (int32 [E/2] each); None if that does not apply."""
        sel = self.half_selection()
        if sel is None:
            return None
        if self._pair_rows is None:
            idx = sel.long()
            self._pair_rows = (self.row0.index_select(0, idx).contiguous(), self.row1.index_select(0, idx).contiguous())
        return self._pair_rows

    @staticmethod
    def from_centre_sorted(row0, row1, offsets, N, symmetric: bool, loops: bool = False) -> "EdgePlan":
        """Edges sorted by (row0, row1) as the radius graph emits them."""
        be = get_backend()
        E = row0.numel()
        if symmetric:
            if not loops and E % 2 == 0 and E > 0 and hasattr(be, "pair_plan"):
                # reverse-edge map, one edge per pair and the edge -> pair index from one library call
                twin, sel, pair_of, _ = be.pair_plan(row0, row1, offsets, N)
                plan = EdgePlan(N, E, row0, row1, offsets, None, row1, offsets, twin, row1, True, loops)
                plan._half, plan._pair_of = sel, pair_of
                return plan
            twin, _ = be.edge_twin(row0, row1, offsets, N)
            # the k-th edge grouped by row1 is the reverse of the k-th edge grouped by row0
            return EdgePlan(N, E, row0, row1, offsets, None, row1, offsets, twin, row1, True, loops)
        return EdgePlan._general(row0, row1, N, ptr_out=offsets, perm_out=None)

    @staticmethod
    def from_edge_index(edge_index: torch.Tensor, N: int) -> "EdgePlan":
        """Any ``[2, E]`` edge list (torch sort / bincount; not the fast path)."""
        row0 = edge_index[0].to(torch.int32).contiguous()
        row1 = edge_index[1].to(torch.int32).contiguous()
        E = row0.numel()
        ordered = bool((row0[1:] >= row0[:-1]).all()) if E > 1 else True
        ptr_out = _ptr_from_index(row0, N)
        perm_out = None if ordered else torch.argsort(row0.to(torch.int64), stable=True).to(torch.int32)
        return EdgePlan._general(row0, row1, N, ptr_out, perm_out)

    @staticmethod
    def _general(row0, row1, N, ptr_out, perm_out) -> "EdgePlan":
        perm_in = torch.argsort(row1.to(torch.int64), stable=True).to(torch.int32)
        nbr_in = row0[perm_in.long()].contiguous()
        nbr_out = row1 if perm_out is None else row1[perm_out.long()].contiguous()
        return EdgePlan(N, row0.numel(), row0, row1, ptr_out, perm_out, nbr_out, _ptr_from_index(row1, N), perm_in, nbr_in, False)


def _ptr_from_index(idx: torch.Tensor, N: int) -> torch.Tensor:
    counts = torch.bincount(idx.to(torch.int64), minlength=N)
    ptr = torch.zeros(N + 1, dtype=torch.int64, device=idx.device)
    torch.cumsum(counts, 0, out=ptr[1:])
    return ptr


def attach_plan(edge_index: torch.Tensor, plan: EdgePlan) -> torch.Tensor:
    edge_index._mlcgb_plan = plan
    return edge_index


def plan_of(edge_index: torch.Tensor, N: int) -> EdgePlan:
    """The plan travelling with an edge list built by this package, else one derived on the spot."""
    plan = getattr(edge_index, "_mlcgb_plan", None)
    if plan is None or plan.N != N or plan.E != edge_index.shape[1]:
        plan = EdgePlan.from_edge_index(edge_index, N)
        edge_index._mlcgb_plan = plan
    return plan


# ------------------------------------------------------------------------------- bilinear family
class SegIn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, V, plan: EdgePlan, v_symmetric: bool = False):
        ctx.plan = plan
        ctx.save_for_backward(a, V)
        be = get_backend()
        if v_symmetric and plan.symmetric:
            # V[e] == V[reverse(e)] bit for bit (it depends on the distance only), so the grouping by
            # row1 can be read as the grouping by row0 and V is streamed in storage order
            return be.seg_mul_sum(a, V, plan.ptr_out, plan.nbr_out, plan.perm_out, plan.N)
        return be.seg_mul_sum(a, V, plan.ptr_in, plan.nbr_in, plan.perm_in, plan.N)

    @staticmethod
    def backward(ctx, g):
        a, V = ctx.saved_tensors
        ga = SegOut.apply(g, V, ctx.plan) if ctx.needs_input_grad[0] else None
        gV = EdgeMul.apply(a, g, ctx.plan) if ctx.needs_input_grad[1] else None
        return ga, gV, None, None


class SegOut(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, V, plan: EdgePlan):
        ctx.plan = plan
        ctx.save_for_backward(a, V)
        return get_backend().seg_mul_sum(a, V, plan.ptr_out, plan.nbr_out, plan.perm_out, plan.N)

    @staticmethod
    def backward(ctx, g):
        a, V = ctx.saved_tensors
        ga = SegIn.apply(g, V, ctx.plan) if ctx.needs_input_grad[0] else None
        gV = EdgeMul.apply(g, a, ctx.plan) if ctx.needs_input_grad[1] else None
        return ga, gV, None


class EdgeMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, plan: EdgePlan):
        ctx.plan = plan
        ctx.save_for_backward(a, b)
        return get_backend().edge_mul(a, b, plan.row0, plan.row1)

    @staticmethod
    def backward(ctx, gV):
        a, b = ctx.saved_tensors
        ga = SegOut.apply(b, gV, ctx.plan) if ctx.needs_input_grad[0] else None
        gb = SegIn.apply(a, gV, ctx.plan) if ctx.needs_input_grad[1] else None
        return ga, gb, None


# ------------------------------------------------------------------------------- the same family with V stored once per pair
# On a symmetric, loop-free list W depends on the pair's distance only, so the filter network can run on one row per unordered
# pair (half the rows of every edge-sized operator of a training step).  With V per pair the two aggregations coincide,
#     SegPair(a, V)[n] = sum_{e: row0(e)=n} a[row1(e)] * V[pair(e)]          PairMul(a, b)[p] = a[i] b[j] + a[j] b[i],  p = {i, j}
# and the family is closed again: d SegPair / da = SegPair(g, V), d SegPair / dV = PairMul(a, g), d PairMul / da = SegPair(b, G).
class SegPair(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, V, plan: EdgePlan):
        ctx.plan = plan
        ctx.save_for_backward(a, V)
        return get_backend().seg_mul_sum(a, V, plan.ptr_out, plan.nbr_out, plan.pair_index(), plan.N)

    @staticmethod
    def backward(ctx, g):
        a, V = ctx.saved_tensors
        ga = SegPair.apply(g, V, ctx.plan) if ctx.needs_input_grad[0] else None
        gV = PairMul.apply(a, g, ctx.plan) if ctx.needs_input_grad[1] else None
        return ga, gV, None


class PairMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, plan: EdgePlan):
        ctx.plan = plan
        ctx.save_for_backward(a, b)
        ia, ib = plan.pair_rows()
        return get_backend().pair_mul(a, b, ia, ib)

    @staticmethod
    def backward(ctx, G):
        a, b = ctx.saved_tensors
        ga = SegPair.apply(b, G, ctx.plan) if ctx.needs_input_grad[0] else None
        gb = SegPair.apply(a, G, ctx.plan) if ctx.needs_input_grad[1] else None
        return ga, gb, None


class PairSelect(torch.autograd.Function):
    """One value per unordered pair out of one per edge (the selected edge's); its gradient goes back to that edge alone."""

    @staticmethod
    def forward(ctx, v, plan: EdgePlan):
        ctx.plan = plan
        return v.index_select(0, plan.half_selection().long())

    @staticmethod
    def backward(ctx, g):
        return PairScatter.apply(g, ctx.plan), None


class PairScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, plan: EdgePlan):
        ctx.plan = plan
        out = torch.zeros((plan.E,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        return out.index_copy_(0, plan.half_selection().long(), g)       # (distinct positions: no accumulation, no atomics)

    @staticmethod
    def backward(ctx, gg):
        return PairSelect.apply(gg, ctx.plan), None


# ------------------------------------------------------------------------------- edge geometry
class EdgeDiff(torch.autograd.Function):
    """dr[e] = pos[row1(e)] - pos[row0(e)] (internal_coordinates.py:93-96, no cell shifts)."""

    @staticmethod
    def forward(ctx, pos, plan: EdgePlan):
        ctx.plan = plan
        return get_backend().edge_diff(pos, plan.row0, plan.row1)

    @staticmethod
    def backward(ctx, g):
        return NodeScatterDiff.apply(g, ctx.plan), None


class NodeScatterDiff(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, plan: EdgePlan):
        ctx.plan = plan
        return get_backend().node_scatter_diff(g, plan.ptr_in, plan.perm_in, plan.ptr_out, plan.perm_out, plan.N)

    @staticmethod
    def backward(ctx, gg):
        return EdgeDiff.apply(gg, ctx.plan), None


def edge_distances(pos: torch.Tensor, plan: EdgePlan) -> torch.Tensor:
    return EdgeDiff.apply(pos, plan).norm(p=2, dim=1)


class EdgeDistanceOnce(torch.autograd.Function):
    """Distances in one kernel with a hand-written first derivative (energy / force evaluation only; the
    composable :func:`edge_distances` serves anything that differentiates twice)."""

    @staticmethod
    def forward(ctx, pos, plan: EdgePlan):
        d = get_backend().edge_distance(pos, plan.row0, plan.row1)
        ctx.plan = plan
        ctx.save_for_backward(pos, d)
        return d

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        pos, d = ctx.saved_tensors
        return get_backend().edge_distance_backward(pos, g, d, ctx.plan), None


# ------------------------------------------------------------------------------- radial basis
MAX_RBF_ORDER = 3


def _rbf_param_grads(ctx, d, G, c):
    """Gradients for the basis parameters handed to RbfExpand / RbfContract as tensors (``None`` where not asked for).  They are
    results of a reduction kernel, not differentiable further: parameter gradients are what the optimiser consumes."""
    want0, want1 = ctx.needs_input_grad[ctx.param_slot], ctx.needs_input_grad[ctx.param_slot + 1]
    if not (want0 or want1):
        return None, None
    with torch.no_grad():
        gp0, gp1 = get_backend().rbf_param_contract(d.detach(), G.detach(), None if c is None else c.detach(), ctx.spec, ctx.order)
    return (gp0.reshape(ctx.p_shapes[0]) if want0 else None), (gp1.reshape(ctx.p_shapes[1]) if want1 else None)


class RbfExpand(torch.autograd.Function):
    """``order``-th distance derivative of basis x envelope, ``[E, R]``.  ``p0`` / ``p1``: the basis' two parameter tensors when
    they are trained (they are the tensors ``spec`` points at; passing them makes autograd ask for their gradients)."""

    @staticmethod
    def forward(ctx, d, spec: RbfSpec, order: int, p0=None, p1=None):
        if order > MAX_RBF_ORDER:
            raise NotImplementedError("radial-basis derivatives beyond third order are not implemented")
        ctx.spec, ctx.order, ctx.param_slot = spec, order, 3
        ctx.p_shapes = (None if p0 is None else p0.shape, None if p1 is None else p1.shape)
        ctx.trained = p0 is not None or p1 is not None
        ctx.save_for_backward(d, p0, p1)
        return get_backend().rbf_expand(d, spec, order)

    @staticmethod
    def backward(ctx, G):
        d, p0, p1 = ctx.saved_tensors
        gd = RbfContract.apply(d, G, ctx.spec, ctx.order + 1, p0, p1) if ctx.needs_input_grad[0] else None
        gp0, gp1 = _rbf_param_grads(ctx, d, G, None) if ctx.trained else (None, None)
        return gd, None, None, gp0, gp1


class RbfContract(torch.autograd.Function):
    """s[e] = sum_k G[e,k] * d^order(basis_k x envelope)/dd^order."""

    @staticmethod
    def forward(ctx, d, G, spec: RbfSpec, order: int, p0=None, p1=None):
        if order > MAX_RBF_ORDER:
            raise NotImplementedError("radial-basis derivatives beyond third order are not implemented")
        ctx.spec, ctx.order, ctx.param_slot = spec, order, 4
        ctx.p_shapes = (None if p0 is None else p0.shape, None if p1 is None else p1.shape)
        ctx.trained = p0 is not None or p1 is not None
        ctx.save_for_backward(d, G, p0, p1)
        return get_backend().rbf_contract(d, G, spec, order)

    @staticmethod
    def backward(ctx, gs):
        d, G, p0, p1 = ctx.saved_tensors
        gd = gs * RbfContract.apply(d, G, ctx.spec, ctx.order + 1, p0, p1) if ctx.needs_input_grad[0] else None
        gG = RowScale.apply(RbfExpand.apply(d, ctx.spec, ctx.order, p0, p1), gs) if ctx.needs_input_grad[1] else None
        gp0, gp1 = _rbf_param_grads(ctx, d, G, gs) if ctx.trained else (None, None)
        return gd, gG, None, None, gp0, gp1


# ------------------------------------------------------------------------------- per-edge scalar x edge row
class RowScale(torch.autograd.Function):
    """out[e,:] = a[e,:] * c[e] (``net(rbf) * C[:, None]``, schnet.py:341); closed under differentiation with RowDot."""

    @staticmethod
    def forward(ctx, a, c):
        ctx.save_for_backward(a, c)
        return get_backend().row_scale(a, c)

    @staticmethod
    def backward(ctx, g):
        a, c = ctx.saved_tensors
        ga = RowScale.apply(g, c) if ctx.needs_input_grad[0] else None
        gc = RowDot.apply(g, a) if ctx.needs_input_grad[1] else None
        return ga, gc


# ------------------------------------------------------------------------------- tanh and its derivatives
class Tanh(torch.autograd.Function):
    """``tanh`` whose derivatives of every order are single elementwise kernels (torch expands the second derivative of tanh
    into several multiplications over the edge-sized tensors of a force-matching step)."""

    @staticmethod
    def forward(ctx, x):
        y = torch.tanh(x)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return TanhGrad.apply(g, y)


class TanhGrad(torch.autograd.Function):
    """g (1 - y^2)."""

    @staticmethod
    def forward(ctx, g, y):
        ctx.save_for_backward(g, y)
        return get_backend().tanh_grad(0, None, g, y)

    @staticmethod
    def backward(ctx, G):
        g, y = ctx.saved_tensors
        gg = TanhGrad.apply(G, y) if ctx.needs_input_grad[0] else None
        gy = TanhGrad2.apply(G, g, y) if ctx.needs_input_grad[1] else None
        return gg, gy


class TanhGrad2(torch.autograd.Function):
    """-2 G g y; beyond this order the derivatives are plain torch products."""

    @staticmethod
    def forward(ctx, G, g, y):
        ctx.save_for_backward(G, g, y)
        return get_backend().tanh_grad(1, G, g, y)

    @staticmethod
    def backward(ctx, u):
        G, g, y = ctx.saved_tensors
        return (-2 * u * g * y if ctx.needs_input_grad[0] else None, -2 * u * G * y if ctx.needs_input_grad[1] else None,
                -2 * u * G * g if ctx.needs_input_grad[2] else None)


def tanh(x: torch.Tensor) -> torch.Tensor:
    """:class:`Tanh` for CUDA tensors that take part in a graph, ``torch.tanh`` otherwise."""
    if x.is_cuda and x.requires_grad and torch.is_grad_enabled() and x.dtype in (torch.float32, torch.float64):
        return Tanh.apply(x)
    return torch.tanh(x)


class RowDot(torch.autograd.Function):
    """out[e] = sum_f a[e,f] * b[e,f]."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return get_backend().row_dot(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        ga = RowScale.apply(b, g) if ctx.needs_input_grad[0] else None
        gb = RowScale.apply(a, g) if ctx.needs_input_grad[1] else None
        return ga, gb


# ------------------------------------------------------------------------------- GEMM family
class MatmulNT(torch.autograd.Function):
    """Y = X W^T (+ bias): ``torch.nn.Linear`` as the filter network applies it (mlp.py:41-58)."""

    @staticmethod
    def forward(ctx, X, W, bias=None):
        ctx.save_for_backward(X, W)
        ctx.has_bias = bias is not None
        return get_backend().gemm(0, X, W, bias)

    @staticmethod
    def backward(ctx, gY):
        X, W = ctx.saved_tensors
        gX = MatmulNN.apply(gY, W) if ctx.needs_input_grad[0] else None
        if ctx.has_bias and ctx.needs_input_grad[2] and ctx.needs_input_grad[1]:
            gW, gb = MatmulTNColsum.apply(gY, X)          # one pass over gY for both
        else:
            gW = MatmulTN.apply(gY, X) if ctx.needs_input_grad[1] else None
            gb = gY.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return gX, gW, gb


class MatmulNN(torch.autograd.Function):
    """Z = G W."""

    @staticmethod
    def forward(ctx, G, W):
        ctx.save_for_backward(G, W)
        return get_backend().gemm(1, G, W)

    @staticmethod
    def backward(ctx, gZ):
        G, W = ctx.saved_tensors
        gG = MatmulNT.apply(gZ, W) if ctx.needs_input_grad[0] else None
        gW = MatmulTN.apply(G, gZ) if ctx.needs_input_grad[1] else None
        return gG, gW


class MatmulTNColsum(torch.autograd.Function):
    """(P, s) = (G^T X, sum over rows of G): the weight and bias gradients of a Linear layer."""

    @staticmethod
    def forward(ctx, G, X):
        ctx.save_for_backward(G, X)
        return get_backend().gemm_tn_colsum(G, X)

    @staticmethod
    def backward(ctx, gP, gs):
        G, X = ctx.saved_tensors
        gG = MatmulNT.apply(X, gP, gs) if ctx.needs_input_grad[0] else None    # X gP^T + gs broadcast over the rows
        gX = MatmulNN.apply(G, gP) if ctx.needs_input_grad[1] else None
        return gG, gX


class MatmulTN(torch.autograd.Function):
    """P = G^T X (contraction over the edge dimension)."""

    @staticmethod
    def forward(ctx, G, X):
        ctx.save_for_backward(G, X)
        return get_backend().gemm(2, G, X)

    @staticmethod
    def backward(ctx, gP):
        G, X = ctx.saved_tensors
        gG = MatmulNT.apply(X, gP) if ctx.needs_input_grad[0] else None
        gX = MatmulNN.apply(G, gP) if ctx.needs_input_grad[1] else None
        return gG, gX


# ------------------------------------------------------------------------------- per-structure sum
class SegmentSum(torch.autograd.Function):
    """out[b] = sum of x over the nodes of structure b (``scatter(energy, batch)``, schnet.py:158)."""

    @staticmethod
    def forward(ctx, x, ptr, batch):
        ctx.save_for_backward(batch)
        ctx.shape = x.shape
        return get_backend().segment_sum(x.reshape(-1), ptr)

    @staticmethod
    def backward(ctx, g):
        (batch,) = ctx.saved_tensors
        return g.index_select(0, batch).reshape(ctx.shape), None, None


# ------------------------------------------------------------------------------- fused eval path
class FusedFilterConv(torch.autograd.Function):
    """agg = SegIn(xl, W(d)) with W(d) = (tanh(phi(d) A1^T + b1) A2^T) C(d) produced by the tensor-core kernel.

    On a symmetric edge list W[e] = W[reverse(e)] (same distance): the filters are evaluated and stored once per
    unordered pair and both aggregations read them through the edge -> pair index.

    First-order only (energies and forces): the backward returns the gradients with respect to ``xl`` and
    ``d`` and is not itself differentiable; training mode uses the composable operators above instead."""

    @staticmethod
    def forward(ctx, xl, d, A1, b1, A2, plan: EdgePlan, spec: RbfSpec, conv_cut, precision: int):
        be = get_backend()
        sel = plan.half_selection()
        keep = bool(ctx.needs_input_grad[1])  # the hidden layer is kept only when the distance gradient will be asked for
        W, status, *hs = be.filter_forward(d, spec, conv_cut[0], conv_cut[1], conv_cut[2], A1, b1, A2, precision, sel, None, save_hidden=keep)
        be.defer_status(status, "fused filter network (forward)")
        if sel is not None:   # W[pair]; grouping by row1 read as the grouping by row0 of the reversed edges
            agg = be.seg_mul_sum(xl, W, plan.ptr_out, plan.nbr_out, plan.pair_index(), plan.N)
        else:
            agg = be.seg_mul_sum(xl, W, plan.ptr_in, plan.nbr_in, plan.perm_in, plan.N)
        ctx.plan, ctx.spec, ctx.conv_cut, ctx.precision = plan, spec, conv_cut, precision
        ctx.hidden = hs[0] if hs else None
        ctx.save_for_backward(xl, d, W, A1, b1, A2)
        return agg

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        xl, d, W, A1, b1, A2 = ctx.saved_tensors
        plan, be = ctx.plan, get_backend()
        g = g.contiguous()
        sel = plan.half_selection()
        gxl = None
        if ctx.needs_input_grad[0]:
            gxl = be.seg_mul_sum(g, W, plan.ptr_out, plan.nbr_out, plan.pair_index() if sel is not None else plan.perm_out, plan.N)
        gd = None
        if ctx.needs_input_grad[1]:     # d(e) and d(reverse(e)) are the same distance: one gradient per pair
            gd, status = be.filter_backward(d, ctx.spec, ctx.conv_cut[0], ctx.conv_cut[1], ctx.conv_cut[2], A1, b1, A2, plan.row0, plan.row1,
                                            xl, g, ctx.precision, sel, plan.perm_in if sel is not None else None, hidden=ctx.hidden)
            be.defer_status(status, "fused filter network (backward)")
        return gxl, gd, None, None, None, None, None, None, None


class FusedInteraction(torch.autograd.Function):
    """One interaction block with its residual sum, eval mode (schnet.py:150, 252-262, 340-350):

        x_new = x + lin( tanh( lin2( CFConv_aggregate( lin1(x), W(d) ) ) ) )

    Ten kernel launches forward and backward together and no elementwise kernel: the activation, its derivative and
    both residual sums are epilogues of the tensor-core GEMMs.  First-order only, weights are constants."""

    @staticmethod
    def forward(ctx, x, d, W1, fA1, fb1, fA2, W2, b2, W3, b3, plan: EdgePlan, spec: RbfSpec, conv_cut, precision: int):
        be = get_backend()
        x = x.contiguous()
        ctx.plan, ctx.spec, ctx.conv_cut, ctx.precision = plan, spec, conv_cut, precision
        if be.interaction_ok(x, plan, x.shape[1], W1.shape[0], W2.shape[0]):        # the whole block in one library call
            d = d.contiguous()
            out, xl, W, a, hs = be.interaction_forward(x, d, plan, spec, conv_cut, W1, fA1, fb1, fA2, W2, b2, W3, b3, precision,
                                                       save_hidden=bool(ctx.needs_input_grad[1]))
            ctx.hidden = hs
            ctx.save_for_backward(xl, d, W, a, W1, fA1, fb1, fA2, W2, W3)
            return out
        xl = be.gemm(0, x, W1)
        sel = plan.half_selection()
        W, status, *hs = be.filter_forward(d, spec, conv_cut[0], conv_cut[1], conv_cut[2], fA1, fb1, fA2, precision, sel, None,
                                           save_hidden=bool(ctx.needs_input_grad[1]))
        ctx.hidden = hs[0] if hs else None
        be.defer_status(status, "fused filter network (forward)")
        if sel is not None:
            agg = be.seg_mul_sum(xl, W, plan.ptr_out, plan.nbr_out, plan.pair_index(), plan.N)
        else:
            agg = be.seg_mul_sum(xl, W, plan.ptr_in, plan.nbr_in, plan.perm_in, plan.N)
        a = be.gemm_fused(0, agg, W2, b2, None, be.EPI_TANH)
        out = be.gemm_fused(0, a, W3, b3, x, be.EPI_ADD)
        ctx.plan, ctx.spec, ctx.conv_cut, ctx.precision = plan, spec, conv_cut, precision
        ctx.save_for_backward(xl, d, W, a, W1, fA1, fb1, fA2, W2, W3)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        xl, d, W, a, W1, fA1, fb1, fA2, W2, W3 = ctx.saved_tensors
        plan, be = ctx.plan, get_backend()
        g = g.contiguous()
        if be.interaction_ok(g, plan, g.shape[1], W1.shape[0], W2.shape[0]):
            gx, gd = be.interaction_backward(g, a, W, xl, ctx.hidden, d, plan, ctx.spec, ctx.conv_cut, W1, fA1, fb1, fA2, W2, W3, ctx.precision,
                                             ctx.needs_input_grad[0], ctx.needs_input_grad[1])
            return (gx, gd) + (None,) * 12
        gy = be.gemm_fused(1, g, W3, None, a, be.EPI_TANH_GRAD)        # through lin and the activation
        gagg = be.gemm(1, gy, W2)
        sel = plan.half_selection()
        gx = gd = None
        if ctx.needs_input_grad[0]:
            gxl = be.seg_mul_sum(gagg, W, plan.ptr_out, plan.nbr_out, plan.pair_index() if sel is not None else plan.perm_out, plan.N)
            gx = be.gemm_fused(1, gxl, W1, None, g, be.EPI_ADD)        # through lin1, plus the residual branch
        if ctx.needs_input_grad[1]:
            gd, status = be.filter_backward(d, ctx.spec, ctx.conv_cut[0], ctx.conv_cut[1], ctx.conv_cut[2], fA1, fb1, fA2, plan.row0, plan.row1,
                                            xl, gagg, ctx.precision, sel, plan.perm_in if sel is not None else None, hidden=ctx.hidden)
            be.defer_status(status, "fused filter network (backward)")
        return (gx, gd) + (None,) * 12


class SchNetEval(torch.autograd.Function):
    """Energies of a standard SchNet with d(sum E)/d(pos) worked out in the same library call (eval mode: the force pass
    always follows).  ``backward`` hands that gradient out, scaled per structure by the incoming gradient; it is not itself
    differentiable."""

    @staticmethod
    def forward(ctx, pos, types, struct_ptr, batch, plan: EdgePlan, spec: RbfSpec, conv_cut, weights, precision: int):
        energy, grad = get_backend().schnet_eval(pos.contiguous(), types, struct_ptr, plan, spec, conv_cut, weights, precision,
                                                 want_grad=ctx.needs_input_grad[0])
        if grad is not None:
            ctx.save_for_backward(grad, batch)
        return energy

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        grad, batch = ctx.saved_tensors
        return (grad * g.index_select(0, batch).unsqueeze(-1),) + (None,) * 8
