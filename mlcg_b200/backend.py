"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw pointers and the current stream.

Every operator of the package goes through the object returned by :func:`get_backend`.  The only
back end is :class:`CudaBackend`; it refuses tensors that are not on a CUDA device, and constructing it
raises if ``libmlcg_b200.so`` is missing.
"""
import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

_DT = {torch.float32: 0, torch.float64: 1}
STATUS_TRUNCATED, STATUS_BAD_INDEX, STATUS_ASYMMETRIC = 1, 2, 4


@dataclass(frozen=True)
class RbfSpec:
    """Host-side description of a radial basis x envelope (mirror of ``mlcgb_rbf_spec``)."""

    kind: int          # 0 Gaussian, 1 exp-normal
    num_rbf: int
    cutoff_kind: int   # 0 identity, 1 cosine
    lower: float
    upper: float
    alpha: float
    p0: torch.Tensor   # offsets | means
    p1: torch.Tensor   # coeff (1 element) | betas


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    """Raw handle of torch's current stream on the current device."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on(device):
    """Device guard for a launch: a real ``torch.cuda.device`` only when ``device`` is not the current one."""
    if device.index is None or device.index == torch._C._cuda_getDevice():
        return _NO_GUARD
    return torch.cuda.device(device)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mlcg_b200 operators run on CUDA tensors only (there is no CPU fallback)")


def _raise_for_status(word: int, what: str) -> None:
    """Status bits the tensor-core kernels set (read lazily, with the next unavoidable host read)."""
    if word & 8:
        raise RuntimeError(f"mlcg_b200: {what}: a tensor-core wait ran out; results are incomplete")
    if word & 32:
        raise RuntimeError(f"mlcg_b200: {what}: the radius graph has more edges than the fixed edge capacity; results are incomplete "
                           "(raise the capacity)")
    if word & 4:
        raise RuntimeError(f"mlcg_b200: {what}: the edge list is not symmetric (an edge without its reverse, e.g. after the neighbour "
                           "cap cut a list short)")
    if word & 16:
        raise RuntimeError(f"mlcg_b200: {what}: a weight is beyond the range of the fp16-pair tensor-core operands (|w| > 512); "
                           "set mlcg_b200.backend.get_backend().tensor_core_gemm = False to run these layers on the CUDA cores")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"mlcg_b200: unsupported dtype {t.dtype}; use float32 or float64") from None


class KernelProfiler:
    """Per-operator launch counts, device time (CUDA events on the launching stream) and algorithmic work.

    Attach with ``get_backend().profiler = KernelProfiler()``; ``summary()`` synchronises and returns
    ``{name: {"calls", "launches", "ms", "bytes", "flops"}}``."""

    def __init__(self, time_kernels: bool = True):
        self.time_kernels = time_kernels
        self.records = []      # (name, start_event, end_event)
        self.stats = {}

    def begin(self, name, launches, nbytes, flops):
        st = self.stats.setdefault(name, {"calls": 0, "launches": 0, "ms": 0.0, "bytes": 0, "flops": 0})
        st["calls"] += 1
        st["launches"] += launches
        st["bytes"] += int(nbytes)
        st["flops"] += int(flops)
        if not self.time_kernels:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def end(self, name, start):
        if start is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.records.append((name, start, ev))

    def summary(self):
        torch.cuda.synchronize()
        for name, a, b in self.records:
            self.stats[name]["ms"] += a.elapsed_time(b)
        self.records = []
        return self.stats

    @property
    def total_launches(self):
        return sum(v["launches"] for v in self.stats.values())


class CudaBackend:
    name = "cuda"

    def __init__(self):
        self.lib = _lib.load()
        self.profiler = None
        self._status = {}
        self.tensor_core_gemm = True   # float32 GEMMs of qualifying shape run on tcgen05 (fp32-equivalent products)
        self._pending = []      # (status tensor, what) of kernels whose status word has not been read yet

    def defer_status(self, status, what):
        """Remember a kernel's status word; it is read together with the next unavoidable host read (the edge
        count of the next radius graph) or by :meth:`check_pending`, so the hot path gains no synchronisation."""
        if not self._pending or (self._pending[-1][0] is not status and not any(s is status for s, _ in self._pending)):
            self._pending.append((status, what))
        if len(self._pending) > 256:
            self.check_pending()

    def check_pending(self):
        pending, self._pending = self._pending, []
        if not pending:
            return
        words = torch.stack([s[0] for s, _ in pending]).cpu().tolist()
        self._raise_pending(words, pending)

    @staticmethod
    def _raise_pending(words, pending):
        """Raise for the first status word that reports a failure; the words are cleared first, so one failure is reported
        once and later evaluations start clean."""
        bad = [(w, what) for w, (_, what) in zip(words, pending) if w & (4 | 8 | 16 | 32)]
        if bad:
            for st, _ in pending:
                st.zero_()
            _raise_for_status(*bad[0])

    # ------------------------------------------------------------------ device time per entry point
    def timeline_begin(self):
        """Start recording a CUDA event pair around every kernel-launching library call made from this thread."""
        _lib.check(self.lib.mlcgb_timeline_begin(), "timeline_begin")

    def timeline_end(self):
        """Stop recording, wait for the events and return ``{entry point: {"calls": n, "ms": total}}``."""
        n = self.lib.mlcgb_timeline_end()
        if n < 0:
            _lib.check(n, "timeline_end")
        out = {}
        name, calls, ms = ctypes.c_char_p(), ctypes.c_int64(), ctypes.c_double()
        for i in range(n):
            _lib.check(self.lib.mlcgb_timeline_entry(i, ctypes.byref(name), ctypes.byref(calls), ctypes.byref(ms)), "timeline_entry")
            out[name.value.decode()] = {"calls": int(calls.value), "ms": float(ms.value)}
        return out

    def _run(self, name, fn, args, what=None, launches=1, nbytes=0, flops=0):
        prof = self.profiler
        ev = prof.begin(name, launches, nbytes, flops) if prof is not None else None
        _lib.check(fn(*args), what or name)
        if prof is not None:
            prof.end(name, ev)

    def _work(self, name, v):
        """Algorithmic bytes / flops and kernel launches of one call (index tensors counted at their stored width); only
        worked out while a profiler is attached."""
        if self.profiler is None:
            return {}
        es = lambda t: t.element_size()
        if name == "radius_count":
            return dict(launches=5, nbytes=v["N"] * (12 + 4 + 8) + v["B"] * 8)
        if name == "radius_fill":
            return dict(launches=1, nbytes=16 * v["E"] + 20 * v["N"])       # [2,E] int64 written, pos + structure ids read
        if name == "seg_mul_sum":
            V, a = v["V"], v["a"]
            return dict(nbytes=V.numel() * es(V) + V.shape[0] * 4 + (a.numel() + v["N"] * v["F"]) * es(V) + v["N"] * 8,
                        flops=2 * V.numel())
        if name == "edge_mul":
            a = v["a"]
            return dict(nbytes=v["E"] * v["F"] * es(a) + v["E"] * 8 + 2 * a.numel() * es(a), flops=v["E"] * v["F"])
        if name == "gemm":
            A = v["A"]
            M, N, K = v["M"], v["N"], v["K"]
            return dict(launches=2 if v["wsb"] else 1, nbytes=(M * K + N * K + M * N) * es(A), flops=2 * M * N * K)
        if name in ("rbf_expand", "rbf_contract"):
            d = v["d"]
            R = v["spec"].num_rbf
            return dict(nbytes=d.numel() * es(d) * (R + 1 + (1 if name == "rbf_contract" else 0)), flops=d.numel() * R * 20)
        if name == "edge_diff":
            return dict(nbytes=v["E"] * (8 + 3 * es(v["pos"])) + v["pos"].numel() * es(v["pos"]))
        if name == "node_scatter_diff":
            g = v["g"]
            return dict(nbytes=2 * g.numel() * es(g) + g.shape[0] * 4 + v["N"] * (16 + 3 * es(g)))
        if name == "prior_terms":
            m = v["mapping"]
            return dict(nbytes=m.numel() * 8 + v["M"] * 8 + v["params"].numel() * es(v["params"]) + 2 * v["pos"].numel() * es(v["pos"]))
        return {}

    # ------------------------------------------------------------------ radius graph
    def batch_to_ptr(self, batch: torch.Tensor, B: int) -> torch.Tensor:
        _need_cuda(batch)
        batch = batch.contiguous()
        ptr = torch.empty(B + 1, dtype=torch.int64, device=batch.device)
        with _on(batch.device):
            self._run("batch_to_ptr", self.lib.mlcgb_batch_to_ptr, (_ptr(batch), batch.numel(), B, _ptr(ptr), _stream(),), **self._work("batch_to_ptr", locals()))
        return ptr

    def radius_graph(self, pos, ptr, r, max_num_neighbors, loop, rule, want_distance=False, want_batch=True, exclude=None):
        """Returns dict(edge_index[2,E] i64, distance|None, mapping_batch|None, row0, row1 (i32), offsets[N+1] i64, status int).
        ``exclude``: ``(exclude_pair_xs, ptr_exclude_pair_xs)`` int64 as ``mlcg::radius_cuda`` takes them (rule "native" only)."""
        _need_cuda(pos, ptr)
        if exclude is not None:
            if int(rule) != 0:
                raise ValueError("excluded pairs go with the neighbour cap of radius.cu (rule 0)")
            ex_xs, ex_ptr = (t.to(device=pos.device, dtype=torch.int64).contiguous() for t in exclude)
            if ex_ptr.numel() != pos.shape[0] + 1:
                raise ValueError("ptr_exclude_pair_xs must have one entry per point plus one")
        pos = pos.detach().contiguous()
        N, B, dev = pos.shape[0], ptr.numel() - 1, pos.device
        dt = _dt(pos)
        with _on(dev):
            ws_bytes = self.lib.mlcgb_radius_workspace_bytes(N, B, dt)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
            deg = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
            offsets = torch.empty(N + 1, dtype=torch.int64, device=dev)
            status = torch.zeros(4, dtype=torch.int32, device=dev)
            if exclude is None:
                self._run("radius_count", self.lib.mlcgb_radius_count, (_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(max_num_neighbors), int(loop), int(rule),
                                                       _ptr(ws), ws_bytes, _ptr(deg), _ptr(offsets), _ptr(status), _stream(),), **self._work("radius_count", locals()))
            else:
                self._run("radius_count", self.lib.mlcgb_radius_count_excl, (_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(max_num_neighbors), int(loop),
                                                       _ptr(ex_xs), _ptr(ex_ptr), _ptr(ws), ws_bytes, _ptr(deg), _ptr(offsets), _ptr(status), _stream(),),
                          **self._work("radius_count", locals()))
            pend, self._pending = self._pending, []
            extra = [s[0].to(torch.int64) for s, _ in pend]
            tail = torch.stack([offsets[N], status[0].to(torch.int64)] + extra).cpu().tolist()   # the one host read
            E, st = int(tail[0]), int(tail[1])
            self._raise_pending(tail[2:], pend)
            ei = torch.empty((2, E), dtype=torch.int64, device=dev)
            dist = torch.empty(E, dtype=pos.dtype, device=dev) if want_distance else None
            mb = torch.empty(E, dtype=torch.int64, device=dev) if want_batch else None
            r0 = torch.empty(E, dtype=torch.int32, device=dev)
            r1 = torch.empty(E, dtype=torch.int32, device=dev)
            if exclude is None:
                self._run("radius_fill", self.lib.mlcgb_radius_fill, (_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(loop), _ptr(ws), ws_bytes, _ptr(offsets), E,
                                                      _ptr(ei), _ptr(dist), _ptr(mb), _ptr(r0), _ptr(r1), _ptr(status), _stream(),), **self._work("radius_fill", locals()))
            else:
                self._run("radius_fill", self.lib.mlcgb_radius_fill_excl, (_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(loop), _ptr(ex_xs), _ptr(ex_ptr), _ptr(ws), ws_bytes,
                                                      _ptr(offsets), E, _ptr(ei), _ptr(dist), _ptr(mb), _ptr(r0), _ptr(r1), _ptr(status), _stream(),),
                          **self._work("radius_fill", locals()))
        return dict(edge_index=ei, distance=dist, mapping_batch=mb, row0=r0, row1=r1, offsets=offsets, status=st)

    def radius_graph_pbc(self, pos, ptr, cells, repeats, r, max_num_neighbors, loop, want_distance=False, want_batch=True):
        """Radius graph of periodic structures: dict(edge_index [2,E] i64 (row 0 = centre), cell_shifts [E,3], distance|None,
        mapping_batch|None, status int).  ``cells`` [B,3,3] in the dtype of ``pos``, ``repeats`` [B,3] copies per cell vector."""
        _need_cuda(pos, ptr, cells, repeats)
        pos = pos.detach().contiguous()
        cells = cells.detach().to(pos.dtype).contiguous()
        repeats = repeats.to(torch.int32).contiguous()
        N, B, dev = pos.shape[0], ptr.numel() - 1, pos.device
        if cells.numel() != 9 * B or repeats.numel() != 3 * B:
            raise ValueError("cells must be [B,3,3] and repeats [B,3]")
        dt = _dt(pos)
        with _on(dev):
            wsb = self.lib.mlcgb_radius_pbc_workspace_bytes(N)
            ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
            deg = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
            offsets = torch.empty(N + 1, dtype=torch.int64, device=dev)
            status = torch.zeros(4, dtype=torch.int32, device=dev)
            self._run("radius_pbc_count", self.lib.mlcgb_radius_pbc_count,
                      (_ptr(pos), dt, _ptr(ptr), N, B, _ptr(cells), _ptr(repeats), float(r), int(max_num_neighbors), int(loop), _ptr(ws), wsb,
                       _ptr(deg), _ptr(offsets), _ptr(status), _stream()), launches=5)
            E, st = (int(v) for v in torch.stack([offsets[N], status[0].to(torch.int64)]).cpu().tolist())
            ei = torch.empty((2, E), dtype=torch.int64, device=dev)
            shifts = torch.empty((E, 3), dtype=pos.dtype, device=dev)
            dist = torch.empty(E, dtype=pos.dtype, device=dev) if want_distance else None
            mb = torch.empty(E, dtype=torch.int64, device=dev) if want_batch else None
            self._run("radius_pbc_fill", self.lib.mlcgb_radius_pbc_fill,
                      (_ptr(pos), dt, _ptr(ptr), N, B, _ptr(cells), _ptr(repeats), float(r), int(max_num_neighbors), int(loop), _ptr(ws), wsb,
                       _ptr(offsets), E, _ptr(ei), _ptr(shifts), _ptr(dist), _ptr(mb), _ptr(status), _stream()), nbytes=E * (16 + 3 * pos.element_size()))
        return dict(edge_index=ei, cell_shifts=shifts, distance=dist, mapping_batch=mb, offsets=offsets, status=st)

    def radius_graph_capacity(self, pos, ptr, r, max_num_neighbors, capacity, rows=None, rule=1):
        """The radius graph into buffers of ``capacity`` edges without reading the edge count on the host:
        dict(row0, row1 (int32 [capacity]), offsets [N+1], counts (int64 [2] on the device: edges, edges / 2)).  ``rows``: an int32
        ``[2, capacity]`` buffer to reuse, whose entries are valid point indices (zeros at first).  An overflow sets bit 5 of the
        backend's accumulating status words (reported by :meth:`check_pending`)."""
        _need_cuda(pos, ptr)
        pos = pos.detach().contiguous()
        N, B, dev = pos.shape[0], ptr.numel() - 1, pos.device
        dt = _dt(pos)
        capacity = int(capacity)
        if capacity < 0 or capacity % 2:
            raise ValueError("capacity must be a non-negative even number of edges")
        if rows is None:
            rows = torch.zeros((2, capacity), dtype=torch.int32, device=dev)
        with _on(dev):
            ws_bytes = self.lib.mlcgb_radius_workspace_bytes(N, B, dt)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
            deg = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
            offsets = torch.empty(N + 1, dtype=torch.int64, device=dev)
            counts = torch.empty(2, dtype=torch.int64, device=dev)
            status = self._sticky_status(dev)
            self._run("radius_graph_capacity", self.lib.mlcgb_radius_graph_capacity,
                      (_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(max_num_neighbors), 0, int(rule), _ptr(ws), ws_bytes, _ptr(deg), _ptr(offsets),
                       capacity, None, _ptr(rows[0]), _ptr(rows[1]), _ptr(counts), _ptr(status), _stream()), launches=7, nbytes=N * 24 + capacity * 8)
        self.defer_status(status, "radius graph with a fixed edge capacity")
        return dict(row0=rows[0], row1=rows[1], offsets=offsets, counts=counts)

    def edge_twin(self, row0, row1, offsets, N, fresh_status: bool = False):
        """twin[e] = position of the reversed edge; second value: the status words (bit 2: an edge without its reverse).  By default
        the words are the backend's accumulating ones; ``fresh_status=True`` gives this call its own."""
        _need_cuda(row0)
        E = row0.numel()
        twin = torch.empty(E, dtype=torch.int32, device=row0.device)
        status = torch.zeros(4, dtype=torch.int32, device=row0.device) if fresh_status else self._sticky_status(row0.device)
        with _on(row0.device):
            self._run("edge_twin", self.lib.mlcgb_edge_twin, (_ptr(row0), _ptr(row1), _ptr(offsets), E, N, _ptr(twin), _ptr(status), _stream(),), **self._work("edge_twin", locals()))
        return twin, status

    def pair_plan(self, row0, row1, offsets, N, fresh_status: bool = False):
        """(twin [E], sel [E/2], pair_of [E], status words) of a symmetric, loop-free, centre-sorted list with an even number of
        edges; status bit 2: a missing reverse edge or a loop."""
        _need_cuda(row0)
        E, dev = row0.numel(), row0.device
        out = torch.zeros(2 * E + E // 2, dtype=torch.int32, device=dev)    # (entries no edge claims stay valid indices)
        twin, pair_of, sel = out[:E], out[E:2 * E], out[2 * E:]
        wsb = self.lib.mlcgb_pair_plan_workspace_bytes(N)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev) if fresh_status else self._sticky_status(dev)
        with _on(dev):
            self._run("pair_plan", self.lib.mlcgb_pair_plan, (_ptr(row0), _ptr(row1), _ptr(offsets), E, N, _ptr(ws), wsb, _ptr(twin), _ptr(sel), _ptr(pair_of),
                                                               _ptr(status), _stream()), launches=5, nbytes=28 * E + 20 * N)
        return twin, sel, pair_of, status

    def pair_index(self, sel, twin):
        """pair_of[e] = k for the k-th selected edge and for its reverse."""
        _need_cuda(sel, twin)
        pair_of = torch.empty(twin.numel(), dtype=torch.int32, device=twin.device)
        with _on(twin.device):
            self._run("pair_index", self.lib.mlcgb_pair_index, (_ptr(sel), _ptr(twin), sel.numel(), _ptr(pair_of), _stream(),), nbytes=12 * sel.numel())
        return pair_of

    # ------------------------------------------------------------------ geometry
    def edge_diff(self, pos, row0, row1):
        _need_cuda(pos, row0, row1)
        pos = pos.contiguous()
        E = row0.numel()
        out = torch.empty((E, 3), dtype=pos.dtype, device=pos.device)
        status = torch.zeros(4, dtype=torch.int32, device=pos.device)
        with _on(pos.device):
            self._run("edge_diff", self.lib.mlcgb_edge_diff, (_ptr(pos), _dt(pos), _ptr(row0), _ptr(row1), E, pos.shape[0], _ptr(out), _ptr(status), _stream(),), **self._work("edge_diff", locals()))
        return out

    def _sticky_status(self, dev):
        """One status array per device for kernels whose status is only ever checked lazily (bits accumulate)."""
        st = self._status.get(dev)
        if st is None:
            st = self._status[dev] = torch.zeros(4, dtype=torch.int32, device=dev)
        return st

    def edge_distance(self, pos, row0, row1):
        _need_cuda(pos, row0, row1)
        pos = pos.contiguous()
        E = row0.numel()
        out = torch.empty(E, dtype=pos.dtype, device=pos.device)
        with _on(pos.device):
            self._run("edge_distance", self.lib.mlcgb_edge_distance,
                      (_ptr(pos), _dt(pos), _ptr(row0), _ptr(row1), E, pos.shape[0], _ptr(out), _ptr(self._sticky_status(pos.device)), _stream()),
                      nbytes=E * (8 + pos.element_size()) + pos.numel() * pos.element_size())
        return out

    def edge_distance_backward(self, pos, g, d, plan):
        _need_cuda(pos, g, d)
        pos, g, d = pos.contiguous(), g.contiguous(), d.contiguous()
        out = torch.empty_like(pos)
        with _on(pos.device):
            self._run("edge_distance_backward", self.lib.mlcgb_edge_distance_backward,
                      (_ptr(pos), _ptr(g), _ptr(d), _dt(pos), _ptr(plan.row0), _ptr(plan.row1), _ptr(plan.ptr_in), _ptr(plan.perm_in),
                       _ptr(plan.ptr_out), _ptr(plan.perm_out), plan.N, plan.E, _ptr(out), _stream()),
                      nbytes=2 * plan.E * (16 + 2 * pos.element_size()) + 2 * pos.numel() * pos.element_size())
        return out

    def node_scatter_diff(self, g, ptr_in, perm_in, ptr_out, perm_out, N):
        _need_cuda(g)
        g = g.contiguous()
        out = torch.empty((N, 3), dtype=g.dtype, device=g.device)
        with _on(g.device):
            self._run("node_scatter_diff", self.lib.mlcgb_node_scatter_diff, (_ptr(g), _dt(g), _ptr(ptr_in), _ptr(perm_in), _ptr(ptr_out), _ptr(perm_out), N,
                                                        g.shape[0], _ptr(out), _stream(),), **self._work("node_scatter_diff", locals()))
        return out

    # ------------------------------------------------------------------ radial basis
    def _spec(self, spec: RbfSpec, dtype):
        p0 = spec.p0.detach().to(dtype).contiguous()
        p1 = spec.p1.detach().to(dtype).reshape(-1).contiguous()
        s = _lib.RbfSpecStruct(spec.kind, spec.num_rbf, spec.cutoff_kind, 0, spec.lower, spec.upper, spec.alpha, p0.data_ptr(), p1.data_ptr())
        return s, (p0, p1)

    def rbf_expand(self, d, spec: RbfSpec, order: int):
        _need_cuda(d, spec.p0, spec.p1)
        d = d.contiguous()
        s, keep = self._spec(spec, d.dtype)
        out = torch.empty((d.numel(), spec.num_rbf), dtype=d.dtype, device=d.device)
        with _on(d.device):
            self._run("rbf_expand", self.lib.mlcgb_rbf_expand, (_ptr(d), _dt(d), d.numel(), ctypes.byref(s), order, _ptr(out), _stream(),), **self._work("rbf_expand", locals()))
        return out

    def rbf_contract(self, d, G, spec: RbfSpec, order: int):
        _need_cuda(d, G, spec.p0, spec.p1)
        d, G = d.contiguous(), G.contiguous()
        s, keep = self._spec(spec, d.dtype)
        out = torch.empty(d.numel(), dtype=d.dtype, device=d.device)
        with _on(d.device):
            self._run("rbf_contract", self.lib.mlcgb_rbf_contract, (_ptr(d), _ptr(G), _dt(d), d.numel(), ctypes.byref(s), order, _ptr(out), _stream(),), **self._work("rbf_contract", locals()))
        return out

    def rbf_param_contract(self, d, G, c, spec: RbfSpec, order: int):
        """``(gp0 [R], gp1 [R] or [1])``: gradients with respect to the two parameter vectors of the basis of
        ``sum_e c[e] sum_k G[e,k] phi_k^(order)(d_e)`` (``c`` may be ``None``)."""
        _need_cuda(d, G, c, spec.p0, spec.p1)
        d, G = d.contiguous(), G.contiguous()
        c = None if c is None else c.contiguous()
        s, keep = self._spec(spec, d.dtype)
        gp0 = torch.empty(spec.num_rbf, dtype=d.dtype, device=d.device)
        gp1 = torch.empty(spec.p1.numel(), dtype=d.dtype, device=d.device)
        nbytes = self.lib.mlcgb_rbf_param_workspace_bytes(d.numel(), spec.num_rbf, _dt(d))
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=d.device)
        with _on(d.device):
            self._run("rbf_param_contract", self.lib.mlcgb_rbf_param_contract,
                      (_ptr(d), _ptr(G), _ptr(c), _dt(d), d.numel(), ctypes.byref(s), order, _ptr(ws), nbytes, _ptr(gp0), _ptr(gp1), _stream(),),
                      **self._work("rbf_param_contract", locals()))
        return gp0, gp1

    # ------------------------------------------------------------------ CFConv primitives
    def seg_mul_sum(self, a, V, ptr, nbr, eperm, N):
        _need_cuda(a, V, ptr, nbr)
        a, V = a.contiguous(), V.contiguous()
        F = V.shape[1]
        out = torch.empty((N, F), dtype=V.dtype, device=V.device)
        with _on(V.device):
            self._run("seg_mul_sum", self.lib.mlcgb_seg_mul_sum, (_ptr(a), _ptr(V), _dt(V), _ptr(ptr), _ptr(nbr), _ptr(eperm), N, V.shape[0], F, _ptr(out), _stream(),), **self._work("seg_mul_sum", locals()))
        return out

    def edge_mul(self, a, b, ia, ib):
        _need_cuda(a, b, ia, ib)
        a, b = a.contiguous(), b.contiguous()
        E, F = ia.numel(), a.shape[1]
        out = torch.empty((E, F), dtype=a.dtype, device=a.device)
        with _on(a.device):
            self._run("edge_mul", self.lib.mlcgb_edge_mul, (_ptr(a), _ptr(b), _dt(a), _ptr(ia), _ptr(ib), E, F, _ptr(out), _stream(),), **self._work("edge_mul", locals()))
        return out

    def pair_mul(self, a, b, ia, ib):
        """out[p,:] = a[ia[p],:] * b[ib[p],:] + a[ib[p],:] * b[ia[p],:]."""
        _need_cuda(a, b, ia, ib)
        a, b = a.contiguous(), b.contiguous()
        E, F = ia.numel(), a.shape[1]
        out = torch.empty((E, F), dtype=a.dtype, device=a.device)
        with _on(a.device):
            self._run("pair_mul", self.lib.mlcgb_pair_mul, (_ptr(a), _ptr(b), _dt(a), _ptr(ia), _ptr(ib), E, F, _ptr(out), _stream(),), **self._work("edge_mul", locals()))
        return out

    def tanh_grad(self, mode: int, G, g, y):
        """mode 0: ``g * (1 - y**2)``; mode 1: ``-2 * G * g * y`` (elementwise; ``G`` is ignored in mode 0)."""
        _need_cuda(G, g, y)
        g, y = g.contiguous(), y.contiguous()
        G = None if G is None else G.contiguous()
        out = torch.empty_like(y)
        with _on(y.device):
            self._run("tanh_grad", self.lib.mlcgb_tanh_grad, (int(mode), _ptr(G), _ptr(g), _ptr(y), _dt(y), y.numel(), _ptr(out), _stream(),),
                      nbytes=(3 + mode) * y.numel() * y.element_size(), flops=(3 + mode) * y.numel())
        return out

    def row_scale(self, a, c):
        """out[e,:] = a[e,:] * c[e]."""
        _need_cuda(a, c)
        a, c = a.contiguous(), c.contiguous()
        E, F = a.shape
        out = torch.empty_like(a)
        with _on(a.device):
            self._run("row_scale", self.lib.mlcgb_row_scale, (_ptr(a), _ptr(c), _dt(a), E, F, _ptr(out), _stream(),), nbytes=(2 * a.numel() + E) * a.element_size())
        return out

    def row_dot(self, a, b):
        """out[e] = sum_f a[e,f] * b[e,f]."""
        _need_cuda(a, b)
        a, b = a.contiguous(), b.contiguous()
        E, F = a.shape
        out = torch.empty(E, dtype=a.dtype, device=a.device)
        with _on(a.device):
            self._run("row_dot", self.lib.mlcgb_row_dot, (_ptr(a), _ptr(b), _dt(a), E, F, _ptr(out), _stream(),), nbytes=(2 * a.numel() + E) * a.element_size(),
                      flops=2 * a.numel())
        return out

    # ------------------------------------------------------------------ GEMM
    def gemm(self, mode: int, A, B, bias=None):
        """mode 0: A[M,K] B[N,K]^T (+bias); 1: A[M,K] B[K,N]; 2: A[K,M]^T B[K,N]."""
        _need_cuda(A, B, bias)
        A, B = A.contiguous(), B.contiguous()
        if mode == 0:
            (M, K), N = A.shape, B.shape[0]
        elif mode == 1:
            (M, K), N = A.shape, B.shape[1]
        else:
            (K, M), N = A.shape, B.shape[1]
        dt = _dt(A)
        C = torch.empty((M, N), dtype=A.dtype, device=A.device)
        tc_ok = (N <= 128 and K <= 128) if mode != 2 else (M <= 128 and N <= 128)      # what mlcgb_gemm_tc_supported tests
        if self.tensor_core_gemm and dt == 0 and min(M, N, K) > 0 and tc_ok:
            with _on(A.device):
                wsb = self.lib.mlcgb_gemm_tc_workspace_bytes(mode, M, N, K) if mode == 2 else 0
                ws = torch.empty(wsb, dtype=torch.uint8, device=A.device) if wsb else None
                if bias is not None:
                    bias = bias.contiguous()
                status = self._sticky_status(A.device)
                self._run("gemm_tc", self.lib.mlcgb_gemm_tc, (mode, _ptr(A), _ptr(B), _ptr(bias), M, N, K, _ptr(C), _ptr(ws), wsb, _ptr(status), _stream()),
                          launches=2 if wsb else 1, nbytes=(M * K + N * K + M * N) * 4, flops=2 * M * N * K)
                self.defer_status(status, "tensor-core GEMM")
            return C
        with _on(A.device):
            wsb = self.lib.mlcgb_gemm_workspace_bytes(mode, M, N, K, dt)
            ws = torch.empty(wsb, dtype=torch.uint8, device=A.device) if wsb else None
            if bias is not None:
                bias = bias.contiguous()
            self._run("gemm", self.lib.mlcgb_gemm, (mode, _ptr(A), _ptr(B), _ptr(bias), dt, M, N, K, _ptr(C), _ptr(ws), wsb, _stream(),), **self._work("gemm", locals()))
        return C

    def gemm_tn_colsum(self, G, X):
        """(G^T X, column sums of G): weight and bias gradient of a Linear layer in one pass over G (contraction over rows)."""
        _need_cuda(G, X)
        G, X = G.contiguous(), X.contiguous()
        (K, M), N = G.shape, X.shape[1]
        if (self.tensor_core_gemm and G.dtype == torch.float32 and min(M, N, K) > 0 and N % 4 == 0 and X.data_ptr() % 16 == 0
                and self.lib.mlcgb_gemm_tc_supported(2, M, N, K)):
            C = torch.empty((M, N), dtype=G.dtype, device=G.device)
            cs = torch.empty(M, dtype=G.dtype, device=G.device)
            with _on(G.device):
                wsb = self.lib.mlcgb_gemm_tc_workspace_bytes(2, M, N, K)
                ws = torch.empty(wsb, dtype=torch.uint8, device=G.device)
                status = self._sticky_status(G.device)
                self._run("gemm_tc", self.lib.mlcgb_gemm_tc_tn_colsum, (_ptr(G), _ptr(X), K, M, N, _ptr(C), _ptr(cs), _ptr(ws), wsb, _ptr(status), _stream()),
                          launches=3, nbytes=(M * K + N * K + M * N) * 4, flops=2 * M * N * K)
                self.defer_status(status, "tensor-core GEMM")
            return C, cs
        return self.gemm(2, G, X), G.sum(0)

    EPI_NONE, EPI_TANH, EPI_ADD, EPI_TANH_GRAD, EPI_IN_TANH_GRAD_VEC = 0, 1, 2, 3, 4

    def gemm_fused_ok(self, mode: int, A, B) -> bool:
        """Whether :meth:`gemm_fused` takes these operands (float32, >= 128 rows, widths multiples of four and <= 128)."""
        if not (self.tensor_core_gemm and A.is_cuda and A.dtype == torch.float32 and A.dim() == 2 and B.dim() == 2):
            return False
        M, K = A.shape
        N = B.shape[0] if mode == 0 else B.shape[1]
        return M >= 128 and K % 4 == 0 and N % 4 == 0 and N <= 128 and K <= 128

    def gemm_fused(self, mode: int, A, B, bias=None, aux=None, epilogue: int = 0):
        """Row-wise tensor-core GEMM (mode 0: A B^T + bias, mode 1: A B) with the elementwise step that follows it:
        1 tanh, 2 ``+ aux``, 3 ``* (1 - aux**2)``; 4 transforms the input instead: ``A <- aux[None, :] * (1 - A**2)`` with a
        vector ``aux`` over the columns of A."""
        _need_cuda(A, B, bias, aux)
        A, B = A.contiguous(), B.detach().contiguous()
        M, K = A.shape
        N = B.shape[0] if mode == 0 else B.shape[1]
        C = torch.empty((M, N), dtype=A.dtype, device=A.device)
        if bias is not None:
            bias = bias.detach().contiguous()
        if aux is not None:
            aux = aux.contiguous()
        status = self._sticky_status(A.device)
        with _on(A.device):
            self._run("gemm_tc", self.lib.mlcgb_gemm_tc_fused, (mode, _ptr(A), _ptr(B), _ptr(bias), _ptr(aux), int(epilogue), M, N, K, _ptr(C), _ptr(status), _stream()),
                      nbytes=(M * K + N * K + M * N * (2 if aux is not None else 1)) * 4, flops=2 * M * N * K)
        self.defer_status(status, "tensor-core GEMM")
        return C

    def gemm_chain2(self, backward: bool, A, Wa, ba, Wb, bb, aux):
        """Two 128-wide layers in one kernel.  Forward: ``mid = tanh(A Wa^T + ba)``, ``C = aux + mid Wb^T + bb`` -> ``(mid, C)``;
        backward: ``C = ((A Wa) * (1 - aux**2)) Wb`` -> ``(None, C)``."""
        _need_cuda(A, Wa, ba, Wb, bb, aux)
        A, aux = A.contiguous(), aux.contiguous()
        Wa, Wb = Wa.detach().contiguous(), Wb.detach().contiguous()
        ba = None if ba is None else ba.detach().contiguous()
        bb = None if bb is None else bb.detach().contiguous()
        if A.dtype != torch.float32 or A.shape[1] != 128 or tuple(Wa.shape) != (128, 128) or tuple(Wb.shape) != (128, 128) or aux.shape != A.shape:
            raise ValueError("gemm_chain2 takes float32 operands of width 128")
        M = A.shape[0]
        mid = None if backward else torch.empty_like(A)
        C = torch.empty_like(A)
        status = self._sticky_status(A.device)
        with _on(A.device):
            self._run("gemm_tc", self.lib.mlcgb_gemm_tc_chain2, (int(bool(backward)), _ptr(A), _ptr(Wa), _ptr(ba), _ptr(Wb), _ptr(bb), _ptr(aux), M, _ptr(mid), _ptr(C),
                                                                   _ptr(status), _stream()),
                      nbytes=(3 if backward else 4) * M * 128 * 4 + 2 * 128 * 128 * 4, flops=4 * M * 128 * 128)
        self.defer_status(status, "tensor-core GEMM")
        return mid, C

    # ------------------------------------------------------------------ one interaction block per call
    def interaction_ok(self, x, plan, H, F, H2) -> bool:
        """Whether the per-block entry points take this case; with a profiler attached the individual kernels are launched
        instead, so that each is timed on its own."""
        return (self.profiler is None and self.tensor_core_gemm and x.dtype == torch.float32 and x.shape[0] >= 128 and F == 128
                and H <= 128 and H2 <= 128 and H % 4 == 0 and H2 % 4 == 0 and plan.half_selection() is not None)

    def interaction_forward(self, x, d, plan, spec: RbfSpec, conv_cut, W1, fA1, fb1, fA2, W2, b2, W3, b3, precision, save_hidden=True):
        """x + lin(tanh(lin2(aggregate(lin1(x), W(d))))) in one library call; returns (x_new, xl, Wp, a, hs) with ``hs`` the
        filter network's hidden layer kept for the backward (None when ``save_hidden`` is off: the backward recomputes it)."""
        N, H = x.shape
        W1, fA1, fb1, fA2, W2, b2, W3, b3 = (t.contiguous() for t in (W1, fA1, fb1, fA2, W2, b2, W3, b3))
        F, H2 = W1.shape[0], W2.shape[0]
        sel, pair_of = plan.half_selection(), plan.pair_index()
        P, dev = sel.numel(), x.device
        s, keep = self._spec(spec, torch.float32)
        new = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        xl, Wp, agg, a, out = new(N, F), new(P, F), new(N, F), new(N, H2), new(N, H)
        hs = new(self.lib.mlcgb_filter_hidden_bytes(P) // 4) if save_hidden else None
        status = self._sticky_status(dev)
        with _on(dev):
            _lib.check(self.lib.mlcgb_interaction_forward(
                _ptr(x), _ptr(d), _ptr(plan.ptr_out), _ptr(plan.nbr_out), _ptr(sel), _ptr(pair_of), ctypes.byref(s), int(conv_cut[0]),
                float(conv_cut[1]), float(conv_cut[2]), _ptr(W1), _ptr(fA1), _ptr(fb1), _ptr(fA2), _ptr(W2), _ptr(b2), _ptr(W3), _ptr(b3),
                N, plan.E, P, H, F, H2, int(precision), _ptr(xl), _ptr(Wp), _ptr(hs), _ptr(agg), _ptr(a), _ptr(out), _ptr(status), _stream()),
                "interaction_forward")
        self.defer_status(status, "interaction block (forward)")
        return out, xl, Wp, a, hs

    def interaction_backward(self, g, a, Wp, xl, hs, d, plan, spec: RbfSpec, conv_cut, W1, fA1, fb1, fA2, W2, W3, precision, want_gx=True, want_gd=True):
        N, H = g.shape
        W1, fA1, fb1, fA2, W2, W3 = (t.contiguous() for t in (W1, fA1, fb1, fA2, W2, W3))
        F, H2 = W1.shape[0], W2.shape[0]
        sel, pair_of = plan.half_selection(), plan.pair_index()
        P, dev = sel.numel(), g.device
        s, keep = self._spec(spec, torch.float32)
        new = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        gy, gagg, gxl = new(N, H2), new(N, F), new(N, F)
        gx = new(N, H) if want_gx else None
        gd = new(plan.E) if want_gd else None
        status = self._sticky_status(dev)
        with _on(dev):
            _lib.check(self.lib.mlcgb_interaction_backward(
                _ptr(g), _ptr(a), _ptr(Wp), _ptr(xl), _ptr(hs), _ptr(d), _ptr(plan.ptr_out), _ptr(plan.nbr_out), _ptr(sel), _ptr(pair_of),
                _ptr(plan.perm_in), _ptr(plan.row0), _ptr(plan.row1), ctypes.byref(s), int(conv_cut[0]), float(conv_cut[1]), float(conv_cut[2]),
                _ptr(W1), _ptr(fA1), _ptr(fb1), _ptr(fA2), _ptr(W2), _ptr(W3), N, plan.E, P, H, F, H2, int(precision),
                _ptr(gy), _ptr(gagg), _ptr(gxl), _ptr(gx), _ptr(gd), _ptr(status), _stream()),
                "interaction_backward")
        self.defer_status(status, "interaction block (backward)")
        return gx, gd

    def schnet_eval(self, pos, types, struct_ptr, plan, spec: RbfSpec, conv_cut, weights, precision, want_grad=True, counts=None):
        """Energies [B] and d(sum of energies)/d(pos) [N,3] of a standard SchNet in one library call.  ``weights`` is what
        :func:`mlcg_b200.nn.schnet.packed_weights` returns: ``(SchnetWeightsStruct, keep-alive objects)``.  ``counts``: the
        device-side (edges, pairs) of a fixed-capacity graph, whose plan is sized by the capacity."""
        wstruct, _keep = weights
        N, dev = pos.shape[0], pos.device
        B = struct_ptr.numel() - 1
        sel, pair_of = plan.half_selection(), plan.pair_index()
        P = sel.numel()
        s, keep = self._spec(spec, torch.float32)
        wsb = self.lib.mlcgb_schnet_eval_workspace_bytes(N, plan.E, P, wstruct.hidden, wstruct.filters, wstruct.conv_out, wstruct.head_width,
                                                         wstruct.num_blocks)
        ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
        energy = torch.empty(B, dtype=torch.float32, device=dev)
        grad = torch.empty((N, 3), dtype=torch.float32, device=dev) if want_grad else None
        status = self._sticky_status(dev)
        with _on(dev):
            _lib.check(self.lib.mlcgb_schnet_eval_counted(
                _ptr(pos), _ptr(types), _ptr(struct_ptr), N, B, _ptr(plan.row0), _ptr(plan.row1), _ptr(plan.ptr_out), _ptr(sel), _ptr(pair_of),
                _ptr(plan.perm_in), plan.E, P, _ptr(counts), ctypes.byref(s), int(conv_cut[0]), float(conv_cut[1]), float(conv_cut[2]), ctypes.byref(wstruct),
                int(precision), _ptr(ws), wsb, _ptr(energy), _ptr(grad), _ptr(status), _stream()), "schnet_eval")
        self.defer_status(status, "SchNet evaluation")
        return energy, grad

    # ------------------------------------------------------------------ fused filter network (tensor cores)
    def filter_forward(self, d, spec: RbfSpec, conv_cutoff_kind, conv_lower, conv_upper, A1, b1, A2, precision=0, sel=None, twin=None, save_hidden=False):
        """W[E,F] = (tanh(phi(d) A1^T + b1) A2^T) * C(d); float32, F = 128, R <= 128.
        ``sel`` / ``twin``: compute one row per unordered pair and write it to both edges (symmetric edge lists);
        ``sel`` alone: W has one row per selected edge, in the order of ``sel``.
        Returns ``(W, status)``, or ``(W, status, hidden)`` with ``save_hidden``: the first layer's output kept (in the kernels'
        own order) for :meth:`filter_backward`."""
        _need_cuda(d, A1, b1, A2, spec.p0, spec.p1)
        if d.dtype != torch.float32:
            raise TypeError("filter_forward is a float32 kernel")
        d, A1, b1, A2 = d.contiguous(), A1.detach().contiguous(), b1.detach().contiguous(), A2.detach().contiguous()
        s, keep = self._spec(spec, d.dtype)
        E, F = d.numel(), A2.shape[0]
        rows = E if sel is None else sel.numel()
        W = torch.empty((E if (sel is None or twin is not None) else rows, F), dtype=d.dtype, device=d.device)
        hs = torch.empty(self.lib.mlcgb_filter_hidden_bytes(rows) // 4, dtype=torch.float32, device=d.device) if save_hidden else None
        status = self._sticky_status(d.device)
        with _on(d.device):
            self._run("filter_forward", self.lib.mlcgb_filter_forward,
                      (_ptr(d), rows, _ptr(sel), _ptr(twin), ctypes.byref(s), int(conv_cutoff_kind), float(conv_lower), float(conv_upper), _ptr(A1), _ptr(b1), _ptr(A2), F,
                       int(precision), _ptr(W), _ptr(hs), _ptr(status), _stream()),
                      nbytes=W.shape[0] * 4 * F + 4 * rows + (hs.numel() * 4 if save_hidden else 0), flops=2 * rows * F * (spec.num_rbf + F))
        return (W, status, hs) if save_hidden else (W, status)

    def filter_backward(self, d, spec: RbfSpec, conv_cutoff_kind, conv_lower, conv_upper, A1, b1, A2, row0, row1, xl, gagg, precision=0,
                        sel=None, twin=None, hidden=None):
        """gd[E] = sum_f (xl[row0] * gagg[row1])_f * dW_f/dd.  ``hidden``: what :meth:`filter_forward` kept for the same
        distances, selection and weights (the hidden layer is recomputed without it)."""
        _need_cuda(d, A1, b1, A2, row0, row1, xl, gagg)
        d, A1, b1, A2 = d.contiguous(), A1.detach().contiguous(), b1.detach().contiguous(), A2.detach().contiguous()
        xl, gagg = xl.detach().contiguous(), gagg.detach().contiguous()
        s, keep = self._spec(spec, d.dtype)
        E, F = d.numel(), A2.shape[0]
        rows = E if sel is None else sel.numel()
        gd = torch.empty(E, dtype=d.dtype, device=d.device)
        status = self._sticky_status(d.device)
        with _on(d.device):
            self._run("filter_backward", self.lib.mlcgb_filter_backward,
                      (_ptr(d), rows, _ptr(sel), _ptr(twin), ctypes.byref(s), int(conv_cutoff_kind), float(conv_lower), float(conv_upper), _ptr(A1), _ptr(b1), _ptr(A2), F,
                       int(precision), _ptr(row0), _ptr(row1), _ptr(xl), _ptr(gagg), xl.shape[0], _ptr(hidden), _ptr(gd), _ptr(status), _stream()),
                      nbytes=E * 16 + 2 * xl.numel() * 4 + (hidden.numel() * 4 if hidden is not None else 0), flops=2 * rows * F * 2 * (spec.num_rbf + F))
        return gd, status

    def segment_sum(self, x, ptr):
        _need_cuda(x, ptr)
        x = x.contiguous()
        B = ptr.numel() - 1
        out = torch.empty(B, dtype=x.dtype, device=x.device)
        with _on(x.device):
            self._run("segment_sum", self.lib.mlcgb_segment_sum, (_ptr(x), _dt(x), _ptr(ptr), B, _ptr(out), _stream(),), **self._work("segment_sum", locals()))
        return out

    # ------------------------------------------------------------------ Langevin integrator
    def langevin_first_half(self, x, v, f, masses, beta_mass_ratio, noise, dt, vscale, noisescale):
        """In place on x and v (both contiguous [N,3])."""
        _need_cuda(x, v, f, masses, beta_mass_ratio, noise)
        assert x.is_contiguous() and v.is_contiguous()
        f, noise = f.contiguous(), noise.contiguous()
        with _on(x.device):
            self._run("langevin_first_half", self.lib.mlcgb_langevin_first_half,
                      (_ptr(x), _ptr(v), _ptr(f), _ptr(masses), _ptr(beta_mass_ratio), _ptr(noise), _dt(x), x.shape[0], float(dt), float(vscale),
                       float(noisescale), _stream()), nbytes=6 * x.numel() * x.element_size())

    def langevin_second_half(self, v, f, masses, dt):
        _need_cuda(v, f, masses)
        assert v.is_contiguous()
        f = f.contiguous()
        with _on(v.device):
            self._run("langevin_second_half", self.lib.mlcgb_langevin_second_half, (_ptr(v), _ptr(f), _ptr(masses), _dt(v), v.shape[0], float(dt), _stream()),
                      nbytes=3 * v.numel() * v.element_size())

    # ------------------------------------------------------------------ priors
    def prior_terms(self, kind, pos, mapping, mapping_batch, params, B, want_grad=True):
        """Returns (energy[B], dE/dpos[N,3] | None)."""
        _need_cuda(pos, mapping, mapping_batch, params)
        pos, mapping, mapping_batch, params = pos.detach().contiguous(), mapping.contiguous(), mapping_batch.contiguous(), params.contiguous()
        M, N = mapping.shape[1], pos.shape[0]
        # the kernel accumulates: one zero-filled buffer holds the gradient (first, so that it stays 16-byte aligned) and the energies
        buf = torch.zeros(3 * N + B if want_grad else B, dtype=pos.dtype, device=pos.device)
        grad = buf[:3 * N].view(N, 3) if want_grad else None
        energy = buf[3 * N:] if want_grad else buf
        status = self._sticky_status(pos.device)       # (bit 1: a term with an index out of range was skipped)
        with _on(pos.device):
            self._run("prior_terms", self.lib.mlcgb_prior_terms, (kind, _ptr(pos), _dt(pos), _ptr(mapping), _ptr(mapping_batch), _ptr(params), params.shape[0], M, N, B,
                                                  _ptr(energy), _ptr(grad), _ptr(status), _stream(),), **self._work("prior_terms", locals()))
        return energy, grad


    def prior_eval(self, lists, pos, struct_of, B, deterministic=True):
        """Every prior list of a model in one launch.  ``lists``: sequence of ``(kind, idx32 [order, M], params [P, M], symmetric,
        run_ptr | None)`` (at most ``_lib.MAX_PRIOR_SEGMENTS``; ``run_ptr`` int64: runs of equal first bead of a symmetric pair list).  Returns ``(energy [n, B], dE/dpos [n, N, 3])``, one row / block per list.
        ``deterministic``: sums formed as 64-bit fixed-point integers (bit-identical from run to run)."""
        _need_cuda(pos, struct_of)
        n = len(lists)
        if n == 0 or n > _lib.MAX_PRIOR_SEGMENTS:
            raise ValueError(f"between 1 and {_lib.MAX_PRIOR_SEGMENTS} prior lists per launch")
        pos = pos.detach().contiguous()
        N, dev = pos.shape[0], pos.device
        arr = (_lib.PriorListStruct * n)()
        keep = []
        for k, (kind, idx, params, symmetric, run_ptr) in enumerate(lists):
            _need_cuda(idx, params, run_ptr)
            if idx.dtype != torch.int32 or params.dtype != pos.dtype or (run_ptr is not None and run_ptr.dtype != torch.int64):
                raise TypeError("prior lists take int32 indices, int64 run pointers and parameters of the positions' dtype")
            idx, params = idx.contiguous(), params.contiguous()
            run_ptr = None if run_ptr is None else run_ptr.contiguous()
            keep += [idx, params, run_ptr]
            arr[k] = _lib.PriorListStruct(int(kind), int(params.shape[0]), int(bool(symmetric)), 0, int(idx.shape[1]), idx.data_ptr(), params.data_ptr(),
                                          _ptr(run_ptr), 0 if run_ptr is None else run_ptr.numel() - 1)
        fixed = 1 if deterministic else 0
        make = torch.empty if fixed else torch.zeros               # (the fixed-point mode writes its outputs, the other adds to them)
        buf = make(n * (3 * N + B), dtype=pos.dtype, device=dev)
        grad, energy = buf[: n * 3 * N].view(n, N, 3), buf[n * 3 * N:].view(n, B)
        status = self._sticky_status(dev)
        with _on(dev):
            wsb = self.lib.mlcgb_prior_eval_workspace_bytes(n, N, B, fixed)
            ws = torch.empty(wsb, dtype=torch.uint8, device=dev) if wsb else None
            M_total = sum(int(l[1].shape[1]) for l in lists)
            self._run("prior_eval", self.lib.mlcgb_prior_eval,
                      (n, arr, _ptr(pos), _dt(pos), _ptr(struct_of), N, B, _ptr(energy), _ptr(grad), fixed, _ptr(ws), wsb, _ptr(status), _stream()),
                      launches=3 if fixed else 1, nbytes=sum(l[1].numel() * 4 + l[2].numel() * pos.element_size() for l in lists) + 2 * pos.numel() * pos.element_size(),
                      flops=40 * M_total)
        return energy, grad


_backend = None


def get_backend():
    global _backend
    if _backend is None:
        _backend = CudaBackend()   # raises ExtensionMissing if the library is absent
    return _backend
