"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw pointers and the current stream.

Every operator of the package goes through the object returned by :func:`get_backend`.  The only
back end shipped is :class:`CudaBackend`; it refuses tensors that are not on a CUDA device.
(:func:`set_backend` exists so that the test-suite can check the autograd wiring on a machine
without a GPU by substituting reference implementations of the same primitives.)
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
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mlcg_b200 operators run on CUDA tensors only (there is no CPU fallback)")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"mlcg_b200: unsupported dtype {t.dtype}; use float32 or float64") from None


class CudaBackend:
    name = "cuda"

    def __init__(self):
        self.lib = _lib.load()

    # ------------------------------------------------------------------ radius graph
    def batch_to_ptr(self, batch: torch.Tensor, B: int) -> torch.Tensor:
        _need_cuda(batch)
        batch = batch.contiguous()
        ptr = torch.empty(B + 1, dtype=torch.int64, device=batch.device)
        with torch.cuda.device(batch.device):
            _lib.check(self.lib.mlcgb_batch_to_ptr(_ptr(batch), batch.numel(), B, _ptr(ptr), _stream()), "batch_to_ptr")
        return ptr

    def radius_graph(self, pos, ptr, r, max_num_neighbors, loop, rule, want_distance=False, want_batch=True):
        """Returns dict(edge_index[2,E] i64, distance|None, mapping_batch|None, row0, row1 (i32), offsets[N+1] i64, status int)."""
        _need_cuda(pos, ptr)
        pos = pos.detach().contiguous()
        N, B, dev = pos.shape[0], ptr.numel() - 1, pos.device
        dt = _dt(pos)
        with torch.cuda.device(dev):
            ws_bytes = self.lib.mlcgb_radius_workspace_bytes(N, B, dt)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
            deg = torch.empty(max(N, 1), dtype=torch.int32, device=dev)
            offsets = torch.empty(N + 1, dtype=torch.int64, device=dev)
            status = torch.zeros(4, dtype=torch.int32, device=dev)
            _lib.check(self.lib.mlcgb_radius_count(_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(max_num_neighbors), int(loop), int(rule),
                                                   _ptr(ws), ws_bytes, _ptr(deg), _ptr(offsets), _ptr(status), _stream()), "radius_count")
            tail = torch.stack([offsets[N], status[0].to(torch.int64)]).cpu()   # the one host read: E and the status word
            E, st = int(tail[0]), int(tail[1])
            ei = torch.empty((2, E), dtype=torch.int64, device=dev)
            dist = torch.empty(E, dtype=pos.dtype, device=dev) if want_distance else None
            mb = torch.empty(E, dtype=torch.int64, device=dev) if want_batch else None
            r0 = torch.empty(E, dtype=torch.int32, device=dev)
            r1 = torch.empty(E, dtype=torch.int32, device=dev)
            _lib.check(self.lib.mlcgb_radius_fill(_ptr(pos), dt, _ptr(ptr), N, B, float(r), int(loop), _ptr(ws), ws_bytes, _ptr(offsets), E,
                                                  _ptr(ei), _ptr(dist), _ptr(mb), _ptr(r0), _ptr(r1), _ptr(status), _stream()), "radius_fill")
        return dict(edge_index=ei, distance=dist, mapping_batch=mb, row0=r0, row1=r1, offsets=offsets, status=st)

    def edge_twin(self, row0, row1, offsets, N):
        """twin[e] = position of the reversed edge; second value: True if every edge has one."""
        _need_cuda(row0)
        E = row0.numel()
        twin = torch.empty(E, dtype=torch.int32, device=row0.device)
        status = torch.zeros(4, dtype=torch.int32, device=row0.device)
        with torch.cuda.device(row0.device):
            _lib.check(self.lib.mlcgb_edge_twin(_ptr(row0), _ptr(row1), _ptr(offsets), E, N, _ptr(twin), _ptr(status), _stream()), "edge_twin")
        return twin, status

    # ------------------------------------------------------------------ geometry
    def edge_diff(self, pos, row0, row1):
        _need_cuda(pos, row0, row1)
        pos = pos.contiguous()
        E = row0.numel()
        out = torch.empty((E, 3), dtype=pos.dtype, device=pos.device)
        status = torch.zeros(4, dtype=torch.int32, device=pos.device)
        with torch.cuda.device(pos.device):
            _lib.check(self.lib.mlcgb_edge_diff(_ptr(pos), _dt(pos), _ptr(row0), _ptr(row1), E, pos.shape[0], _ptr(out), _ptr(status), _stream()), "edge_diff")
        return out

    def node_scatter_diff(self, g, ptr_in, perm_in, ptr_out, perm_out, N):
        _need_cuda(g)
        g = g.contiguous()
        out = torch.empty((N, 3), dtype=g.dtype, device=g.device)
        with torch.cuda.device(g.device):
            _lib.check(self.lib.mlcgb_node_scatter_diff(_ptr(g), _dt(g), _ptr(ptr_in), _ptr(perm_in), _ptr(ptr_out), _ptr(perm_out), N,
                                                        g.shape[0], _ptr(out), _stream()), "node_scatter_diff")
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
        with torch.cuda.device(d.device):
            _lib.check(self.lib.mlcgb_rbf_expand(_ptr(d), _dt(d), d.numel(), ctypes.byref(s), order, _ptr(out), _stream()), "rbf_expand")
        return out

    def rbf_contract(self, d, G, spec: RbfSpec, order: int):
        _need_cuda(d, G, spec.p0, spec.p1)
        d, G = d.contiguous(), G.contiguous()
        s, keep = self._spec(spec, d.dtype)
        out = torch.empty(d.numel(), dtype=d.dtype, device=d.device)
        with torch.cuda.device(d.device):
            _lib.check(self.lib.mlcgb_rbf_contract(_ptr(d), _ptr(G), _dt(d), d.numel(), ctypes.byref(s), order, _ptr(out), _stream()), "rbf_contract")
        return out

    # ------------------------------------------------------------------ CFConv primitives
    def seg_mul_sum(self, a, V, ptr, nbr, eperm, N):
        _need_cuda(a, V, ptr, nbr)
        a, V = a.contiguous(), V.contiguous()
        F = V.shape[1]
        out = torch.empty((N, F), dtype=V.dtype, device=V.device)
        with torch.cuda.device(V.device):
            _lib.check(self.lib.mlcgb_seg_mul_sum(_ptr(a), _ptr(V), _dt(V), _ptr(ptr), _ptr(nbr), _ptr(eperm), N, V.shape[0], F, _ptr(out), _stream()), "seg_mul_sum")
        return out

    def edge_mul(self, a, b, ia, ib):
        _need_cuda(a, b, ia, ib)
        a, b = a.contiguous(), b.contiguous()
        E, F = ia.numel(), a.shape[1]
        out = torch.empty((E, F), dtype=a.dtype, device=a.device)
        with torch.cuda.device(a.device):
            _lib.check(self.lib.mlcgb_edge_mul(_ptr(a), _ptr(b), _dt(a), _ptr(ia), _ptr(ib), E, F, _ptr(out), _stream()), "edge_mul")
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
        with torch.cuda.device(A.device):
            wsb = self.lib.mlcgb_gemm_workspace_bytes(mode, M, N, K, dt)
            ws = torch.empty(wsb, dtype=torch.uint8, device=A.device) if wsb else None
            if bias is not None:
                bias = bias.contiguous()
            _lib.check(self.lib.mlcgb_gemm(mode, _ptr(A), _ptr(B), _ptr(bias), dt, M, N, K, _ptr(C), _ptr(ws), wsb, _stream()), "gemm")
        return C

    def segment_sum(self, x, ptr):
        _need_cuda(x, ptr)
        x = x.contiguous()
        B = ptr.numel() - 1
        out = torch.empty(B, dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(self.lib.mlcgb_segment_sum(_ptr(x), _dt(x), _ptr(ptr), B, _ptr(out), _stream()), "segment_sum")
        return out

    # ------------------------------------------------------------------ priors
    def prior_terms(self, kind, pos, mapping, mapping_batch, params, B, want_grad=True):
        """Returns (energy[B], dE/dpos[N,3] | None)."""
        _need_cuda(pos, mapping, mapping_batch, params)
        pos, mapping, mapping_batch, params = pos.detach().contiguous(), mapping.contiguous(), mapping_batch.contiguous(), params.contiguous()
        M, N = mapping.shape[1], pos.shape[0]
        energy = torch.zeros(B, dtype=pos.dtype, device=pos.device)
        grad = torch.zeros((N, 3), dtype=pos.dtype, device=pos.device) if want_grad else None
        status = torch.zeros(4, dtype=torch.int32, device=pos.device)
        with torch.cuda.device(pos.device):
            _lib.check(self.lib.mlcgb_prior_terms(kind, _ptr(pos), _dt(pos), _ptr(mapping), _ptr(mapping_batch), _ptr(params), params.shape[0], M, N, B,
                                                  _ptr(energy), _ptr(grad), _ptr(status), _stream()), "prior_terms")
        return energy, grad


_backend = None


def get_backend():
    global _backend
    if _backend is None:
        _backend = CudaBackend()   # raises ExtensionMissing if the library is absent
    return _backend


def set_backend(be):
    """Replace the back end (test harness only). Returns the previous one."""
    global _backend
    old, _backend = _backend, be
    return old
