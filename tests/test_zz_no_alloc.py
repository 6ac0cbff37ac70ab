"""The allocation-free radius-graph entry point, called through the C ABI.

Some users of this library cannot allocate GPU memory where they need a neighbour list: the force routine
runs inside someone else's time-step loop, or the embedding program has claimed the device's memory up
front, or the calling thread must never block on an allocator.  For them ``mlcgb_radius_graph_static``
keeps its cell-list scratch in a fixed array inside the library and fills buffers the caller already owns.
This test drives it with plain pointers and checks that it returns exactly the edges of the regular
two-call path, twice in a row on different inputs (the scratch is shared and keeps whatever the previous
call left in it), and that it refuses inputs beyond its built-in limits instead of overrunning.

Collected last on purpose: a failure here stops a ``-x`` run only after every other test has run.
"""
import ctypes

import numpy as np
import pytest
import torch

from mlcg_b200 import _lib
from mlcg_b200.backend import get_backend
from oracle import radius_ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def call_static(pos, ptr, r, max_nn, loop, rule, capacity):
    lib = _lib.load()
    N, B = pos.shape[0], ptr.numel() - 1
    deg = torch.empty(max(N, 1), dtype=torch.int32, device=DEV)
    offsets = torch.empty(N + 1, dtype=torch.int64, device=DEV)
    edge_index = torch.full((2, capacity), -7, dtype=torch.int64, device=DEV)       # caller-owned output
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    n_edges = ctypes.c_int64(-1)
    dt = 0 if pos.dtype == torch.float32 else 1
    with torch.cuda.device(0):
        rc = lib.mlcgb_radius_graph_static(pos.data_ptr(), dt, ptr.data_ptr(), N, B, float(r), max_nn, int(loop), rule, deg.data_ptr(),
                                           offsets.data_ptr(), capacity, edge_index.data_ptr(), ctypes.byref(n_edges), status.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, n_edges.value, edge_index, offsets, int(status[0])


def regular_path(pos, ptr, r, max_nn, loop, rule):
    res = get_backend().radius_graph(pos, ptr, r, max_nn, loop, rule)
    return res["edge_index"], res["offsets"], res["status"]


def inputs(sizes, box, dtype, seed):
    rng = np.random.default_rng(seed)
    ptr = torch.as_tensor(np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64), device=DEV)
    pos = torch.as_tensor((rng.random((int(ptr[-1]), 3)) * box).astype(dtype), device=DEV)
    return pos, ptr


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_two_calls_in_a_row_match_the_regular_path(dtype):
    # first a large, cell-list sized problem, then a small ragged one that reuses the same scratch
    for sizes, box, r, max_nn, loop, rule, seed in [([4000, 3000, 10, 0, 500], 45.0, 8.0, 1000, False, 1, 0),
                                                    ([7, 0, 129, 600], 14.0, 3.0, 5, True, 0, 1)]:
        pos, ptr = inputs(sizes, box, dtype, seed)
        want_ei, want_off, want_status = regular_path(pos, ptr, r, max_nn, loop, rule)
        E = want_ei.shape[1]
        rc, n_edges, ei, off, status = call_static(pos, ptr, r, max_nn, loop, rule, capacity=E + 11)
        assert rc == 0 and n_edges == E
        assert torch.equal(ei[:, :E], want_ei)                      # bit-exact: integer output
        assert bool((ei[:, E:] == -7).all())                        # nothing written past the edges
        assert torch.equal(off, want_off) and status == want_status
        # and directly against the CPU oracle's list for the same inputs
        oracle_ei = radius_ref.radius_graph_c(pos.cpu().numpy(), ptr.cpu().numpy(), r, max_nn, loop, "cluster" if rule == 1 else "native")
        assert np.array_equal(ei[:, :E].cpu().numpy(), oracle_ei)


def test_limits_are_refused_with_an_error_code():
    lib = _lib.load()
    pos, ptr = inputs([300], 10.0, np.float32, 2)
    rc, n_edges, ei, _, _ = call_static(pos, ptr, 4.0, 1000, False, 1, capacity=5)      # edge buffer too small
    assert rc == -4 and n_edges > 5 and bool((ei == -7).all())
    assert b"limit" in lib.mlcgb_strerror(rc)
    big = torch.zeros(1, dtype=torch.int64, device=DEV)
    n = ctypes.c_int64(0)
    # more points than the built-in scratch covers: rejected before anything is launched or read
    rc = lib.mlcgb_radius_graph_static(big.data_ptr(), 0, big.data_ptr(), 65537, 1, 1.0, 10, 0, 1, big.data_ptr(), big.data_ptr(), 0,
                                       big.data_ptr(), ctypes.byref(n), big.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -4


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_the_largest_batch_the_scratch_is_sized_for(dtype):
    """65 536 points in 8 192 structures, the documented limits at once: accepted in both dtypes, same list as the regular path."""
    pos, ptr = inputs([8] * 8192, 6.0, dtype, 4)
    want_ei, want_off, _ = regular_path(pos, ptr, 3.0, 1000, False, 1)
    E = want_ei.shape[1]
    rc, n_edges, ei, off, _ = call_static(pos, ptr, 3.0, 1000, False, 1, capacity=E)
    assert rc == 0 and n_edges == E and torch.equal(ei, want_ei) and torch.equal(off, want_off)
