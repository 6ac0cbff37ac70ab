"""Radius graph on the GPU, through the C ABI, against the CPU oracle: bit-exact edges in the reference's order."""
import math
from itertools import product

import numpy as np
import pytest
import torch

import mlcg_b200
from mlcg_b200.backend import get_backend
from oracle import radius_ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_gpu(pos, ptr, r, max_nn, loop, rule):
    be = get_backend()
    res = be.radius_graph(torch.as_tensor(pos, device=DEV), torch.as_tensor(ptr, device=DEV), r, max_nn, loop,
                          {"native": 0, "cluster": 1}[rule], want_distance=True)
    torch.cuda.synchronize()
    return res


def check_against_oracle(pos, ptr, r, max_nn=1000, loop=False, rule="cluster"):
    res = run_gpu(pos, ptr, r, max_nn, loop, rule)
    ei, dist = radius_ref.radius_graph_c(pos, ptr, r, max_nn, loop, rule, with_distance=True)
    got = res["edge_index"].cpu().numpy()
    assert got.shape == ei.shape, (got.shape, ei.shape)
    assert np.array_equal(got, ei)
    assert np.array_equal(res["distance"].cpu().numpy(), dist)            # sqrt of the same rounded sum: bit-exact too
    seg = np.searchsorted(ptr, ei[0], side="right") - 1
    assert np.array_equal(res["mapping_batch"].cpu().numpy(), seg)
    assert np.array_equal(res["row0"].cpu().numpy(), ei[0]) and np.array_equal(res["row1"].cpu().numpy(), ei[1])
    off = np.zeros(len(pos) + 1, np.int64)
    np.cumsum(np.bincount(ei[0], minlength=len(pos)), out=off[1:])
    assert np.array_equal(res["offsets"].cpu().numpy(), off)
    return res, ei


# the parameter grid of the reference's native-op test (src/opt_radius/mlcg_opt_radius/test_radius.py:28-41)
@pytest.mark.parametrize("x_c,dim,x_range,r,batch_size,loop,dtype",
                         list(product([0, 10, 100], [1, 2, 3], [(-1.0, 1.0), (-10.0, -20.0)], [0.0, 1.0, 10.0],
                                      [(100,), (50, 100), (10, 20, 100)], [True, False], [np.float64, np.float32])))
def test_reference_grid(x_c, dim, x_range, r, batch_size, loop, dtype):
    rng = np.random.default_rng(x_c * 7 + dim)
    lo, hi = x_range
    x = ((hi - lo) * rng.random((x_c, dim)) + lo).astype(dtype)
    sizes, p = [], 0
    for b in batch_size:
        n = math.ceil(x_c * (b / 100)) - p
        sizes.append(n)
        p += n
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    batch = np.repeat(np.arange(len(sizes)), sizes)
    x3 = np.concatenate([x, np.zeros((x_c, 3 - dim), dtype)], axis=1)
    want = radius_ref.radius_graph_c(x3, ptr, r, 100, loop, "native")
    if x_c == 0:
        d, ei = mlcg_b200.radius_distance(torch.as_tensor(x, device=DEV), r, None, loop, 100)
        assert ei.shape == (2, 0)
        return
    d, ei = mlcg_b200.radius_distance(torch.as_tensor(x, device=DEV), r, torch.as_tensor(batch, device=DEV), loop, 100,
                                      batch_size=len(sizes))
    assert np.array_equal(ei.cpu().numpy(), want)
    ref_d = np.linalg.norm(x3[want[1]] - x3[want[0]], axis=-1)
    assert np.allclose(d.cpu().numpy(), ref_d, atol=1e-6)
    same = mlcg_b200.radius_graph(torch.as_tensor(x, device=DEV), r, torch.as_tensor(batch, device=DEV), loop, 100,
                                  flow="target_to_source", batch_size=len(sizes))
    assert np.array_equal(same.cpu().numpy(), radius_ref.radius_graph_c(x3, ptr, r, 100, loop, "cluster"))


@pytest.mark.parametrize("rule", ["native", "cluster"])
@pytest.mark.parametrize("loop", [False, True])
@pytest.mark.parametrize("max_nn", [1, 3, 17, 1000])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_truncation_and_ragged_batches(rule, loop, max_nn, dtype):
    rng = np.random.default_rng(3)
    sizes = [0, 5, 1, 130, 0, 0, 700, 33, 0]            # empty, tiny, brute-force and cell-list structures mixed
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    pos = (rng.random((ptr[-1], 3)) * 12).astype(dtype)
    res, ei = check_against_oracle(pos, ptr, 3.0, max_nn, loop, rule)
    full = radius_ref.radius_graph_c(pos, ptr, 3.0, 10 ** 6, loop, rule)
    assert bool(res["status"] & 1) == (full.shape[1] != ei.shape[1])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_uniform_cube_cell_path(dtype):
    """Four structures of the standalone radius-graph configuration: 4000 points in a 60 A cube, 10 A cutoff."""
    rng = np.random.default_rng(0)
    pos = (rng.random((4 * 4000, 3)) * 60).astype(dtype)
    ptr = np.arange(5, dtype=np.int64) * 4000
    res, ei = check_against_oracle(pos, ptr, 10.0, 1000)
    deg = np.bincount(ei[0], minlength=len(pos))
    assert 40 < deg.mean() < 90 and not res["status"]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("loop", [False, True])
def test_dense_and_uneven_structures(dtype, loop):
    """More candidates than one stage of the block kernels holds, more than 32 centres in a block of cells, hit lists
    that are written out several times, neighbour caps that bite: a dense cube, and a blob inside a sparse cloud."""
    rng = np.random.default_rng(11)
    dense = (rng.random((3000, 3)) * 10).astype(dtype)
    blob = np.concatenate([rng.random((2500, 3)) * 40, 18 + rng.random((1500, 3)) * 4]).astype(dtype)
    blob = blob[rng.permutation(len(blob))]
    for pos, r in ((dense, 4.0), (blob, 5.0)):
        ptr = np.array([0, len(pos)], np.int64)
        for max_nn in (1000, 40):
            check_against_oracle(pos, ptr, r, max_nn, loop, "cluster")
        check_against_oracle(pos, ptr, r, 9, loop, "native")


def test_structure_larger_than_one_bitmask_window():
    rng = np.random.default_rng(1)
    sizes = [20000, 9000]
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    pos = (rng.random((ptr[-1], 3)) * np.array([80, 80, 40])).astype(np.float32)
    check_against_oracle(pos, ptr, 6.0, 1000)
    check_against_oracle(pos, ptr, 6.0, 7)


def test_pairs_exactly_at_the_cutoff():
    """Lattice with spacing 2.5 and cutoff 2.5 / 5.0: d2 == r2 must be rejected (strict <), in both paths."""
    g = np.stack(np.meshgrid(*[np.arange(12)] * 3, indexing="ij"), -1).reshape(-1, 3).astype(np.float32) * 2.5
    for r in (2.5, 5.0, 2.5000002):
        check_against_oracle(g, np.array([0, len(g)], np.int64), r)           # 1728 points: cell path
        check_against_oracle(g[:216], np.array([0, 216], np.int64), r)        # brute-force path


def test_far_from_origin_and_degenerate_boxes():
    rng = np.random.default_rng(5)
    pos = (rng.random((3000, 3)) * 30 + 5000.0).astype(np.float32)              # large offsets: coarse float spacing
    check_against_oracle(pos, np.array([0, 3000], np.int64), 4.0)
    flat = pos.copy()
    flat[:, 2] = 1.0                                                            # planar structure: one cell layer
    check_against_oracle(flat, np.array([0, 3000], np.int64), 4.0)
    same = np.zeros((500, 3), np.float32)                                       # all points coincide
    check_against_oracle(same, np.array([0, 500], np.int64), 1.0, 50)


def test_chain_configurations():
    """Bead chains of the coarse-grained configurations: 10, 100, 73 and 268 beads."""
    from helpers import random_walk_chain
    gen = torch.Generator().manual_seed(0)
    for n, B, rc in [(10, 64, 30.0), (100, 16, 15.0), (73, 16, 10.0), (268, 8, 12.0)]:
        pos = torch.cat([random_walk_chain(n, gen, jitter=0.3) for _ in range(B)]).numpy()
        res, ei = check_against_oracle(pos, np.arange(B + 1, dtype=np.int64) * n, rc)
        twin, st = get_backend().edge_twin(res["row0"], res["row1"], res["offsets"], len(pos), fresh_status=True)
        assert int(st[0]) == 0
        t = twin.cpu().numpy()
        assert np.array_equal(ei[0][t], ei[1]) and np.array_equal(ei[1][t], ei[0])


def test_pair_plan_in_one_call():
    """Reverse-edge map, one edge per unordered pair and the edge -> pair index from `mlcgb_pair_plan` equal the three
    separate steps; a list that lacks a reverse edge, or holds a loop, is reported."""
    from helpers import random_walk_chain
    from oracle.primitives import OracleBackend
    be, gen = get_backend(), torch.Generator().manual_seed(1)
    for n, B, rc in [(2, 1, 30.0), (10, 64, 30.0), (268, 8, 12.0), (1500, 3, 9.0)]:
        pos = torch.cat([random_walk_chain(n, gen, jitter=0.3) for _ in range(B)]).numpy()
        res = run_gpu(pos, np.arange(B + 1, dtype=np.int64) * n, rc, 1000, False, "cluster")
        r0, r1, off = res["row0"], res["row1"], res["offsets"]
        twin, sel, pair_of, st = be.pair_plan(r0, r1, off, len(pos), fresh_status=True)
        assert int(st[0]) == 0
        want = OracleBackend().pair_plan(r0.cpu(), r1.cpu(), off.cpu(), len(pos))
        for got, ref in zip((twin, sel, pair_of), want):
            assert torch.equal(got.cpu(), ref)
        twin2, st = be.edge_twin(r0, r1, off, len(pos), fresh_status=True)
        assert int(st[0]) == 0 and torch.equal(twin, twin2)
        assert torch.equal(pair_of, be.pair_index(sel, twin))
    # drop one edge and its successor (the count stays even): the reverse of a kept edge is missing
    keep = torch.ones(r0.numel(), dtype=torch.bool, device=r0.device)
    keep[5:7] = False
    r0b, r1b = r0[keep].contiguous(), r1[keep].contiguous()
    offb = torch.zeros_like(off)
    offb[1:] = torch.cumsum(torch.bincount(r0b.long(), minlength=len(pos)), 0)
    *_, st = be.pair_plan(r0b, r1b, offb, len(pos), fresh_status=True)
    assert int(st[0]) & 4


def test_full_size_standalone_configuration_properties():
    """256 x 4000 points (65 M edges): size-independent properties on the whole output, oracle on a sample."""
    rng = np.random.default_rng(0)
    B, n = 256, 4000
    pos = (rng.random((B * n, 3)) * 60).astype(np.float32)
    ptr = np.arange(B + 1, dtype=np.int64) * n
    res = run_gpu(pos, ptr, 10.0, 1000, False, "cluster")
    ei, off = res["edge_index"], res["offsets"]
    E = ei.shape[1]
    assert int(off[-1]) == E and not res["status"]
    assert bool((ei[0][1:] >= ei[0][:-1]).all())                                          # centre-major
    same = ei[0][1:] == ei[0][:-1]
    assert bool((ei[1][1:][same] > ei[1][:-1][same]).all())                               # neighbours ascending, no duplicates
    assert bool((ei[0] // n == ei[1] // n).all()) and bool((ei[0] != ei[1]).all())        # same structure, no loops
    p = torch.as_tensor(pos, device=DEV)
    d = (p[ei[1]] - p[ei[0]]).double()             # (the float32 difference is what the kernel squares; products exact in float64)
    d2 = (d[:, 0] * d[:, 0] + d[:, 1] * d[:, 1]) + d[:, 2] * d[:, 2]
    assert bool((d2 < 100.0 * (1 + 2e-7)).all())   # within the two float32 roundings of the fused evaluation of r*r
    twin, st = get_backend().edge_twin(res["row0"], res["row1"], off, B * n, fresh_status=True)              # symmetric: every edge has its reverse
    assert int(st[0]) == 0
    for b in (0, 100, 255):
        want = radius_ref.radius_graph_c(pos[b * n:(b + 1) * n], np.array([0, n], np.int64), 10.0, 1000, False, "cluster") + b * n
        lo, hi = int(off[b * n]), int(off[(b + 1) * n])
        assert np.array_equal(ei[:, lo:hi].cpu().numpy(), want)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("loop", [False, True])
@pytest.mark.parametrize("max_nn", [4, 1000])
def test_excluded_pairs(dtype, loop, max_nn):
    """`mlcg::radius_cuda` with exclusion lists (radius.cu:112-141): brute-force and cell-list structures, with and without
    the neighbour cap, self pairs among the exclusions."""
    from mlcg_b200.neighbor_list import exclusion_pair_to_ptr, radius_cuda, radius_distance
    rng = np.random.default_rng(11)
    sizes = [0, 30, 1, 600, 130]
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    pos = (rng.random((ptr[-1], 3)) * 11).astype(dtype)
    xs_l, ys_l = [], []
    for b in range(len(sizes)):
        lo, hi = int(ptr[b]), int(ptr[b + 1])
        if hi > lo:
            m = 4 * (hi - lo)
            xs_l.append(rng.integers(lo, hi, m)); ys_l.append(rng.integers(lo, hi, m))
    # plus the bonded neighbours of every point, as a topology would list them
    idx = np.arange(ptr[-1] - 1)
    xs_l += [idx, idx + 1]; ys_l += [idx + 1, idx]
    pairs = np.stack([np.concatenate(xs_l), np.concatenate(ys_l)]).astype(np.int64)
    txs, tptr = exclusion_pair_to_ptr(torch.from_numpy(pairs).to(DEV), int(ptr[-1]))
    oxs, optr = radius_ref.exclusion_pair_to_ptr(pairs, int(ptr[-1]))
    assert np.array_equal(txs.cpu().numpy(), oxs) and np.array_equal(tptr.cpu().numpy(), optr)
    want, wdist = radius_ref.radius_graph_numpy(pos, ptr, 3.0, max_nn, loop, "native", with_distance=True, exclude=(oxs, optr))
    x = torch.as_tensor(pos, device=DEV)
    ei, dist = radius_cuda(x, torch.as_tensor(ptr, device=DEV), 3.0, max_nn, not loop, txs, tptr)
    assert np.array_equal(ei.cpu().numpy(), want) and np.array_equal(dist.cpu().numpy(), wdist)
    banned = set(zip(pairs[1].tolist(), pairs[0].tolist()))
    assert not any((i, j) in banned for i, j in zip(want[0].tolist(), want[1].tolist()))
    # the Python-level entry point builds the lists itself
    batch = torch.as_tensor(np.repeat(np.arange(len(sizes)), sizes), device=DEV)
    d2, ei2 = radius_distance(x, 3.0, batch, loop, max_nn, len(sizes), torch.from_numpy(pairs).to(DEV))
    assert np.array_equal(ei2.cpu().numpy(), want)
    assert np.allclose(d2.detach().cpu().numpy(), wdist, rtol=1e-6 if dtype == np.float32 else 1e-12)


@pytest.mark.parametrize("name", ["orthorhombic", "slab", "triclinic"])
def test_periodic_graph_vs_reference_vectors(golden_periodic, name):
    """`mlcgb_radius_pbc_count` / `_fill` against the lists the reference's torch_neighbor_list_pbc returned."""
    from mlcg_b200.neighbor_list import atomic_data2neighbor_list
    import mlcg_b200
    c = golden_periodic[name]
    mk = lambda: mlcg_b200.AtomicData(pos=c["pos"].to(DEV), atom_types=c["atom_types"].to(DEV), batch=c["batch"].to(DEV),
                                      n_atoms=torch.full((c["B"],), c["n"]).to(DEV), cell=c["cells"].to(DEV), pbc=c["pbc"].to(DEV))
    for key, cap, loop in (("1000", 1000, False), ("12", 12, False), ("self", 1000, True)):
        nl = atomic_data2neighbor_list(mk(), c["upper"], self_interaction=loop, max_num_neighbors=cap)
        assert torch.equal(nl["index_mapping"].cpu(), c[f"index_mapping_{key}"])
        assert torch.allclose(nl["cell_shifts"].cpu(), c[f"cell_shifts_{key}"], rtol=1e-6, atol=1e-6)
        if key != "self":
            assert torch.equal(nl["mapping_batch"].cpu(), c[f"mapping_batch_{key}"])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_periodic_graph_vs_oracle(dtype):
    """Random boxes, structures of different sizes, cutoffs from a fraction of the box to more than the box (several copies
    per direction): edges, shifts (bit for bit: same separately rounded arithmetic) and distances against the restatement."""
    rng = np.random.default_rng(5)
    be = get_backend()
    for trial, (rc, cap) in enumerate([(3.0, 1000), (7.0, 1000), (10.5, 1000), (7.0, 9)]):
        sizes = [5, 17, 24, 1, 20]
        ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        B = len(sizes)
        cells = np.zeros((B, 3, 3), dtype)
        for b in range(B):
            cells[b] = np.diag(rng.uniform(6.0, 10.0, 3)) + (rng.uniform(-1.5, 1.5, (3, 3)) if b % 2 else 0.0)
        pbc = np.array([[True, True, True], [True, False, True], [True, True, True], [False, False, True], [True, True, False]])
        frac = rng.uniform(-0.1, 1.1, (int(ptr[-1]), 3))
        pos = np.concatenate([frac[ptr[b]:ptr[b + 1]] @ cells[b].astype(np.float64) for b in range(B)]).astype(dtype)
        ei, shifts = radius_ref.radius_graph_pbc_numpy(pos, ptr, cells, pbc, rc, cap, False)
        reps = torch.as_tensor(radius_ref.pbc_repeats(cells, pbc, rc))
        res = be.radius_graph_pbc(torch.as_tensor(pos, device=DEV), torch.as_tensor(ptr, device=DEV), torch.as_tensor(cells, device=DEV),
                                  reps.to(DEV), rc, cap, False, want_distance=True)
        assert np.array_equal(res["edge_index"].cpu().numpy(), ei), trial
        assert np.array_equal(res["cell_shifts"].cpu().numpy(), shifts), trial
        d = np.sqrt((((pos[ei[1]] + shifts) - pos[ei[0]]) ** 2).sum(1))
        assert np.allclose(res["distance"].cpu().numpy(), d, rtol=1e-6 if dtype == np.float32 else 1e-13, atol=1e-6 if dtype == np.float32 else 1e-12)
        assert np.array_equal(res["mapping_batch"].cpu().numpy(), np.searchsorted(ptr, ei[0], side="right") - 1)
        assert bool(res["status"] & 1) == (cap == 9)


def test_reverse_edge_map_of_a_list_with_self_pairs():
    """Self pairs are their own reverse; a list with them may hold an odd number of edges and is still symmetric."""
    pos = np.array([[0.0, 0, 0], [1.0, 0, 0], [0, 1.0, 0], [5.0, 5, 5], [0.5, 0.5, 0]], np.float32)
    res = run_gpu(pos, np.array([0, 5], np.int64), 2.0, 1000, True, "cluster")
    E = int(res["offsets"][-1])
    assert E % 2 == 1
    twin, st = get_backend().edge_twin(res["row0"], res["row1"], res["offsets"], 5, fresh_status=True)
    assert int(st[0]) == 0
    t = twin.long()
    assert torch.equal(res["row0"][t], res["row1"]) and torch.equal(res["row1"][t], res["row0"])
