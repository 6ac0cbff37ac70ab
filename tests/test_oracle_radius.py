"""The two radius-graph oracles against each other and against hand-checkable cases."""
import numpy as np
import pytest

from oracle import radius_ref


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("rule", ["native", "cluster"])
@pytest.mark.parametrize("loop", [False, True])
@pytest.mark.parametrize("max_nn", [2, 5, 1000])
def test_c_equals_numpy(dtype, rule, loop, max_nn):
    rng = np.random.default_rng(0)
    sizes = [0, 17, 1, 40, 0, 33]
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    pos = (rng.random((ptr[-1], 3)) * 6).astype(dtype)
    a, da = radius_ref.radius_graph_c(pos, ptr, 2.0, max_nn, loop, rule, with_distance=True)
    b, db = radius_ref.radius_graph_numpy(pos, ptr, 2.0, max_nn, loop, rule, with_distance=True)
    assert np.array_equal(a, b) and np.array_equal(da, db)
    assert np.all(np.diff(a[0]) >= 0)                           # centre-major
    same = a[0][1:] == a[0][:-1]
    assert np.all(a[1][1:][same] > a[1][:-1][same])             # neighbours ascending


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_fused_multiply_add_emulation_is_exact(dtype):
    """`fma_exact` (operations of one dtype only) against libm's correctly rounded fma on random, cancelling, tiny and huge
    addends; separately rounded `a*b + c` differs from both on a large share of these inputs."""
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    f = libm.fmaf if dtype == np.float32 else libm.fma
    ct = ctypes.c_float if dtype == np.float32 else ctypes.c_double
    f.restype, f.argtypes = ct, [ct] * 3
    rng = np.random.default_rng(1)
    n = 20000
    a, b = (rng.standard_normal(n) * 10).astype(dtype), (rng.standard_normal(n) * 10).astype(dtype)
    c = (rng.standard_normal(n) * 100).astype(dtype)
    c[: n // 4] = (-(a[: n // 4].astype(np.float64) * b[: n // 4])).astype(dtype)
    c[n // 4: n // 2] *= dtype(1e-6)
    c[n // 2: 3 * n // 4] *= dtype(1e6)
    want = np.array([f(float(x), float(y), float(z)) for x, y, z in zip(a, b, c)], dtype=dtype)
    assert np.array_equal(radius_ref.fma_exact(a, b, c), want)
    assert (a * b + c != want).sum() > n // 10


def test_strict_cutoff_on_a_lattice():
    """Integer lattice, integer cutoff: pairs at exactly r are excluded (strict <, radius.cu:134)."""
    g = np.stack(np.meshgrid(*[np.arange(4)] * 3, indexing="ij"), -1).reshape(-1, 3).astype(np.float32)
    ei = radius_ref.radius_graph_c(g, np.array([0, 64]), 1.0, 1000, False, "cluster")
    assert ei.shape[1] == 0
    ei = radius_ref.radius_graph_c(g, np.array([0, 64]), 1.0000001, 1000, False, "cluster")
    assert ei.shape[1] == 2 * 3 * 4 * 4 * 3                     # axis neighbours only
    assert radius_ref.radius_graph_c(g, np.array([0, 64]), 0.0, 1000, True, "native").shape[1] == 0  # r = 0: nothing, not even loops


def test_truncation_rules_differ_only_when_self_is_not_reached():
    # five collinear points, all within range; max_nn = 2
    pos = np.zeros((5, 3), np.float32)
    pos[:, 0] = np.arange(5) * 0.1
    nat = radius_ref.radius_graph_c(pos, np.array([0, 5]), 1.0, 2, False, "native")
    clu = radius_ref.radius_graph_c(pos, np.array([0, 5]), 1.0, 2, False, "cluster")
    deg_n, deg_c = np.bincount(nat[0], minlength=5), np.bincount(clu[0], minlength=5)
    assert deg_n.tolist() == [2, 2, 2, 2, 2]
    assert deg_c.tolist() == [2, 2, 2, 3, 3]                    # centres 3, 4 have >= 3 lower neighbours: self never reached
    assert clu[1][clu[0] == 4].tolist() == [0, 1, 2]


def test_exclusion_pair_worked_example():
    """The input of the example in the comment at exclusion_pairs.cpp:16-18, with the result the CODE below
    that comment produces (two stable sorts -> ordered by (y, x); pointer indexed by 0-based node, which is
    how radius.cu:122-123 reads it).  The comment's own numbers ([2,1,3,2,2] / [0,1,4,5,5]) do not follow
    from the code: they leave x unsorted inside y = 2 and index the pointer from node 1."""
    pairs = np.array([[2, 1, 3, 2, 2], [1, 2, 2, 2, 3]])
    xs, ptr = radius_ref.exclusion_pair_to_ptr(pairs, 4)
    assert xs.tolist() == [2, 1, 2, 3, 2]
    assert ptr.tolist() == [0, 0, 1, 4, 5]


def _random_exclusions(rng, ptr, per_point, both_directions):
    """Pairs (x, y) inside structures, `per_point` of them per point on average, some of them (i, i)."""
    xs, ys = [], []
    for b in range(len(ptr) - 1):
        lo, hi = int(ptr[b]), int(ptr[b + 1])
        if hi - lo < 1:
            continue
        m = (hi - lo) * per_point
        x, y = rng.integers(lo, hi, m), rng.integers(lo, hi, m)
        xs.append(x); ys.append(y)
        if both_directions:
            xs.append(y); ys.append(x)
    pairs = np.unique(np.stack([np.concatenate(xs), np.concatenate(ys)]), axis=1)     # the kernel's search wants no duplicates? it does not care
    return pairs.astype(np.int64)


@pytest.mark.parametrize("loop", [False, True])
@pytest.mark.parametrize("max_nn", [3, 1000])
def test_excluded_pairs_oracle(loop, max_nn):
    """Exclusions (radius.cu:122-141): without a cap the graph is the plain graph minus the excluded pairs; with a cap the
    excluded points do not use up places."""
    rng = np.random.default_rng(5)
    sizes = [0, 17, 1, 40]
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    pos = (rng.random((ptr[-1], 3)) * 5).astype(np.float32)
    pairs = _random_exclusions(rng, ptr, 3, False)
    xs, y_ptr = radius_ref.exclusion_pair_to_ptr(pairs, int(ptr[-1]))
    plain = radius_ref.radius_graph_numpy(pos, ptr, 2.0, 10 ** 6, loop, "native")
    got = radius_ref.radius_graph_numpy(pos, ptr, 2.0, max_nn, loop, "native", exclude=(xs, y_ptr))
    banned = set(zip(pairs[1].tolist(), pairs[0].tolist()))                     # (centre y, neighbour x)
    want = [(i, j) for i, j in zip(plain[0].tolist(), plain[1].tolist()) if (i, j) not in banned]
    if max_nn < 1000:
        kept, seen = [], {}
        for i, j in want:
            if seen.get(i, 0) < max_nn:
                kept.append((i, j)); seen[i] = seen.get(i, 0) + 1
        want = kept
    assert list(zip(got[0].tolist(), got[1].tolist())) == want


def test_exclusion_pair_to_ptr_torch_version_matches_the_c_restatement():
    import torch
    from mlcg_b200.neighbor_list import exclusion_pair_to_ptr
    rng = np.random.default_rng(2)
    for n, p in [(4, 5), (50, 400), (7, 0), (1, 3)]:
        pairs = rng.integers(0, n, (2, p)).astype(np.int64)
        xs, y_ptr = radius_ref.exclusion_pair_to_ptr(pairs, n)
        txs, tptr = exclusion_pair_to_ptr(torch.from_numpy(pairs), n)
        assert txs.tolist() == xs.tolist() and tptr.tolist() == y_ptr.tolist()
    xs, y_ptr = exclusion_pair_to_ptr(torch.tensor([[2, 1, 3, 2, 2], [1, 2, 2, 2, 3]]), 4)
    assert xs.tolist() == [2, 1, 2, 3, 2] and y_ptr.tolist() == [0, 0, 1, 4, 5]


@pytest.mark.parametrize("name", ["orthorhombic", "slab", "triclinic"])
def test_periodic_graph_restatement_vs_reference(golden_periodic, name):
    """`radius_graph_pbc_numpy` against what the reference's own torch_neighbor_list_pbc returned (torch_impl.py:252-329):
    same edges in the same order with and without the neighbour cap and with self pairs kept; the shift vectors are equal bit
    for bit for the axis-aligned boxes and to rounding for the sheared one."""
    c = golden_periodic[name]
    pos, ptr = c["pos"].numpy(), np.arange(c["B"] + 1, dtype=np.int64) * c["n"]
    for key, cap, loop in (("1000", 1000, False), ("12", 12, False), ("self", 1000, True)):
        ei, shifts = radius_ref.radius_graph_pbc_numpy(pos, ptr, c["cells"].numpy(), c["pbc"].numpy(), c["upper"], cap, loop)
        assert np.array_equal(ei, c[f"index_mapping_{key}"].numpy())
        want = c[f"cell_shifts_{key}"].numpy()
        if name == "triclinic":
            assert np.allclose(shifts, want, rtol=1e-6, atol=1e-6)
        else:
            assert np.array_equal(shifts, want)
