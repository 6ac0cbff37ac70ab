"""The radius graph against the reference's own compiled kernel.

The comparator is ``oracle/_ref/radius_kernel.so``: ``src/opt_radius/mlcg_opt_radius/{binding.cpp, radius.cu,
exclusion_pairs.cpp}`` of mlcg, compiled unmodified by ``oracle/build_ref.py`` with the reference's own flags and run in a child
process (``oracle/ref_runner.py``).  Every case calls ``radius_cuda`` of that binary and ``mlcg_b200.radius_cuda`` with the same
seven arguments and wants the same edges in the same order, and distances equal to a few units in the last place.

Cases: the parameter grid of the reference's own test (``test_radius.py:28-41``: 10 and 100 points, 1 to 3 dimensions, two
coordinate ranges, r in {0, 1, 10}, one to three structures, with and without loops; float64 as there, and float32), the same
grid with a neighbour cap that truncates, an integer lattice with the cutoff on a lattice distance, 4 x 4000 points in a 60 A
cube at 10 A, excluded pairs, and pairs whose squared distance is within one rounding of r*r.
"""
import ctypes
import itertools
import math

import numpy as np
import pytest
import torch

import mlcg_b200
from oracle import ref_runner

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref/radius_kernel.so not built (python oracle/build_ref.py <mlcg checkout>)")]


def _job(x, ptr, r, max_nn, loop, excl=None):
    return dict(op="radius_cuda", x=x, ptr_x=ptr, r=float(r), max_num_neighbors=int(max_nn), ignore_same_index=not loop,
                exclude_pair_xs=None if excl is None else excl[0], ptr_exclude_pair_xs=None if excl is None else excl[1])


def _grid_cases():
    gen = torch.Generator().manual_seed(0)
    cases = []
    for x_c, dim, (x_min, x_max), r, sizes, loop, dtype, max_nn in itertools.product(
            [10, 100], [1, 2, 3], [(-1.0, 1.0), (-10.0, -20.0)], [0.0, 1.0, 10.0], [(100,), (50, 100), (10, 20, 100)], [True, False],
            [torch.float64, torch.float32], [100, 7]):
        x = ((x_max - x_min) * torch.rand((x_c, dim), generator=gen, dtype=torch.float64) + x_min).to(dtype)
        counts, p = [], 0
        for b in sizes:                                     # the split of test_radius.py:71-77
            n = math.ceil(x_c * (b / 100)) - p
            counts.append(n)
            p += n
        ptr = torch.tensor([0] + list(itertools.accumulate(counts)), dtype=torch.int64) if len(sizes) > 1 else None
        cases.append((f"grid n={x_c} dim={dim} range=({x_min},{x_max}) r={r} B={len(sizes)} loop={loop} {dtype} cap={max_nn}", _job(x, ptr, r, max_nn, loop)))
    return cases


def _lattice_cases():
    g = torch.stack(torch.meshgrid(*[torch.arange(5.0)] * 3, indexing="ij"), -1).reshape(-1, 3)
    out = []
    for dtype in (torch.float32, torch.float64):
        for r in (1.0, math.sqrt(2.0), 2.0, 1.0000001):
            out.append((f"lattice r={r} {dtype}", _job(g.to(dtype), None, r, 200, False)))
    return out


def _cube_case():
    gen = torch.Generator().manual_seed(3)
    x = torch.rand(4 * 4000, 3, generator=gen) * 60.0
    return [("cube 4x4000 r=10", _job(x, torch.arange(5, dtype=torch.int64) * 4000, 10.0, 160, False))]


def _exclusion_cases():
    gen = torch.Generator().manual_seed(5)
    out = []
    for dtype, max_nn, loop in itertools.product([torch.float32, torch.float64], [6, 1000], [False, True]):
        sizes = [40, 1, 70, 25]
        ptr = torch.tensor([0] + list(itertools.accumulate(sizes)), dtype=torch.int64)
        n = int(ptr[-1])
        x = (torch.rand(n, 3, generator=gen, dtype=torch.float64) * 6).to(dtype)
        pairs = []
        for lo, hi in zip(ptr[:-1].tolist(), ptr[1:].tolist()):
            m = 4 * (hi - lo)
            pairs.append(torch.stack([torch.randint(lo, hi, (m,), generator=gen), torch.randint(lo, hi, (m,), generator=gen)]))
        pairs = torch.unique(torch.cat(pairs, dim=1), dim=1)
        xs, yptr = mlcg_b200.exclusion_pair_to_ptr(pairs, n)
        out.append((f"exclusions {dtype} cap={max_nn} loop={loop}", _job(x, ptr, 2.5, max_nn, loop, (xs, yptr))))
    return out


def _boundary_cases():
    """Two-point structures whose squared distance comes out one rounding apart under the two ways of evaluating
    dx*dx + dy*dy + dz*dz (every operation rounded on its own / fused multiply-adds, which is how nvcc contracts the loop at
    radius.cu:126-130 by default), with r chosen so that (T)(r*r) is the larger of the two values: the pair is an edge under
    exactly one of the two forms."""
    libm = ctypes.CDLL("libm.so.6")
    libm.fmaf.restype, libm.fmaf.argtypes = ctypes.c_float, [ctypes.c_float] * 3
    libm.fma.restype, libm.fma.argtypes = ctypes.c_double, [ctypes.c_double] * 3
    rng = np.random.default_rng(0)
    out = []
    for dt, fma in ((np.float32, libm.fmaf), (np.float64, libm.fma)):
        found = 0
        while found < 16:
            p = (rng.random((2, 3)) * 10).astype(dt)
            d = p[1] - p[0]
            sep = (d[0] * d[0] + d[1] * d[1]) + d[2] * d[2]
            fused = dt(fma(d[2], d[2], dt(fma(d[1], d[1], dt(d[0] * d[0])))))
            if sep == fused:
                continue
            hi = max(sep, fused)
            r = float(np.sqrt(np.float64(hi)))
            for _ in range(4):
                if dt(r * r) == hi:
                    break
                r = float(np.nextafter(r, 0.0 if dt(r * r) > hi else np.inf))
            if dt(r * r) != hi:
                continue
            found += 1
            out.append((f"boundary {dt.__name__} #{found} edge-if-{'fused' if fused < sep else 'separate'}", _job(torch.from_numpy(p), None, r, 8, False)))
    return out


@pytest.fixture(scope="module")
def compared():
    """(name, job, reference result, product result) for every case; the reference binary runs once, in a child process."""
    cases = _grid_cases() + _lattice_cases() + _cube_case() + _exclusion_cases() + _boundary_cases()
    ref = ref_runner.run([job for _, job in cases], timeout=900)
    out = []
    on = lambda t: None if t is None else t.cuda()
    for (name, job), (rei, rdist) in zip(cases, ref):
        ei, dist = mlcg_b200.radius_cuda(on(job["x"]), on(job["ptr_x"]), job["r"], job["max_num_neighbors"], job["ignore_same_index"],
                                         on(job["exclude_pair_xs"]), on(job["ptr_exclude_pair_xs"]))
        out.append((name, job, rei, rdist, ei.cpu(), dist.cpu()))
    return out


def _check(rows, prefix):
    rows = [r for r in rows if r[0].startswith(prefix)]
    assert rows
    edges = 0
    for name, job, rei, rdist, ei, dist in rows:
        assert rei.shape == ei.shape, f"{name}: {rei.shape[1]} reference edges, {ei.shape[1]} here"
        assert torch.equal(rei, ei), name
        tol = 1e-6 if dist.dtype == torch.float32 else 1e-14
        assert torch.allclose(rdist, dist, rtol=tol, atol=0.0), name
        edges += ei.shape[1]
    return len(rows), edges


def test_reference_parameter_grid(compared):
    n, edges = _check(compared, "grid")
    print(f"{n} grid cases, {edges} edges identical to the reference kernel's")
    assert edges > 100000


def test_lattice_at_the_cutoff(compared):
    _check(compared, "lattice")


def test_uniform_cube_4x4000(compared):
    n, edges = _check(compared, "cube")
    print(f"{edges} edges identical to the reference kernel's")
    assert edges > 900000


def test_excluded_pairs(compared):
    _check(compared, "exclusions")


def test_pairs_within_one_rounding_of_the_cutoff(compared):
    """Says which evaluation of the squared distance the reference binary follows, and wants the same decisions here."""
    rows = [r for r in compared if r[0].startswith("boundary")]
    follows = {"fused": 0, "separate": 0}
    for name, job, rei, rdist, ei, dist in rows:
        edge_if = name.rsplit("-", 1)[1]
        other = "separate" if edge_if == "fused" else "fused"
        follows[edge_if if rei.shape[1] > 0 else other] += 1
    print("reference binary decides like:", follows)
    assert min(follows.values()) == 0, follows          # the binary is one or the other throughout
    _check(compared, "boundary")
