"""TEST INFRASTRUCTURE — CPU oracle for the radius graph (not shipped, not measured as product).

Two independent restatements of the same rule, used to pin each other:

* :func:`radius_graph_numpy` — vectorised numpy, all pairs of one structure at a time, with the fused multiply-adds of the
  squared distance emulated exactly (:func:`fma_exact`);
* :func:`radius_graph_c` — ``radius_ref.c`` compiled with ``-ffp-contract=off`` and OpenMP, using libm's ``fma``.

Both evaluate ``fma(dz, dz, fma(dy, dy, dx*dx)) < (T)(r*r)``, the form the reference's compiled kernel follows (checked against
that kernel on a B200 by ``tests/test_gpu_radius_reference.py``).

The rule follows ``src/opt_radius/mlcg_opt_radius/radius.cu:106-141`` (strict ``<`` on the squared
distance, optional self exclusion, the first ``max_num_neighbors`` hits in index order) and, for
``rule="cluster"``, the ``max_num_neighbors + 1``-then-drop-self behaviour of
``torch_cluster.radius_graph`` 1.6.3 as called from ``src/mlcg/neighbor_list/torch_impl.py:216-224``
with ``flow="target_to_source"`` (row 0 = centre, row 1 = neighbour).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libradius_ref.so")
_SRC = os.path.join(_HERE, "radius_ref.c")
RULES = {"native": 0, "cluster": 1}


def build(force: bool = False) -> str:
    """Compile ``radius_ref.c`` next to itself; returns the path of the shared object."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-o", _SO, _SRC, "-lm"]
        )
    return _SO


_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64p = ctypes.POINTER(ctypes.c_int64)
        for name, fp in (("f32", ctypes.c_float), ("f64", ctypes.c_double)):
            cnt = getattr(_lib, f"radius_ref_{name}_count")
            cnt.restype = ctypes.c_int64
            cnt.argtypes = [ctypes.POINTER(fp), i64p, ctypes.c_int64, ctypes.c_double, ctypes.c_int64,
                            ctypes.c_int, ctypes.c_int, i64p]
            fill = getattr(_lib, f"radius_ref_{name}_fill")
            fill.restype = None
            fill.argtypes = [ctypes.POINTER(fp), i64p, ctypes.c_int64, ctypes.c_double, ctypes.c_int64,
                             ctypes.c_int, ctypes.c_int, i64p, i64p, i64p, ctypes.POINTER(fp)]
        _lib.exclusion_pair_to_ptr_ref.restype = ctypes.c_int
        _lib.exclusion_pair_to_ptr_ref.argtypes = [i64p, ctypes.c_int64, ctypes.c_int64, i64p, i64p]
    return _lib


def _ptr_of(a, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


def _two_sum(a, b):
    s = a + b
    bb = s - a
    return s, (a - (s - bb)) + (b - bb)


def _two_prod(a, b):
    """a*b = p + e exactly (Dekker's product with Veltkamp's splitting; no overflow or underflow at the magnitudes used here)."""
    T = a.dtype.type
    split = T(4097.0) if a.dtype == np.float32 else T(134217729.0)      # 2^12 + 1, 2^27 + 1
    p = a * b
    ca, cb = split * a, split * b
    ah, bh = ca - (ca - a), cb - (cb - b)
    al, bl = a - ah, b - bh
    return p, ((ah * bh - p) + ah * bl + al * bh) + al * bl


def _add_round_to_odd(a, b):
    """a + b rounded to odd: the nearest-rounded sum, moved to its neighbour on the side of the rounding error when the sum
    is inexact and its last mantissa bit is even."""
    s, e = _two_sum(a, b)
    bits = s.view(np.int32 if s.dtype == np.float32 else np.int64)
    fix = (e != 0) & ((bits & 1) == 0)
    toward = np.where(e > 0, np.inf, -np.inf).astype(s.dtype)
    return np.where(fix, np.nextafter(s, toward), s)


def fma_exact(a, b, c):
    """round(a*b + c) with a single rounding, elementwise, in the dtype of the inputs (float32 or float64), from operations
    of that same dtype: exact product, exact sum of its head with c, the two tails added with rounding to odd, one final
    rounding (Boldo and Melquiond's emulation of the fused multiply-add)."""
    a, b, c = np.broadcast_arrays(np.asarray(a), np.asarray(b), np.asarray(c))
    with np.errstate(invalid="ignore", over="ignore"):
        uh, ul = _two_prod(a, b)
        th, tl = _two_sum(c, uh)
        return th + _add_round_to_odd(tl, ul)


def squared_distance(d):
    """fma(dz, dz, fma(dy, dy, dx*dx)) for displacement vectors ``d[..., 3]``."""
    return fma_exact(d[..., 2], d[..., 2], fma_exact(d[..., 1], d[..., 1], d[..., 0] * d[..., 0]))


def batch_to_ptr(batch: np.ndarray, num_structures=None) -> np.ndarray:
    """``ptr[b]`` = first index whose batch id is >= b (radius.py:64-75 uses bucketize for this)."""
    batch = np.asarray(batch, dtype=np.int64)
    B = int(batch.max()) + 1 if num_structures is None else int(num_structures)
    return np.searchsorted(batch, np.arange(B + 1), side="left").astype(np.int64)


def radius_graph_c(pos, ptr, r, max_num_neighbors=1000, loop=False, rule="cluster", with_distance=False):
    """Edges ``[2, E]`` int64 (and distances) from the compiled oracle. ``pos`` is float32 or float64."""
    lib = _load()
    pos = np.ascontiguousarray(pos)
    assert pos.ndim == 2 and pos.shape[1] == 3 and pos.dtype in (np.float32, np.float64)
    tag, ct = ("f32", ctypes.c_float) if pos.dtype == np.float32 else ("f64", ctypes.c_double)
    ptr = np.ascontiguousarray(ptr, dtype=np.int64)
    B, N = len(ptr) - 1, pos.shape[0]
    deg = np.zeros(N, dtype=np.int64)
    E = getattr(lib, f"radius_ref_{tag}_count")(
        _ptr_of(pos, ct), _ptr_of(ptr, ctypes.c_int64), B, float(r), int(max_num_neighbors), int(loop),
        RULES[rule], _ptr_of(deg, ctypes.c_int64))
    off = np.zeros(N + 1, dtype=np.int64)
    np.cumsum(deg, out=off[1:])
    ei = np.empty((2, E), dtype=np.int64)
    dist = np.empty(E, dtype=pos.dtype)
    getattr(lib, f"radius_ref_{tag}_fill")(
        _ptr_of(pos, ct), _ptr_of(ptr, ctypes.c_int64), B, float(r), int(max_num_neighbors), int(loop),
        RULES[rule], _ptr_of(off, ctypes.c_int64), _ptr_of(ei[0], ctypes.c_int64),
        _ptr_of(ei[1], ctypes.c_int64), _ptr_of(dist, ct))
    return (ei, dist) if with_distance else ei


def radius_graph_numpy(pos, ptr, r, max_num_neighbors=1000, loop=False, rule="cluster", with_distance=False, exclude=None):
    """Same rule, all pairs of one structure at a time.

    ``exclude = (xs, y_ptr)`` as :func:`exclusion_pair_to_ptr` returns them (rule "native" only): centre ``i`` never gets a
    neighbour listed in ``xs[y_ptr[i]:y_ptr[i+1]]``, and excluded points do not count towards the cap (radius.cu:122-141)."""
    pos = np.asarray(pos)
    assert exclude is None or rule == "native"
    T = pos.dtype.type
    r2 = T(float(r) * float(r))
    rows0, rows1, dists = [], [], []
    for b in range(len(ptr) - 1):
        lo, hi = int(ptr[b]), int(ptr[b + 1])
        p = pos[lo:hi]
        d = p[None, :, :] - p[:, None, :]          # d[i, j] = pos[j] - pos[i]
        d2 = squared_distance(d)
        hit = d2 < r2
        n = hi - lo
        eye = np.eye(n, dtype=bool)
        if exclude is not None:
            xs, y_ptr = exclude
            for i in range(lo, hi):
                for x in xs[int(y_ptr[i]):int(y_ptr[i + 1])]:
                    if lo <= x < hi:
                        hit[i - lo, int(x) - lo] = False
        if loop:
            counted, cap = hit, max_num_neighbors
        elif rule == "cluster":
            counted, cap = hit, max_num_neighbors + 1   # self counts towards the cap ...
        else:
            counted, cap = hit & ~eye, max_num_neighbors
        rank = np.cumsum(counted, axis=1)               # 1-based rank of each counted hit
        keep = counted & (rank <= cap)
        if not loop:
            keep &= ~eye                                # ... and is dropped afterwards
        i, j = np.nonzero(keep)
        rows0.append(i + lo)
        rows1.append(j + lo)
        dists.append(np.sqrt(d2[i, j]))
    ei = np.stack([np.concatenate(rows0), np.concatenate(rows1)]).astype(np.int64) if rows0 else np.zeros((2, 0), np.int64)
    if with_distance:
        return ei, (np.concatenate(dists) if dists else np.zeros(0, pos.dtype))
    return ei


def pbc_repeats(cells, pbc, r):
    """Copies per cell vector, compute_images (src/mlcg/neighbor_list/torch_impl.py:113-120): ceil(r * norm of the rows of the
    transposed inverse cell), zero along non-periodic directions.  cells [B,3,3], pbc [B,3] bool -> [B,3] int."""
    cells = np.asarray(cells).reshape(-1, 3, 3)
    pbc = np.asarray(pbc).reshape(-1, 3).astype(bool)
    recip = np.transpose(np.linalg.inv(cells), (0, 2, 1))
    inv_d = np.sqrt((recip * recip).sum(-1))
    rep = np.ceil(cells.dtype.type(r) * inv_d).astype(np.int64)
    return np.where(pbc, rep, 0)


def radius_graph_pbc_numpy(pos, ptr, cells, pbc, r, max_num_neighbors=1000, loop=False):
    """torch_neighbor_list_pbc (torch_impl.py:252-329) restated: every structure is copied along its periodic cell vectors
    (shift triples in cartesian-product order, last index fastest; copy = pos + shift, rounded once), the original points are
    searched against all copies (squared distance < r*r, neighbours in the order of the copies, at most
    ``max_num_neighbors``), the copy index is folded back to the point index, and the pair (i, i, zero shift) is dropped
    unless ``loop``.  The shift vector is ((s1 c1 + s2 c2) + s3 c3) with separately rounded operations.
    Returns (edge_index [2,E] with row 0 = centre, cell_shifts [E,3])."""
    pos = np.asarray(pos)
    T = pos.dtype.type
    cells = np.asarray(cells, dtype=pos.dtype).reshape(-1, 3, 3)
    reps = pbc_repeats(cells, pbc, r)
    r2 = T(float(r) * float(r))
    rows0, rows1, shifts_out = [], [], []
    for b in range(len(ptr) - 1):
        lo, hi = int(ptr[b]), int(ptr[b + 1])
        p, n, c = pos[lo:hi], hi - lo, cells[b]
        n1, n2, n3 = (int(v) for v in reps[b])
        idx = np.array([(a, bb, cc) for a in range(-n1, n1 + 1) for bb in range(-n2, n2 + 1) for cc in range(-n3, n3 + 1)], dtype=np.int64)
        sf = idx.astype(pos.dtype)
        shifts = (sf[:, 0:1] * c[0][None, :] + sf[:, 1:2] * c[1][None, :]) + sf[:, 2:3] * c[2][None, :]     # [S,3]
        images = (p[None, :, :] + shifts[:, None, :]).reshape(-1, 3)                                   # copy-major
        d = images[None, :, :] - p[:, None, :]
        d2 = squared_distance(d)
        hit = d2 < r2
        keep = hit & (np.cumsum(hit, axis=1) <= max_num_neighbors)
        i, im = np.nonzero(keep)
        j, s = im % n, im // n
        if not loop:
            central = (idx[s] == 0).all(axis=1)
            sel = ~(central & (i == j))
            i, j, s = i[sel], j[sel], s[sel]
        rows0.append(i + lo)
        rows1.append(j + lo)
        shifts_out.append(shifts[s])
    if not rows0:
        return np.zeros((2, 0), np.int64), np.zeros((0, 3), pos.dtype)
    return np.stack([np.concatenate(rows0), np.concatenate(rows1)]).astype(np.int64), np.concatenate(shifts_out).astype(pos.dtype)


def exclusion_pair_to_ptr(pairs, num_nodes):
    """``exclusion_pairs.cpp:7-62``: pairs ``[2, P]`` (x, y) -> xs sorted by (y, x), CSR pointer over y."""
    lib = _load()
    pairs = np.ascontiguousarray(pairs, dtype=np.int64)
    P = pairs.shape[1]
    xs = np.empty(P, dtype=np.int64)
    y_ptr = np.empty(num_nodes + 1, dtype=np.int64)
    rc = lib.exclusion_pair_to_ptr_ref(_ptr_of(pairs, ctypes.c_int64), P, int(num_nodes),
                                       _ptr_of(xs, ctypes.c_int64), _ptr_of(y_ptr, ctypes.c_int64))
    assert rc == 0
    return xs, y_ptr
