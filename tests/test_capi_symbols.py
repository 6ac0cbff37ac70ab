"""The C-ABI library loads and exports exactly what include/mlcg_b200.h declares (no compute calls)."""
import ctypes
import os
import re

import pytest

from mlcg_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mlcg_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlcgb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_something():
    syms = declared_symbols()
    assert "mlcgb_radius_count" in syms and "mlcgb_seg_mul_sum" in syms and len(syms) >= 15


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        from mlcg_b200 import build
        build.build()
    try:
        lib = ctypes.CDLL(_lib.LIB_PATH)
    except OSError as exc:
        pytest.skip(f"library cannot be loaded on this machine: {exc}")
    for name in declared_symbols():
        assert hasattr(lib, name), name
    lib.mlcgb_strerror.restype = ctypes.c_char_p
    assert lib.mlcgb_strerror(0) == b"ok" and b"workspace" in lib.mlcgb_strerror(-2)
    assert lib.mlcgb_version() >= 100


def test_workspace_size_queries_are_host_only():
    lib = _lib.load()
    assert lib.mlcgb_radius_workspace_bytes(0, 0, 0) >= 0
    small, big = lib.mlcgb_radius_workspace_bytes(1000, 10, 0), lib.mlcgb_radius_workspace_bytes(100000, 10, 0)
    assert 0 < small < big
    assert lib.mlcgb_gemm_workspace_bytes(0, 1000, 128, 128, 0) == 0
    assert lib.mlcgb_gemm_workspace_bytes(2, 128, 128, 1000000, 0) > 0


def test_radius_workspace_fits_the_built_in_scratch_at_its_limits():
    """`mlcgb_radius_graph_static` owns 17 x 512 KiB of scratch and accepts up to 65 536 points in 8 192 structures: the
    workspace of the two-call interface at those sizes must fit in both precisions, and grow with the points (the hit masks)."""
    lib = _lib.load()
    scratch = 17 << 19
    f32, f64 = lib.mlcgb_radius_workspace_bytes(65536, 8192, 0), lib.mlcgb_radius_workspace_bytes(65536, 8192, 1)
    assert 0 < f64 <= scratch and 0 < f32 <= scratch
    per_point = (lib.mlcgb_radius_workspace_bytes(200000, 10, 0) - lib.mlcgb_radius_workspace_bytes(100000, 10, 0)) / 100000
    assert 100 <= per_point <= 160            # points, cell tables, indices, 24 mask words, a flag
