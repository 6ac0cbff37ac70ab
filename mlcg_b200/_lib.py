"""ctypes binding of ``libmlcg_b200.so`` — the C ABI declared in ``include/mlcg_b200.h``.

The library is the only compute back end of this package.  If it cannot be loaded the import of
:mod:`mlcg_b200` still works (so CPU-only tooling can inspect the modules), but every operator call
raises: there is no CPU or pure-torch fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
#: the library next to this file, unless MLCGB_LIBRARY names another build of the same sources (e.g. one with extra checks)
LIB_PATH = os.environ.get("MLCGB_LIBRARY") or os.path.join(_HERE, "libmlcg_b200.so")

c_i64, c_int, c_dbl, c_vp, c_sz = ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t


class RbfSpecStruct(ctypes.Structure):
    """Mirror of ``mlcgb_rbf_spec``."""

    _fields_ = [("kind", c_int), ("num_rbf", c_int), ("cutoff_kind", c_int), ("reserved", c_int),
                ("lower", c_dbl), ("upper", c_dbl), ("alpha", c_dbl), ("p0", c_vp), ("p1", c_vp)]


class SchnetBlockStruct(ctypes.Structure):
    """Mirror of ``mlcgb_schnet_block``."""

    _fields_ = [(n, c_vp) for n in ("lin1_w", "filter_w1", "filter_b1", "filter_w2", "lin2_w", "lin2_b", "lin_w", "lin_b")]


class SchnetWeightsStruct(ctypes.Structure):
    """Mirror of ``mlcgb_schnet_weights``."""

    _fields_ = [("hidden", c_i64), ("filters", c_i64), ("conv_out", c_i64), ("head_width", c_i64), ("num_blocks", c_i64), ("num_types", c_i64),
                ("blocks", ctypes.POINTER(SchnetBlockStruct)), ("embedding", c_vp), ("head_W", c_vp), ("head_b", c_vp), ("head_out", c_vp),
                ("head_out_b", c_vp)]


class PriorListStruct(ctypes.Structure):
    """Mirror of ``mlcgb_prior_list``."""

    _fields_ = [("kind", c_int), ("n_params", c_int), ("symmetric", c_int), ("reserved", c_int), ("M", c_i64), ("idx", c_vp), ("params", c_vp),
                ("run_ptr", c_vp), ("n_runs", c_i64)]


MAX_PRIOR_SEGMENTS = 8

# name -> (restype, argtypes); one entry per symbol declared in include/mlcg_b200.h
SIGNATURES = {
    "mlcgb_strerror": (ctypes.c_char_p, [c_int]),
    "mlcgb_last_cuda_error": (c_int, []),
    "mlcgb_version": (c_int, []),
    "mlcgb_timeline_begin": (c_int, []),
    "mlcgb_timeline_end": (c_int, []),
    "mlcgb_timeline_entry": (c_int, [c_int, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(c_i64), ctypes.POINTER(c_dbl)]),
    "mlcgb_batch_to_ptr": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_radius_workspace_bytes": (c_sz, [c_i64, c_i64, c_int]),
    "mlcgb_radius_count": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_dbl, c_i64, c_int, c_int, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_radius_fill": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_dbl, c_int, c_vp, c_sz, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_radius_count_excl": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_dbl, c_i64, c_int, c_vp, c_vp, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_radius_fill_excl": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_dbl, c_int, c_vp, c_vp, c_vp, c_sz, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp,
                                       c_vp, c_vp]),
    "mlcgb_radius_graph_static": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_dbl, c_i64, c_int, c_int, c_vp, c_vp, c_i64, c_vp,
                                          ctypes.POINTER(c_i64), c_vp, c_vp]),
    "mlcgb_edge_twin": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "mlcgb_pair_plan_workspace_bytes": (c_sz, [c_i64]),
    "mlcgb_pair_plan": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_pair_index": (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp]),
    "mlcgb_edge_diff": (c_int, [c_vp, c_int, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "mlcgb_edge_distance": (c_int, [c_vp, c_int, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "mlcgb_edge_distance_backward": (c_int, [c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_node_scatter_diff": (c_int, [c_vp, c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_rbf_expand": (c_int, [c_vp, c_int, c_i64, ctypes.POINTER(RbfSpecStruct), c_int, c_vp, c_vp]),
    "mlcgb_rbf_contract": (c_int, [c_vp, c_vp, c_int, c_i64, ctypes.POINTER(RbfSpecStruct), c_int, c_vp, c_vp]),
    "mlcgb_rbf_param_workspace_bytes": (c_sz, [c_i64, c_int, c_int]),
    "mlcgb_rbf_param_contract": (c_int, [c_vp, c_vp, c_vp, c_int, c_i64, ctypes.POINTER(RbfSpecStruct), c_int, c_vp, c_sz, c_vp, c_vp, c_vp]),
    "mlcgb_seg_mul_sum": (c_int, [c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_edge_mul": (c_int, [c_vp, c_vp, c_int, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_pair_mul": (c_int, [c_vp, c_vp, c_int, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_gemm_workspace_bytes": (c_sz, [c_int, c_i64, c_i64, c_i64, c_int]),
    "mlcgb_gemm": (c_int, [c_int, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "mlcgb_gemm_tc_supported": (c_int, [c_int, c_i64, c_i64, c_i64]),
    "mlcgb_gemm_tc_workspace_bytes": (c_sz, [c_int, c_i64, c_i64, c_i64]),
    "mlcgb_gemm_tc": (c_int, [c_int, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp, c_vp]),
    "mlcgb_gemm_tc_chain2": (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_tanh_grad": (c_int, [c_int, c_vp, c_vp, c_vp, c_int, c_i64, c_vp, c_vp]),
    "mlcgb_row_scale": (c_int, [c_vp, c_vp, c_int, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_row_dot": (c_int, [c_vp, c_vp, c_int, c_i64, c_i64, c_vp, c_vp]),
    "mlcgb_gemm_tc_tn_colsum": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_sz, c_vp, c_vp]),
    "mlcgb_interaction_forward": (c_int, [c_vp] * 6 + [c_vp, c_int, c_dbl, c_dbl] + [c_vp] * 8 + [c_i64] * 6 + [c_int] + [c_vp] * 8),
    "mlcgb_interaction_backward": (c_int, [c_vp] * 13 + [c_vp, c_int, c_dbl, c_dbl] + [c_vp] * 6 + [c_i64] * 6 + [c_int] + [c_vp] * 7),
    "mlcgb_schnet_eval_workspace_bytes": (c_sz, [c_i64] * 8),
    "mlcgb_radius_pbc_workspace_bytes": (c_sz, [c_i64]),
    "mlcgb_radius_pbc_count": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_vp, c_vp, c_dbl, c_i64, c_int, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_radius_pbc_fill": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_vp, c_vp, c_dbl, c_i64, c_int, c_vp, c_sz, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp,
                                      c_vp, c_vp]),
    "mlcgb_radius_graph_capacity": (c_int, [c_vp, c_int, c_vp, c_i64, c_i64, c_dbl, c_i64, c_int, c_int, c_vp, c_sz, c_vp, c_vp, c_i64, c_vp, c_vp,
                                            c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_filter_forward_counted": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, ctypes.POINTER(RbfSpecStruct), c_int, c_dbl, c_dbl, c_vp, c_vp, c_vp, c_i64,
                                             c_int, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_filter_hidden_bytes": (c_sz, [c_i64]),
    "mlcgb_filter_backward_counted": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, ctypes.POINTER(RbfSpecStruct), c_int, c_dbl, c_dbl, c_vp, c_vp, c_vp, c_i64,
                                              c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_int, c_vp, c_vp]),
    "mlcgb_schnet_eval_counted": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_int, c_dbl,
                                          c_dbl, c_vp, c_int, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_schnet_eval": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_int, c_dbl, c_dbl,
                                  c_vp, c_int, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_gemm_tc_fused": (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "mlcgb_filter_forward": (c_int, [c_vp, c_i64, c_vp, c_vp, ctypes.POINTER(RbfSpecStruct), c_int, c_dbl, c_dbl, c_vp, c_vp, c_vp, c_i64, c_int, c_vp, c_vp, c_vp,
                                     c_vp]),
    "mlcgb_filter_backward": (c_int, [c_vp, c_i64, c_vp, c_vp, ctypes.POINTER(RbfSpecStruct), c_int, c_dbl, c_dbl, c_vp, c_vp, c_vp, c_i64, c_int,
                                      c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_segment_sum": (c_int, [c_vp, c_int, c_vp, c_i64, c_vp, c_vp]),
    "mlcgb_langevin_first_half": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_dbl, c_dbl, c_dbl, c_vp]),
    "mlcgb_langevin_second_half": (c_int, [c_vp, c_vp, c_vp, c_int, c_i64, c_dbl, c_vp]),
    "mlcgb_prior_terms": (c_int, [c_int, c_vp, c_int, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "mlcgb_prior_eval_workspace_bytes": (c_sz, [c_int, c_i64, c_i64, c_int]),
    "mlcgb_prior_eval": (c_int, [c_int, ctypes.POINTER(PriorListStruct), c_vp, c_int, c_vp, c_i64, c_i64, c_vp, c_vp, c_int, c_vp, c_sz, c_vp, c_vp]),
}

_lib = None
_load_error = None


class ExtensionMissing(RuntimeError):
    pass


def load():
    """Return the loaded library or raise :class:`ExtensionMissing` (never falls back)."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        _load_error = f"{LIB_PATH} not found; build it with `python -m mlcg_b200.build`"
        raise ExtensionMissing(_load_error)
    try:
        lib = ctypes.CDLL(LIB_PATH)
    except OSError as exc:  # e.g. libcudart missing
        _load_error = f"cannot load {LIB_PATH}: {exc}"
        raise ExtensionMissing(_load_error) from exc
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(code: int, what: str):
    if code != 0:
        lib = load()
        msg = lib.mlcgb_strerror(code).decode()
        extra = f" (cudaError {lib.mlcgb_last_cuda_error()})" if code == -3 else ""
        raise RuntimeError(f"mlcg_b200: {what} failed: {msg}{extra}")
