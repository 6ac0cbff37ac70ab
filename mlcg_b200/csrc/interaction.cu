// One interaction block per call: the kernel sequences of the eval-mode forward and force pass of
//   x_new = x + lin( tanh( lin2( sum_j lin1(x)_j * W(d_ij) ) ) )            src/mlcg/nn/schnet.py:150, 252-262, 340-350
// issued from C, so that a host in any language pays one foreign call per block and direction instead of one per kernel
// (for small systems the evaluation time is the host's launch path, not the GPU).  Symmetric edge lists only (one filter
// row per unordered pair); everything else goes through the individual entry points.
#include "common.cuh"

using namespace mlcgb;

extern "C" {

int mlcgb_interaction_forward(const void *x, const void *d, const int64_t *ptr_out, const int32_t *nbr_out, const int32_t *sel,
                              const int32_t *pair_of, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower,
                              double conv_upper, const void *W1, const void *fA1, const void *fb1, const void *fA2, const void *W2,
                              const void *b2, const void *W3, const void *b3, int64_t N, int64_t E, int64_t P, int64_t H, int64_t F,
                              int64_t H2, int precision, void *xl, void *Wp, void *agg, void *a, void *out, int32_t *status,
                              void *stream) {
    if (N < 0 || E < 0 || P < 0 || !status) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!x || !ptr_out || !W1 || !W2 || !b2 || !W3 || !b3 || !xl || !agg || !a || !out) return MLCGB_E_ARG;
    if (P > 0 && (!d || !nbr_out || !sel || !pair_of || !Wp)) return MLCGB_E_ARG;
    if (N < 128 || (H & 3) || (F & 3) || (H2 & 3) || H > 128 || F != 128 || H2 > 128) return MLCGB_E_LIMIT;
    int rc = mlcgb_gemm_tc_fused(0, x, W1, nullptr, nullptr, 0, N, F, H, xl, status, stream);                 // lin1 (no bias)
    if (rc) return rc;
    rc = mlcgb_filter_forward(d, P, sel, nullptr, rbf, conv_cutoff_kind, conv_lower, conv_upper, fA1, fb1, fA2, F, precision, Wp, status, stream);
    if (rc) return rc;
    rc = mlcgb_seg_mul_sum(xl, Wp, MLCGB_F32, ptr_out, nbr_out, pair_of, N, P, F, agg, stream);                // aggregation
    if (rc) return rc;
    rc = mlcgb_gemm_tc_fused(0, agg, W2, b2, nullptr, 1, N, H2, F, a, status, stream);                         // lin2 + tanh
    if (rc) return rc;
    return mlcgb_gemm_tc_fused(0, a, W3, b3, x, 2, N, H, H2, out, status, stream);                             // lin + residual
}

int mlcgb_interaction_backward(const void *g, const void *a, const void *Wp, const void *xl, const void *d, const int64_t *ptr_out,
                               const int32_t *nbr_out, const int32_t *sel, const int32_t *pair_of, const int32_t *twin,
                               const int32_t *row0, const int32_t *row1, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind,
                               double conv_lower, double conv_upper, const void *W1, const void *fA1, const void *fb1,
                               const void *fA2, const void *W2, const void *W3, int64_t N, int64_t E, int64_t P, int64_t H, int64_t F,
                               int64_t H2, int precision, void *gy, void *gagg, void *gxl, void *gx /* or NULL */,
                               void *gd /* [E] or NULL */, int32_t *status, void *stream) {
    if (N < 0 || E < 0 || P < 0 || !status) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!g || !a || !xl || !ptr_out || !W1 || !W2 || !W3 || !gy || !gagg || !gxl) return MLCGB_E_ARG;
    if (P > 0 && (!d || !nbr_out || !sel || !pair_of || !twin || !row0 || !row1 || !Wp)) return MLCGB_E_ARG;
    if (N < 128 || (H & 3) || (F & 3) || (H2 & 3) || H > 128 || F != 128 || H2 > 128) return MLCGB_E_LIMIT;
    int rc = mlcgb_gemm_tc_fused(1, g, W3, nullptr, a, 3, N, H2, H, gy, status, stream);                      // through lin and tanh
    if (rc) return rc;
    rc = mlcgb_gemm_tc_fused(1, gy, W2, nullptr, nullptr, 0, N, F, H2, gagg, status, stream);                  // through lin2
    if (rc) return rc;
    if (gx) {
        rc = mlcgb_seg_mul_sum(gagg, Wp, MLCGB_F32, ptr_out, nbr_out, pair_of, N, P, F, gxl, stream);          // to the gathered features
        if (rc) return rc;
        rc = mlcgb_gemm_tc_fused(1, gxl, W1, nullptr, g, 2, N, H, F, gx, status, stream);                     // through lin1, + residual branch
        if (rc) return rc;
    }
    if (gd && E > 0)
        rc = mlcgb_filter_backward(d, P, sel, twin, rbf, conv_cutoff_kind, conv_lower, conv_upper, fA1, fb1, fA2, F, precision, row0, row1,
                                   xl, gagg, N, gd, status, stream);
    return rc;
}

}  // extern "C"
