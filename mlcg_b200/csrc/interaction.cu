// One interaction block per call: the kernel sequences of the eval-mode forward and force pass of
//   x_new = x + lin( tanh( lin2( sum_j lin1(x)_j * W(d_ij) ) ) )            src/mlcg/nn/schnet.py:150, 252-262, 340-350
// issued from C, so that a host in any language pays one foreign call per block and direction instead of one per kernel
// (for small systems the evaluation time is the host's launch path, not the GPU).  Symmetric edge lists only (one filter
// row per unordered pair); everything else goes through the individual entry points.
#include "common.cuh"

using namespace mlcgb;

extern "C" {

static int interaction_forward_counted(const void *x, const void *d, const int64_t *ptr_out, const int32_t *nbr_out, const int32_t *sel,
                                      const int32_t *pair_of, const int64_t *pairs_dev, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind,
                                      double conv_lower, double conv_upper, const void *W1, const void *fA1, const void *fb1,
                                      const void *fA2, const void *W2, const void *b2, const void *W3, const void *b3, int64_t N, int64_t E,
                                      int64_t P, int64_t H, int64_t F, int64_t H2, int precision, void *xl, void *Wp, void *hsave, void *agg, void *a,
                                      void *out, int32_t *status, void *stream);
static int interaction_backward_counted(const void *g, const void *a, const void *Wp, const void *xl, const void *hsave, const void *d, const int64_t *ptr_out,
                                       const int32_t *nbr_out, const int32_t *sel, const int32_t *pair_of, const int32_t *twin,
                                       const int64_t *pairs_dev, const int32_t *row0, const int32_t *row1, const mlcgb_rbf_spec *rbf,
                                       int conv_cutoff_kind, double conv_lower, double conv_upper, const void *W1, const void *fA1,
                                       const void *fb1, const void *fA2, const void *W2, const void *W3, int64_t N, int64_t E, int64_t P,
                                       int64_t H, int64_t F, int64_t H2, int precision, void *gy, void *gagg, void *gxl, void *gx,
                                       void *gd, int gd_accumulate, int32_t *status, void *stream);

int mlcgb_interaction_forward(const void *x, const void *d, const int64_t *ptr_out, const int32_t *nbr_out, const int32_t *sel,
                              const int32_t *pair_of, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower,
                              double conv_upper, const void *W1, const void *fA1, const void *fb1, const void *fA2, const void *W2,
                              const void *b2, const void *W3, const void *b3, int64_t N, int64_t E, int64_t P, int64_t H, int64_t F,
                              int64_t H2, int precision, void *xl, void *Wp, void *hsave, void *agg, void *a, void *out,
                              int32_t *status, void *stream) {
    return interaction_forward_counted(x, d, ptr_out, nbr_out, sel, pair_of, nullptr, rbf, conv_cutoff_kind, conv_lower, conv_upper, W1,
                                             fA1, fb1, fA2, W2, b2, W3, b3, N, E, P, H, F, H2, precision, xl, Wp, hsave, agg, a, out, status,
                                             stream);
}

// pairs_dev: NULL, or the number of pairs in device memory; P then only sizes the buffers (see mlcgb_filter_forward_counted)
static int interaction_forward_counted(const void *x, const void *d, const int64_t *ptr_out, const int32_t *nbr_out, const int32_t *sel,
                                      const int32_t *pair_of, const int64_t *pairs_dev, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind,
                                      double conv_lower, double conv_upper, const void *W1, const void *fA1, const void *fb1,
                                      const void *fA2, const void *W2, const void *b2, const void *W3, const void *b3, int64_t N, int64_t E,
                                      int64_t P, int64_t H, int64_t F, int64_t H2, int precision, void *xl, void *Wp, void *hsave, void *agg, void *a,
                                      void *out, int32_t *status, void *stream) {
    if (N < 0 || E < 0 || P < 0 || !status) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!x || !ptr_out || !W1 || !W2 || !b2 || !W3 || !b3 || !xl || !agg || !a || !out) return MLCGB_E_ARG;
    if (P > 0 && (!d || !nbr_out || !sel || !pair_of || !Wp)) return MLCGB_E_ARG;
    if (N < 128 || (H & 3) || (F & 3) || (H2 & 3) || H > 128 || F != 128 || H2 > 128) return MLCGB_E_LIMIT;
    int rc = mlcgb_gemm_tc_fused(0, x, W1, nullptr, nullptr, 0, N, F, H, xl, status, stream);                 // lin1 (no bias)
    if (rc) return rc;
    rc = mlcgb_filter_forward_counted(d, P, pairs_dev, sel, nullptr, rbf, conv_cutoff_kind, conv_lower, conv_upper, fA1, fb1, fA2, F, precision,
                                      Wp, hsave, status, stream);
    if (rc) return rc;
    rc = mlcgb_seg_mul_sum(xl, Wp, MLCGB_F32, ptr_out, nbr_out, pair_of, N, P, F, agg, stream);                // aggregation
    if (rc) return rc;
    if (H == 128 && F == 128 && H2 == 128) {                                                                   // lin2 + tanh -> lin + residual, one kernel
        rc = mlcgb_gemm_tc_chain2(0, agg, W2, b2, W3, b3, x, N, a, out, status, stream);
        if (rc != MLCGB_E_LIMIT) return rc;
    }
    rc = mlcgb_gemm_tc_fused(0, agg, W2, b2, nullptr, 1, N, H2, F, a, status, stream);                         // lin2 + tanh
    if (rc) return rc;
    return mlcgb_gemm_tc_fused(0, a, W3, b3, x, 2, N, H, H2, out, status, stream);                             // lin + residual
}

int mlcgb_interaction_backward(const void *g, const void *a, const void *Wp, const void *xl, const void *hsave, const void *d, const int64_t *ptr_out,
                               const int32_t *nbr_out, const int32_t *sel, const int32_t *pair_of, const int32_t *twin,
                               const int32_t *row0, const int32_t *row1, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind,
                               double conv_lower, double conv_upper, const void *W1, const void *fA1, const void *fb1,
                               const void *fA2, const void *W2, const void *W3, int64_t N, int64_t E, int64_t P, int64_t H, int64_t F,
                               int64_t H2, int precision, void *gy, void *gagg, void *gxl, void *gx /* or NULL */,
                               void *gd /* [E] or NULL */, int32_t *status, void *stream) {
    return interaction_backward_counted(g, a, Wp, xl, hsave, d, ptr_out, nbr_out, sel, pair_of, twin, nullptr, row0, row1, rbf, conv_cutoff_kind,
                                              conv_lower, conv_upper, W1, fA1, fb1, fA2, W2, W3, N, E, P, H, F, H2, precision, gy, gagg, gxl,
                                              gx, gd, 0, status, stream);
}

static int interaction_backward_counted(const void *g, const void *a, const void *Wp, const void *xl, const void *hsave, const void *d, const int64_t *ptr_out,
                                       const int32_t *nbr_out, const int32_t *sel, const int32_t *pair_of, const int32_t *twin,
                                       const int64_t *pairs_dev, const int32_t *row0, const int32_t *row1, const mlcgb_rbf_spec *rbf,
                                       int conv_cutoff_kind, double conv_lower, double conv_upper, const void *W1, const void *fA1,
                                       const void *fb1, const void *fA2, const void *W2, const void *W3, int64_t N, int64_t E, int64_t P,
                                       int64_t H, int64_t F, int64_t H2, int precision, void *gy, void *gagg, void *gxl,
                                       void *gx /* or NULL */, void *gd /* [E] or NULL */, int gd_accumulate, int32_t *status,
                                       void *stream) {
    if (N < 0 || E < 0 || P < 0 || !status) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!g || !a || !xl || !ptr_out || !W1 || !W2 || !W3 || !gy || !gagg || !gxl) return MLCGB_E_ARG;
    if (P > 0 && (!d || !nbr_out || !sel || !pair_of || !twin || !row0 || !row1 || !Wp)) return MLCGB_E_ARG;
    if (N < 128 || (H & 3) || (F & 3) || (H2 & 3) || H > 128 || F != 128 || H2 > 128) return MLCGB_E_LIMIT;
    int rc = MLCGB_E_LIMIT;
    if (H == 128 && F == 128 && H2 == 128)                                                                     // through lin, tanh and lin2, one kernel
        rc = mlcgb_gemm_tc_chain2(1, g, W3, nullptr, W2, nullptr, a, N, nullptr, gagg, status, stream);
    if (rc == MLCGB_E_LIMIT) {
        rc = mlcgb_gemm_tc_fused(1, g, W3, nullptr, a, 3, N, H2, H, gy, status, stream);                      // through lin and tanh
        if (rc) return rc;
        rc = mlcgb_gemm_tc_fused(1, gy, W2, nullptr, nullptr, 0, N, F, H2, gagg, status, stream);              // through lin2
    }
    if (rc) return rc;
    if (gx) {
        rc = mlcgb_seg_mul_sum(gagg, Wp, MLCGB_F32, ptr_out, nbr_out, pair_of, N, P, F, gxl, stream);          // to the gathered features
        if (rc) return rc;
        rc = mlcgb_gemm_tc_fused(1, gxl, W1, nullptr, g, 2, N, H, F, gx, status, stream);                     // through lin1, + residual branch
        if (rc) return rc;
    }
    if (gd && E > 0)
        rc = mlcgb_filter_backward_counted(d, P, pairs_dev, sel, twin, rbf, conv_cutoff_kind, conv_lower, conv_upper, fA1, fb1, fA2, F, precision,
                                           row0, row1, xl, gagg, N, hsave, gd, gd_accumulate, status, stream);
    return rc;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// The whole SchNet evaluation — embedding, interaction blocks, output network, per-structure sum and the force pass — as
// one kernel sequence issued from C (src/mlcg/nn/schnet.py:116-162 and its derivative, src/mlcg/nn/gradients.py:191-230).
// ------------------------------------------------------------------------------------------------
namespace mlcgb {

__global__ void embedding_rows_kernel(const float *__restrict__ table, const int64_t *__restrict__ types, int64_t N, int64_t H, int64_t T,
                                      float *__restrict__ x, int32_t *__restrict__ status) {
    const int64_t Hv = H >> 2, total = N * Hv;
    pdl_wait();
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = t / Hv, c = t - n * Hv;
        int64_t ty = types[n];
        if (ty < 0 || ty >= T) {
            atomicOr(status, (int)kBadIndex);
            ty = 0;
        }
        reinterpret_cast<float4 *>(x)[t] = __ldg(reinterpret_cast<const float4 *>(table + ty * H) + c);
    }
}

// e[n] = sum_f a[n,f] w[f] + b: the last Linear layer of the output network (one output); one warp per node
__global__ void head_out_kernel(const float *__restrict__ a, const float *__restrict__ w, const float *__restrict__ b, int64_t N, int64_t F,
                                float *__restrict__ e) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    pdl_wait();
    for (int64_t n = warp; n < N; n += nwarps) {
        float s = 0.f;
        for (int64_t f = lane; f < F; f += 32) s = fmaf(a[n * F + f], w[f], s);
        s = warp_sum(s);
        if (lane == 0) e[n] = s + (b ? b[0] : 0.f);
    }
}

static inline int64_t up4(int64_t n) { return (n + 3) & ~(int64_t)3; }

struct SchnetLayout {
    int64_t d, x[2], g[2], agg, gy, gxl, ah, en, gd, block0, block_stride, xl_off, a_off, wp_off, h_off, total;
};
static SchnetLayout schnet_layout(int64_t N, int64_t E, int64_t P, int64_t H, int64_t F, int64_t H2, int64_t Wh, int64_t L) {
    SchnetLayout o;
    int64_t at = 0;
    auto take = [&](int64_t n) { const int64_t r = at; at += up4(n); return r; };
    o.d = take(E);
    o.x[0] = take(N * H); o.x[1] = take(N * H);
    o.g[0] = take(N * H); o.g[1] = take(N * H);
    o.agg = take(N * F); o.gy = take(N * H2); o.gxl = take(N * F);
    o.ah = take(N * Wh); o.en = take(N);
    o.gd = take(E);
    o.xl_off = 0; o.a_off = up4(N * F); o.wp_off = o.a_off + up4(N * H2);
    o.h_off = o.wp_off + up4(P * F);                                         // hidden layer of the filter network, whole tiles
    o.block_stride = o.h_off + (int64_t)(mlcgb_filter_hidden_bytes(P) / sizeof(float));
    o.block0 = at;
    at += L * o.block_stride;
    o.total = at;
    return o;
}

}  // namespace mlcgb

extern "C" {

size_t mlcgb_schnet_eval_workspace_bytes(int64_t N, int64_t E, int64_t P, int64_t H, int64_t F, int64_t H2, int64_t head_width,
                                         int64_t num_blocks) {
    if (N < 0 || E < 0 || P < 0 || H <= 0 || F <= 0 || H2 <= 0 || head_width <= 0 || num_blocks < 0) return 0;
    return (size_t)schnet_layout(N, E, P, H, F, H2, head_width, num_blocks).total * sizeof(float);
}

int mlcgb_schnet_eval(const void *pos, const int64_t *types, const int64_t *struct_ptr, int64_t N, int64_t B, const int32_t *row0,
                      const int32_t *row1, const int64_t *offsets, const int32_t *sel, const int32_t *pair_of, const int32_t *twin,
                      int64_t E, int64_t P, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper,
                      const mlcgb_schnet_weights *w, int precision, void *workspace, size_t workspace_bytes, void *energy,
                      void *grad_pos, int32_t *status, void *stream) {
    return mlcgb_schnet_eval_counted(pos, types, struct_ptr, N, B, row0, row1, offsets, sel, pair_of, twin, E, P, nullptr, rbf,
                                     conv_cutoff_kind, conv_lower, conv_upper, w, precision, workspace, workspace_bytes, energy, grad_pos,
                                     status, stream);
}

// counts: NULL, or {edges, pairs} in device memory as mlcgb_radius_graph_capacity leaves them.  E and P are then the
// capacities of the index arrays (whose entries past the live ones must be valid node / edge indices, e.g. zero): the
// edge-sized elementwise kernels run over the capacity, the filter kernels over the live pairs, everything else over nodes.
int mlcgb_schnet_eval_counted(const void *pos, const int64_t *types, const int64_t *struct_ptr, int64_t N, int64_t B,
                              const int32_t *row0, const int32_t *row1, const int64_t *offsets, const int32_t *sel,
                              const int32_t *pair_of, const int32_t *twin, int64_t E, int64_t P, const int64_t *counts,
                              const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper,
                              const mlcgb_schnet_weights *w, int precision, void *workspace, size_t workspace_bytes, void *energy,
                              void *grad_pos, int32_t *status, void *stream) {
    const int64_t *pairs_dev = counts ? counts + 1 : nullptr;
    if (N < 0 || B < 0 || E < 0 || P < 0 || !w || !status || !energy || !struct_ptr) return MLCGB_E_ARG;
    if (B == 0) return MLCGB_OK;
    const int64_t H = w->hidden, F = w->filters, H2 = w->conv_out, Wh = w->head_width, L = w->num_blocks;
    if (N < 128 || F != 128 || H > 128 || H2 > 128 || Wh > 128 || (H & 3) || (H2 & 3) || (Wh & 3) || L < 1) return MLCGB_E_LIMIT;
    if (!pos || !types || !offsets || !w->embedding || !w->blocks || !w->head_W || !w->head_b || !w->head_out || !workspace) return MLCGB_E_ARG;
    if (E > 0 && (!row0 || !row1 || !sel || !pair_of || !twin || 2 * P != E)) return MLCGB_E_ARG;
    const SchnetLayout lay = schnet_layout(N, E, P, H, F, H2, Wh, L);
    if (workspace_bytes < (size_t)lay.total * sizeof(float)) return MLCGB_E_WORKSPACE;
    float *ws = (float *)workspace;
    auto st = (cudaStream_t)stream;
    float *d = ws + lay.d;
    int rc = mlcgb_edge_distance(pos, MLCGB_F32, row0, row1, E, N, d, status, stream);
    if (rc) return rc;
    {
        TimelineScope timeline_scope("embedding", stream);
        launch_pdl(embedding_rows_kernel, dim3(grid_for(N * (H >> 2), 256)), dim3(256), 0, st, (const float *)w->embedding, types, N, H, w->num_types, ws + lay.x[0], status);
    }
    int cur = 0;
    for (int64_t l = 0; l < L; l++) {
        const mlcgb_schnet_block &bw = w->blocks[l];
        float *blk = ws + lay.block0 + l * lay.block_stride;
        rc = interaction_forward_counted(ws + lay.x[cur], d, offsets, row1, sel, pair_of, pairs_dev, rbf, conv_cutoff_kind, conv_lower, conv_upper, bw.lin1_w,
                                       bw.filter_w1, bw.filter_b1, bw.filter_w2, bw.lin2_w, bw.lin2_b, bw.lin_w, bw.lin_b, N, E, P, H, F, H2,
                                       precision, blk + lay.xl_off, blk + lay.wp_off, grad_pos ? blk + lay.h_off : nullptr, ws + lay.agg, blk + lay.a_off,
                                       ws + lay.x[cur ^ 1], status, stream);
        if (rc) return rc;
        cur ^= 1;
    }
    // output network: tanh(x W^T + b) . w_out (+ b_out), summed per structure
    rc = mlcgb_gemm_tc_fused(0, ws + lay.x[cur], w->head_W, w->head_b, nullptr, 1, N, Wh, H, ws + lay.ah, status, stream);
    if (rc) return rc;
    {
        TimelineScope timeline_scope("head_out", stream);
        launch_pdl(head_out_kernel, dim3(grid_for(N * 32, 256)), dim3(256), 0, st, (const float *)(ws + lay.ah), (const float *)w->head_out, (const float *)w->head_out_b, N, Wh, ws + lay.en);
    }
    rc = mlcgb_segment_sum(ws + lay.en, MLCGB_F32, struct_ptr, B, energy, stream);
    if (rc || !grad_pos) return rc ? rc : check_launch();

    // force pass: d(sum of energies)/d(pos)
    // through the output network: g = (w_out * (1 - a^2)) head_W, the factor applied as the GEMM reads its input tile
    int gcur = 0;
    rc = mlcgb_gemm_tc_fused(1, ws + lay.ah, w->head_W, nullptr, w->head_out, 4, N, H, Wh, ws + lay.g[gcur], status, stream);
    if (rc) return rc;
    for (int64_t l = L - 1; l >= 0; l--) {
        const mlcgb_schnet_block &bw = w->blocks[l];
        float *blk = ws + lay.block0 + l * lay.block_stride;
        // every block's filter kernel writes the same rows of gd (one edge per pair): the last block sets them, the others add
        rc = interaction_backward_counted(ws + lay.g[gcur], blk + lay.a_off, blk + lay.wp_off, blk + lay.xl_off, blk + lay.h_off, d, offsets, row1, sel, pair_of, twin,
                                        pairs_dev, row0, row1, rbf, conv_cutoff_kind, conv_lower, conv_upper, bw.lin1_w, bw.filter_w1, bw.filter_b1,
                                        bw.filter_w2, bw.lin2_w, bw.lin_w, N, E, P, H, F, H2, precision, ws + lay.gy, ws + lay.agg, ws + lay.gxl,
                                        l > 0 ? ws + lay.g[gcur ^ 1] : nullptr, E > 0 ? ws + lay.gd : nullptr, l != L - 1, status, stream);
        if (rc) return rc;
        gcur ^= 1;
    }
    // symmetric centre-sorted list: grouped by row0 in place, grouped by row1 through the reverse-edge map
    return mlcgb_edge_distance_backward(pos, ws + lay.gd, d, MLCGB_F32, row0, row1, offsets, twin, offsets, nullptr, N, E, grad_pos, stream);
}

}  // extern "C"
