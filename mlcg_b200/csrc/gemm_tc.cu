// Edge-sized GEMMs of the filter network on the sm_100a tensor cores, fp32-equivalent.
//
// The composable (training) path needs plain GEMMs whose tall dimension is the edge count and whose
// other two dimensions are the widths of the filter network (128 and at most 128):
//   NT  C[E,N] = A[E,K] B[N,K]^T (+ bias)     forward of a Linear layer
//   NN  C[E,N] = A[E,K] B[K,N]                gradient w.r.t. the layer input
//   TN  C[M,N] = A[E,M]^T B[E,N]              gradient w.r.t. the weight (contraction over edges)
// Every fp32 operand is carried as an fp16 pair (hi + lo, ~22 bits) and each product runs as
// hi*hi + hi*lo + lo*hi with fp32 accumulation in tensor memory, like the fused eval-mode kernels.
// Rows of A (NT/NN) are scaled by a power of two so that their largest magnitude sits in [8,16);
// TN scales each 128-edge tile of A and of B by one power of two and accumulates the tiles in registers.
#include "tc_common.cuh"
#include "tensor_map.cuh"

namespace mlcgb {

constexpr int kGT = 512;   // threads: thread = (row of the tile, 32-column quarter)

struct GemmTcSmem {
    static constexpr int kB = 0;                 // operand tile hi | lo (2 x 32 KB)
    static constexpr int kStageA = 65536;        // fp32 stage 64 KB
    static constexpr int kStageB = 131072;       // fp32 stage 64 KB (TN only)
    static constexpr int kMisc = 196608;         // exchange [4][128] f32, bias [128], barrier, TMEM slot, flags
    static constexpr int kTotal = kMisc + 4096 + 1024;
};

__device__ __forceinline__ float4 *gstage(uint8_t *stage, int row, int chunk) {
    return reinterpret_cast<float4 *>(stage + row * 512 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ float *gstage_elem(uint8_t *stage, int row, int col) {
    return reinterpret_cast<float *>(stage + row * 512 + ((((col >> 2) ^ (row & 7)) << 4) | ((col & 3) << 2)));
}

// rows [row0, row0+128) x cols [0, ncols) of a row-major [nrows_total, ncols] fp32 matrix -> stage, zero-filled
// outside; whole rows are read by consecutive lanes
__device__ __forceinline__ void load_tile_to_stage(uint8_t *stage, const float *__restrict__ src, int64_t row0, int64_t nrows_total,
                                                   int ncols) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (ncols & 3) == 0 && ((uintptr_t)src & 15) == 0;
#pragma unroll 1
    for (int i = 0; i < 8; i++) {
        const int row = warp * 8 + i;
        const int64_t gr = row0 + row;
        if (vec) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gr < nrows_total && lane * 4 < ncols) v = __ldcs(reinterpret_cast<const float4 *>(src + gr * ncols) + lane);
            *gstage(stage, row, lane) = v;
        } else {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int col = lane + 32 * c;
                *gstage_elem(stage, row, col) = (gr < nrows_total && col < ncols) ? src[gr * ncols + col] : 0.f;
            }
        }
    }
}

// The same, asynchronously (cp.async, 16 bytes per lane) for rows whose length is a multiple of four floats: used to
// fetch the next tile while the current one is processed.  Out-of-range chunks are zero-filled by the copy itself.
__device__ __forceinline__ void prefetch_tile_to_stage(uint8_t *stage, const float *__restrict__ src, int64_t row0, int64_t nrows_total,
                                                       int ncols) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = warp * 8 + i;
        const int64_t gr = row0 + row;
        const bool ok = gr < nrows_total && lane * 4 < ncols;
        const float *g = ok ? src + gr * ncols + lane * 4 : src;
        const uint32_t dst = tc::smem_u32(gstage(stage, row, lane));
        const int nbytes = ok ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(g), "r"(nbytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// rows [row0, row0+128) of a row-major [nrows_total, ncols] fp32 matrix (ncols a multiple of four) -> 32-column boxes in
// the 128-byte swizzle, asynchronously; whole rows are read by consecutive lanes
__device__ __forceinline__ void prefetch_tile_to_boxes(uint8_t *stage, const float *__restrict__ src, int64_t row0, int64_t nrows_total,
                                                       int ncols) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = warp * 8 + i;
        const int64_t gr = row0 + row;
        const bool ok = gr < nrows_total && lane * 4 < ncols;
        const float *g = ok ? src + gr * ncols + lane * 4 : src;
        const uint32_t dst = tc::smem_u32(box_chunk(stage, lane >> 3, row, lane & 7));
        const int nbytes = ok ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(g), "r"(nbytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void wait_prefetch() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ NT / NN
template <int MODE>   // 0 NT, 1 NN
__global__ void __launch_bounds__(kGT, 1)
gemm_tc_rows_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias, int64_t E, int N, int K,
                    float *__restrict__ C, int32_t *__restrict__ status) {
    using namespace tc;
    using L = GemmTcSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sB_hi = smem + L::kB, *sB_lo = sB_hi + 32768;
    uint8_t *stages[2] = {smem + L::kStageA, smem + L::kStageB};   // input tiles, double-buffered; outputs reuse the current one
    float *s_red = reinterpret_cast<float *>(smem + L::kMisc);
    float *s_bias = s_red + 512;
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_bias + 128);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = tid & 127, qt = tid >> 7, col0 = qt * 32;
    constexpr float kWS = 64.f;
    // operand tile of the weight: NT: rows = n, K-major;  NN: rows = k, read as an MN-major operand
    const int wrows = MODE == 0 ? N : K, wcols = MODE == 0 ? K : N;
    const int wpad = wcols <= 64 ? 64 : 128;
    if (load_weight_tile<true>(sB_hi, sB_lo, B, wrows, wcols, wpad, kWS) && blockIdx.x == 0) atomicOr(status, (int)kWeightRange);
    if (tid < 128) s_bias[tid] = (bias && tid < N) ? bias[tid] : 0.f;
    const uint32_t bar = smem_u32(s_bar);
    if (tid == 0) {
        mbar_init(bar, 1);
        *s_err = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), 256);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const int ksteps = MODE == 0 ? wpad / 16 : (K + 15) / 16;
    const int nmma = MODE == 0 ? 128 : wpad;
    uint32_t phase = 0;

    const int64_t ntiles = (E + kRows - 1) / kRows;
    const bool async_in = (K & 3) == 0 && ((uintptr_t)A & 15) == 0;
    int sidx = 0;
    if (async_in && blockIdx.x < ntiles) prefetch_tile_to_stage(stages[0], A, (int64_t)blockIdx.x * kRows, E, K);
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, sidx ^= 1) {
        uint8_t *stage = stages[sidx];
        if (async_in) {
            wait_prefetch();
            __syncthreads();          // this tile has landed; the other stage was fully consumed one iteration ago
            const int64_t next = tile + gridDim.x;
            if (next < ntiles) prefetch_tile_to_stage(stages[sidx ^ 1], A, next * kRows, E, K);
        } else {
            load_tile_to_stage(stage, A, tile * kRows, E, K);
            __syncthreads();
        }
        float x[32];
        float rmax = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const float4 v = *gstage(stage, r, (col0 >> 2) + w);
            x[4 * w] = v.x; x[4 * w + 1] = v.y; x[4 * w + 2] = v.z; x[4 * w + 3] = v.w;
            rmax = fmaxf(fmaxf(rmax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        s_red[qt * 128 + r] = rmax;
        __syncthreads();
        const float sc = row_scale(fmaxf(fmaxf(s_red[r], s_red[128 + r]), fmaxf(s_red[256 + r], s_red[384 + r])));
        if (col0 < ksteps * 16) store_a_tmem<true>(tmem + 128 + lane_off, col0, x, sc);
        tmem_wait_st();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            issue_gemm_ts<true>(tmem, tmem + 128, smem_u32(sB_hi), smem_u32(sB_lo), ksteps, MODE, nmma);
            mma_commit(bar);
        }
        if (!mbar_wait(bar, phase)) *s_err = 1;
        phase ^= 1;
        tc_fence_after();
        if (col0 < nmma) {
            float v[32];
            tmem_ld32(tmem + lane_off + col0, v);
            const float inv = 1.f / (sc * kWS);
#pragma unroll
            for (int w = 0; w < 8; w++)
                *gstage(stage, r, (col0 >> 2) + w) = make_float4(fmaf(v[4 * w], inv, s_bias[col0 + 4 * w]), fmaf(v[4 * w + 1], inv, s_bias[col0 + 4 * w + 1]),
                                                                 fmaf(v[4 * w + 2], inv, s_bias[col0 + 4 * w + 2]), fmaf(v[4 * w + 3], inv, s_bias[col0 + 4 * w + 3]));
        }
        tc_fence_before();
        __syncthreads();
        if (*s_err) break;
        const bool vec = (N & 3) == 0 && ((uintptr_t)C & 15) == 0;
#pragma unroll 1
        for (int i = 0; i < 8; i++) {
            const int row = warp * 8 + i;
            const int64_t gr = tile * kRows + row;
            if (gr >= E) continue;
            if (vec) {
                if (lane * 4 < N) __stcs(reinterpret_cast<float4 *>(C + gr * N) + lane, *gstage(stage, row, lane));
            } else {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int col = lane + 32 * c;
                    if (col < N) C[gr * N + col] = *gstage_elem(stage, row, col);
                }
            }
        }
        __syncthreads();
    }
    tc_fence_before();
    __syncthreads();
    if (*s_err && tid == 0) atomicOr(status, 8);
    if (warp == 0) tmem_free(tmem, 256);
}

// ------------------------------------------------------------------------------------------------ NT / NN, pipelined
// Fast path of the two row-wise modes (K and N multiples of four, 16-byte aligned A and C, at least one full tile):
//  * input tiles arrive in one shared-memory stage by cp.async (whole rows per warp); the copy of tile i+2 is issued
//    as soon as tile i+1 has been read out of the stage;
//  * two operand blocks and two accumulators in tensor memory: the conversion of tile i+1 (row scale, fp16 hi/lo, store
//    to TMEM) and its MMAs are issued before the epilogue of tile i, so the tensor core works under both;
//  * the output tile goes to a second stage (32-column boxes, 128-byte swizzle) and leaves through tensor stores that
//    drain while the next tile is processed.
// Epilogues (EPI): 0 none; 1 tanh; 2 + aux; 3 * (1 - aux^2), the derivative of tanh given its output.  `aux` is a matrix
// shaped like C; its tile is copied into the output stage while the next tile is converted and combined there.
// EPI 4 is a transform of the input instead: A[m,k] <- aux[k] * (1 - A[m,k]^2) with a vector aux[K], applied as the tile is read
// (the derivative of a tanh layer followed by a dot product with aux, fed straight into the next GEMM).
enum { kEpiNone = 0, kEpiTanh = 1, kEpiAdd = 2, kEpiTanhGrad = 3, kProTanhGradVec = 4 };
template <int MODE>   // 0 NT, 1 NN
__global__ void __launch_bounds__(kGT, 1)
gemm_tc_rows_pipe_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias, int64_t E, int N, int K,
                         const float *__restrict__ aux, int epi, const __grid_constant__ CUtensorMap cmap, int32_t *__restrict__ status) {
    using namespace tc;
    using L = GemmTcSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sB_hi = smem + L::kB, *sB_lo = sB_hi + 32768;
    uint8_t *s_in = smem + L::kStageA, *s_out = smem + L::kStageB;
    float *s_red = reinterpret_cast<float *>(smem + L::kMisc);
    float *s_bias = s_red + 512;
    float *s_vec = s_bias + 128;                                     // input-transform vector (EPI 4)
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_vec + 128);     // two barriers, one per accumulator
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 2);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int r = tid & 127, qt = tid >> 7, col0 = qt * 32;
    constexpr float kWS = 64.f;
    const int64_t ntiles = (E + kRows - 1) / kRows;
    const int64_t step = gridDim.x, t0 = blockIdx.x;
    const int wrows = MODE == 0 ? N : K, wcols = MODE == 0 ? K : N;
    const int wpad = wcols <= 64 ? 64 : 128;
    if (load_weight_tile<true>(sB_hi, sB_lo, B, wrows, wcols, wpad, kWS) && blockIdx.x == 0) atomicOr(status, (int)kWeightRange);
    if (tid < 128) {
        s_bias[tid] = (bias && tid < N) ? bias[tid] : 0.f;
        s_vec[tid] = (epi == kProTanhGradVec && tid < K) ? aux[tid] : 0.f;      // (a parameter vector, not a result of the kernels before)
    }
    const uint32_t bar0 = smem_u32(s_bar);
    if (tid == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        *s_err = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), 512);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();                                    // set-up done (weights only); A, aux and C belong to the kernels before
    pdl_launch_dependents();
    if (t0 < ntiles) prefetch_tile_to_stage(s_in, A, t0 * kRows, E, K);
    const uint32_t tmem = *s_tmem;                 // accumulators at columns [0,128) [128,256), operands at [256,384) [384,512)
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const int ksteps = MODE == 0 ? wpad / 16 : (K + 15) / 16;
    const int nmma = MODE == 0 ? 128 : wpad;
    const uint32_t b_hi = smem_u32(sB_hi), b_lo = smem_u32(sB_lo);
    uint32_t phase_bits = 0;          // bit b: parity the next wait on barrier b looks for

    // the tile that has landed in the input stage: row scale, operand store, MMAs into accumulator `buf`; then the copy of
    // tile `following` (if any) into the stage.  Returns the row's scale.
    auto convert_issue = [&](int buf, int64_t following) {
        wait_prefetch();
        __syncthreads();
        float x[32];
        float rmax = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            float4 v = *gstage(s_in, r, (col0 >> 2) + w);
            if (epi == kProTanhGradVec) {
                const float4 u = *reinterpret_cast<const float4 *>(s_vec + col0 + 4 * w);
                v = make_float4(u.x * fmaf(-v.x, v.x, 1.f), u.y * fmaf(-v.y, v.y, 1.f), u.z * fmaf(-v.z, v.z, 1.f), u.w * fmaf(-v.w, v.w, 1.f));
            }
            x[4 * w] = v.x; x[4 * w + 1] = v.y; x[4 * w + 2] = v.z; x[4 * w + 3] = v.w;
            rmax = fmaxf(fmaxf(rmax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        s_red[qt * 128 + r] = rmax;
        __syncthreads();                            // also: everybody has read the stage
        if (following < ntiles) prefetch_tile_to_stage(s_in, A, following * kRows, E, K);
        const float sc = row_scale(fmaxf(fmaxf(s_red[r], s_red[128 + r]), fmaxf(s_red[256 + r], s_red[384 + r])));
        const uint32_t ta = tmem + 256 + buf * 128;
        if (col0 < ksteps * 16) store_a_tmem<true>(ta + lane_off, col0, x, sc);
        tmem_wait_st();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            issue_gemm_ts<true>(tmem + buf * 128, ta, b_hi, b_lo, ksteps, MODE, nmma);
            mma_commit(bar0 + 8 * buf);
        }
        return sc;
    };

    float sc_cur = 1.f;
    if (t0 < ntiles) sc_cur = convert_issue(0, t0 + step);
    int buf = 0;
    const int nboxes = (N + 31) >> 5;
    for (int64_t tile = t0; tile < ntiles; tile += step, buf ^= 1) {
        float sc_next = 1.f;
        const bool with_aux = epi == kEpiAdd || epi == kEpiTanhGrad;
        if (with_aux) {                             // the aux tile travels to the output stage under the conversion below
            if (tid == 0) bulk_wait_read<0>();      // the stores of the previous tile have read the output stage
            __syncthreads();
            prefetch_tile_to_boxes(s_out, aux, tile * kRows, E, N);
        }
        if (tile + step < ntiles) sc_next = convert_issue(buf ^ 1, tile + 2 * step);
        if (!mbar_wait(bar0 + 8 * buf, (phase_bits >> buf) & 1u)) *s_err = 1;
        phase_bits ^= 1u << buf;
        tc_fence_after();
        if (with_aux) wait_prefetch();              // (also waits for the input tile just requested)
        else if (tid == 0) bulk_wait_read<0>();
        __syncthreads();
        if (col0 < nmma) {
            float v[32];
            tmem_ld32(tmem + buf * 128 + lane_off + col0, v);
            const float inv = 1.f / (sc_cur * kWS);
#pragma unroll
            for (int w = 0; w < 8; w++) {
                float4 o = make_float4(fmaf(v[4 * w], inv, s_bias[col0 + 4 * w]), fmaf(v[4 * w + 1], inv, s_bias[col0 + 4 * w + 1]),
                                       fmaf(v[4 * w + 2], inv, s_bias[col0 + 4 * w + 2]), fmaf(v[4 * w + 3], inv, s_bias[col0 + 4 * w + 3]));
                float4 *slot = box_chunk(s_out, qt, r, w);
                if (epi == kEpiTanh) {
                    o = make_float4(tanh_ex2(o.x), tanh_ex2(o.y), tanh_ex2(o.z), tanh_ex2(o.w));
                } else if (epi == kEpiAdd) {
                    const float4 a4 = *slot;
                    o = make_float4(o.x + a4.x, o.y + a4.y, o.z + a4.z, o.w + a4.w);
                } else if (epi == kEpiTanhGrad) {
                    const float4 a4 = *slot;
                    o = make_float4(o.x * fmaf(-a4.x, a4.x, 1.f), o.y * fmaf(-a4.y, a4.y, 1.f), o.z * fmaf(-a4.z, a4.z, 1.f), o.w * fmaf(-a4.w, a4.w, 1.f));
                }
                *slot = o;
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (*s_err) break;
        if (tid == 0) {
            for (int b = 0; b < nboxes; b++) tensor_store_box(&cmap, 32 * b, (int)(tile * kRows), s_out + b * 16384);
            bulk_commit();
        }
        sc_cur = sc_next;
    }
    wait_prefetch();
    bulk_wait_all();
    tc_fence_before();
    __syncthreads();
    if (*s_err && tid == 0) atomicOr(status, 8);
    if (warp == 0) tmem_free(tmem, 512);
}

// ------------------------------------------------------------------------------------------------ two Linear layers chained
// The two node-sized layers that follow the aggregation of an interaction block, and their counterparts in the force pass,
// as one kernel: the 128-row tile stays on the chip between the two GEMMs.
//   FWD (NT, NT):  mid = tanh(A Wa^T + ba)  (stored: the force pass reads it)      C = aux + mid Wb^T + bb
//   BWD (NN, NN):  mid = (A Wa) * (1 - aux^2)                                       C = mid Wb
// All widths are 128.  Shared memory: both weight tiles as fp16 hi/lo pairs (2 x 64 KB) and one 64 KB stage through which
// every tile enters and leaves in whole rows.  One accumulator and one operand block of tensor memory, used by both GEMMs of
// a tile one after the other.
struct ChainSmem {
    static constexpr int kWa = 0, kWb = 65536, kStage = 131072, kMisc = 196608;
    static constexpr int kTotal = kMisc + 4096 + 1024;
};

template <int BWD>
__global__ void __launch_bounds__(kGT, 1)
gemm_tc_chain2_kernel(const float *__restrict__ A, const float *__restrict__ Wa, const float *__restrict__ ba, const float *__restrict__ Wb,
                      const float *__restrict__ bb, const float *__restrict__ aux, int64_t E, float *__restrict__ mid_out,
                      float *__restrict__ C, int32_t *__restrict__ status) {
    using namespace tc;
    using L = ChainSmem;
    constexpr int W = 128, MODE = BWD ? 1 : 0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sWa_hi = smem + L::kWa, *sWa_lo = sWa_hi + 32768, *sWb_hi = smem + L::kWb, *sWb_lo = sWb_hi + 32768;
    uint8_t *stage = smem + L::kStage;
    float *s_red = reinterpret_cast<float *>(smem + L::kMisc);
    float *s_ba = s_red + 512, *s_bb = s_ba + 128;
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_bb + 128);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = tid & 127, qt = tid >> 7, col0 = qt * 32;
    constexpr float kWS = 64.f;
    bool range = load_weight_tile<true>(sWa_hi, sWa_lo, Wa, W, W, W, kWS);
    range = load_weight_tile<true>(sWb_hi, sWb_lo, Wb, W, W, W, kWS) || range;
    if (range && blockIdx.x == 0) atomicOr(status, (int)kWeightRange);
    if (tid < 128) {
        s_ba[tid] = ba ? ba[tid] : 0.f;
        s_bb[tid] = bb ? bb[tid] : 0.f;
    }
    const uint32_t bar = smem_u32(s_bar);
    if (tid == 0) {
        mbar_init(bar, 1);
        *s_err = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), 256);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();                                    // set-up done (weights only); A and aux belong to the kernels before
    pdl_launch_dependents();
    const uint32_t tmem = *s_tmem;                 // accumulator at columns [0,128), operand at [128,256)
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ta = tmem + 128;
    const int64_t ntiles = (E + kRows - 1) / kRows;
    uint32_t phase = 0;
    bool failed = false;
    if (blockIdx.x < ntiles) prefetch_tile_to_stage(stage, A, (int64_t)blockIdx.x * kRows, E, W);

    // this thread's 32 values -> operand block (row-scaled fp16 pairs); returns the row's scale.  `fetch`: a tile to copy into
    // the stage as soon as everybody has read the current contents out of it (rows of `fetch` starting at `fetch_row0`)
    auto to_operand = [&](const float (&x)[32], const float *fetch, int64_t fetch_row0) {
        float rmax = 0.f;
#pragma unroll
        for (int c = 0; c < 32; c++) rmax = fmaxf(rmax, fabsf(x[c]));
        s_red[qt * 128 + r] = rmax;
        __syncthreads();
        if (fetch) prefetch_tile_to_stage(stage, fetch, fetch_row0, E, W);
        const float sc = row_scale(fmaxf(fmaxf(s_red[r], s_red[128 + r]), fmaxf(s_red[256 + r], s_red[384 + r])));
        store_a_tmem<true>(ta + lane_off, col0, x, sc);
        tmem_wait_st();
        tc_fence_before();
        __syncthreads();
        return sc;
    };
    auto gemm = [&](uint8_t *w_hi, uint8_t *w_lo) {
        if (tid == 0) {
            tc_fence_after();
            issue_gemm_ts<true>(tmem, ta, smem_u32(w_hi), smem_u32(w_lo), W / 16, MODE, W);
            mma_commit(bar);
        }
    };
    auto await = [&]() {
        if (!failed && !mbar_wait(bar, phase)) failed = true;
        phase ^= 1;
        tc_fence_after();
    };
    // rows of the stage -> global memory, whole rows by consecutive lanes, eight rows per warp in flight
    auto store_stage = [&](float *dst, int64_t tile) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = *gstage(stage, warp * 8 + i, lane);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int64_t gr = tile * kRows + warp * 8 + i;
            if (gr < E) __stcs(reinterpret_cast<float4 *>(dst + gr * W) + lane, v[i]);
        }
    };

    // Everything that crosses to or from global memory goes through the stage in whole rows (a thread's own 32 columns of a
    // row are 128 bytes: 32 separate lines per warp instruction if moved directly).  The stage holds, in turn: the input tile;
    // BWD: the tile of tanh outputs; FWD: mid on its way out, then the residual tile; the output tile on its way out.
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        wait_prefetch();
        __syncthreads();                            // the input tile has landed
        float x[32];
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const float4 v = *gstage(stage, r, (col0 >> 2) + w);
            x[4 * w] = v.x; x[4 * w + 1] = v.y; x[4 * w + 2] = v.z; x[4 * w + 3] = v.w;
        }
        const float sc1 = to_operand(x, BWD ? aux : nullptr, tile * kRows);      // BWD: the tanh outputs arrive under the first GEMM
        gemm(sWa_hi, sWa_lo);
        await();
        if (BWD) {
            wait_prefetch();
            __syncthreads();
        }
        {
            float v[32];
            tmem_ld32(tmem + lane_off + col0, v);
            const float inv = 1.f / (sc1 * kWS);
#pragma unroll
            for (int w = 0; w < 8; w++) {
                float4 o = make_float4(fmaf(v[4 * w], inv, s_ba[col0 + 4 * w]), fmaf(v[4 * w + 1], inv, s_ba[col0 + 4 * w + 1]),
                                       fmaf(v[4 * w + 2], inv, s_ba[col0 + 4 * w + 2]), fmaf(v[4 * w + 3], inv, s_ba[col0 + 4 * w + 3]));
                float4 *slot = gstage(stage, r, (col0 >> 2) + w);
                if (BWD) {
                    const float4 t4 = *slot;
                    o = make_float4(o.x * fmaf(-t4.x, t4.x, 1.f), o.y * fmaf(-t4.y, t4.y, 1.f), o.z * fmaf(-t4.z, t4.z, 1.f), o.w * fmaf(-t4.w, t4.w, 1.f));
                } else {
                    o = make_float4(tanh_ex2(o.x), tanh_ex2(o.y), tanh_ex2(o.z), tanh_ex2(o.w));
                    *slot = o;                       // on its way to mid_out
                }
                x[4 * w] = o.x; x[4 * w + 1] = o.y; x[4 * w + 2] = o.z; x[4 * w + 3] = o.w;
            }
        }
        const float sc2 = to_operand(x, nullptr, 0);     // (the accumulator has been read, the first GEMM's operand consumed)
        gemm(sWb_hi, sWb_lo);
        if (!BWD) {                                  // under the second GEMM: mid leaves, the residual tile arrives
            store_stage(mid_out, tile);
            __syncthreads();
            prefetch_tile_to_stage(stage, aux, tile * kRows, E, W);
        }
        await();
        if (!BWD) {
            wait_prefetch();
            __syncthreads();
        }
        {
            float v[32];
            tmem_ld32(tmem + lane_off + col0, v);
            const float inv = 1.f / (sc2 * kWS);
#pragma unroll
            for (int w = 0; w < 8; w++) {
                float4 o = make_float4(fmaf(v[4 * w], inv, s_bb[col0 + 4 * w]), fmaf(v[4 * w + 1], inv, s_bb[col0 + 4 * w + 1]),
                                       fmaf(v[4 * w + 2], inv, s_bb[col0 + 4 * w + 2]), fmaf(v[4 * w + 3], inv, s_bb[col0 + 4 * w + 3]));
                float4 *slot = gstage(stage, r, (col0 >> 2) + w);
                if (!BWD) {
                    const float4 t4 = *slot;
                    o = make_float4(o.x + t4.x, o.y + t4.y, o.z + t4.z, o.w + t4.w);
                }
                *slot = o;
            }
        }
        tc_fence_before();
        __syncthreads();
        store_stage(C, tile);
        __syncthreads();                            // the stage is free for the next input tile
        const int64_t next = tile + gridDim.x;
        if (next < ntiles) prefetch_tile_to_stage(stage, A, next * kRows, E, W);
    }
    wait_prefetch();
    if (failed) *s_err = 1;
    tc_fence_before();
    __syncthreads();
    if (*s_err && tid == 0) atomicOr(status, 8);
    if (warp == 0) tmem_free(tmem, 256);
}

// ------------------------------------------------------------------------------------------------ TN
__device__ __forceinline__ float block_max_512(float v, float *s_red) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = s_red[0];
#pragma unroll
    for (int i = 1; i < 16; i++) m = fmaxf(m, s_red[i]);
    __syncthreads();
    return m;
}

__global__ void __launch_bounds__(kGT, 1)
gemm_tc_tn_kernel(const float *__restrict__ A, const float *__restrict__ B, int64_t E, int M, int N, float *__restrict__ partial,
                  int32_t *__restrict__ status) {
    using namespace tc;
    using L = GemmTcSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sB_hi = smem + L::kB, *sB_lo = sB_hi + 32768, *stageA = smem + L::kStageA, *stageB = smem + L::kStageB;
    float *s_red = reinterpret_cast<float *>(smem + L::kMisc);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_red + 640);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int r = tid & 127, qt = tid >> 7, col0 = qt * 32;   // r: output row m (TMEM lane); col0: edge sub-range / output column range
    const int npad = N <= 64 ? 64 : 128;
    const uint32_t bar = smem_u32(s_bar);
    if (tid == 0) {
        mbar_init(bar, 1);
        *s_err = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), 256);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t phase = 0;
    float acc[32];
#pragma unroll
    for (int j = 0; j < 32; j++) acc[j] = 0.f;

    const int64_t ntiles = (E + kRows - 1) / kRows;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        load_tile_to_stage(stageA, A, tile * kRows, E, M);
        load_tile_to_stage(stageB, B, tile * kRows, E, N);
        __syncthreads();
        // A operand: lane = output row m, K = edge: x[j] = A[edge col0 + j][m]
        float x[32];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            x[j] = *gstage_elem(stageA, col0 + j, r);
            amax = fmaxf(amax, fabsf(x[j]));
        }
        float bmax = 0.f;
        for (int idx = tid; idx < kRows * 32; idx += kGT) {
            const float4 v = *reinterpret_cast<const float4 *>(stageB + idx * 16);
            bmax = fmaxf(fmaxf(bmax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        const float sa = row_scale(block_max_512(amax, s_red));
        const float sb = row_scale(block_max_512(bmax, s_red));
        store_a_tmem<true>(tmem + 128 + lane_off, col0, x, sa);
        // B operand tile [edge rows][n cols], read MN-major
        for (int idx = tid; idx < kRows * npad; idx += kGT) {
            const int er = idx / npad, n = idx - er * npad;
            const float w = *gstage_elem(stageB, er, n) * sb;
            const uint32_t off = elem_offset(er, n);
            const __half a = __float2half_rn(w);
            *reinterpret_cast<__half *>(sB_hi + off) = a;
            *reinterpret_cast<__half *>(sB_lo + off) = __float2half_rn(w - __half2float(a));
        }
        tmem_wait_st();
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            issue_gemm_ts<true>(tmem, tmem + 128, smem_u32(sB_hi), smem_u32(sB_lo), kRows / 16, 1, npad);
            mma_commit(bar);
        }
        if (!mbar_wait(bar, phase)) *s_err = 1;
        phase ^= 1;
        tc_fence_after();
        if (col0 < npad) {
            float v[32];
            tmem_ld32(tmem + lane_off + col0, v);
            const float inv = 1.f / (sa * sb);
#pragma unroll
            for (int j = 0; j < 32; j++) acc[j] = fmaf(v[j], inv, acc[j]);
        }
        tc_fence_before();
        __syncthreads();
        if (*s_err) break;
    }
    // this CTA's partial [M][N]
    if (r < M)
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (col0 + j < N) partial[((int64_t)blockIdx.x * M + r) * N + col0 + j] = acc[j];
    tc_fence_before();
    __syncthreads();
    if (*s_err && tid == 0) atomicOr(status, 8);
    if (warp == 0) tmem_free(tmem, 256);
}

// ------------------------------------------------------------------------------------------------ TN, pipelined
// C[M,N] = A[E,M]^T B[E,N], the contraction runs over the edges.  Per 128-edge tile:
//  * A operand (lane = output row m, K = edge): every thread reads its 32 values A[e][m] straight from global memory —
//    for one edge the 128 threads of a lane quarter read 128 consecutive floats;
//  * B operand (rows = edges, read MN-major): float4 per thread from global memory, converted to fp16 hi/lo and written
//    as 8-byte pieces of the swizzled operand tile;
//  * both are scaled by one power of two per tile (largest magnitude to [8,16)), so every tile has its own scale and
//    its product is read out of tensor memory and added to an fp32 accumulator tile in shared memory;
//  * two operand buffers (TMEM for A, shared memory for B) and two accumulators: the loads and conversion of tile i+1
//    run under the MMAs of tile i.
// Needs N % 4 == 0 and a 16-byte aligned B; the one-tile-at-a-time kernel below takes everything else.
struct GemmTnSmem {
    static constexpr int kB0 = 0, kB1 = 65536;        // operand tiles hi | lo, two buffers
    static constexpr int kAcc = 131072;               // fp32 accumulators [128][128], chunk-swizzled
    static constexpr int kMisc = 196608;
    static constexpr int kTotal = kMisc + 1024 + 1024;
};

__global__ void __launch_bounds__(kGT, 1)
gemm_tc_tn_pipe_kernel(const float *__restrict__ A, const float *__restrict__ B, int64_t E, int M, int N, float *__restrict__ partial,
                       float *__restrict__ colsum_partial /* [gridDim.x][M] or NULL: column sums of A */, int32_t *__restrict__ status) {
    using namespace tc;
    using L = GemmTnSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *s_acc = smem + L::kAcc;
    float2 *s_red = reinterpret_cast<float2 *>(smem + L::kMisc);          // [16] per-warp maxima of (A, B)
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + L::kMisc + 256);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 2);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = tid & 127, qt = tid >> 7, col0 = qt * 32;   // r: output row m (TMEM lane); col0: edge sub-range / output columns
    const int npad = N <= 64 ? 64 : 128;
    const int qpr = npad >> 2;                                  // float4 pieces per row of the B tile
    const uint32_t bar0 = smem_u32(s_bar);
    if (tid == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        *s_err = 0;
    }
#pragma unroll
    for (int w = 0; w < 8; w++) *gstage(s_acc, r, (col0 >> 2) + w) = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), 512);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;                 // accumulators [0,128) [128,256); A operands [256,384) [384,512)
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t phase_bits = 0;

    const int64_t ntiles = (E + kRows - 1) / kRows;
    const int64_t step = gridDim.x;
    float xa[32];
    float4 xb[8];
    float csum = 0.f;                               // this thread's share of sum_e A[e][r]
    auto load_tile = [&](int64_t tile) {
        const int64_t e0 = tile * kRows;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int64_t e = e0 + col0 + j;
            xa[j] = (e < E && r < M) ? __ldg(A + e * M + r) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = tid + u * kGT;
            const int er = idx / qpr, n4 = (idx - er * qpr) << 2;
            const int64_t e = e0 + er;
            xb[u] = (er < kRows && e < E && n4 < N) ? __ldg(reinterpret_cast<const float4 *>(B + e * N + n4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    // scales, operand stores and MMAs of the tile held in xa / xb into buffer `buf`; returns 1 / (sa sb)
    auto convert_issue = [&](int buf) {
        float amax = 0.f, bmax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            amax = fmaxf(amax, fabsf(xa[j]));
            csum += xa[j];
        }
#pragma unroll
        for (int u = 0; u < 8; u++) bmax = fmaxf(fmaxf(bmax, fmaxf(fabsf(xb[u].x), fabsf(xb[u].y))), fmaxf(fabsf(xb[u].z), fabsf(xb[u].w)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
        }
        if (lane == 0) s_red[warp] = make_float2(amax, bmax);
        __syncthreads();
        if (*s_err) return -1.f;      // written before this barrier, so every thread takes the same branch
#pragma unroll
        for (int w = 0; w < 16; w++) {
            const float2 m = s_red[w];
            amax = fmaxf(amax, m.x);
            bmax = fmaxf(bmax, m.y);
        }
        const float sa = row_scale(amax), sb = row_scale(bmax);
        const uint32_t ta = tmem + 256 + buf * 128;
        store_a_tmem<true>(ta + lane_off, col0, xa, sa);
        uint8_t *b_hi = smem + (buf ? L::kB1 : L::kB0), *b_lo = b_hi + 32768;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = tid + u * kGT;
            const int er = idx / qpr, n4 = (idx - er * qpr) << 2;
            if (er < kRows) {
                const float4 w = make_float4(xb[u].x * sb, xb[u].y * sb, xb[u].z * sb, xb[u].w * sb);
                const uint32_t off = elem_offset(er, n4);
                const __half2 a0 = __floats2half2_rn(w.x, w.y), a1 = __floats2half2_rn(w.z, w.w);
                const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
                const __half2 c0 = __floats2half2_rn(w.x - f0.x, w.y - f0.y), c1 = __floats2half2_rn(w.z - f1.x, w.w - f1.y);
                *reinterpret_cast<uint2 *>(b_hi + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1));
                *reinterpret_cast<uint2 *>(b_lo + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&c0), *reinterpret_cast<const uint32_t *>(&c1));
            }
        }
        tmem_wait_st();
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            issue_gemm_ts<true>(tmem + buf * 128, ta, smem_u32(b_hi), smem_u32(b_lo), kRows / 16, 1, npad);
            mma_commit(bar0 + 8 * buf);
        }
        return 1.f / (sa * sb);
    };
    // product of the tile in accumulator `buf` -> shared-memory accumulator
    auto collect = [&](int buf, float inv) {
        if (!mbar_wait(bar0 + 8 * buf, (phase_bits >> buf) & 1u)) *s_err = 1;
        phase_bits ^= 1u << buf;
        tc_fence_after();
        if (col0 < npad) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float v[16];
                tmem_ld16(tmem + buf * 128 + lane_off + col0 + half * 16, v);
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    float4 *slot = gstage(s_acc, r, (col0 >> 2) + half * 4 + w);
                    float4 a4 = *slot;
                    a4.x = fmaf(v[4 * w], inv, a4.x); a4.y = fmaf(v[4 * w + 1], inv, a4.y);
                    a4.z = fmaf(v[4 * w + 2], inv, a4.z); a4.w = fmaf(v[4 * w + 3], inv, a4.w);
                    *slot = a4;
                }
            }
        }
        tc_fence_before();
    };

    const int64_t t0 = blockIdx.x;
    float inv_prev = 0.f;
    int buf = 0;
    if (t0 < ntiles) load_tile(t0);
    for (int64_t tile = t0; tile < ntiles; tile += step, buf ^= 1) {
        const float inv_cur = convert_issue(buf);
        if (inv_cur < 0.f) break;                                   // a wait ran out (all threads leave together)
        if (tile + step < ntiles) load_tile(tile + step);           // in flight under the MMAs just issued
        if (tile != t0) collect(buf ^ 1, inv_prev);
        inv_prev = inv_cur;
    }
    __syncthreads();
    if (t0 < ntiles && !*s_err) collect(buf ^ 1, inv_prev);
    __syncthreads();
    if (r < M)
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const float4 a4 = *gstage(s_acc, r, (col0 >> 2) + w);
            const float o[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (col0 + 4 * w + j < N) partial[((int64_t)blockIdx.x * M + r) * N + col0 + 4 * w + j] = o[j];
        }
    if (colsum_partial) {                           // the four edge sub-ranges of each output row, in a fixed order
        float *s_cs = reinterpret_cast<float *>(s_acc);
        __syncthreads();
        s_cs[qt * 128 + r] = csum;
        __syncthreads();
        if (qt == 0 && r < M) colsum_partial[(int64_t)blockIdx.x * M + r] = (s_cs[r] + s_cs[128 + r]) + (s_cs[256 + r] + s_cs[384 + r]);
    }
    tc_fence_before();
    __syncthreads();
    if (*s_err && tid == 0) atomicOr(status, 8);
    if (warp == 0) tmem_free(tmem, 512);
}

// C = the partials added in their order (eight loads in flight at a time; the additions stay in sequence, so the result does
// not depend on how the loop is unrolled)
__global__ void gemm_tc_reduce_kernel(const float *__restrict__ partial, int64_t MN, int parts, float *__restrict__ C) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN; i += (int64_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        int z = 0;
        for (; z + 8 <= parts; z += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = __ldg(partial + (int64_t)(z + u) * MN + i);
#pragma unroll
            for (int u = 0; u < 8; u++) s += v[u];
        }
        for (; z < parts; z++) s += __ldg(partial + (int64_t)z * MN + i);
        C[i] = s;
    }
}

// The same for two sets of partials in one launch (a weight gradient and its bias gradient): element i < MN of the first,
// element i - MN of the second
__global__ void gemm_tc_reduce2_kernel(const float *__restrict__ partial, int64_t MN, const float *__restrict__ partial2, int64_t M2, int parts,
                                       float *__restrict__ C, float *__restrict__ C2) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN + M2; i += (int64_t)gridDim.x * blockDim.x) {
        const bool second = i >= MN;
        const float *src = second ? partial2 + (i - MN) : partial + i;
        const int64_t stride = second ? M2 : MN;
        float s = 0.f;
        int z = 0;
        for (; z + 8 <= parts; z += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = __ldg(src + (int64_t)(z + u) * stride);
#pragma unroll
            for (int u = 0; u < 8; u++) s += v[u];
        }
        for (; z < parts; z++) s += __ldg(src + (int64_t)z * stride);
        if (second) C2[i - MN] = s;
        else C[i] = s;
    }
}

// CTAs of the TN kernels (each writes one [M,N] partial): one per SM for edge-sized contractions; for short ones two tiles
// per CTA (one, two and four measured within a per cent of one another on a node-sized contraction)
static int tn_parts(int64_t K) {
    const int64_t ntiles = (K + tc::kRows - 1) / tc::kRows;
    int64_t parts = (ntiles + 1) / 2;
    if (parts > kNumSM) parts = kNumSM;
    return (int)(parts < 1 ? 1 : parts);
}

template <typename Kern>
static int set_smem(Kern kern, bool *done) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmTcSmem::kTotal) != cudaSuccess) return check_launch();
        done[dev] = true;
    }
    return MLCGB_OK;
}

// Pipelined row-wise kernel; MLCGB_E_LIMIT when its conditions on shape and alignment do not hold.
static int rows_pipe_launch(int mode, const void *A, const void *B, const void *bias, const void *aux, int epi, int64_t M, int64_t N, int64_t K,
                            void *C, int32_t *status, cudaStream_t st) {
    CUtensorMap cmap;
    if ((K & 3) != 0 || ((uintptr_t)A & 15) != 0 || (aux && epi != kProTanhGradVec && ((uintptr_t)aux & 15) != 0) || !make_rows_map(&cmap, (float *)C, M, N))
        return MLCGB_E_LIMIT;
    const int64_t ntiles = (M + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    static bool p0[64] = {false}, p1[64] = {false};
    if (mode == 0) {
        if (int rc = set_smem(gemm_tc_rows_pipe_kernel<0>, p0)) return rc;
        launch_pdl(gemm_tc_rows_pipe_kernel<0>, dim3(grid), dim3(kGT), GemmTcSmem::kTotal, st, (const float *)A, (const float *)B, (const float *)bias, M,
                   (int)N, (int)K, (const float *)aux, epi, cmap, status);
    } else {
        if (int rc = set_smem(gemm_tc_rows_pipe_kernel<1>, p1)) return rc;
        launch_pdl(gemm_tc_rows_pipe_kernel<1>, dim3(grid), dim3(kGT), GemmTcSmem::kTotal, st, (const float *)A, (const float *)B, (const float *)bias, M,
                   (int)N, (int)K, (const float *)aux, epi, cmap, status);
    }
    return check_launch();
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

int mlcgb_gemm_tc_fused(int mode, const void *A, const void *B, const void *bias, const void *aux, int epilogue, int64_t M, int64_t N,
                        int64_t K, void *C, int32_t *status, void *stream) {
    TimelineScope timeline_scope("gemm_tc_fused", stream);
    if ((mode != 0 && mode != 1) || epilogue < 0 || epilogue > 4 || !status) return MLCGB_E_ARG;
    if ((epilogue == kEpiAdd || epilogue == kEpiTanhGrad || epilogue == kProTanhGradVec) && !aux) return MLCGB_E_ARG;
    if (!mlcgb_gemm_tc_supported(mode, M, N, K)) return MLCGB_E_LIMIT;
    if (M == 0) return MLCGB_OK;
    if (!A || !B || !C) return MLCGB_E_ARG;
    return rows_pipe_launch(mode, A, B, bias, aux, epilogue, M, N, K, C, status, (cudaStream_t)stream);
}


int mlcgb_gemm_tc_chain2(int backward, const void *A, const void *Wa, const void *ba, const void *Wb, const void *bb, const void *aux,
                         int64_t M, void *mid_out, void *C, int32_t *status, void *stream) {
    TimelineScope timeline_scope("gemm_tc_chain2", stream);
    if (M < 0 || !status) return MLCGB_E_ARG;
    if (M == 0) return MLCGB_OK;
    if (!A || !Wa || !Wb || !aux || !C || (!backward && !mid_out)) return MLCGB_E_ARG;
    if ((((uintptr_t)A | (uintptr_t)aux | (uintptr_t)C | (uintptr_t)mid_out) & 15) != 0) return MLCGB_E_LIMIT;
    auto st = (cudaStream_t)stream;
    const int64_t ntiles = (M + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    static bool f0[64] = {false}, f1[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    bool *flag = backward ? f1 : f0;
    if (dev >= 0 && dev < 64 && !flag[dev]) {
        const cudaError_t e = backward ? cudaFuncSetAttribute(gemm_tc_chain2_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, ChainSmem::kTotal)
                                       : cudaFuncSetAttribute(gemm_tc_chain2_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, ChainSmem::kTotal);
        if (e != cudaSuccess) return check_launch();
        flag[dev] = true;
    }
    if (backward)
        launch_pdl(gemm_tc_chain2_kernel<1>, dim3(grid), dim3(kGT), ChainSmem::kTotal, st, (const float *)A, (const float *)Wa, (const float *)ba,
                   (const float *)Wb, (const float *)bb, (const float *)aux, M, (float *)mid_out, (float *)C, status);
    else
        launch_pdl(gemm_tc_chain2_kernel<0>, dim3(grid), dim3(kGT), ChainSmem::kTotal, st, (const float *)A, (const float *)Wa, (const float *)ba,
                   (const float *)Wb, (const float *)bb, (const float *)aux, M, (float *)mid_out, (float *)C, status);
    return check_launch();
}

int mlcgb_gemm_tc_tn_colsum(const void *A, const void *B, int64_t K, int64_t M, int64_t N, void *C, void *colsum, void *workspace,
                            size_t workspace_bytes, int32_t *status, void *stream) {
    TimelineScope timeline_scope("gemm_tc_tn_colsum", stream);
    if (!A || !B || !C || !colsum || !status) return MLCGB_E_ARG;
    if (!mlcgb_gemm_tc_supported(2, M, N, K) || (N & 3) != 0 || ((uintptr_t)B & 15) != 0) return MLCGB_E_LIMIT;
    const int parts = tn_parts(K);
    if (!workspace || workspace_bytes < (size_t)parts * M * (N + 1) * sizeof(float)) return MLCGB_E_WORKSPACE;
    auto st = (cudaStream_t)stream;
    static bool done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !done[dev]) {
        if (cudaFuncSetAttribute(gemm_tc_tn_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmTnSmem::kTotal) != cudaSuccess) return check_launch();
        done[dev] = true;
    }
    float *part = (float *)workspace, *cpart = part + (size_t)parts * M * N;
    gemm_tc_tn_pipe_kernel<<<parts, kGT, GemmTnSmem::kTotal, st>>>((const float *)A, (const float *)B, K, (int)M, (int)N, part, cpart, status);
    gemm_tc_reduce2_kernel<<<grid_for(M * N + M, 256), 256, 0, st>>>(part, M * N, cpart, M, parts, (float *)C, (float *)colsum);
    return check_launch();
}

int mlcgb_gemm_tc_supported(int mode, int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (mode == 0 || mode == 1) return N <= 128 && K <= 128;   // M = edges
    if (mode == 2) return M <= 128 && N <= 128;                // K = edges
    return 0;
}

size_t mlcgb_gemm_tc_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K) {
    if (mode != 2 || !mlcgb_gemm_tc_supported(mode, M, N, K)) return 0;
    return (size_t)tn_parts(K) * (size_t)M * (size_t)(N + 1) * sizeof(float);   // partial products, and partial column sums
}

int mlcgb_gemm_tc(int mode, const void *A, const void *B, const void *bias, int64_t M, int64_t N, int64_t K, void *C, void *workspace,
                  size_t workspace_bytes, int32_t *status, void *stream) {
    TimelineScope timeline_scope("gemm_tc", stream);
    if (!A || !B || !C || !status) return MLCGB_E_ARG;
    if (!mlcgb_gemm_tc_supported(mode, M, N, K)) return MLCGB_E_LIMIT;
    auto st = (cudaStream_t)stream;
    static bool c0[64] = {false}, c1[64] = {false}, c2[64] = {false};
    if (mode == 0 || mode == 1) {
        const int64_t ntiles = (M + tc::kRows - 1) / tc::kRows;
        const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
        const int rc = rows_pipe_launch(mode, A, B, bias, nullptr, kEpiNone, M, N, K, C, status, st);
        if (rc != MLCGB_E_LIMIT) return rc;            // else: shapes or alignment the pipelined kernel does not take
        if (mode == 0) {
            if (int rc = set_smem(gemm_tc_rows_kernel<0>, c0)) return rc;
            gemm_tc_rows_kernel<0><<<grid, kGT, GemmTcSmem::kTotal, st>>>((const float *)A, (const float *)B, (const float *)bias, M, (int)N, (int)K, (float *)C, status);
        } else {
            if (int rc = set_smem(gemm_tc_rows_kernel<1>, c1)) return rc;
            gemm_tc_rows_kernel<1><<<grid, kGT, GemmTcSmem::kTotal, st>>>((const float *)A, (const float *)B, nullptr, M, (int)N, (int)K, (float *)C, status);
        }
        return check_launch();
    }
    const int parts = tn_parts(K);
    if (!workspace || workspace_bytes < (size_t)parts * M * N * sizeof(float)) return MLCGB_E_WORKSPACE;
    if ((N & 3) == 0 && ((uintptr_t)B & 15) == 0) {
        static bool c3[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !c3[dev]) {
            if (cudaFuncSetAttribute(gemm_tc_tn_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmTnSmem::kTotal) != cudaSuccess) return check_launch();
            c3[dev] = true;
        }
        gemm_tc_tn_pipe_kernel<<<parts, kGT, GemmTnSmem::kTotal, st>>>((const float *)A, (const float *)B, K, (int)M, (int)N, (float *)workspace, nullptr, status);
    } else {
        if (int rc = set_smem(gemm_tc_tn_kernel, c2)) return rc;
        gemm_tc_tn_kernel<<<parts, kGT, GemmTcSmem::kTotal, st>>>((const float *)A, (const float *)B, K, (int)M, (int)N, (float *)workspace, status);
    }
    gemm_tc_reduce_kernel<<<grid_for(M * N, 256), 256, 0, st>>>((const float *)workspace, M * N, parts, (float *)C);
    return check_launch();
}

}  // extern "C"
