// Fused filter-generating network on the sm_100a tensor cores (tcgen05 + TMEM).
//
//   W[e,:] = ( tanh( phi(d_e) A1^T + b1 ) A2^T ) * C(d_e)            src/mlcg/nn/schnet.py:340-341
//
// One persistent CTA per SM walks 128-edge tiles.  Per tile: the radial basis is evaluated straight
// into the A operand in shared memory (it never exists in HBM), GEMM 1 accumulates in tensor memory,
// its epilogue (bias, tanh) writes the hidden activations back to shared memory as the A operand of
// GEMM 2, and the second epilogue applies the cutoff envelope and stores W.  Weights are converted
// once per CTA and stay resident in shared memory.
//
// Precision modes.  0: every fp32 value is carried as an fp16 pair (value = hi + lo, ~22 bits) and
// each GEMM runs hi*hi + hi*lo + lo*hi with fp32 accumulation — the products an fp32 GEMM forms, at
// half-precision tensor-core rate.  1: operands rounded to bf16, one product, tanh.approx.
#include "rbf_device.cuh"
#include "tc_common.cuh"

namespace mlcgb {

constexpr int kF = 128;                 // filters / hidden width of the filter network
constexpr int kTcThreads = 256;         // thread t: row t % 128, column half t / 128
constexpr float kWScale = 64.f;         // power-of-two operand scalings keep the fp16 "low" parts normal
constexpr float kActScale = 16.f;

struct FilterFwdParams {
    const float *d;      // [E]
    int64_t E;
    RbfDev<float> rbf;   // basis and its envelope
    RbfDev<float> conv;  // only cutoff_kind / lower / upper are used: the CFConv cutoff C(d)
    const float *A1;     // [kF][R]
    const float *b1;     // [kF]
    const float *A2;     // [kF][kF]
    float *W;            // [E][kF]
    int32_t *status;
};

template <bool SPLIT>
struct FilterSmem {
    static constexpr int kTile = SPLIT ? 2 * 32768 : 32768;   // one 128x128 operand tile (hi [+ lo])
    static constexpr int kA = 0, kB1 = kTile, kB2 = 2 * kTile, kMisc = 3 * kTile;
    static constexpr int kTotal = kMisc + 4096 + 1024;        // + misc (bias, barrier, exchange buffers) + alignment slack
};

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool SPLIT>
__global__ void __launch_bounds__(kTcThreads, 1) filter_fwd_tc_kernel(FilterFwdParams p) {
    using namespace tc;
    using L = FilterSmem<SPLIT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sA_hi = smem + L::kA, *sA_lo = sA_hi + 32768;
    uint8_t *sB1_hi = smem + L::kB1, *sB1_lo = sB1_hi + 32768;
    uint8_t *sB2_hi = smem + L::kB2, *sB2_lo = sB2_hi + 32768;
    float *s_b1 = reinterpret_cast<float *>(smem + L::kMisc);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_b1 + kF);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int r = tid & 127, ch = tid >> 7;            // row of the tile, column half
    const int R = p.rbf.R;
    const int Kpad1 = R <= 64 ? 64 : 128;
    const float wscale = SPLIT ? kWScale : 1.f, ascale = SPLIT ? kActScale : 1.f;
    const float unscale = 1.f / (wscale * ascale);

    load_weight_tile<SPLIT>(sB1_hi, sB1_lo, p.A1, kF, R, Kpad1, wscale);
    load_weight_tile<SPLIT>(sB2_hi, sB2_lo, p.A2, kF, kF, kF, wscale);
    if (tid < kF) s_b1[tid] = p.b1[tid];
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
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 TMEM lanes
    uint32_t phase = 0;

    const int64_t ntiles = (p.E + kRows - 1) / kRows;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t e = tile * kRows + r;
        const bool live = e < p.E;
        const float de = live ? p.d[e] : 1.f;

        // ---- A operand of GEMM 1: phi_k(d) for this thread's 64 columns
        if (ch * 64 < Kpad1) {
            const Jet<float, 0> env = envelope_jet<float, 0>(de, p.rbf);
            const Jet<float, 0> ej = edge_jet<float, 0>(de, p.rbf);
#pragma unroll 2
            for (int c = 0; c < 8; c++) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int k = ch * 64 + c * 8 + j;
                    x[j] = k < R ? ascale * phi_deriv<float, 0>(ej, env, k, p.rbf) : 0.f;
                }
                uint4 hi, lo;
                pack8<SPLIT>(x, hi, lo);
                const uint32_t off = chunk_offset(r, ch * 64 + c * 8);
                *reinterpret_cast<uint4 *>(sA_hi + off) = hi;
                if (SPLIT) *reinterpret_cast<uint4 *>(sA_lo + off) = lo;
            }
        }
        fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            issue_gemm<SPLIT>(tmem, smem_u32(sA_hi), smem_u32(sA_lo), smem_u32(sB1_hi), smem_u32(sB1_lo), Kpad1 / 16, 0);
            mma_commit(bar);
        }
        if (!mbar_wait(bar, phase)) *s_err = 1;
        phase ^= 1;
        tc_fence_after();
        __syncthreads();
        if (*s_err) break;

        // ---- epilogue 1: h = tanh(z + b1) -> A operand of GEMM 2 (GEMM 1 has finished reading sA)
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            const int col0 = ch * 64 + half * 32;
            float v[32];
            tmem_ld32(t_lane + col0, v);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float z = v[c * 8 + j] * unscale + s_b1[col0 + c * 8 + j];
                    x[j] = ascale * (SPLIT ? tanhf(z) : tanh_fast(z));
                }
                uint4 hi, lo;
                pack8<SPLIT>(x, hi, lo);
                const uint32_t off = chunk_offset(r, col0 + c * 8);
                *reinterpret_cast<uint4 *>(sA_hi + off) = hi;
                if (SPLIT) *reinterpret_cast<uint4 *>(sA_lo + off) = lo;
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            issue_gemm<SPLIT>(tmem + 128, smem_u32(sA_hi), smem_u32(sA_lo), smem_u32(sB2_hi), smem_u32(sB2_lo), kF / 16, 0);
            mma_commit(bar);
        }
        if (!mbar_wait(bar, phase)) *s_err = 1;
        phase ^= 1;
        tc_fence_after();
        __syncthreads();
        if (*s_err) break;

        // ---- epilogue 2: W = y * C(d)
        const float C = envelope_jet<float, 0>(de, p.conv).c[0] * unscale;
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            const int col0 = ch * 64 + half * 32;
            float v[32];
            tmem_ld32(t_lane + 128 + col0, v);
            if (live) {
                float4 *dst = reinterpret_cast<float4 *>(p.W + e * kF + col0);
#pragma unroll
                for (int q = 0; q < 8; q++) dst[q] = make_float4(v[4 * q] * C, v[4 * q + 1] * C, v[4 * q + 2] * C, v[4 * q + 3] * C);
            }
        }
        tc_fence_before();
        __syncthreads();   // TMEM and sA are reused by the next tile
    }

    if (*s_err && tid == 0) atomicOr(p.status, 8);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_free(tmem, 256);
}

template <bool SPLIT>
static int filter_fwd_launch(const FilterFwdParams &p, cudaStream_t st) {
    using L = FilterSmem<SPLIT>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(filter_fwd_tc_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
            return check_launch();
        configured[dev] = true;
    }
    const int64_t ntiles = (p.E + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    filter_fwd_tc_kernel<SPLIT><<<grid, kTcThreads, L::kTotal, st>>>(p);
    return check_launch();
}


// ------------------------------------------------------------------------------------------------
// Backward of the fused filter network + message product with respect to the distance:
//
//   gd[e] = sum_f gW[e,f] * dW[e,f]/dd_e ,   gW[e,:] = xl[row0(e),:] * gagg[row1(e),:]
//
// (gW is the gradient the aggregation sends to the filters; it is formed on the fly from two gathered
// node rows and never written to HBM.)  Per 128-edge tile the forward quantities are recomputed
// (phi, z, h, y) and four GEMMs run on the tensor cores:
//   Z = phi A1^T          Y = h A2^T          GH = (gW C) A2          GPHI = (GH (1-h^2)) A1
// then gd = sum_r GPHI_r phi'_r(d) + (sum_f gW_f y_f) C'(d).  The weight tiles in shared memory serve
// GEMM 3 and 4 as MN-major operands, so no transposed copies are needed; h waits in tensor memory.
// ------------------------------------------------------------------------------------------------
struct FilterBwdParams {
    FilterFwdParams f;       // d, E, rbf, conv, A1, b1, A2, status (W unused)
    const int32_t *row0, *row1;
    const float *xl, *gagg;  // [N][kF]
    float *gd;               // [E]
};

template <bool SPLIT>
__global__ void __launch_bounds__(kTcThreads, 1) filter_bwd_tc_kernel(FilterBwdParams q) {
    using namespace tc;
    using L = FilterSmem<SPLIT>;
    const FilterFwdParams &p = q.f;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sA_hi = smem + L::kA, *sA_lo = sA_hi + 32768;
    uint8_t *sB1_hi = smem + L::kB1, *sB1_lo = sB1_hi + 32768;
    uint8_t *sB2_hi = smem + L::kB2, *sB2_lo = sB2_hi + 32768;
    float *s_b1 = reinterpret_cast<float *>(smem + L::kMisc);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_b1 + kF);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);
    float *s_red = reinterpret_cast<float *>(smem + L::kMisc + 1024);   // [2][128] exchange between the two column halves
    float *s_red2 = s_red + 256;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int r = tid & 127, ch = tid >> 7;
    const int R = p.rbf.R;
    const int Kpad1 = R <= 64 ? 64 : 128;
    const float wscale = SPLIT ? kWScale : 1.f, ascale = SPLIT ? kActScale : 1.f;
    const float unscale = 1.f / (wscale * ascale);

    load_weight_tile<SPLIT>(sB1_hi, sB1_lo, p.A1, kF, R, Kpad1, wscale);
    load_weight_tile<SPLIT>(sB2_hi, sB2_lo, p.A2, kF, kF, kF, wscale);
    if (tid < kF) s_b1[tid] = p.b1[tid];
    const uint32_t bar = smem_u32(s_bar);
    if (tid == 0) {
        mbar_init(bar, 1);
        *s_err = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), 512);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t a_hi = smem_u32(sA_hi), a_lo = smem_u32(sA_lo);
    uint32_t phase = 0;

// one GEMM issued by thread 0 and awaited by everybody; leaves the loop if the wait runs out
#define RUN_GEMM(TCOL, BHI, BLO, KSTEPS, BMN, NN)                                         \
    fence_async_smem();                                                                   \
    tc_fence_before();                                                                    \
    __syncthreads();                                                                      \
    if (tid == 0) {                                                                       \
        tc_fence_after();                                                                 \
        issue_gemm<SPLIT>(tmem + (TCOL), a_hi, a_lo, smem_u32(BHI), smem_u32(BLO), (KSTEPS), (BMN), (NN)); \
        mma_commit(bar);                                                                  \
    }                                                                                     \
    if (!mbar_wait(bar, phase)) *s_err = 1;                                               \
    phase ^= 1;                                                                           \
    tc_fence_after();                                                                     \
    __syncthreads();                                                                      \
    if (*s_err) break;

    const int64_t ntiles = (p.E + kRows - 1) / kRows;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t e = tile * kRows + r;
        const bool live = e < p.E;
        const float de = live ? p.d[e] : 1.f;
        const int64_t i0 = live ? q.row0[e] : 0, i1 = live ? q.row1[e] : 0;
        const Jet<float, 1> env = envelope_jet<float, 1>(de, p.rbf);
        const Jet<float, 1> ej = edge_jet<float, 1>(de, p.rbf);
        const Jet<float, 0> env0{{env.c[0]}}, ej0{{ej.c[0]}};

        // ---- step 1: phi -> A operand, Z = phi A1^T
        if (ch * 64 < Kpad1) {
#pragma unroll 2
            for (int c = 0; c < 8; c++) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int k = ch * 64 + c * 8 + j;
                    x[j] = k < R ? ascale * phi_deriv<float, 0>(ej0, env0, k, p.rbf) : 0.f;
                }
                uint4 hi, lo;
                pack8<SPLIT>(x, hi, lo);
                const uint32_t off = chunk_offset(r, ch * 64 + c * 8);
                *reinterpret_cast<uint4 *>(sA_hi + off) = hi;
                if (SPLIT) *reinterpret_cast<uint4 *>(sA_lo + off) = lo;
            }
        }
        RUN_GEMM(0, sB1_hi, sB1_lo, Kpad1 / 16, 0, 128)

        // ---- step 2: h = tanh(z + b1): kept in tensor memory (over z) and written as the A operand; Y = h A2^T
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            const int col0 = ch * 64 + half * 32;
            float v[32];
            tmem_ld32(t_lane + col0, v);
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float z = v[j] * unscale + s_b1[col0 + j];
                v[j] = SPLIT ? tanhf(z) : tanh_fast(z);
            }
            tmem_st32(t_lane + col0, v);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] = ascale * v[c * 8 + j];
                uint4 hi, lo;
                pack8<SPLIT>(x, hi, lo);
                const uint32_t off = chunk_offset(r, col0 + c * 8);
                *reinterpret_cast<uint4 *>(sA_hi + off) = hi;
                if (SPLIT) *reinterpret_cast<uint4 *>(sA_lo + off) = lo;
            }
        }
        RUN_GEMM(128, sB2_hi, sB2_lo, kF / 16, 0, 128)

        // ---- step 3: gW from the two gathered node rows; gC = sum gW*y; gy = gW*C -> A operand; GH = gy A2
        const Jet<float, 1> cj = envelope_jet<float, 1>(de, p.conv);
        float g[64];
        float gC = 0.f, rmax = 0.f;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int col0 = ch * 64 + half * 32;
            float v[32];
            tmem_ld32(t_lane + 128 + col0, v);
            const float4 *xa = reinterpret_cast<const float4 *>(q.xl + i0 * kF + col0);
            const float4 *ga = reinterpret_cast<const float4 *>(q.gagg + i1 * kF + col0);
#pragma unroll
            for (int w = 0; w < 8; w++) {
                const float4 a = __ldg(xa + w), b = __ldg(ga + w);
                const float gw[4] = {a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float t = live ? gw[j] : 0.f;
                    gC = fmaf(t, v[4 * w + j] * unscale, gC);
                    const float gy = t * cj.c[0];
                    g[half * 32 + 4 * w + j] = gy;
                    rmax = fmaxf(rmax, fabsf(gy));
                }
            }
        }
        s_red[ch * 128 + r] = rmax;
        s_red2[ch * 128 + r] = gC;
        __syncthreads();
        gC = s_red2[r] + s_red2[128 + r];
        const float sc3 = SPLIT ? row_scale(fmaxf(s_red[r], s_red[128 + r])) : 1.f;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = g[c * 8 + j] * sc3;
            uint4 hi, lo;
            pack8<SPLIT>(x, hi, lo);
            const uint32_t off = chunk_offset(r, ch * 64 + c * 8);
            *reinterpret_cast<uint4 *>(sA_hi + off) = hi;
            if (SPLIT) *reinterpret_cast<uint4 *>(sA_lo + off) = lo;
        }
        RUN_GEMM(256, sB2_hi, sB2_lo, kF / 16, 1, 128)

        // ---- step 4: gz = gh (1 - h^2) -> A operand; GPHI = gz A1
        const float inv3 = 1.f / (sc3 * wscale);
        rmax = 0.f;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int col0 = ch * 64 + half * 32;
            float v[32], h[32];
            tmem_ld32(t_lane + 256 + col0, v);
            tmem_ld32(t_lane + col0, h);
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float gz = v[j] * inv3 * (1.f - h[j] * h[j]);
                g[half * 32 + j] = gz;
                rmax = fmaxf(rmax, fabsf(gz));
            }
        }
        __syncthreads();            // everyone has read s_red of step 3
        s_red[ch * 128 + r] = rmax;
        __syncthreads();
        const float sc4 = SPLIT ? row_scale(fmaxf(s_red[r], s_red[128 + r])) : 1.f;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = g[c * 8 + j] * sc4;
            uint4 hi, lo;
            pack8<SPLIT>(x, hi, lo);
            const uint32_t off = chunk_offset(r, ch * 64 + c * 8);
            *reinterpret_cast<uint4 *>(sA_hi + off) = hi;
            if (SPLIT) *reinterpret_cast<uint4 *>(sA_lo + off) = lo;
        }
        RUN_GEMM(384, sB1_hi, sB1_lo, kF / 16, 1, Kpad1)

        // ---- step 5: gd = sum_r gphi_r phi'_r(d) + gC C'(d)
        float acc = 0.f;
        if (ch * 64 < Kpad1) {
#pragma unroll 1
            for (int half = 0; half < 2; half++) {
                const int col0 = ch * 64 + half * 32;
                float v[32];
                tmem_ld32(t_lane + 384 + col0, v);
#pragma unroll 4
                for (int j = 0; j < 32; j++) {
                    const int k = col0 + j;
                    if (k < R) acc = fmaf(v[j], phi_deriv<float, 1>(ej, env, k, p.rbf), acc);
                }
            }
            acc *= 1.f / (sc4 * wscale);
        }
        if (ch == 0) acc = fmaf(gC, cj.c[1], acc);
        __syncthreads();            // s_red of step 4 has been read by everyone
        s_red[ch * 128 + r] = acc;
        tc_fence_before();
        __syncthreads();
        if (ch == 0 && live) q.gd[e] = s_red[r] + s_red[128 + r];
    }
#undef RUN_GEMM

    if (*s_err && tid == 0) atomicOr(p.status, 8);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_free(tmem, 512);
}

template <bool SPLIT>
static int filter_bwd_launch(const FilterBwdParams &q, cudaStream_t st) {
    using L = FilterSmem<SPLIT>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(filter_bwd_tc_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
            return check_launch();
        configured[dev] = true;
    }
    const int64_t ntiles = (q.f.E + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    filter_bwd_tc_kernel<SPLIT><<<grid, kTcThreads, L::kTotal, st>>>(q);
    return check_launch();
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" int mlcgb_filter_forward(const void *d, int64_t E, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower,
                                    double conv_upper, const void *A1, const void *b1, const void *A2, int64_t F, int precision,
                                    void *W, int32_t *status, void *stream) {
    if (int rc = check_spec(rbf, 0)) return rc;
    if (E < 0 || !status || (precision != 0 && precision != 1) || (conv_cutoff_kind != 0 && conv_cutoff_kind != 1)) return MLCGB_E_ARG;
    if (F != kF || rbf->num_rbf > 128) return MLCGB_E_LIMIT;
    if (E == 0) return MLCGB_OK;
    if (!d || !A1 || !b1 || !A2 || !W) return MLCGB_E_ARG;
    FilterFwdParams p;
    p.d = (const float *)d;
    p.E = E;
    p.rbf = to_dev<float>(rbf);
    p.conv = p.rbf;
    p.conv.cutoff_kind = conv_cutoff_kind;
    p.conv.lower = (float)conv_lower;
    p.conv.upper = (float)conv_upper;
    p.A1 = (const float *)A1;
    p.b1 = (const float *)b1;
    p.A2 = (const float *)A2;
    p.W = (float *)W;
    p.status = status;
    return precision == 0 ? filter_fwd_launch<true>(p, (cudaStream_t)stream) : filter_fwd_launch<false>(p, (cudaStream_t)stream);
}

extern "C" int mlcgb_filter_backward(const void *d, int64_t E, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower,
                                     double conv_upper, const void *A1, const void *b1, const void *A2, int64_t F, int precision,
                                     const int32_t *row0, const int32_t *row1, const void *xl, const void *gagg, int64_t N, void *gd,
                                     int32_t *status, void *stream) {
    if (int rc = check_spec(rbf, 1)) return rc;
    if (E < 0 || N < 0 || !status || (precision != 0 && precision != 1) || (conv_cutoff_kind != 0 && conv_cutoff_kind != 1)) return MLCGB_E_ARG;
    if (F != kF || rbf->num_rbf > 128) return MLCGB_E_LIMIT;
    if (E == 0) return MLCGB_OK;
    if (!d || !A1 || !b1 || !A2 || !row0 || !row1 || !xl || !gagg || !gd) return MLCGB_E_ARG;
    FilterBwdParams q;
    q.f.d = (const float *)d;
    q.f.E = E;
    q.f.rbf = to_dev<float>(rbf);
    q.f.conv = q.f.rbf;
    q.f.conv.cutoff_kind = conv_cutoff_kind;
    q.f.conv.lower = (float)conv_lower;
    q.f.conv.upper = (float)conv_upper;
    q.f.A1 = (const float *)A1;
    q.f.b1 = (const float *)b1;
    q.f.A2 = (const float *)A2;
    q.f.W = nullptr;
    q.f.status = status;
    q.row0 = row0;
    q.row1 = row1;
    q.xl = (const float *)xl;
    q.gagg = (const float *)gagg;
    q.gd = (float *)gd;
    return precision == 0 ? filter_bwd_launch<true>(q, (cudaStream_t)stream) : filter_bwd_launch<false>(q, (cudaStream_t)stream);
}
