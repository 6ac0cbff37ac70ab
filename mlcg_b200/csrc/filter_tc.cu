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
    static constexpr int kTotal = kMisc + 1024 + 1024;        // + misc + alignment slack
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
