// Fused filter-generating network on the sm_100a tensor cores (tcgen05 + TMEM).
//
//   W[e,:] = ( tanh( phi(d_e) A1^T + b1 ) A2^T ) * C(d_e)            src/mlcg/nn/schnet.py:340-341
//
// One persistent CTA per SM (512 threads: thread = one tile row x 32 columns) walks 128-edge tiles.  The
// radial basis is evaluated straight into the A operand (it never exists in HBM); A operands live in
// tensor memory (fp16 pairs packed two per 32-bit column), accumulators too; the weight tiles are
// converted once per CTA and stay in shared memory (K-major, 128-byte swizzle), and serve the backward
// GEMMs as MN-major operands.  W leaves through a swizzled shared-memory stage as whole 512-byte rows.
//
// Precision modes.  0: every fp32 value is carried as an fp16 pair (value = hi + lo, ~22 bits) and
// each GEMM runs hi*hi + hi*lo + lo*hi with fp32 accumulation — the products an fp32 GEMM forms, at
// half-precision tensor-core rate.  1: operands rounded to bf16, one product, tanh.approx.
#include <type_traits>

#include "rbf_device.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"

namespace mlcgb {

// Phase timing of the saved-hidden-layer backward (development builds only, -DMLCGB_PHASE_TIMING): thread 0 of every block adds
// the cycles between consecutive marks to per-phase totals that mlcgb_debug_phase_cycles reads back.
#ifdef MLCGB_PHASE_TIMING
__device__ unsigned long long g_phase_cycles[16];
#define PHASE_DECL long long ph_last = clock64();
#define PHASE(k)                                                          \
    if (tid == 0) {                                                       \
        const long long ph_now = clock64();                               \
        atomicAdd(&g_phase_cycles[k], (unsigned long long)(ph_now - ph_last)); \
        ph_last = clock64();                                              \
    }
#else
#define PHASE_DECL
#define PHASE(k)
#endif

constexpr int kF = 128;                 // filters / hidden width of the filter network
constexpr int kTcThreads = 512;         // thread t: row t % 128 of the tile, 32-column quarter t / 128
constexpr float kWScale = 64.f;         // power-of-two weight scaling keeps the fp16 "low" parts of the weights normal
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

struct FilterFwdParams {
    const float *d;      // [E]
    int64_t E;           // rows to process: all edges, or one edge per unordered pair when `sel` is given
    const int64_t *rows_dev;  // NULL, or the row count in device memory (written by an earlier kernel on the stream): the
                              // kernel then processes min(E, *rows_dev) rows and E only sizes the grid and the buffers
    const int32_t *sel;  // [E] edge handled by row k (NULL: k itself)
    const int32_t *twin; // reverse edge of each edge (NULL: none); with `sel`, results go to both edges of a pair
                         // (forward with `sel` alone: W has E rows, row k is the filter of edge sel[k])
    RbfDev<float> rbf;   // basis and its envelope
    RbfDev<float> conv;  // only cutoff_kind / lower / upper are used: the CFConv cutoff C(d)
    const float *A1;     // [kF][R]
    const float *b1;     // [kF]
    const float *A2;     // [kF][kF]
    float *W;            // [E][kF]
    float *H;            // NULL, or where the forward keeps h = tanh(phi A1^T + b1) for the backward (hidden_offset() order)
    int32_t *status;
};

// The hidden layer of a tile is kept in the order the threads hold it: thread (row r, 32-column quarter q) owns eight 16-byte
// chunks j; chunk (q, j) of all 128 rows is contiguous, so both kernels move it with fully coalesced 128-bit accesses and
// no staging.  Offset, in float4 units, of chunk j of quarter q of row r of tile t; a tile takes 16384 floats.
__device__ __forceinline__ int64_t hidden_offset(int64_t tile, int q, int j, int r) { return ((tile * 4 + q) * 8 + j) * 128 + r; }

// rows the kernel works on; read after the wait on the preceding kernels
__device__ __forceinline__ int64_t live_rows(const FilterFwdParams &p) {
    if (!p.rows_dev) return p.E;
    const int64_t n = *reinterpret_cast<const volatile int64_t *>(p.rows_dev);
    return n < 0 ? 0 : (n < p.E ? n : p.E);
}

template <bool SPLIT>
struct FilterSmem {
    static constexpr int kTile = SPLIT ? 2 * 32768 : 32768;   // one 128x128 operand tile (hi [+ lo])
    static constexpr int kStageBytes = 65536;                 // fp32 staging tile: 128 rows of 512 B
    static constexpr int kASize = SPLIT ? kStageBytes : kTile;
    static constexpr int kA = 0, kB1 = kASize, kB2 = kASize + kTile, kMisc = kASize + 2 * kTile;
    // misc: bias, scaled bias [2][128] f32 | basis table [128] float2 | exchange [4][128] f32 x2 | barrier, TMEM slot, error flag
    static constexpr int kBias = 0, kTable = 1024, kRed = 2048, kRed2 = 4096, kBar = 6144;
    // fp32 staging tile for coalesced global traffic: in the A region (free when the A operands live in TMEM) or its own
    static constexpr int kStage = SPLIT ? kA : kMisc + 7168;
    static constexpr int kTotal = kMisc + 7168 + (SPLIT ? 0 : kStageBytes) + 1024;   // + alignment slack
    // the backward that reads the saved hidden layer: two more [4][128] f32 exchange arrays behind everything else
    static constexpr int kExtra = kMisc + 7168 + (SPLIT ? 0 : kStageBytes);
    static constexpr int kTotalExtra = kExtra + 4096 + 1024;
};

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Per-edge part of the basis: value t(d) the basis functions are centred on and its derivative.
//   Gaussian:   g_k = exp(coeff (d - offset_k)^2)                 t = d,                 t' = 1
//   exp-normal: g_k = exp(-beta_k (u - mean_k)^2), u = exp(alpha (lower - d)):  t = u,   t' = -alpha u
// The table holds (c_k, w_k) with g_k = 2^(-w_k (t - c_k)^2), w_k = width_k log2(e)
// (widths are positive: -coeff for the Gaussian, beta_k for the exp-normal basis).
__device__ __forceinline__ void edge_arg(float d, const RbfDev<float> &s, float &t, float &dt) {
    if (s.kind == 0) {
        t = d;
        dt = 1.f;
    } else {
        t = expf(s.alpha * (-d + s.lower));
        dt = -s.alpha * t;
    }
}

// Shared set-up of both kernels: weight tiles, bias, basis table, barrier, tensor memory.
template <bool SPLIT>
__device__ __forceinline__ uint32_t filter_setup(const FilterFwdParams &p, uint8_t *smem, int Kpad1, uint32_t tmem_cols) {
    using namespace tc;
    using L = FilterSmem<SPLIT>;
    const int tid = threadIdx.x, warp = tid >> 5;
    const float wscale = SPLIT ? kWScale : 1.f;
    const bool over1 = load_weight_tile<SPLIT>(smem + L::kB1, smem + L::kB1 + 32768, p.A1, kF, p.rbf.R, Kpad1, wscale);
    const bool over2 = load_weight_tile<SPLIT>(smem + L::kB2, smem + L::kB2 + 32768, p.A2, kF, kF, kF, wscale);
    if ((over1 || over2) && blockIdx.x == 0) atomicOr(p.status, (int)kWeightRange);
    float *s_b1 = reinterpret_cast<float *>(smem + L::kMisc + L::kBias);
    float2 *s_tab = reinterpret_cast<float2 *>(smem + L::kMisc + L::kTable);
    if (tid < kF) {
        s_b1[tid] = p.b1[tid];
        float c = 1e4f, w = 1.f;                       // beyond R: 2^(-(t - 1e4)^2) = 0
        if (tid < p.rbf.R) {
            c = p.rbf.p0[tid];
            w = (p.rbf.kind == 0 ? -p.rbf.p1[0] : p.rbf.p1[tid]) * kLog2e;
        }
        s_tab[tid] = make_float2(c, w);
        s_b1[kF + tid] = p.b1[tid] * (2.f * kLog2e);    // bias pre-multiplied for the exp2-based tanh
    }
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + L::kMisc + L::kBar);
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(s_bar + 1);
    int *s_err = reinterpret_cast<int *>(s_tmem + 1);
    if (tid == 0) {
        mbar_init(smem_u32(s_bar), 1);
        *s_err = 0;
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(smem_u32(s_tmem), tmem_cols);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    return *s_tmem;
}

// h = tanh(z) for this thread's accumulator values, z = v * unscale + b1, through exp2: tanh z = sign(z) (1 - 2/(2^{|zz|} + 1)),
// zz = 2 log2(e) z.  |zz| is clamped at 30, where the result has long rounded to 1, so that four denominators can share one
// reciprocal (1/A = B C D / (A B C D), ...): five special-function operations per four values instead of eight — this phase
// runs at the special-function unit's rate — for nine extra multiplies.
template <bool SPLIT, int NC = 32>
__device__ __forceinline__ void tanh_row32(float (&v)[NC], const float *s_b1s, int col0, float unscale2) {
    const float4 *b4 = reinterpret_cast<const float4 *>(s_b1s + col0);
#pragma unroll
    for (int q = 0; q < NC / 4; q++) {
        const float4 bq = b4[q];
        const float bb[4] = {bq.x, bq.y, bq.z, bq.w};
        if (SPLIT) {
            float zz[4], den[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                zz[i] = fmaf(v[4 * q + i], unscale2, bb[i]);
                den[i] = ex2_fast(fminf(fabsf(zz[i]), 30.f)) + 1.f;
            }
            const float p01 = den[0] * den[1], p23 = den[2] * den[3];
            const float r = rcp_fast(p01 * p23);
            const float r01 = r * p23, r23 = r * p01;
            const float inv[4] = {r01 * den[1], r01 * den[0], r23 * den[3], r23 * den[2]};
#pragma unroll
            for (int i = 0; i < 4; i++) v[4 * q + i] = copysignf(fmaf(-2.f, inv[i], 1.f), zz[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) v[4 * q + i] = tanh_fast(fmaf(v[4 * q + i], unscale2, bb[i]) * (0.5f * kLn2));
        }
    }
}

// fp32 staging tile [128 rows][32 chunks of 16 B], chunk index XOR-ed with (row & 7): a thread writing its own
// row and a warp reading one whole row are both free of bank conflicts
__device__ __forceinline__ float4 *stage_chunk(uint8_t *stage, int row, int chunk) {
    return reinterpret_cast<float4 *>(stage + row * 512 + ((chunk ^ (row & 7)) << 4));
}

// ------------------------------------------------------------------------------------------------
// Forward, pipelined: the A operands (phi, h) live in tensor memory instead of shared memory, which
// leaves room for two tiles in flight.  TMEM columns: D1 [0,128) | D2 [128,256) | A of even tiles
// [256,384) | A of odd tiles [384,512) (fp16 hi in the first 64 columns of an A block, lo in the last 64).
// While GEMM 1 of tile i runs the threads store W of tile i-1; while GEMM 2 of tile i runs they evaluate
// the radial basis of tile i+1.  NT compute threads and one more warp that only issues the tensor-core instructions, when
// the compute warps have told it (one mbarrier arrival each) that an operand block is written.
// ------------------------------------------------------------------------------------------------
template <bool SPLIT, int NT>
__global__ void __launch_bounds__(NT + 32, 1) filter_fwd_pipe_kernel(FilterFwdParams p, const __grid_constant__ CUtensorMap wmap, int use_map) {
    constexpr int NC = 128 * 128 / NT;      // columns per thread: 32 with 512 threads (1024 threads x 16 columns measured no faster)
    constexpr int RPW = 128 * 32 / NT;      // rows each warp writes out: 8 or 4
    using namespace tc;
    using L = FilterSmem<SPLIT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *stage = smem + L::kA;                       // the A region of the layout is free here (split) ...
    if (!SPLIT) stage = smem + L::kStage;                // ... or the separate staging region
    const float *s_b1 = reinterpret_cast<const float *>(smem + L::kMisc + L::kBias);
    const float2 *s_tab = reinterpret_cast<const float2 *>(smem + L::kMisc + L::kTable);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + L::kMisc + L::kBar);
    uint64_t *s_bar2 = reinterpret_cast<uint64_t *>(smem + L::kMisc + L::kBar + 64);
    uint64_t *s_r1 = s_bar2 + 1, *s_r2 = s_bar2 + 2;      // operands of GEMM 1 / GEMM 2 ready (one arrival per compute warp)
    int *s_err = reinterpret_cast<int *>(reinterpret_cast<uint32_t *>(s_bar + 1) + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = tid & 127, col0 = (tid >> 7) * NC;
    const int R = p.rbf.R;
    const int Kpad1 = R <= 64 ? 64 : 128;
    const float wscale = SPLIT ? kWScale : 1.f;
    const float unscale = 1.f / wscale;

    const uint32_t tmem = filter_setup<SPLIT>(p, smem, Kpad1, 512);
    if (tid == 0) {
        mbar_init(smem_u32(s_bar2), 1);
        mbar_init(smem_u32(s_r1), NT / 32);
        mbar_init(smem_u32(s_r2), NT / 32);
    }
    __syncthreads();
    pdl_wait();                    // set-up done (weights only); from here on the distances of the previous kernels are read
    pdl_launch_dependents();
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_lane = tmem + lane_off;
    const uint32_t bar1 = smem_u32(s_bar), bar2 = smem_u32(s_bar2);
    const uint32_t b1_hi = smem_u32(smem + L::kB1), b1_lo = b1_hi + 32768, b2_hi = smem_u32(smem + L::kB2), b2_lo = b2_hi + 32768;
    uint32_t ph1 = 0, ph2 = 0;
    bool failed = false;

    const int64_t nE = live_rows(p);
    const int64_t ntiles = (nE + kRows - 1) / kRows;
    const int64_t first = blockIdx.x, step = gridDim.x;

    auto load_d = [&](int64_t tile) {
        const int64_t k = tile * kRows + r;
        return k < nE ? p.d[p.sel ? (int64_t)p.sel[k] : k] : 1.f;
    };
    const bool same_env = p.conv.cutoff_kind == p.rbf.cutoff_kind && p.conv.lower == p.rbf.lower && p.conv.upper == p.rbf.upper;
    // phi_k(d) for this thread's columns -> A operand; returns the CFConv cutoff C(d) of the row (the envelope of the basis
    // when both use the same cutoff, as SchNet builds them)
    auto basis_to_tmem = [&](float de, uint32_t ta) {
        const float env = envelope_jet<float, 0>(de, p.rbf).c[0];
        if (col0 < Kpad1) {
            float t, dt;
            edge_arg(de, p.rbf, t, dt);
            const float l2a = log2f(env);
            float x[NC];
            const float4 *tab4 = reinterpret_cast<const float4 *>(s_tab + col0);   // two (centre, width) pairs per 128-bit read
#pragma unroll
            for (int j = 0; j < NC / 2; j++) {
                const float4 cw = tab4[j];
                const float u0 = t - cw.x, u1 = t - cw.z;
                x[2 * j] = ex2_fast(fmaf(-cw.y * u0, u0, l2a));
                x[2 * j + 1] = ex2_fast(fmaf(-cw.w * u1, u1, l2a));
            }
            store_a_tmem_cols<SPLIT, NC>(ta + lane_off, col0, x, 1.f);
        }
        tmem_wait_st();
        return same_env ? env : envelope_jet<float, 0>(de, p.conv).c[0];
    };
    auto compute_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); };     // the compute warps (not the issuing one)
    // W = y * C(d): D2 -> shared-memory stage -> global memory.  With a tensor map (rows written in order) the stage is four
    // 32-column boxes in the 128-byte swizzle and one thread hands them to the copy engine, which drains them while the
    // CTA goes on; otherwise (rows scattered to an edge and its reverse) warps copy whole 512-byte rows themselves.
    auto store_w = [&](int64_t tile, float C) {
        C *= unscale;
        float v[NC];
        tmem_ld_cols<NC>(t_lane + 128 + col0, v);
        if (tid == 0) bulk_wait_read<0>();                      // the copies of the tile before have read the stage
        compute_sync();                                         // ... and every thread is done with it
        if (use_map) {
            const int chunk0 = (col0 & 31) >> 2;
#pragma unroll
            for (int q = 0; q < NC / 4; q++)
                *box_chunk(stage, col0 >> 5, r, chunk0 + q) = make_float4(v[4 * q] * C, v[4 * q + 1] * C, v[4 * q + 2] * C, v[4 * q + 3] * C);
            fence_async_smem();                                 // the copy engine reads the stage through the async proxy
            compute_sync();
            if (tid == 0) {
#pragma unroll
                for (int b = 0; b < 4; b++) tensor_store_box(&wmap, 32 * b, (int)(tile * kRows), stage + b * 16384);
                bulk_commit();
            }
            return;
        }
#pragma unroll
        for (int q = 0; q < NC / 4; q++)
            *stage_chunk(stage, r, (col0 >> 2) + q) = make_float4(v[4 * q] * C, v[4 * q + 1] * C, v[4 * q + 2] * C, v[4 * q + 3] * C);
        compute_sync();
#pragma unroll
        for (int i = 0; i < RPW; i++) {
            const int row = warp * RPW + i;
            const int64_t kr = tile * kRows + row;
            if (kr < nE) {
                const int64_t er = (p.sel && p.twin) ? (int64_t)p.sel[kr] : kr;   // sel without twin: one row per pair, in order
                const float4 w4 = *stage_chunk(stage, row, lane);
                __stcs(reinterpret_cast<float4 *>(p.W + er * kF) + lane, w4);
                if (p.sel && p.twin) __stcs(reinterpret_cast<float4 *>(p.W + (int64_t)p.twin[er] * kF) + lane, w4);   // same distance, same filter
            }
        }
    };

    // a wait that has run out is not repeated: the block runs on (on whatever the accumulators hold), so that every barrier
    // of the schedule is still reached by everybody, and reports the failure at the end
    auto await = [&](uint32_t bar, uint32_t parity) {
        if (!failed && !mbar_wait(bar, parity)) failed = true;
        tc_fence_after();
    };
    const int64_t n_local = first < ntiles ? (ntiles - first + step - 1) / step : 0;
    if (warp == NT / 32) {
        // ---- the issuing warp: per tile GEMM 1 when the basis is in its operand block, GEMM 2 when the hidden layer is.  The
        //      tensor core's queue is short, so issuing a GEMM takes about as long as the GEMM: kept off the compute warps
        for (int64_t j = 0; j < n_local; j++) {
            const uint32_t ta = tmem + 256 + (uint32_t)(j & 1) * 128, par = (uint32_t)(j & 1);
            await(smem_u32(s_r1), par);
            if (lane == 0) {
                issue_gemm_ts<SPLIT>(tmem, ta, b1_hi, b1_lo, Kpad1 / 16, 0, 128);
                mma_commit(bar1);
            }
            __syncwarp();
            await(smem_u32(s_r2), par);
            if (lane == 0) {
                issue_gemm_ts<SPLIT>(tmem + 128, ta, b2_hi, b2_lo, kF / 16, 0, 128);
                mma_commit(bar2);
            }
            __syncwarp();
        }
    } else {
        // this warp's operand stores and accumulator reads are done: one arrival on the barrier the issuing warp waits for
        auto signal = [&](uint64_t *bar) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(bar));
        };
        float c_cur = 0.f, c_prev = 0.f;
        if (n_local > 0) {
            c_cur = basis_to_tmem(load_d(first), tmem + 256);
            signal(s_r1);
        }
        int s = 0;
        for (int64_t tile = first; tile < ntiles; tile += step, s ^= 1) {
            const uint32_t ta = tmem + 256 + s * 128, ta_next = tmem + 256 + (s ^ 1) * 128;
            const int64_t next = tile + step;
            const float d_next = next < ntiles ? load_d(next) : 1.f;      // (two dependent loads: on their way while (a) and (b) run)
            // (a) GEMM 1 of this tile is running (or about to): GEMM 2 of the previous tile done -> write out its W
            if (tile != first) {
                await(bar2, ph2);
                ph2 ^= 1;
                store_w(tile - step, c_prev);
            }
            // (b) h = tanh(z + b1) -> A operand (over phi, which GEMM 1 has finished reading); GEMM 2 can go
            await(bar1, ph1);
            ph1 ^= 1;
            {
                float v[NC];
                tmem_ld_cols<NC>(t_lane + col0, v);
                tanh_row32<SPLIT, NC>(v, s_b1 + kF, col0, unscale * (2.f * kLog2e));
                store_a_tmem_cols<SPLIT, NC>(ta + lane_off, col0, v, 1.f);
                if (NC == 32 && p.H) {                               // kept for the backward (rows past the end hold finite filler)
                    float4 *hb = reinterpret_cast<float4 *>(p.H);
#pragma unroll
                    for (int j = 0; j < NC / 4; j++) __stcs(hb + hidden_offset(tile, col0 >> 5, j, r), make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
                }
                tmem_wait_st();
            }
            signal(s_r2);
            // (c) radial basis of the next tile into the other A block (GEMM 2 of the previous tile, its last reader, is done:
            //     waited for in (a)); GEMM 1 of the next tile can go (its accumulator was read in (b))
            c_prev = c_cur;
            if (next < ntiles) {
                c_cur = basis_to_tmem(d_next, ta_next);
                signal(s_r1);
            }
        }
        if (n_local > 0) {                       // W of the last tile
            await(bar2, ph2);
            store_w(first + (n_local - 1) * step, c_prev);
        }
    }

    if (failed) s_err[0] = 1;
    bulk_wait_all();
    tc_fence_before();
    __syncthreads();
    if (s_err[0] && tid == 0) atomicOr(p.status, 8);
    if (warp == 0) tmem_free(tmem, 512);
}

template <bool SPLIT>
static int filter_fwd_launch(const FilterFwdParams &p, cudaStream_t st) {
    using L = FilterSmem<SPLIT>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(filter_fwd_pipe_kernel<SPLIT, kTcThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
            return check_launch();
        configured[dev] = true;
    }
    // rows written in order (no scatter to reverse edges): the copy engine stores the tiles
    CUtensorMap wmap;
    const int use_map = (make_rows_map(&wmap, p.W, p.E, kF) && !(p.sel && p.twin)) ? 1 : 0;
    const int64_t ntiles = (p.E + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    launch_pdl(filter_fwd_pipe_kernel<SPLIT, kTcThreads>, dim3(grid), dim3(kTcThreads + 32), L::kTotal, st, p, wmap, use_map);
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
    const float *H;          // NULL (recompute the forward per tile), or the hidden layer the forward kept
    float *gd;               // [E]
    int accumulate;          // 0: gd[e] is set (and the reverse edge's entry zeroed in pair mode); 1: added to what gd holds
};

// ------------------------------------------------------------------------------------------------
// Backward, pipelined.  A operands (phi, h, gy, gz) go through one 128-column block of tensor memory;
// accumulators: T0 = Z then h (fp32) | T1 = Y then GH | T2 = GPHI.  Work placed under the GEMMs:
// the gather of gW under GEMM 2, the basis derivatives under GEMM 4, the final reduction and the store
// of gd under GEMM 1 of the next tile.
// ------------------------------------------------------------------------------------------------
template <bool SPLIT>
__global__ void __launch_bounds__(kTcThreads, 1) filter_bwd_pipe_kernel(FilterBwdParams q) {
    using namespace tc;
    using L = FilterSmem<SPLIT>;
    const FilterFwdParams &p = q.f;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *stage = SPLIT ? smem + L::kA : smem + L::kStage;
    const float *s_b1 = reinterpret_cast<const float *>(smem + L::kMisc + L::kBias);
    const float2 *s_tab = reinterpret_cast<const float2 *>(smem + L::kMisc + L::kTable);
    float *s_red = reinterpret_cast<float *>(smem + L::kMisc + L::kRed);
    float *s_red2 = reinterpret_cast<float *>(smem + L::kMisc + L::kRed2);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + L::kMisc + L::kBar);
    int *s_err = reinterpret_cast<int *>(reinterpret_cast<uint32_t *>(s_bar + 1) + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = tid & 127, qt = tid >> 7, col0 = qt * 32;
    const int R = p.rbf.R;
    const int Kpad1 = R <= 64 ? 64 : 128;
    const float wscale = SPLIT ? kWScale : 1.f;
    const float unscale = 1.f / wscale;

    const uint32_t tmem = filter_setup<SPLIT>(p, smem, Kpad1, 512);
    pdl_wait();                    // set-up done (weights only); everything below reads what earlier kernels wrote
    pdl_launch_dependents();
    const int64_t nE = live_rows(p);
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_lane = tmem + lane_off;
    const uint32_t T0 = 0, T1 = 128, T2 = 256, TA = 384;
    const uint32_t bar = smem_u32(s_bar);
    const uint32_t b1_hi = smem_u32(smem + L::kB1), b1_lo = b1_hi + 32768, b2_hi = smem_u32(smem + L::kB2), b2_lo = b2_hi + 32768;
    uint32_t phase = 0;
    bool failed = false;

    // issue one GEMM (A in tensor memory) after everybody's operand stores are visible
#define ISSUE(TCOL, BHI, BLO, KSTEPS, BMN, NN)                                                  \
    tc_fence_before();                                                                          \
    __syncthreads();                                                                            \
    if (tid == 0) {                                                                             \
        tc_fence_after();                                                                       \
        issue_gemm_ts<SPLIT>(tmem + (TCOL), tmem + TA, (BHI), (BLO), (KSTEPS), (BMN), (NN));    \
        mma_commit(bar);                                                                        \
    }
#define AWAIT()                                   \
    if (!mbar_wait(bar, phase)) failed = true;    \
    phase ^= 1;                                   \
    tc_fence_after();

    // per-row scalars: basis argument and its derivative, envelope of the basis and its derivative, CFConv cutoff C(d) and
    // C'(d) (the envelope again when both use the same cutoff, as SchNet builds them)
    const bool same_env = p.conv.cutoff_kind == p.rbf.cutoff_kind && p.conv.lower == p.rbf.lower && p.conv.upper == p.rbf.upper;
    // The four column quarters of a row sit in warps w, w+4, w+8, w+12: exchanges between them (row maxima, row sums) need only
    // those 128 threads, on a named barrier of their own (ids 1-4; every such exchange is separated from the next use of its
    // shared-memory slots by a CTA-wide barrier of the GEMM issue).
    auto row_group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + (warp & 3)) : "memory"); };
    struct EdgeScalars { float t, dt, e0, e1, c0, c1; };
    auto scalars = [&](float de) {
        EdgeScalars s;
        edge_arg(de, p.rbf, s.t, s.dt);
        const Jet<float, 1> env = envelope_jet<float, 1>(de, p.rbf);
        s.e0 = env.c[0];
        s.e1 = env.c[1];
        if (same_env) {
            s.c0 = s.e0;
            s.c1 = s.e1;
        } else {
            const Jet<float, 1> cj = envelope_jet<float, 1>(de, p.conv);
            s.c0 = cj.c[0];
            s.c1 = cj.c[1];
        }
        return s;
    };
    // row of the tile -> edge and its two nodes (0 for rows past the end)
    struct RowIdx { int64_t e; int32_t i0, i1; bool live; };
    auto row_index = [&](int64_t tile) {
        RowIdx x;
        const int64_t krow = tile * kRows + r;
        x.live = krow < nE;
        x.e = x.live ? (p.sel ? (int64_t)p.sel[krow] : krow) : 0;
        x.i0 = x.live ? q.row0[x.e] : 0;
        x.i1 = x.live ? q.row1[x.e] : 0;
        return x;
    };
    auto basis_to_tmem = [&](const EdgeScalars &es) {
        if (col0 < Kpad1) {
            const float l2a = log2f(es.e0);
            float x[32];
            const float4 *tab4 = reinterpret_cast<const float4 *>(s_tab + col0);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const float4 cw = tab4[j];
                const float u0 = es.t - cw.x, u1 = es.t - cw.z;
                x[2 * j] = ex2_fast(fmaf(-cw.y * u0, u0, l2a));
                x[2 * j + 1] = ex2_fast(fmaf(-cw.w * u1, u1, l2a));
            }
            store_a_tmem<SPLIT>(tmem + TA + lane_off, col0, x, 1.f);
        }
        tmem_wait_st();
    };

    const int64_t ntiles = (nE + kRows - 1) / kRows;
    const int64_t first = blockIdx.x, step = gridDim.x;
    EdgeScalars es{};
    RowIdx ri{0, 0, 0, false};
    const bool paired = p.sel && p.twin;          // one row per unordered pair: both directions' gW are summed
    if (first < ntiles) {
        ri = row_index(first);
        es = scalars(ri.live ? p.d[ri.e] : 1.f);
        basis_to_tmem(es);
        ISSUE(T0, b1_hi, b1_lo, Kpad1 / 16, 0, 128)
    }
    for (int64_t tile = first; tile < ntiles; tile += step) {
        const bool live = ri.live;
        const int64_t e = ri.e;
        const int64_t i0 = ri.i0, i1 = ri.i1;

        // ---- GEMM 1 done: h = tanh(z + b1) kept in T0 (fp32) and written as the A operand; issue Y = h A2^T
        AWAIT()
        {
            float v[32];
            tmem_ld32(t_lane + T0 + col0, v);
            tanh_row32<SPLIT>(v, s_b1 + kF, col0, unscale * (2.f * kLog2e));
            tmem_st32(t_lane + T0 + col0, v);
            store_a_tmem<SPLIT>(tmem + TA + lane_off, col0, v, 1.f);
            tmem_wait_st();
        }
        ISSUE(T1, b2_hi, b2_lo, kF / 16, 0, 128)

        // ---- under GEMM 2: gW = xl[row0] * gagg[row1] for this warp's 32 rows x 32 columns, four rows per instruction,
        //      turned row-per-lane through shared memory; the loads of four instructions' worth of rows are issued together
        {
            const int sub = lane >> 3, cc = (col0 >> 2) + (lane & 7);
            auto gather = [&](auto paired_tag) {
                constexpr bool kPaired = decltype(paired_tag)::value;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    float4 a[4], b[4], a2[4], b2[4];
                    float m[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int rl = (half * 4 + u) * 4 + sub;
                        const int64_t j0 = __shfl_sync(0xffffffffu, i0, rl), j1 = __shfl_sync(0xffffffffu, i1, rl);
                        m[u] = __shfl_sync(0xffffffffu, (int)live, rl) ? 1.f : 0.f;
                        a[u] = __ldg(reinterpret_cast<const float4 *>(q.xl + j0 * kF) + cc);
                        b[u] = __ldg(reinterpret_cast<const float4 *>(q.gagg + j1 * kF) + cc);
                        if (kPaired) {   // the reverse edge: xl[row1] * gagg[row0]
                            a2[u] = __ldg(reinterpret_cast<const float4 *>(q.xl + j1 * kF) + cc);
                            b2[u] = __ldg(reinterpret_cast<const float4 *>(q.gagg + j0 * kF) + cc);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int rl = (half * 4 + u) * 4 + sub;
                        float4 gw = make_float4(a[u].x * b[u].x * m[u], a[u].y * b[u].y * m[u], a[u].z * b[u].z * m[u], a[u].w * b[u].w * m[u]);
                        if (kPaired) {
                            gw.x = fmaf(a2[u].x * b2[u].x, m[u], gw.x); gw.y = fmaf(a2[u].y * b2[u].y, m[u], gw.y);
                            gw.z = fmaf(a2[u].z * b2[u].z, m[u], gw.z); gw.w = fmaf(a2[u].w * b2[u].w, m[u], gw.w);
                        }
                        *stage_chunk(stage, (r & ~31) + rl, cc) = gw;
                    }
                }
            };
            if (paired) gather(std::true_type{});
            else gather(std::false_type{});
            __syncwarp();
        }
        AWAIT()

        // ---- gC = sum gW*y; gy = gW*C -> A operand (row-scaled); issue GH = gy A2 (over Y)
        float g[32];
        float gC = 0.f, rmax = 0.f;
        {
            float v[32];
            tmem_ld32(t_lane + T1 + col0, v);
#pragma unroll
            for (int w = 0; w < 8; w++) {
                const float4 gw4 = *stage_chunk(stage, r, (col0 >> 2) + w);
                const float gw[4] = {gw4.x, gw4.y, gw4.z, gw4.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    gC = fmaf(gw[j], v[4 * w + j], gC);
                    const float gy = gw[j] * es.c0;
                    g[4 * w + j] = gy;
                    rmax = fmaxf(rmax, fabsf(gy));
                }
            }
        }
        s_red[qt * 128 + r] = rmax;
        s_red2[qt * 128 + r] = gC * unscale;
        row_group_sync();
        gC = (s_red2[r] + s_red2[128 + r]) + (s_red2[256 + r] + s_red2[384 + r]);
        const float sc3 = SPLIT ? row_scale(fmaxf(fmaxf(s_red[r], s_red[128 + r]), fmaxf(s_red[256 + r], s_red[384 + r]))) : 1.f;
        store_a_tmem<SPLIT>(tmem + TA + lane_off, col0, g, sc3);
        tmem_wait_st();
        ISSUE(T1, b2_hi, b2_lo, kF / 16, 1, 128)
        // under GEMM 3: indices and per-row scalars of the next tile
        const int64_t next = tile + step;
        EdgeScalars es_next{};
        RowIdx ri_next{0, 0, 0, false};
        if (next < ntiles) {
            ri_next = row_index(next);
            es_next = scalars(ri_next.live ? p.d[ri_next.e] : 1.f);
        }
        AWAIT()

        // ---- gz = gh (1 - h^2) -> A operand (row-scaled); issue GPHI = gz A1
        {
            const float inv3 = 1.f / (sc3 * wscale);
            rmax = 0.f;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float v[16], h[16];
                tmem_ld16(t_lane + T1 + col0 + half * 16, v);
                tmem_ld16(t_lane + T0 + col0 + half * 16, h);
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float gz = v[j] * inv3 * fmaf(-h[j], h[j], 1.f);
                    g[half * 16 + j] = gz;
                    rmax = fmaxf(rmax, fabsf(gz));
                }
            }
        }
        s_red[qt * 128 + r] = rmax;
        row_group_sync();
        const float sc4 = SPLIT ? row_scale(fmaxf(fmaxf(s_red[r], s_red[128 + r]), fmaxf(s_red[256 + r], s_red[384 + r]))) : 1.f;
        store_a_tmem<SPLIT>(tmem + TA + lane_off, col0, g, sc4);
        tmem_wait_st();
        ISSUE(T2, b1_hi, b1_lo, kF / 16, 1, Kpad1)

        // ---- under GEMM 4: basis derivatives phi'_k = g_k (env' - env 2 ln2 w_k (t - c_k) t') for this thread's columns
        if (col0 < Kpad1) {
            const float m2 = -2.f * kLn2 * es.dt * es.e0;
            const float4 *tab4 = reinterpret_cast<const float4 *>(s_tab + col0);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const float4 cw = tab4[j];
                const float u0 = es.t - cw.x, wu0 = cw.y * u0, u1 = es.t - cw.z, wu1 = cw.w * u1;
                g[2 * j] = ex2_fast(-wu0 * u0) * fmaf(m2, wu0, es.e1);      // columns at or beyond R: exactly 0
                g[2 * j + 1] = ex2_fast(-wu1 * u1) * fmaf(m2, wu1, es.e1);
            }
        }
        const float gC_dC = gC * es.c1, inv4 = 1.f / (sc4 * wscale);
        AWAIT()
        if (failed) s_err[0] = 1;

        // ---- next tile's basis -> A operand (GEMM 4 has consumed gz), issue its GEMM 1 (T0's h was consumed above)
        if (next < ntiles) basis_to_tmem(es_next);
        tc_fence_before();
        __syncthreads();
        if (s_err[0]) break;
        if (next < ntiles && tid == 0) {
            tc_fence_after();
            issue_gemm_ts<SPLIT>(tmem + T0, tmem + TA, b1_hi, b1_lo, Kpad1 / 16, 0, 128);
            mma_commit(bar);
        }

        // ---- under the next GEMM 1: gd = sum_r gphi_r phi'_r(d) + gC C'(d)
        float acc = 0.f;
        if (col0 < Kpad1) {
            float v[32];
            tmem_ld32(t_lane + T2 + col0, v);
#pragma unroll
            for (int j = 0; j < 32; j++) acc = fmaf(v[j], g[j], acc);
            acc *= inv4;
        }
        if (qt == 0) acc += gC_dC;
        s_red2[qt * 128 + r] = acc;
        tc_fence_before();
        row_group_sync();
        if (qt == 0 && live) {
            const float v = (s_red2[r] + s_red2[128 + r]) + (s_red2[256 + r] + s_red2[384 + r]);
            if (q.accumulate) {
                q.gd[e] += v;
            } else {
                q.gd[e] = v;
                if (paired) q.gd[p.twin[e]] = 0.f;   // the pair's whole gradient is carried by one of its two edges
            }
        }
        es = es_next;
        ri = ri_next;
    }
#undef ISSUE
#undef AWAIT

    tc_fence_before();
    __syncthreads();
    if (s_err[0] && tid == 0) atomicOr(p.status, 8);
    if (warp == 0) tmem_free(tmem, 512);
}

// ------------------------------------------------------------------------------------------------
// Backward with the forward's hidden layer at hand (FilterBwdParams::H): nothing of the forward is recomputed and two GEMMs
// per tile remain,
//   GH' = gW A2        gC = sum_k h_k GH'_k        gz = C(d) GH' (1 - h^2)        GPHI = gz A1
//   gd  = sum_r GPHI_r phi'_r(d) + gC C'(d)
// (gC is sum_f gW_f y_f of the kernel above: y = h A2^T, so sum_f gW_f y_f = sum_k h_k (gW A2)_k — the filter output is not
// needed either.)  A tile holds one accumulator block and one operand block of tensor memory, so two tiles are in flight
// and the tensor core works on one tile while the threads work on the other:
//
//   iteration j:   B(j)   wait GH'(j); gC, gz -> operand; issue GPHI(j)
//                  C(j)   basis derivatives under that GEMM; wait; reduce; store gd
//                  A(j+2) gather gW of tile j+2 into the slot tile j has left, issue GH'(j+2)
//
// GH'(j+1), issued an iteration earlier, has the whole of B(j) and C(j) to finish.  The index rows and distances of a tile
// are loaded two iterations, its edge ids three iterations before they are used; the hidden rows are prefetched into L2
// one phase ahead and loaded at the top of the iteration.
// ------------------------------------------------------------------------------------------------
constexpr int kSavedThreads = kTcThreads + 32;     // 16 compute warps + one warp that only issues the tensor-core instructions

template <bool SPLIT>
__global__ void __launch_bounds__(kSavedThreads, 1) filter_bwd_saved_kernel(FilterBwdParams q) {
    using namespace tc;
    using L = FilterSmem<SPLIT>;
    const FilterFwdParams &p = q.f;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *stage = SPLIT ? smem + L::kA : smem + L::kStage;
    const float2 *s_tab = reinterpret_cast<const float2 *>(smem + L::kMisc + L::kTable);
    float *s_redA = reinterpret_cast<float *>(smem + L::kMisc + L::kRed);       // row maxima of gW
    float *s_redB = reinterpret_cast<float *>(smem + L::kMisc + L::kRed2);      // row maxima of gz
    float *s_redB2 = reinterpret_cast<float *>(smem + L::kExtra);               // partial sums of gC
    float *s_redC = reinterpret_cast<float *>(smem + L::kExtra + 2048);         // partial sums of gd
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + L::kMisc + L::kBar);
    // GEMM finished: GH' of slot 0, 1; GPHI of slot 0, 1 (one arrival, from tcgen05.commit).  Operands ready and accumulator
    // free: the same four (one arrival per compute warp).
    uint64_t *s_done = reinterpret_cast<uint64_t *>(smem + L::kMisc + L::kBar + 64);
    uint64_t *s_ready = s_done + 4;
    int *s_err = reinterpret_cast<int *>(reinterpret_cast<uint32_t *>(s_bar + 1) + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = tid & 127, qt = (tid >> 7) & 3, col0 = qt * 32;
    const int R = p.rbf.R;
    const int Kpad1 = R <= 64 ? 64 : 128;
    const float wscale = SPLIT ? kWScale : 1.f;

    const uint32_t tmem = filter_setup<SPLIT>(p, smem, Kpad1, 512);
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            mbar_init(smem_u32(s_done + i), 1);
            mbar_init(smem_u32(s_ready + i), kTcThreads / 32);
        }
    }
    __syncthreads();
    pdl_wait();                    // set-up done (weights only); everything below reads what earlier kernels wrote
    pdl_launch_dependents();
    const int64_t nE = live_rows(p);
    const uint32_t b1_hi = smem_u32(smem + L::kB1), b1_lo = b1_hi + 32768, b2_hi = smem_u32(smem + L::kB2), b2_lo = b2_hi + 32768;
    const int64_t ntiles = (nE + kRows - 1) / kRows;
    const int64_t first = blockIdx.x, step = gridDim.x;
    const int64_t n_local = first < ntiles ? (ntiles - first + step - 1) / step : 0;
    bool failed = false;
    // a wait that has run out is not repeated: the block runs on (on whatever the accumulators hold), so that every
    // barrier of the schedule below is still reached by everybody, and reports the failure at the end
    auto await = [&](uint64_t *bar, uint32_t parity) {
        if (!failed && !mbar_wait(smem_u32(bar), parity)) failed = true;
        tc_fence_after();
    };

    if (warp == kTcThreads / 32) {
        // ---- the issuing warp: GH'(0), GH'(1), then per tile GPHI(j), GH'(j+2), each when its operands are ready.  The
        //      tensor core's queue is short, so issuing a GEMM takes about as long as the GEMM: kept off the compute warps
        auto gemm = [&](int s, bool gphi) {
            if (lane == 0) {
                if (gphi) issue_gemm_ts<SPLIT>(tmem + 128 * s, tmem + 256 + 128 * s, b1_hi, b1_lo, kF / 16, 1, Kpad1);
                else issue_gemm_ts<SPLIT>(tmem + 128 * s, tmem + 256 + 128 * s, b2_hi, b2_lo, kF / 16, 1, 128);
                mma_commit(smem_u32(s_done + (gphi ? 2 : 0) + s));
            }
            __syncwarp();
        };
        for (int64_t t = 0; t < 2 && t < n_local; t++) {
            await(s_ready + t, 0);
            gemm((int)t, false);
        }
        for (int64_t j = 0; j < n_local; j++) {
            const int s = (int)(j & 1);
            await(s_ready + 2 + s, (uint32_t)((j >> 1) & 1));
            gemm(s, true);
            if (j + 2 < n_local) {
                await(s_ready + s, (uint32_t)(((j + 2) >> 1) & 1));
                gemm(s, false);
            }
        }
    } else {
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t t_lane = tmem + lane_off;
        // tensor memory: accumulator of slot s at columns [128 s, 128 s + 128), operand of slot s at [256 + 128 s, ...)
        const bool same_env = p.conv.cutoff_kind == p.rbf.cutoff_kind && p.conv.lower == p.rbf.lower && p.conv.upper == p.rbf.upper;
        // The four column quarters of a row sit in warps w, w+4, w+8, w+12: exchanges between them need only those 128 threads,
        // on a named barrier of their own (ids 1-4).  Nothing in the loop below synchronises the whole block: the four row groups
        // meet only through the GEMMs, so that one group computes while another waits for memory.
        auto row_group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + (warp & 3)) : "memory"); };
        // this warp's operand stores and accumulator reads are done: one arrival on the barrier the issuing warp waits for
        auto signal = [&](uint64_t *bar) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(bar));
        };
        struct EdgeScalars { float t, dt, e0, e1, c0, c1; };
        auto scalars = [&](float de) {
            EdgeScalars s;
            edge_arg(de, p.rbf, s.t, s.dt);
            const Jet<float, 1> env = envelope_jet<float, 1>(de, p.rbf);
            s.e0 = env.c[0];
            s.e1 = env.c[1];
            if (same_env) {
                s.c0 = s.e0;
                s.c1 = s.e1;
            } else {
                const Jet<float, 1> cj = envelope_jet<float, 1>(de, p.conv);
                s.c0 = cj.c[0];
                s.c1 = cj.c[1];
            }
            return s;
        };
        const bool paired = p.sel && p.twin;          // one row per unordered pair: both directions' gW are summed
        const bool zero_twin = paired && !q.accumulate && qt == 0;
        auto tile_of = [&](int64_t j) { return first + j * step; };
        auto edge_of = [&](int64_t j) -> int32_t {      // edge handled by this thread's row of local tile j (-1: past the end)
            if (j >= n_local) return -1;
            const int64_t krow = tile_of(j) * kRows + r;
            if (krow >= nE) return -1;
            return p.sel ? p.sel[krow] : (int32_t)krow;
        };

        // gW = xl[row0] * gagg[row1] (+ the reverse edge's product in pair mode) of one tile -> operand block `ta`, rows scaled
        // by a power of two; returns the row's scale.  Four rows per load instruction, turned row-per-lane through this warp's
        // own 32 x 32 block of the stage.  Rows past the end use node 0: finite values nobody reads.
        auto gather_pack = [&](int32_t i0, int32_t i1, uint32_t ta) -> float {
            const int sub = lane >> 3, cc = (col0 >> 2) + (lane & 7);
            auto gather = [&](auto paired_tag) {
                constexpr bool kPaired = decltype(paired_tag)::value;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    float4 a[4], b[4], a2[4], b2[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int rl = (half * 4 + u) * 4 + sub;
                        const int64_t j0 = __shfl_sync(0xffffffffu, i0, rl), j1 = __shfl_sync(0xffffffffu, i1, rl);
                        a[u] = __ldg(reinterpret_cast<const float4 *>(q.xl + j0 * kF) + cc);
                        b[u] = __ldg(reinterpret_cast<const float4 *>(q.gagg + j1 * kF) + cc);
                        if (kPaired) {   // the reverse edge: xl[row1] * gagg[row0]
                            a2[u] = __ldg(reinterpret_cast<const float4 *>(q.xl + j1 * kF) + cc);
                            b2[u] = __ldg(reinterpret_cast<const float4 *>(q.gagg + j0 * kF) + cc);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int rl = (half * 4 + u) * 4 + sub;
                        float4 gw = make_float4(a[u].x * b[u].x, a[u].y * b[u].y, a[u].z * b[u].z, a[u].w * b[u].w);
                        if (kPaired) {
                            gw.x = fmaf(a2[u].x, b2[u].x, gw.x); gw.y = fmaf(a2[u].y, b2[u].y, gw.y);
                            gw.z = fmaf(a2[u].z, b2[u].z, gw.z); gw.w = fmaf(a2[u].w, b2[u].w, gw.w);
                        }
                        *stage_chunk(stage, (r & ~31) + rl, cc) = gw;
                    }
                }
            };
            if (paired) gather(std::true_type{});
            else gather(std::false_type{});
            __syncwarp();
            float g[32];
            float rmax = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) {
                const float4 gw4 = *stage_chunk(stage, r, (col0 >> 2) + w);
                g[4 * w] = gw4.x; g[4 * w + 1] = gw4.y; g[4 * w + 2] = gw4.z; g[4 * w + 3] = gw4.w;
                rmax = fmaxf(fmaxf(rmax, fmaxf(fabsf(gw4.x), fabsf(gw4.y))), fmaxf(fabsf(gw4.z), fabsf(gw4.w)));
            }
            __syncwarp();
            s_redA[qt * 128 + r] = rmax;
            row_group_sync();
            const float sc = SPLIT ? row_scale(fmaxf(fmaxf(s_redA[r], s_redA[128 + r]), fmaxf(s_redA[256 + r], s_redA[384 + r]))) : 1.f;
            store_a_tmem<SPLIT>(ta + lane_off, col0, g, sc);
            tmem_wait_st();
            return sc;
        };
        auto prefetch_hidden = [&](int64_t j) {      // the tile's 64 KB of hidden rows into L2, one 128-byte line per thread
            if (j < n_local) asm volatile("prefetch.global.L2 [%0];" ::"l"(q.H + tile_of(j) * (kRows * kF) + tid * 32));
        };

        // ---- state of the tiles in flight: (edge, reverse edge, scalars, gW scale) of tile j (being finished) and j+1 (GH' issued)
        int32_t e_cur = -1, e_nx = -1, tw_cur = 0, tw_nx = 0;
        EdgeScalars es_cur{}, es_nx{};
        float sc3_cur = 1.f, sc3_nx = 1.f;
        // prologue: gather tiles 0 and 1
        {
            const int32_t e_a = edge_of(0), e_b = edge_of(1);
            const bool la = e_a >= 0, lb = e_b >= 0;
            const int32_t a0 = la ? q.row0[e_a] : 0, a1 = la ? q.row1[e_a] : 0, b0 = lb ? q.row0[e_b] : 0, b1i = lb ? q.row1[e_b] : 0;
            const float da = la ? p.d[e_a] : 1.f, db = lb ? p.d[e_b] : 1.f;
            if (n_local > 0) {
                prefetch_hidden(0);
                e_cur = e_a;
                tw_cur = (zero_twin && la) ? p.twin[e_a] : 0;
                es_cur = scalars(da);
                sc3_cur = gather_pack(a0, a1, tmem + 256);
                signal(s_ready + 0);
            }
            if (n_local > 1) {
                prefetch_hidden(1);
                e_nx = e_b;
                tw_nx = (zero_twin && lb) ? p.twin[e_b] : 0;
                es_nx = scalars(db);
                sc3_nx = gather_pack(b0, b1i, tmem + 256 + 128);
                signal(s_ready + 1);
            }
        }
        int32_t e_pre = edge_of(2);                   // edge id of the tile after those: its rows are loaded in the first iteration
        PHASE_DECL
        for (int64_t j = 0; j < n_local; j++) {
            PHASE(0)
            const int s = (int)(j & 1);
            const uint32_t par = (uint32_t)((j >> 1) & 1);
            const uint32_t D = 128u * s, TA = 256u + 128u * s;
            const bool live = e_cur >= 0;
            // ---- loads whose results are needed later: the hidden rows of this tile (B), rows, distance and reverse edge of tile
            //      j+2 (A below), edge id of tile j+3 (next iteration)
            float4 hq[8];
            {
                const float4 *hb = reinterpret_cast<const float4 *>(q.H);
                const int64_t t = tile_of(j);
#pragma unroll
                for (int c = 0; c < 8; c++) hq[c] = hb[hidden_offset(t, qt, c, r)];
            }
            const int32_t e_g = e_pre;                 // tile j+2
            const bool lg = e_g >= 0;
            const int32_t g0 = lg ? q.row0[e_g] : 0, g1 = lg ? q.row1[e_g] : 0;
            const float dg = lg ? p.d[e_g] : 1.f;
            const int32_t tw_g = (zero_twin && lg) ? p.twin[e_g] : 0;
            e_pre = edge_of(j + 3);

            // ---- B(j): GH' done.  gC = sum h GH', gz = C GH' (1 - h^2) -> operand (row-scaled); GPHI = gz A1 can go
            PHASE(1)
            await(s_done + s, par);
            PHASE(2)
            float g[32];
            float gC = 0.f, rmax = 0.f;
            {
                const float inv3 = 1.f / (sc3_cur * wscale);
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    float v[16];
                    tmem_ld16(t_lane + D + col0 + half * 16, v);
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float4 h4 = hq[half * 4 + c];
                        const float hh[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float gh = v[4 * c + i] * inv3;
                            gC = fmaf(hh[i], gh, gC);
                            const float gz = es_cur.c0 * gh * fmaf(-hh[i], hh[i], 1.f);
                            g[half * 16 + 4 * c + i] = gz;
                            rmax = fmaxf(rmax, fabsf(gz));
                        }
                    }
                }
            }
            PHASE(3)
            s_redB[qt * 128 + r] = rmax;
            s_redB2[qt * 128 + r] = gC;
            row_group_sync();
            gC = (s_redB2[r] + s_redB2[128 + r]) + (s_redB2[256 + r] + s_redB2[384 + r]);
            const float sc4 = SPLIT ? row_scale(fmaxf(fmaxf(s_redB[r], s_redB[128 + r]), fmaxf(s_redB[256 + r], s_redB[384 + r]))) : 1.f;
            store_a_tmem<SPLIT>(tmem + TA + lane_off, col0, g, sc4);
            tmem_wait_st();
            PHASE(4)
            signal(s_ready + 2 + s);
            PHASE(5)

            // ---- C(j), under GPHI: basis derivatives phi'_k = g_k (env' - env 2 ln2 w_k (t - c_k) t') for this thread's columns,
            //      and the per-row scalars of tile j+2
            if (col0 < Kpad1) {
                const float m2 = -2.f * kLn2 * es_cur.dt * es_cur.e0;
                const float4 *tab4 = reinterpret_cast<const float4 *>(s_tab + col0);
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    const float4 cw = tab4[c];
                    const float u0 = es_cur.t - cw.x, wu0 = cw.y * u0, u1 = es_cur.t - cw.z, wu1 = cw.w * u1;
                    g[2 * c] = ex2_fast(-wu0 * u0) * fmaf(m2, wu0, es_cur.e1);      // columns at or beyond R: exactly 0
                    g[2 * c + 1] = ex2_fast(-wu1 * u1) * fmaf(m2, wu1, es_cur.e1);
                }
            }
            const float gC_dC = gC * es_cur.c1, inv4 = 1.f / (sc4 * wscale);
            if (j + 1 < n_local) prefetch_hidden(j + 1);
            const EdgeScalars es_g = scalars(dg);
            PHASE(6)
            await(s_done + 2 + s, par);
            PHASE(7)
            float acc = 0.f;
            if (col0 < Kpad1) {
                float v[32];
                tmem_ld32(t_lane + D + col0, v);
#pragma unroll
                for (int c = 0; c < 32; c++) acc = fmaf(v[c], g[c], acc);
                acc *= inv4;
            }
            if (qt == 0) acc += gC_dC;
            s_redC[qt * 128 + r] = acc;
            row_group_sync();
            if (qt == 0 && live) {
                const float v = (s_redC[r] + s_redC[128 + r]) + (s_redC[256 + r] + s_redC[384 + r]);
                if (q.accumulate) {
                    atomicAdd(q.gd + e_cur, v);         // (one addition per entry and launch: the result does not depend on timing)
                } else {
                    q.gd[e_cur] = v;
                    if (paired) q.gd[tw_cur] = 0.f;     // the pair's whole gradient is carried by one of its two edges
                }
            }
            PHASE(8)

            // ---- A(j+2): the slot is free (GPHI(j) has been read): gather gW of tile j+2 into it; its GH' can go
            e_cur = e_nx;
            tw_cur = tw_nx;
            es_cur = es_nx;
            sc3_cur = sc3_nx;
            if (j + 2 < n_local) {
                e_nx = e_g;
                tw_nx = tw_g;
                es_nx = es_g;
                PHASE(9)
                sc3_nx = gather_pack(g0, g1, tmem + TA);
                PHASE(10)
                signal(s_ready + s);
                PHASE(11)
            }
        }
    }

    if (failed) s_err[0] = 1;
    tc_fence_before();
    __syncthreads();
    if (s_err[0] && tid == 0) atomicOr(p.status, 8);
    if (warp == 0) tmem_free(tmem, 512);
}

template <bool SPLIT>
static int filter_bwd_saved_launch(const FilterBwdParams &q, cudaStream_t st) {
    using L = FilterSmem<SPLIT>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(filter_bwd_saved_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotalExtra) != cudaSuccess)
            return check_launch();
        configured[dev] = true;
    }
    const int64_t ntiles = (q.f.E + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    launch_pdl(filter_bwd_saved_kernel<SPLIT>, dim3(grid), dim3(kSavedThreads), L::kTotalExtra, st, q);
    return check_launch();
}

template <bool SPLIT>
static int filter_bwd_launch(const FilterBwdParams &q, cudaStream_t st) {
    using L = FilterSmem<SPLIT>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(filter_bwd_pipe_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
            return check_launch();
        configured[dev] = true;
    }
    const int64_t ntiles = (q.f.E + tc::kRows - 1) / tc::kRows;
    const int grid = (int)(ntiles < kNumSM ? ntiles : kNumSM);
    launch_pdl(filter_bwd_pipe_kernel<SPLIT>, dim3(grid), dim3(kTcThreads), L::kTotal, st, q);
    return check_launch();
}

}  // namespace mlcgb

using namespace mlcgb;

#ifdef MLCGB_PHASE_TIMING
extern "C" int mlcgb_debug_phase_cycles(unsigned long long *out, int n, int reset) {
    unsigned long long host[16];
    if (cudaMemcpyFromSymbol(host, mlcgb::g_phase_cycles, sizeof(host)) != cudaSuccess) return MLCGB_E_LAUNCH;
    for (int i = 0; i < n && i < 16; i++) out[i] = host[i];
    if (reset) {
        unsigned long long zero[16] = {0};
        if (cudaMemcpyToSymbol(mlcgb::g_phase_cycles, zero, sizeof(zero)) != cudaSuccess) return MLCGB_E_LAUNCH;
    }
    return MLCGB_OK;
}
#endif

extern "C" size_t mlcgb_filter_hidden_bytes(int64_t rows) {
    return rows <= 0 ? 0 : (size_t)((rows + tc::kRows - 1) / tc::kRows) * tc::kRows * kF * sizeof(float);
}

extern "C" int mlcgb_filter_forward_counted(const void *d, int64_t E, const int64_t *rows_dev, const int32_t *sel, const int32_t *twin,
                                            const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper,
                                            const void *A1, const void *b1, const void *A2, int64_t F, int precision, void *W,
                                            void *h_save, int32_t *status, void *stream) {
    TimelineScope timeline_scope("filter_forward", stream);
    if (int rc = check_spec(rbf, 0)) return rc;
    if (E < 0 || !status || (precision != 0 && precision != 1) || (conv_cutoff_kind != 0 && conv_cutoff_kind != 1)) return MLCGB_E_ARG;
    if (F != kF || rbf->num_rbf > 128) return MLCGB_E_LIMIT;
    if (E == 0) return MLCGB_OK;
    if (!d || !A1 || !b1 || !A2 || !W) return MLCGB_E_ARG;
    FilterFwdParams p;
    p.d = (const float *)d;
    p.E = E;
    p.rows_dev = rows_dev;
    p.sel = sel;
    p.twin = twin;
    p.rbf = to_dev<float>(rbf);
    p.conv = p.rbf;
    p.conv.cutoff_kind = conv_cutoff_kind;
    p.conv.lower = (float)conv_lower;
    p.conv.upper = (float)conv_upper;
    p.A1 = (const float *)A1;
    p.b1 = (const float *)b1;
    p.A2 = (const float *)A2;
    p.W = (float *)W;
    p.H = (float *)h_save;
    p.status = status;
    return precision == 0 ? filter_fwd_launch<true>(p, (cudaStream_t)stream) : filter_fwd_launch<false>(p, (cudaStream_t)stream);
}

extern "C" int mlcgb_filter_forward(const void *d, int64_t E, const int32_t *sel, const int32_t *twin, const mlcgb_rbf_spec *rbf,
                                    int conv_cutoff_kind, double conv_lower, double conv_upper, const void *A1, const void *b1,
                                    const void *A2, int64_t F, int precision, void *W, void *h_save, int32_t *status, void *stream) {
    TimelineScope timeline_scope("filter_forward", stream);
    return mlcgb_filter_forward_counted(d, E, nullptr, sel, twin, rbf, conv_cutoff_kind, conv_lower, conv_upper, A1, b1, A2, F, precision, W,
                                        h_save, status, stream);
}

extern "C" int mlcgb_filter_backward_counted(const void *d, int64_t E, const int64_t *rows_dev, const int32_t *sel, const int32_t *twin,
                                             const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper,
                                             const void *A1, const void *b1, const void *A2, int64_t F, int precision,
                                             const int32_t *row0, const int32_t *row1, const void *xl, const void *gagg, int64_t N,
                                             const void *h_saved, void *gd, int accumulate, int32_t *status, void *stream) {
    TimelineScope timeline_scope("filter_backward", stream);
    if (int rc = check_spec(rbf, 1)) return rc;
    if (E < 0 || N < 0 || !status || (precision != 0 && precision != 1) || (conv_cutoff_kind != 0 && conv_cutoff_kind != 1)) return MLCGB_E_ARG;
    if (F != kF || rbf->num_rbf > 128) return MLCGB_E_LIMIT;
    if (E == 0) return MLCGB_OK;
    if (!d || !A1 || !b1 || !A2 || !row0 || !row1 || !xl || !gagg || !gd) return MLCGB_E_ARG;
    FilterBwdParams q;
    q.f.d = (const float *)d;
    q.f.E = E;
    q.f.rows_dev = rows_dev;
    q.f.sel = sel;
    q.f.twin = twin;
    q.f.rbf = to_dev<float>(rbf);
    q.f.conv = q.f.rbf;
    q.f.conv.cutoff_kind = conv_cutoff_kind;
    q.f.conv.lower = (float)conv_lower;
    q.f.conv.upper = (float)conv_upper;
    q.f.A1 = (const float *)A1;
    q.f.b1 = (const float *)b1;
    q.f.A2 = (const float *)A2;
    q.f.W = nullptr;
    q.f.H = nullptr;
    q.f.status = status;
    q.row0 = row0;
    q.row1 = row1;
    q.xl = (const float *)xl;
    q.gagg = (const float *)gagg;
    q.H = (const float *)h_saved;
    q.gd = (float *)gd;
    q.accumulate = accumulate ? 1 : 0;
    if (q.H) return precision == 0 ? filter_bwd_saved_launch<true>(q, (cudaStream_t)stream) : filter_bwd_saved_launch<false>(q, (cudaStream_t)stream);
    return precision == 0 ? filter_bwd_launch<true>(q, (cudaStream_t)stream) : filter_bwd_launch<false>(q, (cudaStream_t)stream);
}

extern "C" int mlcgb_filter_backward(const void *d, int64_t E, const int32_t *sel, const int32_t *twin, const mlcgb_rbf_spec *rbf,
                                     int conv_cutoff_kind, double conv_lower, double conv_upper, const void *A1, const void *b1,
                                     const void *A2, int64_t F, int precision, const int32_t *row0, const int32_t *row1, const void *xl,
                                     const void *gagg, int64_t N, const void *h_saved, void *gd, int32_t *status, void *stream) {
    TimelineScope timeline_scope("filter_backward", stream);
    return mlcgb_filter_backward_counted(d, E, nullptr, sel, twin, rbf, conv_cutoff_kind, conv_lower, conv_upper, A1, b1, A2, F, precision,
                                         row0, row1, xl, gagg, N, h_saved, gd, 0, status, stream);
}
