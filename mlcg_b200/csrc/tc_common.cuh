// sm_100a tensor-core plumbing shared by the fused filter-network kernels and the tensor-core GEMMs:
// shared-memory layout of the B (weight) operand (K-major, 128-byte swizzle), UMMA descriptors,
// tcgen05.mma with the A operand in tensor memory, commit / ld / st, TMEM allocation, bounded mbarrier waits,
// fp16 hi/lo packing.
//
// Weight tiles hold 2-byte elements (bf16 or fp16).  A [rows][K] tile is stored as K/64 "atoms";
// one atom is [rows][64 elements] = rows x 128 bytes, rows grouped by 8 (1024 bytes per group), and
// inside a group the 16-byte chunk index of a row is XOR-ed with the row index modulo 8.  That is
// the canonical K-major SWIZZLE_128B layout the tensor core reads through a matrix descriptor with
// stride-byte-offset 1024; the same bytes can be read as an MN-major operand (rows = K index) with
// leading-byte-offset = the atom size.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.cuh"

namespace mlcgb {
namespace tc {

constexpr int kRows = 128;                       // tile rows (M of the MMA, edges per tile)
constexpr int kAtomBytes = kRows * 128;          // one 64-element column block of a 128-row tile
constexpr uint32_t kSpinLimit = 1u << 22;        // bounded wait on an mbarrier

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of the 16-byte chunk holding elements [k0, k0+8) of row r (k0 a multiple of 8)
__device__ __forceinline__ uint32_t chunk_offset(int r, int k0) {
    const int atom = k0 >> 6, chunk = (k0 & 63) >> 3;
    return (uint32_t)(atom * kAtomBytes + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}
// byte offset of a single 2-byte element (used when filling the weight tiles)
__device__ __forceinline__ uint32_t elem_offset(int r, int k) { return chunk_offset(r, k & ~7) + ((k & 7) << 1); }

// ---- matrix descriptors --------------------------------------------------------------------------
// bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
// [46,48) version (1 on sm_100), [61,64) layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// the same storage read with rows as the K index and the 64-element blocks along N (MN-major)
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(kAtomBytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// descriptor of K-step ks (16 elements) of a K-major tile
__device__ __forceinline__ uint64_t kstep_kmajor(uint64_t base, int ks) {
    return base + (uint64_t)(((ks >> 2) * kAtomBytes + (ks & 3) * 32) >> 4);
}
// descriptor of K-step ks (16 rows) of an MN-major tile
__device__ __forceinline__ uint64_t kstep_mnmajor(uint64_t base, int ks) { return base + (uint64_t)((ks * 16 * 128) >> 4); }

// instruction descriptor: fp32 accumulate, A/B format fmt (0 = fp16, 1 = bf16), M = 128, N = n (multiple of 16)
__device__ __forceinline__ uint32_t instr_desc(int fmt, int b_mn_major, int n) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)b_mn_major << 16) | (((uint32_t)n >> 3) << 17) |
           ((128u >> 4) << 24);
}

__device__ __forceinline__ void mma_commit(uint32_t bar_saddr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_saddr) : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar_saddr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_saddr), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar_saddr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_saddr) : "memory");
}

// Waits for the phase with the given parity; gives up after kSpinLimit polls and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar_saddr, uint32_t parity) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(bar_saddr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// ---- tensor memory ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t slot_saddr, uint32_t ncols) {   // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_saddr), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t ncols) {         // the same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 consecutive columns of this thread's TMEM lane (lane = 32*(warp%4) + laneid): v[j] = D[row][col0 + j]
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
}

// 16 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Fill a [128][Kpad] weight tile (and its low part) from a row-major fp32 matrix src[rows][K], scaled by `scale`.
// Four consecutive K elements of a row are 8 contiguous bytes of the swizzled tile, so with K % 4 == 0 and a 16-byte
// aligned source every thread moves float4 -> 8 bytes, with all its loads issued before the first conversion.
// Returns true if this thread saw a scaled weight too large for a 16-bit operand (|w * scale| > 32768 with fp16 pairs):
// the caller reports it through its status word instead of computing with infinities.
template <bool SPLIT>
__device__ __forceinline__ bool load_weight_tile(uint8_t *hi, uint8_t *lo, const float *__restrict__ src, int rows, int K, int Kpad,
                                                 float scale) {
    float wmax = 0.f;
    auto put4 = [&](int n, int k, float4 w) {
        wmax = fmaxf(fmaxf(wmax, fmaxf(fabsf(w.x), fabsf(w.y))), fmaxf(fabsf(w.z), fabsf(w.w)));
        const uint32_t off = elem_offset(n, k);
        if (SPLIT) {
            const __half2 a0 = __floats2half2_rn(w.x * scale, w.y * scale), a1 = __floats2half2_rn(w.z * scale, w.w * scale);
            const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
            const __half2 c0 = __floats2half2_rn(w.x * scale - f0.x, w.y * scale - f0.y), c1 = __floats2half2_rn(w.z * scale - f1.x, w.w * scale - f1.y);
            *reinterpret_cast<uint2 *>(hi + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1));
            *reinterpret_cast<uint2 *>(lo + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&c0), *reinterpret_cast<const uint32_t *>(&c1));
        } else {
            const __nv_bfloat162 a0 = __floats2bfloat162_rn(w.x * scale, w.y * scale), a1 = __floats2bfloat162_rn(w.z * scale, w.w * scale);
            *reinterpret_cast<uint2 *>(hi + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1));
        }
    };
    const int qpr = Kpad >> 2, nquads = kRows * qpr;          // quads per row, quads in the tile
    if ((K & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        constexpr int kBatch = 8;
        for (int base = threadIdx.x; base < nquads; base += kBatch * blockDim.x) {
            float4 w[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; u++) {
                const int qd = base + u * blockDim.x;
                const int n = qd / qpr, k = (qd - n * qpr) << 2;
                w[u] = (qd < nquads && n < rows && k < K) ? __ldg(reinterpret_cast<const float4 *>(src + (int64_t)n * K + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < kBatch; u++) {
                const int qd = base + u * blockDim.x;
                if (qd < nquads) {
                    const int n = qd / qpr;
                    put4(n, (qd - n * qpr) << 2, w[u]);
                }
            }
        }
        return SPLIT && !(wmax * scale <= 32768.f);
    }
    for (int qd = threadIdx.x; qd < nquads; qd += blockDim.x) {
        const int n = qd / qpr, k = (qd - n * qpr) << 2;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = (n < rows && k + j < K) ? src[(int64_t)n * K + k + j] : 0.f;
        put4(n, k, make_float4(v[0], v[1], v[2], v[3]));
    }
    return SPLIT && !(wmax * scale <= 32768.f);     // (also true for NaN weights)
}

// ---- A operand in tensor memory -----------------------------------------------------------------------
// For 16-bit operands the tensor core can read A straight from TMEM: lane = row, each 32-bit column holds two
// consecutive K elements (even k in the low half), so a K-step of 16 spans 8 columns.
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 fp32 values of one row (K range [k0, k0+32)) -> 16 packed columns of the high part (and of the low part)
template <bool SPLIT>
__device__ __forceinline__ void pack32(const float (&x)[32], float scale, uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const float a0 = x[2 * i] * scale, a1 = x[2 * i + 1] * scale;
        if (SPLIT) {
            const __half2 a = __floats2half2_rn(a0, a1);
            const float2 b = __half22float2(a);
            const __half2 c = __floats2half2_rn(a0 - b.x, a1 - b.y);
            hi[i] = *reinterpret_cast<const uint32_t *>(&a);
            lo[i] = *reinterpret_cast<const uint32_t *>(&c);
        } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(a0, a1);
            hi[i] = *reinterpret_cast<const uint32_t *>(&a);
            lo[i] = 0u;
        }
    }
}

// write this thread's 32 K-elements of its row into the TMEM A operand (hi block at ta, lo block 64 columns further)
template <bool SPLIT>
__device__ __forceinline__ void store_a_tmem(uint32_t ta_lane, int k0, const float (&x)[32], float scale) {
    uint32_t hi[16], lo[16];
    pack32<SPLIT>(x, scale, hi, lo);
    tmem_st16(ta_lane + (k0 >> 1), hi);
    if (SPLIT) tmem_st16(ta_lane + 64 + (k0 >> 1), lo);
}


__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
        : "memory");
}

// N = 32 or 16 columns per thread
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, float (&v)[N]);
template <> __device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, float (&v)[32]) { tmem_ld32(taddr, v); }
template <> __device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, float (&v)[16]) { tmem_ld16(taddr, v); }

// N fp32 values of one row (K range [k0, k0+N)) -> N/2 packed columns of the A operand in TMEM (hi block at ta, lo block 64
// columns further)
template <bool SPLIT, int N>
__device__ __forceinline__ void store_a_tmem_cols(uint32_t ta_lane, int k0, const float (&x)[N], float scale) {
    uint32_t hi[N / 2], lo[N / 2];
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
        const float a0 = x[2 * i] * scale, a1 = x[2 * i + 1] * scale;
        if (SPLIT) {
            const __half2 a = __floats2half2_rn(a0, a1);
            const float2 b = __half22float2(a);
            const __half2 c = __floats2half2_rn(a0 - b.x, a1 - b.y);
            hi[i] = *reinterpret_cast<const uint32_t *>(&a);
            lo[i] = *reinterpret_cast<const uint32_t *>(&c);
        } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(a0, a1);
            hi[i] = *reinterpret_cast<const uint32_t *>(&a);
            lo[i] = 0u;
        }
    }
    if constexpr (N == 32) {
        tmem_st16(ta_lane + (k0 >> 1), hi);
        if (SPLIT) tmem_st16(ta_lane + 64 + (k0 >> 1), lo);
    } else {
        tmem_st8(ta_lane + (k0 >> 1), hi);
        if (SPLIT) tmem_st8(ta_lane + 64 + (k0 >> 1), lo);
    }
}

// GEMM with the A operand in tensor memory (hi at ta, lo at ta + 64 columns)
template <bool SPLIT>
__device__ __forceinline__ void issue_gemm_ts(uint32_t tmem_d, uint32_t ta, uint32_t b_hi, uint32_t b_lo, int ksteps, int b_mn, int n = 128) {
    const uint32_t idesc = instr_desc(SPLIT ? 0 : 1, b_mn, n);
    const uint64_t dbh = b_mn ? desc_mnmajor(b_hi) : desc_kmajor(b_hi), dbl = b_mn ? desc_mnmajor(b_lo) : desc_kmajor(b_lo);
    for (int ks = 0; ks < ksteps; ks++) {
        const uint64_t bh = b_mn ? kstep_mnmajor(dbh, ks) : kstep_kmajor(dbh, ks);
        const uint64_t bl = b_mn ? kstep_mnmajor(dbl, ks) : kstep_kmajor(dbl, ks);
        mma_f16_ts(tmem_d, ta + ks * 8, bh, idesc, ks > 0 ? 1u : 0u);
        if (SPLIT) {
            mma_f16_ts(tmem_d, ta + ks * 8, bl, idesc, 1u);
            mma_f16_ts(tmem_d, ta + 64 + ks * 8, bh, idesc, 1u);
        }
    }
}

// tanh through exp2: tanh z = sign(z) (1 - 2 / (2^{2 log2(e) |z|} + 1)); 2^x overflowing to inf gives exactly 1.
// Two special-function operations, about 1e-6 relative accuracy.
__device__ __forceinline__ float tanh_ex2(float z) {
    const float zz = z * 2.8853900817779268f;
    float t, rr;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fabsf(zz)));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rr) : "f"(t + 1.f));
    return copysignf(fmaf(-2.f, rr, 1.f), zz);
}

// Power-of-two factor that brings a row whose largest magnitude is `rmax` to [8, 16): exact to apply and to
// undo, keeps fp16 operands far from overflow and their low parts out of the subnormal range.
__device__ __forceinline__ float row_scale(float rmax) {
    if (!(rmax > 0.f) || !isfinite(rmax)) return 1.f;
    int ex = (int)((__float_as_uint(rmax) >> 23) & 0xffu) - 126;   // rmax = m * 2^ex, m in [0.5, 1)
    ex = ex < -100 ? -100 : (ex > 100 ? 100 : ex);
    return __uint_as_float((uint32_t)(127 + 4 - ex) << 23);
}

}  // namespace tc
}  // namespace mlcgb
