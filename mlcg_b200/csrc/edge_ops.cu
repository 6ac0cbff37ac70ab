// Gather / segmented-sum primitives of the continuous-filter convolution and of the edge geometry.
//
// All of them are bandwidth kernels: an [E,F] edge tensor is streamed once with 128-bit loads
// (one warp covers a 512-byte row when F = 128), node rows are gathered (they stay L2-resident:
// N*F*4 bytes is a few tens of MB), and sums run over a CSR segment in edge order, so results are
// reproducible run to run and no atomics are issued.
#include "common.cuh"

namespace mlcgb {

template <typename T> struct VecIO;
template <> struct VecIO<float> {
    using V = float4;
    static constexpr int W = 4;
};
template <> struct VecIO<double> {
    using V = double2;
    static constexpr int W = 2;
};

__device__ __forceinline__ float4 vmul(const float4 &a, const float4 &b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ double2 vmul(const double2 &a, const double2 &b) { return make_double2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ void vfma(float4 &acc, const float4 &a, const float4 &b) {
    acc.x = fmaf(a.x, b.x, acc.x); acc.y = fmaf(a.y, b.y, acc.y); acc.z = fmaf(a.z, b.z, acc.z); acc.w = fmaf(a.w, b.w, acc.w);
}
__device__ __forceinline__ void vfma(double2 &acc, const double2 &a, const double2 &b) {
    acc.x = fma(a.x, b.x, acc.x); acc.y = fma(a.y, b.y, acc.y);
}
__device__ __forceinline__ float4 vzero(float4 *) { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ double2 vzero(double2 *) { return make_double2(0.0, 0.0); }

// streaming (evict-first) load for edge tensors that are read exactly once
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ double2 ld_stream(const double2 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, const float4 &v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(double2 *p, const double2 &v) { __stcs(p, v); }

// ------------------------------------------------------------------------------- seg_mul_sum
// One group of G lanes per destination row; G*W elements per pass over the feature dimension.
// PERM: rows of V are picked through eperm.  Such rows may be shared between destination rows (a filter stored once
// per pair of a symmetric list is read from both ends), so they are loaded with the default cache policy and the
// second reader finds them in L2; rows read in order are read once and loaded with the streaming hint.
template <typename T, int G, bool VEC, bool PERM>
__global__ void __launch_bounds__(256)
seg_mul_sum_kernel(const T *__restrict__ a, const T *__restrict__ V, const int64_t *__restrict__ ptr,
                   const int32_t *__restrict__ nbr, const int32_t *__restrict__ eperm, int64_t N, int64_t F,
                   T *__restrict__ out) {
    using VT = typename VecIO<T>::V;
    constexpr int W = VEC ? VecIO<T>::W : 1;
    const int gl = threadIdx.x % G;
    const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) / G;
    const int64_t Fv = F / W;  // vectors per row
    for (int64_t n = group; n < N; n += ngroups) {
        const int64_t k0 = ptr[n], k1 = ptr[n + 1];
        for (int64_t c = gl; c < Fv; c += G) {
            if (VEC) {
                VT acc0 = vzero((VT *)nullptr), acc1 = vzero((VT *)nullptr);
                int64_t k = k0;
                for (; k + 3 < k1; k += 4) {  // four edges in flight per lane
                    int64_t e[4];
                    int32_t j[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) { j[u] = nbr[k + u]; e[u] = PERM ? (int64_t)eperm[k + u] : k + u; }
                    VT v[4], x[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const VT *vp = reinterpret_cast<const VT *>(V + e[u] * F) + c;
                        v[u] = PERM ? __ldg(vp) : ld_stream(vp);
                        x[u] = __ldg(reinterpret_cast<const VT *>(a + (int64_t)j[u] * F) + c);
                    }
                    vfma(acc0, x[0], v[0]);
                    vfma(acc1, x[1], v[1]);
                    vfma(acc0, x[2], v[2]);
                    vfma(acc1, x[3], v[3]);
                }
                for (; k < k1; k++) {
                    const int64_t e = PERM ? (int64_t)eperm[k] : k;
                    const VT *vp = reinterpret_cast<const VT *>(V + e * F) + c;
                    const VT v = PERM ? __ldg(vp) : ld_stream(vp);
                    const VT x = __ldg(reinterpret_cast<const VT *>(a + (int64_t)nbr[k] * F) + c);
                    vfma(acc0, x, v);
                }
                VT r;
                if constexpr (sizeof(T) == 4) {
                    r = make_float4(acc0.x + acc1.x, acc0.y + acc1.y, acc0.z + acc1.z, acc0.w + acc1.w);
                } else {
                    r = make_double2(acc0.x + acc1.x, acc0.y + acc1.y);
                }
                reinterpret_cast<VT *>(out + n * F)[c] = r;
            } else {
                T acc = T(0);
                for (int64_t k = k0; k < k1; k++) {
                    const int64_t e = PERM ? (int64_t)eperm[k] : k;
                    acc = fma(a[(int64_t)nbr[k] * F + c], V[e * F + c], acc);
                }
                out[n * F + c] = acc;
            }
        }
    }
}

// The float32, 128-feature case (every configuration of the model): the rows of V — the one operand that comes from HBM — are
// copied asynchronously into a ring of shared-memory slots, sixteen rows (8 KB) per warp in flight, instead of four per lane
// through registers: the kernel above is bound by the latency of those loads at the number it can keep in flight.  A lane
// copies and later reads its own 16 bytes of a row, so no synchronisation is needed beyond the copy groups.  Edge order
// and accumulation order are those of the kernel above: identical results.
constexpr int kSegSlots = 16, kSegWarps = 8;

template <bool PERM>
__global__ void __launch_bounds__(kSegWarps * 32)
seg_mul_sum_async_kernel(const float *__restrict__ a, const float *__restrict__ V, const int64_t *__restrict__ ptr, const int32_t *__restrict__ nbr,
                         const int32_t *__restrict__ eperm, int64_t N, float *__restrict__ out) {
    extern __shared__ float4 seg_ring[];       // [warps][kSegSlots][32]
    const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float4 *ring = seg_ring + (warp_in_block * kSegSlots) * 32 + lane;             // this lane's 16 bytes of slot s: ring[s * 32]
    const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
    const float4 *a4 = reinterpret_cast<const float4 *>(a) + lane, *V4 = reinterpret_cast<const float4 *>(V) + lane;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t n = warp; n < N; n += nwarps) {
        const int64_t k0 = ptr[n], k1 = ptr[n + 1];
        float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
        for (int64_t c0 = k0; c0 < k1; c0 += 32) {               // the row's edges, 32 at a time: lane t holds edge c0 + t
            const int len = (int)(k1 - c0 < 32 ? k1 - c0 : 32);
            int32_t my_j = 0;
            int64_t my_e = 0;
            if (lane < len) {
                my_j = nbr[c0 + lane];
                my_e = PERM ? (int64_t)eperm[c0 + lane] : c0 + lane;
            }
            const int ngroups = (len + 3) >> 2;
            // group g = edges 4g .. 4g+3 of the chunk -> slots (4g + u) % kSegSlots
            auto issue = [&](int g) {
                if (g < ngroups) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int t = 4 * g + u;
                        const int64_t e = __shfl_sync(0xffffffffu, my_e, t & 31);
                        if (t < len)
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_addr + (uint32_t)((t % kSegSlots) * 512)), "l"(V4 + e * 32) : "memory");
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");       // (an empty group keeps the count of pending groups fixed)
            };
#pragma unroll
            for (int g = 0; g < kSegSlots / 4; g++) issue(g);
            for (int g = 0; g < ngroups; g++) {
                float4 x[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int t = 4 * g + u;
                    const int32_t j = __shfl_sync(0xffffffffu, my_j, t & 31);
                    x[u] = t < len ? __ldg(a4 + (int64_t)j * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                asm volatile("cp.async.wait_group %0;" ::"n"(kSegSlots / 4 - 1) : "memory");
                const int full = 4 * g + 3 < len;
                if (full) {
                    const float4 v0 = ring[((4 * g) % kSegSlots) * 32], v1 = ring[((4 * g + 1) % kSegSlots) * 32];
                    const float4 v2 = ring[((4 * g + 2) % kSegSlots) * 32], v3 = ring[((4 * g + 3) % kSegSlots) * 32];
                    vfma(acc0, x[0], v0);
                    vfma(acc1, x[1], v1);
                    vfma(acc0, x[2], v2);
                    vfma(acc1, x[3], v3);
                } else {                                          // the last edges of the row, one by one into the first sum
#pragma unroll
                    for (int u = 0; u < 3; u++)
                        if (4 * g + u < len) vfma(acc0, x[u], ring[((4 * g + u) % kSegSlots) * 32]);
                }
                issue(g + kSegSlots / 4);
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        reinterpret_cast<float4 *>(out)[n * 32 + lane] = make_float4(acc0.x + acc1.x, acc0.y + acc1.y, acc0.z + acc1.z, acc0.w + acc1.w);
    }
}

// V[p,:] = a[ia[p],:] * b[ib[p],:] + a[ib[p],:] * b[ia[p],:]: the two directed edges of an unordered pair share their row of V,
// so the gradient with respect to that row is the sum of both edges' products
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
pair_mul_kernel(const T *__restrict__ a, const T *__restrict__ b, const int32_t *__restrict__ ia,
                const int32_t *__restrict__ ib, int64_t P, int64_t F, T *__restrict__ V) {
    using VT = typename VecIO<T>::V;
    constexpr int W = VEC ? VecIO<T>::W : 1;
    const int64_t Fv = F / W;
    const int64_t total = P * Fv;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = t / Fv, c = t - e * Fv;
        const int64_t i = ia[e], j = ib[e];
        if (VEC) {
            const VT ai = __ldg(reinterpret_cast<const VT *>(a + i * F) + c), bj = __ldg(reinterpret_cast<const VT *>(b + j * F) + c);
            const VT aj = __ldg(reinterpret_cast<const VT *>(a + j * F) + c), bi = __ldg(reinterpret_cast<const VT *>(b + i * F) + c);
            VT acc = vmul(ai, bj);
            vfma(acc, aj, bi);
            st_stream(reinterpret_cast<VT *>(V + e * F) + c, acc);
        } else {
            V[e * F + c] = fma(a[j * F + c], b[i * F + c], a[i * F + c] * b[j * F + c]);
        }
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
edge_mul_kernel(const T *__restrict__ a, const T *__restrict__ b, const int32_t *__restrict__ ia,
                const int32_t *__restrict__ ib, int64_t E, int64_t F, T *__restrict__ V) {
    using VT = typename VecIO<T>::V;
    constexpr int W = VEC ? VecIO<T>::W : 1;
    const int64_t Fv = F / W;
    const int64_t total = E * Fv;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = t / Fv, c = t - e * Fv;
        if (VEC) {
            const VT x = __ldg(reinterpret_cast<const VT *>(a + (int64_t)ia[e] * F) + c);
            const VT y = __ldg(reinterpret_cast<const VT *>(b + (int64_t)ib[e] * F) + c);
            st_stream(reinterpret_cast<VT *>(V + e * F) + c, vmul(x, y));
        } else {
            V[e * F + c] = a[(int64_t)ia[e] * F + c] * b[(int64_t)ib[e] * F + c];
        }
    }
}

// --------------------------------------------------------------------------------- edge geometry
template <typename T>
__global__ void edge_diff_kernel(const T *__restrict__ pos, const int32_t *__restrict__ row0,
                                 const int32_t *__restrict__ row1, int64_t E, int64_t N, T *__restrict__ dr,
                                 int32_t *__restrict__ status) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t a = row0[e], b = row1[e];
        if (a < 0 || a >= N || b < 0 || b >= N) {
            atomicOr(status, (int)kBadIndex);
            dr[e * 3] = dr[e * 3 + 1] = dr[e * 3 + 2] = T(0);
            continue;
        }
#pragma unroll
        for (int c = 0; c < 3; c++) dr[e * 3 + c] = pos[b * 3 + c] - pos[a * 3 + c];
    }
}

// one warp per node; lanes stride over the node's edges, fixed-shape shuffle reduction
template <typename T>
__global__ void __launch_bounds__(256)
node_scatter_diff_kernel(const T *__restrict__ g, const int64_t *__restrict__ ptr_in, const int32_t *__restrict__ perm_in,
                         const int64_t *__restrict__ ptr_out, const int32_t *__restrict__ perm_out, int64_t N,
                         T *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t n = warp; n < N; n += nwarps) {
        T s0 = T(0), s1 = T(0), s2 = T(0);
        for (int64_t k = ptr_in[n] + lane; k < ptr_in[n + 1]; k += 32) {
            const int64_t e = perm_in ? (int64_t)perm_in[k] : k;
            s0 += g[e * 3]; s1 += g[e * 3 + 1]; s2 += g[e * 3 + 2];
        }
        for (int64_t k = ptr_out[n] + lane; k < ptr_out[n + 1]; k += 32) {
            const int64_t e = perm_out ? (int64_t)perm_out[k] : k;
            s0 -= g[e * 3]; s1 -= g[e * 3 + 1]; s2 -= g[e * 3 + 2];
        }
        s0 = warp_sum(s0); s1 = warp_sum(s1); s2 = warp_sum(s2);
        if (lane == 0) { out[n * 3] = s0; out[n * 3 + 1] = s1; out[n * 3 + 2] = s2; }
    }
}


// d[e] = |pos[row1] - pos[row0]|  (compute_distances, internal_coordinates.py:72-100, in one kernel)
template <typename T>
__global__ void edge_distance_kernel(const T *__restrict__ pos, const int32_t *__restrict__ row0,
                                     const int32_t *__restrict__ row1, int64_t E, int64_t N, T *__restrict__ d,
                                     int32_t *__restrict__ status) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t a = row0[e], b = row1[e];
        if (a < 0 || a >= N || b < 0 || b >= N) {
            atomicOr(status, (int)kBadIndex);
            d[e] = T(0);
            continue;
        }
        const T dx = pos[b * 3] - pos[a * 3], dy = pos[b * 3 + 1] - pos[a * 3 + 1], dz = pos[b * 3 + 2] - pos[a * 3 + 2];
        d[e] = sqrt(dx * dx + dy * dy + dz * dz);
    }
}

// gpos[n] = sum_{e: row1(e)=n} (g_e/d_e) dr_e - sum_{e: row0(e)=n} (g_e/d_e) dr_e,  dr_e = pos[row1] - pos[row0]
// one warp per node, ordered, no atomics
template <typename T>
__global__ void __launch_bounds__(256)
edge_distance_bwd_kernel(const T *__restrict__ pos, const T *__restrict__ g, const T *__restrict__ d,
                         const int32_t *__restrict__ row0, const int32_t *__restrict__ row1,
                         const int64_t *__restrict__ ptr_in, const int32_t *__restrict__ perm_in,
                         const int64_t *__restrict__ ptr_out, const int32_t *__restrict__ perm_out, int64_t N,
                         T *__restrict__ gpos) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t n = warp; n < N; n += nwarps) {
        T s0 = T(0), s1 = T(0), s2 = T(0);
        for (int pass = 0; pass < 2; pass++) {
            const int64_t *ptr = pass ? ptr_out : ptr_in;
            const int32_t *perm = pass ? perm_out : perm_in;
            const T sign = pass ? T(-1) : T(1);
            for (int64_t k = ptr[n] + lane; k < ptr[n + 1]; k += 32) {
                const int64_t e = perm ? (int64_t)perm[k] : k;
                const int64_t a = row0[e], b = row1[e];
                const T w = sign * g[e] / d[e];
                s0 = fma(w, pos[b * 3] - pos[a * 3], s0);
                s1 = fma(w, pos[b * 3 + 1] - pos[a * 3 + 1], s1);
                s2 = fma(w, pos[b * 3 + 2] - pos[a * 3 + 2], s2);
            }
        }
        s0 = warp_sum(s0); s1 = warp_sum(s1); s2 = warp_sum(s2);
        if (lane == 0) { gpos[n * 3] = s0; gpos[n * 3 + 1] = s1; gpos[n * 3 + 2] = s2; }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
segment_sum_kernel(const T *__restrict__ x, const int64_t *__restrict__ ptr, int64_t B, T *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp; b < B; b += nwarps) {
        T s = T(0);
        for (int64_t k = ptr[b] + lane; k < ptr[b + 1]; k += 32) s += x[k];
        s = warp_sum(s);
        if (lane == 0) out[b] = s;
    }
}

// ---------------------------------------------------------------------------- per-edge scalar times edge row
// out[e,:] = a[e,:] * c[e]   (W = net(rbf) * C[:,None], schnet.py:341, and every derivative of that product)
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
row_scale_kernel(const T *__restrict__ a, const T *__restrict__ c, int64_t E, int64_t F, T *__restrict__ out) {
    using VT = typename VecIO<T>::V;
    constexpr int W = VEC ? VecIO<T>::W : 1;
    const int64_t Fv = F / W, total = E * Fv;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = t / Fv;
        const T s = c[e];
        if (VEC) {
            VT v = ld_stream(reinterpret_cast<const VT *>(a) + t);
            if constexpr (sizeof(T) == 4) v = make_float4(v.x * s, v.y * s, v.z * s, v.w * s);
            else v = make_double2(v.x * s, v.y * s);
            reinterpret_cast<VT *>(out)[t] = v;
        } else {
            out[t] = a[t] * s;
        }
    }
}

// The derivative of tanh given its output, and the derivative of that (the activation of the filter network and of the
// interaction blocks, src/mlcg/nn/schnet.py:252-262, 446-450, differentiated once for the forces and again for force matching):
//   MODE 0: out = g (1 - y^2)          MODE 1: out = -2 G g y
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
tanh_grad_kernel(const T *__restrict__ G, const T *__restrict__ g, const T *__restrict__ y, int64_t n, T *__restrict__ out) {
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
        const T yy = y[t], gg = g[t];
        out[t] = MODE == 0 ? gg * (T(1) - yy * yy) : T(-2) * G[t] * gg * yy;
    }
}
template <int MODE>
__global__ void __launch_bounds__(256)
tanh_grad_vec_kernel(const float4 *__restrict__ G, const float4 *__restrict__ g, const float4 *__restrict__ y, int64_t n4, float4 *__restrict__ out) {
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n4; t += (int64_t)gridDim.x * blockDim.x) {
        const float4 yy = ld_stream(y + t), gg = ld_stream(g + t);
        float4 o;
        if (MODE == 0) {
            o = make_float4(gg.x * fmaf(-yy.x, yy.x, 1.f), gg.y * fmaf(-yy.y, yy.y, 1.f), gg.z * fmaf(-yy.z, yy.z, 1.f), gg.w * fmaf(-yy.w, yy.w, 1.f));
        } else {
            const float4 GG = ld_stream(G + t);
            o = make_float4(-2.f * GG.x * gg.x * yy.x, -2.f * GG.y * gg.y * yy.y, -2.f * GG.z * gg.z * yy.z, -2.f * GG.w * gg.w * yy.w);
        }
        out[t] = o;
    }
}

// out[e] = sum_f a[e,f] * b[e,f]: one warp per row, fixed-shape shuffle reduction
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
row_dot_kernel(const T *__restrict__ a, const T *__restrict__ b, int64_t E, int64_t F, T *__restrict__ out) {
    using VT = typename VecIO<T>::V;
    constexpr int W = VEC ? VecIO<T>::W : 1;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t Fv = F / W;
    for (int64_t e = warp; e < E; e += nwarps) {
        T s = T(0);
        for (int64_t k = lane; k < Fv; k += 32) {
            if (VEC) {
                const VT x = ld_stream(reinterpret_cast<const VT *>(a + e * F) + k), y = ld_stream(reinterpret_cast<const VT *>(b + e * F) + k);
                if constexpr (sizeof(T) == 4) s = fmaf(x.w, y.w, fmaf(x.z, y.z, fmaf(x.y, y.y, fmaf(x.x, y.x, s))));
                else s = fma(x.y, y.y, fma(x.x, y.x, s));
            } else {
                s = fma(a[e * F + k], b[e * F + k], s);
            }
        }
        s = warp_sum(s);
        if (lane == 0) out[e] = s;
    }
}

template <typename T>
static int seg_mul_sum_launch(const void *a, const void *V, const int64_t *ptr, const int32_t *nbr, const int32_t *eperm,
                              int64_t N, int64_t F, void *out, cudaStream_t st) {
    constexpr int W = VecIO<T>::W;
    const bool vec = (F % W == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)V % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const int64_t Fv = vec ? F / W : F;
    if constexpr (sizeof(T) == 4) {
        if (vec && F == 128) {
            constexpr int kSmem = kSegWarps * kSegSlots * 512;
            static bool done[64] = {false};
            int dev = 0;
            cudaGetDevice(&dev);
            if (dev >= 0 && dev < 64 && !done[dev]) {
                if (cudaFuncSetAttribute(seg_mul_sum_async_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess ||
                    cudaFuncSetAttribute(seg_mul_sum_async_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
                    return check_launch();
                done[dev] = true;
            }
            const int64_t want = (N + kSegWarps - 1) / kSegWarps;
            const int grid = (int)(want < (int64_t)kNumSM * 3 ? want : (int64_t)kNumSM * 3);      // three blocks of 64 KB per SM
            if (eperm) seg_mul_sum_async_kernel<true><<<grid, kSegWarps * 32, kSmem, st>>>((const float *)a, (const float *)V, ptr, nbr, eperm, N, (float *)out);
            else seg_mul_sum_async_kernel<false><<<grid, kSegWarps * 32, kSmem, st>>>((const float *)a, (const float *)V, ptr, nbr, eperm, N, (float *)out);
            return check_launch();
        }
    }
    int G = 32;
    while (G > 1 && G / 2 >= Fv) G /= 2;  // smallest power of two >= Fv, capped at a warp
    const int grid = grid_for(N * G, 256, 16);
#define LAUNCH2(GG, VV)                                                                                                              \
    if (eperm) seg_mul_sum_kernel<T, GG, VV, true><<<grid, 256, 0, st>>>((const T *)a, (const T *)V, ptr, nbr, eperm, N, F, (T *)out);  \
    else seg_mul_sum_kernel<T, GG, VV, false><<<grid, 256, 0, st>>>((const T *)a, (const T *)V, ptr, nbr, eperm, N, F, (T *)out)
#define LAUNCH(GG)                \
    if (vec) { LAUNCH2(GG, true); } \
    else { LAUNCH2(GG, false); }
    switch (G) {
        case 32: LAUNCH(32); break;
        case 16: LAUNCH(16); break;
        case 8: LAUNCH(8); break;
        case 4: LAUNCH(4); break;
        case 2: LAUNCH(2); break;
        default: LAUNCH(1); break;
    }
#undef LAUNCH
#undef LAUNCH2
    return check_launch();
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

int mlcgb_seg_mul_sum(const void *a, const void *V, int dtype, const int64_t *ptr, const int32_t *nbr, const int32_t *eperm,
                      int64_t N, int64_t E, int64_t F, void *out, void *stream) {
    TimelineScope timeline_scope("seg_mul_sum", stream);
    if (N < 0 || E < 0 || F <= 0) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!ptr || !out || (E > 0 && (!a || !V || !nbr))) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] { return seg_mul_sum_launch<scalar_t>(a, V, ptr, nbr, eperm, N, F, out, (cudaStream_t)stream); });
}

int mlcgb_edge_mul(const void *a, const void *b, int dtype, const int32_t *ia, const int32_t *ib, int64_t E, int64_t F, void *V,
                   void *stream) {
    TimelineScope timeline_scope("edge_mul", stream);
    if (E < 0 || F <= 0) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!a || !b || !ia || !ib || !V) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        constexpr int W = VecIO<scalar_t>::W;
        const bool vec = (F % W == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)V % 16 == 0);
        const int64_t work = E * (vec ? F / W : F);
        const int grid = grid_for(work, 256, 32);
        if (vec) edge_mul_kernel<scalar_t, true><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)b, ia, ib, E, F, (scalar_t *)V);
        else edge_mul_kernel<scalar_t, false><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)b, ia, ib, E, F, (scalar_t *)V);
        return check_launch();
    });
}

int mlcgb_pair_mul(const void *a, const void *b, int dtype, const int32_t *ia, const int32_t *ib, int64_t P, int64_t F, void *V,
                   void *stream) {
    TimelineScope timeline_scope("pair_mul", stream);
    if (P < 0 || F <= 0) return MLCGB_E_ARG;
    if (P == 0) return MLCGB_OK;
    if (!a || !b || !ia || !ib || !V) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        constexpr int W = VecIO<scalar_t>::W;
        const bool vec = (F % W == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)V % 16 == 0);
        const int64_t work = P * (vec ? F / W : F);
        const int grid = grid_for(work, 256, 32);
        if (vec) pair_mul_kernel<scalar_t, true><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)b, ia, ib, P, F, (scalar_t *)V);
        else pair_mul_kernel<scalar_t, false><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)b, ia, ib, P, F, (scalar_t *)V);
        return check_launch();
    });
}

int mlcgb_edge_diff(const void *pos, int dtype, const int32_t *row0, const int32_t *row1, int64_t E, int64_t N, void *dr,
                    int32_t *status, void *stream) {
    TimelineScope timeline_scope("edge_diff", stream);
    if (E < 0 || N < 0 || !status) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!pos || !row0 || !row1 || !dr) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        edge_diff_kernel<scalar_t><<<grid_for(E, 256), 256, 0, (cudaStream_t)stream>>>((const scalar_t *)pos, row0, row1, E, N, (scalar_t *)dr, status);
        return check_launch();
    });
}

int mlcgb_node_scatter_diff(const void *g, int dtype, const int64_t *ptr_in, const int32_t *perm_in, const int64_t *ptr_out,
                            const int32_t *perm_out, int64_t N, int64_t E, void *out, void *stream) {
    TimelineScope timeline_scope("node_scatter_diff", stream);
    if (N < 0 || E < 0) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!ptr_in || !ptr_out || !out || (E > 0 && !g)) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        node_scatter_diff_kernel<scalar_t><<<grid_for(N * 32, 256), 256, 0, (cudaStream_t)stream>>>((const scalar_t *)g, ptr_in, perm_in, ptr_out, perm_out, N, (scalar_t *)out);
        return check_launch();
    });
}

int mlcgb_segment_sum(const void *x, int dtype, const int64_t *ptr, int64_t B, void *out, void *stream) {
    TimelineScope timeline_scope("segment_sum", stream);
    if (B < 0) return MLCGB_E_ARG;
    if (B == 0) return MLCGB_OK;
    if (!x || !ptr || !out) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        segment_sum_kernel<scalar_t><<<grid_for(B * 32, 256), 256, 0, (cudaStream_t)stream>>>((const scalar_t *)x, ptr, B, (scalar_t *)out);
        return check_launch();
    });
}

int mlcgb_row_scale(const void *a, const void *c, int dtype, int64_t E, int64_t F, void *out, void *stream) {
    TimelineScope timeline_scope("row_scale", stream);
    if (E < 0 || F <= 0) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!a || !c || !out) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        constexpr int W = VecIO<scalar_t>::W;
        const bool vec = (F % W == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)out % 16 == 0);
        const int grid = grid_for(E * (vec ? F / W : F), 256, 32);
        if (vec) row_scale_kernel<scalar_t, true><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)c, E, F, (scalar_t *)out);
        else row_scale_kernel<scalar_t, false><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)c, E, F, (scalar_t *)out);
        return check_launch();
    });
}

int mlcgb_tanh_grad(int mode, const void *G, const void *g, const void *y, int dtype, int64_t n, void *out, void *stream) {
    TimelineScope timeline_scope("tanh_grad", stream);
    if (n < 0 || (mode != 0 && mode != 1)) return MLCGB_E_ARG;
    if (n == 0) return MLCGB_OK;
    if (!g || !y || !out || (mode == 1 && !G)) return MLCGB_E_ARG;
    auto st = (cudaStream_t)stream;
    if (dtype == MLCGB_F32 && (n & 3) == 0 && (((uintptr_t)g | (uintptr_t)y | (uintptr_t)out | (uintptr_t)G) & 15) == 0) {
        const int grid = grid_for(n / 4, 256, 32);
        if (mode == 0) tanh_grad_vec_kernel<0><<<grid, 256, 0, st>>>((const float4 *)G, (const float4 *)g, (const float4 *)y, n / 4, (float4 *)out);
        else tanh_grad_vec_kernel<1><<<grid, 256, 0, st>>>((const float4 *)G, (const float4 *)g, (const float4 *)y, n / 4, (float4 *)out);
        return check_launch();
    }
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        const int grid = grid_for(n, 256, 32);
        if (mode == 0) tanh_grad_kernel<scalar_t, 0><<<grid, 256, 0, st>>>((const scalar_t *)G, (const scalar_t *)g, (const scalar_t *)y, n, (scalar_t *)out);
        else tanh_grad_kernel<scalar_t, 1><<<grid, 256, 0, st>>>((const scalar_t *)G, (const scalar_t *)g, (const scalar_t *)y, n, (scalar_t *)out);
        return check_launch();
    });
}

int mlcgb_row_dot(const void *a, const void *b, int dtype, int64_t E, int64_t F, void *out, void *stream) {
    TimelineScope timeline_scope("row_dot", stream);
    if (E < 0 || F <= 0) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!a || !b || !out) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        constexpr int W = VecIO<scalar_t>::W;
        const bool vec = (F % W == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0);
        const int grid = grid_for(E * 32, 256, 32);
        if (vec) row_dot_kernel<scalar_t, true><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)b, E, F, (scalar_t *)out);
        else row_dot_kernel<scalar_t, false><<<grid, 256, 0, (cudaStream_t)stream>>>((const scalar_t *)a, (const scalar_t *)b, E, F, (scalar_t *)out);
        return check_launch();
    });
}

int mlcgb_edge_distance(const void *pos, int dtype, const int32_t *row0, const int32_t *row1, int64_t E, int64_t N, void *d,
                        int32_t *status, void *stream) {
    TimelineScope timeline_scope("edge_distance", stream);
    if (E < 0 || N < 0 || !status) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!pos || !row0 || !row1 || !d) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        edge_distance_kernel<scalar_t><<<grid_for(E, 256), 256, 0, (cudaStream_t)stream>>>((const scalar_t *)pos, row0, row1, E, N, (scalar_t *)d, status);
        return check_launch();
    });
}

int mlcgb_edge_distance_backward(const void *pos, const void *g, const void *d, int dtype, const int32_t *row0, const int32_t *row1,
                                 const int64_t *ptr_in, const int32_t *perm_in, const int64_t *ptr_out, const int32_t *perm_out,
                                 int64_t N, int64_t E, void *gpos, void *stream) {
    TimelineScope timeline_scope("edge_distance_backward", stream);
    if (N < 0 || E < 0) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!ptr_in || !ptr_out || !gpos || (E > 0 && (!pos || !g || !d || !row0 || !row1))) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        edge_distance_bwd_kernel<scalar_t><<<grid_for(N * 32, 256), 256, 0, (cudaStream_t)stream>>>(
            (const scalar_t *)pos, (const scalar_t *)g, (const scalar_t *)d, row0, row1, ptr_in, perm_in, ptr_out, perm_out, N, (scalar_t *)gpos);
        return check_launch();
    });
}

}  // extern "C"
