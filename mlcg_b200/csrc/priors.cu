// Classical prior terms (bonds, angles, dihedrals, repulsion): energy per structure and dE/dpos in
// one pass over the static index lists.  One thread per term; the term's energy is reduced inside
// the warp when all 32 terms belong to the same structure (the common case, lists are ordered by
// structure), gradients go out as floating-point atomics.
#include "common.cuh"

namespace mlcgb {

template <typename T> struct V3 { T x, y, z; };
template <typename T> __device__ __forceinline__ V3<T> ld3(const T *p, int64_t i) { return V3<T>{p[i * 3], p[i * 3 + 1], p[i * 3 + 2]}; }
template <typename T> __device__ __forceinline__ V3<T> sub(const V3<T> &a, const V3<T> &b) { return V3<T>{a.x - b.x, a.y - b.y, a.z - b.z}; }
template <typename T> __device__ __forceinline__ T dot(const V3<T> &a, const V3<T> &b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
template <typename T> __device__ __forceinline__ V3<T> cross(const V3<T> &a, const V3<T> &b) {
    return V3<T>{a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x};
}
template <typename T> __device__ __forceinline__ V3<T> scale(const V3<T> &a, T s) { return V3<T>{a.x * s, a.y * s, a.z * s}; }
template <typename T> __device__ __forceinline__ V3<T> axpy(T s, const V3<T> &a, const V3<T> &b) { return V3<T>{s * a.x + b.x, s * a.y + b.y, s * a.z + b.z}; }
template <typename T> __device__ __forceinline__ void atomic_add3(T *g, int64_t i, const V3<T> &v) {
    atomicAdd(g + i * 3, v.x);
    atomicAdd(g + i * 3 + 1, v.y);
    atomicAdd(g + i * 3 + 2, v.z);
}

// Adds v into g[i] with one atomic per run of consecutive lanes that share the same index i (pair lists are
// usually grouped by their first index, so a warp holds one or two runs).  Every lane of the warp must call this;
// lanes without a contribution pass i = -1.
template <typename T>
__device__ __forceinline__ void run_add3(T *g, int64_t i, V3<T> v, int lane) {
    const int64_t prev = __shfl_up_sync(0xffffffffu, i, 1);
    const bool head = lane == 0 || prev != i;
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    // end of this lane's run = position of the next head above it
    const unsigned above = lane == 31 ? 0u : (heads >> (lane + 1));
    const int run_end = above ? lane + __ffs(above) : 32;   // exclusive
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T x = __shfl_down_sync(0xffffffffu, v.x, o), y = __shfl_down_sync(0xffffffffu, v.y, o), z = __shfl_down_sync(0xffffffffu, v.z, o);
        if (lane + o < run_end) { v.x += x; v.y += y; v.z += z; }
    }
    if (head && i >= 0) atomic_add3(g, i, v);
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256)
prior_kernel(const T *__restrict__ pos, const int64_t *__restrict__ mapping, const int64_t *__restrict__ mapping_batch,
             const T *__restrict__ params, int n_params, int64_t M, int64_t N, int64_t B, T *__restrict__ energy,
             T *__restrict__ grad, int32_t *__restrict__ status) {
    constexpr int ORDER = KIND == 0 || KIND == 3 ? 2 : (KIND == 1 ? 3 : 4);
    const int lane = threadIdx.x & 31;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x - lane;  // warp-uniform base
    for (int64_t base = first; base < M; base += stride) {
        const int64_t t = base + lane;
        bool valid = t < M;
        int64_t idx[ORDER];
        int64_t mb = 0;
        if (valid) {
#pragma unroll
            for (int o = 0; o < ORDER; o++) {
                idx[o] = mapping[(int64_t)o * M + t];
                if (idx[o] < 0 || idx[o] >= N) valid = false;
            }
            mb = mapping_batch[t];
            if (mb < 0 || mb >= B) valid = false;
            if (!valid) atomicOr(status, (int)kBadIndex);
        }
        T e = T(0);
        V3<T> g0{T(0), T(0), T(0)};   // pair terms: gradient on the first index, reduced over runs below
        if (valid) {
            if (KIND == 0 || KIND == 3) {
                const V3<T> dr = sub(ld3(pos, idx[1]), ld3(pos, idx[0]));
                const T d = sqrt(dot(dr, dr));
                T dEdd;
                if (KIND == 0) {
                    const T x0 = params[t], k = params[M + t];
                    e = k * (d - x0) * (d - x0);
                    dEdd = T(2) * k * (d - x0);
                } else {
                    const T q = params[t] / d;
                    const T rr = q * q;
                    e = rr * rr * rr;
                    dEdd = T(-6) * e / d;
                }
                if (grad) {
                    const V3<T> g1 = scale(dr, dEdd / d);
                    atomic_add3(grad, idx[1], g1);
                    g0 = scale(g1, T(-1));
                }
            } else if (KIND == 1) {
                const V3<T> p1 = ld3(pos, idx[1]);
                const V3<T> a = sub(ld3(pos, idx[0]), p1), b = sub(ld3(pos, idx[2]), p1);
                const T na = sqrt(dot(a, a)), nb = sqrt(dot(b, b));
                const T c = dot(a, b) / na / nb;
                const T x0 = params[t], k = params[M + t];
                e = k * (c - x0) * (c - x0);
                if (grad) {
                    const T dEdc = T(2) * k * (c - x0);
                    const T inv = T(1) / (na * nb);
                    const V3<T> ga = scale(axpy(-c / (na * na), a, scale(b, inv)), dEdc);
                    const V3<T> gb = scale(axpy(-c / (nb * nb), b, scale(a, inv)), dEdc);
                    atomic_add3(grad, idx[0], ga);
                    atomic_add3(grad, idx[2], gb);
                    atomic_add3(grad, idx[1], V3<T>{-ga.x - gb.x, -ga.y - gb.y, -ga.z - gb.z});
                }
            } else {
                const V3<T> p0 = ld3(pos, idx[0]), p1 = ld3(pos, idx[1]), p2 = ld3(pos, idx[2]), p3 = ld3(pos, idx[3]);
                // angle exactly as compute_torsions builds it (unit bond vectors, atan2(-m.n2, n1.n2))
                V3<T> b1 = sub(p1, p0), b2 = sub(p2, p1), b3 = sub(p3, p2);
                const V3<T> u1 = scale(b1, T(1) / sqrt(dot(b1, b1)));
                const V3<T> u2 = scale(b2, T(1) / sqrt(dot(b2, b2)));
                const V3<T> u3 = scale(b3, T(1) / sqrt(dot(b3, b3)));
                const V3<T> n1 = cross(u1, u2), n2 = cross(u2, u3), m1 = cross(n1, u2);
                const T theta = atan2(-dot(m1, n2), dot(n1, n2));
                const int n_degs = (n_params - 1) / 2;
                e = params[t];
                T dEdth = T(0);
                for (int n = 1; n <= n_degs; n++) {
                    T sn, cs;
                    sincos(T(n) * theta, &sn, &cs);
                    const T k1 = params[(int64_t)n * M + t], k2 = params[(int64_t)(n_degs + n) * M + t];
                    e += k1 * sn + k2 * cs;
                    dEdth += T(n) * (k1 * cs - k2 * sn);
                }
                if (grad) {
                    // d(theta)/d(positions): F = p0-p1, G = p1-p2, H = p3-p2, A = F x G, B = H x G
                    const V3<T> F = sub(p0, p1), G = sub(p1, p2), H = sub(p3, p2);
                    const V3<T> A = cross(F, G), Bv = cross(H, G);
                    const T A2 = dot(A, A), B2 = dot(Bv, Bv), Gn = sqrt(dot(G, G));
                    const T fg = dot(F, G) / (A2 * Gn), hg = dot(H, G) / (B2 * Gn);
                    const V3<T> d0 = scale(A, -Gn / A2);
                    const V3<T> d3 = scale(Bv, Gn / B2);
                    const V3<T> d1 = axpy(-hg, Bv, scale(A, Gn / A2 + fg));
                    const V3<T> d2 = axpy(hg, Bv, axpy(-fg, A, scale(Bv, -Gn / B2)));
                    atomic_add3(grad, idx[0], scale(d0, dEdth));
                    atomic_add3(grad, idx[1], scale(d1, dEdth));
                    atomic_add3(grad, idx[2], scale(d2, dEdth));
                    atomic_add3(grad, idx[3], scale(d3, dEdth));
                }
            }
        }
        if ((KIND == 0 || KIND == 3) && grad) run_add3(grad, valid ? idx[0] : (int64_t)-1, g0, lane);
        // energy: one atomic per warp when the whole warp sits in one structure
        const int64_t mb0 = __shfl_sync(0xffffffffu, mb, 0);
        const bool same = __all_sync(0xffffffffu, !valid || mb == mb0);
        const bool lane0_valid = __shfl_sync(0xffffffffu, (int)valid, 0) != 0;
        if (same && lane0_valid) {
            const T s = warp_sum(e);
            if (lane == 0) atomicAdd(energy + mb0, s);
        } else if (valid) {
            atomicAdd(energy + mb, e);
        }
    }
}

template <typename T>
static int prior_launch(int kind, const void *pos, const int64_t *mapping, const int64_t *mapping_batch, const void *params,
                        int n_params, int64_t M, int64_t N, int64_t B, void *energy, void *grad, int32_t *status,
                        cudaStream_t st) {
    const int grid = grid_for(M, 256, 16);
#define GO(K) prior_kernel<T, K><<<grid, 256, 0, st>>>((const T *)pos, mapping, mapping_batch, (const T *)params, n_params, M, N, B, (T *)energy, (T *)grad, status)
    switch (kind) {
        case 0: GO(0); break;
        case 1: GO(1); break;
        case 2: GO(2); break;
        default: GO(3); break;
    }
#undef GO
    return check_launch();
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" int mlcgb_prior_terms(int kind, const void *pos, int dtype, const int64_t *mapping, const int64_t *mapping_batch,
                                 const void *params, int n_params, int64_t M, int64_t N, int64_t B, void *energy, void *grad,
                                 int32_t *status, void *stream) {
    TimelineScope timeline_scope("prior_terms", stream);
    if (kind < 0 || kind > 3 || M < 0 || N < 0 || B < 0 || !status) return MLCGB_E_ARG;
    if (M == 0) return MLCGB_OK;
    if (!pos || !mapping || !mapping_batch || !params || !energy) return MLCGB_E_ARG;
    const int need = kind == 3 ? 1 : (kind == 2 ? 3 : 2);
    if (n_params < need || (kind == 2 && (n_params - 1) % 2 != 0)) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        return prior_launch<scalar_t>(kind, pos, mapping, mapping_batch, params, n_params, M, N, B, energy, grad, status,
                                      (cudaStream_t)stream);
    });
}
