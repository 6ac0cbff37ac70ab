// Classical prior terms (bonds, angles, dihedrals, repulsion): energy per structure and dE/dpos in
// one pass over the static index lists.  One thread per term; the term's energy is reduced inside
// the warp when all 32 terms belong to the same structure (the common case, lists are ordered by
// structure), gradients go out as floating-point atomics.
#include "common.cuh"

#include <type_traits>

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

// Bonds, angles and dihedrals are evaluated in double precision whatever the storage type: their lists are short (one term
// per bead, where a repulsion list has hundreds), and in float32 a harmonic bond loses most of its digits in d - x0 and a
// torsion gradient in the cross products of nearly collinear bonds.  Positions and parameters are read as stored; energy and
// gradient are rounded to the storage type once, at the end.
template <typename T> __device__ __forceinline__ V3<double> ld3d(const T *p, int64_t i) {
    return V3<double>{(double)p[i * 3], (double)p[i * 3 + 1], (double)p[i * 3 + 2]};
}
template <typename T> __device__ __forceinline__ V3<T> narrow(const V3<double> &a) { return V3<T>{(T)a.x, (T)a.y, (T)a.z}; }

// harmonic bond k (d - x0)^2: energy; g1 = dE/dpos[i1] (dE/dpos[i0] = -g1)
template <typename T>
__device__ __forceinline__ double bond_term(const T *pos, int64_t i0, int64_t i1, double x0, double k, V3<double> &g1) {
    const V3<double> dr = sub(ld3d(pos, i1), ld3d(pos, i0));
    const double d = sqrt(dot(dr, dr));
    g1 = scale(dr, 2.0 * k * (d - x0) / d);
    return k * (d - x0) * (d - x0);
}

// harmonic angle in the cosine, k (cos - x0)^2: ga = dE/dpos[i0], gb = dE/dpos[i2] (dE/dpos[i1] = -ga - gb)
template <typename T>
__device__ __forceinline__ double angle_term(const T *pos, int64_t i0, int64_t i1, int64_t i2, double x0, double k, V3<double> &ga, V3<double> &gb) {
    const V3<double> p1 = ld3d(pos, i1);
    const V3<double> a = sub(ld3d(pos, i0), p1), b = sub(ld3d(pos, i2), p1);
    const double na = sqrt(dot(a, a)), nb = sqrt(dot(b, b));
    const double c = dot(a, b) / na / nb;
    const double dEdc = 2.0 * k * (c - x0);
    const double inv = 1.0 / (na * nb);
    ga = scale(axpy(-c / (na * na), a, scale(b, inv)), dEdc);
    gb = scale(axpy(-c / (nb * nb), b, scale(a, inv)), dEdc);
    return k * (c - x0) * (c - x0);
}

// Fourier series in the torsion angle, built as compute_torsions builds it (unit bond vectors, atan2(-m.n2, n1.n2)):
// params rows v0, k1_1..k1_n, k2_1..k2_n with stride M; g[0..3] = dE/dpos of the four beads
template <typename T>
__device__ __forceinline__ double torsion_term(const T *pos, int64_t i0, int64_t i1, int64_t i2, int64_t i3, const T *params, int64_t M,
                                               int64_t t, int n_degs, V3<double> (&g)[4]) {
    const V3<double> p0 = ld3d(pos, i0), p1 = ld3d(pos, i1), p2 = ld3d(pos, i2), p3 = ld3d(pos, i3);
    const V3<double> b1 = sub(p1, p0), b2 = sub(p2, p1), b3 = sub(p3, p2);
    const V3<double> u1 = scale(b1, 1.0 / sqrt(dot(b1, b1)));
    const V3<double> u2 = scale(b2, 1.0 / sqrt(dot(b2, b2)));
    const V3<double> u3 = scale(b3, 1.0 / sqrt(dot(b3, b3)));
    const V3<double> n1 = cross(u1, u2), n2 = cross(u2, u3), m1 = cross(n1, u2);
    const double theta = atan2(-dot(m1, n2), dot(n1, n2));
    double e = (double)params[t], dEdth = 0.0;
    for (int n = 1; n <= n_degs; n++) {
        double sn, cs;
        sincos((double)n * theta, &sn, &cs);
        const double k1 = (double)params[(int64_t)n * M + t], k2 = (double)params[(int64_t)(n_degs + n) * M + t];
        e += k1 * sn + k2 * cs;
        dEdth += (double)n * (k1 * cs - k2 * sn);
    }
    // d(theta)/d(positions): F = p0-p1, G = p1-p2, H = p3-p2, A = F x G, B = H x G
    const V3<double> F = sub(p0, p1), G = sub(p1, p2), H = sub(p3, p2);
    const V3<double> A = cross(F, G), Bv = cross(H, G);
    const double A2 = dot(A, A), B2 = dot(Bv, Bv), Gn = sqrt(dot(G, G));
    const double fg = dot(F, G) / (A2 * Gn), hg = dot(H, G) / (B2 * Gn);
    g[0] = scale(scale(A, -Gn / A2), dEdth);
    g[3] = scale(scale(Bv, Gn / B2), dEdth);
    g[1] = scale(axpy(-hg, Bv, scale(A, Gn / A2 + fg)), dEdth);
    g[2] = scale(axpy(hg, Bv, axpy(-fg, A, scale(Bv, -Gn / B2))), dEdth);
    return e;
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
            if (KIND == 0) {
                V3<double> g1;
                e = (T)bond_term(pos, idx[0], idx[1], (double)params[t], (double)params[M + t], g1);
                if (grad) {
                    atomic_add3(grad, idx[1], narrow<T>(g1));
                    g0 = narrow<T>(scale(g1, -1.0));
                }
            } else if (KIND == 3) {
                const V3<T> dr = sub(ld3(pos, idx[1]), ld3(pos, idx[0]));
                const T d = sqrt(dot(dr, dr));
                const T q = params[t] / d;
                const T rr = q * q;
                e = rr * rr * rr;
                if (grad) {
                    const V3<T> g1 = scale(dr, T(-6) * e / d / d);
                    atomic_add3(grad, idx[1], g1);
                    g0 = scale(g1, T(-1));
                }
            } else if (KIND == 1) {
                V3<double> ga, gb;
                e = (T)angle_term(pos, idx[0], idx[1], idx[2], (double)params[t], (double)params[M + t], ga, gb);
                if (grad) {
                    atomic_add3(grad, idx[0], narrow<T>(ga));
                    atomic_add3(grad, idx[2], narrow<T>(gb));
                    atomic_add3(grad, idx[1], narrow<T>(V3<double>{-ga.x - gb.x, -ga.y - gb.y, -ga.z - gb.z}));
                }
            } else {
                V3<double> g[4];
                e = (T)torsion_term(pos, idx[0], idx[1], idx[2], idx[3], params, M, t, (n_params - 1) / 2, g);
                if (grad) {
#pragma unroll
                    for (int o = 0; o < 4; o++) atomic_add3(grad, idx[o], narrow<T>(g[o]));
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

// ------------------------------------------------------------------------------------------------
// All prior classes of a model in one launch.  The terms of up to kMaxPriorSegments index lists are laid end to end (each
// list's share of the thread space rounded up to whole warps, so that a warp never mixes kinds); indices are 32-bit, the
// structure of a term is looked up from its first bead, and every list has its own energy row and gradient block, so the
// caller still gets one energy / force set per prior (src/mlcg/nn/gradients.py:111-117 adds them up afterwards).
//   pair lists that hold both (i, j) and (j, i) ("symmetric"): the gradient on bead i is twice the sum over i's own terms,
//   so only the first bead of a term is written, through the reduction over runs of equal first index: no scatter.
//   FIXED: energies and gradients are accumulated as 64-bit fixed-point integers (integer addition is associative: the
//   result does not depend on the order in which the threads arrive) and converted afterwards.
// ------------------------------------------------------------------------------------------------
constexpr int kFixedShift = 36;          // fixed point: 2^-36 resolution, +-1.3e8 range

struct PriorSegments {
    int n;
    int kind[MLCGB_MAX_PRIOR_SEGMENTS], n_params[MLCGB_MAX_PRIOR_SEGMENTS], symmetric[MLCGB_MAX_PRIOR_SEGMENTS];
    int64_t M[MLCGB_MAX_PRIOR_SEGMENTS], vstart[MLCGB_MAX_PRIOR_SEGMENTS + 1];     // terms; first thread of the list (multiple of 32)
    const int32_t *idx[MLCGB_MAX_PRIOR_SEGMENTS];                                  // [order, M]
    const void *params[MLCGB_MAX_PRIOR_SEGMENTS];                                  // [n_params, M]
    const int64_t *run_ptr[MLCGB_MAX_PRIOR_SEGMENTS];                              // NULL, or [n_runs + 1]: runs of equal first bead
    int64_t n_runs[MLCGB_MAX_PRIOR_SEGMENTS];
};

template <typename T> __device__ __forceinline__ long long to_fixed(T v) { return __double2ll_rn((double)v * (double)(1ll << kFixedShift)); }

template <typename T, bool FIXED> struct Accum;
template <typename T> struct Accum<T, false> {
    T *e, *g;
    __device__ __forceinline__ void energy(int64_t at, T v) const { atomicAdd(e + at, v); }
    __device__ __forceinline__ void grad3(int64_t at, const V3<T> &v) const { atomic_add3(g, at, v); }
};
template <typename T> struct Accum<T, true> {
    unsigned long long *e, *g;
    __device__ __forceinline__ void energy(int64_t at, T v) const { atomicAdd(e + at, (unsigned long long)to_fixed(v)); }
    __device__ __forceinline__ void grad3(int64_t at, const V3<T> &v) const {
        atomicAdd(g + at * 3, (unsigned long long)to_fixed(v.x));
        atomicAdd(g + at * 3 + 1, (unsigned long long)to_fixed(v.y));
        atomicAdd(g + at * 3 + 2, (unsigned long long)to_fixed(v.z));
    }
};

// v summed over runs of consecutive lanes with equal index i, added once per run (every lane calls; i = -1: nothing)
template <typename T, typename A>
__device__ __forceinline__ void run_accumulate(const A &acc, int64_t block0, int32_t i, V3<T> v, int lane) {
    const int32_t prev = __shfl_up_sync(0xffffffffu, i, 1);
    const bool head = lane == 0 || prev != i;
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    const unsigned above = lane == 31 ? 0u : (heads >> (lane + 1));
    const int run_end = above ? lane + __ffs(above) : 32;   // exclusive
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T x = __shfl_down_sync(0xffffffffu, v.x, o), y = __shfl_down_sync(0xffffffffu, v.y, o), z = __shfl_down_sync(0xffffffffu, v.z, o);
        if (lane + o < run_end) { v.x += x; v.y += y; v.z += z; }
    }
    if (head && i >= 0) acc.grad3(block0 + i, v);
}

template <typename T, bool FIXED>
__global__ void __launch_bounds__(256, 4)      // four blocks per SM (64 registers): the long pair lists are bound by memory latency
prior_eval_kernel(PriorSegments seg, const T *__restrict__ pos, const int32_t *__restrict__ struct_of, int64_t N, int64_t B,
                  typename std::conditional<FIXED, unsigned long long, T>::type *__restrict__ energy,
                  typename std::conditional<FIXED, unsigned long long, T>::type *__restrict__ grad, int32_t *__restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t vtotal = seg.vstart[seg.n];
    Accum<T, FIXED> acc{energy, grad};
    for (int64_t vbase = (int64_t)blockIdx.x * blockDim.x + threadIdx.x - lane; vbase < vtotal; vbase += stride) {
        int s = 0;
        while (s + 1 < seg.n && vbase >= seg.vstart[s + 1]) s++;               // warp-uniform: lists start on warp boundaries
        const int kind = seg.kind[s];
        const int64_t M = seg.M[s], t = vbase - seg.vstart[s] + lane;
        const int32_t *idx = seg.idx[s];
        const T *params = (const T *)seg.params[s];
        const int64_t e_row = (int64_t)s * B, g_block = (int64_t)s * N;
        if (seg.run_ptr[s]) {
            // A symmetric pair list given with its runs of equal first bead: one warp per run.  The bead's position is read once,
            // energy and gradient are summed in registers over the run and reduced across the warp: one addition per bead and
            // component, no scatter (the reverse terms of the list carry the other half of every pair's gradient).
            const int64_t run = (vbase - seg.vstart[s]) >> 5;
            if (run >= seg.n_runs[s]) continue;
            const int64_t k0 = seg.run_ptr[s][run], k1 = seg.run_ptr[s][run + 1];
            if (k0 < 0 || k1 > M || k1 <= k0) {
                if (k1 != k0 && lane == 0) atomicOr(status, (int)kBadIndex);
                continue;
            }
            const int32_t c0 = idx[k0];
            if (c0 < 0 || c0 >= N) {
                if (lane == 0) atomicOr(status, (int)kBadIndex);
                continue;
            }
            const int32_t mbr = struct_of[c0];
            const V3<T> p0 = ld3(pos, c0);
            T es = T(0);
            V3<T> gs{T(0), T(0), T(0)};
            bool bad = mbr < 0 || mbr >= B;
            // four terms per lane and round: their index, parameter and position loads are issued before any is used
            for (int64_t k = k0 + lane; k < k1; k += 128) {
                int32_t j[4];
                bool ok[4];
                T pa[4], pb[4];
                V3<T> pj[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t ku = k + 32 * u;
                    ok[u] = ku < k1;
                    j[u] = ok[u] ? idx[M + ku] : c0;
                    pa[u] = ok[u] ? params[ku] : T(0);
                    pb[u] = (ok[u] && kind == 0) ? params[M + ku] : T(0);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (j[u] < 0 || j[u] >= N) {
                        bad = true;
                        j[u] = c0;
                        ok[u] = false;
                    }
                    pj[u] = ld3(pos, j[u]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const V3<T> dr = sub(pj[u], p0);
                    const T d2 = dot(dr, dr);
                    const T inv_d = rsqrt(d2);
                    T ee, dEdd_over_d;
                    if (kind == 0) {
                        const T d = d2 * inv_d;
                        ee = pb[u] * (d - pa[u]) * (d - pa[u]);
                        dEdd_over_d = T(2) * pb[u] * (d - pa[u]) * inv_d;
                    } else {
                        const T q = pa[u] * inv_d;
                        const T rr = q * q;
                        ee = rr * rr * rr;
                        dEdd_over_d = T(-6) * ee * inv_d * inv_d;
                    }
                    if (ok[u]) {  // a padded or rejected slot computed on the bead itself (distance 0): dropped here
                        es += ee;
                        gs.x += dr.x * dEdd_over_d; gs.y += dr.y * dEdd_over_d; gs.z += dr.z * dEdd_over_d;
                    }
                }
            }
            es = warp_sum(es);
            gs.x = warp_sum(gs.x); gs.y = warp_sum(gs.y); gs.z = warp_sum(gs.z);
            if (__any_sync(0xffffffffu, bad)) {
                if (lane == 0) atomicOr(status, (int)kBadIndex);
                continue;
            }
            if (lane == 0) {
                acc.grad3(g_block + c0, scale(gs, T(-2)));
                acc.energy(e_row + mbr, es);
            }
            continue;
        }
        bool valid = t < M;
        int32_t i0 = 0, i1 = 0, i2 = 0, i3 = 0;
        if (valid) {
            i0 = idx[t];
            i1 = idx[M + t];
            if (kind == 1 || kind == 2) i2 = idx[2 * M + t];
            if (kind == 2) i3 = idx[3 * M + t];
            if (i0 < 0 || i0 >= N || i1 < 0 || i1 >= N || i2 < 0 || i2 >= N || i3 < 0 || i3 >= N) {
                valid = false;
                atomicOr(status, (int)kBadIndex);
            }
        }
        int32_t mb = valid ? struct_of[i0] : 0;
        if (valid && (mb < 0 || mb >= B)) {
            valid = false;
            atomicOr(status, (int)kBadIndex);
        }
        T e = T(0);
        V3<T> g0{T(0), T(0), T(0)};
        if (valid) {
            if (kind == 0 || kind == 3) {
                V3<T> g1;
                if (kind == 0) {
                    V3<double> g1d;
                    e = (T)bond_term(pos, i0, i1, (double)params[t], (double)params[M + t], g1d);
                    g1 = narrow<T>(g1d);
                } else {
                    const V3<T> dr = sub(ld3(pos, i1), ld3(pos, i0));
                    const T d = sqrt(dot(dr, dr));
                    const T q = params[t] / d;
                    const T rr = q * q;
                    e = rr * rr * rr;
                    g1 = scale(dr, T(-6) * e / d / d);
                }
                if (seg.symmetric[s]) {
                    g0 = scale(g1, T(-2));                       // the reverse term of the list adds the same again
                } else {
                    acc.grad3(g_block + i1, g1);
                    g0 = scale(g1, T(-1));
                }
            } else if (kind == 1) {
                V3<double> ga, gb;
                e = (T)angle_term(pos, i0, i1, i2, (double)params[t], (double)params[M + t], ga, gb);
                acc.grad3(g_block + i0, narrow<T>(ga));
                acc.grad3(g_block + i2, narrow<T>(gb));
                acc.grad3(g_block + i1, narrow<T>(V3<double>{-ga.x - gb.x, -ga.y - gb.y, -ga.z - gb.z}));
            } else {
                V3<double> g[4];
                e = (T)torsion_term(pos, i0, i1, i2, i3, params, M, t, (seg.n_params[s] - 1) / 2, g);
                acc.grad3(g_block + i0, narrow<T>(g[0]));
                acc.grad3(g_block + i1, narrow<T>(g[1]));
                acc.grad3(g_block + i2, narrow<T>(g[2]));
                acc.grad3(g_block + i3, narrow<T>(g[3]));
            }
        }
        if (kind == 0 || kind == 3) run_accumulate<T>(acc, g_block, valid ? i0 : -1, g0, lane);
        // energy: one addition per warp when the whole warp sits in one structure
        const int32_t mb0 = __shfl_sync(0xffffffffu, mb, 0);
        const bool same = __all_sync(0xffffffffu, !valid || mb == mb0);
        const bool lane0_valid = __shfl_sync(0xffffffffu, (int)valid, 0) != 0;
        if (same && lane0_valid) {
            const T sum = warp_sum(e);
            if (lane == 0) acc.energy(e_row + mb0, sum);
        } else if (valid) {
            acc.energy(e_row + mb, e);
        }
    }
}

template <typename T>
__global__ void fixed_to_float_kernel(const unsigned long long *__restrict__ in, int64_t n, T *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (T)((double)(long long)in[i] * (1.0 / (double)(1ll << kFixedShift)));
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

extern "C" size_t mlcgb_prior_eval_workspace_bytes(int n_lists, int64_t N, int64_t B, int fixed_point) {
    if (n_lists <= 0 || N < 0 || B < 0 || !fixed_point) return 0;
    return (size_t)n_lists * (size_t)(3 * N + B) * sizeof(unsigned long long);
}

extern "C" int mlcgb_prior_eval(int n_lists, const mlcgb_prior_list *lists, const void *pos, int dtype, const int32_t *struct_of, int64_t N,
                                int64_t B, void *energy, void *grad, int fixed_point, void *workspace, size_t workspace_bytes,
                                int32_t *status, void *stream) {
    TimelineScope timeline_scope("prior_eval", stream);
    if (n_lists < 0 || n_lists > MLCGB_MAX_PRIOR_SEGMENTS || N < 0 || B < 0 || !status) return MLCGB_E_ARG;
    if (n_lists == 0) return MLCGB_OK;
    if (!lists || !pos || !struct_of || !energy || !grad || N >= ((int64_t)1 << 31)) return MLCGB_E_ARG;
    PriorSegments seg;
    seg.n = n_lists;
    int64_t v = 0;
    for (int i = 0; i < n_lists; i++) {
        const mlcgb_prior_list &l = lists[i];
        const int need = l.kind == 3 ? 1 : (l.kind == 2 ? 3 : 2);
        if (l.kind < 0 || l.kind > 3 || l.M < 0 || l.n_params < need || (l.kind == 2 && (l.n_params - 1) % 2 != 0)) return MLCGB_E_ARG;
        if (l.M > 0 && (!l.idx || !l.params)) return MLCGB_E_ARG;
        seg.kind[i] = l.kind;
        seg.n_params[i] = l.n_params;
        seg.symmetric[i] = (l.kind == 0 || l.kind == 3) && l.symmetric ? 1 : 0;
        seg.M[i] = l.M;
        seg.idx[i] = l.idx;
        seg.params[i] = l.params;
        const bool runs = seg.symmetric[i] && l.run_ptr && l.n_runs > 0;
        seg.run_ptr[i] = runs ? l.run_ptr : nullptr;
        seg.n_runs[i] = runs ? l.n_runs : 0;
        seg.vstart[i] = v;
        v += runs ? l.n_runs * 32 : (l.M + 31) / 32 * 32;
    }
    seg.vstart[n_lists] = v;
    if (v == 0) return MLCGB_OK;
    auto st = (cudaStream_t)stream;
    const int grid = grid_for(v, 256, 16);
    const int64_t n_acc = (int64_t)n_lists * (3 * N + B);
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        if (fixed_point) {
            // accumulators: [n_lists][B] energies, then [n_lists][N][3] gradients, zeroed here, converted into energy / grad
            if (workspace_bytes < (size_t)n_acc * sizeof(unsigned long long) || !workspace) return MLCGB_E_WORKSPACE;
            auto *acc = (unsigned long long *)workspace;
            cudaMemsetAsync(acc, 0, (size_t)n_acc * sizeof(unsigned long long), st);
            prior_eval_kernel<scalar_t, true><<<grid, 256, 0, st>>>(seg, (const scalar_t *)pos, struct_of, N, B, acc, acc + (int64_t)n_lists * B, status);
            fixed_to_float_kernel<scalar_t><<<grid_for((int64_t)n_lists * B, 256), 256, 0, st>>>(acc, (int64_t)n_lists * B, (scalar_t *)energy);
            fixed_to_float_kernel<scalar_t><<<grid_for((int64_t)n_lists * N * 3, 256), 256, 0, st>>>(acc + (int64_t)n_lists * B, (int64_t)n_lists * N * 3, (scalar_t *)grad);
        } else {
            prior_eval_kernel<scalar_t, false><<<grid, 256, 0, st>>>(seg, (const scalar_t *)pos, struct_of, N, B, (scalar_t *)energy, (scalar_t *)grad, status);
        }
        return check_launch();
    });
}
