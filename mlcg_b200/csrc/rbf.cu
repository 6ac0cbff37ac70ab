// Radial basis x cutoff envelope and its distance derivatives up to third order.
//
// phi_k(d) = basis_k(d) * envelope(d).  Derivatives are needed because forces are -dE/dpos
// (first order) and force matching differentiates the forces again (second order, third when the
// positions themselves carry a gradient).  They are evaluated with truncated Taylor arithmetic:
// every quantity carries its coefficients c[m] = f^(m)(d)/m! for m = 0..ORDER, products are
// Cauchy products and exp() uses the standard recurrence, so one code path serves every order.
#include "common.cuh"

namespace mlcgb {

template <typename T, int O>
struct Jet {
    T c[O + 1];
};

template <typename T, int O>
__device__ __forceinline__ Jet<T, O> jet_mul(const Jet<T, O> &a, const Jet<T, O> &b) {
    Jet<T, O> r;
#pragma unroll
    for (int m = 0; m <= O; m++) {
        T s = T(0);
#pragma unroll
        for (int j = 0; j <= m; j++) s += a.c[j] * b.c[m - j];
        r.c[m] = s;
    }
    return r;
}

template <typename T, int O>
__device__ __forceinline__ Jet<T, O> jet_exp(const Jet<T, O> &a) {
    Jet<T, O> e;
    e.c[0] = exp(a.c[0]);
#pragma unroll
    for (int m = 1; m <= O; m++) {
        T s = T(0);
#pragma unroll
        for (int j = 1; j <= m; j++) s += T(j) * a.c[j] * e.c[m - j];
        e.c[m] = s / T(m);
    }
    return e;
}

template <typename T>
struct RbfDev {
    int kind, R, cutoff_kind;
    T lower, upper, alpha;
    const T *p0, *p1;
};

// envelope(d) as a jet.  Masks (d < upper, d > lower) are piecewise constant: zero derivative.
template <typename T, int O>
__device__ __forceinline__ Jet<T, O> envelope_jet(T d, const RbfDev<T> &s) {
    Jet<T, O> r;
    if (s.cutoff_kind == 0) {
        r.c[0] = T(1);
#pragma unroll
        for (int m = 1; m <= O; m++) r.c[m] = T(0);
        return r;
    }
    const T pi = T(3.14159265358979323846);
    T arg, a, mask;
    if (s.lower > T(0)) {
        const T w = s.upper - s.lower;
        arg = pi * (T(2) * (d - s.lower) / w + T(1));  // same operation order as the reference
        a = T(2) * pi / w;
        mask = (d < s.upper && d > s.lower) ? T(1) : T(0);
    } else {
        arg = d * pi / s.upper;
        a = pi / s.upper;
        mask = d < s.upper ? T(1) : T(0);
    }
    T sn, cs;
    sincos(arg, &sn, &cs);
    const T half = T(0.5) * mask;
    // 0.5*(cos(a d + phase) + 1): derivatives cycle through -a sin, -a^2 cos, a^3 sin
    r.c[0] = half * (cs + T(1));
    if (O >= 1) r.c[O >= 1 ? 1 : 0] = -half * a * sn;
    if (O >= 2) r.c[O >= 2 ? 2 : 0] = -half * a * a * cs * T(0.5);
    if (O >= 3) r.c[O >= 3 ? 3 : 0] = half * a * a * a * sn * T(1.0 / 6.0);
    return r;
}

// per-edge part of the basis: Gaussian -> jet of d itself; exp-normal -> jet of u = exp(alpha*(lower-d))
template <typename T, int O>
__device__ __forceinline__ Jet<T, O> edge_jet(T d, const RbfDev<T> &s) {
    Jet<T, O> r;
    if (s.kind == 0) {
        r.c[0] = d;
        if (O >= 1) r.c[O >= 1 ? 1 : 0] = T(1);
#pragma unroll
        for (int m = 2; m <= O; m++) r.c[m] = T(0);
    } else {
        const T u = exp(s.alpha * (-d + s.lower));
        r.c[0] = u;
        T f = u;
#pragma unroll
        for (int m = 1; m <= O; m++) {
            f = f * (-s.alpha) / T(m);
            r.c[m] = f;
        }
    }
    return r;
}

// basis_k as a jet, given the per-edge jet
template <typename T, int O>
__device__ __forceinline__ Jet<T, O> basis_jet(const Jet<T, O> &ej, int k, const RbfDev<T> &s) {
    Jet<T, O> v = ej;
    v.c[0] -= s.p0[k];                       // d - offset_k   |   u - mean_k
    Jet<T, O> q = jet_mul<T, O>(v, v);       // squared
    const T scale = s.kind == 0 ? s.p1[0] : -s.p1[k];
#pragma unroll
    for (int m = 0; m <= O; m++) q.c[m] *= scale;
    return jet_exp<T, O>(q);
}

template <int O> struct Fact;
template <> struct Fact<0> { static constexpr double v = 1.0; };
template <> struct Fact<1> { static constexpr double v = 1.0; };
template <> struct Fact<2> { static constexpr double v = 2.0; };
template <> struct Fact<3> { static constexpr double v = 6.0; };

template <typename T, int O>
__device__ __forceinline__ T phi_deriv(const Jet<T, O> &ej, const Jet<T, O> &env, int k, const RbfDev<T> &s) {
    const Jet<T, O> b = basis_jet<T, O>(ej, k, s);
    T acc = T(0);
#pragma unroll
    for (int j = 0; j <= O; j++) acc += b.c[j] * env.c[O - j];
    return acc * T(Fact<O>::v);
}

// out[e,k]: one warp per edge row, lanes stride over k (coalesced row writes)
template <typename T, int O>
__global__ void __launch_bounds__(256)
rbf_expand_kernel(const T *__restrict__ d, int64_t E, RbfDev<T> s, T *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t e = warp; e < E; e += nwarps) {
        const T de = d[e];
        const Jet<T, O> env = envelope_jet<T, O>(de, s);
        const Jet<T, O> ej = edge_jet<T, O>(de, s);
        for (int k = lane; k < s.R; k += 32) out[e * s.R + k] = phi_deriv<T, O>(ej, env, k, s);
    }
}

template <typename T, int O>
__global__ void __launch_bounds__(256)
rbf_contract_kernel(const T *__restrict__ d, const T *__restrict__ G, int64_t E, RbfDev<T> s, T *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t e = warp; e < E; e += nwarps) {
        const T de = d[e];
        const Jet<T, O> env = envelope_jet<T, O>(de, s);
        const Jet<T, O> ej = edge_jet<T, O>(de, s);
        T acc = T(0);
        for (int k = lane; k < s.R; k += 32) acc += G[e * s.R + k] * phi_deriv<T, O>(ej, env, k, s);
        acc = warp_sum(acc);
        if (lane == 0) out[e] = acc;
    }
}

template <typename T>
static RbfDev<T> to_dev(const mlcgb_rbf_spec *sp) {
    RbfDev<T> s;
    s.kind = sp->kind;
    s.R = sp->num_rbf;
    s.cutoff_kind = sp->cutoff_kind;
    s.lower = (T)sp->lower;
    s.upper = (T)sp->upper;
    s.alpha = (T)sp->alpha;
    s.p0 = (const T *)sp->p0;
    s.p1 = (const T *)sp->p1;
    return s;
}

static int check_spec(const mlcgb_rbf_spec *sp, int order) {
    if (!sp || order < 0 || order > 3) return MLCGB_E_ARG;
    if ((sp->kind != 0 && sp->kind != 1) || (sp->cutoff_kind != 0 && sp->cutoff_kind != 1)) return MLCGB_E_ARG;
    if (sp->num_rbf <= 0 || !sp->p0 || !sp->p1) return MLCGB_E_ARG;
    return MLCGB_OK;
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

int mlcgb_rbf_expand(const void *d, int dtype, int64_t E, const mlcgb_rbf_spec *spec, int order, void *out, void *stream) {
    if (int rc = check_spec(spec, order)) return rc;
    if (E < 0) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!d || !out) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        const RbfDev<scalar_t> s = to_dev<scalar_t>(spec);
        const int grid = grid_for(E * 32, 256, 32);
        auto st = (cudaStream_t)stream;
        switch (order) {
            case 0: rbf_expand_kernel<scalar_t, 0><<<grid, 256, 0, st>>>((const scalar_t *)d, E, s, (scalar_t *)out); break;
            case 1: rbf_expand_kernel<scalar_t, 1><<<grid, 256, 0, st>>>((const scalar_t *)d, E, s, (scalar_t *)out); break;
            case 2: rbf_expand_kernel<scalar_t, 2><<<grid, 256, 0, st>>>((const scalar_t *)d, E, s, (scalar_t *)out); break;
            default: rbf_expand_kernel<scalar_t, 3><<<grid, 256, 0, st>>>((const scalar_t *)d, E, s, (scalar_t *)out); break;
        }
        return check_launch();
    });
}

int mlcgb_rbf_contract(const void *d, const void *G, int dtype, int64_t E, const mlcgb_rbf_spec *spec, int order, void *s_out,
                       void *stream) {
    if (int rc = check_spec(spec, order)) return rc;
    if (E < 0) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!d || !G || !s_out) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        const RbfDev<scalar_t> s = to_dev<scalar_t>(spec);
        const int grid = grid_for(E * 32, 256, 32);
        auto st = (cudaStream_t)stream;
        switch (order) {
            case 0: rbf_contract_kernel<scalar_t, 0><<<grid, 256, 0, st>>>((const scalar_t *)d, (const scalar_t *)G, E, s, (scalar_t *)s_out); break;
            case 1: rbf_contract_kernel<scalar_t, 1><<<grid, 256, 0, st>>>((const scalar_t *)d, (const scalar_t *)G, E, s, (scalar_t *)s_out); break;
            case 2: rbf_contract_kernel<scalar_t, 2><<<grid, 256, 0, st>>>((const scalar_t *)d, (const scalar_t *)G, E, s, (scalar_t *)s_out); break;
            default: rbf_contract_kernel<scalar_t, 3><<<grid, 256, 0, st>>>((const scalar_t *)d, (const scalar_t *)G, E, s, (scalar_t *)s_out); break;
        }
        return check_launch();
    });
}

}  // extern "C"
