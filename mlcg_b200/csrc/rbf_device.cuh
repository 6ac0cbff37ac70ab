// Device-side radial basis x envelope with distance derivatives by truncated Taylor arithmetic.
//
// phi_k(d) = basis_k(d) * envelope(d).  Every quantity carries its coefficients c[m] = f^(m)(d)/m!
// for m = 0..ORDER; products are Cauchy products and exp() uses the standard recurrence, so one
// code path serves every derivative order.
#pragma once
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

// d(basis_k)/d(p0_k) and d(basis_k)/d(p1) as jets in the distance, given the per-edge jet.  basis = exp(q), q = s v^2,
// v = w(d) - p0_k, s = p1 (Gaussian: the shared coefficient) or -p1_k (exp-normal):
//   d basis / d p0 = basis * (-2 s v)        d basis / d p1 = basis * (+v^2 | -v^2)
template <typename T, int O>
__device__ __forceinline__ void basis_param_jets(const Jet<T, O> &ej, int k, const RbfDev<T> &s, Jet<T, O> &dp0, Jet<T, O> &dp1) {
    Jet<T, O> v = ej;
    v.c[0] -= s.p0[k];
    const Jet<T, O> v2 = jet_mul<T, O>(v, v);
    const T scale = s.kind == 0 ? s.p1[0] : -s.p1[k];
    Jet<T, O> q = v2;
#pragma unroll
    for (int m = 0; m <= O; m++) q.c[m] *= scale;
    const Jet<T, O> b = jet_exp<T, O>(q);
    Jet<T, O> f0 = v, f1 = v2;
    const T sign1 = s.kind == 0 ? T(1) : T(-1);
#pragma unroll
    for (int m = 0; m <= O; m++) {
        f0.c[m] *= T(-2) * scale;
        f1.c[m] *= sign1;
    }
    dp0 = jet_mul<T, O>(b, f0);
    dp1 = jet_mul<T, O>(b, f1);
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


// order-O distance derivative of d(basis_k x envelope)/d(parameter), for both parameters
template <typename T, int O>
__device__ __forceinline__ void phi_param_deriv(const Jet<T, O> &ej, const Jet<T, O> &env, int k, const RbfDev<T> &s, T &g0, T &g1) {
    Jet<T, O> dp0, dp1;
    basis_param_jets<T, O>(ej, k, s, dp0, dp1);
    T a0 = T(0), a1 = T(0);
#pragma unroll
    for (int j = 0; j <= O; j++) {
        a0 += dp0.c[j] * env.c[O - j];
        a1 += dp1.c[j] * env.c[O - j];
    }
    g0 = a0 * T(Fact<O>::v);
    g1 = a1 * T(Fact<O>::v);
}

template <typename T>
static inline RbfDev<T> to_dev(const mlcgb_rbf_spec *sp) {
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

static inline int check_spec(const mlcgb_rbf_spec *sp, int order) {
    if (!sp || order < 0 || order > 3) return MLCGB_E_ARG;
    if ((sp->kind != 0 && sp->kind != 1) || (sp->cutoff_kind != 0 && sp->cutoff_kind != 1)) return MLCGB_E_ARG;
    if (sp->num_rbf <= 0 || !sp->p0 || !sp->p1) return MLCGB_E_ARG;
    return MLCGB_OK;
}

}  // namespace mlcgb
