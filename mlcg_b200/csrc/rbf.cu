// Radial basis x cutoff envelope and its distance derivatives up to third order (stand-alone kernels).
//
// Derivatives are needed because forces are -dE/dpos (first order) and force matching differentiates
// the forces again (second order, third when the positions themselves carry a gradient).
#include "rbf_device.cuh"

namespace mlcgb {

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

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

int mlcgb_rbf_expand(const void *d, int dtype, int64_t E, const mlcgb_rbf_spec *spec, int order, void *out, void *stream) {
    TimelineScope timeline_scope("rbf_expand", stream);
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
    TimelineScope timeline_scope("rbf_contract", stream);
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
