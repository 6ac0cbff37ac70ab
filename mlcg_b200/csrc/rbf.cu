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

// Gradients with respect to the basis parameters (offsets | means; coefficient | betas):
//   gp0[k] = sum_e c[e] G[e,k] d/dp0_k phi_k^(O)(d_e)        gp1 likewise
// One warp per edge row, lanes stride over k and keep their k's partial sums over the block's edges; the block's warps are
// added up in shared memory in a fixed order and written as one partial row per block; a second kernel adds the blocks'
// rows in order (no atomics: the result does not depend on scheduling).  At most kParamMaxR basis functions.
constexpr int kParamMaxR = 256, kParamPerLane = kParamMaxR / 32, kParamBlock = 256;

template <typename T, int O>
__global__ void __launch_bounds__(kParamBlock)
rbf_param_partial_kernel(const T *__restrict__ d, const T *__restrict__ G, const T *__restrict__ c, int64_t E, RbfDev<T> s,
                         T *__restrict__ partial /* [gridDim.x, 2, R] */) {
    __shared__ T s_acc[kParamBlock / 32][2][kParamMaxR];
    const int lane = threadIdx.x & 31, warp_in_block = threadIdx.x >> 5;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    T a0[kParamPerLane], a1[kParamPerLane];
#pragma unroll
    for (int j = 0; j < kParamPerLane; j++) a0[j] = a1[j] = T(0);
    for (int64_t e = warp; e < E; e += nwarps) {
        const T de = d[e];
        const T ce = c ? c[e] : T(1);
        const Jet<T, O> env = envelope_jet<T, O>(de, s);
        const Jet<T, O> ej = edge_jet<T, O>(de, s);
#pragma unroll
        for (int j = 0; j < kParamPerLane; j++) {
            const int k = lane + 32 * j;
            if (k < s.R) {
                T g0, g1;
                phi_param_deriv<T, O>(ej, env, k, s, g0, g1);
                const T w = ce * G[e * s.R + k];
                a0[j] += w * g0;
                a1[j] += w * g1;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kParamPerLane; j++) {
        s_acc[warp_in_block][0][lane + 32 * j] = a0[j];
        s_acc[warp_in_block][1][lane + 32 * j] = a1[j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * s.R; i += blockDim.x) {
        const int which = i / s.R, k = i % s.R;
        T sum = T(0);
#pragma unroll
        for (int w = 0; w < kParamBlock / 32; w++) sum += s_acc[w][which][k];
        partial[((int64_t)blockIdx.x * 2 + which) * s.R + k] = sum;
    }
}

// gp0[k], gp1[k] = sums over the blocks' partial rows, in block order; a Gaussian basis has one shared coefficient: gp1[0]
// = the sum over k as well
template <typename T>
__global__ void rbf_param_reduce_kernel(const T *__restrict__ partial, int nblocks, int R, int shared_p1, T *__restrict__ gp0, T *__restrict__ gp1) {
    __shared__ T s_p1[kParamMaxR];
    const int k = threadIdx.x;
    T s0 = T(0), s1 = T(0);
    if (k < R) {
        for (int b = 0; b < nblocks; b++) {
            s0 += partial[((int64_t)b * 2) * R + k];
            s1 += partial[((int64_t)b * 2 + 1) * R + k];
        }
        gp0[k] = s0;
        if (!shared_p1) gp1[k] = s1;
    }
    if (shared_p1) {
        s_p1[k] = k < R ? s1 : T(0);
        __syncthreads();
        if (k == 0) {
            T t = T(0);
            for (int i = 0; i < R; i++) t += s_p1[i];
            gp1[0] = t;
        }
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

static int param_blocks(int64_t E) {
    const int64_t want = (E + kParamBlock / 32 - 1) / (kParamBlock / 32);
    return (int)(want < 1 ? 1 : (want > 4 * kNumSM ? 4 * kNumSM : want));
}

size_t mlcgb_rbf_param_workspace_bytes(int64_t E, int num_rbf, int dtype) {
    if (E < 0 || num_rbf <= 0) return 0;
    return (size_t)param_blocks(E) * 2 * (size_t)num_rbf * (dtype == MLCGB_F64 ? 8 : 4);
}

int mlcgb_rbf_param_contract(const void *d, const void *G, const void *c, int dtype, int64_t E, const mlcgb_rbf_spec *spec, int order,
                             void *workspace, size_t workspace_bytes, void *gp0, void *gp1, void *stream) {
    TimelineScope timeline_scope("rbf_param_contract", stream);
    if (int rc = check_spec(spec, order)) return rc;
    if (E < 0 || !gp0 || !gp1) return MLCGB_E_ARG;
    if (spec->num_rbf > kParamMaxR) return MLCGB_E_LIMIT;
    if (E > 0 && (!d || !G || !workspace)) return MLCGB_E_ARG;
    if (workspace_bytes < mlcgb_rbf_param_workspace_bytes(E, spec->num_rbf, dtype)) return MLCGB_E_WORKSPACE;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        const RbfDev<scalar_t> s = to_dev<scalar_t>(spec);
        auto st = (cudaStream_t)stream;
        const int grid = E > 0 ? param_blocks(E) : 0;
        auto *ws = (scalar_t *)workspace;
        if (grid > 0) {
            const auto *dd = (const scalar_t *)d, *GG = (const scalar_t *)G, *cc = (const scalar_t *)c;
            switch (order) {
                case 0: rbf_param_partial_kernel<scalar_t, 0><<<grid, kParamBlock, 0, st>>>(dd, GG, cc, E, s, ws); break;
                case 1: rbf_param_partial_kernel<scalar_t, 1><<<grid, kParamBlock, 0, st>>>(dd, GG, cc, E, s, ws); break;
                case 2: rbf_param_partial_kernel<scalar_t, 2><<<grid, kParamBlock, 0, st>>>(dd, GG, cc, E, s, ws); break;
                default: rbf_param_partial_kernel<scalar_t, 3><<<grid, kParamBlock, 0, st>>>(dd, GG, cc, E, s, ws); break;
            }
        }
        rbf_param_reduce_kernel<scalar_t><<<1, kParamMaxR, 0, st>>>(ws, grid, s.R, s.kind == 0 ? 1 : 0, (scalar_t *)gp0, (scalar_t *)gp1);
        return check_launch();
    });
}

}  // extern "C"
