// BAOAB Langevin integrator, the two halves around the force evaluation
// (LangevinSimulation.timestep, src/mlcg/simulation/langevin.py:100-144).
//
//   first half  (B, A, O, A):  v <- v + dt/2 f/m;  x <- x + dt/2 v;  v <- vscale v + noisescale sqrt(1/(beta m)) xi;
//                              x <- x + dt/2 v
//   second half (B):           v <- v + dt/2 f/m      with the forces at the new positions
// The normal deviates xi are an input, so the random stream stays the caller's (torch.Generator) and is the
// same as the reference's.  Pure streaming kernels: 3 reads + 2 writes (first half) per coordinate.
#include "common.cuh"

namespace mlcgb {

template <typename T>
__global__ void langevin_first_half_kernel(T *__restrict__ x, T *__restrict__ v, const T *__restrict__ f, const T *__restrict__ masses,
                                           const T *__restrict__ beta_mass_ratio, const T *__restrict__ noise, int64_t N, T dt, T vscale,
                                           T noisescale) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < 3 * N; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / 3;
        const T half = T(0.5) * dt;
        T vn = v[i] + half * f[i] / masses[n];
        T xn = x[i] + vn * half;
        vn = vn * vscale + noisescale * (beta_mass_ratio[n] * noise[i]);
        xn = xn + vn * half;
        x[i] = xn;
        v[i] = vn;
    }
}

template <typename T>
__global__ void langevin_second_half_kernel(T *__restrict__ v, const T *__restrict__ f, const T *__restrict__ masses, int64_t N, T dt) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < 3 * N; i += (int64_t)gridDim.x * blockDim.x)
        v[i] = v[i] + T(0.5) * dt * f[i] / masses[i / 3];
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

int mlcgb_langevin_first_half(void *x, void *v, const void *f, const void *masses, const void *beta_mass_ratio, const void *noise, int dtype,
                              int64_t N, double dt, double vscale, double noisescale, void *stream) {
    TimelineScope timeline_scope("langevin_first_half", stream);
    if (N < 0) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!x || !v || !f || !masses || !beta_mass_ratio || !noise) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        using T = scalar_t;
        langevin_first_half_kernel<T><<<grid_for(3 * N, 256), 256, 0, (cudaStream_t)stream>>>((T *)x, (T *)v, (const T *)f, (const T *)masses,
                                                                                             (const T *)beta_mass_ratio, (const T *)noise, N, (T)dt,
                                                                                             (T)vscale, (T)noisescale);
        return check_launch();
    });
}

int mlcgb_langevin_second_half(void *v, const void *f, const void *masses, int dtype, int64_t N, double dt, void *stream) {
    TimelineScope timeline_scope("langevin_second_half", stream);
    if (N < 0) return MLCGB_E_ARG;
    if (N == 0) return MLCGB_OK;
    if (!v || !f || !masses) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        using T = scalar_t;
        langevin_second_half_kernel<T><<<grid_for(3 * N, 256), 256, 0, (cudaStream_t)stream>>>((T *)v, (const T *)f, (const T *)masses, N, (T)dt);
        return check_launch();
    });
}

}  // extern "C"
