// Shared helpers for the sm_100a kernels of mlcg_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/mlcg_b200.h"

namespace mlcgb {

constexpr int kNumSM = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

enum StatusBits : int { kTruncated = 1, kBadIndex = 2, kAsymmetric = 4, kTensorWait = 8, kWeightRange = 16, kCapacity = 32 };

extern thread_local int g_last_cuda_error;

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return MLCGB_E_LAUNCH;
    }
    return MLCGB_OK;
}

// Device time per entry point, for hosts that want to know where an evaluation's time goes without a profiler attached:
// while the calling host thread has a timeline open (mlcgb_timeline_begin), every kernel-launching entry point brackets its
// launches with a CUDA event pair on its stream (only the outermost such entry point of a nest records).  Off, the scope
// costs one thread-local read.
struct TimelineScope {
    int slot;
    cudaStream_t st;
    TimelineScope(const char *name, void *stream);
    ~TimelineScope();
    TimelineScope(const TimelineScope &) = delete;
    TimelineScope &operator=(const TimelineScope &) = delete;
};

// Programmatic dependent launch: a kernel launched this way may start (on SMs the previous kernel of the stream has
// already left) before that kernel has finished as a whole; it runs its own set-up — weight tiles, barriers, tensor-memory
// allocation, nothing that depends on the previous kernel — and calls pdl_wait() before it touches any activation.
// pdl_wait() returns once the previous kernel has completed and its writes are visible; it is a no-op for a plain launch.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);      // errors surface through cudaGetLastError() in check_launch()
}
#endif

inline int grid_for(int64_t work_items, int per_block, int max_waves = 64) {
    int64_t blocks = (work_items + per_block - 1) / per_block;
    int64_t cap = (int64_t)kNumSM * max_waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <typename T> struct Vec4;
template <> struct Vec4<float> { using type = float4; };
template <> struct Vec4<double> { using type = double4; };

// Explicitly rounded arithmetic for the pair test.  The squared distance is evaluated the way the reference's compiled
// kernels evaluate it: `dist += diff * diff` over the three coordinates (src/opt_radius/mlcg_opt_radius/radius.cu:126-130,
// and the same loop in torch_cluster's radius kernel), which nvcc contracts into fused multiply-adds by default:
//   d2 = fma(dz, dz, fma(dy, dy, dx * dx)).
// Writing the roundings out (instead of leaving the contraction to the compiler) fixes the decision for every pair,
// including pairs within one rounding of the cutoff; the host oracle evaluates the same expression with libm's fma.
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float fma_rn(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ double fma_rn(double a, double b, double c) { return __fma_rn(a, b, c); }

template <typename T>
__device__ __forceinline__ T dist2_rn(T xi, T yi, T zi, T xj, T yj, T zj) {
    const T dx = sub_rn(xj, xi), dy = sub_rn(yj, yi), dz = sub_rn(zj, zi);
    return fma_rn(dz, dz, fma_rn(dy, dy, mul_rn(dx, dx)));
}

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace mlcgb

#define MLCGB_DISPATCH_DTYPE(dtype, ...)                     \
    [&]() -> int {                                           \
        if ((dtype) == MLCGB_F32) {                          \
            using scalar_t = float;                          \
            return __VA_ARGS__();                            \
        } else if ((dtype) == MLCGB_F64) {                   \
            using scalar_t = double;                         \
            return __VA_ARGS__();                            \
        }                                                    \
        return MLCGB_E_ARG;                                  \
    }()
