// Full-precision GEMMs of the filter-generating network (edge-sized: M or K is the edge count).
//
// CUDA-core FMA path: fp32 (and fp64 for derivative checks) products with fp32/fp64 accumulation,
// which is what the 1e-5 energy / 1e-4 force parity bar needs.  128x128 CTA tile, 8x8 register
// tile per thread, operands staged through shared memory with the contraction index outermost so
// the inner product reads are conflict-free broadcasts.
//   mode 0 (NT): C[M,N] = A[M,K] * B[N,K]^T (+ bias)
//   mode 1 (NN): C[M,N] = A[M,K] * B[K,N]
//   mode 2 (TN): C[M,N] = A[K,M]^T * B[K,N], K split across CTAs, partial tiles summed in order
#include "common.cuh"

namespace mlcgb {

constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN_ = 8;
constexpr int kGemmThreads = (BM / TM) * (BN / TN_);  // 256

// A is addressed as A(m,k) = A[m*sa_m + k*sa_k]; B as B(k,n) = B[k*sb_k + n*sb_n].
template <typename T>
__global__ void __launch_bounds__(kGemmThreads)
gemm_kernel(const T *__restrict__ A, int64_t sa_m, int64_t sa_k, const T *__restrict__ B, int64_t sb_k, int64_t sb_n,
            const T *__restrict__ bias, int64_t M, int64_t N, int64_t K, int64_t k_chunk, T *__restrict__ C,
            int64_t c_split_stride) {
    __shared__ T As[BK][BM + 4];
    __shared__ T Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int64_t m0 = (int64_t)blockIdx.x * BM, n0 = (int64_t)blockIdx.y * BN;
    const int64_t kbeg = (int64_t)blockIdx.z * k_chunk;
    const int64_t kend = kbeg + k_chunk < K ? kbeg + k_chunk : K;
    const int tx = tid % (BN / TN_), ty = tid / (BN / TN_);
    T acc[TM][TN_];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN_; j++) acc[i][j] = T(0);

    // The tile loaders walk the faster-varying index of each operand with consecutive threads.
    const bool a_kfast = sa_k == 1;
    const bool b_nfast = sb_n == 1;
    for (int64_t kt = kbeg; kt < kend; kt += BK) {
        for (int idx = tid; idx < BM * BK; idx += kGemmThreads) {
            int mm, kk;
            if (a_kfast) { kk = idx % BK; mm = idx / BK; } else { mm = idx % BM; kk = idx / BM; }
            const int64_t m = m0 + mm, k = kt + kk;
            As[kk][mm] = (m < M && k < kend) ? A[m * sa_m + k * sa_k] : T(0);
        }
        for (int idx = tid; idx < BN * BK; idx += kGemmThreads) {
            int nn, kk;
            if (b_nfast) { nn = idx % BN; kk = idx / BN; } else { kk = idx % BK; nn = idx / BK; }
            const int64_t n = n0 + nn, k = kt + kk;
            Bs[kk][nn] = (n < N && k < kend) ? B[k * sb_k + n * sb_n] : T(0);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            // each thread owns rows {ty*4..+3, 64+ty*4..+3} and columns {tx*4..+3, 64+tx*4..+3}:
            // a half-warp reads 16 consecutive 4-element groups, so shared reads are conflict-free
            T a[TM], b[TN_];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = As[kk][ty * 4 + i]; a[4 + i] = As[kk][64 + ty * 4 + i]; }
#pragma unroll
            for (int j = 0; j < 4; j++) { b[j] = Bs[kk][tx * 4 + j]; b[4 + j] = Bs[kk][64 + tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN_; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    T *Cout = C + (int64_t)blockIdx.z * c_split_stride;
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int64_t m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN_; j++) {
            const int64_t n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n < N) Cout[m * N + n] = acc[i][j] + (bias ? bias[n] : T(0));
        }
    }
}

template <typename T>
__global__ void splitk_reduce_kernel(const T *__restrict__ part, int64_t MN, int splits, T *__restrict__ C) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN; i += (int64_t)gridDim.x * blockDim.x) {
        T s = T(0);
        for (int z = 0; z < splits; z++) s += part[(int64_t)z * MN + i];
        C[i] = s;
    }
}

static int tn_splits(int64_t M, int64_t N, int64_t K) {
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    int64_t s = (2 * kNumSM + tiles - 1) / tiles;
    const int64_t max_by_k = (K + 4 * BK - 1) / (4 * BK);  // at least four k-tiles per split
    if (s > max_by_k) s = max_by_k;
    if (s < 1) s = 1;
    if (s > 1024) s = 1024;
    return (int)s;
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

size_t mlcgb_gemm_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K, int dtype) {
    if (mode != 2 || M <= 0 || N <= 0 || K <= 0) return 0;
    const int s = tn_splits(M, N, K);
    return s > 1 ? (size_t)s * (size_t)M * (size_t)N * (dtype == MLCGB_F64 ? 8 : 4) : 0;
}

int mlcgb_gemm(int mode, const void *A, const void *B, const void *bias, int dtype, int64_t M, int64_t N, int64_t K, void *C,
               void *workspace, size_t workspace_bytes, void *stream) {
    TimelineScope timeline_scope("gemm", stream);
    if (mode < 0 || mode > 2 || M < 0 || N < 0 || K < 0) return MLCGB_E_ARG;
    if (M == 0 || N == 0) return MLCGB_OK;
    if (!C || (K > 0 && (!A || !B))) return MLCGB_E_ARG;
    auto st = (cudaStream_t)stream;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        using T = scalar_t;
        int64_t sa_m, sa_k, sb_k, sb_n;
        if (mode == 0) { sa_m = K; sa_k = 1; sb_k = 1; sb_n = K; }
        else if (mode == 1) { sa_m = K; sa_k = 1; sb_k = N; sb_n = 1; }
        else { sa_m = 1; sa_k = M; sb_k = N; sb_n = 1; }
        int splits = 1;
        T *dst = (T *)C;
        if (mode == 2) {
            splits = tn_splits(M, N, K);
            if (splits > 1) {
                if (!workspace || workspace_bytes < (size_t)splits * M * N * sizeof(T)) return MLCGB_E_WORKSPACE;
                dst = (T *)workspace;
            }
        }
        int64_t k_chunk = (K + splits - 1) / splits;
        k_chunk = ((k_chunk + BK - 1) / BK) * BK;
        if (k_chunk < BK) k_chunk = BK;
        dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)((N + BN - 1) / BN), (unsigned)splits);
        if (grid.y > 65535 || grid.z > 65535) return MLCGB_E_LIMIT;
        gemm_kernel<T><<<grid, kGemmThreads, 0, st>>>((const T *)A, sa_m, sa_k, (const T *)B, sb_k, sb_n,
                                                      mode == 0 ? (const T *)bias : nullptr, M, N, K, k_chunk, dst, M * N);
        if (splits > 1)
            splitk_reduce_kernel<T><<<grid_for(M * N, 256), 256, 0, st>>>((const T *)workspace, M * N, splits, (T *)C);
        return check_launch();
    });
}

}  // extern "C"
