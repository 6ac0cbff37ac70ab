/*
 * mlcg_b200 — C ABI of the B200 (sm_100a) kernels behind mlcg's coarse-grained force-field hot path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host". The library never allocates,
 *     frees or synchronises (one entry point, mlcgb_radius_graph_static, waits for its stream once and says so):
 *     the caller owns inputs, outputs and workspaces and passes the stream.
 *   - `dtype`: 0 = float32, 1 = float64 (the type of positions and of every floating tensor of a call).
 *   - Node tensors are row-major [N, F]; edge tensors are row-major [E, F]; index rows are contiguous.
 *   - Return value: 0 on success, a negative MLCGB_E_* code otherwise (mlcgb_strerror gives the text).
 *     Data-dependent conditions are reported through a 4-word device `status` array the caller zeroes:
 *     status[0] bit 0 = a centre had more neighbours than max_num_neighbors (list truncated),
 *     status[0] bit 1 = an index was out of range and the element was skipped,
 *     status[0] bit 2 = an edge had no reverse partner (graph not symmetric).
 *   - `stream` is a cudaStream_t passed as void*.
 *
 * Each entry point names the reference interface it stands in for (path inside the mlcg repository).
 */
#ifndef MLCG_B200_H
#define MLCG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLCGB_OK 0
#define MLCGB_E_ARG (-1)       /* null pointer, negative size, unsupported dtype / option */
#define MLCGB_E_WORKSPACE (-2) /* workspace too small */
#define MLCGB_E_LAUNCH (-3)    /* the CUDA runtime refused a launch (see mlcgb_last_cuda_error) */
#define MLCGB_E_LIMIT (-4)     /* a size is beyond what the entry point supports */

#define MLCGB_F32 0
#define MLCGB_F64 1

#define MLCGB_RULE_NATIVE 0  /* mlcg_opt_radius: skip self, keep the first max_num_neighbors by index */
#define MLCGB_RULE_CLUSTER 1 /* torch_cluster.radius_graph: max_num_neighbors+1 incl. self, self dropped */

const char *mlcgb_strerror(int code);
int mlcgb_last_cuda_error(void); /* cudaError_t of the last failed launch on this host thread */
int mlcgb_version(void);

/* Device time per entry point, without a profiler.  No counterpart in the reference (mlcg times whole steps on the host).
 * Between mlcgb_timeline_begin and mlcgb_timeline_end, every kernel-launching entry point called from the same host thread
 * brackets its launches with a CUDA event pair on its stream (the events are created on first use and kept: host-side
 * objects, no device memory).  mlcgb_timeline_end waits for the recorded events and returns the number of distinct entry
 * points seen (or a negative code); mlcgb_timeline_entry(i, ...) then gives name, number of calls and summed milliseconds of
 * the i-th.  Entry points that only sequence others (mlcgb_interaction_*, mlcgb_schnet_eval*) are not recorded themselves:
 * their parts are.  A recorded launch cannot overlap its set-up with the tail of the launch before it, so a recorded step
 * is a little slower than an unrecorded one. */
int mlcgb_timeline_begin(void);
int mlcgb_timeline_end(void);
int mlcgb_timeline_entry(int index, const char **name /* out: static string */, int64_t *calls, double *ms);

/* ------------------------------------------------------------------------------------------------
 * Radius graph.  Replaces torch_cluster.radius_graph as called at
 * src/mlcg/neighbor_list/torch_impl.py:216-224 and mlcg::radius_cuda
 * (src/opt_radius/mlcg_opt_radius/radius.cu:197-307).  Two calls around one host read of the edge
 * count: `count` builds the per-structure cell lists in the workspace, writes deg[N] and the
 * exclusive prefix sum offsets[N+1] (offsets[N] = E), and leaves in the workspace what it found (a
 * mask of each point's neighbours among the candidates it tested, about 100 bytes per float32
 * point); `fill`, given the same workspace untouched and the same pos, ptr, r and loop, writes the
 * edges, centre-major with neighbours ascending, which is the order both reference back ends
 * produce.
 * The pair test is fma(dz, dz, fma(dy, dy, dx*dx)) < (T)(r*r): the loop of radius.cu:126-130 as nvcc contracts it, which is
 * what the reference's compiled kernel decides by (compared with it pair by pair, tests/test_gpu_radius_reference.py).
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_batch_to_ptr(const int64_t *batch, int64_t N, int64_t B, int64_t *ptr /* [B+1] */, void *stream);
/* radius.py:64-75 (bucketize of arange(B+1) into the sorted batch vector). */

size_t mlcgb_radius_workspace_bytes(int64_t N, int64_t B, int dtype);

int mlcgb_radius_count(const void *pos /* [N,3] */, int dtype, const int64_t *ptr /* [B+1] */, int64_t N, int64_t B,
                       double r, int64_t max_num_neighbors, int loop, int rule, void *workspace, size_t workspace_bytes,
                       int32_t *deg /* [N] */, int64_t *offsets /* [N+1] */, int32_t *status, void *stream);

int mlcgb_radius_fill(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int loop,
                      const void *workspace, size_t workspace_bytes, const int64_t *offsets, int64_t E,
                      int64_t *edge_index /* [2,E]: row 0 centre, row 1 neighbour */,
                      void *distance /* [E] or NULL */, int64_t *mapping_batch /* [E] or NULL */,
                      int32_t *row0_i32 /* [E] or NULL */, int32_t *row1_i32 /* [E] or NULL */, int32_t *status,
                      void *stream);

/* The same two calls with excluded pairs, the last two arguments of mlcg::radius_cuda
 * (src/opt_radius/mlcg_opt_radius/radius.cu:112-133,197-203): exclude_pair_xs[ptr_exclude_pair_xs[i] ..
 * ptr_exclude_pair_xs[i+1]) lists, in ascending order, the points that centre i must not get as neighbours — the
 * layout mlcg::exclusion_pair_to_ptr produces (exclusion_pairs.cpp:7-62).  Neighbour cap as in radius.cu (the first
 * max_num_neighbors non-excluded hits by index).  Both pointers NULL: no exclusions. */
int mlcgb_radius_count_excl(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r,
                            int64_t max_num_neighbors, int loop, const int64_t *exclude_pair_xs,
                            const int64_t *ptr_exclude_pair_xs /* [N+1] */, void *workspace, size_t workspace_bytes,
                            int32_t *deg, int64_t *offsets, int32_t *status, void *stream);
int mlcgb_radius_fill_excl(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int loop,
                           const int64_t *exclude_pair_xs, const int64_t *ptr_exclude_pair_xs, const void *workspace,
                           size_t workspace_bytes, const int64_t *offsets, int64_t E, int64_t *edge_index, void *distance,
                           int64_t *mapping_batch, int32_t *row0_i32, int32_t *row1_i32, int32_t *status, void *stream);

/* Radius graph in one call that allocates nothing.  No counterpart in the reference (mlcg sizes its
 * outputs with torch and a host read, src/opt_radius/mlcg_opt_radius/radius.cu:236-241,288-292); it exists
 * for callers that may not allocate device memory at the point of the call: a force routine invoked from
 * inside another program's integration loop, a plug-in whose host owns all of the GPU's memory, a thread
 * that must stay off the allocator's locks.  The cell-list scratch is a fixed 3 MiB array inside the
 * library image (every GPU that loads the library holds it until the process exits); the limits are
 * N <= 65536 points and B <= 8192 structures, and larger inputs return MLCGB_E_LIMIT.
 *   deg[N], offsets[N+1] and edge_index[2, capacity] are the caller's; row 0 starts at edge_index, row 1 at
 *   edge_index + capacity; *n_edges_host (a HOST pointer) receives the number of edges, also when it
 *   exceeds `capacity`, in which case nothing is written to edge_index and MLCGB_E_LIMIT is returned.
 * Every call copies the edge count to the host and waits for the stream, so the entry point cannot be used while the stream
 * is being captured into a CUDA graph (mlcgb_radius_graph_capacity is the capturable form; it takes a caller's workspace).
 * The first call on each device also looks up the scratch address; concurrent first calls from several host threads may both
 * do the look-up and store the same value.  All calls on a device share the scratch: calls that may overlap on the GPU
 * (different streams or threads) race on it and must be serialised by the caller.  Nothing in the scratch has to start at zero
 * and nothing is kept between calls. */
int mlcgb_radius_graph_static(const void *pos /* [N,3] */, int dtype, const int64_t *ptr /* [B+1] */, int64_t N, int64_t B,
                              double r, int64_t max_num_neighbors, int loop, int rule, int32_t *deg /* [N] */,
                              int64_t *offsets /* [N+1] */, int64_t capacity, int64_t *edge_index /* [2,capacity] */,
                              int64_t *n_edges_host /* host */, int32_t *status, void *stream);

/* For each edge (a,b) of a centre-sorted list, the position of (b,a); -1 and status bit 2 if absent.
 * No reference counterpart: PyG aggregates at edge_index[1] with atomics (src/mlcg/nn/schnet.py:346);
 * this permutation is what lets the aggregation run as an ordered segmented sum instead. */
int mlcgb_edge_twin(const int32_t *row0, const int32_t *row1, const int64_t *offsets, int64_t E, int64_t N,
                    int32_t *twin /* [E] */, int32_t *status, void *stream);

/* pair_of[sel[k]] = pair_of[twin[sel[k]]] = k for k < P: the row that holds a pair's filter when the filters of a
 * symmetric list are stored once per unordered pair (mlcgb_filter_forward with `sel` and no `twin`); passed to
 * mlcgb_seg_mul_sum as `eperm`.  No reference counterpart. */
int mlcgb_pair_index(const int32_t *sel /* [P] */, const int32_t *twin /* [E] */, int64_t P, int32_t *pair_of /* [E] */,
                     void *stream);

/* mlcgb_edge_twin, the selection of one edge per unordered pair (row0 < row1, in list order: sel[P], P = E/2) and
 * mlcgb_pair_index in one call, for a symmetric, loop-free, centre-sorted list.  An edge without its reverse or a loop sets
 * status bit 2: the outputs are then not a valid plan, but every entry written is a valid index (twin[e] = e, pair_of[e] = 0
 * for such an edge), so that kernels already queued behind the call stay inside their arrays.  `sel` entries that no pair
 * claims are left as they were: zero the array first if that can happen.  The edge count is read from offsets[N] on the
 * device (E may be the larger capacity of the arrays).  No reference counterpart. */
size_t mlcgb_pair_plan_workspace_bytes(int64_t N);
int mlcgb_pair_plan(const int32_t *row0, const int32_t *row1, const int64_t *offsets /* [N+1] */, int64_t E, int64_t N,
                    void *workspace, size_t workspace_bytes, int32_t *twin /* [E] */, int32_t *sel /* [E/2] */,
                    int32_t *pair_of /* [E] */, int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Edge geometry.  compute_distances, src/mlcg/geometry/internal_coordinates.py:72-100, split into
 * its linear part dr = pos[row1] - pos[row0] and that part's transpose (used by every derivative).
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_edge_diff(const void *pos /* [N,3] */, int dtype, const int32_t *row0, const int32_t *row1, int64_t E,
                    int64_t N, void *dr /* [E,3] */, int32_t *status, void *stream);

/* out[n] = sum_{k in [ptr_in[n],ptr_in[n+1])} g[perm_in ? perm_in[k] : k] - sum_{k in [ptr_out..)} g[perm_out ? ... : k]
 * ("in" = edges whose row1 is n, "out" = edges whose row0 is n). Ordered, no atomics. */
int mlcgb_node_scatter_diff(const void *g /* [E,3] */, int dtype, const int64_t *ptr_in, const int32_t *perm_in,
                            const int64_t *ptr_out, const int32_t *perm_out, int64_t N, int64_t E,
                            void *out /* [N,3] */, void *stream);

/* The same distance in one kernel, d[e] = |pos[row1[e]] - pos[row0[e]]|, and its first derivative
 * gpos[n] = sum_{e: row1=n} (g_e/d_e) dr_e - sum_{e: row0=n} (g_e/d_e) dr_e (ordered, no atomics): the force path
 * of energy/force evaluation, where nothing has to be differentiated a second time. */
int mlcgb_edge_distance(const void *pos, int dtype, const int32_t *row0, const int32_t *row1, int64_t E, int64_t N,
                        void *d /* [E] */, int32_t *status, void *stream);
int mlcgb_edge_distance_backward(const void *pos, const void *g /* [E] */, const void *d /* [E] */, int dtype,
                                 const int32_t *row0, const int32_t *row1, const int64_t *ptr_in, const int32_t *perm_in,
                                 const int64_t *ptr_out, const int32_t *perm_out, int64_t N, int64_t E, void *gpos /* [N,3] */,
                                 void *stream);

/* ------------------------------------------------------------------------------------------------
 * Radial basis times cutoff envelope, and its derivatives with respect to the distance.
 * GaussianBasis.forward src/mlcg/nn/radial_basis/gaussian.py:83-102, ExpNormalBasis.forward
 * src/mlcg/nn/radial_basis/exp_normal.py:104-124, CosineCutoff.forward src/mlcg/nn/cutoff.py:110-153.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int kind;         /* 0 Gaussian: exp(p1[0]*(d-p0[k])^2); 1 exp-normal: exp(-p1[k]*(exp(alpha*(lower-d))-p0[k])^2) */
    int num_rbf;      /* R */
    int cutoff_kind;  /* 0 identity, 1 cosine */
    int reserved;
    double lower, upper; /* envelope bounds */
    double alpha;        /* exp-normal only: 5/(upper-lower) */
    const void *p0;      /* [R] offsets | means (device) */
    const void *p1;      /* [1] coeff   | [R] betas (device) */
} mlcgb_rbf_spec;

/* out[e,k] = d^order/dd^order ( basis_k(d_e) * envelope(d_e) ), order 0..3 */
int mlcgb_rbf_expand(const void *d /* [E] */, int dtype, int64_t E, const mlcgb_rbf_spec *spec /* host */, int order,
                     void *out /* [E,R] */, void *stream);
/* s[e] = sum_k G[e,k] * d^order/dd^order( basis_k * envelope )(d_e) */
int mlcgb_rbf_contract(const void *d, const void *G /* [E,R] */, int dtype, int64_t E, const mlcgb_rbf_spec *spec,
                       int order, void *s /* [E] */, void *stream);
/* Gradients with respect to the basis parameters, which the reference trains by default (ExpNormalBasis(trainable=True),
 * src/mlcg/nn/radial_basis/exp_normal.py:52,80-94; GaussianBasis(trainable=True), gaussian.py:64-75):
 *   gp0[k] = sum_e c[e] G[e,k] d/dp0_k [ d^order/dd^order( basis_k * envelope )(d_e) ]      (offsets | means)
 *   gp1[k] = the same for p1                                                                (betas; Gaussian: gp1[0], the shared coeff)
 * c may be NULL (all ones).  order 0..3, num_rbf <= 256.  Sums are formed block by block and added in a fixed order (no atomics).
 * workspace: mlcgb_rbf_param_workspace_bytes(E, num_rbf, dtype) bytes. */
size_t mlcgb_rbf_param_workspace_bytes(int64_t E, int num_rbf, int dtype);
int mlcgb_rbf_param_contract(const void *d /* [E] */, const void *G /* [E,R] */, const void *c /* [E] or NULL */, int dtype, int64_t E,
                             const mlcgb_rbf_spec *spec, int order, void *workspace, size_t workspace_bytes, void *gp0 /* [R] */,
                             void *gp1 /* [R] | [1] */, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Continuous-filter convolution primitives.  CFConv.forward / .message, src/mlcg/nn/schnet.py:312-368:
 * x_j = x[edge_index[0]], message x_j * W, sum at edge_index[1].  Forward, backward and double
 * backward are all instances of these two kernels with the roles of the index rows exchanged.
 * ---------------------------------------------------------------------------------------------- */
/* out[n,:] = sum_{k in [ptr[n],ptr[n+1])} a[nbr[k],:] * V[eperm ? eperm[k] : k, :]   (ordered, no atomics) */
int mlcgb_seg_mul_sum(const void *a /* [Na,F] */, const void *V /* [E,F] */, int dtype, const int64_t *ptr /* [N+1] */,
                      const int32_t *nbr /* [E] */, const int32_t *eperm /* [E] or NULL */, int64_t N, int64_t E,
                      int64_t F, void *out /* [N,F] */, void *stream);
/* V[e,:] = a[ia[e],:] * b[ib[e],:] */
int mlcgb_edge_mul(const void *a, const void *b, int dtype, const int32_t *ia, const int32_t *ib, int64_t E, int64_t F,
                   void *V /* [E,F] */, void *stream);
/* V[p,:] = a[ia[p],:] * b[ib[p],:] + a[ib[p],:] * b[ia[p],:]: on a symmetric edge list the filter depends on the pair's distance
 * only (W = net(rbf(d)) * C(d), src/mlcg/nn/schnet.py:340-341), so it can be kept once per unordered pair; this is the
 * gradient of the aggregation (mlcgb_seg_mul_sum with eperm = the edge -> pair index) with respect to such a row. */
int mlcgb_pair_mul(const void *a, const void *b, int dtype, const int32_t *ia /* [P] */, const int32_t *ib /* [P] */, int64_t P,
                   int64_t F, void *V /* [P,F] */, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Filter-generating network GEMMs.  MLP([R,F,F]) built at src/mlcg/nn/schnet.py:446-450 and run by
 * src/mlcg/nn/mlp.py:56-58 (torch.nn.Linear -> cuBLAS in the reference).  fp32/fp64 accumulate.
 *   mode 0 (NT): C[M,N] = A[M,K] * B[N,K]^T (+ bias[N])      forward of a Linear layer
 *   mode 1 (NN): C[M,N] = A[M,K] * B[K,N]                    gradient w.r.t. the layer input
 *   mode 2 (TN): C[M,N] = A[K,M]^T * B[K,N]                  gradient w.r.t. the weight (K = edges)
 * `workspace` is only used by mode 2 (split over K); size from mlcgb_gemm_workspace_bytes.
 * ---------------------------------------------------------------------------------------------- */
size_t mlcgb_gemm_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K, int dtype);
int mlcgb_gemm(int mode, const void *A, const void *B, const void *bias /* [N] or NULL */, int dtype, int64_t M,
               int64_t N, int64_t K, void *C, void *workspace, size_t workspace_bytes, void *stream);

/* The same three GEMMs on the tensor cores (tcgen05, fp16 hi/lo pairs, three products per GEMM, fp32
 * accumulation in tensor memory): float32 only, the two weight-sized dimensions at most 128 (modes 0/1: N, K <= 128,
 * M = edges; mode 2: M, N <= 128, K = edges).  mlcgb_gemm_tc_supported tells whether a shape qualifies;
 * status bit 3 reports a tensor-core wait that ran out, bit 4 a weight beyond the range of the fp16-pair operands
 * (|w| > 512: the result is then not to be used; mlcgb_gemm computes such layers on the CUDA cores). */
int mlcgb_gemm_tc_supported(int mode, int64_t M, int64_t N, int64_t K);
size_t mlcgb_gemm_tc_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K);
int mlcgb_gemm_tc(int mode, const void *A, const void *B, const void *bias, int64_t M, int64_t N, int64_t K, void *C,
                  void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/* Mode 2 together with the column sums of A: C[M,N] = A[K,M]^T B[K,N], colsum[M] = sum_k A[k,:] — the weight and bias
 * gradients of one Linear layer (torch.nn.Linear's backward) from one pass over the incoming gradient A.  Needs N % 4 == 0
 * and a 16-byte aligned B (MLCGB_E_LIMIT otherwise); workspace as for mode 2. */
int mlcgb_gemm_tc_tn_colsum(const void *A, const void *B, int64_t K, int64_t M, int64_t N, void *C, void *colsum /* [M] */,
                            void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/* Modes 0 and 1 of the above with the elementwise step that follows the Linear layer in an interaction block fused into
 * the store of C (src/mlcg/nn/schnet.py:252-262: activation after CFConv, Linear, and the residual sum at
 * schnet.py:150; their derivatives in the force pass).  `epilogue`:
 *   0  C = A op(B) + bias                      1  C = tanh(A op(B) + bias)
 *   2  C = A op(B) + bias + aux                3  C = (A op(B) + bias) * (1 - aux^2)      (aux = tanh output)
 *   4  C = A' op(B) + bias with A'[m,k] = aux[k] * (1 - A[m,k]^2), aux a vector [K]: the derivative of a tanh layer followed
 *      by a dot product with aux (the output network, src/mlcg/nn/schnet.py:157), applied as the input tile is read
 * `aux` is [M,N] like C for 2 and 3 (NULL for 0 and 1); C may alias aux.  Needs M >= 128, N and K multiples of four and 16-byte aligned
 * A, C and aux; MLCGB_E_LIMIT otherwise (use mlcgb_gemm_tc and separate elementwise steps). */
int mlcgb_gemm_tc_fused(int mode, const void *A, const void *B, const void *bias, const void *aux, int epilogue, int64_t M,
                        int64_t N, int64_t K, void *C, int32_t *status, void *stream);

/* Two of those layers chained in one kernel, all widths 128 (the row tile stays on the chip between the GEMMs): the tail of an
 * interaction block, src/mlcg/nn/schnet.py:252-262 with the residual sum at schnet.py:150, and its part of the force pass.
 *   backward = 0:  mid = tanh(A Wa^T + ba) -> mid_out [M,128];   C = aux + mid Wb^T + bb        (Wa, Wb as torch.nn.Linear stores them)
 *   backward = 1:  mid = (A Wa) * (1 - aux^2)  (not stored);      C = mid Wb                     (ba, bb, mid_out ignored)
 * aux [M,128]: the block's input x (forward) or the stored tanh output (backward).  16-byte aligned A, aux, C, mid_out
 * (MLCGB_E_LIMIT otherwise).  Same arithmetic as two calls of mlcgb_gemm_tc_fused. */
int mlcgb_gemm_tc_chain2(int backward, const void *A, const void *Wa, const void *ba, const void *Wb, const void *bb, const void *aux,
                         int64_t M, void *mid_out, void *C, int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Fused filter network on the tensor cores (tcgen05 / TMEM):
 *   W[e,:] = ( tanh( phi(d_e) A1^T + b1 ) A2^T ) * C(d_e)
 * i.e. rbf_layer -> filter_network -> cutoff of CFConv.forward, src/mlcg/nn/schnet.py:340-341 with the
 * basis of src/mlcg/nn/radial_basis (gaussian.py, exp_normal.py) evaluated in the GEMM prologue.  float32 in / out, F = 128,
 * R <= 128, tanh activation.  precision 0: fp32-equivalent products (fp16 hi/lo pairs, three tensor-core
 * products per GEMM, fp32 accumulation); precision 1: bf16 operands, one product.
 * status bit 3 is set if a tensor-core wait ran out (the output is then incomplete), bit 4 if a weight of the filter
 * network is beyond the range of the fp16-pair operands (|w| > 512, precision 0).
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_filter_forward(const void *d /* [.] */, int64_t rows, const int32_t *sel /* [rows] or NULL */,
                         const int32_t *twin /* [E] or NULL */, const mlcgb_rbf_spec *rbf /* host */, int conv_cutoff_kind,
                         double conv_lower, double conv_upper, const void *A1 /* [F,R] */, const void *b1 /* [F] */,
                         const void *A2 /* [F,F] */, int64_t F, int precision, void *W /* [E,F] or [rows,F] */,
                         void *h_save /* mlcgb_filter_hidden_bytes(rows) or NULL */, int32_t *status, void *stream);
/* `h_save`: where the hidden layer tanh(phi(d) A1^T + b1) of every computed row is kept for mlcgb_filter_backward (in the
 * kernels' own tile order; opaque to the caller).  What autograd keeps of the filter network's first layer in the reference
 * (src/mlcg/nn/mlp.py:56-58), here at 512 bytes per computed row. */
size_t mlcgb_filter_hidden_bytes(int64_t rows);
/* `rows` = E and sel = twin = NULL: row k is edge k.  For a symmetric edge list the filter of an edge equals that of its
 * reverse (same distance), so the caller may pass one edge per unordered pair in `sel` (rows = E/2).  With the
 * reverse-edge map `twin` (mlcgb_edge_twin) each computed row is written to both edges of W[E,F]; without it W has
 * `rows` rows and row k holds the filter of edge sel[k] and of its reverse (half the HBM traffic; the aggregation then
 * reads W through mlcgb_pair_index).  The backward below, given `sel` and `twin`, sums the two directions' incoming
 * gradients and returns the pair's gradient on the selected edge (zero on its twin). */

/* Backward of the above with respect to the distance, fused with the message product:
 *   gd[e] = sum_f gW[e,f] * dW[e,f]/dd_e,  gW[e,:] = xl[row0[e],:] * gagg[row1[e],:]
 * (the gradient CFConv's aggregation, src/mlcg/nn/schnet.py:346,350-368, sends back to its filters).
 * With `h_saved` (what mlcgb_filter_forward left in `h_save` for the same d, rows, sel and weights): two tensor-core GEMMs per
 * tile, two tiles in flight, nothing recomputed.  With h_saved = NULL the forward is recomputed per tile (four GEMMs) and
 * nothing edge-sized is read or written in HBM except d, the two index rows and gd. */
int mlcgb_filter_backward(const void *d, int64_t rows, const int32_t *sel, const int32_t *twin, const mlcgb_rbf_spec *rbf,
                          int conv_cutoff_kind, double conv_lower, double conv_upper, const void *A1, const void *b1, const void *A2,
                          int64_t F, int precision, const int32_t *row0, const int32_t *row1, const void *xl /* [N,F] */,
                          const void *gagg /* [N,F] */, int64_t N, const void *h_saved /* or NULL */, void *gd /* [E] */,
                          int32_t *status, void *stream);

/* The product of the filter network's output with the per-edge cutoff, W = net(rbf) * C[:, None]
 * (src/mlcg/nn/schnet.py:341), and the contraction its derivatives need:
 *   row_scale: out[e,:] = a[e,:] * c[e]          row_dot: out[e] = sum_f a[e,f] * b[e,f] */
int mlcgb_row_scale(const void *a /* [E,F] */, const void *c /* [E] */, int dtype, int64_t E, int64_t F, void *out /* [E,F] */,
                    void *stream);
int mlcgb_row_dot(const void *a /* [E,F] */, const void *b /* [E,F] */, int dtype, int64_t E, int64_t F, void *out /* [E] */,
                  void *stream);
/* The derivative of the tanh activation (src/mlcg/nn/schnet.py:252-262, 446-450) given its output y, over n elements:
 *   mode 0: out = g * (1 - y^2)   (first derivative: the force pass)       mode 1: out = -2 * G * g * y   (its derivative with
 * respect to y: the second-order pass of force matching).  G is ignored in mode 0. */
int mlcgb_tanh_grad(int mode, const void *G, const void *g, const void *y, int dtype, int64_t n, void *out, void *stream);

/* ------------------------------------------------------------------------------------------------
 * One interaction block per call (eval mode, symmetric edge list, float32, 128 filters):
 *   x_new = x + lin( tanh( lin2( sum_j lin1(x)_j * W(d_ij) ) ) )     src/mlcg/nn/schnet.py:150, 252-262, 340-350
 * forward  = mlcgb_gemm_tc_fused (lin1) -> mlcgb_filter_forward (one row per pair) -> mlcgb_seg_mul_sum ->
 *            mlcgb_gemm_tc_fused (lin2 + tanh) -> mlcgb_gemm_tc_fused (lin + residual);
 * backward = the force pass through the same block: gx (gradient w.r.t. x, residual branch included; skipped if NULL)
 *            and gd (gradient w.r.t. the distances; skipped if NULL) from g = dE/dx_new.
 * They exist so that a host pays one foreign call per block and direction: for small systems the evaluation time is the
 * launch path.  W1 [F,H] (no bias), fA1 [F,R], fb1 [F], fA2 [F,F] the filter network, W2 [H2,F], b2, W3 [H,H2], b3.
 * sel [P] one edge per unordered pair, pair_of [E] (mlcgb_pair_index), twin [E] (mlcgb_edge_twin), ptr_out / nbr_out the
 * CSR of the centre-sorted list.  xl [N,F], Wp [P,F], a [N,H2] and hsave (mlcgb_filter_hidden_bytes(P) bytes, or NULL: the
 * backward then recomputes the filter network's hidden layer) are written by the forward and read by the backward; agg,
 * gy, gagg, gxl are scratch of the shapes [N,F], [N,H2], [N,F], [N,F].  MLCGB_E_LIMIT when N < 128 or a width is not a
 * multiple of four / beyond 128 (use the individual entry points then).
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_interaction_forward(const void *x, const void *d, const int64_t *ptr_out, const int32_t *nbr_out, const int32_t *sel,
                              const int32_t *pair_of, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower,
                              double conv_upper, const void *W1, const void *fA1, const void *fb1, const void *fA2, const void *W2,
                              const void *b2, const void *W3, const void *b3, int64_t N, int64_t E, int64_t P, int64_t H, int64_t F,
                              int64_t H2, int precision, void *xl, void *Wp, void *hsave, void *agg, void *a, void *out,
                              int32_t *status, void *stream);
int mlcgb_interaction_backward(const void *g, const void *a, const void *Wp, const void *xl, const void *hsave, const void *d, const int64_t *ptr_out,
                               const int32_t *nbr_out, const int32_t *sel, const int32_t *pair_of, const int32_t *twin,
                               const int32_t *row0, const int32_t *row1, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind,
                               double conv_lower, double conv_upper, const void *W1, const void *fA1, const void *fb1,
                               const void *fA2, const void *W2, const void *W3, int64_t N, int64_t E, int64_t P, int64_t H, int64_t F,
                               int64_t H2, int precision, void *gy, void *gagg, void *gxl, void *gx, void *gd, int32_t *status,
                               void *stream);

/* ------------------------------------------------------------------------------------------------
 * The whole evaluation of a SchNet with the standard layout in one call: embedding, interaction blocks, output network
 * MLP([H, head_width, 1]) with tanh, per-structure energy sum (src/mlcg/nn/schnet.py:116-162) and, if grad_pos is given,
 * d(sum of energies)/d(pos) (what GradientsOut differentiates, src/mlcg/nn/gradients.py:191-230; forces are its negative).
 * Same kernels as the per-block entry points; float32, symmetric centre-sorted edge list with its pair selection, pair
 * index and reverse-edge map, N >= 128, widths multiples of four and at most 128, 128 filters (MLCGB_E_LIMIT otherwise).
 * All weight pointers are device pointers; the two structs live on the host.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    const void *lin1_w;                            /* [F,H], no bias       CFConv.lin1 */
    const void *filter_w1, *filter_b1, *filter_w2; /* [F,R], [F], [F,F]    CFConv.filter_network */
    const void *lin2_w, *lin2_b;                   /* [H2,F], [H2]         CFConv.lin2 */
    const void *lin_w, *lin_b;                     /* [H,H2], [H]          InteractionBlock.lin */
} mlcgb_schnet_block;

typedef struct {
    int64_t hidden, filters, conv_out, head_width; /* H, F, H2, width of the output network's hidden layer */
    int64_t num_blocks, num_types;
    const mlcgb_schnet_block *blocks;              /* host array [num_blocks] */
    const void *embedding;                         /* [num_types, H] */
    const void *head_W, *head_b;                   /* [head_width, H], [head_width] */
    const void *head_out, *head_out_b;             /* [head_width], [1] or NULL */
} mlcgb_schnet_weights;

size_t mlcgb_schnet_eval_workspace_bytes(int64_t N, int64_t E, int64_t P, int64_t H, int64_t F, int64_t H2, int64_t head_width,
                                         int64_t num_blocks);
int mlcgb_schnet_eval(const void *pos /* [N,3] */, const int64_t *types /* [N] */, const int64_t *struct_ptr /* [B+1] */, int64_t N,
                      int64_t B, const int32_t *row0, const int32_t *row1, const int64_t *offsets /* [N+1] */,
                      const int32_t *sel /* [P] */, const int32_t *pair_of /* [E] */, const int32_t *twin /* [E] */, int64_t E,
                      int64_t P, const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper,
                      const mlcgb_schnet_weights *weights, int precision, void *workspace, size_t workspace_bytes,
                      void *energy /* [B] */, void *grad_pos /* [N,3] or NULL */, int32_t *status, void *stream);

/* out[b] = sum_{n in [ptr[b],ptr[b+1])} x[n]  — the per-structure energy sum, src/mlcg/nn/schnet.py:158 */
int mlcgb_segment_sum(const void *x /* [N] */, int dtype, const int64_t *ptr /* [B+1] */, int64_t B, void *out /* [B] */,
                      void *stream);

/* ------------------------------------------------------------------------------------------------
 * Radius graph of periodic structures, torch_neighbor_list_pbc + compute_images,
 * src/mlcg/neighbor_list/torch_impl.py:102-163, 252-329: neighbours are (point j, periodic shift); per centre they are listed
 * in the reference's order (shift triples (s1,s2,s3) in [-n_k, n_k] with s3 running fastest, points in order), cut after
 * max_nn, the pair (j = i, zero shift) dropped afterwards unless `loop`.  cells is [B,3,3] (rows = cell vectors), repeats
 * [B,3] int32 = n_k (zero along non-periodic directions).  Outputs: edge_index [2,E] (row 0 = centre), cell_shifts [E,3]
 * (the shift in length units, as compute_distances adds it to pos[j]), optional distance [E] and mapping_batch [E].
 * Two calls around one host read of offsets[N], like mlcgb_radius_count / mlcgb_radius_fill; the fill call takes the
 * workspace as the count call left it.  Status bit 0: a centre reached max_nn.
 * ---------------------------------------------------------------------------------------------- */
size_t mlcgb_radius_pbc_workspace_bytes(int64_t N);
int mlcgb_radius_pbc_count(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, const void *cells, const int32_t *repeats,
                           double r, int64_t max_nn, int loop, void *workspace, size_t workspace_bytes, int32_t *deg, int64_t *offsets,
                           int32_t *status, void *stream);
int mlcgb_radius_pbc_fill(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, const void *cells, const int32_t *repeats,
                          double r, int64_t max_nn, int loop, const void *workspace, size_t workspace_bytes, const int64_t *offsets,
                          int64_t E, int64_t *edge_index, void *cell_shifts, void *distance /* or NULL */,
                          int64_t *mapping_batch /* or NULL */, int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Capacity mode: the whole evaluation without a host read of the edge count, so that a molecular-dynamics step can be
 * recorded into a CUDA graph (the reference reads the count on the host in every step, radius.cu:288).
 *
 * mlcgb_radius_graph_capacity = mlcgb_radius_count + mlcgb_radius_fill into buffers of `capacity` edges: offsets beyond the
 * capacity are clamped, so at most `capacity` edges are written, and status bit 5 (32) reports the overflow (the list is
 * then incomplete).  counts[0] = edges written, counts[1] = counts[0] / 2, both in device memory.  edge_index ([2,capacity]
 * int64) may be NULL when only the int32 rows are wanted.
 *
 * The *_counted entry points take such a device-side count next to the host-side size: the host-side size is the capacity of
 * the buffers and sizes the launch, the kernels work on min(size, *count) rows.  Index arrays must hold valid indices
 * (e.g. zero) in their unused tail.  mlcgb_pair_plan reads the edge count from offsets[N], so it needs no extra argument.
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_radius_graph_capacity(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int64_t max_nn,
                                int loop, int rule, void *workspace, size_t workspace_bytes, int32_t *deg /* [N] */,
                                int64_t *offsets /* [N+1] */, int64_t capacity, int64_t *edge_index /* [2,capacity] or NULL */,
                                int32_t *row0_i32 /* [capacity] */, int32_t *row1_i32 /* [capacity] */, int64_t *counts /* [2] */,
                                int32_t *status, void *stream);
int mlcgb_filter_forward_counted(const void *d, int64_t E, const int64_t *rows_dev, const int32_t *sel, const int32_t *twin,
                                 const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper, const void *A1,
                                 const void *b1, const void *A2, int64_t F, int precision, void *W, void *h_save, int32_t *status,
                                 void *stream);
int mlcgb_filter_backward_counted(const void *d, int64_t E, const int64_t *rows_dev, const int32_t *sel, const int32_t *twin,
                                  const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper, const void *A1,
                                  const void *b1, const void *A2, int64_t F, int precision, const int32_t *row0, const int32_t *row1,
                                  const void *xl, const void *gagg, int64_t N, const void *h_saved, void *gd,
                                  int accumulate /* 1: add to gd (same rows as the call that set it) instead of setting it */,
                                  int32_t *status, void *stream);
int mlcgb_schnet_eval_counted(const void *pos, const int64_t *types, const int64_t *struct_ptr, int64_t N, int64_t B,
                              const int32_t *row0, const int32_t *row1, const int64_t *offsets, const int32_t *sel,
                              const int32_t *pair_of, const int32_t *twin, int64_t E, int64_t P, const int64_t *counts /* [2] or NULL */,
                              const mlcgb_rbf_spec *rbf, int conv_cutoff_kind, double conv_lower, double conv_upper,
                              const mlcgb_schnet_weights *weights, int precision, void *workspace, size_t workspace_bytes,
                              void *energy, void *grad_pos, int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Prior energy terms with analytic gradients.  `kind`:
 *   0 bond      k (d - x0)^2                       src/mlcg/nn/prior/harmonic.py:110-120,229-242
 *   1 angle     k (cos(theta) - x0)^2              src/mlcg/nn/prior/harmonic.py:284-297
 *   2 dihedral  v0 + sum_n k1_n sin(n phi) + k2_n cos(n phi)   src/mlcg/nn/prior/fourier_series.py:105-198
 *   3 repulsion (sigma/d)^6                        src/mlcg/nn/prior/repulsion.py:88-140
 * `mapping` is [order, M] int64 as the neighbour-list dictionary holds it; `params` is [P, M] with one
 * row per parameter (bond/angle: x0,k; dihedral: v0,k1_1..k1_n,k2_1..k2_n; repulsion: sigma).
 * energy[B] and grad[N,3] (= dE/dpos, not its negative) are ACCUMULATED into: zero them first.
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_prior_terms(int kind, const void *pos /* [N,3] */, int dtype, const int64_t *mapping, const int64_t *mapping_batch,
                      const void *params, int n_params, int64_t M, int64_t N, int64_t B, void *energy /* [B] */,
                      void *grad /* [N,3] or NULL */, int32_t *status, void *stream);

/* Every prior of a model in one launch (what SumOut.forward adds up one model at a time, src/mlcg/nn/gradients.py:111-117, over
 * the flat per-term parameters that condense_all_priors_for_simulation prepares, src/mlcg/simulation/specialize_prior.py:75-206).
 * Each list has 32-bit indices idx [order, M], per-term parameters params [n_params, M] as for mlcgb_prior_terms, and its own
 * row of energy [n_lists, B] and block of grad [n_lists, N, 3]; the structure of a term is struct_of[its first bead].
 * `symmetric` (pair kinds only): the list holds (j, i) for every (i, j), as mlcg's fully connected lists do
 * (src/mlcg/geometry/topology.py:131-135); the gradient of bead i is then formed from i's own terms alone (twice their sum)
 * and nothing is scattered to the second bead; with `run_ptr` (lists grouped by first bead, as those lists are) a warp takes a
 * whole run and adds once per bead, otherwise the reduction runs over what a warp happens to hold.  fixed_point = 0: energy and grad are ACCUMULATED into with floating-point
 * atomics (zero them first; the order of the additions, and so the last bits, vary from run to run).  fixed_point = 1:
 * sums are formed as 64-bit fixed-point integers in `workspace` (mlcgb_prior_eval_workspace_bytes) and then WRITTEN to energy and
 * grad: bit-identical from run to run, resolution 2^-36, magnitudes up to 1.3e8. */
#define MLCGB_MAX_PRIOR_SEGMENTS 8
typedef struct {
    int kind, n_params, symmetric, reserved;
    int64_t M;
    const int32_t *idx;
    const void *params;
    const int64_t *run_ptr; /* NULL, or [n_runs + 1]: the terms [run_ptr[k], run_ptr[k+1]) of a symmetric list share their first bead */
    int64_t n_runs;
} mlcgb_prior_list;
size_t mlcgb_prior_eval_workspace_bytes(int n_lists, int64_t N, int64_t B, int fixed_point);
int mlcgb_prior_eval(int n_lists, const mlcgb_prior_list *lists /* host */, const void *pos /* [N,3] */, int dtype,
                     const int32_t *struct_of /* [N] */, int64_t N, int64_t B, void *energy /* [n_lists,B] */,
                     void *grad /* [n_lists,N,3] */, int fixed_point, void *workspace, size_t workspace_bytes, int32_t *status,
                     void *stream);

/* ------------------------------------------------------------------------------------------------
 * BAOAB Langevin step around the force evaluation, LangevinSimulation.timestep,
 * src/mlcg/simulation/langevin.py:100-144.  x, v are updated in place; `noise` holds the normal deviates
 * (drawn by the caller, so the random stream is the reference's); beta_mass_ratio[n] = sqrt(1/(beta_n m_n))
 * (langevin.py:176-180); vscale = exp(-dt*friction), noisescale = sqrt(1 - vscale^2) (langevin.py:74-76).
 * ---------------------------------------------------------------------------------------------- */
int mlcgb_langevin_first_half(void *x /* [N,3] */, void *v /* [N,3] */, const void *f /* [N,3] */, const void *masses /* [N] */,
                              const void *beta_mass_ratio /* [N] */, const void *noise /* [N,3] */, int dtype, int64_t N, double dt,
                              double vscale, double noisescale, void *stream);
int mlcgb_langevin_second_half(void *v, const void *f, const void *masses, int dtype, int64_t N, double dt, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MLCG_B200_H */
