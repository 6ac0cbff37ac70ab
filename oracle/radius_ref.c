/*
 * TEST INFRASTRUCTURE — CPU oracle for the radius graph. Not part of the product:
 * only the tests, the smoke check and the bench's CPU-baseline leg may load this.
 *
 * Restates the edge rule of the reference's radius graph:
 *   - mlcg's own native kernel, src/opt_radius/mlcg_opt_radius/radius.cu:106-141
 *     (one query point scans every point of its own structure in index order, keeps a
 *     pair when the squared distance is strictly below r*r, optionally skips itself,
 *     stops after max_num_neighbors hits), with r*r rounded once to the scalar type
 *     (radius.cu:250);
 *   - torch_cluster.radius_graph (torch-cluster 1.6.3, not vendored), the call SchNet
 *     makes through src/mlcg/neighbor_list/torch_impl.py:216-224: the same scan, but
 *     when loops are excluded it searches with max_num_neighbors+1 hits *including*
 *     the point itself and removes the self pair afterwards.
 * Output order is what both produce: centre index ascending, neighbour index ascending.
 *
 * The squared distance is fma(dz, dz, fma(dy, dy, dx*dx)): the loop `dist += diff * diff`
 * of radius.cu:126-130 as nvcc compiles it with its default contraction into fused
 * multiply-adds (compile this file with -ffp-contract=off so that nothing else is fused).
 *
 * Parity status: PINNED.  The reference's kernel, compiled unmodified (oracle/build_ref.py),
 * was run on a B200 against this rule through the product's kernels on the reference's own
 * test grid, lattices, a 4 x 4000 cube, exclusion lists and pairs whose squared distance is
 * within one rounding of r*r (tests/test_gpu_radius_reference.py): the reference decides
 * every such pair as the fused form does, never as separately rounded operations would.
 * torch_cluster itself (not vendored, not installable here) stays unpinned; its CUDA kernel
 * has the same loop.  The numpy restatement in radius_ref.py emulates the fused operations
 * exactly and pins this file on the CPU (tests/test_oracle_radius.py).
 */
#include <stdint.h>
#include <math.h>
#include <stdlib.h>

#define RULE_NATIVE 0   /* radius.cu: skip self first, keep first max_nn hits        */
#define RULE_CLUSTER 1  /* torch_cluster: cap = max_nn+1 with self counted, drop self */

#define DEFINE_ORACLE(NAME, T, SQRT, FMA)                                                \
    static int64_t NAME##_centre(const T *pos, int64_t lo, int64_t hi, int64_t i, T r2, \
                                 int64_t max_nn, int loop, int rule, int64_t *oi,       \
                                 int64_t *oj, T *od) {                                   \
        const T xi = pos[3 * i], yi = pos[3 * i + 1], zi = pos[3 * i + 2];               \
        const int count_self = loop || rule == RULE_CLUSTER;                             \
        const int64_t cap = (!loop && rule == RULE_CLUSTER) ? max_nn + 1 : max_nn;       \
        int64_t hits = 0, kept = 0;                                                      \
        for (int64_t j = lo; j < hi && hits < cap; j++) {                                \
            const T dx = pos[3 * j] - xi, dy = pos[3 * j + 1] - yi,                      \
                    dz = pos[3 * j + 2] - zi;                                            \
            const T d2 = FMA(dz, dz, FMA(dy, dy, dx * dx));                              \
            if (!(d2 < r2)) continue;                                                    \
            if (j == i) {                                                                \
                if (!count_self) continue;                                               \
                hits++;                                                                  \
                if (!loop) continue; /* counted towards the cap, removed afterwards */   \
            } else {                                                                     \
                hits++;                                                                  \
            }                                                                            \
            if (oi) {                                                                    \
                oi[kept] = i;                                                            \
                oj[kept] = j;                                                            \
                if (od) od[kept] = SQRT(d2);                                             \
            }                                                                            \
            kept++;                                                                      \
        }                                                                                \
        return kept;                                                                     \
    }                                                                                    \
    /* deg[N] <- kept neighbours per centre; returns the total. */                       \
    int64_t NAME##_count(const T *pos, const int64_t *ptr, int64_t B, double r,          \
                         int64_t max_nn, int loop, int rule, int64_t *deg) {             \
        const T r2 = (T)(r * r);                                                         \
        int64_t total = 0;                                                               \
        _Pragma("omp parallel for schedule(dynamic, 1) reduction(+ : total)")           \
        for (int64_t b = 0; b < B; b++)                                                  \
            for (int64_t i = ptr[b]; i < ptr[b + 1]; i++) {                              \
                deg[i] = NAME##_centre(pos, ptr[b], ptr[b + 1], i, r2, max_nn, loop,     \
                                       rule, 0, 0, 0);                                   \
                total += deg[i];                                                         \
            }                                                                            \
        return total;                                                                    \
    }                                                                                    \
    /* off[N] = exclusive prefix sum of deg; writes edges in (centre, neighbour) order */\
    void NAME##_fill(const T *pos, const int64_t *ptr, int64_t B, double r,              \
                     int64_t max_nn, int loop, int rule, const int64_t *off,             \
                     int64_t *row0, int64_t *row1, T *dist) {                            \
        const T r2 = (T)(r * r);                                                         \
        _Pragma("omp parallel for schedule(dynamic, 1)")                                \
        for (int64_t b = 0; b < B; b++)                                                  \
            for (int64_t i = ptr[b]; i < ptr[b + 1]; i++)                                \
                NAME##_centre(pos, ptr[b], ptr[b + 1], i, r2, max_nn, loop, rule,        \
                              row0 + off[i], row1 + off[i], dist ? dist + off[i] : 0);   \
    }

DEFINE_ORACLE(radius_ref_f32, float, sqrtf, fmaf)
DEFINE_ORACLE(radius_ref_f64, double, sqrt, fma)

/*
 * exclusion_pairs.cpp:7-62 — sort pairs (x, y) by (y, x), return the xs and a CSR
 * pointer over y of length num_nodes+1, indexed by 0-based node as radius.cu:122-123 reads it.
 * For the input of the comment at exclusion_pairs.cpp:16-18, pairs [(2,1),(1,2),(3,2),(2,2),(2,3)]
 * with num_nodes 4, the code gives xs [2,1,2,3,2], ptr [0,0,1,4,5] (the numbers printed in that
 * comment are not what the code below it computes; the code is followed here).
 */
typedef struct { int64_t x, y; } pair_t;
static int pair_cmp(const void *a, const void *b) {
    const pair_t *p = (const pair_t *)a, *q = (const pair_t *)b;
    if (p->y != q->y) return p->y < q->y ? -1 : 1;
    if (p->x != q->x) return p->x < q->x ? -1 : 1;
    return 0;
}
int exclusion_pair_to_ptr_ref(const int64_t *pairs /* [2,P] row-major */, int64_t P,
                              int64_t num_nodes, int64_t *xs, int64_t *y_ptr) {
    pair_t *buf = (pair_t *)malloc((size_t)(P > 0 ? P : 1) * sizeof(pair_t));
    if (!buf) return -1;
    for (int64_t k = 0; k < P; k++) { buf[k].x = pairs[k]; buf[k].y = pairs[P + k]; }
    qsort(buf, (size_t)P, sizeof(pair_t), pair_cmp);
    int64_t k = 0;
    y_ptr[0] = 0;
    for (int64_t n = 0; n < num_nodes; n++) {
        while (k < P && buf[k].y == n) k++;
        y_ptr[n + 1] = k;
    }
    for (int64_t q = 0; q < P; q++) xs[q] = buf[q].x;
    free(buf);
    return 0;
}
