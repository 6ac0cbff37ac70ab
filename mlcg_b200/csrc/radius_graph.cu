// Radius graph for batches of independent structures (non-periodic), sm_100a.
//
// Output contract (same as torch_cluster.radius_graph(flow="target_to_source") and mlcg::radius_cuda):
// edges (centre i, neighbour j), both in the same structure, squared distance strictly below r*r,
// centre-major with neighbours in ascending index order, at most max_num_neighbors per centre.
//
// Plan:  build_cells (one CTA per large structure: bounding box, cell grid with cells of half the cutoff
//        where the structure has points enough, counting sort of the points by cell, all counters in
//        shared memory; the size of the blocks of cells the block kernels work on)
//     -> neighbours_block_count for structures of up to 8192 points with a cell grid: a warp takes a
//        block of cells of one layer (about 24 centres), stages every point within reach of the block
//        in shared memory once, in ascending order of index, and each lane tests its centre against
//        the whole staged list; the hits, a bit per staged candidate, stay in the workspace;
//        neighbours<COUNT> for the rest (one warp per centre over the rows of cells within reach, each
//        row a contiguous run of cell-sorted points; small structures scan all their points instead)
//     -> exclusive scan of the degrees (three small kernels, no spin-waits)
//     -> [host reads E] -> neighbours_block_expand (the same blocks: the kept bits become edges, in
//        the order the edges are listed in, without another distance test), neighbours_block_fill for
//        the blocks with more candidates than a stage holds (tested again, two warps per block; it
//        leaves at once when there are none), and neighbours<FILL> (hits are marked in a bitmask in
//        shared memory indexed by local point index, per centre, then emitted in ascending order).
#include "common.cuh"

#include <atomic>

namespace mlcgb {

#ifdef MLCGB_PHASE_TIMING
__device__ unsigned long long g_radius_phase_cycles[16];
#define RPHASE_DECL long long ph_last = clock64();
#define RPHASE(k)                                                                  \
    if (threadIdx.x == 0) {                                                        \
        const long long ph_now = clock64();                                        \
        atomicAdd(&g_radius_phase_cycles[k], (unsigned long long)(ph_now - ph_last)); \
        ph_last = clock64();                                                       \
    }
#else
#define RPHASE_DECL
#define RPHASE(k)
#endif

constexpr int kBruteMax = 384;     // structures up to this size scan all their points
constexpr int kSmemCells = 8192;   // upper bound on cells per structure (shared-memory counters)
constexpr int kNbrWarps = 8;       // warps per CTA in the neighbour kernels
constexpr int kCapBits = 8192;     // bitmask window per warp (local point indices per pass)
constexpr int kBuildThreads = 512;
constexpr int kScanBlock = 1024;

// Cell grid of one structure.  reach: cells to either side that can hold a neighbour (1: cell edge >= cutoff, 2: >= half
// of it); tile: handled by the block kernels (ngroups work items: blocks of bx x by cells, pad = bx | by << 8, in every
// layer), else by the warp kernels.
struct CellParam { int gx, gy, gz, use_cells, reach, tile, ngroups, pad; };

constexpr int kHitWordsF32 = 24, kHitWordsF64 = 12;          // block kernels: words of a centre's hit mask (= staged candidates / 32)
constexpr int kBlkMaxBY = 8;                               // block kernels: rows of cells in a block, at most
constexpr int kBlkTargetCentres = 24;                      // mean number of centres per block the block's size aims at

template <typename T> using V4 = typename Vec4<T>::type;

__device__ __forceinline__ int idx_of(const float4 &p) { return __float_as_int(p.w); }
__device__ __forceinline__ int idx_of(const double4 &p) { return (int)__double_as_longlong(p.w); }
__device__ __forceinline__ float4 make_v4(float x, float y, float z, int i) { return make_float4(x, y, z, __int_as_float(i)); }
__device__ __forceinline__ double4 make_v4(double x, double y, double z, int i) {
    return make_double4(x, y, z, __longlong_as_double((long long)i));
}

struct WsLayout {
    size_t spos, cellparam, cell_of, cell_start, struct_of, bsum, group_ptr, hits, cidx, item_flag, total;
};
static inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
static WsLayout ws_layout(int64_t N, int64_t B, int dtype) {
    WsLayout L;
    size_t v4 = dtype == MLCGB_F64 ? 32 : 16;
    size_t o = 0;
    L.spos = o;        o += align256((size_t)N * v4);
    L.cellparam = o;   o += align256((size_t)B * sizeof(CellParam));
    L.cell_of = o;     o += align256((size_t)N * 4);
    L.cell_start = o;  o += align256((size_t)(N + B) * 4);
    L.struct_of = o;   o += align256((size_t)N * 4);
    L.bsum = o;        o += align256((size_t)((N + kScanBlock - 1) / kScanBlock + 1) * 8);
    L.group_ptr = o;   o += align256((size_t)(B + 3) * 4);
    L.hits = o;        o += align256((size_t)N * (dtype == MLCGB_F64 ? kHitWordsF64 : kHitWordsF32) * 4);   // hit words per point
    L.cidx = o;        o += align256((size_t)N * 4);                      // local index of every cell-sorted point (= spos[].w, compact)
    L.item_flag = o;   o += align256((size_t)N);                          // per work item (at most one per cell, cells <= points): 1 = no hit masks
    L.total = o;
    return L;
}

// ------------------------------------------------------------------------------------------ build
template <typename T>
__global__ void __launch_bounds__(kBuildThreads)
build_cells_kernel(const T *__restrict__ pos, const int64_t *__restrict__ ptr, int64_t B, T rcut, int allow_tile,
                   V4<T> *__restrict__ spos, CellParam *__restrict__ cellparam, int32_t *__restrict__ cell_of,
                   int32_t *__restrict__ cell_start, int32_t *__restrict__ struct_of, int32_t *__restrict__ cidx) {
    __shared__ int counts[kSmemCells + 1];
    __shared__ T red[6][kBuildThreads / 32];
    __shared__ T s_org[3];
    __shared__ T s_invh;
    __shared__ int s_g[3];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int64_t b = blockIdx.x; b < B; b += gridDim.x) {
        const int64_t lo = ptr[b];
        const int64_t n64 = ptr[b + 1] - lo;
        for (int64_t i = tid; i < n64; i += kBuildThreads) struct_of[lo + i] = (int32_t)b;   // structure of every point
        if (n64 <= kBruteMax) {
            if (tid == 0) cellparam[b] = CellParam{0, 0, 0, 0, 0, 0, 0, 0};
            continue;
        }
        const int n = (int)n64;
        // bounding box
        T mn[3] = {T(INFINITY), T(INFINITY), T(INFINITY)}, mx[3] = {T(-INFINITY), T(-INFINITY), T(-INFINITY)};
        for (int i = tid; i < n; i += kBuildThreads)
#pragma unroll
            for (int a = 0; a < 3; a++) {
                const T v = pos[(lo + i) * 3 + a];
                mn[a] = fmin(mn[a], v);
                mx[a] = fmax(mx[a], v);
            }
#pragma unroll
        for (int a = 0; a < 3; a++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                mn[a] = fmin(mn[a], __shfl_xor_sync(0xffffffffu, mn[a], o));
                mx[a] = fmax(mx[a], __shfl_xor_sync(0xffffffffu, mx[a], o));
            }
            if (lane == 0) { red[a][warp] = mn[a]; red[3 + a][warp] = mx[a]; }
        }
        __syncthreads();
        if (tid == 0) {
            double lo3[3], ext[3], extmax = 0.0;
            bool finite = true;
            for (int a = 0; a < 3; a++) {
                T m0 = red[a][0], m1 = red[3 + a][0];
                for (int w = 1; w < kBuildThreads / 32; w++) { m0 = fmin(m0, red[a][w]); m1 = fmax(m1, red[3 + a][w]); }
                lo3[a] = (double)m0;
                ext[a] = (double)m1 - (double)m0;
                if (!(ext[a] >= 0.0) || !isfinite(ext[a]) || !isfinite(lo3[a])) finite = false;
                if (ext[a] > extmax) extmax = ext[a];
            }
            int g[3] = {1, 1, 1};
            double h = 1.0, reach_len = 1.0;
            if (finite && rcut > T(0)) {
                // Reach: the cutoff plus a margin that covers every rounding between the pair test and the cell
                // assignment, so that two points passing the test are less than this apart along every axis.  Cells
                // start at half of it (a neighbour then sits at most two cells away, and fewer candidates are tested
                // per hit) and grow until the grid fits the counters.
                reach_len = (double)rcut * 1.001 + extmax * 1e-6 + 1e-30;
                h = 0.5 * reach_len;
                const int maxcells = n < kSmemCells ? n : kSmemCells;
                for (int it = 0; it < 64; it++) {
                    double prod = 1.0;
                    for (int a = 0; a < 3; a++) {
                        double ga = floor(ext[a] / h) + 1.0;
                        g[a] = ga > 2000000.0 ? 2000000 : (int)ga;
                        prod *= ga;
                    }
                    if (prod <= (double)maxcells) break;
                    h *= 1.2599210498948732;  // cbrt(2): halve the cell count per step
                }
                if ((double)g[0] * g[1] * g[2] > (double)maxcells) { g[0] = g[1] = g[2] = 1; }
            } else if (!finite) {
                lo3[0] = lo3[1] = lo3[2] = 0.0;
            }
            for (int a = 0; a < 3; a++) { s_org[a] = (T)lo3[a]; s_g[a] = g[a]; }
            s_invh = (T)(1.0 / h);
            // cells per reach, rounded up (the cell index is floor((x - origin) / h) with a rounded 1/h: one more cell of slack
            // is cheap next to a missed pair when h is within rounding of a whole fraction of the reach)
            int reach = (int)ceil(reach_len / h * (1.0 + 1e-9));
            if (!(finite && rcut > T(0))) reach = 1;
            if (reach > 2) reach = 2;                      // h >= reach_len / 2 by construction
            const int tile = allow_tile && n <= kCapBits;
            // block of cells per work item of the block kernels: about kBlkTargetCentres points, as square as the grid allows
            int bx = 1, by = 1;
            if (tile) {
                const double dens = (double)n / ((double)g[0] * g[1] * g[2]);
                int area = (int)floor(kBlkTargetCentres / dens + 0.5);
                if (area < 1) area = 1;
                bx = (int)floor(sqrt((double)area) + 0.5);
                bx = bx < 1 ? 1 : (bx > g[0] ? g[0] : bx);
                by = (area + bx - 1) / bx;
                const int by_max = g[1] < kBlkMaxBY ? g[1] : kBlkMaxBY;
                by = by > by_max ? by_max : by;
                if (bx * by < area) {
                    bx = (area + by - 1) / by;
                    bx = bx > g[0] ? g[0] : (bx > 255 ? 255 : bx);
                }
            }
            cellparam[b] = CellParam{g[0], g[1], g[2], 1, reach, tile, tile ? g[2] * ((g[1] + by - 1) / by) * ((g[0] + bx - 1) / bx) : 0, bx | (by << 8)};
        }
        __syncthreads();
        const int gx = s_g[0], gy = s_g[1], gz = s_g[2];
        const int ncell = gx * gy * gz;
        for (int c = tid; c <= ncell; c += kBuildThreads) counts[c] = 0;
        __syncthreads();
        const T ox = s_org[0], oy = s_org[1], oz = s_org[2], invh = s_invh;
        for (int i = tid; i < n; i += kBuildThreads) {
            const T x = pos[(lo + i) * 3], y = pos[(lo + i) * 3 + 1], z = pos[(lo + i) * 3 + 2];
            int cx = (int)floor((x - ox) * invh), cy = (int)floor((y - oy) * invh), cz = (int)floor((z - oz) * invh);
            cx = min(max(cx, 0), gx - 1);
            cy = min(max(cy, 0), gy - 1);
            cz = min(max(cz, 0), gz - 1);
            const int c = cx + gx * (cy + gy * cz);
            cell_of[lo + i] = c;
            atomicAdd(&counts[c], 1);
        }
        __syncthreads();
        // exclusive scan of counts[0..ncell) by warp 0: each lane owns a contiguous chunk
        if (warp == 0) {
            const int chunk = (ncell + 31) / 32;
            const int c0 = lane * chunk, c1 = min(c0 + chunk, ncell);
            int s = 0;
            for (int c = c0; c < c1; c++) s += counts[c];
            int incl = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            int run = incl - s;
            for (int c = c0; c < c1; c++) { int t = counts[c]; counts[c] = run; run += t; }
            if (lane == 31) counts[ncell] = incl;
        }
        __syncthreads();
        int32_t *cs = cell_start + lo + b;
        for (int c = tid; c <= ncell; c += kBuildThreads) cs[c] = counts[c];
        __syncthreads();
        for (int i = tid; i < n; i += kBuildThreads) {
            const int c = cell_of[lo + i];
            const int slot = atomicAdd(&counts[c], 1);
            spos[lo + slot] = make_v4(pos[(lo + i) * 3], pos[(lo + i) * 3 + 1], pos[(lo + i) * 3 + 2], i);
            cidx[lo + slot] = i;
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------- neighbours
struct FillOut {
    int64_t *row0, *row1, *mapping_batch;
    void *distance;
    int32_t *row0_32, *row1_32;
};

template <typename T>
__device__ __forceinline__ void emit_edge(const FillOut &o, int64_t slot, int64_t i, int64_t j, int64_t b, T d2) {
    if (o.row0) {
        o.row0[slot] = i;
        o.row1[slot] = j;
    }
    if (o.mapping_batch) o.mapping_batch[slot] = b;
    if (o.distance) ((T *)o.distance)[slot] = sqrt(d2);
    if (o.row0_32) o.row0_32[slot] = (int32_t)i;
    if (o.row1_32) o.row1_32[slot] = (int32_t)j;
}

// Pairs never to be listed (radius.cu:112-133): xs[ptr[i] .. ptr[i+1]) holds, in ascending order, the neighbours that
// centre i must not get.  Both pointers NULL: nothing is excluded.
struct Exclusion {
    const int64_t *xs = nullptr, *ptr = nullptr;
};
__device__ __forceinline__ bool is_excluded(const int64_t *__restrict__ xs, int64_t e0, int64_t e1, int64_t j) {
    while (e0 < e1) {                                  // binary search in the centre's sorted segment
        const int64_t mid = (e0 + e1) >> 1;
        const int64_t v = xs[mid];
        if (v == j) return true;
        if (v < j) e0 = mid + 1; else e1 = mid;
    }
    return false;
}

// EXCL: compiled with the exclusion test (kept out of the plain kernels, whose inner loop is issue-bound)
template <typename T, bool FILL, bool EXCL>
__global__ void __launch_bounds__(kNbrWarps * 32)
neighbours_kernel(const T *__restrict__ pos, const int64_t *__restrict__ ptr, int64_t N, int64_t B, T r2,
                  int64_t max_nn, int loop, int rule, const V4<T> *__restrict__ spos,
                  const CellParam *__restrict__ cellparam, const int32_t *__restrict__ cell_of,
                  const int32_t *__restrict__ cell_start, const int32_t *__restrict__ struct_of, int32_t *__restrict__ deg,
                  const int64_t *__restrict__ offsets, FillOut out, Exclusion ex, int32_t *__restrict__ status,
                  const int32_t *__restrict__ n_plain) {
    if (n_plain && *n_plain == 0) return;          // every structure belongs to the block kernels
    __shared__ unsigned s_mask[FILL ? kNbrWarps * (kCapBits / 32) : 1];
    __shared__ unsigned short s_list[FILL ? kNbrWarps * 1024 : 1];   // per warp: bit positions of one 32-word chunk
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned *mask = s_mask + (FILL ? warp * (kCapBits / 32) : 0);
    unsigned short *list = s_list + (FILL ? warp * 1024 : 0);
    const unsigned lt = lanemask_lt();

    for (int64_t i = (int64_t)blockIdx.x * kNbrWarps + warp; i < N; i += (int64_t)gridDim.x * kNbrWarps) {
        const int64_t b = struct_of[i];
        const int64_t lo = ptr[b];
        const int n = (int)(ptr[b + 1] - lo);
        const int il = (int)(i - lo);
        const int64_t ex0 = EXCL ? ex.ptr[i] : 0, ex1 = EXCL ? ex.ptr[i + 1] : 0;   // this centre's excluded neighbours
        const CellParam cp = cellparam[b];
        if (cp.tile) continue;                       // this structure's centres belong to the block kernels
        const T xi = pos[i * 3], yi = pos[i * 3 + 1], zi = pos[i * 3 + 2];

        int64_t kept = 0, base_off = 0;
        if (FILL) {
            base_off = offsets[i];
            kept = offsets[i + 1] - base_off;
            if (kept == 0) continue;
        }
        int cnt_lo = 0, cnt_hi = 0;  // COUNT: hits with j < il / j > il (per lane)

        if (!cp.use_cells) {
            int64_t emitted = 0;
            for (int jb = 0; jb < n; jb += 32) {
                const int j = jb + lane;
                bool hit = false;
                T d2 = T(0);
                if (j < n) {
                    const int64_t gj = lo + j;
                    d2 = dist2_rn(xi, yi, zi, pos[gj * 3], pos[gj * 3 + 1], pos[gj * 3 + 2]);
                    hit = d2 < r2 && !(EXCL && ex1 > ex0 && is_excluded(ex.xs, ex0, ex1, gj));
                }
                if (FILL) {
                    hit = hit && (loop || j != il);
                    const unsigned bal = __ballot_sync(0xffffffffu, hit);
                    const int64_t rank = emitted + __popc(bal & lt);
                    if (hit && rank < kept) emit_edge<T>(out, base_off + rank, i, lo + j, b, d2);
                    emitted += __popc(bal);
                    if (emitted >= kept) break;
                } else if (hit) {
                    cnt_lo += (j < il);
                    cnt_hi += (j > il);
                }
            }
        } else {
            const int gx = cp.gx, gy = cp.gy, gz = cp.gz;
            const int c = cell_of[i];
            const int cx = c % gx, cy = (c / gx) % gy, cz = c / (gx * gy);
            const int reach = cp.reach, side = 2 * reach + 1, nrows = side * side;
            const int x0 = max(cx - reach, 0), x1 = min(cx + reach, gx - 1);
            const int32_t *cs = cell_start + lo + b;
            const V4<T> *sp = spos + lo;
            const int nwin = FILL ? (n + kCapBits - 1) / kCapBits : 1;
            int64_t emitted = 0;
            for (int win = 0; win < nwin; win++) {
                const int wbase = win * kCapBits;
                const int wbits = FILL ? min(kCapBits, n - wbase) : 0;
                const int nwords = (wbits + 31) >> 5;
                if (FILL) {
                    for (int w = lane; w < nwords; w += 32) mask[w] = 0u;
                    __syncwarp();
                }
                // the first lanes fetch the candidate run of one (dy, dz) row each (9 rows at reach 1, 25 at reach 2), so
                // the pairs of cell-start reads are in flight together; every lane then keeps two loads per row in flight
                int rk0 = 0, rk1 = 0;
                if (lane < nrows) {
                    const int yy = cy + lane % side - reach, zz = cz + lane / side - reach;
                    if (yy >= 0 && yy < gy && zz >= 0 && zz < gz) {
                        const int rowbase = gx * (yy + gy * zz);
                        rk0 = cs[rowbase + x0];
                        rk1 = cs[rowbase + x1 + 1];
                    }
                }
                auto test = [&](const V4<T> &p) {
                    const int j = idx_of(p);
                    const T d2 = dist2_rn(xi, yi, zi, p.x, p.y, p.z);
                    if (d2 < r2 && !(EXCL && ex1 > ex0 && is_excluded(ex.xs, ex0, ex1, lo + j))) {
                        if (FILL) {
                            const int jw = j - wbase;
                            if ((loop || j != il) && jw >= 0 && jw < wbits) atomicOr(&mask[jw >> 5], 1u << (jw & 31));
                        } else {
                            cnt_lo += (j < il);
                            cnt_hi += (j > il);
                        }
                    }
                };
                for (int row = 0; row < nrows; row++) {
                    const int k0 = __shfl_sync(0xffffffffu, rk0, row), k1 = __shfl_sync(0xffffffffu, rk1, row);
                    const int ka = k0 + lane, kb = ka + 32;
                    V4<T> pa, pb;
                    if (ka < k1) pa = sp[ka];
                    if (kb < k1) pb = sp[kb];
                    if (ka < k1) test(pa);
                    if (kb < k1) test(pb);
                    for (int k = kb + 32; k < k1; k += 32) test(sp[k]);
                }
                if (FILL) {
                    __syncwarp();
                    for (int w0 = 0; w0 < nwords; w0 += 32) {
                        const int w = w0 + lane;
                        unsigned bits = w < nwords ? mask[w] : 0u;
                        const int cbits = __popc(bits);
                        int incl = cbits;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const int t = __shfl_up_sync(0xffffffffu, incl, o);
                            if (lane >= o) incl += t;
                        }
                        const int total = __shfl_sync(0xffffffffu, incl, 31);
                        // compact the set bits of these 32 words into a dense list in shared memory ...
                        int pos_in = incl - cbits;
                        while (bits) {
                            const int t = __ffs(bits) - 1;
                            bits &= bits - 1;
                            list[pos_in++] = (unsigned short)(((w - w0) << 5) + t);
                        }
                        __syncwarp();
                        // ... and write the edges with consecutive lanes on consecutive slots
                        const int64_t room = kept - emitted;
                        const int take = (int64_t)total < room ? total : (int)room;
                        for (int t = lane; t < take; t += 32) {
                            const int j = wbase + (w0 << 5) + (int)list[t];
                            T d2 = T(0);
                            if (out.distance) {
                                const int64_t gj = lo + j;
                                d2 = dist2_rn(xi, yi, zi, pos[gj * 3], pos[gj * 3 + 1], pos[gj * 3 + 2]);
                            }
                            emit_edge<T>(out, base_off + emitted + t, i, lo + j, b, d2);
                        }
                        __syncwarp();
                        emitted += total;
                        if (emitted >= kept) break;
                    }
                    __syncwarp();
                    if (emitted >= kept) break;
                }
            }
        }

        if (!FILL) {
            const int64_t nlo = warp_sum(cnt_lo), nhi = warp_sum(cnt_hi);
            const int self_hit = (dist2_rn(xi, yi, zi, xi, yi, zi) < r2 && !(EXCL && ex1 > ex0 && is_excluded(ex.xs, ex0, ex1, i))) ? 1 : 0;
            int64_t total, k;
            if (loop) {
                total = nlo + nhi + self_hit;
                k = total < max_nn ? total : max_nn;
            } else if (rule == MLCGB_RULE_CLUSTER && self_hit) {
                total = nlo + nhi;
                if (nlo >= max_nn + 1) k = max_nn + 1;
                else k = total < max_nn ? total : max_nn;
            } else {
                total = nlo + nhi;
                k = total < max_nn ? total : max_nn;
            }
            if (lane == 0) {
                deg[i] = (int32_t)k;
                if (k < total) atomicOr(status, (int)kTruncated);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------- scan
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *s_warp, int64_t *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int64_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int64_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int64_t w = lane < nwarp ? s_warp[lane] : 0;
        int64_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int64_t t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        if (lane < nwarp) s_warp[lane] = wi - w;
        if (lane == 31) s_warp[32] = wi;
    }
    __syncthreads();
    const int64_t r = s_warp[warp] + incl - v;
    if (total) *total = s_warp[32];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(kScanBlock) scan_block_sums_kernel(const int32_t *deg, int64_t N, int64_t *bsum) {
    __shared__ int64_t s_warp[33];
    const int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
    int64_t total;
    block_exclusive_scan(i < N ? (int64_t)deg[i] : 0, s_warp, &total);
    if (threadIdx.x == 0) bsum[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanBlock) scan_of_sums_kernel(int64_t *bsum, int64_t nb, int64_t *grand_total) {
    __shared__ int64_t s_warp[33];
    int64_t carry = 0;
    for (int64_t c0 = 0; c0 < nb; c0 += kScanBlock) {
        const int64_t k = c0 + threadIdx.x;
        const int64_t v = k < nb ? bsum[k] : 0;
        int64_t total;
        const int64_t ex = block_exclusive_scan(v, s_warp, &total);
        if (k < nb) bsum[k] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) *grand_total = carry;
}

__global__ void __launch_bounds__(kScanBlock)
scan_apply_kernel(const int32_t *deg, int64_t N, const int64_t *bsum, int64_t *offsets) {
    __shared__ int64_t s_warp[33];
    const int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
    const int64_t ex = block_exclusive_scan(i < N ? (int64_t)deg[i] : 0, s_warp, nullptr);
    if (i < N) offsets[i] = bsum[blockIdx.x] + ex;
}

// inputs of at most one scan block: exclusive scan and grand total in one launch
__global__ void __launch_bounds__(kScanBlock) scan_single_block_kernel(const int32_t *deg, int64_t N, int64_t *offsets) {
    __shared__ int64_t s_warp[33];
    const int64_t i = threadIdx.x;
    int64_t total;
    const int64_t ex = block_exclusive_scan(i < N ? (int64_t)deg[i] : 0, s_warp, &total);
    if (i < N) offsets[i] = ex;
    if (i == 0) offsets[N] = total;
}

// offsets[0..N] = exclusive scan of deg[0..N), offsets[N] = total; bsum: (N + kScanBlock - 1) / kScanBlock + 1 words of scratch
static void launch_scan(const int32_t *deg, int64_t N, int64_t *bsum, int64_t *offsets, cudaStream_t st) {
    const int64_t nb = (N + kScanBlock - 1) / kScanBlock;
    if (nb <= 1) {
        scan_single_block_kernel<<<1, kScanBlock, 0, st>>>(deg, N, offsets);
        return;
    }
    scan_block_sums_kernel<<<(unsigned)nb, kScanBlock, 0, st>>>(deg, N, bsum);
    scan_of_sums_kernel<<<1, kScanBlock, 0, st>>>(bsum, nb, offsets + N);
    scan_apply_kernel<<<(unsigned)nb, kScanBlock, 0, st>>>(deg, N, bsum, offsets);
}

// ---------------------------------------------------------------------------- work items of the block kernels
// group_ptr[b] = work items of the structures before b (exclusive scan of CellParam::ngroups), group_ptr[B] = all of them,
// group_ptr[B + 1] = structures that have no work items (left to the warp kernels), group_ptr[B + 2] = 0: set by the
// counting kernel when an item has more candidates than one stage holds (such items keep no hit masks)
__global__ void __launch_bounds__(kScanBlock) group_scan_kernel(const CellParam *__restrict__ cellparam, int64_t B, int32_t *__restrict__ group_ptr) {
    __shared__ int64_t s_warp[33];
    int64_t carry = 0;
    int plain = 0;
    for (int64_t c0 = 0; c0 < B; c0 += kScanBlock) {
        const int64_t k = c0 + threadIdx.x;
        const int64_t v = k < B ? cellparam[k].ngroups : 0;
        plain += __syncthreads_count(k < B && cellparam[k].tile == 0);
        int64_t total;
        const int64_t ex = block_exclusive_scan(v, s_warp, &total);
        if (k < B) group_ptr[k] = (int32_t)(carry + ex);
        carry += total;
    }
    if (threadIdx.x == 0) {
        group_ptr[B] = (int32_t)carry;
        group_ptr[B + 1] = plain;
        group_ptr[B + 2] = 0;
    }
}

// ------------------------------------------------------------------------------------ block kernels
// One work item = the centres in a block of bx x by cells of one layer (z) of one structure, about kBlkTargetCentres of
// them, taken by ONE WARP (a block of 32 threads: the warps share nothing and never meet): a lane per centre.  Their
// candidates are the cells within `reach` of the block: (by + 2 reach) x (2 reach + 1) runs of the cell-sorted points.
//   COUNT stages them in shared memory in ascending order of their local index: the warp marks the indices in a bitmask
//   over the structure (at most kCapBits points), a prefix sum of the mask's population counts gives every candidate its
//   rank, and the candidate is copied to that position.  Every lane then tests its centre against the whole staged list:
//   the list is read with broadcast loads, the loop is the same for all lanes, and a test is nine instructions (load, six
//   for the squared distance as the reference rounds it, compare, bit).  The hits, a bit per staged candidate, go to the
//   workspace; they are in the order the edges are listed in.
//   EXPAND (after the scan of the degrees) puts the item's indices in the same order, turns every centre's words into a
//   list of neighbours and writes the edges, consecutive lanes on consecutive slots: no second distance test, no
//   per-centre sort.
//   FILL takes the items with more candidates than the stage holds: those leave no masks, are counted in windows as the
//   candidates come, and are tested again, in windows of ranks, by two warps per item.
// More than 32 centres are taken in passes, more neighbours than a list holds in several rounds.
template <typename T> struct BlockCap { static constexpr int value = 768; };
template <> struct BlockCap<double> { static constexpr int value = 384; };
constexpr int kItemRun = 2;                               // consecutive work items a block takes at a time

template <typename T> __device__ __forceinline__ V4<T> far_point();
template <> __device__ __forceinline__ float4 far_point<float>() { return make_float4(INFINITY, INFINITY, INFINITY, 0.f); }
template <> __device__ __forceinline__ double4 far_point<double>() { return make_double4((double)INFINITY, (double)INFINITY, (double)INFINITY, 0.0); }

// d2 < r2 (false for NaN, like the C++ comparison): the 16-bit value goes to the shared-memory address `end`, which moves on
// by one entry.  Two predicated instructions after the comparison; as a branch the compiler makes of the same, the hit path
// of almost every test (some lane hits) costs several times that.
__device__ __forceinline__ void push_if_below(float d2, float r2, uint32_t &end, int value) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.f32 p, %1, %2;\n\t@p st.shared.u16 [%0], %3;\n\t@p add.u32 %0, %0, 2;\n\t}"
                 : "+r"(end) : "f"(d2), "f"(r2), "h"((unsigned short)value));
}
__device__ __forceinline__ void push_if_below(double d2, double r2, uint32_t &end, int value) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.f64 p, %1, %2;\n\t@p st.shared.u16 [%0], %3;\n\t@p add.u32 %0, %0, 2;\n\t}"
                 : "+r"(end) : "d"(d2), "d"(r2), "h"((unsigned short)value));
}

// The structure a work item belongs to and its cell grid, kept from item to item (a run of items seldom changes structure).
struct ItemStruct {
    int b = -1, item_lo = 0, item_hi = 0;                  // structure, and the items it owns
    int gx = 0, gy = 0, gz = 0, reach = 0, bx = 1, by = 1, n = 0;
    int64_t lo = 0;
};
__device__ __forceinline__ void find_struct(ItemStruct &q, int item, int64_t B, const int64_t *__restrict__ ptr,
                                            const CellParam *__restrict__ cellparam, const int32_t *__restrict__ group_ptr, int lane) {
    if (q.b >= 0 && item < q.item_hi) return;
    int b = 0, span = (int)B;
    // largest b with group_ptr[b] <= item: every round looks at 32 entries of the range that is left
    while (span > 1) {
        const int step = (span + 31) >> 5, k = b + lane * step;
        const unsigned below = __ballot_sync(0xffffffffu, lane * step < span && group_ptr[k] <= item);     // (lane 0 always)
        const int last = 31 - __clz(below);
        span = min(step, span - last * step);
        b += last * step;
    }
    const CellParam cp = cellparam[b];
    q.b = b;
    q.gx = cp.gx; q.gy = cp.gy; q.gz = cp.gz; q.reach = cp.reach; q.bx = cp.pad & 255; q.by = cp.pad >> 8;
    q.lo = ptr[b];
    q.n = (int)(ptr[b + 1] - q.lo);
    q.item_lo = group_ptr[b];
    q.item_hi = group_ptr[b + 1];
}
// A work item: block [x0, x1) x [y0, y1) of layer cz of the structure's cells; its candidates lie in cells [xa, xb] of the
// nrows = ny x nz rows of cells from (ya, za) on.
struct BlockGeom { int cz, x0, x1, y0, y1, xa, xb, ya, za, ny, nrows; };
__device__ __forceinline__ BlockGeom block_geom(const ItemStruct &q, int item) {
    BlockGeom o;
    const int g = item - q.item_lo;
    const int nbx = (q.gx + q.bx - 1) / q.bx, nby = (q.gy + q.by - 1) / q.by, gr = g % (nbx * nby);
    o.cz = g / (nbx * nby);
    o.y0 = (gr / nbx) * q.by; o.x0 = (gr % nbx) * q.bx;
    o.y1 = min(o.y0 + q.by, q.gy); o.x1 = min(o.x0 + q.bx, q.gx);
    o.ya = max(o.y0 - q.reach, 0); o.za = max(o.cz - q.reach, 0);
    const int yb = min(o.y1 - 1 + q.reach, q.gy - 1), zb = min(o.cz + q.reach, q.gz - 1);
    o.ny = yb - o.ya + 1; o.nrows = o.ny * (zb - o.za + 1);
    o.xa = max(o.x0 - q.reach, 0); o.xb = min(o.x1 - 1 + q.reach, q.gx - 1);
    return o;
}
// This lane's part of an item's tables: the run of centres in row `lane` of the block, and candidate runs 2 lane, 2 lane + 1
// (positions in the structure's cell-sorted points).  Read an item ahead, under the tests of the item before.
struct ItemRuns { int run_k, run_len, k0[2], len[2]; };
__device__ __forceinline__ ItemRuns load_runs(const int32_t *__restrict__ cs, const ItemStruct &q, const BlockGeom &o, int lane) {
    ItemRuns r;
    r.run_k = r.run_len = 0;
    if (lane < o.y1 - o.y0) {
        const int rb = q.gx * (o.y0 + lane + q.gy * o.cz);
        r.run_k = cs[rb + o.x0];
        r.run_len = cs[rb + o.x1] - r.run_k;
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int rw = 2 * lane + h;
        r.k0[h] = r.len[h] = 0;
        if (rw < o.nrows) {
            const int rb = q.gx * (o.ya + rw % o.ny + q.gy * (o.za + rw / o.ny));
            r.k0[h] = cs[rb + o.xa];
            r.len[h] = cs[rb + o.xb + 1] - r.k0[h];
        }
    }
    return r;
}
// position, among the block's centres, -> position in the structure's cell-sorted points (-1: past the last centre)
__device__ __forceinline__ int centre_at(int q, const ItemRuns &r, int rows) {
    int kc = -1;
    for (int rr = 0; rr < rows; rr++) {
        const int len = __shfl_sync(0xffffffffu, r.run_len, rr), st = __shfl_sync(0xffffffffu, r.run_k, rr);
        if (kc < 0 && q >= 0 && q < len) kc = st + q;
        q -= len;
    }
    return kc;
}

// Exclusive prefix, over the warp's lanes, of the lengths of an item's candidate runs (two per lane): where this lane's first
// run starts in the concatenated list; returns the length of the whole list.
__device__ __forceinline__ int run_offsets(const ItemRuns &r, int lane, int &excl) {
    int incl = r.len[0] + r.len[1];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += t;
    }
    excl = incl - r.len[0] - r.len[1];
    return __shfl_sync(0xffffffffu, incl, 31);
}
// Where candidates [0, cap) of the concatenated list come from (positions in the structure's cell-sorted points): every lane
// writes out its own two runs.
__device__ __forceinline__ void write_sources(unsigned short *src, const ItemRuns &r, int excl, int cap) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int off = excl + (h ? r.len[0] : 0), kb = min(r.len[h], cap - off);
        for (int k = 0; k < kb; k++) src[off + k] = (unsigned short)(r.k0[h] + k);
    }
}

template <typename T> struct HitWords { static constexpr int value = BlockCap<T>::value / 32; };
static_assert(HitWords<float>::value == kHitWordsF32 && HitWords<double>::value == kHitWordsF64, "the workspace is sized with these");

template <typename T>
struct CountSmem {
    static constexpr int kCap = BlockCap<T>::value;
    static constexpr size_t cand = 0;                                         // V4<T>[kCap]: staged candidates
    static constexpr size_t src = cand + (size_t)kCap * sizeof(V4<T>);        // u16[kCap]: where the candidates of a stage come from
    static constexpr size_t ssrc = src + (size_t)kCap * 2;                    // u16[kCap]: the same in ascending order of index
    static constexpr size_t mask = ssrc + (size_t)kCap * 2;                   // u32[kCapBits / 32]: marks of the candidates' indices
    static constexpr size_t pref = mask + kCapBits / 8;                       // u16[kCapBits / 32]: marks before a word
    static constexpr size_t rows = pref + kCapBits / 16;                      // int k0[64], off[65]
    static constexpr size_t total = (rows + 544 + 31) & ~(size_t)31;
};

// The marks of an item's candidates (a bit per local index) -> pref[w] = marks before word w, by one warp.
__device__ __forceinline__ void rank_marks(const unsigned *mask, unsigned short *pref, int nwords, int lane) {
    constexpr int kPer = kCapBits / 32 / 32;         // words per lane
    int cnt[kPer], sum = 0;
#pragma unroll
    for (int q = 0; q < kPer; q++) {
        const int w = kPer * lane + q;
        cnt[q] = w < nwords ? __popc(mask[w]) : 0;
        sum += cnt[q];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    int run = incl - sum;
#pragma unroll
    for (int q = 0; q < kPer; q++) {
        const int w = kPer * lane + q;
        if (w < nwords) pref[w] = (unsigned short)run;
        run += cnt[q];
    }
}

// The local indices of the M candidates src[] names -> sj[f] (asynchronous copies, all in flight together), a mark per index
// in mask[], and pref[w] = marks before word w: the rank of a candidate among the item's candidates, in ascending order of
// index, is pref[j >> 5] + the marks below bit j & 31 of word j >> 5.  One warp; the loops are not unrolled (the
// instruction cache is small).
__device__ __forceinline__ void mark_and_rank(const int32_t *__restrict__ ci, const unsigned short *src, int M, int *sj, unsigned *mask,
                                              unsigned short *pref, int nwords, int lane) {
    for (int w = lane; w < nwords; w += 32) mask[w] = 0u;
    const uint32_t sj0 = (uint32_t)__cvta_generic_to_shared(sj);
#pragma unroll 4
    for (int f = lane; f < M; f += 32)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sj0 + 4u * (uint32_t)f), "l"(ci + src[f]) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
#pragma unroll 4
    for (int f = lane; f < M; f += 32) {
        const int j = sj[f];
        atomicOr(&mask[j >> 5], 1u << (j & 31));
    }
    __syncwarp();
    rank_marks(mask, pref, nwords, lane);
    __syncwarp();
}

// COUNT.  An item whose candidates fit one stage (the rule) is staged in ascending order of the candidates' indices, as FILL
// needs them: the centre's hits, a bit per staged candidate, go to the workspace (hits[point][word], the centre's own bit
// cleared unless loops are wanted), and the filling pass only expands them: the distance tests are done once.  The degree
// under the neighbour-cap rule comes from the same words (hits before / after the centre's own place).  An item with more
// candidates is counted in windows, as they come, sets the flag word after the work-item prefix and leaves no masks.
template <typename T>
__global__ void __launch_bounds__(32, 12)                  // (shared memory allows 12 one-warp blocks per SM)
neighbours_block_count_kernel(const int64_t *__restrict__ ptr, int64_t B, T r2, int64_t max_nn, int loop, int rule,
                              const V4<T> *__restrict__ spos, const CellParam *__restrict__ cellparam,
                              const int32_t *__restrict__ cell_start, int32_t *__restrict__ group_ptr, int32_t *__restrict__ deg,
                              const int32_t *__restrict__ cidx, unsigned *__restrict__ hits, unsigned char *__restrict__ item_flag,
                              int32_t *__restrict__ status) {
    using S = CountSmem<T>;
    constexpr int kCap = S::kCap, kPerLane = kCap / 32, kWords = HitWords<T>::value;
    extern __shared__ __align__(32) unsigned char blk_smem[];
    const int lane = threadIdx.x;
    V4<T> *cand = reinterpret_cast<V4<T> *>(blk_smem + S::cand);
    unsigned short *src = reinterpret_cast<unsigned short *>(blk_smem + S::src);
    unsigned short *ssrc = reinterpret_cast<unsigned short *>(blk_smem + S::ssrc);
    unsigned *mask = reinterpret_cast<unsigned *>(blk_smem + S::mask);
    unsigned short *pref = reinterpret_cast<unsigned short *>(blk_smem + S::pref);
    int *s_k0 = reinterpret_cast<int *>(blk_smem + S::rows), *s_off = s_k0 + 64;
    const unsigned full = 0xffffffffu;
    const int G = group_ptr[B];
    RPHASE_DECL

    // Items are dealt in runs of kItemRun consecutive ones: neighbouring blocks of one structure, whose structure look-up and
    // parameters are then read once per run and whose candidates overlap in the L2.
    ItemStruct q;
    ItemRuns ahead;
    bool have_ahead = false;
    const int nruns = (G + kItemRun - 1) / kItemRun;
    for (int run = blockIdx.x; run < nruns; run += gridDim.x)
    for (int item = run * kItemRun, item_end = min(G, (run + 1) * kItemRun); item < item_end; item++) {
        RPHASE(10)
        find_struct(q, item, B, ptr, cellparam, group_ptr, lane);
        const BlockGeom o = block_geom(q, item);
        const int32_t *cs = cell_start + q.lo + q.b;
        const V4<T> *sp = spos + q.lo;
        const ItemRuns rn = have_ahead ? ahead : load_runs(cs, q, o, lane);
        have_ahead = false;
        const int nc = warp_sum(rn.run_len), rows = o.y1 - o.y0;
        // the first 32 centres' points: on their way while the candidates are staged
        const int kc0 = centre_at(lane, rn, rows);
        const V4<T> pc0 = sp[max(kc0, 0)];

        // ---- the candidate runs: exclusive prefix of their lengths; every lane writes out where its two runs come from
        int excl;
        const int M = run_offsets(rn, lane, excl);
        if (nc > 0) {
            if (2 * lane < o.nrows) { s_k0[2 * lane] = rn.k0[0]; s_off[2 * lane] = excl; }
            if (2 * lane + 1 < o.nrows) { s_k0[2 * lane + 1] = rn.k0[1]; s_off[2 * lane + 1] = excl + rn.len[0]; }
            if (lane == 0) s_off[o.nrows] = M;
            write_sources(src, rn, excl, kCap);
        }
        __syncwarp();
        const bool single = M <= kCap;
        RPHASE(11)
        bool first_src = true;                         // src[] still holds the sources of candidates [0, kCap)
        auto build_src = [&](int c0) {                 // sources of candidates [c0, c0 + kCap) of the concatenated runs; half a warp per run
            const int half = lane >> 4, l16 = lane & 15;
            for (int rw = half; rw < o.nrows; rw += 2) {
                const int off = s_off[rw] - c0, len = s_off[rw + 1] - s_off[rw], k0 = s_k0[rw];
                const int ka = max(0, -off), kb = min(len, kCap - off);
                for (int k = ka + l16; k < kb; k += 16) src[off + k] = (unsigned short)(k0 + k);
            }
            __syncwarp();
        };
        // the points from[f] names, f < mc, into the stage without passing through registers, all copies in flight together
        auto copy_in = [&](const unsigned short *from_idx, int mc) {
            const uint32_t dst0 = (uint32_t)__cvta_generic_to_shared(cand);
#pragma unroll
            for (int u = 0; u < kPerLane; u++) {
                const int f = u * 32 + lane;
                if (f < mc) {
                    const V4<T> *from = sp + from_idx[f];
#pragma unroll
                    for (int h = 0; h < (int)sizeof(V4<T>) / 16; h++)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst0 + (uint32_t)(f * sizeof(V4<T>) + 16 * h)),
                                     "l"(reinterpret_cast<const char *>(from) + 16 * h) : "memory");
                }
            }
            {   // the rest of the last 32 staged entries: points that hit nothing
                const int f = mc + lane;
                if (f < ((mc + 31) & ~31)) cand[f] = far_point<T>();
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
        };
        auto stage_plain = [&](int c0) {               // candidates [c0, c0 + kCap) as they come
            if (c0 > 0 || !first_src) build_src(c0);
            first_src = false;
            copy_in(src, min(kCap, M - c0));
        };
        auto rank_of = [&](int j) { return (int)pref[j >> 5] + __popc(mask[j >> 5] & ((1u << (j & 31)) - 1u)); };
        if (nc > 0 && single) {
            // ---- in ascending order of index: mark the indices, rank the marks, sources by rank, copy
            // the candidates' indices go through the stage, which is still empty
            int *sj = reinterpret_cast<int *>(cand);
            mark_and_rank(cidx + q.lo, src, M, sj, mask, pref, (q.n + 31) >> 5, lane);      // (n <= kCapBits)
#pragma unroll 1
            for (int f0 = lane; f0 < M; f0 += 256) {
                // (eight ranks first, then their stores: a load of shared memory cannot be moved above an earlier store)
                int rk[8];
#pragma unroll
                for (int u = 0; u < 8; u++) rk[u] = rank_of(sj[min(f0 + 32 * u, M - 1)]);
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (f0 + 32 * u < M) ssrc[rk[u]] = src[f0 + 32 * u];
            }
            __syncwarp();
            copy_in(ssrc, M);
        } else if (nc > 0 && lane == 0) {
            atomicOr(group_ptr + B + 2, 1);                      // an item without hit masks: the filling pass tests it again
        }
        if (lane == 0) item_flag[item] = (nc > 0 && !single) ? 1 : 0;
        // the next item's tables: read under this item's tests
        if (item + 1 < min(item_end, q.item_hi)) {
            ahead = load_runs(cs, q, block_geom(q, item + 1), lane);
            have_ahead = true;
        }
        RPHASE(12)

        for (int cp0 = 0; cp0 < nc; cp0 += 32) {
            // ---- this lane's centre
            const int kc = cp0 == 0 ? kc0 : centre_at(cp0 + lane, rn, rows);
            const bool active = kc >= 0;
            const V4<T> pc = cp0 == 0 ? pc0 : sp[max(kc, 0)];
            const int il = idx_of(pc);
            // (a lane without a centre sits at infinity: no hits)
            const T xi = active ? pc.x : T(INFINITY), yi = active ? pc.y : T(INFINITY), zi = active ? pc.z : T(INFINITY);
            RPHASE(13)
            const int self_hit = dist2_rn(xi, yi, zi, xi, yi, zi) < r2 ? 1 : 0;      // (the centre is one of its candidates)
            int cnt = 0, cnt_lo = 0;                             // hits (the centre included), hits below the centre's own index
            if (single) {
                const int nw = (M + 31) >> 5;
                const int self_rank = active ? rank_of(il) : -1, self_w = self_rank >> 5;
                const unsigned self_bit = 1u << (self_rank & 31);
                unsigned *my_words = hits + (size_t)(q.lo + il) * kWords;
                for (int w = 0; w < nw; w++) {
                    const V4<T> *cw = cand + w * 32;
                    unsigned word = 0u;
#pragma unroll
                    for (int u = 0; u < 32; u++) {
                        const V4<T> p = cw[u];
                        const T d2 = dist2_rn(xi, yi, zi, p.x, p.y, p.z);
                        if (d2 < r2) word |= 1u << u;
                    }
                    cnt += __popc(word);
                    if (w < self_w) cnt_lo += __popc(word);
                    if (w == self_w) {
                        cnt_lo += __popc(word & (self_bit - 1u));
                        if (!loop) word &= ~self_bit;
                    }
                    if (active) my_words[w] = word;
                }
            } else {
                auto count_windows = [&](auto with_lo_tag) {
                    constexpr bool kLo = decltype(with_lo_tag)::value;
                    cnt = cnt_lo = 0;
                    for (int wb = 0; wb < M; wb += kCap) {
                        stage_plain(wb);
                        const int mw = min(kCap, M - wb), nw = (mw + 31) >> 5;
                        for (int w = 0; w < nw; w++) {
                            const V4<T> *cw = cand + w * 32;
#pragma unroll 8
                            for (int u = 0; u < 32; u++) {
                                const V4<T> p = cw[u];
                                const T d2 = dist2_rn(xi, yi, zi, p.x, p.y, p.z);
                                if (d2 < r2) {
                                    cnt++;
                                    if (kLo) cnt_lo += idx_of(p) < il;
                                }
                            }
                        }
                        __syncwarp();
                    }
                };
                count_windows(std::false_type{});
                // hits below the centre's own index matter only where the neighbour cap bites: counted in a second walk
                const bool over = active && (int64_t)(loop ? cnt : cnt - self_hit) > max_nn;
                if (__any_sync(full, over)) count_windows(std::true_type{});
            }
            RPHASE(14)
            if (active) {
                const int64_t nlo = cnt_lo, nhi = cnt - self_hit - cnt_lo;
                int64_t total, k;
                if (loop) {
                    total = nlo + nhi + self_hit;
                    k = total < max_nn ? total : max_nn;
                } else if (rule == MLCGB_RULE_CLUSTER && self_hit) {
                    total = nlo + nhi;
                    if (nlo >= max_nn + 1) k = max_nn + 1;
                    else k = total < max_nn ? total : max_nn;
                } else {
                    total = nlo + nhi;
                    k = total < max_nn ? total : max_nn;
                }
                deg[q.lo + il] = (int32_t)k;
                if (k < total) atomicOr(status, (int)kTruncated);
            }
        }
        __syncwarp();          // the stage and its tables are rewritten by the next item
    }
}

// FILL for the items that left no hit masks (more candidates than a stage holds: tested again here, in windows of ranks), with
// the candidates of an item split between the warps of a block (kFillWarps of them): the same work item, the same
// staged list, lane l of every warp the same centre, warp w the w-th part of the (ascending) list.  A centre's edges are then
// warp 0's hits followed by warp 1's: each warp writes its own, warp 1 after warp 0 has published how many it had.  Warp 0
// publishes its counts when its tests are done, before it writes its own edges, and arrives on a named barrier; warp 1 waits
// on that barrier before its first emission.  Warp 0 never waits for warp 1 inside a window, so nobody waits in a circle, and
// both warps write at the same time.  Twice the warps per staged list hide twice the latency: the staging, the pushes and
// the emission are chains of dependent shared-memory operations, and shared memory, not registers, is what limits the
// blocks per SM.  The emission takes what it needs of a centre (count, place of the centre's own entry, first slot, index)
// from a table in shared memory, half a warp per centre, and reads the next pair's entries while this pair's edges go out.
constexpr int kFillWarps = 2;
constexpr int kFillList = 80;                              // entries of a warp's hit list of a centre between two emissions
constexpr int kFillListStride = kFillList + 2;             // (in 16-bit entries: an odd number of words, so that lanes at the same
                                                           //  position of their lists use different banks)

template <typename T>
struct FillSmem {
    static constexpr int kCap = BlockCap<T>::value;
    static constexpr size_t cand = 0;                                          // V4<T>[kCap]: staged candidates, ascending
    static constexpr size_t hits = cand + (size_t)kCap * sizeof(V4<T>);        // u16[kFillWarps][32][kFillListStride]
    static constexpr size_t hits_bytes = (size_t)kFillWarps * 32 * kFillListStride * 2;
    // while an item is staged the lists are empty and their space holds:
    static constexpr size_t src = hits;                                        // u16[kCap]: where a chunk's candidates come from
    static constexpr size_t ssrc = src + (size_t)kCap * 2;                     // u16[kCap]: the same in ascending order
    static constexpr size_t mask = ssrc + (size_t)kCap * 2;                    // u32[kCapBits / 32]
    static constexpr size_t pref = mask + kCapBits / 8;                        // u16[kCapBits / 32]
    static_assert(pref + kCapBits / 16 <= hits + hits_bytes, "staging tables must fit the space of the hit lists");
    static constexpr size_t rows = hits + hits_bytes;                          // int k0[64], off[65]
    static constexpr size_t avail = rows + 544;                                // int[kFillWarps][32]: entries the warps had
    static constexpr size_t par = (avail + (size_t)kFillWarps * 32 * 4 + 15) & ~(size_t)15;   // int4[kFillWarps][32]: what an emission needs of a centre
    static constexpr size_t total = (par + (size_t)kFillWarps * 32 * 16 + 31) & ~(size_t)31;
};

static_assert(kFillWarps == 2, "the hand-over below is written for two warps: one named barrier, warp 0 arrives, warp 1 waits");
__device__ __forceinline__ void fill_handover_wait() { asm volatile("bar.sync 1, 64;" ::: "memory"); }
__device__ __forceinline__ void fill_handover_arrive() { asm volatile("bar.arrive 1, 64;" ::: "memory"); }

template <typename T>
__global__ void __launch_bounds__(kFillWarps * 32, 8)      // (shared memory allows nine blocks per SM; with eight nothing spills)
neighbours_block_fill_kernel(const T *__restrict__ pos, const int64_t *__restrict__ ptr, int64_t B, T r2, int loop,
                             const V4<T> *__restrict__ spos, const CellParam *__restrict__ cellparam,
                             const int32_t *__restrict__ cell_start, const int32_t *__restrict__ group_ptr,
                             const unsigned char *__restrict__ item_flag, const int64_t *__restrict__ offsets, FillOut out) {
    using S = FillSmem<T>;
    constexpr int kCap = S::kCap, kPerThread = kCap / (kFillWarps * 32), kThreads = kFillWarps * 32;
    extern __shared__ __align__(32) unsigned char blk_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    V4<T> *cand = reinterpret_cast<V4<T> *>(blk_smem + S::cand);
    unsigned short *src = reinterpret_cast<unsigned short *>(blk_smem + S::src);
    unsigned short *ssrc = reinterpret_cast<unsigned short *>(blk_smem + S::ssrc);
    unsigned *mask = reinterpret_cast<unsigned *>(blk_smem + S::mask);
    unsigned short *pref = reinterpret_cast<unsigned short *>(blk_smem + S::pref);
    int *s_k0 = reinterpret_cast<int *>(blk_smem + S::rows), *s_off = s_k0 + 64;
    int *s_avail = reinterpret_cast<int *>(blk_smem + S::avail);
    int4 *s_par = reinterpret_cast<int4 *>(blk_smem + S::par) + warp * 32;
    unsigned short *warp_hits = reinterpret_cast<unsigned short *>(blk_smem + S::hits) + warp * 32 * kFillListStride;
    unsigned short *my_hits = warp_hits + lane * kFillListStride;
    const unsigned full = 0xffffffffu;
    const int G = group_ptr[B];
    if (group_ptr[B + 2] == 0) return;                     // every item left its hit masks: the expanding kernel fills them all
    // (the output pointers as scalars: read through the parameter struct inside the lambdas below they end up in local
    //  memory, and with all of the L1 given to shared memory every such read is a trip to the L2)
    int64_t *const o_row0 = out.row0, *const o_row1 = out.row1, *const o_batch = out.mapping_batch;
    T *const o_dist = reinterpret_cast<T *>(out.distance);
    int32_t *const o_row0_32 = out.row0_32, *const o_row1_32 = out.row1_32;
    RPHASE_DECL

    // The items the counting pass has flagged, found 32 flags at a time.  (Every warp reads the flags and decodes an item for
    // itself: the same loads, no exchange.)
    ItemStruct q;
    ItemRuns ahead;
    bool have_ahead = false;
    const int item_end = 0;                                  // (nothing is read ahead here: the items are few and far between)
    for (int base = blockIdx.x * 32; base < G; base += gridDim.x * 32)
    for (unsigned todo = __ballot_sync(full, base + lane < G && item_flag[base + lane] != 0); todo; todo &= todo - 1) {
        const int item = base + __ffs(todo) - 1;
        RPHASE(0)
        find_struct(q, item, B, ptr, cellparam, group_ptr, lane);
        const BlockGeom o = block_geom(q, item);
        const int b = q.b, n = q.n, nrows = o.nrows, rows = o.y1 - o.y0;
        const int64_t lo = q.lo;
        const int32_t *cs = cell_start + lo + b;
        const V4<T> *sp = spos + lo;
        const ItemRuns rn = have_ahead ? ahead : load_runs(cs, q, o, lane);
        have_ahead = false;
        const int nc = warp_sum(rn.run_len);
        // the first 32 centres' points: on their way while the candidates are staged
        const int kc0 = centre_at(lane, rn, rows);
        const V4<T> pc0 = sp[max(kc0, 0)];
        int M;
        {   // the candidate runs: exclusive prefix of the lengths; warp w writes out where run 2 lane + w comes from
            int excl;
            M = run_offsets(rn, lane, excl);
            // (an item that fits one stage left its hit masks: the expanding kernel's.  Before anything of it is written to
            //  shared memory: the warps meet only in the items this kernel takes.  The same in every warp.)
            if (M <= kCap) continue;
            const int h = warp & 1, off = excl + (h ? rn.len[0] : 0), k0h = h ? rn.k0[1] : rn.k0[0], lenh = h ? rn.len[1] : rn.len[0];
            if (nc > 0 && warp < 2) {
                if (2 * lane + h < nrows) { s_k0[2 * lane + h] = k0h; s_off[2 * lane + h] = off; }
                if (tid == 0) s_off[nrows] = M;
                const int kb = min(lenh, kCap - off);
                for (int k = 0; k < kb; k++) src[off + k] = (unsigned short)(k0h + k);
            }
        }
        __syncthreads();
        RPHASE(1)
        bool src_fresh = true;                               // src[] holds the sources of candidates [0, kCap)

        auto build_src = [&](int c0) {                       // sources of candidates [c0, c0 + kCap) of the concatenated runs
            const int half = tid >> 4, l16 = tid & 15;
            for (int rw = half; rw < nrows; rw += kThreads / 16) {
                const int off = s_off[rw] - c0, len = s_off[rw + 1] - s_off[rw], k0 = s_k0[rw];
                const int ka = max(0, -off), kb = min(len, kCap - off);
                for (int k = ka + l16; k < kb; k += 16) src[off + k] = (unsigned short)(k0 + k);
            }
            __syncthreads();
        };
        auto rank_of = [&](int j) { return (int)pref[j >> 5] + __popc(mask[j >> 5] & ((1u << (j & 31)) - 1u)); };
        // candidates of ranks [wb, wb + kCap) -> the stage, ascending (the lists are empty: their space holds the tables)
        auto stage = [&](int wb) {
            const int nwords = (n + 31) >> 5;                // (n <= kCapBits)
            for (int w = tid; w < nwords; w += kThreads) mask[w] = 0u;
            __syncthreads();
            int jj[kPerThread];                              // local indices of this thread's candidates of a chunk
            for (int c0 = 0; c0 < M; c0 += kCap) {
                const int mc = min(kCap, M - c0);
                if (c0 > 0 || !src_fresh) build_src(c0);
                src_fresh = false;
#pragma unroll
                for (int u = 0; u < kPerThread; u++) jj[u] = idx_of(sp[src[min(u * kThreads + tid, mc - 1)]]);
#pragma unroll
                for (int u = 0; u < kPerThread; u++)
                    if (u * kThreads + tid < mc) atomicOr(&mask[jj[u] >> 5], 1u << (jj[u] & 31));
                __syncthreads();
            }
            if (warp == 0) {
                constexpr int kPer = kCapBits / 32 / 32;     // words per lane
                int cnt[kPer], sum = 0;
#pragma unroll
                for (int q = 0; q < kPer; q++) {
                    const int w = kPer * lane + q;
                    cnt[q] = w < nwords ? __popc(mask[w]) : 0;
                    sum += cnt[q];
                }
                int incl = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(full, incl, o);
                    if (lane >= o) incl += t;
                }
                int run = incl - sum;
#pragma unroll
                for (int q = 0; q < kPer; q++) {
                    const int w = kPer * lane + q;
                    if (w < nwords) pref[w] = (unsigned short)run;
                    run += cnt[q];
                }
            }
            __syncthreads();
            const int mw = min(kCap, M - wb);
            const uint32_t dst0 = (uint32_t)__cvta_generic_to_shared(cand);
            auto copy_sorted = [&](int count) {              // cand[f] <- the point ssrc[f] names, f < count: asynchronous copies
#pragma unroll
                for (int u = 0; u < kPerThread; u++) {
                    const int f = u * kThreads + tid;
                    if (f < count) {
                        const V4<T> *from = sp + ssrc[f];
#pragma unroll
                        for (int h = 0; h < (int)sizeof(V4<T>) / 16; h++)
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst0 + (uint32_t)(f * sizeof(V4<T>) + 16 * h)),
                                         "l"(reinterpret_cast<const char *>(from) + 16 * h) : "memory");
                    }
                }
            };
            // (a chunk's sources that fall into the window go to their place in ssrc, chunk after chunk)
            for (int c0 = 0; c0 < M; c0 += kCap) {
                const int mc = min(kCap, M - c0);
                build_src(c0);
#pragma unroll
                for (int u = 0; u < kPerThread; u++) jj[u] = idx_of(sp[src[min(u * kThreads + tid, mc - 1)]]);
#pragma unroll
                for (int u = 0; u < kPerThread; u++)
                    if (u * kThreads + tid < mc) {
                        const int rw = rank_of(jj[u]) - wb;
                        if (rw >= 0 && rw < kCap) ssrc[rw] = src[u * kThreads + tid];
                    }
                __syncthreads();
            }
            copy_sorted(mw);
            {   // the rest of the last 32 staged entries: points that hit nothing
                const int f = mw + tid;
                if (f < ((mw + 31) & ~31)) cand[f] = far_point<T>();
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
        };
        // the first 32 centres' places in the output (their points have arrived by now), read under the tests: the first
        // window is tested without looking at them
        int64_t base0 = 0, end0 = 0;
        if (kc0 >= 0) {
            base0 = offsets[lo + idx_of(pc0)];
            end0 = offsets[lo + idx_of(pc0) + 1];
        }
        // the next item's tables: read under this item's tests
        if (item + 1 < min(item_end, q.item_hi)) {
            ahead = load_runs(cs, q, block_geom(q, item + 1), lane);
            have_ahead = true;
        }
        RPHASE(2)

        for (int cp0 = 0; cp0 < nc; cp0 += 32) {
            // ---- this lane's centre (the same in every warp)
            const int kc = cp0 == 0 ? kc0 : centre_at(cp0 + lane, rn, rows);
            const bool active = kc >= 0;
            const V4<T> pc = cp0 == 0 ? pc0 : sp[max(kc, 0)];
            const int il = idx_of(pc);
            // (a lane without a centre sits at infinity: no hits)
            const T xi = active ? pc.x : T(INFINITY), yi = active ? pc.y : T(INFINITY), zi = active ? pc.z : T(INFINITY);
            int64_t base_off = base0, end_off = end0;
            int emitted = 0;                                 // entries (other than the centre itself) gone by so far
            if (cp0 > 0) {
                base_off = end_off = 0;
                if (active) {
                    base_off = offsets[lo + il];
                    end_off = offsets[lo + il + 1];
                }
            }
            const uint32_t list0 = (uint32_t)__cvta_generic_to_shared(my_hits);
            RPHASE(3)

            for (int wb = 0; wb < M; wb += kCap) {
                if (wb > 0 && !__any_sync(full, active && emitted < (int)(end_off - base_off))) break;      // (the same in every warp)
                stage(wb);
                const int mw = min(kCap, M - wb), nw = (mw + 31) >> 5, nwh = (nw + kFillWarps - 1) / kFillWarps;
                const int w_lo = min(warp * nwh, nw), w_hi = min(w_lo + nwh, nw);
                uint32_t list_end = list0;                   // shared-memory address past the last entry of this lane's list
                int flushed = 0;                             // entries of this window this warp has dealt with, for this lane's centre
                bool waited = warp == 0;
                // this warp's lists so far -> edges, a centre at a time, consecutive lanes on consecutive slots; the centre's
                // own entry is skipped (unless loops are wanted), entries beyond the centre's count are not written
                auto emit_lists = [&](bool last) {
                    __syncwarp();
                    RPHASE(4)
                    const int nh = (int)(list_end - list0) >> 1;
                    int self_at = INT_MAX;                   // where the centre itself sits in its (ascending) list
                    if (!loop) {
                        int lo_t = 0, hi_t = nh;
                        while (lo_t < hi_t) {
                            const int mid = (lo_t + hi_t) >> 1;
                            if ((int)my_hits[mid] < il) lo_t = mid + 1; else hi_t = mid;
                        }
                        if (lo_t < nh && (int)my_hits[lo_t] == il) self_at = lo_t;
                    }
                    const int avail = nh - (self_at != INT_MAX ? 1 : 0);
                    if (last) {                              // this warp's count of the window is final: the next warp may go ahead
                        s_avail[warp * 32 + lane] = flushed + avail;
                        __threadfence_block();
                        if (warp == 0) fill_handover_arrive();
                    }
                    if (!waited) {                           // the warps before this one are through: their counts are there
                        fill_handover_wait();
                        waited = true;
                    }
                    int start = emitted + flushed;
                    for (int w2 = 0; w2 < warp; w2++) start += s_avail[w2 * 32 + lane];
                    const int take = max(0, min(avail, (int)(end_off - base_off) - start));
                    const int64_t slot0 = base_off + start;
                    RPHASE(5)
                    // what the emission needs of a centre goes through a table: half a warp takes a centre, two centres at a
                    // time, and the next pair's entries are read while this pair's edges are written
                    s_par[lane] = make_int4(take | (min(self_at, 0xffff) << 16), il, (int)(uint32_t)slot0, (int)(slot0 >> 32));
                    __syncwarp();
                    const int hsel = lane >> 4, l16 = lane & 15;
                    int4 nxt = s_par[hsel];
                    for (int pp = 0; pp < 16; pp++) {
                        const int4 cur = nxt;
                        const int cc = 2 * pp + hsel;
                        if (pp < 15) nxt = s_par[cc + 2];
                        const int tk = cur.x & 0xffff, at = (int)((unsigned)cur.x >> 16);
                        const int64_t slot_c = (int64_t)(((uint64_t)(uint32_t)cur.w << 32) | (uint32_t)cur.z), ic = lo + cur.y;
                        T cxi = T(0), cyi = T(0), czi = T(0);
                        if (o_dist) { cxi = __shfl_sync(full, xi, cc); cyi = __shfl_sync(full, yi, cc); czi = __shfl_sync(full, zi, cc); }
                        const unsigned short *hl = warp_hits + cc * kFillListStride;
                        for (int t = l16; t < tk; t += 16) {
                            const int64_t gj = lo + (int)hl[t + (t >= at ? 1 : 0)], slot = slot_c + t;
                            if (o_row0) { o_row0[slot] = ic; o_row1[slot] = gj; }
                            if (o_batch) o_batch[slot] = b;
                            if (o_dist) o_dist[slot] = sqrt(dist2_rn(cxi, cyi, czi, pos[gj * 3], pos[gj * 3 + 1], pos[gj * 3 + 2]));
                            if (o_row0_32) { o_row0_32[slot] = (int32_t)ic; o_row1_32[slot] = (int32_t)gj; }
                        }
                    }
                    flushed += avail;
                    list_end = list0;
                    __syncwarp();
                    RPHASE(6)
                };
                for (int w = w_lo; w < w_hi; w++) {
                    if (__any_sync(full, list_end > list0 + 2 * (kFillList - 32))) emit_lists(false);   // room for this word's hits in every list
                    const V4<T> *cw = cand + w * 32;
                    // (eight loads and distances, then their pushes: a load cannot be moved above an earlier store to
                    //  shared memory, so interleaved they would run one test at a time)
#pragma unroll
                    for (int g8 = 0; g8 < 4; g8++) {
                        T d2[8];
                        int id[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            const V4<T> q = cw[g8 * 8 + u];
                            d2[u] = dist2_rn(xi, yi, zi, q.x, q.y, q.z);
                            id[u] = idx_of(q);
                        }
#pragma unroll
                        for (int u = 0; u < 8; u++) push_if_below(d2[u], r2, list_end, id[u]);
                    }
                    asm volatile("" ::: "memory");           // (the pushes write shared memory behind the compiler's back)
                }
                emit_lists(true);
                __syncthreads();                             // everybody's counts of the window are there
#pragma unroll
                for (int w2 = 0; w2 < kFillWarps; w2++) emitted += s_avail[w2 * 32 + lane];
                __syncthreads();                             // before the counts, the lists and the stage are written again
            }
        }
    }
}

// FILL for the items whose hit masks the counting pass has left in the workspace: no distance tests.  A warp takes an item,
// puts the indices of the item's candidates in ascending order (the marks and ranks of the counting pass again, without the
// points themselves), and every lane turns its centre's words into the centre's list of neighbours, which half a warp
// per centre then writes out, consecutive lanes on consecutive slots.
constexpr int kExpList = 128;                              // entries of a centre's list between two emissions
constexpr int kExpListStride = kExpList + 2;               // (16-bit entries: an odd number of words)

template <typename T>
struct ExpandSmem {
    static constexpr int kCap = BlockCap<T>::value;
    static constexpr size_t sidx = 0;                                          // u16[kCap]: the candidates' local indices, ascending
    static constexpr size_t src = sidx + (size_t)kCap * 2;                     // u16[kCap]: where the candidates come from
    static constexpr size_t mask = src + (size_t)kCap * 2;                     // u32[kCapBits / 32]
    static constexpr size_t pref = mask + kCapBits / 8;                        // u16[kCapBits / 32]
    // once the indices are in order, src / mask / pref are free: the centres' hit words, u32[kCap / 32][32], go there
    static constexpr size_t words = src;
    static_assert((size_t)kCap * 4 <= (size_t)kCap * 2 + kCapBits / 8 + kCapBits / 16, "the hit words must fit the staging tables");
    static constexpr size_t lists = pref + kCapBits / 16;                      // u16[32][kExpListStride]; while staging: int[kCap] indices
    static_assert((size_t)kCap * 4 <= (size_t)32 * kExpListStride * 2, "the staged indices must fit the space of the lists");
    static constexpr size_t par = (lists + (size_t)32 * kExpListStride * 2 + 15) & ~(size_t)15;   // int4[32]
    static constexpr size_t total = (par + 32 * 16 + 31) & ~(size_t)31;
};

template <typename T>
__global__ void __launch_bounds__(32, 16)
neighbours_block_expand_kernel(const T *__restrict__ pos, const int64_t *__restrict__ ptr, int64_t B, int loop,
                               const V4<T> *__restrict__ spos, const CellParam *__restrict__ cellparam,
                               const int32_t *__restrict__ cell_start, const int32_t *__restrict__ group_ptr,
                               const int32_t *__restrict__ cidx, const unsigned *__restrict__ hits, const int64_t *__restrict__ offsets,
                               FillOut out) {
    using S = ExpandSmem<T>;
    constexpr int kCap = S::kCap, kWords = HitWords<T>::value;
    extern __shared__ __align__(32) unsigned char blk_smem[];
    const int lane = threadIdx.x;
    unsigned short *src = reinterpret_cast<unsigned short *>(blk_smem + S::src);
    unsigned short *sidx = reinterpret_cast<unsigned short *>(blk_smem + S::sidx);
    unsigned *mask = reinterpret_cast<unsigned *>(blk_smem + S::mask);
    unsigned short *pref = reinterpret_cast<unsigned short *>(blk_smem + S::pref);
    unsigned short *all_lists = reinterpret_cast<unsigned short *>(blk_smem + S::lists);
    unsigned short *my_list = all_lists + lane * kExpListStride;
    int4 *s_par = reinterpret_cast<int4 *>(blk_smem + S::par);
    unsigned *my_hw = reinterpret_cast<unsigned *>(blk_smem + S::words) + lane;          // word w of this lane's centre at [32 w]
    const unsigned full = 0xffffffffu;
    const int G = group_ptr[B];
    int64_t *const o_row0 = out.row0, *const o_row1 = out.row1, *const o_batch = out.mapping_batch;
    T *const o_dist = reinterpret_cast<T *>(out.distance);
    int32_t *const o_row0_32 = out.row0_32, *const o_row1_32 = out.row1_32;

    RPHASE_DECL
    ItemStruct q;
    ItemRuns ahead;
    bool have_ahead = false;
    const int nruns = (G + kItemRun - 1) / kItemRun;
    for (int run = blockIdx.x; run < nruns; run += gridDim.x)
    for (int item = run * kItemRun, item_end = min(G, (run + 1) * kItemRun); item < item_end; item++) {
        RPHASE(0)
        find_struct(q, item, B, ptr, cellparam, group_ptr, lane);
        const BlockGeom o = block_geom(q, item);
        const int b = q.b, rows = o.y1 - o.y0;
        const int64_t lo = q.lo;
        const int32_t *cs = cell_start + lo + b;
        const V4<T> *sp = spos + lo;
        const ItemRuns rn = have_ahead ? ahead : load_runs(cs, q, o, lane);
        have_ahead = false;
        const int nc = warp_sum(rn.run_len);
        const int kc0 = centre_at(lane, rn, rows);
        const V4<T> pc0 = sp[max(kc0, 0)];                  // the first 32 centres' points: on their way during the staging
        int excl;
        const int M = run_offsets(rn, lane, excl);
        RPHASE(1)
        const bool mine = nc > 0 && M <= kCap;              // (items with more candidates have no masks: the testing kernel fills them)
        if (mine) {
            write_sources(src, rn, excl, kCap);
            // the candidates' indices go through the space of the lists, empty now
            int *sj = reinterpret_cast<int *>(all_lists);
            mark_and_rank(cidx + lo, src, M, sj, mask, pref, (q.n + 31) >> 5, lane);
#pragma unroll 1
            for (int f0 = lane; f0 < M; f0 += 256) {
                // (eight ranks first, then their stores: a load of shared memory cannot be moved above an earlier store)
                int jj[8], rk[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    jj[u] = sj[min(f0 + 32 * u, M - 1)];
                    rk[u] = (int)pref[jj[u] >> 5] + __popc(mask[jj[u] >> 5] & ((1u << (jj[u] & 31)) - 1u));
                }
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (f0 + 32 * u < M) sidx[rk[u]] = (unsigned short)jj[u];
            }
            __syncwarp();
        }
        if (item + 1 < min(item_end, q.item_hi)) {          // the next item's tables: read under this item's work
            ahead = load_runs(cs, q, block_geom(q, item + 1), lane);
            have_ahead = true;
        }
        RPHASE(2)
        if (!mine) continue;
        const int nw = (M + 31) >> 5;

        for (int cp0 = 0; cp0 < nc; cp0 += 32) {
            const int kc = cp0 == 0 ? kc0 : centre_at(cp0 + lane, rn, rows);
            const bool active = kc >= 0;
            const V4<T> pc = cp0 == 0 ? pc0 : sp[max(kc, 0)];
            const int il = idx_of(pc);
            int64_t base_off = 0;
            int kept = 0;
            const unsigned *my_words = hits + (size_t)(lo + il) * kWords;
            if (active) {
                base_off = offsets[lo + il];
                kept = (int)(offsets[lo + il + 1] - base_off);
            }
            // the centre's words: loaded together, parked in shared memory (the loop over them below is not unrolled)
            {
                uint4 wd[kWords / 4];
#pragma unroll
                for (int g4 = 0; g4 < kWords / 4; g4++) {
                    wd[g4] = make_uint4(0u, 0u, 0u, 0u);
                    if (active && 4 * g4 < nw) wd[g4] = *reinterpret_cast<const uint4 *>(my_words + 4 * g4);
                }
#pragma unroll
                for (int g4 = 0; g4 < kWords / 4; g4++) {
                    my_hw[32 * (4 * g4)] = wd[g4].x; my_hw[32 * (4 * g4 + 1)] = wd[g4].y;
                    my_hw[32 * (4 * g4 + 2)] = wd[g4].z; my_hw[32 * (4 * g4 + 3)] = wd[g4].w;
                }
            }
            RPHASE(3)
            // Entries [first, first + kExpList) of every centre's neighbours at a time (one round, unless a centre has more than
            // kExpList neighbours to write): a word's set bits become entries of the centre's list, positions in the ascending
            // candidate list, turned into indices when the edges are written (the centre's own bit was cleared by the counting
            // pass unless loops are wanted).  One copy of the expansion and of the emission: the instruction cache is small.
            for (int first = 0; __any_sync(full, first < kept); first += kExpList) {
                int ord = 0;                                     // ordinal of the next set bit among the centre's neighbours
#pragma unroll 1
                for (int w = 0; w < nw; w++) {
                    unsigned word = (ord < kept && ord < first + kExpList) ? my_hw[32 * w] : 0u;
                    if (ord + __popc(word) <= first) {           // all of them before the window
                        ord += __popc(word);
                        word = 0u;
                    }
                    while (word) {
                        const int t = __ffs(word) - 1;
                        word &= word - 1;
                        if ((unsigned)(ord - first) < (unsigned)kExpList) my_list[ord - first] = (unsigned short)(w * 32 + t);
                        ord++;
                    }
                }
                __syncwarp();
                RPHASE(4)
                // ---- the lists -> edges: half a warp per centre, what it needs of the centre from a table, the next pair's
                //      entries read while this pair's edges are written
                const int take = max(0, min(min(ord, kept) - first, kExpList));
                const int64_t slot0 = base_off + first;
                s_par[lane] = make_int4(take, il, (int)(uint32_t)slot0, (int)(slot0 >> 32));
                __syncwarp();
                const int hsel = lane >> 4, l16 = lane & 15;
                int4 nxt = s_par[hsel];
                for (int pp = 0; pp < 16; pp++) {
                    const int4 cur = nxt;
                    const int cc = 2 * pp + hsel;
                    if (pp < 15) nxt = s_par[cc + 2];
                    const int tk = cur.x;
                    const int64_t slot_c = (int64_t)(((uint64_t)(uint32_t)cur.w << 32) | (uint32_t)cur.z), ic = lo + cur.y;
                    T cxi = T(0), cyi = T(0), czi = T(0);
                    if (o_dist) { cxi = __shfl_sync(full, pc.x, cc); cyi = __shfl_sync(full, pc.y, cc); czi = __shfl_sync(full, pc.z, cc); }
                    const unsigned short *hl = all_lists + cc * kExpListStride;
                    // (four rounds at a time: their list entries and indices are read together, then the edges written)
                    for (int t0 = l16; t0 < tk; t0 += 64) {
                        int jv[4];
#pragma unroll
                        for (int r = 0; r < 4; r++) jv[r] = t0 + 16 * r < tk ? (int)hl[t0 + 16 * r] : 0;
#pragma unroll
                        for (int r = 0; r < 4; r++) jv[r] = (int)sidx[jv[r]];
#pragma unroll
                        for (int r = 0; r < 4; r++) {
                            const int t = t0 + 16 * r;
                            if (t < tk) {
                                const int64_t gj = lo + jv[r], slot = slot_c + t;
                                if (o_row0) { o_row0[slot] = ic; o_row1[slot] = gj; }
                                if (o_batch) o_batch[slot] = b;
                                if (o_dist) o_dist[slot] = sqrt(dist2_rn(cxi, cyi, czi, pos[gj * 3], pos[gj * 3 + 1], pos[gj * 3 + 2]));
                                if (o_row0_32) { o_row0_32[slot] = (int32_t)ic; o_row1_32[slot] = (int32_t)gj; }
                            }
                        }
                    }
                }
                __syncwarp();
                RPHASE(5)
            }
        }
        __syncwarp();
    }
}

template <typename T>
static int expand_kernel_grid(int *grid) {
    static std::atomic<int> cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MLCGB_E_LAUNCH;
    int per_sm = cached[dev].load(std::memory_order_relaxed);
    if (per_sm == 0) {
        const size_t bytes = ExpandSmem<T>::total;
        if (cudaFuncSetAttribute(neighbours_block_expand_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess ||
            cudaFuncSetAttribute(neighbours_block_expand_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, 100) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, neighbours_block_expand_kernel<T>, 32, bytes) != cudaSuccess)
            return check_launch();
        if (per_sm < 1) per_sm = 1;
        cached[dev].store(per_sm, std::memory_order_relaxed);
    }
    *grid = kNumSM * per_sm;
    return MLCGB_OK;
}

template <typename T>
static int fill_kernel_grid(int *grid) {
    static std::atomic<int> cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MLCGB_E_LAUNCH;
    int per_sm = cached[dev].load(std::memory_order_relaxed);
    if (per_sm == 0) {
        const size_t bytes = FillSmem<T>::total;
        if (cudaFuncSetAttribute(neighbours_block_fill_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess ||
            cudaFuncSetAttribute(neighbours_block_fill_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, 100) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, neighbours_block_fill_kernel<T>, kFillWarps * 32, bytes) != cudaSuccess)
            return check_launch();
        if (per_sm < 1) per_sm = 1;
        cached[dev].store(per_sm, std::memory_order_relaxed);
    }
    *grid = kNumSM * per_sm;
    return MLCGB_OK;
}

template <typename T>
static int count_kernel_grid(int *grid) {
    // resident blocks per SM, asked once per device and kernel
    static std::atomic<int> cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MLCGB_E_LAUNCH;
    int per_sm = cached[dev].load(std::memory_order_relaxed);
    if (per_sm == 0) {
        const size_t bytes = CountSmem<T>::total;
        if (cudaFuncSetAttribute(neighbours_block_count_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess ||
            cudaFuncSetAttribute(neighbours_block_count_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, 100) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, neighbours_block_count_kernel<T>, 32, bytes) != cudaSuccess)
            return check_launch();
        if (per_sm < 1) per_sm = 1;
        cached[dev].store(per_sm, std::memory_order_relaxed);
    }
    *grid = kNumSM * per_sm;
    return MLCGB_OK;
}

#ifdef MLCGB_PHASE_TIMING
extern "C" int mlcgb_debug_radius_phase_cycles(unsigned long long *out, int n, int reset) {
    unsigned long long host[16];
    if (cudaMemcpyFromSymbol(host, g_radius_phase_cycles, sizeof(host)) != cudaSuccess) return MLCGB_E_LAUNCH;
    for (int i = 0; i < n && i < 16; i++) out[i] = host[i];
    if (reset) {
        unsigned long long zero[16] = {0};
        if (cudaMemcpyToSymbol(g_radius_phase_cycles, zero, sizeof(zero)) != cudaSuccess) return MLCGB_E_LAUNCH;
    }
    return MLCGB_OK;
}
#endif

__global__ void batch_to_ptr_kernel(const int64_t *__restrict__ batch, int64_t N, int64_t B, int64_t *__restrict__ ptr) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b > B) return;
    int64_t lo = 0, hi = N;  // first index with batch[idx] >= b
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (batch[mid] < b) lo = mid + 1; else hi = mid;
    }
    ptr[b] = lo;
}

__global__ void edge_twin_kernel(const int32_t *__restrict__ row0, const int32_t *__restrict__ row1,
                                 const int64_t *__restrict__ offsets, int64_t E, int64_t N, int32_t *__restrict__ twin,
                                 int32_t *__restrict__ status) {
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x) {
        const int a = row0[e], b = row1[e];
        int32_t t = -1;
        if (a >= 0 && a < N && b >= 0 && b < N) {
            int64_t lo = offsets[b], hi = offsets[b + 1];  // first k in b's segment with row1[k] >= a
            while (lo < hi) {
                const int64_t mid = (lo + hi) >> 1;
                if (row1[mid] < a) lo = mid + 1; else hi = mid;
            }
            if (lo < offsets[b + 1] && row1[lo] == a) t = (int32_t)lo;
        } else {
            atomicOr(status, (int)kBadIndex);
        }
        if (t < 0) atomicOr(status, (int)kAsymmetric);
        twin[e] = t;
    }
}

// pair_of[e] = k for the k-th selected edge and for its reverse
__global__ void pair_index_kernel(const int32_t *__restrict__ sel, const int32_t *__restrict__ twin, int64_t P,
                                  int32_t *__restrict__ pair_of) {
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < P; k += (int64_t)gridDim.x * blockDim.x) {
        const int32_t e = sel[k];
        pair_of[e] = (int32_t)k;
        const int32_t t = twin[e];
        if (t >= 0) pair_of[t] = (int32_t)k;
    }
}

// ---- pair plan of a symmetric, loop-free, centre-sorted list in one pass over the nodes, a scan and one pass over the edges.
// In centre i's segment the neighbours ascend, so its edges with row1 > i ("upper" edges, one per unordered pair) are the
// tail of the segment: upper[i] of them.
__global__ void upper_count_kernel(const int32_t *__restrict__ row1, const int64_t *__restrict__ offsets, int64_t N,
                                   int32_t *__restrict__ upper) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t lo = offsets[i], hi = offsets[i + 1];
        const int64_t end = hi;
        while (lo < hi) {                      // first k with row1[k] > i
            const int64_t mid = (lo + hi) >> 1;
            if (row1[mid] <= i) lo = mid + 1; else hi = mid;
        }
        upper[i] = (int32_t)(end - lo);
    }
}

// twin[e] as edge_twin_kernel; sel[p] = e and pair_of[e] = pair_of[twin[e]] = p, p = rank of the upper edge among all
// upper edges in list order (uoff = exclusive scan of upper)
__global__ void pair_plan_kernel(const int32_t *__restrict__ row0, const int32_t *__restrict__ row1, const int64_t *__restrict__ offsets,
                                 const int32_t *__restrict__ upper, const int64_t *__restrict__ uoff, int64_t E, int64_t N,
                                 int32_t *__restrict__ twin, int32_t *__restrict__ sel, int32_t *__restrict__ pair_of,
                                 int32_t *__restrict__ status) {
    // offsets[N] is the list's edge count; E may be the (larger) capacity of the buffers
    const int64_t total = offsets[N];
    const int64_t nE = total < E ? total : E;
    if ((nE & 1) && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, (int)kAsymmetric);
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nE; e += (int64_t)gridDim.x * blockDim.x) {
        const int a = row0[e], b = row1[e];
        int32_t t = -1;
        if (a >= 0 && a < N && b >= 0 && b < N) {
            int64_t lo = offsets[b], hi = offsets[b + 1];
            while (lo < hi) {
                const int64_t mid = (lo + hi) >> 1;
                if (row1[mid] < a) lo = mid + 1; else hi = mid;
            }
            if (lo < offsets[b + 1] && row1[lo] == a) t = (int32_t)lo;
        } else {
            atomicOr(status, (int)kBadIndex);
        }
        if (t < 0 || a == b) {               // not a valid plan: reported, and every index written stays inside its array
            atomicOr(status, (int)kAsymmetric);
            twin[e] = (int32_t)e;
            pair_of[e] = 0;
            continue;
        }
        twin[e] = t;
        if (b > a) {
            const int64_t p = uoff[a] + (e - (offsets[a + 1] - upper[a]));
            if (p >= (nE >> 1)) {              // more upper than lower edges: not symmetric
                atomicOr(status, (int)kAsymmetric);
                pair_of[e] = 0;
                continue;
            }
            sel[p] = (int32_t)e;
            pair_of[e] = (int32_t)p;
        } else {
            pair_of[e] = (int32_t)(uoff[b] + (t - (offsets[b + 1] - upper[b])));
        }
    }
}

// Capacity mode: the edge count stays on the device.  Offsets beyond the capacity of the edge buffers are clamped (the fill
// then writes at most `capacity` edges and the overflow is reported in the status word); counts = {edges, edges / 2}.
__global__ void clamp_offsets_kernel(int64_t *__restrict__ offsets, int64_t N, int64_t capacity, int64_t *__restrict__ counts,
                                     int32_t *__restrict__ status) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= N; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t o = offsets[i];
        if (o > capacity) {
            offsets[i] = o = capacity;
            if (i == N) atomicOr(status, (int)kCapacity);
        }
        if (i == N) {
            counts[0] = o;
            counts[1] = o >> 1;
        }
    }
}


// ------------------------------------------------------------------------------------------------
// Periodic structures (src/mlcg/neighbor_list/torch_impl.py:102-163, 252-329): the reference copies every structure
// (2 n_k + 1) times along each periodic cell vector, n_k = ceil(rcut * |row k of the transposed inverse cell|), and runs a
// bipartite radius search of the original points against all copies; a neighbour is (point j, shift s), listed per centre
// in the order of the copies (shift triples with the last index running fastest, points in order inside a copy), cut after
// max_num_neighbors, and the pair (j = i, s = 0) is dropped afterwards unless self pairs are asked for.
// Here the copies are never built: one warp per centre walks the shift triples and tests the structure's points, 32 at a
// time, against the centre; the copy's coordinates are pos[j] + shift, rounded once, as the reference stores them.
// shift = (s1 * c1 + s2 * c2) + s3 * c3 per component with separately rounded products and sums — exact for a cell with
// one non-zero entry per column (orthorhombic boxes); for a general cell a matrix-product routine may round differently.
// ------------------------------------------------------------------------------------------------
struct PbcOut {
    int64_t *row0, *row1, *mapping_batch;
    void *shifts, *distance;      // [E,3], [E]
};

template <typename T>
__device__ __forceinline__ void shift_vector(const T *__restrict__ cell, int s1, int s2, int s3, T &sx, T &sy, T &sz) {
    const T a = (T)s1, b = (T)s2, c = (T)s3;
    sx = add_rn(add_rn(mul_rn(a, cell[0]), mul_rn(b, cell[3])), mul_rn(c, cell[6]));
    sy = add_rn(add_rn(mul_rn(a, cell[1]), mul_rn(b, cell[4])), mul_rn(c, cell[7]));
    sz = add_rn(add_rn(mul_rn(a, cell[2]), mul_rn(b, cell[5])), mul_rn(c, cell[8]));
}

template <typename T, bool FILL>
__global__ void __launch_bounds__(256)
radius_pbc_kernel(const T *__restrict__ pos, const int64_t *__restrict__ ptr, const int32_t *__restrict__ struct_of, int64_t N,
                  const T *__restrict__ cells /* [B,3,3] */, const int32_t *__restrict__ repeats /* [B,3] */, T r2, int64_t max_nn,
                  int loop, int32_t *__restrict__ deg, const int64_t *__restrict__ offsets, PbcOut out, int32_t *__restrict__ status) {
    const int lane = threadIdx.x & 31;
    const unsigned lt = lanemask_lt();
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp; i < N; i += nwarps) {
        const int64_t b = struct_of[i];
        const int64_t lo = ptr[b];
        const int n = (int)(ptr[b + 1] - lo);
        const T *cell = cells + b * 9;
        const int n1 = repeats[b * 3], n2 = repeats[b * 3 + 1], n3 = repeats[b * 3 + 2];
        const T xi = pos[i * 3], yi = pos[i * 3 + 1], zi = pos[i * 3 + 2];
        int64_t kept = max_nn, base = 0;
        if (FILL) {
            base = offsets[i];
            if (offsets[i + 1] == base) continue;
        }
        int64_t hits = 0, emitted = 0;       // hits so far in list order (self included); edges written
        bool self_kept = false;
        for (int s1 = -n1; s1 <= n1 && hits < kept; s1++)
            for (int s2 = -n2; s2 <= n2 && hits < kept; s2++)
                for (int s3 = -n3; s3 <= n3 && hits < kept; s3++) {
                    T sx, sy, sz;
                    shift_vector<T>(cell, s1, s2, s3, sx, sy, sz);
                    const bool central = s1 == 0 && s2 == 0 && s3 == 0;
                    for (int jb = 0; jb < n && hits < kept; jb += 32) {
                        const int j = jb + lane;
                        bool hit = false;
                        T d2 = T(0);
                        if (j < n) {
                            const int64_t gj = lo + j;
                            d2 = dist2_rn(xi, yi, zi, add_rn(pos[gj * 3], sx), add_rn(pos[gj * 3 + 1], sy), add_rn(pos[gj * 3 + 2], sz));
                            hit = d2 < r2;
                        }
                        const unsigned bal = __ballot_sync(0xffffffffu, hit);
                        const int64_t rank = hits + __popc(bal & lt);
                        const bool in_list = hit && rank < kept;
                        const bool is_self = central && lo + j == i;
                        if (FILL) {
                            const bool write = in_list && (loop || !is_self);
                            const unsigned wbal = __ballot_sync(0xffffffffu, write);
                            if (write) {
                                const int64_t slot = base + emitted + __popc(wbal & lt);
                                out.row0[slot] = i;
                                out.row1[slot] = lo + j;
                                if (out.mapping_batch) out.mapping_batch[slot] = b;
                                T *sh = (T *)out.shifts + slot * 3;
                                sh[0] = sx; sh[1] = sy; sh[2] = sz;
                                if (out.distance) ((T *)out.distance)[slot] = sqrt(d2);
                            }
                            emitted += __popc(wbal);
                        } else {
                            self_kept = self_kept || __any_sync(0xffffffffu, in_list && is_self);
                        }
                        hits += __popc(bal);
                    }
                }
        if (!FILL && lane == 0) {
            const int64_t k = hits < kept ? hits : kept;
            deg[i] = (int32_t)(k - ((self_kept && !loop) ? 1 : 0));
            if (hits >= kept && kept > 0) {
                // the walk stopped at the cap: whether more would have followed is not known without finishing it; the cap
                // was reached, which is what callers need to know
                atomicOr(status, (int)kTruncated);
            }
        }
    }
}

__global__ void struct_of_kernel(const int64_t *__restrict__ ptr, int64_t B, int32_t *__restrict__ struct_of) {
    for (int64_t b = blockIdx.x; b < B; b += gridDim.x)
        for (int64_t i = ptr[b] + threadIdx.x; i < ptr[b + 1]; i += blockDim.x) struct_of[i] = (int32_t)b;
}

template <typename T>
static int radius_launch(bool fill, const void *pos_, const int64_t *ptr, int64_t N, int64_t B, double r, int64_t max_nn,
                         int loop, int rule, void *ws, size_t ws_bytes, int dtype, int32_t *deg, int64_t *offsets,
                         FillOut out, int32_t *status, cudaStream_t st, Exclusion ex = Exclusion{}) {
    const WsLayout L = ws_layout(N, B, dtype);
    if (ws_bytes < L.total) return MLCGB_E_WORKSPACE;
    char *w = (char *)ws;
    const T *pos = (const T *)pos_;
    auto *spos = (V4<T> *)(w + L.spos);
    auto *cellparam = (CellParam *)(w + L.cellparam);
    auto *cell_of = (int32_t *)(w + L.cell_of);
    auto *cell_start = (int32_t *)(w + L.cell_start);
    auto *struct_of = (int32_t *)(w + L.struct_of);
    auto *bsum = (int64_t *)(w + L.bsum);
    auto *group_ptr = (int32_t *)(w + L.group_ptr);
    auto *hits = (unsigned *)(w + L.hits);
    auto *cidx = (int32_t *)(w + L.cidx);
    auto *item_flag = (unsigned char *)(w + L.item_flag);
    const T r2 = (T)(r * r);
    const int nbr_grid = grid_for(N, kNbrWarps, 32);
    // the block kernels take structures with a cell grid and at most kCapBits points (none when pairs are excluded); a batch
    // of small structures only (fewer points than one cell-grid structure needs, on average) cannot hold one
    const bool tiles = !ex.ptr && N > kBruteMax;
    const int32_t *n_plain = tiles ? group_ptr + B + 1 : nullptr;
    if (!fill) {
        build_cells_kernel<T><<<grid_for(B, 1, 8), kBuildThreads, 0, st>>>(pos, ptr, B, (T)r, tiles ? 1 : 0, spos, cellparam, cell_of, cell_start, struct_of, cidx);
        if (tiles) {
            group_scan_kernel<<<1, kScanBlock, 0, st>>>(cellparam, B, group_ptr);
            int grid = 0;
            const int rc = count_kernel_grid<T>(&grid);
            if (rc != MLCGB_OK) return rc;
            neighbours_block_count_kernel<T><<<grid, 32, CountSmem<T>::total, st>>>(ptr, B, r2, max_nn, loop, rule, spos, cellparam, cell_start,
                                                                                 group_ptr, deg, cidx, hits, item_flag, status);
        }
        if (ex.ptr)
            neighbours_kernel<T, false, true><<<nbr_grid, kNbrWarps * 32, 0, st>>>(pos, ptr, N, B, r2, max_nn, loop, rule, spos, cellparam,
                                                                                   cell_of, cell_start, struct_of, deg, nullptr, out, ex, status, n_plain);
        else
            neighbours_kernel<T, false, false><<<nbr_grid, kNbrWarps * 32, 0, st>>>(pos, ptr, N, B, r2, max_nn, loop, rule, spos, cellparam,
                                                                                    cell_of, cell_start, struct_of, deg, nullptr, out, ex, status, n_plain);
        launch_scan(deg, N, bsum, offsets, st);
    } else {
        if (tiles) {
            int grid = 0;
            int rc = expand_kernel_grid<T>(&grid);
            if (rc != MLCGB_OK) return rc;
            neighbours_block_expand_kernel<T><<<grid, 32, ExpandSmem<T>::total, st>>>(pos, ptr, B, loop, spos, cellparam, cell_start, group_ptr,
                                                                                    cidx, hits, offsets, out);
            // (the items that left no hit masks, if the counting pass met any: tested again)
            rc = fill_kernel_grid<T>(&grid);
            if (rc != MLCGB_OK) return rc;
            neighbours_block_fill_kernel<T><<<grid, kFillWarps * 32, FillSmem<T>::total, st>>>(
                pos, ptr, B, r2, loop, spos, cellparam, cell_start, group_ptr, item_flag, offsets, out);
        }
        if (ex.ptr)
            neighbours_kernel<T, true, true><<<nbr_grid, kNbrWarps * 32, 0, st>>>(pos, ptr, N, B, r2, max_nn, loop, rule, spos, cellparam,
                                                                                  cell_of, cell_start, struct_of, nullptr, offsets, out, ex, status, n_plain);
        else
            neighbours_kernel<T, true, false><<<nbr_grid, kNbrWarps * 32, 0, st>>>(pos, ptr, N, B, r2, max_nn, loop, rule, spos, cellparam,
                                                                                   cell_of, cell_start, struct_of, nullptr, offsets, out, ex, status, n_plain);
    }
    return check_launch();
}

}  // namespace mlcgb

using namespace mlcgb;

extern "C" {

int mlcgb_batch_to_ptr(const int64_t *batch, int64_t N, int64_t B, int64_t *ptr, void *stream) {
    TimelineScope timeline_scope("batch_to_ptr", stream);
    if (N < 0 || B < 0 || !ptr || (N > 0 && !batch)) return MLCGB_E_ARG;
    batch_to_ptr_kernel<<<(unsigned)((B + 1 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(batch, N, B, ptr);
    return check_launch();
}

size_t mlcgb_radius_workspace_bytes(int64_t N, int64_t B, int dtype) {
    if (N < 0 || B < 0) return 0;
    return ws_layout(N, B, dtype).total;
}

static int radius_count_impl(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int64_t max_nn, int loop,
                             int rule, void *workspace, size_t workspace_bytes, int32_t *deg, int64_t *offsets, int32_t *status,
                             void *stream, Exclusion ex) {
    if (N < 0 || B < 0 || max_nn < 0 || !offsets || !status || !ptr || !workspace) return MLCGB_E_ARG;
    if (N >= (int64_t)1 << 31) return MLCGB_E_LIMIT;
    if (rule != MLCGB_RULE_NATIVE && rule != MLCGB_RULE_CLUSTER) return MLCGB_E_ARG;
    if (N == 0) {
        cudaMemsetAsync(offsets, 0, sizeof(int64_t), (cudaStream_t)stream);
        return check_launch();
    }
    if (!pos || !deg || B == 0) return MLCGB_E_ARG;
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        return radius_launch<scalar_t>(false, pos, ptr, N, B, r, max_nn, loop, rule, workspace, workspace_bytes, dtype, deg,
                                       offsets, FillOut{}, status, (cudaStream_t)stream, ex);
    });
}

int mlcgb_radius_count(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int64_t max_nn, int loop,
                       int rule, void *workspace, size_t workspace_bytes, int32_t *deg, int64_t *offsets, int32_t *status,
                       void *stream) {
    TimelineScope timeline_scope("radius_count", stream);
    return radius_count_impl(pos, dtype, ptr, N, B, r, max_nn, loop, rule, workspace, workspace_bytes, deg, offsets, status, stream, Exclusion{});
}

int mlcgb_radius_count_excl(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int64_t max_nn, int loop,
                            const int64_t *exclude_pair_xs, const int64_t *ptr_exclude_pair_xs, void *workspace, size_t workspace_bytes,
                            int32_t *deg, int64_t *offsets, int32_t *status, void *stream) {
    TimelineScope timeline_scope("radius_count", stream);
    if (!exclude_pair_xs != !ptr_exclude_pair_xs) return MLCGB_E_ARG;
    Exclusion ex;
    ex.xs = exclude_pair_xs;
    ex.ptr = ptr_exclude_pair_xs;
    return radius_count_impl(pos, dtype, ptr, N, B, r, max_nn, loop, MLCGB_RULE_NATIVE, workspace, workspace_bytes, deg, offsets, status, stream, ex);
}

static int radius_fill_impl(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int loop,
                            const void *workspace, size_t workspace_bytes, const int64_t *offsets, int64_t E, int64_t *edge_index,
                            void *distance, int64_t *mapping_batch, int32_t *row0_i32, int32_t *row1_i32, int32_t *status,
                            void *stream, Exclusion ex) {
    if (N < 0 || B < 0 || E < 0 || !offsets || !status || !ptr || !workspace) return MLCGB_E_ARG;
    if (E == 0 || N == 0) return MLCGB_OK;
    if (!pos || !edge_index) return MLCGB_E_ARG;
    FillOut out{edge_index, edge_index + E, mapping_batch, distance, row0_i32, row1_i32};
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        return radius_launch<scalar_t>(true, pos, ptr, N, B, r, 0, loop, 0, const_cast<void *>(workspace), workspace_bytes, dtype,
                                       nullptr, const_cast<int64_t *>(offsets), out, status, (cudaStream_t)stream, ex);
    });
}

int mlcgb_radius_fill(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int loop,
                      const void *workspace, size_t workspace_bytes, const int64_t *offsets, int64_t E, int64_t *edge_index,
                      void *distance, int64_t *mapping_batch, int32_t *row0_i32, int32_t *row1_i32, int32_t *status,
                      void *stream) {
    TimelineScope timeline_scope("radius_fill", stream);
    return radius_fill_impl(pos, dtype, ptr, N, B, r, loop, workspace, workspace_bytes, offsets, E, edge_index, distance, mapping_batch,
                            row0_i32, row1_i32, status, stream, Exclusion{});
}

int mlcgb_radius_fill_excl(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int loop,
                           const int64_t *exclude_pair_xs, const int64_t *ptr_exclude_pair_xs, const void *workspace,
                           size_t workspace_bytes, const int64_t *offsets, int64_t E, int64_t *edge_index, void *distance,
                           int64_t *mapping_batch, int32_t *row0_i32, int32_t *row1_i32, int32_t *status, void *stream) {
    TimelineScope timeline_scope("radius_fill", stream);
    if (!exclude_pair_xs != !ptr_exclude_pair_xs) return MLCGB_E_ARG;
    Exclusion ex;
    ex.xs = exclude_pair_xs;
    ex.ptr = ptr_exclude_pair_xs;
    return radius_fill_impl(pos, dtype, ptr, N, B, r, loop, workspace, workspace_bytes, offsets, E, edge_index, distance, mapping_batch,
                            row0_i32, row1_i32, status, stream, ex);
}

int mlcgb_edge_twin(const int32_t *row0, const int32_t *row1, const int64_t *offsets, int64_t E, int64_t N, int32_t *twin,
                    int32_t *status, void *stream) {
    TimelineScope timeline_scope("edge_twin", stream);
    if (E < 0 || N < 0 || !status) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!row0 || !row1 || !offsets || !twin) return MLCGB_E_ARG;
    edge_twin_kernel<<<grid_for(E, 256), 256, 0, (cudaStream_t)stream>>>(row0, row1, offsets, E, N, twin, status);
    return check_launch();
}

size_t mlcgb_pair_plan_workspace_bytes(int64_t N) {
    if (N < 0) return 0;
    return align256((size_t)N * 4) + align256((size_t)(N + 1) * 8) + align256((size_t)((N + kScanBlock - 1) / kScanBlock + 1) * 8);
}

int mlcgb_pair_plan(const int32_t *row0, const int32_t *row1, const int64_t *offsets, int64_t E, int64_t N, void *workspace,
                    size_t workspace_bytes, int32_t *twin, int32_t *sel, int32_t *pair_of, int32_t *status, void *stream) {
    TimelineScope timeline_scope("pair_plan", stream);
    if (E < 0 || N < 0 || (E & 1) || !status) return MLCGB_E_ARG;
    if (E == 0) return MLCGB_OK;
    if (!row0 || !row1 || !offsets || !twin || !sel || !pair_of || !workspace) return MLCGB_E_ARG;
    if (workspace_bytes < mlcgb_pair_plan_workspace_bytes(N)) return MLCGB_E_WORKSPACE;
    auto st = (cudaStream_t)stream;
    char *w = (char *)workspace;
    auto *upper = (int32_t *)w;
    auto *uoff = (int64_t *)(w + align256((size_t)N * 4));
    auto *bsum = (int64_t *)(w + align256((size_t)N * 4) + align256((size_t)(N + 1) * 8));
    upper_count_kernel<<<grid_for(N, 256), 256, 0, st>>>(row1, offsets, N, upper);
    launch_scan(upper, N, bsum, uoff, st);
    pair_plan_kernel<<<grid_for(E, 256), 256, 0, st>>>(row0, row1, offsets, upper, uoff, E, N, twin, sel, pair_of, status);
    return check_launch();
}

size_t mlcgb_radius_pbc_workspace_bytes(int64_t N) {
    if (N < 0) return 0;
    return align256((size_t)N * 4) + align256((size_t)((N + kScanBlock - 1) / kScanBlock + 1) * 8);
}

int mlcgb_radius_pbc_count(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, const void *cells, const int32_t *repeats,
                           double r, int64_t max_nn, int loop, void *workspace, size_t workspace_bytes, int32_t *deg, int64_t *offsets,
                           int32_t *status, void *stream) {
    TimelineScope timeline_scope("radius_pbc_count", stream);
    if (N < 0 || B < 0 || max_nn < 0 || !offsets || !status || !ptr || !workspace) return MLCGB_E_ARG;
    if (N >= (int64_t)1 << 31) return MLCGB_E_LIMIT;
    auto st = (cudaStream_t)stream;
    if (N == 0) {
        cudaMemsetAsync(offsets, 0, sizeof(int64_t), st);
        return check_launch();
    }
    if (!pos || !deg || !cells || !repeats || B == 0) return MLCGB_E_ARG;
    if (workspace_bytes < mlcgb_radius_pbc_workspace_bytes(N)) return MLCGB_E_WORKSPACE;
    auto *struct_of = (int32_t *)workspace;
    auto *bsum = (int64_t *)((char *)workspace + align256((size_t)N * 4));
    struct_of_kernel<<<grid_for(B, 1, 8), 256, 0, st>>>(ptr, B, struct_of);
    int rc = MLCGB_DISPATCH_DTYPE(dtype, [&] {
        const scalar_t r2 = (scalar_t)(r * r);
        radius_pbc_kernel<scalar_t, false><<<grid_for(N * 32, 256), 256, 0, st>>>((const scalar_t *)pos, ptr, struct_of, N, (const scalar_t *)cells,
                                                                                  repeats, r2, max_nn, loop, deg, nullptr, PbcOut{}, status);
        return MLCGB_OK;
    });
    if (rc) return rc;
    launch_scan(deg, N, bsum, offsets, st);
    return check_launch();
}

int mlcgb_radius_pbc_fill(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, const void *cells, const int32_t *repeats,
                          double r, int64_t max_nn, int loop, const void *workspace, size_t workspace_bytes, const int64_t *offsets,
                          int64_t E, int64_t *edge_index, void *cell_shifts, void *distance, int64_t *mapping_batch, int32_t *status,
                          void *stream) {
    TimelineScope timeline_scope("radius_pbc_fill", stream);
    if (N < 0 || B < 0 || E < 0 || max_nn < 0 || !offsets || !status || !ptr || !workspace) return MLCGB_E_ARG;
    if (E == 0 || N == 0) return MLCGB_OK;
    if (!pos || !cells || !repeats || !edge_index || !cell_shifts) return MLCGB_E_ARG;
    if (workspace_bytes < mlcgb_radius_pbc_workspace_bytes(N)) return MLCGB_E_WORKSPACE;
    auto st = (cudaStream_t)stream;
    const auto *struct_of = (const int32_t *)workspace;      // as the count call left it
    PbcOut out{edge_index, edge_index + E, mapping_batch, cell_shifts, distance};
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        const scalar_t r2 = (scalar_t)(r * r);
        radius_pbc_kernel<scalar_t, true><<<grid_for(N * 32, 256), 256, 0, st>>>((const scalar_t *)pos, ptr, struct_of, N, (const scalar_t *)cells,
                                                                                 repeats, r2, max_nn, loop, nullptr, offsets, out, status);
        return check_launch();
    });
}

int mlcgb_pair_index(const int32_t *sel, const int32_t *twin, int64_t P, int32_t *pair_of, void *stream) {
    TimelineScope timeline_scope("pair_index", stream);
    if (P < 0) return MLCGB_E_ARG;
    if (P == 0) return MLCGB_OK;
    if (!sel || !twin || !pair_of) return MLCGB_E_ARG;
    pair_index_kernel<<<grid_for(P, 256), 256, 0, (cudaStream_t)stream>>>(sel, twin, P, pair_of);
    return check_launch();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Radius graph for callers that cannot allocate device memory.
//
// The two-call path above takes its workspace from the caller (the Python wrapper gets it from torch's
// caching allocator).  Code that runs where no allocator may be called — a force callback inside
// another engine's time-step loop, a plug-in whose host forbids cudaMalloc after start-up, a thread
// that must not take the allocator's locks — uses this single call instead: the cell-list scratch
// lives in a fixed array that is part of the library image, and inputs and outputs stay the caller's.
// ------------------------------------------------------------------------------------------------
namespace mlcgb {
constexpr int64_t kStaticMaxPoints = 65536;
constexpr int64_t kStaticMaxStructures = 8192;
constexpr size_t kStaticScratchBytes = (size_t)17 << 19;  // 8.5 MB >= ws_layout(65536, 8192, float32).total = 8 782 848 (float64: 6 685 696)
static __device__ __align__(256) unsigned char g_radius_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::atomic<void *> g_scratch_addr[kMaxDevices];      // zero-initialised; every writer stores the same address per device

// The array's name is only a host-side handle; the device address has to be asked for, once per
// device, with that device current.
static int static_scratch_address(void **out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MLCGB_E_ARG;
    void *p = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_radius_scratch);
        if (e != cudaSuccess || !p) {
            g_last_cuda_error = (int)e;
            return MLCGB_E_LAUNCH;
        }
        g_scratch_addr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return MLCGB_OK;
}
}  // namespace mlcgb

extern "C" int mlcgb_radius_graph_capacity(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r, int64_t max_nn,
                                           int loop, int rule, void *workspace, size_t workspace_bytes, int32_t *deg, int64_t *offsets,
                                           int64_t capacity, int64_t *edge_index, int32_t *row0_i32, int32_t *row1_i32,
                                           int64_t *counts, int32_t *status, void *stream) {
    TimelineScope timeline_scope("radius_graph_capacity", stream);
    if (capacity < 0 || !counts || (!edge_index && (!row0_i32 || !row1_i32))) return MLCGB_E_ARG;
    if (N <= 0 || B <= 0) return MLCGB_E_ARG;
    int rc = mlcgb_radius_count(pos, dtype, ptr, N, B, r, max_nn, loop, rule, workspace, workspace_bytes, deg, offsets, status, stream);
    if (rc != MLCGB_OK) return rc;
    auto st = (cudaStream_t)stream;
    clamp_offsets_kernel<<<grid_for(N + 1, 256), 256, 0, st>>>(offsets, N, capacity, counts, status);
    if (capacity == 0) return check_launch();
    FillOut out{edge_index, edge_index ? edge_index + capacity : nullptr, nullptr, nullptr, row0_i32, row1_i32};
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        return radius_launch<scalar_t>(true, pos, ptr, N, B, r, 0, loop, 0, workspace, workspace_bytes, dtype, nullptr, offsets, out, status,
                                       st);
    });
}

extern "C" int mlcgb_radius_graph_static(const void *pos, int dtype, const int64_t *ptr, int64_t N, int64_t B, double r,
                                         int64_t max_nn, int loop, int rule, int32_t *deg, int64_t *offsets, int64_t capacity,
                                         int64_t *edge_index, int64_t *n_edges_host, int32_t *status, void *stream) {
    TimelineScope timeline_scope("radius_graph_static", stream);
    if (N < 0 || B < 0 || max_nn < 0 || capacity < 0 || !offsets || !status || !ptr || !n_edges_host) return MLCGB_E_ARG;
    if (dtype != MLCGB_F32 && dtype != MLCGB_F64) return MLCGB_E_ARG;
    if (N > kStaticMaxPoints || B > kStaticMaxStructures) return MLCGB_E_LIMIT;   // beyond the built-in scratch
    if (ws_layout(N, B, dtype).total > kStaticScratchBytes) return MLCGB_E_LIMIT;
    void *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    auto st = (cudaStream_t)stream;
    *n_edges_host = 0;
    int rc = mlcgb_radius_count(pos, dtype, ptr, N, B, r, max_nn, loop, rule, scratch, kStaticScratchBytes, deg, offsets, status, stream);
    if (rc != MLCGB_OK) return rc;
    int64_t E = 0;
    cudaError_t e = cudaMemcpyAsync(&E, offsets + N, sizeof(int64_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return MLCGB_E_LAUNCH;
    }
    *n_edges_host = E;
    if (E > capacity) return MLCGB_E_LIMIT;   // the caller's edge buffer is too small; n_edges_host says how many are needed
    if (E == 0 || N == 0) return MLCGB_OK;
    if (!pos || !edge_index) return MLCGB_E_ARG;
    // rows of the caller's [2, capacity] buffer
    FillOut out{edge_index, edge_index + capacity, nullptr, nullptr, nullptr, nullptr};
    return MLCGB_DISPATCH_DTYPE(dtype, [&] {
        return radius_launch<scalar_t>(true, pos, ptr, N, B, r, 0, loop, 0, scratch, kStaticScratchBytes, dtype, nullptr, offsets, out,
                                       status, st);
    });
}
