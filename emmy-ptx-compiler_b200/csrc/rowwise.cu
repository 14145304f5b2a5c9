// Row-wise reductions over the last axis of a contiguous fp32 [rows, cols] array, and the normalisations built
// on them (softmax, log-softmax, layer norm, RMS norm, L2 normalise).
//
// In the reference a reduction is a per-thread `Accum` loop (emmyptx/kernel.py:786-797) whose partial states
// are merged by a `WarpShuffle` butterfly (:856-866) and, across warps, by a `TreeHalve` over shared slabs
// (:868-900); the combine step is an ordinary Assign program. The cases are those of
// tools/torch_cases/reductions.py:6-19 and fused.py:6-13. Here the same three levels are fixed in CUDA:
//
//   * rowwise_cached_kernel: a row is held in registers by a group of G threads (8 to 256, by row length) or,
//     beyond 8192 elements, by the 2, 4 or 8 CTAs of a thread-block cluster, which exchange their partial
//     results through distributed shared memory; so the array is read once and written at most once, with
//     128-bit accesses; the grid is a multiple of the SM count and walks the rows.
//   * rowwise_split_kernel: rows longer than a group can hold are cut into pieces, one CTA each; a piece's state
//     goes to workspace memory and the CTA that takes the last ticket of a row merges the pieces in index order
//     (so the result does not depend on which CTA that was). No CTA waits for another.
//   * rowwise_map_kernel: the second pass of a normalisation over such long rows.
//
// Across pieces every op is a mergeable state: sums; extrema (NaN wins, as torch); products; (n, mean, M2) merged
// with Chan's formula; (max, sum of exp) for the softmax family; (value, first index) for argmax. Within a cached
// row the moments and the softmax family take two rounds of plain all-reduces instead (sum, then squared
// deviations; max, then exponentials), which is cheaper than merging pairs and costs no second read.
#include <limits.h>
#include <math_constants.h>

#include <mutex>

#include "common.cuh"
#include "emmy_math.cuh"
#include "reduce_state.cuh"

namespace emmy {
namespace {

// ---- thread-block clusters: a row wider than one CTA's registers is held by up to 8 CTAs -------------------------
__device__ __forceinline__ uint32_t cluster_size() { uint32_t v; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(v)); return v; }
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t v; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(v)); return v; }
// A hardware barrier over the CTAs of the cluster (they are scheduled together); release / acquire so that shared
// memory written before it is visible to the peers after it.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Reads a float at the same shared-memory offset in the CTA of rank `rank`.
__device__ __forceinline__ float peer_shared_load(const float* local, uint32_t rank) {
    uint32_t addr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// Shared memory of the all-reduce: [2][32] per-warp states and [2] per-CTA states, alternated by `round` so that one
// barrier per reduction is enough (a buffer is rewritten two reductions later, after a barrier every reader has
// passed).
struct ReduceSlabs {
    St warp[64];
    St cta[2];
};

// All-reduce over a group of G consecutive threads (a part of a warp, a warp, or the whole CTA) and then, if the
// CTA belongs to a cluster, over the CTAs of the cluster in rank order. Every thread returns the same bits.
template <int K, int G>
__device__ __forceinline__ St group_allreduce(St s, ReduceSlabs* slabs, int& round) {
    const int lane = threadIdx.x & 31;
    s = warp_allreduce<K>(s, G < 32 ? G : 32, lane);
    if constexpr (G > 32) {
        const int buf = round & 1;
        ++round;
        St* slab = slabs->warp + buf * 32;
        if (lane == 0) slab[threadIdx.x >> 5] = s;
        const int first_warp = (threadIdx.x / G) * (G / 32);    // of this group
        if constexpr (G == 256) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + (int)threadIdx.x / G), "n"(G) : "memory");      // the group only
        s = lane < G / 32 ? slab[first_warp + lane] : st_identity<K>();
        s = warp_allreduce<K>(s, 32, lane);                     // identities in the upper lanes: every lane gets the result
    }
    return s;
}

// All-reduce of per-CTA states (every thread of a CTA holding its CTA's) over the cluster, in rank order: one
// hardware barrier, then each CTA reads its peers' states through distributed shared memory.
template <int K>
__device__ __forceinline__ St cluster_allreduce(St s, ReduceSlabs* slabs, int& cround, uint32_t csize) {
    const int lane = threadIdx.x & 31;
    const int buf = cround & 1;
    ++cround;
    if (threadIdx.x == 0) slabs->cta[buf] = s;
    cluster_barrier();
    St o = st_identity<K>();
    if ((uint32_t)lane < csize) {
        o.a = peer_shared_load(&slabs->cta[buf].a, lane);
        if constexpr (K == K_MOM || K == K_LSE || K == K_DOT3) o.b = peer_shared_load(&slabs->cta[buf].b, lane);
        if constexpr (K == K_MOM || K == K_ARG || K == K_DOT3) o.c = peer_shared_load(&slabs->cta[buf].c, lane);
    }
    s = warp_allreduce<K>(o, 8, lane);                          // at most 8 CTAs, in lanes 0-7
    s.a = __shfl_sync(0xffffffffu, s.a, 0);
    if constexpr (K == K_MOM || K == K_LSE || K == K_DOT3) s.b = __shfl_sync(0xffffffffu, s.b, 0);
    if constexpr (K == K_MOM || K == K_ARG || K == K_DOT3) s.c = __shfl_sync(0xffffffffu, s.c, 0);
    return s;
}

struct RowArgs {
    const float* x;
    const float* w;
    const float* b;
    void* y;
    int64_t rows;
    int64_t cols;
    float eps;
};

// Final statistics of a row: what a reducing op stores, or the two numbers a map needs.
// ---- rows that fit a group's registers -----------------------------------------------------------------------
constexpr int kPerThread = 32;     // elements a thread holds
constexpr int kMaxCluster = 8;     // the portable cluster size

// G threads hold a row; with G = 256 the CTAs of a cluster hold consecutive 256 * 32-element slices of it.
template <int OP, int G, int VEC>
__global__ void __launch_bounds__(256) rowwise_cached_kernel(RowArgs a) {
    constexpr int K = kind_of(OP);
    constexpr int kRowsPerBlock = 256 / G;
    constexpr int kIter = kPerThread / VEC;
    __shared__ ReduceSlabs slabs;
    int round = 0, cround = 0;
    const uint32_t csize = G == 256 ? cluster_size() : 1u;
    const uint32_t crank = G == 256 ? cluster_rank() : 0u;
    const int t = threadIdx.x % G, g = threadIdx.x / G;
    const int cols = (int)a.cols;
    const int first = (int)crank * kIter * G + t;               // this thread's first access, in units of VEC elements
    const int slice_end = ((int)crank * kIter) * G * VEC;       // (columns before this CTA's slice)
    const int64_t unit = blockIdx.x / csize, n_units = gridDim.x / csize;

    for (int64_t rb = unit * kRowsPerBlock; rb < a.rows; rb += n_units * kRowsPerBlock) {
        const int64_t row = rb + g;
        const bool live = row < a.rows;
        const float* xr = a.x + row * a.cols;
        float v[kPerThread];
        // All loads first. Column of element (i, e) is (first + i * G) * VEC + e.
#pragma unroll
        for (int i = 0; i < kIter; ++i) {
            if (slice_end + i * G * VEC >= cols) break;         // uniform over the CTA: the rest of the row does not exist
            const int c = (first + i * G) * VEC;
            if (live && c < cols) {
                if constexpr (VEC == 4) {
                    const float4 q = __ldcs(reinterpret_cast<const float4*>(xr + c));
                    v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
                    if constexpr (OP == EMMYB200_ROW_DOT) {     // the products with the vector are what is summed
                        const float4 wq = __ldg(reinterpret_cast<const float4*>(a.w + c));
                        v[4 * i] *= wq.x; v[4 * i + 1] *= wq.y; v[4 * i + 2] *= wq.z; v[4 * i + 3] *= wq.w;
                    }
                } else {
                    v[i] = __ldcs(xr + c);
                    if constexpr (OP == EMMYB200_ROW_DOT) v[i] *= __ldg(a.w + c);
                }
            }
        }
        // Statistics in one or two rounds of plain all-reduces (the held values make a second pass free): sum, then
        // squared deviations from the mean; max, then exponentials against it; max, then the first column equal to it.
        constexpr int K1 = K == K_MOM ? K_ADD : ((K == K_LSE || K == K_ARG) ? K_MAX : K);
        St s = st_identity<K1>();
        // Extrema go through the one-instruction hardware max / min, which drops NaNs; a sum of x * 2^-120 on the FMA
        // pipe (NaN iff the values hold a NaN, or infinities of both signs) tells when the careful version is needed.
        float nan_probe = 0.0f;
#pragma unroll
        for (int i = 0; i < kIter; ++i) {
            if (slice_end + i * G * VEC >= cols) break;
            const int c = (first + i * G) * VEC;
            if (live && c < cols) {
#pragma unroll
                float wv[VEC];
                if constexpr (K1 == K_DOT3) {                   // the second matrix streams by: it is not needed again
                    const float* wr = a.w + row * a.cols + c;
                    if constexpr (VEC == 4) { const float4 q = __ldcs(reinterpret_cast<const float4*>(wr)); wv[0] = q.x; wv[1] = q.y; wv[2] = q.z; wv[3] = q.w; }
                    else wv[0] = __ldcs(wr);
                }
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const float x = v[VEC * i + e];
                    if constexpr (K1 == K_DOT3) { s.a = fmaf(x, wv[e], s.a); s.b = fmaf(x, x, s.b); s.c = fmaf(wv[e], wv[e], s.c); }
                    else if constexpr (K1 == K_ADD) s.a += x;
                    else if constexpr (K1 == K_SQ) s.a = fmaf(x, x, s.a);
                    else if constexpr (K1 == K_MAX) { s.a = fmaxf(s.a, x); nan_probe = fmaf(x, 0x1p-120f, nan_probe); }
                    else if constexpr (K1 == K_MIN) { s.a = fminf(s.a, x); nan_probe = fmaf(x, 0x1p-120f, nan_probe); }
                    else s.a *= x;
                }
            }
        }
        if constexpr (K1 == K_MAX || K1 == K_MIN) {
            if (nan_probe != nan_probe) {
#pragma unroll
                for (int i = 0; i < kIter; ++i) {
                    if (slice_end + i * G * VEC >= cols) break;
                    const int c = (first + i * G) * VEC;
                    if (live && c < cols) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) s.a = K1 == K_MAX ? nan_max(s.a, v[VEC * i + e]) : nan_min(s.a, v[VEC * i + e]);
                    }
                }
            }
        }
        const float own = s.a;                                  // this thread's extremum (argmax looks only where it is the row's)
        s = group_allreduce<K1, G>(s, &slabs, round);           // over the row, or over this CTA's slice of it
        if constexpr (K == K_MOM || K == K_LSE || K == K_ARG) {
            // of the slice this CTA holds (the whole row without a cluster): its mean, or its max
            const int held = min(cols - slice_end, kIter * G * VEC);
            const float centre = K == K_MOM ? (held > 0 ? s.a / (float)held : 0.0f) : s.a;
            const bool max_is_nan = centre != centre;
            int hit = INT_MAX;
            St s2 = st_identity<K == K_ARG ? K_MIN : K_ADD>();
#pragma unroll
            for (int i = kIter - 1; i >= 0; --i) {                          // downwards: the lowest matching column is kept
                const int c = (first + i * G) * VEC;
                if constexpr (K == K_ARG) {
                    if (!(own == centre || max_is_nan)) break;               // the maximum is not among this thread's values
                }
                if (slice_end + i * G * VEC < cols && live && c < cols) {
#pragma unroll
                    for (int e = VEC - 1; e >= 0; --e) {
                        const float x = v[VEC * i + e];
                        if constexpr (K == K_MOM) {
                            const float d = x - centre;
                            s2.a = fmaf(d, d, s2.a);
                        } else if constexpr (K == K_LSE) {
                            const float p = centre == -CUDART_INF_F ? 0.0f : exp_le0(x - centre);
                            s2.a += p;
                            if constexpr (OP == EMMYB200_ROW_SOFTMAX) v[VEC * i + e] = p;
                        } else {
                            if (x == centre || (max_is_nan && x != x)) hit = i * G * VEC + e;      // a constant: no index registers
                        }
                    }
                }
            }
            // columns < 2^24 are exact as floats; INT_MAX stands for "none here"
            if constexpr (K == K_ARG) s2.a = hit == INT_MAX ? (float)INT_MAX : (float)(hit + first * VEC);
            s2 = group_allreduce<K == K_ARG ? K_MIN : K_ADD, G>(s2, &slabs, round);
            if constexpr (K == K_MOM) s = {(float)max(held, 0), centre, s2.a};
            else if constexpr (K == K_LSE) s = {centre, s2.a, 0.0f};
            else s = {centre, 0.0f, __int_as_float((int)s2.a)};
        }
        const float own_centre = s.a;                           // softmax: the max the held exponentials were taken against
        if constexpr (G == 256) {
            if (csize > 1) s = cluster_allreduce<K>(s, &slabs, cround, csize);      // one exchange of whole states per row
        }
        const float2 r = row_finish<OP>(s, (float)cols, a.eps);

        if constexpr (!is_map(OP)) {
            if (live && t == 0 && crank == 0) store_reduced<OP>(a.y, row, s, r);
        } else {
            float* yr = static_cast<float*>(a.y) + row * a.cols;
            // softmax: exp(x - row max) / sum = the held exp(x - slice max) * exp(slice max - row max) / sum
            float soft = r.y;
            if constexpr (OP == EMMYB200_ROW_SOFTMAX && G == 256) {
                if (csize > 1) soft = exp_le0(own_centre - r.x) * r.y;
            }
#pragma unroll
            for (int i = 0; i < kIter; ++i) {
                if (slice_end + i * G * VEC >= cols) break;
                const int c = (first + i * G) * VEC;
                if (live && c < cols) {
                    float wv[VEC], bv[VEC], o[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) { wv[e] = 1.0f; bv[e] = 0.0f; }
                    if constexpr (OP == EMMYB200_ROW_LAYER_NORM || OP == EMMYB200_ROW_RMS_NORM) {
                        if constexpr (VEC == 4) {
                            if (a.w) { const float4 q = __ldg(reinterpret_cast<const float4*>(a.w + c)); wv[0] = q.x; wv[1] = q.y; wv[2] = q.z; wv[3] = q.w; }
                            if (a.b) { const float4 q = __ldg(reinterpret_cast<const float4*>(a.b + c)); bv[0] = q.x; bv[1] = q.y; bv[2] = q.z; bv[3] = q.w; }
                        } else {
                            if (a.w) wv[0] = __ldg(a.w + c);
                            if (a.b) bv[0] = __ldg(a.b + c);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        if constexpr (OP == EMMYB200_ROW_SOFTMAX) o[e] = v[VEC * i + e] * soft;     // the exponential is held
                        else o[e] = row_map<OP>(v[VEC * i + e], r, wv[e], bv[e]);
                    }
                    if constexpr (VEC == 4) __stcs(reinterpret_cast<float4*>(yr + c), make_float4(o[0], o[1], o[2], o[3]));
                    else __stcs(yr + c, o[0]);
                }
            }
        }
    }
    if (csize > 1) cluster_barrier();       // no CTA leaves while a peer may still read its shared memory
}

// ---- rows cut into pieces ------------------------------------------------------------------------------------
constexpr int kSplitThreads = 256;

// Folds elements [c0, c1) of one row into a state, kSplitThreads threads together; every thread returns it.
template <int K, int VEC>
__device__ __forceinline__ St piece_state(const float* xr, const float* w, int64_t c0, int64_t c1, ReduceSlabs* slabs, int& round) {
    St s = st_identity<K>();
    float shift = 0.0f, s1 = 0.0f, s2 = 0.0f, cnt = 0.0f;
    if constexpr (K == K_MOM) shift = __ldg(xr + c0);          // sums are taken about a sample of the piece
    constexpr int kTrip = 4;                                    // accesses in flight per thread
    const int64_t step = (int64_t)kSplitThreads * VEC;
    for (int64_t base = c0 + (int64_t)threadIdx.x * VEC; base < c1; base += step * kTrip) {
        float v[kTrip][VEC];
        float wv[K == K_DOT3 ? kTrip : 1][VEC];
#pragma unroll
        for (int k = 0; k < kTrip; ++k) {
            const int64_t c = base + k * step;
            if (c < c1) {
                if constexpr (VEC == 4) {
                    const float4 q = __ldcs(reinterpret_cast<const float4*>(xr + c));
                    v[k][0] = q.x; v[k][1] = q.y; v[k][2] = q.z; v[k][3] = q.w;
                } else {
                    v[k][0] = __ldcs(xr + c);
                }
                if constexpr (K == K_DOT3) {                    // cosine: w is the same row of the second matrix
#pragma unroll
                    for (int e = 0; e < VEC; ++e) wv[k][e] = __ldcs(w + c + e);
                } else if (w != nullptr) {                      // dot product: fold x * w (uniform over the grid)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) v[k][e] *= __ldg(w + c + e);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < kTrip; ++k) {
            const int64_t c = base + k * step;
            if (c >= c1) continue;
            if constexpr (K == K_LSE) {
                float m = v[k][0];
#pragma unroll
                for (int e = 1; e < VEC; ++e) m = nan_max(m, v[k][e]);
                if (m > s.a || m != m) {                       // raise the max, rescale what was summed so far
                    s.b = s.a == -CUDART_INF_F ? 0.0f : s.b * exp_le0(s.a - m);
                    s.a = m;
                }
                if (s.a != -CUDART_INF_F) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) s.b += exp_le0(v[k][e] - s.a);
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const float x = v[k][e];
                    if constexpr (K == K_DOT3) { const float y = wv[k][e]; s.a = fmaf(x, y, s.a); s.b = fmaf(x, x, s.b); s.c = fmaf(y, y, s.c); }
                    else if constexpr (K == K_ADD) s.a += x;
                    else if constexpr (K == K_SQ) s.a = fmaf(x, x, s.a);
                    else if constexpr (K == K_MAX) s.a = nan_max(s.a, x);
                    else if constexpr (K == K_MIN) s.a = nan_min(s.a, x);
                    else if constexpr (K == K_MUL) s.a *= x;
                    else if constexpr (K == K_MOM) { const float d = x - shift; s1 += d; s2 = fmaf(d, d, s2); }
                    else arg_push(s, x, (int)(c + e));
                }
                cnt += (float)VEC;
            }
        }
    }
    if constexpr (K == K_MOM) {
        if (cnt > 0.0f) {
            const float dm = s1 / cnt;
            s = {cnt, shift + dm, fmaxf(s2 - s1 * dm, 0.0f)};
        }
    }
    return group_allreduce<K, kSplitThreads>(s, slabs, round);
}

// grid = rows * pieces. `partials` [rows][pieces] states, `tickets` [rows] zeroed before the launch (and left
// zero after it), `stats` [rows] the finished pair of a mapping op.
template <int OP, int VEC>
__global__ void __launch_bounds__(kSplitThreads) rowwise_split_kernel(RowArgs a, int pieces, int64_t piece_len, float4* partials,
                                                                       unsigned int* tickets, float2* stats) {
    constexpr int K = kind_of(OP);
    __shared__ ReduceSlabs slabs;
    __shared__ int is_last;
    int round = 0;
    const int64_t row = blockIdx.x / pieces;
    const int piece = blockIdx.x % pieces;
    const float* xr = a.x + row * a.cols;
    const int64_t c0 = (int64_t)piece * piece_len;
    const int64_t c1 = c0 + piece_len < a.cols ? c0 + piece_len : a.cols;
    St s = piece_state<K, VEC>(xr, OP == EMMYB200_ROW_DOT ? a.w : (OP == EMMYB200_ROW_COSINE ? a.w + row * a.cols : nullptr), c0, c1, &slabs, round);
    if (pieces > 1) {
        if (threadIdx.x == 0) {
            partials[row * pieces + piece] = make_float4(s.a, s.b, s.c, 0.0f);
            __threadfence();
            const unsigned int ticket = atomicAdd(tickets + row, 1u);
            is_last = ticket == (unsigned int)pieces - 1u;
            if (is_last) tickets[row] = 0;                      // ready for the next launch
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        // pieces in index order: thread t takes a contiguous run, then the ordered butterfly
        const int per = (pieces + kSplitThreads - 1) / kSplitThreads;
        s = st_identity<K>();
        for (int i = 0; i < per; ++i) {
            const int q = threadIdx.x * per + i;
            if (q < pieces) {
                const float4 f = __ldcg(partials + row * pieces + q);
                s = st_merge<K>(s, St{f.x, f.y, f.z});
            }
        }
        s = group_allreduce<K, kSplitThreads>(s, &slabs, round);
    }
    if (threadIdx.x == 0) {
        const float2 r = row_finish<OP>(s, (float)a.cols, a.eps);
        if constexpr (is_map(OP)) stats[row] = r;
        else store_reduced<OP>(a.y, row, s, r);
    }
}

// y = map(x, stats[row]) over long rows: blockIdx.y walks the rows, blockIdx.x the columns.
template <int OP, int VEC>
__global__ void __launch_bounds__(256) rowwise_map_kernel(RowArgs a, const float2* stats) {
    for (int64_t row = blockIdx.y; row < a.rows; row += gridDim.y) {
        const float2 r = stats[row];
        const float* xr = a.x + row * a.cols;
        float* yr = static_cast<float*>(a.y) + row * a.cols;
        for (int64_t c = ((int64_t)blockIdx.x * 256 + threadIdx.x) * VEC; c < a.cols; c += (int64_t)gridDim.x * 256 * VEC) {
            float xv[VEC], wv[VEC], bv[VEC], o[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) { wv[e] = 1.0f; bv[e] = 0.0f; }
            if constexpr (VEC == 4) {
                const float4 q = __ldcs(reinterpret_cast<const float4*>(xr + c));
                xv[0] = q.x; xv[1] = q.y; xv[2] = q.z; xv[3] = q.w;
                if constexpr (OP == EMMYB200_ROW_LAYER_NORM || OP == EMMYB200_ROW_RMS_NORM) {
                    if (a.w) { const float4 p = __ldg(reinterpret_cast<const float4*>(a.w + c)); wv[0] = p.x; wv[1] = p.y; wv[2] = p.z; wv[3] = p.w; }
                    if (a.b) { const float4 p = __ldg(reinterpret_cast<const float4*>(a.b + c)); bv[0] = p.x; bv[1] = p.y; bv[2] = p.z; bv[3] = p.w; }
                }
            } else {
                xv[0] = __ldcs(xr + c);
                if constexpr (OP == EMMYB200_ROW_LAYER_NORM || OP == EMMYB200_ROW_RMS_NORM) {
                    if (a.w) wv[0] = __ldg(a.w + c);
                    if (a.b) bv[0] = __ldg(a.b + c);
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[e] = row_map<OP>(xv[e], r, wv[e], bv[e]);
            if constexpr (VEC == 4) __stcs(reinterpret_cast<float4*>(yr + c), make_float4(o[0], o[1], o[2], o[3]));
            else __stcs(yr + c, o[0]);
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------------------
constexpr int64_t kMaxCachedCols = (int64_t)kMaxCluster * 256 * kPerThread;      // 8 CTAs of 256 threads, 32 elements each
constexpr int64_t kMinPiece = 8192;

struct SplitPlan {
    int pieces;
    int64_t piece_len;
    size_t partial_bytes, ticket_bytes, stat_bytes;
    size_t total() const { return partial_bytes + ticket_bytes + stat_bytes; }
};

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

SplitPlan plan_split(int64_t rows, int64_t cols) {
    SplitPlan p;
    const int64_t by_len = (cols + kMinPiece - 1) / kMinPiece;
    const int64_t by_fill = (4 * (int64_t)sm_count() + rows - 1) / (rows > 0 ? rows : 1);
    int64_t pieces = by_len < by_fill ? by_len : by_fill;
    if (pieces < 1) pieces = 1;
    if (pieces > 1024) pieces = 1024;
    int64_t len = (cols + pieces - 1) / pieces;
    len = (len + 3) / 4 * 4;                                    // pieces start on 16-byte boundaries of the row
    p.piece_len = len;
    p.pieces = (int)((cols + len - 1) / len);
    p.partial_bytes = round_up((size_t)rows * p.pieces * sizeof(float4), 256);
    p.ticket_bytes = round_up((size_t)rows * sizeof(unsigned int), 256);
    p.stat_bytes = round_up((size_t)rows * sizeof(float2), 256);
    return p;
}

template <int OP, int G, int VEC>
int launch_cached(const RowArgs& a, int cluster, cudaStream_t s) {
    constexpr int kRowsPerBlock = 256 / G;
    const int64_t units = (a.rows + kRowsPerBlock - 1) / kRowsPerBlock;
    const int64_t cap = (int64_t)sm_count() * 16 / cluster;         // a few waves of 256-thread CTAs
    const int64_t n_units = units < cap ? units : cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_units * cluster));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)cluster;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = cluster > 1 ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, rowwise_cached_kernel<OP, G, VEC>, a);
    if (e != cudaSuccess) return cuda_fail(e, "launch of rowwise_cached_kernel");
    return launch_status("rowwise_cached_kernel");
}

template <int OP, int VEC>
int launch_op(const RowArgs& a, void* ws, cudaStream_t s) {
    const int64_t per = a.cols / VEC + (a.cols % VEC != 0);      // accesses per row
    if (a.cols <= kMaxCachedCols) {
        constexpr int kIter = kPerThread / VEC;
        if (per <= 8 * kIter) return launch_cached<OP, 8, VEC>(a, 1, s);
        if (per <= 16 * kIter) return launch_cached<OP, 16, VEC>(a, 1, s);
        if (per <= 32 * kIter) return launch_cached<OP, 32, VEC>(a, 1, s);
        if (per <= 64 * kIter) return launch_cached<OP, 64, VEC>(a, 1, s);
        if (per <= 128 * kIter) return launch_cached<OP, 128, VEC>(a, 1, s);
        const int64_t slices = (per + 256 * kIter - 1) / (256 * kIter);
        return launch_cached<OP, 256, VEC>(a, slices <= 1 ? 1 : (slices <= 2 ? 2 : (slices <= 4 ? 4 : 8)), s);
    }
    const SplitPlan p = plan_split(a.rows, a.cols);
    char* base = static_cast<char*>(ws);
    float4* partials = reinterpret_cast<float4*>(base);
    unsigned int* tickets = reinterpret_cast<unsigned int*>(base + p.partial_bytes);
    float2* stats = reinterpret_cast<float2*>(base + p.partial_bytes + p.ticket_bytes);
    if (p.pieces > 1) EMMY_CUDA(cudaMemsetAsync(tickets, 0, (size_t)a.rows * sizeof(unsigned int), s));
    rowwise_split_kernel<OP, VEC><<<(unsigned)(a.rows * p.pieces), kSplitThreads, 0, s>>>(a, p.pieces, p.piece_len, partials, tickets, stats);
    int rc = launch_status("rowwise_split_kernel");
    if (rc != EMMYB200_OK) return rc;
    if constexpr (is_map(OP)) {
        const int64_t col_blocks = (per + 256 * 4 - 1) / (256 * 4);
        dim3 grid((unsigned)(col_blocks < 65535 ? col_blocks : 65535), (unsigned)(a.rows < 65535 ? a.rows : 65535));
        rowwise_map_kernel<OP, VEC><<<grid, 256, 0, s>>>(a, stats);
        rc = launch_status("rowwise_map_kernel");
    }
    return rc;
}

template <int VEC>
int dispatch(int op, const RowArgs& a, void* ws, cudaStream_t s) {
    switch (op) {
#define EMMY_ROW_CASE(name) case EMMYB200_ROW_##name: return launch_op<EMMYB200_ROW_##name, VEC>(a, ws, s);
        EMMY_ROW_CASE(SUM) EMMY_ROW_CASE(MEAN) EMMY_ROW_CASE(AMAX) EMMY_ROW_CASE(AMIN) EMMY_ROW_CASE(PROD)
        EMMY_ROW_CASE(VAR) EMMY_ROW_CASE(STD) EMMY_ROW_CASE(NORM2) EMMY_ROW_CASE(LOGSUMEXP) EMMY_ROW_CASE(ARGMAX) EMMY_ROW_CASE(DOT) EMMY_ROW_CASE(COSINE)
        EMMY_ROW_CASE(SOFTMAX) EMMY_ROW_CASE(LOG_SOFTMAX) EMMY_ROW_CASE(LAYER_NORM) EMMY_ROW_CASE(RMS_NORM)
        EMMY_ROW_CASE(NORMALIZE)
#undef EMMY_ROW_CASE
    }
    return fail(EMMYB200_ERR_ARG, "rowwise: unknown op %d", op);
}

bool known_op(int op) { return (op >= EMMYB200_ROW_SUM && op <= EMMYB200_ROW_COSINE) || (op >= EMMYB200_ROW_SOFTMAX && op <= EMMYB200_ROW_NORMALIZE); }

}  // namespace
}  // namespace emmy

extern "C" int64_t emmyb200_rowwise_workspace_bytes(int op, int64_t rows, int64_t cols) {
    using namespace emmy;
    if (!known_op(op) || rows < 0 || cols < 1 || cols >= ((int64_t)1 << 31)) return -1;
    if (rows == 0 || cols <= kMaxCachedCols) return 0;
    return (int64_t)plan_split(rows, cols).total();
}

extern "C" int emmyb200_rowwise_f32(int op, const float* x, const float* weight, const float* bias, void* y, int64_t rows,
                                    int64_t cols, float eps, void* workspace, int64_t workspace_bytes, void* cuda_stream) {
    using namespace emmy;
    if (!known_op(op)) return fail(EMMYB200_ERR_ARG, "rowwise: unknown op %d", op);
    if (rows < 0 || cols < 0) return fail(EMMYB200_ERR_ARG, "rowwise: negative extent");
    if (rows == 0) return EMMYB200_OK;
    if (cols < 1) return fail(EMMYB200_ERR_SHAPE, "rowwise: a row needs at least one element");
    if (cols >= ((int64_t)1 << 31) || rows >= ((int64_t)1 << 31)) return fail(EMMYB200_ERR_SHAPE, "rowwise: extents are limited to 2^31 - 1");
    if (x == nullptr || y == nullptr) return fail(EMMYB200_ERR_ARG, "rowwise: null buffer");
    const bool affine = op == EMMYB200_ROW_LAYER_NORM || op == EMMYB200_ROW_RMS_NORM;
    if (op == EMMYB200_ROW_DOT || op == EMMYB200_ROW_COSINE) {
        if (weight == nullptr || bias != nullptr) return fail(EMMYB200_ERR_ARG, "rowwise: dot and cosine take their second operand as `weight` and no bias");
    } else if (!affine && (weight != nullptr || bias != nullptr)) {
        return fail(EMMYB200_ERR_ARG, "rowwise: only layer_norm, rms_norm and dot take a weight or bias");
    }
    if (op == EMMYB200_ROW_RMS_NORM && bias != nullptr) return fail(EMMYB200_ERR_ARG, "rowwise: rms_norm has no bias");
    if (!aligned(x, 4) || !aligned(y, is_map(op) ? 4 : (op == EMMYB200_ROW_ARGMAX ? 8 : 4)))
        return fail(EMMYB200_ERR_ALIGN, "rowwise: buffers must be aligned to their element size");
    const int64_t need = emmyb200_rowwise_workspace_bytes(op, rows, cols);
    if (need > 0) {
        if (workspace == nullptr || workspace_bytes < need)
            return fail(EMMYB200_ERR_ARG, "rowwise: rows of %lld elements need %lld bytes of workspace", (long long)cols, (long long)need);
        if (!aligned(workspace, 256)) return fail(EMMYB200_ERR_ALIGN, "rowwise: the workspace must be 256-byte aligned");
        if (rows * (int64_t)plan_split(rows, cols).pieces >= ((int64_t)1 << 31)) return fail(EMMYB200_ERR_SHAPE, "rowwise: too many pieces");
    }
    RowArgs a{x, weight, bias, y, rows, cols, eps};
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    const bool vec = cols % 4 == 0 && aligned(x, 16) && (!is_map(op) || aligned(y, 16)) &&
                     (weight == nullptr || aligned(weight, 16)) && (bias == nullptr || aligned(bias, 16));
    return vec ? dispatch<4>(op, a, workspace, s) : dispatch<1>(op, a, workspace, s);
}

// ---- the same call with the library's own scratch memory -----------------------------------------------------------
// Piece states, tickets and row statistics of the split path live in a fixed array in the library's device image
// instead of caller memory. Its address is looked up once per device; nothing is allocated or freed, here or later.
namespace emmy {
namespace {
constexpr int64_t kStaticScratchBytes = 1 << 20;
static __device__ __align__(256) unsigned char g_row_scratch[kStaticScratchBytes];

int static_scratch(void** out) {
    static void* cached[64];
    static std::mutex lock;
    int dev = 0;
    EMMY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(EMMYB200_ERR_DEVICE, "rowwise_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> guard(lock);
    if (cached[dev] == nullptr) EMMY_CUDA(cudaGetSymbolAddress(&cached[dev], g_row_scratch));
    *out = cached[dev];
    return EMMYB200_OK;
}
}  // namespace
}  // namespace emmy

extern "C" int64_t emmyb200_rowwise_static_capacity(void) { return emmy::kStaticScratchBytes; }

extern "C" int emmyb200_rowwise_f32_static(int op, const float* x, const float* weight, const float* bias, void* y, int64_t rows,
                                           int64_t cols, float eps, void* cuda_stream) {
    using namespace emmy;
    const int64_t need = emmyb200_rowwise_workspace_bytes(op, rows, cols);
    if (need > kStaticScratchBytes)
        return fail(EMMYB200_ERR_SHAPE, "rowwise_static: %lld rows of %lld elements need %lld bytes of scratch, the library holds %lld",
                    (long long)rows, (long long)cols, (long long)need, (long long)kStaticScratchBytes);
    void* scratch = nullptr;
    if (need > 0) {
        const int rc = static_scratch(&scratch);
        if (rc != EMMYB200_OK) return rc;
    }
    return emmyb200_rowwise_f32(op, x, weight, bias, y, rows, cols, eps, scratch, need > 0 ? kStaticScratchBytes : 0, cuda_stream);
}
