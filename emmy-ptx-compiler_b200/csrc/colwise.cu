// Reductions over the middle axis of a contiguous fp32 [outer, rows, cols] array (a reduction over dim 0 of a
// matrix is outer = 1), the normalisations over that axis, and the running sum along the last axis.
//
// The reference's cases: tools/torch_cases/reductions.py:9-10 (`x.sum(0)`, `x.sum((0, 2))` as a row pass followed by
// this one), :18 (`cumsum`), fused.py:7 (`softmax(x, 0)`). Its kernels walk the reduced axis with an `Accum` loop per
// output element (emmyptx/kernel.py:786-797); here the walk is arranged for the memory system:
//
//   * colwise_kernel: a CTA is 32 column lanes (one 128-bit load each, so a warp reads 512 contiguous bytes of a row)
//     by 8 row lanes; it folds a slice of the rows for 128 columns, the 8 row lanes merge through shared memory, and
//     when the rows were split over several CTAs the slice states go to workspace memory and the CTA that draws the
//     last ticket of its column tile merges them in a fixed order (no CTA waits for another; the result does not
//     depend on block scheduling). The states are those of the row kernels (reduce_state.cuh).
//   * colwise_map_kernel: the second pass of softmax / log-softmax / normalise over that axis.
//   * cumsum_kernel: a group of 32 or 256 threads streams a row slab by slab (128-bit accesses), scanning inside a
//     thread, across the group by shuffles (and shared memory between warps), and carrying the slab total on.
#include "common.cuh"
#include "emmy_math.cuh"
#include "reduce_state.cuh"

namespace emmy {
namespace {

constexpr int kColLanes = 32, kRowLanes = 8, kColThreads = kColLanes * kRowLanes;

// Folds one element (index `idx` along the reduced axis) into a state. MOM accumulates sums about `shift`.
template <int K>
__device__ __forceinline__ void st_push(St& s, float x, int idx, float shift) {
    if constexpr (K == K_ADD) s.a += x;
    else if constexpr (K == K_SQ) s.a = fmaf(x, x, s.a);
    else if constexpr (K == K_MAX) s.a = nan_max(s.a, x);
    else if constexpr (K == K_MIN) s.a = nan_min(s.a, x);
    else if constexpr (K == K_MUL) s.a *= x;
    else if constexpr (K == K_MOM) { const float d = x - shift; s.b += d; s.c = fmaf(d, d, s.c); }      // the count is set by the caller
    else if constexpr (K == K_LSE) {
        if (x > s.a || x != x) {                            // a new maximum: rescale what was summed so far
            s.b = (s.a == -CUDART_INF_F ? 0.0f : s.b * exp_le0(s.a - x)) + exp_le0(x - x);      // 1, or NaN for an infinity, as torch
            s.a = x;
        } else if (s.a != -CUDART_INF_F) {
            s.b += exp_le0(x - s.a);
        }
    } else {
        arg_push(s, x, idx);
    }
}

// (count, sum of d, sum of d^2) about `shift` -> (n, mean, M2)
__device__ __forceinline__ St moments_from_shifted(St s, float shift) {
    if (s.a == 0.0f) return {0.0f, 0.0f, 0.0f};
    const float dm = s.b / s.a;
    return {s.a, shift + dm, fmaxf(s.c - s.b * dm, 0.0f)};
}

struct ColArgs {
    const float* x;
    void* y;
    int64_t outer, rows, cols;
    float eps;
    int splits;             // CTAs along the reduced axis
    int64_t rows_per_split;
};

// grid = (column tiles, splits, outer). partials: [outer][splits][cols] states; tickets: [outer][column tiles];
// stats: [outer][cols], the finished pair of a mapping op.
template <int OP, int VEC>
__global__ void __launch_bounds__(kColThreads) colwise_kernel(ColArgs a, float4* partials, unsigned int* tickets, float2* stats) {
    constexpr int K = kind_of(OP);
    __shared__ float4 slab[kRowLanes][kColLanes * VEC];
    __shared__ int is_last;
    const int cx = threadIdx.x % kColLanes, ry = threadIdx.x / kColLanes;
    const int64_t col0 = ((int64_t)blockIdx.x * kColLanes + cx) * VEC;
    const int split = blockIdx.y;
    const int64_t o = blockIdx.z;
    const bool in_cols = col0 < a.cols;                         // cols % VEC == 0 when VEC == 4
    const int64_t r_begin = (int64_t)split * a.rows_per_split;
    const int64_t r_end = r_begin + a.rows_per_split < a.rows ? r_begin + a.rows_per_split : a.rows;
    const float* base = a.x + o * a.rows * a.cols + col0;

    St s[VEC];
    float shift[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) { s[e] = (K == K_MOM) ? St{0.0f, 0.0f, 0.0f} : st_identity<K>(); shift[e] = 0.0f; }
    if constexpr (K == K_MOM) {
        if (in_cols && r_begin < r_end) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) shift[e] = __ldg(base + r_begin * a.cols + e);
        }
    }
    if (in_cols) {
        constexpr int kTrip = 4;                                // rows in flight per thread
        const int rb = (int)r_begin, re = (int)r_end;           // rows < 2^31
        for (int r = rb + ry; r < re; r += kRowLanes * kTrip) {
            float v[kTrip][VEC];
            const float* row = base + (int64_t)r * a.cols;
#pragma unroll
            for (int k = 0; k < kTrip; ++k) {
                if (r + k * kRowLanes < re) {
                    if constexpr (VEC == 4) {
                        const float4 q = __ldcs(reinterpret_cast<const float4*>(row + (int64_t)k * kRowLanes * a.cols));
                        v[k][0] = q.x; v[k][1] = q.y; v[k][2] = q.z; v[k][3] = q.w;
                    } else {
                        v[k][0] = __ldcs(row + (int64_t)k * kRowLanes * a.cols);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < kTrip; ++k) {
                if (r + k * kRowLanes < re) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) st_push<K>(s[e], v[k][e], r + k * kRowLanes, shift[e]);
                }
            }
        }
        if constexpr (K == K_MOM) {                             // rows rb + ry, rb + ry + 8, ... below re
            const int mine = re - rb > ry ? (re - rb - ry + kRowLanes - 1) / kRowLanes : 0;
#pragma unroll
            for (int e = 0; e < VEC; ++e) s[e].a = (float)mine;
        }
    }
    // the 8 row lanes of a column merge in lane order (lane ry holds rows ry, ry + 8, ...: for argmax the merge
    // compares indices, for everything else the order only fixes the rounding)
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        const St t = (K == K_MOM) ? moments_from_shifted(s[e], shift[e]) : s[e];
        slab[ry][cx * VEC + e] = make_float4(t.a, t.b, t.c, 0.0f);
    }
    __syncthreads();
    St m[VEC];
    if (ry == 0) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            m[e] = St{slab[0][cx * VEC + e].x, slab[0][cx * VEC + e].y, slab[0][cx * VEC + e].z};
            for (int l = 1; l < kRowLanes; ++l) {
                const float4 f = slab[l][cx * VEC + e];
                m[e] = st_merge<K>(m[e], St{f.x, f.y, f.z});
            }
        }
    }
    if (a.splits > 1) {
        if (ry == 0 && in_cols) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) partials[(o * a.splits + split) * a.cols + col0 + e] = make_float4(m[e].a, m[e].b, m[e].c, 0.0f);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int* t = tickets + o * gridDim.x + blockIdx.x;
            const unsigned int ticket = atomicAdd(t, 1u);
            is_last = ticket == (unsigned int)a.splits - 1u;
            if (is_last) *t = 0;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        // The slices are merged in a fixed order whichever CTA does it: row lane ry folds slices ry, ry + 8, ..., then
        // the eight lanes fold through shared memory as above.
        St t[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) t[e] = st_identity<K>();
        if (in_cols) {
            for (int sp = ry; sp < a.splits; sp += kRowLanes) {
                const float4* src = partials + (o * a.splits + sp) * a.cols + col0;
                float4 f[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) f[e] = __ldcg(src + e);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = st_merge<K>(t[e], St{f[e].x, f[e].y, f[e].z});
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) slab[ry][cx * VEC + e] = make_float4(t[e].a, t[e].b, t[e].c, 0.0f);
        __syncthreads();
        if (ry == 0) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                m[e] = St{slab[0][cx * VEC + e].x, slab[0][cx * VEC + e].y, slab[0][cx * VEC + e].z};
                for (int l = 1; l < kRowLanes; ++l) {
                    const float4 f = slab[l][cx * VEC + e];
                    m[e] = st_merge<K>(m[e], St{f.x, f.y, f.z});
                }
            }
        }
    }
    if (ry == 0 && in_cols) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float2 r = row_finish<OP>(m[e], (float)a.rows, a.eps);
            if constexpr (is_map(OP)) stats[o * a.cols + col0 + e] = r;
            else store_reduced<OP>(a.y, o * a.cols + col0 + e, m[e], r);
        }
    }
}

template <int OP, int VEC>
__global__ void __launch_bounds__(256) colwise_map_kernel(ColArgs a, const float2* stats) {
    const int64_t per_row = a.cols / VEC;
    const int64_t total = a.outer * a.rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t c = (i % per_row) * VEC;
        const int64_t o = i / (per_row * a.rows);
        const float* xp = a.x + i * VEC;
        float* yp = static_cast<float*>(a.y) + i * VEC;
        if constexpr (VEC == 4) {
            const float4 q = __ldcs(reinterpret_cast<const float4*>(xp));
            const float2 r0 = stats[o * a.cols + c], r1 = stats[o * a.cols + c + 1], r2 = stats[o * a.cols + c + 2], r3 = stats[o * a.cols + c + 3];
            __stcs(reinterpret_cast<float4*>(yp), make_float4(row_map<OP>(q.x, r0, 1.0f, 0.0f), row_map<OP>(q.y, r1, 1.0f, 0.0f),
                                                              row_map<OP>(q.z, r2, 1.0f, 0.0f), row_map<OP>(q.w, r3, 1.0f, 0.0f)));
        } else {
            __stcs(yp, row_map<OP>(__ldcs(xp), stats[o * a.cols + c], 1.0f, 0.0f));
        }
    }
}

// ---- running sum along the last axis ---------------------------------------------------------------------------
// G threads per row (32: a warp, 8 rows per CTA; 256: the CTA). A slab is G * VEC consecutive elements.
template <int G, int VEC>
__global__ void __launch_bounds__(256) cumsum_kernel(const float* x, float* y, int64_t rows, int64_t cols) {
    constexpr int kRowsPerBlock = 256 / G;
    __shared__ float warp_tot[2][8];
    const int t = threadIdx.x % G, g = threadIdx.x / G, lane = threadIdx.x & 31;
    int round = 0;
    for (int64_t rb = (int64_t)blockIdx.x * kRowsPerBlock; rb < rows; rb += (int64_t)gridDim.x * kRowsPerBlock) {
        const int64_t row = rb + g;
        const bool live = row < rows;
        const float* xr = x + row * cols;
        float* yr = y + row * cols;
        float carry = 0.0f;
        for (int64_t c0 = 0; c0 < cols; c0 += (int64_t)G * VEC) {
            const int64_t c = c0 + (int64_t)t * VEC;
            float v[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = 0.0f;
            if (live && c < cols) {
                if constexpr (VEC == 4) {
                    const float4 q = __ldcs(reinterpret_cast<const float4*>(xr + c));
                    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
                } else {
                    v[0] = __ldcs(xr + c);
                }
            }
#pragma unroll
            for (int e = 1; e < VEC; ++e) v[e] += v[e - 1];      // inside the thread
            float incl = v[VEC - 1];                            // inclusive scan of the thread totals over the warp
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += up;
            }
            float before = __shfl_up_sync(0xffffffffu, incl, 1);    // total of the lower lanes of this warp
            if (lane == 0) before = 0.0f;
            float slab_total = __shfl_sync(0xffffffffu, incl, 31);
            if constexpr (G == 256) {                           // and of the lower warps
                const int buf = round & 1;
                ++round;
                if (lane == 31) warp_tot[buf][threadIdx.x >> 5] = incl;
                __syncthreads();
                float lower = 0.0f, all = 0.0f;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const float tw = warp_tot[buf][w];
                    if (w < (int)(threadIdx.x >> 5)) lower += tw;
                    all += tw;
                }
                before += lower;
                slab_total = all;
            }
            if (live && c < cols) {
                const float add = carry + before;
                if constexpr (VEC == 4) __stcs(reinterpret_cast<float4*>(yr + c), make_float4(v[0] + add, v[1] + add, v[2] + add, v[3] + add));
                else __stcs(yr + c, v[0] + add);
            }
            carry += slab_total;
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------------------
size_t round_up256(size_t v) { return (v + 255) / 256 * 256; }

struct ColPlan {
    int splits;
    int64_t rows_per_split, col_tiles;
    size_t partial_bytes, ticket_bytes, stat_bytes;
    size_t total() const { return partial_bytes + ticket_bytes + stat_bytes; }
};

ColPlan plan_cols(int op, int64_t outer, int64_t rows, int64_t cols, int vec) {
    ColPlan p;
    p.col_tiles = (cols + kColLanes * vec - 1) / (kColLanes * vec);
    const int64_t ctas = p.col_tiles * outer;
    int64_t want = (6 * (int64_t)sm_count() + ctas - 1) / ctas;          // enough CTAs to fill the GPU a few times
    const int64_t most = rows / 64 > 0 ? rows / 64 : 1;                   // at least 64 rows per slice
    if (want > most) want = most;
    if (want > 1024) want = 1024;
    if (want < 1) want = 1;
    p.rows_per_split = (rows + want - 1) / want;
    p.splits = (int)((rows + p.rows_per_split - 1) / p.rows_per_split);
    p.partial_bytes = p.splits > 1 ? round_up256((size_t)outer * p.splits * cols * sizeof(float4)) : 0;
    p.ticket_bytes = p.splits > 1 ? round_up256((size_t)outer * p.col_tiles * sizeof(unsigned int)) : 0;
    p.stat_bytes = is_map(op) ? round_up256((size_t)outer * cols * sizeof(float2)) : 0;
    return p;
}

bool col_op(int op) {
    return (op >= EMMYB200_ROW_SUM && op <= EMMYB200_ROW_ARGMAX) || op == EMMYB200_ROW_SOFTMAX || op == EMMYB200_ROW_LOG_SOFTMAX ||
           op == EMMYB200_ROW_NORMALIZE;
}

template <int OP, int VEC>
int launch_col(const ColArgs& a0, const ColPlan& p, void* ws, cudaStream_t s) {
    ColArgs a = a0;
    a.splits = p.splits;
    a.rows_per_split = p.rows_per_split;
    char* base = static_cast<char*>(ws);
    float4* partials = reinterpret_cast<float4*>(base);
    unsigned int* tickets = reinterpret_cast<unsigned int*>(base + p.partial_bytes);
    float2* stats = reinterpret_cast<float2*>(base + p.partial_bytes + p.ticket_bytes);
    if (p.splits > 1) EMMY_CUDA(cudaMemsetAsync(tickets, 0, (size_t)a.outer * p.col_tiles * sizeof(unsigned int), s));
    dim3 grid((unsigned)p.col_tiles, (unsigned)p.splits, (unsigned)a.outer);
    colwise_kernel<OP, VEC><<<grid, kColThreads, 0, s>>>(a, partials, tickets, stats);
    int rc = launch_status("colwise_kernel");
    if (rc != EMMYB200_OK) return rc;
    if constexpr (is_map(OP)) {
        const int64_t work = a.outer * a.rows * (a.cols / VEC);
        const int64_t blocks = (work + 255) / 256, cap = (int64_t)sm_count() * 32;
        colwise_map_kernel<OP, VEC><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, s>>>(a, stats);
        rc = launch_status("colwise_map_kernel");
    }
    return rc;
}

template <int VEC>
int dispatch_col(int op, const ColArgs& a, const ColPlan& p, void* ws, cudaStream_t s) {
    switch (op) {
#define EMMY_COL_CASE(name) case EMMYB200_ROW_##name: return launch_col<EMMYB200_ROW_##name, VEC>(a, p, ws, s);
        EMMY_COL_CASE(SUM) EMMY_COL_CASE(MEAN) EMMY_COL_CASE(AMAX) EMMY_COL_CASE(AMIN) EMMY_COL_CASE(PROD) EMMY_COL_CASE(VAR)
        EMMY_COL_CASE(STD) EMMY_COL_CASE(NORM2) EMMY_COL_CASE(LOGSUMEXP) EMMY_COL_CASE(ARGMAX) EMMY_COL_CASE(SOFTMAX)
        EMMY_COL_CASE(LOG_SOFTMAX) EMMY_COL_CASE(NORMALIZE)
#undef EMMY_COL_CASE
    }
    return fail(EMMYB200_ERR_ARG, "colwise: unknown op %d", op);
}

bool col_vec(const float* x, const void* y, int op, int64_t cols) {
    return cols % 4 == 0 && aligned(x, 16) && (!is_map(op) || aligned(y, 16));
}

}  // namespace
}  // namespace emmy

extern "C" int64_t emmyb200_colwise_workspace_bytes(int op, int64_t outer, int64_t rows, int64_t cols) {
    using namespace emmy;
    if (!col_op(op) || outer < 0 || rows < 1 || cols < 1 || rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31) || outer > 65535) return -1;
    if (outer == 0) return 0;
    // the vector width only changes the number of column tiles, i.e. the ticket count: size for the narrow one
    const ColPlan p4 = plan_cols(op, outer, rows, cols, 4), p1 = plan_cols(op, outer, rows, cols, 1);
    const size_t a = p4.total(), b = p1.total();
    return (int64_t)(a > b ? a : b);
}

extern "C" int emmyb200_colwise_f32(int op, const float* x, void* y, int64_t outer, int64_t rows, int64_t cols, float eps, void* workspace,
                                    int64_t workspace_bytes, void* cuda_stream) {
    using namespace emmy;
    if (!col_op(op)) return fail(EMMYB200_ERR_ARG, "colwise: op %d is not a reduction over the middle axis", op);
    if (outer < 0 || rows < 0 || cols < 0) return fail(EMMYB200_ERR_ARG, "colwise: negative extent");
    if (outer == 0 || cols == 0) return EMMYB200_OK;
    if (rows < 1) return fail(EMMYB200_ERR_SHAPE, "colwise: the reduced axis needs at least one element");
    if (rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31) || outer > 65535)
        return fail(EMMYB200_ERR_SHAPE, "colwise: rows and cols are limited to 2^31 - 1, outer to 65535");
    if (x == nullptr || y == nullptr) return fail(EMMYB200_ERR_ARG, "colwise: null buffer");
    if (!aligned(x, 4) || !aligned(y, op == EMMYB200_ROW_ARGMAX ? 8 : 4)) return fail(EMMYB200_ERR_ALIGN, "colwise: buffers must be aligned to their element size");
    const bool vec = col_vec(x, y, op, cols);
    const ColPlan p = plan_cols(op, outer, rows, cols, vec ? 4 : 1);
    if (p.splits > 65535) return fail(EMMYB200_ERR_SHAPE, "colwise: too many row slices");
    if (p.total() > 0) {
        if (workspace == nullptr || workspace_bytes < (int64_t)p.total())
            return fail(EMMYB200_ERR_ARG, "colwise: this shape needs %lld bytes of workspace", (long long)p.total());
        if (!aligned(workspace, 256)) return fail(EMMYB200_ERR_ALIGN, "colwise: the workspace must be 256-byte aligned");
    }
    ColArgs a{x, y, outer, rows, cols, eps, 1, rows};
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    return vec ? dispatch_col<4>(op, a, p, workspace, s) : dispatch_col<1>(op, a, p, workspace, s);
}

extern "C" int emmyb200_cumsum_f32(const float* x, float* y, int64_t rows, int64_t cols, void* cuda_stream) {
    using namespace emmy;
    if (rows < 0 || cols < 0) return fail(EMMYB200_ERR_ARG, "cumsum: negative extent");
    if (rows == 0 || cols == 0) return EMMYB200_OK;
    if (rows >= ((int64_t)1 << 31)) return fail(EMMYB200_ERR_SHAPE, "cumsum: rows are limited to 2^31 - 1");
    if (x == nullptr || y == nullptr) return fail(EMMYB200_ERR_ARG, "cumsum: null buffer");
    if (!aligned(x, 4) || !aligned(y, 4)) return fail(EMMYB200_ERR_ALIGN, "cumsum: buffers must be 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    const bool vec = cols % 4 == 0 && aligned(x, 16) && aligned(y, 16);
    const bool wide = cols > 2048;                              // a CTA per row instead of a warp
    const int64_t units = wide ? rows : (rows + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    const unsigned grid = (unsigned)(units < cap ? units : cap);
    if (wide) {
        if (vec) cumsum_kernel<256, 4><<<grid, 256, 0, s>>>(x, y, rows, cols);
        else cumsum_kernel<256, 1><<<grid, 256, 0, s>>>(x, y, rows, cols);
    } else {
        if (vec) cumsum_kernel<32, 4><<<grid, 256, 0, s>>>(x, y, rows, cols);
        else cumsum_kernel<32, 1><<<grid, 256, 0, s>>>(x, y, rows, cols);
    }
    return launch_status("cumsum_kernel");
}
