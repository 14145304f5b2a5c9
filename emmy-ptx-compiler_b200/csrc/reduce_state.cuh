// The mergeable states behind the reduction kernels (row-wise and column-wise): what a partial reduction holds for
// each kind of op, how an element is folded in, how two partial states merge (in index order), and how the final
// state becomes what is stored. The reference spells the same combine steps as Assign programs inside its
// `WarpShuffle` / `TreeHalve` statements (emmyptx/kernel.py:856-900).
#pragma once
#include <limits.h>
#include <math_constants.h>

#include "common.cuh"

namespace emmy {
namespace {

enum Kind { K_ADD, K_SQ, K_MAX, K_MIN, K_MUL, K_MOM, K_LSE, K_ARG, K_DOT3 };

constexpr int kind_of(int op) {
    switch (op) {
        case EMMYB200_ROW_SUM: case EMMYB200_ROW_MEAN: case EMMYB200_ROW_DOT: return K_ADD;
        case EMMYB200_ROW_NORM2: case EMMYB200_ROW_RMS_NORM: case EMMYB200_ROW_NORMALIZE: return K_SQ;
        case EMMYB200_ROW_AMAX: return K_MAX;
        case EMMYB200_ROW_AMIN: return K_MIN;
        case EMMYB200_ROW_PROD: return K_MUL;
        case EMMYB200_ROW_VAR: case EMMYB200_ROW_STD: case EMMYB200_ROW_LAYER_NORM: return K_MOM;
        case EMMYB200_ROW_LOGSUMEXP: case EMMYB200_ROW_SOFTMAX: case EMMYB200_ROW_LOG_SOFTMAX: return K_LSE;
        case EMMYB200_ROW_COSINE: return K_DOT3;
        default: return K_ARG;
    }
}
constexpr bool is_map(int op) { return op >= EMMYB200_ROW_SOFTMAX; }

// The state of a partial reduction. Which members mean something depends on the kind:
//   ADD, SQ, MAX, MIN, MUL: a.   MOM: a = n, b = mean, c = M2.   LSE: a = max, b = sum of exp(x - max).
//   ARG: a = value, c = index (bits of an int).
struct St {
    float a, b, c;
};

// e^d for the softmax family, where d = x - max <= 0: one multiply and the hardware 2^t (the reference's `exp_fast`,
// emmyptx/ops.py:49-77). The rounding of d * log2(e) costs |d| * 6e-8 of relative accuracy, which only matters
// for terms too small to count; -inf gives 0, NaN stays NaN.
__device__ __forceinline__ float exp_le0(float d) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(d * 1.4426950408889634f));
    return y;
}

__device__ __forceinline__ float nan_max(float x, float y) { return (x > y || x != x) ? x : y; }
__device__ __forceinline__ float nan_min(float x, float y) { return (x < y || x != x) ? x : y; }

template <int K>
__device__ __forceinline__ St st_identity() {
    if constexpr (K == K_MAX) return {-CUDART_INF_F, 0.0f, 0.0f};
    else if constexpr (K == K_MIN) return {CUDART_INF_F, 0.0f, 0.0f};
    else if constexpr (K == K_MUL) return {1.0f, 0.0f, 0.0f};
    else if constexpr (K == K_LSE) return {-CUDART_INF_F, 0.0f, 0.0f};
    else if constexpr (K == K_ARG) return {-CUDART_INF_F, 0.0f, __int_as_float(INT_MAX)};
    else return {0.0f, 0.0f, 0.0f};
}

// True if (va, ia) precedes (vb, ib) for argmax: larger value, NaN above everything, ties to the lower index.
__device__ __forceinline__ bool arg_before(float va, int ia, float vb, int ib) {
    const bool na = va != va, nb = vb != vb;
    if (na || nb) return na && (!nb || ia < ib);
    return va > vb || (va == vb && ia < ib);
}

// Folding the next element (a higher index than anything folded so far) into a thread's own (value, index).
__device__ __forceinline__ void arg_push(St& s, float x, int idx) {
    const bool first = __float_as_int(s.c) == INT_MAX;
    if (first || x > s.a || (x != x && s.a == s.a)) { s.a = x; s.c = __int_as_float(idx); }
}

// x covers the elements before y's.
template <int K>
__device__ __forceinline__ St st_merge(St x, St y) {
    if constexpr (K == K_ADD || K == K_SQ) return {x.a + y.a, 0.0f, 0.0f};
    else if constexpr (K == K_DOT3) return {x.a + y.a, x.b + y.b, x.c + y.c};      // sum of x w, of x^2, of w^2
    else if constexpr (K == K_MAX) return {nan_max(x.a, y.a), 0.0f, 0.0f};
    else if constexpr (K == K_MIN) return {nan_min(x.a, y.a), 0.0f, 0.0f};
    else if constexpr (K == K_MUL) return {x.a * y.a, 0.0f, 0.0f};
    else if constexpr (K == K_MOM) {
        const float n = x.a + y.a;
        if (n == 0.0f) return x;
        const float d = y.b - x.b, f = __fdividef(y.a, n);      // counts are small integers: 2 ulp is plenty
        return {n, x.b + d * f, x.c + y.c + d * d * x.a * f};
    } else if constexpr (K == K_LSE) {
        const float m = nan_max(x.a, y.a);
        if (m == -CUDART_INF_F) return {m, 0.0f, 0.0f};
        // an empty side has max -inf and contributes exp(-inf) * 0 = 0
        return {m, x.b * exp_le0(x.a - m) + y.b * exp_le0(y.a - m), 0.0f};
    } else {
        return arg_before(y.a, __float_as_int(y.c), x.a, __float_as_int(x.c)) ? y : x;
    }
}

template <int K>
__device__ __forceinline__ St st_shfl_xor(St s, int off) {
    St o = s;
    o.a = __shfl_xor_sync(0xffffffffu, s.a, off);
    if constexpr (K == K_MOM || K == K_LSE || K == K_DOT3) o.b = __shfl_xor_sync(0xffffffffu, s.b, off);
    if constexpr (K == K_MOM || K == K_ARG || K == K_DOT3) o.c = __shfl_xor_sync(0xffffffffu, s.c, off);
    return o;
}

// Butterfly over `width` lanes; the lower lane's state is always the left operand, so every lane ends with the
// same bits.
template <int K>
__device__ __forceinline__ St warp_allreduce(St s, int width, int lane) {
    for (int off = 1; off < width; off <<= 1) {
        const St o = st_shfl_xor<K>(s, off);
        const bool upper = lane & off;
        const St lo = upper ? o : s, hi = upper ? s : o;        // one merge per level, operands in lane order
        s = st_merge<K>(lo, hi);
    }
    return s;
}

template <int OP>
__device__ __forceinline__ float2 row_finish(St s, float cols, float eps) {
    if constexpr (OP == EMMYB200_ROW_MEAN) return {s.a / cols, 0.0f};
    else if constexpr (OP == EMMYB200_ROW_NORM2) return {sqrtf(s.a), 0.0f};
    else if constexpr (OP == EMMYB200_ROW_VAR) return {s.c / (cols - 1.0f), 0.0f};
    else if constexpr (OP == EMMYB200_ROW_STD) return {sqrtf(s.c / (cols - 1.0f)), 0.0f};
    else if constexpr (OP == EMMYB200_ROW_LOGSUMEXP) return {fabsf(s.a) == CUDART_INF_F ? s.a : s.a + logf(s.b), 0.0f};
    else if constexpr (OP == EMMYB200_ROW_SOFTMAX) return {s.a, 1.0f / s.b};
    else if constexpr (OP == EMMYB200_ROW_LOG_SOFTMAX) return {s.a + logf(s.b), 0.0f};
    else if constexpr (OP == EMMYB200_ROW_LAYER_NORM) return {s.b, 1.0f / sqrtf(s.c / cols + eps)};
    else if constexpr (OP == EMMYB200_ROW_RMS_NORM) return {0.0f, 1.0f / sqrtf(s.a / cols + eps)};
    else if constexpr (OP == EMMYB200_ROW_NORMALIZE) return {0.0f, 1.0f / fmaxf(sqrtf(s.a), eps)};
    else if constexpr (OP == EMMYB200_ROW_COSINE) return {s.a / fmaxf(sqrtf(s.b) * sqrtf(s.c), eps), 0.0f};
    else return {s.a, 0.0f};      // SUM, AMAX, AMIN, PROD (ARGMAX stores s.c)
}

template <int OP>
__device__ __forceinline__ float row_map(float x, float2 r, float w, float b) {
    if constexpr (OP == EMMYB200_ROW_SOFTMAX) return exp_le0(x - r.x) * r.y;
    else if constexpr (OP == EMMYB200_ROW_LOG_SOFTMAX) return x - r.x;
    else if constexpr (OP == EMMYB200_ROW_LAYER_NORM) return (x - r.x) * r.y * w + b;
    else if constexpr (OP == EMMYB200_ROW_RMS_NORM) return x * r.y * w;
    else return x * r.y;          // NORMALIZE
}

template <int OP>
__device__ __forceinline__ void store_reduced(void* y, int64_t row, St s, float2 r) {
    if constexpr (OP == EMMYB200_ROW_ARGMAX) static_cast<int64_t*>(y)[row] = (int64_t)__float_as_int(s.c);
    else static_cast<float*>(y)[row] = r.x;
}

}  // namespace
}  // namespace emmy
