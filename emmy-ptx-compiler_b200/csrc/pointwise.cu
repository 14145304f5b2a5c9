// Streaming fp32 elementwise kernels: y[i] = op(x[i]).
//
// The reference lowers a one-axis `Tile` to one thread per element with 4-byte accesses and no
// loop (emmyptx/kernel.py:551-585 for the thread map, :632-677 / :714-733 for the scalar
// ld/st, emmyptx/ops.py:212-290 for the op bodies). Here each thread moves 128-bit vectors,
// several per trip of a grid-stride loop, so every warp access is four full 128-byte lines and
// a few independent loads are in flight per thread; the grid is capped at a multiple of the SM
// count. The op bodies are the <= 2 ulp functions of emmy_math.cuh.
#include "common.cuh"
#include "emmy_math.cuh"
#include "emmy_math_x2.cuh"

namespace emmy {

template <int OP>
__device__ __forceinline__ float apply_op(float x) {
    if constexpr (OP == EMMYB200_OP_EXP_SIN_TANH) return emmy_exp_sin_tanh(x);
    else if constexpr (OP == EMMYB200_OP_EXP) return emmy_expf(x);
    else if constexpr (OP == EMMYB200_OP_SIN) return emmy_sinf(x);
    else if constexpr (OP == EMMYB200_OP_COS) return emmy_cosf(x);
    else if constexpr (OP == EMMYB200_OP_TANH) return emmy_tanhf(x);
    else if constexpr (OP == EMMYB200_OP_SIGMOID) return emmy_sigmoidf(x);
    else if constexpr (OP == EMMYB200_OP_SILU) return emmy_siluf(x);
    else if constexpr (OP == EMMYB200_OP_RELU) return emmy_reluf(x);
    else return emmy_gelu_tanhf(x);
}

#ifndef EMMY_PW_THREADS
#define EMMY_PW_THREADS 256
#endif
#ifndef EMMY_PW_VECS
#define EMMY_PW_VECS 4
#endif
#ifndef EMMY_PW_MIN_CTAS
#define EMMY_PW_MIN_CTAS 1
#endif
constexpr int kThreads = EMMY_PW_THREADS;
constexpr int kVecPerTrip = EMMY_PW_VECS;     // float4 vectors per thread and trip (and as many again requested ahead)

// x and y are not __restrict__: the op may run in place.
template <int OP>
__global__ void __launch_bounds__(kThreads, EMMY_PW_MIN_CTAS) pointwise_vec4_kernel(const float4* x, float4* y, int64_t n4,
                                                                   const float* x_tail, float* y_tail, int tail) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    int64_t base = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    // The vectors of the next trip are requested before this trip's arithmetic starts (a few hundred instructions per
    // thread), so a warp's own work covers its memory latency instead of the other warps' alone.
    float4 v[kVecPerTrip];
#pragma unroll
    for (int k = 0; k < kVecPerTrip; ++k)
        if (base + k * stride < n4) v[k] = __ldcs(x + base + k * stride);
    for (; base < n4; base += stride * kVecPerTrip) {
        const int64_t next = base + stride * kVecPerTrip;
        float4 ahead[kVecPerTrip];
#pragma unroll
        for (int k = 0; k < kVecPerTrip; ++k)
            if (next + k * stride < n4) ahead[k] = __ldcs(x + next + k * stride);
#pragma unroll
        for (int k = 0; k < kVecPerTrip; ++k) {
            int64_t idx = base + k * stride;
            if (idx < n4) {
                float4 r;
                if constexpr (PackedOp<OP>::kHas) {
                    // One range test for the four elements picks the packed straight-line path
                    // (a NaN makes the comparison false).
                    const float big = fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w)));
                    const float sum = (v[k].x + v[k].y) + (v[k].z + v[k].w);      // NaN if any element is
                    if (big <= PackedOp<OP>::kBound && sum == sum) {
                        const float2 lo = PackedOp<OP>::apply(make_float2(v[k].x, v[k].y));
                        const float2 hi = PackedOp<OP>::apply(make_float2(v[k].z, v[k].w));
                        r = make_float4(lo.x, lo.y, hi.x, hi.y);
                        __stcs(y + idx, r);
                        continue;
                    }
                }
                r.x = apply_op<OP>(v[k].x);
                r.y = apply_op<OP>(v[k].y);
                r.z = apply_op<OP>(v[k].z);
                r.w = apply_op<OP>(v[k].w);
                __stcs(y + idx, r);
            }
        }
#pragma unroll
        for (int k = 0; k < kVecPerTrip; ++k) v[k] = ahead[k];
    }
    if (blockIdx.x == 0 && (int)threadIdx.x < tail) y_tail[threadIdx.x] = apply_op<OP>(x_tail[threadIdx.x]);
}

// Buffers that are not 16-byte aligned (a view into a larger allocation): 4-byte accesses,
// still one full line per warp.
template <int OP>
__global__ void __launch_bounds__(kThreads) pointwise_scalar_kernel(const float* x, float* y, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) y[i] = apply_op<OP>(x[i]);
}

// CTAs of a kernel that fit one SM at once (registers decide: 40 per thread leave room for 6 CTAs of 256 threads,
// not 8). A grid-stride grid larger than what is resident runs a second, thin wave with little latency hiding.
template <typename K>
static int resident_ctas(K kernel) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
    return per_sm;
}

template <int OP>
static int launch_pointwise(const float* x, float* y, int64_t n, cudaStream_t stream) {
    if (aligned(x, 16) && aligned(y, 16)) {
        static const int per_sm = resident_ctas(pointwise_vec4_kernel<OP>);
        const int64_t max_blocks = (int64_t)sm_count() * per_sm;
        int64_t n4 = n / 4;
        int tail = (int)(n - n4 * 4);
        int64_t want = (n4 + (int64_t)kThreads * kVecPerTrip - 1) / ((int64_t)kThreads * kVecPerTrip);
        int64_t blocks = want < 1 ? 1 : (want > max_blocks ? max_blocks : want);
        pointwise_vec4_kernel<OP><<<(unsigned)blocks, kThreads, 0, stream>>>(
            reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), n4, x + n4 * 4, y + n4 * 4, tail);
        return launch_status("pointwise_vec4_kernel");
    }
    static const int per_sm_scalar = resident_ctas(pointwise_scalar_kernel<OP>);
    const int64_t max_blocks = (int64_t)sm_count() * per_sm_scalar;
    int64_t want = (n + kThreads - 1) / kThreads;
    int64_t blocks = want > max_blocks ? max_blocks : want;
    pointwise_scalar_kernel<OP><<<(unsigned)blocks, kThreads, 0, stream>>>(x, y, n);
    return launch_status("pointwise_scalar_kernel");
}

}  // namespace emmy

extern "C" int emmyb200_pointwise_f32(int op, const float* x, float* y, int64_t n, void* cuda_stream) {
    using namespace emmy;
    if (n < 0) return fail(EMMYB200_ERR_SHAPE, "pointwise: n = %lld is negative", (long long)n);
    if (n == 0) return EMMYB200_OK;
    if (x == nullptr || y == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise: null buffer");
    if (!aligned(x, 4) || !aligned(y, 4)) return fail(EMMYB200_ERR_ALIGN, "pointwise: buffers must be 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    switch (op) {
        case EMMYB200_OP_EXP_SIN_TANH: return launch_pointwise<EMMYB200_OP_EXP_SIN_TANH>(x, y, n, s);
        case EMMYB200_OP_EXP: return launch_pointwise<EMMYB200_OP_EXP>(x, y, n, s);
        case EMMYB200_OP_SIN: return launch_pointwise<EMMYB200_OP_SIN>(x, y, n, s);
        case EMMYB200_OP_COS: return launch_pointwise<EMMYB200_OP_COS>(x, y, n, s);
        case EMMYB200_OP_TANH: return launch_pointwise<EMMYB200_OP_TANH>(x, y, n, s);
        case EMMYB200_OP_GELU_TANH: return launch_pointwise<EMMYB200_OP_GELU_TANH>(x, y, n, s);
        case EMMYB200_OP_SIGMOID: return launch_pointwise<EMMYB200_OP_SIGMOID>(x, y, n, s);
        case EMMYB200_OP_SILU: return launch_pointwise<EMMYB200_OP_SILU>(x, y, n, s);
        case EMMYB200_OP_RELU: return launch_pointwise<EMMYB200_OP_RELU>(x, y, n, s);
        default: return fail(EMMYB200_ERR_ARG, "pointwise: unknown op %d", op);
    }
}
