// Attention forward in fp32 arithmetic on the CUDA cores: O = softmax(Q K^T * scale) V for fp32 buffers, and for
// head sizes the tensor-core kernels do not take (any multiple of 32 up to 128).
//
// These are the shapes of the reference's own attention cases -- fp32 q, k, v with d = 32 or 64 and 64 to 128
// positions (tools/torch_cases/fused.py:21-22, 31-36; models.py:17-19) -- which it lowers to per-thread dot-product
// loops, `WarpShuffle` row reductions and its `_exp` (emmyptx/kernel.py:786-822, 856-900; emmyptx/ops.py:49-77),
// all in fp32. A 16-bit tensor-core pass would not be fp32 arithmetic, so this kernel keeps every product and sum in
// fp32: a CTA of 8 warps takes 32 query rows (4 per warp) of one unit and walks the keys 32 at a time. K and V tiles
// are staged in shared memory with coalesced loads (K rows padded by one word, so that lane j reads key j without
// bank conflicts); lane j of a warp computes the score of key j for the warp's four rows, the row maximum and sum
// go through shuffles (online softmax, exponentials as exp2 of log2(e)-scaled scores), and for P V every lane owns
// d / 32 output columns and receives p_j by shuffle. Causal: keys 0..i for query i; tiles past the CTA's last row
// are skipped.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"

namespace emmy {

constexpr int kAfWarps = 8;
constexpr int kAfRowsPerWarp = 4;
constexpr int kAfRows = kAfWarps * kAfRowsPerWarp;      // query rows per CTA
constexpr int kAfKeys = 32;                             // keys per tile: one per lane

template <typename T> __device__ __forceinline__ float af_load(const T* p, int64_t i);
template <> __device__ __forceinline__ float af_load<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float af_load<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float af_load<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void af_store(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void af_store(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void af_store(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

template <int D, typename T>
__global__ void __launch_bounds__(kAfWarps * 32) attention_fwd_f32_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                                                                           T* __restrict__ O, int seq_q, int seq_k, float scale_log2e, int causal) {
    constexpr int DPL = D / 32;                         // output columns per lane
    extern __shared__ float af_smem[];                  // 48.1 KiB at D = 128: dynamic, above the static limit
    float (*q_s)[D] = reinterpret_cast<float (*)[D]>(af_smem);
    float (*k_s)[D + 1] = reinterpret_cast<float (*)[D + 1]>(af_smem + kAfRows * D);
    float (*v_s)[D] = reinterpret_cast<float (*)[D]>(af_smem + kAfRows * D + kAfKeys * (D + 1));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t unit = blockIdx.y;
    const int row0 = blockIdx.x * kAfRows;
    const T* q_u = Q + unit * (int64_t)seq_q * D;
    const T* k_u = K + unit * (int64_t)seq_k * D;
    const T* v_u = V + unit * (int64_t)seq_k * D;
    T* o_u = O + unit * (int64_t)seq_q * D;

    for (int e = tid; e < kAfRows * D; e += kAfWarps * 32) {
        const int r = e / D, c = e % D;
        q_s[r][c] = row0 + r < seq_q ? af_load(q_u, (int64_t)(row0 + r) * D + c) : 0.0f;
    }
    float m[kAfRowsPerWarp], l[kAfRowsPerWarp], acc[kAfRowsPerWarp][DPL];
#pragma unroll
    for (int r = 0; r < kAfRowsPerWarp; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int dd = 0; dd < DPL; ++dd) acc[r][dd] = 0.0f;
    }
    const int last_row = min(row0 + kAfRows, seq_q) - 1;
    const int key_end = causal ? min(seq_k, last_row + 1) : seq_k;          // keys beyond it are masked for every row here
    for (int j0 = 0; j0 < key_end; j0 += kAfKeys) {
        __syncthreads();                                                    // q_s written / previous tile consumed
        for (int e = tid; e < kAfKeys * D; e += kAfWarps * 32) {
            const int j = e / D, c = e % D;
            const bool live = j0 + j < seq_k;
            k_s[j][c] = live ? af_load(k_u, (int64_t)(j0 + j) * D + c) : 0.0f;
            v_s[j][c] = live ? af_load(v_u, (int64_t)(j0 + j) * D + c) : 0.0f;
        }
        __syncthreads();
        float s[kAfRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kAfRowsPerWarp; ++r) s[r] = 0.0f;
#pragma unroll 8
        for (int c = 0; c < D; ++c) {
            const float kv = k_s[lane][c];
#pragma unroll
            for (int r = 0; r < kAfRowsPerWarp; ++r) s[r] = fmaf(q_s[warp * kAfRowsPerWarp + r][c], kv, s[r]);
        }
        const int key = j0 + lane;
#pragma unroll
        for (int r = 0; r < kAfRowsPerWarp; ++r) {
            const int row = row0 + warp * kAfRowsPerWarp + r;
            float t = s[r] * scale_log2e;
            if (key >= seq_k || (causal && key > row)) t = -INFINITY;
            float tile_max = t;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, off));
            const float m_new = fmaxf(m[r], tile_max);
            const float m_ref = m_new == -INFINITY ? 0.0f : m_new;          // every key so far masked: nothing to rescale
            const float p = exp2f(t - m_ref);                               // a masked key gives exp2(-inf) = 0
            const float corr = exp2f(m[r] - m_ref);
            float tile_sum = p;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, off);
            l[r] = fmaf(l[r], corr, tile_sum);
            m[r] = m_new;
#pragma unroll
            for (int dd = 0; dd < DPL; ++dd) acc[r][dd] *= corr;
#pragma unroll 8
            for (int j = 0; j < kAfKeys; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int dd = 0; dd < DPL; ++dd) acc[r][dd] = fmaf(pj, v_s[j][lane + 32 * dd], acc[r][dd]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kAfRowsPerWarp; ++r) {
        const int row = row0 + warp * kAfRowsPerWarp + r;
        if (row >= seq_q) continue;
        const float inv = 1.0f / l[r];
#pragma unroll
        for (int dd = 0; dd < DPL; ++dd) af_store(o_u, (int64_t)row * D + lane + 32 * dd, acc[r][dd] * inv);
    }
}

template <typename T>
static int launch_attention_f32(const void* Q, const void* K, const void* V, void* O, int64_t units, int64_t seq_q, int64_t seq_k, int64_t d,
                                float scale, bool causal, cudaStream_t s) {
    const dim3 grid((unsigned)((seq_q + kAfRows - 1) / kAfRows), (unsigned)units);
    const float sl = scale * 1.4426950408889634f;
    const T* q = static_cast<const T*>(Q);
    const T* k = static_cast<const T*>(K);
    const T* v = static_cast<const T*>(V);
    T* o = static_cast<T*>(O);
    auto run = [&](auto kernel, int D) -> cudaError_t {
        const size_t smem = sizeof(float) * (size_t)(kAfRows * D + kAfKeys * (D + 1) + kAfKeys * D);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        kernel<<<grid, kAfWarps * 32, smem, s>>>(q, k, v, o, (int)seq_q, (int)seq_k, sl, causal ? 1 : 0);
        return cudaSuccess;
    };
    cudaError_t e;
    switch (d) {
        case 32: e = run(attention_fwd_f32_kernel<32, T>, 32); break;
        case 64: e = run(attention_fwd_f32_kernel<64, T>, 64); break;
        case 96: e = run(attention_fwd_f32_kernel<96, T>, 96); break;
        default: e = run(attention_fwd_f32_kernel<128, T>, 128); break;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute (attention_fwd_f32_kernel)");
    return launch_status("attention_fwd_f32_kernel");
}

// Called by the attention entry point for fp32 buffers and for 16-bit buffers whose head size the tensor-core
// kernels do not take. Arguments are already checked for null pointers, sign and size.
int attention_cuda_cores(int dtype, bool causal, const void* Q, const void* K, const void* V, void* O, int64_t units, int64_t seq_q,
                         int64_t seq_k, int64_t d, float scale, cudaStream_t s) {
    if (d % 32 != 0 || d < 32 || d > 128) return fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: head dim %lld (a multiple of 32 up to 128)", (long long)d);
    if (units > 65535) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: %lld units for the CUDA-core kernel (65535 at most)", (long long)units);
    if (dtype == EMMYB200_F32) return launch_attention_f32<float>(Q, K, V, O, units, seq_q, seq_k, d, scale, causal, s);
    if (dtype == EMMYB200_F16) return launch_attention_f32<__half>(Q, K, V, O, units, seq_q, seq_k, d, scale, causal, s);
    return launch_attention_f32<__nv_bfloat16>(Q, K, V, O, units, seq_q, seq_k, d, scale, causal, s);
}

}  // namespace emmy
