// Attention forward O = softmax(Q K^T * scale) V, per (batch, head) unit, non-causal, fp32 softmax.
//
// The reference has no attention lowering: the tracer fuses the expression into generic statements --
// dot-product `Loop`s whose `Accum` becomes an FMA (emmyptx/kernel.py:786-797), row max / row sum through
// `WarpShuffle` butterflies or `TreeHalve` shared-memory trees (:856-900), `exp` through the libm-style
// expansion (emmyptx/ops.py:49-77), S = Q K^T held per tile in registers or shared memory; its largest
// tested sequence is 512. This kernel is the sm_100a form of that computation:
//
//   * one CTA per 128-query tile of one unit, two CTAs resident per SM (each owns half of tensor
//     memory), so one CTA's softmax overlaps the other's MMAs;
//   * warp 0 (one thread): TMA loads of the Q tile once and of 128-key K and V tiles, each single
//     buffered and re-armed as soon as the MMA that read it has completed;
//   * warp 1 (one thread): S = Q K^T as tcgen05.mma 128x128x16 from shared memory into tensor memory;
//     O += P V with P read from tensor memory and V as an MN-major shared-memory operand;
//   * warps 2-5: one query row per thread. Row max and exponentials on the fp32 S read with
//     tcgen05.ld, P written back over S as packed 16-bit pairs (tcgen05.st), running row sums in
//     registers. The running max is only raised when it grows by more than 8 (in log2 units), so the
//     O accumulator is rescaled in tensor memory rarely; the final 1/rowsum is applied on the way out.
//
// All waits are bounded; keys beyond seq_k are masked to -inf, rows beyond seq_q are not stored.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace emmy {

int check_sm100();

constexpr int kAttThreads = 192;
constexpr int kTileQ = 128, kTileK = 128;

template <int D>
struct AttSmem {
    static constexpr int kQBytes = kTileQ * D * 2;
    static constexpr int kKBytes = kTileK * D * 2;
    static constexpr int kVBytes = kTileK * D * 2;
    static constexpr int kBarOffset = kQBytes + kKBytes + kVBytes;
    // at least 80 KiB, so that no more than two CTAs (2 x 256 tensor-memory columns) share an SM
    static constexpr int kTotal = (kBarOffset + 128 + 1024) > 81920 ? (kBarOffset + 128 + 1024) : 81920;
};

struct AttParams {
    void* O;
    int seq_q, seq_k;
    int q_tiles;
    float scale_log2;       // scale * log2(e)
    uint32_t* status;
};

__device__ uint32_t g_att_status;

template <bool BF16>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttThreads, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, AttParams p) {
    using S = AttSmem<D>;
    constexpr int kChunks = D / 64;                 // 64-element (128-byte) pieces of a head row
    constexpr uint32_t kTmemCols = 256;             // S / P: columns 0-127, O: 128 .. 128 + D
    constexpr uint32_t kColO = 128;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t q_smem = smem_base, k_smem = smem_base + S::kQBytes, v_smem = k_smem + S::kKBytes;
    const uint32_t bar_base = smem_base + S::kBarOffset;
    const uint32_t q_full = bar_base, k_full = bar_base + 8, v_full = bar_base + 16, k_empty = bar_base + 24,
                   v_empty = bar_base + 32, s_full = bar_base + 40, p_full = bar_base + 48, o_full = bar_base + 56;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + S::kBarOffset + 64);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x / p.q_tiles, qt = blockIdx.x % p.q_tiles;
    const int kv_tiles = (p.seq_k + kTileK - 1) / kTileK;
    const WaitCtx wctx{abort_flag, p.status};

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1); ptx::mbar_init(k_full, 1); ptx::mbar_init(v_full, 1);
        ptx::mbar_init(k_empty, 1); ptx::mbar_init(v_empty, 1);
        ptx::mbar_init(s_full, 1); ptx::mbar_init(p_full, 4); ptx::mbar_init(o_full, 1);
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&map_q); ptx::prefetch_tensormap(&map_k); ptx::prefetch_tensormap(&map_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer ------------------------------------------------------------------------------
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(q_full, S::kQBytes);
#pragma unroll
            for (int c = 0; c < kChunks; ++c)
                ptx::tma_load_3d(q_smem + c * (kTileQ * 128), &map_q, q_full, c * 64, qt * kTileQ, unit);
            for (int j = 0; j < kv_tiles; ++j) {
                const uint32_t ph = j & 1;
                if (!bounded_wait(wctx, k_empty, ph ^ 1, 0x02010000u | (j & 0xffff))) break;
                ptx::mbar_arrive_expect_tx(k_full, S::kKBytes);
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
                    ptx::tma_load_3d(k_smem + c * (kTileK * 128), &map_k, k_full, c * 64, j * kTileK, unit);
                if (!bounded_wait(wctx, v_empty, ph ^ 1, 0x02020000u | (j & 0xffff))) break;
                ptx::mbar_arrive_expect_tx(v_full, S::kVBytes);
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
                    ptx::tma_load_3d(v_smem + c * (kTileK * 128), &map_v, v_full, c * 64, j * kTileK, unit);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = ptx::mma_idesc_f16(BF16, false, false, kTileQ, kTileK);
            constexpr uint32_t idesc_o = ptx::mma_idesc_f16(BF16, false, true, kTileQ, D);
            const uint32_t s_tmem = tmem_base, o_tmem = tmem_base + kColO;
            bool ok = bounded_wait(wctx, q_full, 0, 0x02030000u);
            for (int j = 0; j < kv_tiles && ok; ++j) {
                const uint32_t ph = j & 1;
                if (!(ok = bounded_wait(wctx, k_full, ph, 0x02040000u | (j & 0xffff)))) break;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {           // S = Q K^T, contraction over the head dim
                    const uint32_t off = (kk / 4) * (kTileQ * 128) + (kk % 4) * 32;
                    ptx::mma_ss(s_tmem, ptx::smem_desc_sw128(q_smem + off, 16, 1024),
                                ptx::smem_desc_sw128(k_smem + off, 16, 1024), idesc_s, kk != 0);
                }
                ptx::mma_commit(k_empty);
                ptx::mma_commit(s_full);
                if (!(ok = bounded_wait(wctx, p_full, ph, 0x02050000u | (j & 0xffff)))) break;
                if (!(ok = bounded_wait(wctx, v_full, ph, 0x02060000u | (j & 0xffff)))) break;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kTileK / 16; ++kk) {      // O += P V, contraction over the keys
                    ptx::mma_ts(o_tmem, s_tmem + kk * 8,
                                ptx::smem_desc_sw128(v_smem + kk * (16 * 128), kTileK * 128, 1024), idesc_o,
                                (j | kk) != 0);
                }
                ptx::mma_commit(v_empty);
            }
            if (ok) ptx::mma_commit(o_full);
        }
        __syncwarp();
    } else {
        // ---- softmax: thread = one query row ---------------------------------------------------------------
        const int quarter = warp & 3;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_row = tmem_base + lane_base, o_row = tmem_base + lane_base + kColO;
        const float c = p.scale_log2;
        float m_run = -CUDART_INF_F;      // the max the exponentials are taken against (log2 units)
        float l_run = 0.0f;               // running row sum
        bool ok = true;
        for (int j = 0; j < kv_tiles && ok; ++j) {
            ok = __all_sync(0xffffffffu, bounded_wait(wctx, s_full, j & 1, 0x02070000u | (j & 0xffff)));      // warp-uniform
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const int valid = p.seq_k - j * kTileK;             // keys of this tile inside the sequence
            float m_tile = -CUDART_INF_F;
#pragma unroll 1
            for (int ch = 0; ch < kTileK / 32; ++ch) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(s_row + ch * 32, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(r[i]) * c;
                    if (ch * 32 + i >= valid) s = -CUDART_INF_F;
                    m_tile = fmaxf(m_tile, s);
                }
            }
            // Raise the running max only when it would grow by more than 8: exponentials then stay
            // below 2^8, and the accumulator needs rescaling rarely.
            const bool raise = m_tile > m_run + 8.0f;
            const float m_new = raise ? m_tile : m_run;
            if (__any_sync(0xffffffffu, raise) && j > 0) {
                const float f = ptx::ex2_approx(m_run - m_new);     // 1 for rows that keep their max
#pragma unroll 1
                for (int ch = 0; ch < D / 32; ++ch) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(o_row + ch * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(__uint_as_float(r[16 * h + i]) * f);
                        ptx::tmem_st_32x32b_x16(o_row + ch * 32 + h * 16, w);
                    }
                }
                l_run *= f;
            }
            m_run = m_new;
            float l_tile = 0.0f;
#pragma unroll 1
            for (int ch = 0; ch < kTileK / 32; ++ch) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(s_row + ch * 32, r);
                ptx::tmem_ld_wait();
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float e0 = ptx::ex2_approx(fmaf(__uint_as_float(r[2 * i]), c, -m_run));
                    float e1 = ptx::ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), c, -m_run));
                    if (ch * 32 + 2 * i >= valid) e0 = 0.0f;
                    if (ch * 32 + 2 * i + 1 >= valid) e1 = 0.0f;
                    l_tile += e0 + e1;
                    w[i] = pack_pair<BF16>(e0, e1);
                }
                ptx::tmem_st_32x32b_x16(s_row + ch * 16, w);        // P over the consumed part of S
            }
            l_run += l_tile;
            ptx::tmem_st_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
        }
        if (ok && __all_sync(0xffffffffu, bounded_wait(wctx, o_full, 0, 0x02080000u))) {
            ptx::tc_fence_after_sync();
            const float inv = 1.0f / l_run;
            const int row = qt * kTileQ + quarter * 32 + lane;
            uint16_t* out = reinterpret_cast<uint16_t*>(p.O) + ((int64_t)unit * p.seq_q + row) * D;
#pragma unroll 1
            for (int ch = 0; ch < D / 32; ++ch) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(o_row + ch * 32, r);
                ptx::tmem_ld_wait();
                if (row < p.seq_q) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        o.x = pack_pair<BF16>(__uint_as_float(r[8 * q + 0]) * inv, __uint_as_float(r[8 * q + 1]) * inv);
                        o.y = pack_pair<BF16>(__uint_as_float(r[8 * q + 2]) * inv, __uint_as_float(r[8 * q + 3]) * inv);
                        o.z = pack_pair<BF16>(__uint_as_float(r[8 * q + 4]) * inv, __uint_as_float(r[8 * q + 5]) * inv);
                        o.w = pack_pair<BF16>(__uint_as_float(r[8 * q + 6]) * inv, __uint_as_float(r[8 * q + 7]) * inv);
                        *reinterpret_cast<uint4*>(out + ch * 32 + q * 8) = o;
                    }
                }
            }
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

int attention_read_status(uint32_t* out) {
    uint32_t zero = 0;
    EMMY_CUDA(cudaDeviceSynchronize());
    EMMY_CUDA(cudaMemcpyFromSymbol(out, g_att_status, sizeof(uint32_t)));
    if (*out) EMMY_CUDA(cudaMemcpyToSymbol(g_att_status, &zero, sizeof(uint32_t)));
    return EMMYB200_OK;
}

template <int D, bool BF16>
static int launch_attention(const void* Q, const void* K, const void* V, void* O, int64_t units, int64_t seq_q,
                            int64_t seq_k, float scale, cudaStream_t stream) {
    using S = AttSmem<D>;
    CUtensorMap mq, mk, mv;
    int rc = make_tensor_map_3d(&mq, Q, (uint64_t)units, (uint64_t)seq_q, D, kTileQ, 64);
    if (rc == EMMYB200_OK) rc = make_tensor_map_3d(&mk, K, (uint64_t)units, (uint64_t)seq_k, D, kTileK, 64);
    if (rc == EMMYB200_OK) rc = make_tensor_map_3d(&mv, V, (uint64_t)units, (uint64_t)seq_k, D, kTileK, 64);
    if (rc != EMMYB200_OK) return rc;
    auto kernel = attention_fwd_kernel<D, BF16>;
    EMMY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    AttParams p;
    p.O = O; p.seq_q = (int)seq_q; p.seq_k = (int)seq_k;
    p.q_tiles = (int)((seq_q + kTileQ - 1) / kTileQ);
    p.scale_log2 = scale * 1.4426950408889634f;
    EMMY_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_att_status));
    const int64_t ctas = units * p.q_tiles;
    if (ctas >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: %lld query tiles exceed the grid limit", (long long)ctas);
    kernel<<<(unsigned)ctas, kAttThreads, S::kTotal, stream>>>(mq, mk, mv, p);
    return launch_status("attention_fwd_kernel");
}

}  // namespace emmy

extern "C" int emmyb200_attention_fwd(int dtype, const void* Q, const void* K, const void* V, void* O, int64_t units,
                                      int64_t seq_q, int64_t seq_k, int64_t d, float scale, void* cuda_stream) {
    using namespace emmy;
    if (dtype != EMMYB200_F16 && dtype != EMMYB200_BF16) return fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: dtype %d (f16 and bf16 only)", dtype);
    if (units < 0 || seq_q < 0 || seq_k < 0) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: negative extent");
    if (units == 0 || seq_q == 0) return EMMYB200_OK;
    if (seq_k == 0) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: seq_k = 0 (softmax over no keys)");
    if (d != 64 && d != 128) return fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: head dim %lld (64 and 128 only)", (long long)d);
    if (seq_q >= (1ll << 31) || seq_k >= (1ll << 31) || units >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: extents must be below 2^31");
    if (Q == nullptr || K == nullptr || V == nullptr || O == nullptr) return fail(EMMYB200_ERR_ARG, "attention_fwd: null buffer");
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16)) return fail(EMMYB200_ERR_ALIGN, "attention_fwd: buffers must be 16-byte aligned");
    if (!(scale == scale) || scale == 0.0f) return fail(EMMYB200_ERR_ARG, "attention_fwd: scale must be a non-zero number");
    int rc = check_sm100();
    if (rc != EMMYB200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    const bool bf16 = dtype == EMMYB200_BF16;
    if (d == 128) return bf16 ? launch_attention<128, true>(Q, K, V, O, units, seq_q, seq_k, scale, s)
                              : launch_attention<128, false>(Q, K, V, O, units, seq_q, seq_k, scale, s);
    return bf16 ? launch_attention<64, true>(Q, K, V, O, units, seq_q, seq_k, scale, s)
                : launch_attention<64, false>(Q, K, V, O, units, seq_q, seq_k, scale, s);
}
