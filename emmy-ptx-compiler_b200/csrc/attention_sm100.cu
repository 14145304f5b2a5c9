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
//   * warps 2-9: two threads per query row, 64 keys of each tile apiece. Row max and exponentials on
//     the fp32 S read with tcgen05.ld (one pass, values held in registers), P written back over S as
//     packed 16-bit pairs (tcgen05.st), running row sums in registers. The running max is only raised when it grows by
//     more than 8 (in log2 units), so the O accumulator is rescaled in tensor memory rarely; the final
//     1/rowsum is applied on the way out.
//
// All waits are bounded; keys beyond seq_k (and, with the causal flag, keys after the query) are masked to -inf,
// rows beyond seq_q are not stored.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace emmy {

int check_sm100();

constexpr int kAttThreads = 320;     // TMA warp, MMA warp, eight softmax warps
constexpr int kTileQ = 128, kTileK = 128;

template <int D>
struct AttSmem {
    static constexpr int kQBytes = kTileQ * D * 2;
    static constexpr int kKBytes = kTileK * D * 2;
    static constexpr int kVBytes = kTileK * D * 2;
    static constexpr int kBarOffset = kQBytes + kKBytes + kVBytes;
    // at least 80 KiB, so that no more than two CTAs (2 x 256 tensor-memory columns) share an SM
    static constexpr int kTotal = (kBarOffset + 256 + 2048 + 1024) > 81920 ? (kBarOffset + 256 + 2048 + 1024) : 81920;
};

constexpr int kMaxDst = 8;
constexpr float kTruncBiasLog2 = 0.0028150156f;      // log2(1 + 2^-9): centres the error of truncating an fp32 to bf16

struct AttOutMaps {
    CUtensorMap m[kMaxDst];
};

struct AttParams {
    int n_dst;              // destinations of every output tile (1 = the local O only)
    int causal;             // 1: query i sees keys 0 .. i only
    unsigned long long mc_base;     // != 0: O as a multicast address, written once with multimem.st for every GPU
    int units, seq_q, seq_k;
    int q_tiles;
    float scale_log2;       // scale * log2(e)
    unsigned long long wait_limit_ns;       // after which a pipeline wait gives up
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

// Packed fp32 pairs (one issue slot for two elements), rounding spelled out.
__device__ __forceinline__ uint64_t as_u64(float2 v) { return *reinterpret_cast<uint64_t*>(&v); }
__device__ __forceinline__ float2 as_f2(uint64_t v) { return *reinterpret_cast<float2*>(&v); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(as_u64(a)), "l"(as_u64(b)), "l"(as_u64(c)));
    return as_f2(d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(as_u64(a)), "l"(as_u64(b)));
    return as_f2(d);
}

// The two warps that share a lane quarter publish per-row values in shared memory and then trade a flag:
// each writes `token` to its own flag and polls the partner's, with the same time limit and abort handling
// as every other wait in the kernel. Returns false (warp-uniformly) when the wait was given up.
__device__ __forceinline__ bool pair_exchange(const WaitCtx& ctx, volatile uint32_t* flags, int half, int quarter, int lane,
                                              uint32_t token, uint32_t code) {
    __threadfence_block();
    __syncwarp();
    bool ok = true;
    if (lane == 0) {
        flags[half * 4 + quarter] = token;
        volatile uint32_t* other = flags + (half ^ 1) * 4 + quarter;
        uint64_t t0 = 0;
        for (uint32_t spin = 1; *other != token; ++spin) {
            if ((spin & 255u) == 0) {
                if (*ctx.abort_flag) { ok = false; break; }
                const uint64_t now = ptx::global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > ctx.limit_ns) {
                    atomicCAS(ctx.status_word, 0u, code);
                    *ctx.abort_flag = 1;
                    ok = false;
                    break;
                }
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    __threadfence_block();
    return ok;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttThreads, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttOutMaps out, AttParams p) {
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
                   v_empty = bar_base + 32, s_full = bar_base + 40, p_full = bar_base + 48, o_full = bar_base + 56,
                   o_staged = bar_base + 64;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + S::kBarOffset + 80);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* pair_flags = tmem_slot + 4;                                 // [2 buffers][2 halves][4 quarters]
    float* xchg = reinterpret_cast<float*>(smem_gen + S::kBarOffset + 256);        // [2][2][128] row maxima / sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Causal tiles differ in length (tile qt runs qt + 1 key tiles): the longest of each unit are launched first.
    const int unit = blockIdx.x / p.q_tiles;
    const int qt = p.causal ? p.q_tiles - 1 - (int)(blockIdx.x % p.q_tiles) : (int)(blockIdx.x % p.q_tiles);
    // Causal: keys beyond the tile's last query are never seen, so the tiles past the diagonal are skipped.
    const int kv_all = (p.seq_k + kTileK - 1) / kTileK;
    const int kv_tiles = p.causal ? min(kv_all, (qt * kTileQ + kTileQ + kTileK - 1) / kTileK) : kv_all;
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1); ptx::mbar_init(k_full, 1); ptx::mbar_init(v_full, 1);
        ptx::mbar_init(k_empty, 1); ptx::mbar_init(v_empty, 1);
        ptx::mbar_init(s_full, 1); ptx::mbar_init(p_full, 8); ptx::mbar_init(o_full, 1); ptx::mbar_init(o_staged, 8);
        for (int q = 0; q < 16; ++q) pair_flags[q] = 0;
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
            // descriptors of every k-step, built once
            uint64_t q_desc[D / 16], k_desc[D / 16], v_desc[kTileK / 16];
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk / 4) * (kTileQ * 128) + (kk % 4) * 32;
                q_desc[kk] = ptx::smem_desc_sw128(q_smem + off, 16, 1024);
                k_desc[kk] = ptx::smem_desc_sw128(k_smem + off, 16, 1024);
            }
#pragma unroll
            for (int kk = 0; kk < kTileK / 16; ++kk) v_desc[kk] = ptx::smem_desc_sw128(v_smem + kk * (16 * 128), kTileK * 128, 1024);
            bool ok = bounded_wait(wctx, q_full, 0, 0x02030000u);
            for (int j = 0; j < kv_tiles && ok; ++j) {
                const uint32_t ph = j & 1;
                if (!(ok = bounded_wait(wctx, k_full, ph, 0x02040000u | (j & 0xffff)))) break;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)             // S = Q K^T, contraction over the head dim
                    ptx::mma_ss(s_tmem, q_desc[kk], k_desc[kk], idesc_s, kk != 0);
                ptx::mma_commit(k_empty);
                ptx::mma_commit(s_full);
                if (!(ok = bounded_wait(wctx, p_full, ph, 0x02050000u | (j & 0xffff)))) break;
                if (!(ok = bounded_wait(wctx, v_full, ph, 0x02060000u | (j & 0xffff)))) break;
                ptx::tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < kTileK / 16; ++kk)        // O += P V, contraction over the keys
                    ptx::mma_ts(o_tmem, s_tmem + kk * 8, v_desc[kk], idesc_o, (j | kk) != 0);
                ptx::mma_commit(v_empty);
            }
            if (ok) ptx::mma_commit(o_full);
        }
        __syncwarp();
    } else {
        // ---- softmax: two threads per query row, 64 keys of each tile apiece ----------------------------------
        // Warp w reads tensor-memory lanes 32 (w % 4) .. +32; warps w and w + 4 share those rows and take the
        // lower and upper half of the columns. They agree on the row max through shared memory (an mbarrier
        // per lane quarter, so the wait is bounded); partial row sums are merged once, at the end.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_row = tmem_base + lane_base + half * (kTileK / 2);      // this thread's 64 S columns
        const uint32_t p_row = tmem_base + lane_base + half * (kTileK / 4);      // and where its 64 P values go
        const uint32_t o_row = tmem_base + lane_base + kColO + half * (D / 2);   // its half of the O row
        const float c = p.scale_log2;
        float m_run = -CUDART_INF_F;      // the max the exponentials are taken against (log2 units)
        float l_run = 0.0f;               // running sum over this thread's columns
        bool ok = true;
        for (int j = 0; j < kv_tiles && ok; ++j) {
            ok = __all_sync(0xffffffffu, bounded_wait(wctx, s_full, j & 1, 0x02070000u | (j & 0xffff)));      // warp-uniform
            if (!ok) break;
            ptx::tc_fence_after_sync();
            uint32_t r[kTileK / 2];
#pragma unroll
            for (int ch = 0; ch < kTileK / 64; ++ch) ptx::tmem_ld_32x32b_x32(s_row + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[ch * 32]));
            ptx::tmem_ld_wait();
            int valid = p.seq_k - j * kTileK - half * (kTileK / 2);             // of this thread's columns
            if (p.causal) valid = min(valid, qt * kTileQ + row_in_tile - j * kTileK - half * (kTileK / 2) + 1);
            if (valid < kTileK / 2) {                           // ragged last tile, or the causal diagonal
#pragma unroll
                for (int i = 0; i < kTileK / 2; ++i)
                    if (i >= valid) r[i] = __float_as_uint(c > 0.0f ? -CUDART_INF_F : CUDART_INF_F);
            }
            // max of c * s = c * (max or min of s); eight independent chains for latency
            float ext[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ext[i] = __uint_as_float(r[i]);
            if (c > 0.0f) {
#pragma unroll
                for (int i = 8; i < kTileK / 2; ++i) ext[i & 7] = fmaxf(ext[i & 7], __uint_as_float(r[i]));
                ext[0] = fmaxf(fmaxf(fmaxf(ext[0], ext[1]), fmaxf(ext[2], ext[3])), fmaxf(fmaxf(ext[4], ext[5]), fmaxf(ext[6], ext[7])));
            } else {
#pragma unroll
                for (int i = 8; i < kTileK / 2; ++i) ext[i & 7] = fminf(ext[i & 7], __uint_as_float(r[i]));
                ext[0] = fminf(fminf(fminf(ext[0], ext[1]), fminf(ext[2], ext[3])), fminf(fminf(ext[4], ext[5]), fminf(ext[6], ext[7])));
            }
            // exchange with the thread that owns the other half of the row (both S halves are in registers by
            // now, so P may overwrite S afterwards)
            volatile float* slot = xchg + (j & 1) * 256;
            slot[half * 128 + row_in_tile] = ext[0] * c;
            ok = pair_exchange(wctx, pair_flags + (j & 1) * 8, half, quarter, lane, (uint32_t)j + 1, 0x02090000u | (j & 0xffff));
            if (!ok) break;
            const float m_tile = fmaxf(ext[0] * c, slot[(half ^ 1) * 128 + row_in_tile]);
            // Raise the running max only when it would grow by more than 8: exponentials then stay
            // below 2^8, and the accumulator needs rescaling rarely.
            const bool raise = m_tile > m_run + 8.0f;
            const float m_new = raise ? m_tile : m_run;
            if (__any_sync(0xffffffffu, raise) && j > 0) {
                const float f = ptx::ex2_approx(m_run - m_new);     // 1 for rows that keep their max
#pragma unroll 1
                for (int col = 0; col < D / 2; col += 8) {          // few registers: the S row is still live
                    uint32_t o[8];
                    ptx::tmem_ld_32x32b_x8(o_row + col, o);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                    ptx::tmem_st_32x32b_x8(o_row + col, o);
                }
                l_run *= f;
            }
            m_run = m_new;
            // p = 2^(c s - m): packed fma for the exponent, MUFU ex2 (moving part of the exponentials to a
            // polynomial on the FMA pipe was measured slower at every fraction tried).
            // (bf16: P is the upper half of the fp32 pattern -- one byte-permute per pair instead of a conversion, which
            // would run on the transcendental unit like the exponentials; the truncation's mean loss of half a 16-bit
            // ulp is made up by taking every exponent kTruncBiasLog2 higher and scaling the row sum back at the end)
            const float shift = BF16 ? kTruncBiasLog2 - m_run : -m_run;
            const float2 c2 = make_float2(c, c), nm2 = make_float2(shift, shift);
            float2 sum2[4] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int ch = 0; ch < kTileK / 64; ++ch) {
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 sv = make_float2(__uint_as_float(r[ch * 32 + 2 * i]), __uint_as_float(r[ch * 32 + 2 * i + 1]));
                    const float2 y = fma2(sv, c2, nm2);
                    const float2 e = make_float2(ptx::ex2_approx(y.x), ptx::ex2_approx(y.y));
                    sum2[i & 3] = add2(sum2[i & 3], e);
                    if constexpr (BF16) w[i] = __byte_perm(__float_as_uint(e.x), __float_as_uint(e.y), 0x7632);
                    else w[i] = pack_pair<false>(e.x, e.y);
                }
                ptx::tmem_st_32x32b_x16(p_row + ch * 16, w);
            }
            const float2 tot = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
            l_run += tot.x + tot.y;
            ptx::tmem_st_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
        }
        // merge the two partial row sums, then write this thread's half of the output row
        if (ok) {
            volatile float* slot = xchg + (kv_tiles & 1) * 256;
            slot[half * 128 + row_in_tile] = l_run;
            ok = pair_exchange(wctx, pair_flags + (kv_tiles & 1) * 8, half, quarter, lane, (uint32_t)kv_tiles + 1, 0x020a0000u);
            if (ok) l_run += slot[(half ^ 1) * 128 + row_in_tile];
        }
        if (ok && __all_sync(0xffffffffu, bounded_wait(wctx, o_full, 0, 0x02080000u))) {
            // Every MMA has completed, so the Q tile's shared memory is free: the normalised output tile is
            // staged there in the same swizzled 128 x 64 halves and leaves through TMA stores (which drop the
            // rows beyond seq_q), one per destination.
            ptx::tc_fence_after_sync();
            const float inv = (BF16 ? 1.001953125f : 1.0f) / l_run;        // the bf16 exponentials carried a factor 1 + 2^-9
            const uint32_t row_smem = q_smem + half * (kTileQ * 128) + row_in_tile * 128;
            if constexpr (D == 128) {
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t o[32];
                    ptx::tmem_ld_32x32b_x32(o_row + ch * 32, o);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t slot = (uint32_t)(4 * ch + q) ^ (uint32_t)(row_in_tile & 7);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_smem + slot * 16),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv)),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv)),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv)),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv))
                                     : "memory");
                    }
                }
            } else {                                            // D == 64: one 128 x 64 piece, 32 columns per thread
                uint32_t o[32];
                ptx::tmem_ld_32x32b_x32(o_row, o);
                ptx::tmem_ld_wait();
                const uint32_t row64 = q_smem + row_in_tile * 128;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t slot = (uint32_t)(4 * half + q) ^ (uint32_t)(row_in_tile & 7);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row64 + slot * 16),
                                 "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv)),
                                 "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv)),
                                 "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv)),
                                 "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv))
                                 : "memory");
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(o_staged);
            if (p.mc_base != 0) {
                // every softmax thread waits for the staged tile, then the 256 of them copy it out: 16 (d = 128) or 8
                // (d = 64) threads per row, so each multicast store of a warp covers whole rows
                if (__all_sync(0xffffffffu, bounded_wait(wctx, o_staged, 0, 0x020b0000u))) {
                    constexpr int kSlots = D / 8;                   // 16-byte slots per output row
                    const int tt = (int)threadIdx.x - 64, slot = tt % kSlots;
                    const uint32_t chunk_smem = q_smem + (slot >> 3) * (kTileQ * 128);
#pragma unroll
                    for (int i = 0; i < kTileQ * kSlots / 256; ++i) {
                        const int r = tt / kSlots + (256 / kSlots) * i;
                        if (qt * kTileQ + r < p.seq_q) {
                            uint32_t w0, w1, w2, w3;
                            ptx::ld_shared_16B(chunk_smem + r * 128 + (((slot & 7) ^ (r & 7)) << 4), w0, w1, w2, w3);
                            const unsigned long long elem = ((unsigned long long)unit * p.seq_q + qt * kTileQ + r) * D + slot * 8;
                            ptx::multimem_st_16B(p.mc_base + elem * 2ull, w0, w1, w2, w3);
                        }
                    }
                }
            } else if (threadIdx.x == 64) {                     // first softmax thread: owns the stores
                if (bounded_wait(wctx, o_staged, 0, 0x020b0000u)) {
                    for (int d = 0; d < p.n_dst; ++d)
#pragma unroll
                        for (int c = 0; c < kChunks; ++c)
                            ptx::tma_store_3d(&out.m[d], q_smem + c * (kTileQ * 128), c * 64, qt * kTileQ, unit);
                    ptx::tma_store_commit();
                    ptx::tma_store_wait<0>();
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


// ---- two query tiles per CTA ------------------------------------------------------------------------------------------
// The kernel above overlaps one CTA's softmax with the other resident CTA's MMAs; inside a CTA the score product, the
// softmax and the value product of a key tile still run one after the other. This form keeps the tensor pipe fed from
// within one CTA: a persistent CTA per SM owns TWO 128-query tiles of one unit (S0, S1, O0, O1 = all 512 tensor-memory
// columns) and walks the key tiles once for both.
//   warp 0     TMA: the two Q tiles, then K_j / V_j through a four-stage ring (32 KiB each at d = 128)
//   warp 1     MMA issue, in the order  S0(0) S1(0) | O0+=P0 V(j)  S0(j+1)  O1+=P1 V(j)  S1(j+1) | ...  so that
//              while one tile's probabilities are being made the tensor pipe works on the other tile; descriptor
//              words are built once and a k-step costs the thread one add
//   warps 4-7, 8-11   softmax of tile 0 / tile 1, one thread per query row with the whole row of scores in registers
//              (setmaxnreg moves registers to these warps): no exchange between threads anywhere. The exponentials
//              are taken against a reference maximum fixed BEFORE the tile arrives (the first tile's own maximum,
//              raised between tiles when a later maximum exceeds it by more than 2^8): floating point does not care
//              how far from 1 the values sit, so the tile's own maximum is only needed for the next reference and is
//              computed after P has been handed to the MMA warp. A tile whose sum shows scores far above the
//              reference (2^64: never on ordinary data) is done again against a raised reference. The thread
//              rescales its own row of O in tensor memory on the rare raise. P (16-bit pairs) overwrites S.
//   warps 12-15  output: normalise O_i by the row sums, stage it in shared memory and store it (TMA, or multimem.st
//              for a multicast destination) while the MMA warp is already working on the next pair of tiles.
// Work items (unit, pair of query tiles) are dealt round-robin. With the causal flag a pair's cost grows with its
// position, so the pairs of all units are dealt longest first in rounds that alternate direction (pair_item): the
// static deal stays balanced to within a few key tiles per CTA. Every wait is bounded; the groups meet only
// through mbarriers (no bar.sync inside the role loops), so a wait that gives up cannot strand another warp.
constexpr int kPairThreads = 512;
constexpr int kKvStages = 4;
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
template <int D>
struct PairSmem {
    static constexpr int kQBytes = kTileQ * D * 2;
    static constexpr int kKvBytes = kTileK * D * 2;
    static constexpr int kOBytes = kTileQ * D * 2;
    static constexpr int kKvOffset = 2 * kQBytes;
    static constexpr int kOOffset = kKvOffset + kKvStages * kKvBytes;
    static constexpr int kBarOffset = kOOffset + kOBytes;
    static constexpr int kFloatOffset = kBarOffset + 512;            // corr[2][128], lsum[2][128]
    static constexpr int kTotal = kFloatOffset + 4 * 128 * 4;        // the base must be 1024-byte aligned (checked)
};

struct PairItem {
    int unit, row0;     // unit and first query row of tile 0
    int n[2];           // key tiles of tile 0 / tile 1 (0: the tile does not exist; n[0] == 0: nothing to do)
};

// Item `it` of this CTA. Returns false when the CTA's share is exhausted.
__device__ __forceinline__ bool pair_item(const AttParams& p, int it, PairItem& w) {
    const int q_pairs = (p.q_tiles + 1) >> 1;
    int unit, pr;
    if (!p.causal) {
        const long long t = (long long)blockIdx.x + (long long)it * gridDim.x;
        if (t >= (long long)p.units * q_pairs) return false;
        unit = (int)(t / q_pairs);
        pr = (int)(t % q_pairs);
    } else {
        // Pairs of every unit sorted by length, longest first (pair pr walks 2 pr + 2 key tiles), dealt in rounds of
        // gridDim.x that alternate direction: after every two rounds the CTAs' sums differ by at most one step of the
        // length, and the last, partial round holds the shortest pairs.
        const long long total = (long long)p.units * q_pairs;
        const long long pos = (it & 1) ? (long long)gridDim.x - 1 - blockIdx.x : (long long)blockIdx.x;
        const long long t = (long long)it * gridDim.x + pos;
        if (t >= total) return false;
        unit = (int)(t % p.units);
        pr = q_pairs - 1 - (int)(t / p.units);
    }
    const int kv_all = (p.seq_k + kTileK - 1) / kTileK;
    w.unit = unit;
    w.row0 = pr * 2 * kTileQ;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = w.row0 + i * kTileQ;
        w.n[i] = r >= p.seq_q ? 0 : (p.causal ? min(kv_all, r / kTileK + 1) : kv_all);
    }
    return true;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kPairThreads, 1)
attention_fwd_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttOutMaps out, AttParams p) {
    using S = PairSmem<D>;
    constexpr int kChunks = D / 64;
    constexpr uint32_t kColS = 128, kColO = 256, kColOStride = 128;     // S_i at i * 128, O_i at 256 + i * 128
    extern __shared__ __align__(1024) uint8_t smem_pair_raw[];
    const uint32_t smem_base = ptx::smem_u32(smem_pair_raw);
    if (smem_base & 1023u) {                                            // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, 0x02ff0000u);
        return;
    }
    uint8_t* smem_gen = smem_pair_raw;
    auto q_smem = [&](int i) { return smem_base + (uint32_t)i * S::kQBytes; };
    auto kv_smem = [&](uint32_t s) { return smem_base + S::kKvOffset + s * S::kKvBytes; };
    const uint32_t o_smem = smem_base + S::kOOffset;
    const uint32_t bar_base = smem_base + S::kBarOffset;
    auto bar = [&](int idx) { return bar_base + 8u * idx; };
    // barrier indices
    constexpr int Q_FULL = 0, Q_EMPTY = 2, KV_FULL = 4, KV_EMPTY = 8, S_FULL = 12, P_FULL = 14, O_FULL = 16, O_FREE = 18,
                  L_READY = 20, STAGE_READY = 28, STAGE_FREE = 29, N_BARS = 30;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + S::kBarOffset + 8 * N_BARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* lsum = reinterpret_cast<float*>(smem_gen + S::kFloatOffset);        // [2][128] final row sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(bar(Q_FULL + i), 1); ptx::mbar_init(bar(Q_EMPTY + i), 1); ptx::mbar_init(bar(S_FULL + i), 1);
            ptx::mbar_init(bar(P_FULL + i), 4); ptx::mbar_init(bar(O_FULL + i), 1);
            ptx::mbar_init(bar(O_FREE + i), 4);
            for (int w = 0; w < 4; ++w) ptx::mbar_init(bar(L_READY + 4 * i + w), 1);
        }
        for (int s = 0; s < kKvStages; ++s) { ptx::mbar_init(bar(KV_FULL + s), 1); ptx::mbar_init(bar(KV_EMPTY + s), 1); }
        ptx::mbar_init(bar(STAGE_READY), 4); ptx::mbar_init(bar(STAGE_FREE), p.mc_base != 0 ? 4 : 1);
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&map_q); ptx::prefetch_tensormap(&map_k); ptx::prefetch_tensormap(&map_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // Registers follow the work: 512 threads start with 128 each; the softmax warps (a whole row of scores per thread)
    // take 184, paid for by the correction warps and by the first warpgroup, whose threads mostly wait.
    // (Each role's branch starts with its own setmaxnreg, so that the register allocator sees one limit per branch.)
    constexpr int kRegsFirst = 64, kRegsSoftmax = 184, kRegsCorrection = 80;
    static_assert(4 * kRegsFirst + 8 * kRegsSoftmax + 4 * kRegsCorrection == 16 * 128, "the register file is 64 K registers");

    if (warp == 0) {
        // ---- TMA producer --------------------------------------------------------------------------------------------
        ptx::setmaxnreg_dec<kRegsFirst>();
        if (lane == 0) {
            uint32_t kvr = 0, cq[2] = {0, 0};
            bool ok = true;
            PairItem w;
            auto load_kv = [&](const CUtensorMap* map, int j) -> bool {
                const uint32_t s = kvr & (kKvStages - 1), ph = (kvr / kKvStages) & 1;
                if (!bounded_wait(wctx, bar(KV_EMPTY + s), ph ^ 1, 0x03010000u | (kvr & 0xffff))) return false;
                ptx::mbar_arrive_expect_tx(bar(KV_FULL + s), S::kKvBytes);
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
                    ptx::tma_load_3d(kv_smem(s) + c * (kTileK * 128), map, bar(KV_FULL + s), c * 64, j * kTileK, w.unit);
                ++kvr;
                return true;
            };
            for (int it = 0; ok && pair_item(p, it, w); ++it) {
                if (w.n[0] == 0) continue;
                const int nmax = max(w.n[0], w.n[1]);
                if (!(ok = load_kv(&map_k, 0))) break;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (w.n[i] == 0 || !ok) continue;
                    if (!(ok = bounded_wait(wctx, bar(Q_EMPTY + i), (cq[i] & 1) ^ 1, 0x03020000u | i))) break;
                    ++cq[i];
                    ptx::mbar_arrive_expect_tx(bar(Q_FULL + i), S::kQBytes);
#pragma unroll
                    for (int c = 0; c < kChunks; ++c)
                        ptx::tma_load_3d(q_smem(i) + c * (kTileQ * 128), &map_q, bar(Q_FULL + i), c * 64, w.row0 + i * kTileQ, w.unit);
                }
                if (!ok || !(ok = load_kv(&map_v, 0))) break;
                for (int j = 1; j < nmax && ok; ++j) ok = load_kv(&map_k, j) && load_kv(&map_v, j);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------------------------
        ptx::setmaxnreg_dec<kRegsFirst>();
        if (lane == 0) {
            constexpr uint32_t idesc_s = ptx::mma_idesc_f16(BF16, false, false, kTileQ, kTileK);
            constexpr uint32_t idesc_o = ptx::mma_idesc_f16(BF16, false, true, kTileQ, D);
            uint32_t kvr = 0, cq[2] = {0, 0}, cp[2] = {0, 0}, cof[2] = {0, 0};
            bool ok = true;
            PairItem w;
            // This thread's waits sit on the chain P ready -> MMAs -> S ready of both tiles: it polls (bounded_spin)
            // instead of parking in try_wait, whose resume latency would be paid twice per key tile.
            auto kv_wait = [&](uint32_t r, uint32_t code) {
                return bounded_spin(wctx, bar(KV_FULL + (r & (kKvStages - 1))), (r / kKvStages) & 1, code | (r & 0xffff));
            };
            // Descriptor words built once: per k-step the issuing thread adds a constant to a low word.
            constexpr uint32_t kDescHi = ptx::smem_desc_sw128_hi(1024);
            const uint32_t q_lo0 = ptx::smem_desc_sw128_lo(q_smem(0), 16), q_lo1 = ptx::smem_desc_sw128_lo(q_smem(1), 16);
            const uint32_t k_lo = ptx::smem_desc_sw128_lo(kv_smem(0), 16), v_lo = ptx::smem_desc_sw128_lo(kv_smem(0), kTileK * 128);
            auto issue_s = [&](int i, uint32_t r) {                      // S_i = Q_i K^T with K in ring slot r
                const uint32_t kb = k_lo + (r & (kKvStages - 1)) * (S::kKvBytes >> 4), qb = i ? q_lo1 : q_lo0;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    constexpr uint32_t kChunk = (kTileQ * 128) >> 4;
                    const uint32_t off = (kk / 4) * kChunk + (kk % 4) * 2;          // in 16-byte units
                    ptx::mma_ss_words(tmem_base + i * kColS, qb + off, kb + off, kDescHi, idesc_s, kk != 0);
                }
                ptx::mma_commit(bar(S_FULL + i));
            };
            auto issue_pv = [&](int i, uint32_t r, bool first) {         // O_i (+)= P_i V with V in ring slot r
                const uint32_t vb = v_lo + (r & (kKvStages - 1)) * (S::kKvBytes >> 4);
#pragma unroll
                for (int kk = 0; kk < kTileK / 16; ++kk)
                    ptx::mma_ts_words(tmem_base + kColO + i * kColOStride, tmem_base + i * kColS + kk * 8, vb + kk * ((16 * 128) >> 4), kDescHi,
                                      idesc_o, !(first && kk == 0));
            };
            for (int it = 0; ok && pair_item(p, it, w); ++it) {
                if (w.n[0] == 0) continue;
                const int nmax = max(w.n[0], w.n[1]);
                if (!(ok = kv_wait(kvr, 0x03030000u))) break;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (w.n[i] == 0 || !ok) continue;
                    if (!(ok = bounded_spin(wctx, bar(Q_FULL + i), cq[i] & 1, 0x03040000u | i))) break;
                    ++cq[i];
                    ptx::tc_fence_after_sync();
                    issue_s(i, kvr);
                    if (w.n[i] == 1) ptx::mma_commit(bar(Q_EMPTY + i));
                }
                if (!ok) break;
                ptx::mma_commit(bar(KV_EMPTY + (kvr & (kKvStages - 1))));
                for (int j = 0; j < nmax && ok; ++j) {
                    const uint32_t rv = kvr + 2 * j + 1, rk = rv + 1;
                    bool v_waited = false, k_waited = false;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        if (j >= w.n[i] || !ok) continue;
                        if (!(ok = bounded_spin(wctx, bar(P_FULL + i), cp[i] & 1, 0x03050000u | (j & 0xffff)))) break;
                        ++cp[i];
                        if (j == 0) {                               // the previous item's O_i has been read out
                            if (!(ok = bounded_spin(wctx, bar(O_FREE + i), (cof[i] & 1) ^ 1, 0x03060000u | i))) break;
                            ++cof[i];
                        }
                        if (!v_waited) {
                            if (!(ok = kv_wait(rv, 0x03080000u))) break;
                            v_waited = true;
                        }
                        ptx::tc_fence_after_sync();
                        issue_pv(i, rv, j == 0);
                        if (j == w.n[i] - 1) ptx::mma_commit(bar(O_FULL + i));
                        if (j + 1 < w.n[i]) {
                            if (!k_waited) {
                                if (!(ok = kv_wait(rk, 0x03090000u))) break;
                                k_waited = true;
                                ptx::tc_fence_after_sync();
                            }
                            issue_s(i, rk);
                            if (j + 2 == w.n[i]) ptx::mma_commit(bar(Q_EMPTY + i));
                        }
                    }
                    if (!ok) break;
                    ptx::mma_commit(bar(KV_EMPTY + (rv & (kKvStages - 1))));
                    if (j + 1 < nmax) ptx::mma_commit(bar(KV_EMPTY + (rk & (kKvStages - 1))));
                }
                kvr += 2 * nmax;
            }
        }
        __syncwarp();
    } else if (warp < 4) {
        ptx::setmaxnreg_dec<kRegsFirst>();                             // the two spare warps of the first warpgroup
    } else if (warp < 12) {
        // ---- softmax of tile g: one thread per query row ---------------------------------------------------------------
        ptx::setmaxnreg_inc<kRegsSoftmax>();
        const int g = (warp - 4) >> 2, wq = warp & 3;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t s_row = tmem_base + lane_base + g * kColS;       // this row's 128 scores; P goes over their first 64 columns
        const float c = p.scale_log2;
        const float fill = c > 0.0f ? -CUDART_INF_F : CUDART_INF_F;
        uint32_t cs = 0;
        bool ok = true;
        PairItem w;
        // O_g row *= f, eight columns at a time (few registers: it runs beside a live row of scores); whole warps only
        auto rescale_o = [&](float f) {
            ptx::tc_fence_after_sync();
            const uint32_t o_row = tmem_base + lane_base + kColO + g * kColOStride;
#pragma unroll 1
            for (int col = 0; col < D; col += 8) {
                uint32_t o[8];
                ptx::tmem_ld_32x32b_x8(o_row + col, o);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                ptx::tmem_st_32x32b_x8(o_row + col, o);
            }
            ptx::tmem_st_wait();
        };
        for (int it = 0; ok && pair_item(p, it, w); ++it) {
            if (w.n[g] == 0) continue;
            const int q_row = w.row0 + g * kTileQ + row;
            float m_run = -CUDART_INF_F, l_run = 0.0f, f_pend = 1.0f;
            for (int j = 0; j < w.n[g] && ok; ++j) {
                ok = __all_sync(0xffffffffu, bounded_wait(wctx, bar(S_FULL + g), cs & 1, 0x030a0000u | (j & 0xffff)));
                if (!ok) break;
                ++cs;
                ptx::tc_fence_after_sync();
                int valid = p.seq_k - j * kTileK;
                if (p.causal) valid = min(valid, q_row - j * kTileK + 1);
                const bool ragged = valid < kTileK;
                // S_i(j) is ready, so O_i holds every product up to tile j - 1: this is where a raise of the reference
                // decided at the previous tile is applied to the accumulator (rare) and to the running sum.
                if (j > 0) {
                    if (__any_sync(0xffffffffu, f_pend != 1.0f)) rescale_o(f_pend);
                    l_run *= f_pend;
                }
                // the whole row of scores into registers: four loads in flight, one wait
                uint32_t r[kTileK];
#pragma unroll
                for (int ch = 0; ch < kTileK / 32; ++ch) ptx::tmem_ld_32x32b_x32(s_row + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[ch * 32]));
                ptx::tmem_ld_wait();
                if (ragged) {                                           // last key tile, or the causal diagonal
#pragma unroll
                    for (int i = 0; i < kTileK; ++i)
                        if (i >= valid) r[i] = __float_as_uint(fill);
                }
                // c * (row extremum): four chains of three-input max / min
                auto row_max = [&]() -> float {
                    float ext[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) ext[i] = __uint_as_float(r[i]);
                    if (c > 0.0f) {
#pragma unroll
                        for (int i = 4; i < kTileK; i += 8) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int a0 = i + 2 * q, a1 = a0 + 1;
                                if (a1 < kTileK) ext[q] = max3(ext[q], __uint_as_float(r[a0]), __uint_as_float(r[a1]));
                                else if (a0 < kTileK) ext[q] = fmaxf(ext[q], __uint_as_float(r[a0]));
                            }
                        }
                        return fmaxf(fmaxf(ext[0], ext[1]), fmaxf(ext[2], ext[3])) * c;
                    }
#pragma unroll
                    for (int i = 4; i < kTileK; i += 8) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int a0 = i + 2 * q, a1 = a0 + 1;
                            if (a1 < kTileK) ext[q] = min3(ext[q], __uint_as_float(r[a0]), __uint_as_float(r[a1]));
                            else if (a0 < kTileK) ext[q] = fminf(ext[q], __uint_as_float(r[a0]));
                        }
                    }
                    return fminf(fminf(ext[0], ext[1]), fminf(ext[2], ext[3])) * c;
                };
                // The exponentials are taken against the reference m_run that was fixed BEFORE this tile (the first tile's
                // own maximum, afterwards raised between tiles only): floating point does not care how far below or above
                // 1 the values sit, so this tile's maximum is needed only to decide the next reference and to guard
                // against overflow -- it is computed beside the exponentials, off the path from S to P.
                float m_tile = 0.0f;
                if (j == 0) m_run = m_tile = row_max();
                // p = 2^(c s - m). bf16: P is the upper half of the fp32 bit pattern, one byte-permute per pair, because the
                // conversion of a pair of floats to 16 bits runs on the transcendental unit like the exponentials, which
                // is the unit this loop is bound by. Truncation loses half a 16-bit ulp on average, so every exponent is
                // taken kTruncBiasLog2 higher (a factor 1 + 2^-9) and the row sum is scaled back once at the end.
                float2 sum2[2];
                auto emit = [&]() {
                    const float shift = BF16 ? kTruncBiasLog2 - m_run : -m_run;
                    const float2 c2 = make_float2(c, c), nm2 = make_float2(shift, shift);
                    sum2[0] = sum2[1] = make_float2(0.0f, 0.0f);
#pragma unroll
                    for (int ch = 0; ch < kTileK / 32; ++ch) {
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int e0 = ch * 32 + 2 * i;
                            const float2 y = fma2(make_float2(__uint_as_float(r[e0]), __uint_as_float(r[e0 + 1])), c2, nm2);
                            const float2 e = make_float2(ptx::ex2_approx(y.x), ptx::ex2_approx(y.y));
                            sum2[i & 1] = add2(sum2[i & 1], e);
                            if constexpr (BF16) pk[i] = __byte_perm(__float_as_uint(e.x), __float_as_uint(e.y), 0x7632);
                            else pk[i] = pack_pair<false>(e.x, e.y);
                        }
                        ptx::tmem_st_32x32b_x16(s_row + ch * 16, pk);
                    }
                };
                emit();
                float2 tot = add2(sum2[0], sum2[1]);
                // Scores far above the reference show in the tile's sum: beyond 2^64 (never on ordinary data) the
                // reference is raised now, the accumulator and the sum are brought along, and this tile's exponentials
                // are taken again.
                if (j > 0 && __any_sync(0xffffffffu, !(tot.x + tot.y < 1.8446744e19f))) {
                    m_tile = row_max();
                    const bool over = m_tile > m_run + 32.0f;
                    const float f = over ? ptx::ex2_approx(m_run - m_tile) : 1.0f;
                    rescale_o(f);
                    l_run *= f;
                    if (over) m_run = m_tile;
                    emit();
                    tot = add2(sum2[0], sum2[1]);
                }
                l_run += tot.x + tot.y;
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar(P_FULL + g));
                // With P handed over, the tile's own maximum and from it the reference for the next tile: raised only
                // when the maximum exceeds the current one by more than 2^8.
                if (j > 0) m_tile = row_max();
                {
                    const bool raise = m_tile > m_run + 8.0f;
                    f_pend = raise ? ptx::ex2_approx(m_run - m_tile) : 1.0f;
                    m_run = raise ? m_tile : m_run;
                }
            }
            if (!ok) break;
            lsum[g * 128 + row] = BF16 ? l_run * (1.0f / 1.001953125f) : l_run;      // the exponentials carried a factor 1 + 2^-9
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(L_READY + 4 * g + wq));
        }
    } else {
        // ---- correction and output ---------------------------------------------------------------------------------------
        ptx::setmaxnreg_dec<kRegsCorrection>();
        const int wq = warp & 3;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const bool issuer = threadIdx.x == 12 * 32;
        uint32_t cl[2] = {0, 0}, cfull[2] = {0, 0}, cstage = 0;
        bool ok = true;
        PairItem w;
        for (int it = 0; ok && pair_item(p, it, w); ++it) {
            if (w.n[0] == 0) continue;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (w.n[i] == 0 || !ok) continue;
                ok = __all_sync(0xffffffffu, bounded_wait(wctx, bar(L_READY + 4 * i + wq), cl[i] & 1, 0x030c0000u | i));
                if (!ok) break;
                ++cl[i];
                const float inv = 1.0f / lsum[i * 128 + row];
                ok = __all_sync(0xffffffffu, bounded_wait(wctx, bar(O_FULL + i), cfull[i] & 1, 0x030d0000u | i));
                if (!ok) break;
                ++cfull[i];
                // the staging tile is free once the previous tile's stores (or multicast copies) have read it
                ok = __all_sync(0xffffffffu, bounded_wait(wctx, bar(STAGE_FREE), (cstage & 1) ^ 1, 0x030e0000u | i));
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t o_row = tmem_base + lane_base + kColO + i * kColOStride;
#pragma unroll 1
                for (int ch = 0; ch < D / 32; ++ch) {
                    uint32_t o[32];
                    ptx::tmem_ld_32x32b_x32(o_row + ch * 32, o);
                    ptx::tmem_ld_wait();
                    const uint32_t row_smem = o_smem + (ch >> 1) * (kTileQ * 128) + row * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t slot = (uint32_t)(4 * (ch & 1) + q) ^ (uint32_t)(row & 7);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_smem + slot * 16),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv)),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv)),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv)),
                                     "r"(pack_pair<BF16>(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv))
                                     : "memory");
                    }
                }
                ptx::tc_fence_before_sync();
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(bar(O_FREE + i));                  // O_i may be overwritten by the next item's first value product
                    ptx::mbar_arrive(bar(STAGE_READY));
                }
                const int tile_row0 = w.row0 + i * kTileQ;
                if (p.mc_base != 0) {
                    ok = __all_sync(0xffffffffu, bounded_wait(wctx, bar(STAGE_READY), cstage & 1, 0x030f0000u | i));
                    if (!ok) break;
                    constexpr int kSlots = D / 8;                       // 16-byte slots per output row
                    const int tt = (int)threadIdx.x - 12 * 32, slot = tt % kSlots;
                    const uint32_t chunk_smem = o_smem + (slot >> 3) * (kTileQ * 128);
#pragma unroll
                    for (int e = 0; e < kTileQ * kSlots / 128; ++e) {
                        const int r = tt / kSlots + (128 / kSlots) * e;
                        if (tile_row0 + r < p.seq_q) {
                            uint32_t w0, w1, w2, w3;
                            ptx::ld_shared_16B(chunk_smem + r * 128 + (((slot & 7) ^ (r & 7)) << 4), w0, w1, w2, w3);
                            const unsigned long long elem = ((unsigned long long)w.unit * p.seq_q + tile_row0 + r) * D + slot * 8;
                            ptx::multimem_st_16B(p.mc_base + elem * 2ull, w0, w1, w2, w3);
                        }
                    }
                    // the next tile's staging writes must come after these reads: every warp reports when it is done
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar(STAGE_FREE));
                } else if (issuer) {
                    if (bounded_wait(wctx, bar(STAGE_READY), cstage & 1, 0x030f0000u | i)) {
                        for (int d = 0; d < p.n_dst; ++d)
#pragma unroll
                            for (int cc2 = 0; cc2 < kChunks; ++cc2)
                                ptx::tma_store_3d(&out.m[d], o_smem + cc2 * (kTileQ * 128), cc2 * 64, tile_row0, w.unit);
                        ptx::tma_store_commit();
                        ptx::tma_store_wait_read<0>();
                    }
                    ptx::mbar_arrive(bar(STAGE_FREE));
                }
                ++cstage;
            }
        }
        if (issuer) ptx::tma_store_wait<0>();
        if (p.mc_base != 0) __threadfence_system();
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 512);
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
static int launch_attention(const void* Q, const void* K, const void* V, void* const* O, int n_dst, bool causal, bool multicast, int form_flags, int64_t units,
                            int64_t seq_q, int64_t seq_k, float scale, cudaStream_t stream) {
    using S = AttSmem<D>;
    CUtensorMap mq, mk, mv;
    int rc = make_tensor_map_3d(&mq, Q, (uint64_t)units, (uint64_t)seq_q, D, kTileQ, 64);
    if (rc == EMMYB200_OK) rc = make_tensor_map_3d(&mk, K, (uint64_t)units, (uint64_t)seq_k, D, kTileK, 64);
    if (rc == EMMYB200_OK) rc = make_tensor_map_3d(&mv, V, (uint64_t)units, (uint64_t)seq_k, D, kTileK, 64);
    AttOutMaps out;
    for (int d = 0; d < kMaxDst && rc == EMMYB200_OK; ++d) {
        if (multicast) out.m[d] = mq;                               // unused: the stores go through multimem.st
        else rc = make_tensor_map_3d(&out.m[d], O[d < n_dst ? d : 0], (uint64_t)units, (uint64_t)seq_q, D, kTileQ, 64);
    }
    if (rc != EMMYB200_OK) return rc;
    AttParams p;
    p.n_dst = n_dst; p.causal = causal ? 1 : 0; p.units = (int)units; p.seq_q = (int)seq_q; p.seq_k = (int)seq_k;
    p.mc_base = multicast ? (unsigned long long)(uintptr_t)O[0] : 0ull;
    p.q_tiles = (int)((seq_q + kTileQ - 1) / kTileQ);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.wait_limit_ns = wait_limit_ns();
    EMMY_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_att_status));
    const int64_t ctas = units * p.q_tiles;
    if (ctas >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: %lld query tiles exceed the grid limit", (long long)ctas);
    // Which form. Measured over units x sequence length x head size, with and without the causal flag (bf16, both forms
    // forced in the same run): the two-tile form is 2-34 % faster once a unit has eight or more key tiles and there is
    // at least one pair of query tiles per SM (its persistent CTAs walk the keys once for two tiles, and with the causal
    // flag its sorted, alternating deal of the pairs keeps every SM busy to the end); for short sequences or few work items the
    // one-tile form, with twice as many and smaller work items, is 1-67 % faster. A flag overrides the choice.
    const int64_t pair_items = units * ((p.q_tiles + 1) / 2);
    const bool two_tiles = (form_flags & EMMYB200_ATT_FORM_TWO_TILES) ? true
                         : ((form_flags & EMMYB200_ATT_FORM_ONE_TILE) ? false : (pair_items >= sm_count() && seq_k >= 8 * kTileK));
    if (two_tiles) {
        using P = PairSmem<D>;
        auto pair_kernel = attention_fwd_pair_kernel<D, BF16>;
        EMMY_CUDA(cudaFuncSetAttribute(pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::kTotal));
        const int64_t q_pairs = (p.q_tiles + 1) / 2;
        const int64_t deals = units * q_pairs;
        const int grid = (int)(deals < sm_count() ? deals : sm_count());
        pair_kernel<<<grid, kPairThreads, P::kTotal, stream>>>(mq, mk, mv, out, p);
        return launch_status("attention_fwd_pair_kernel");
    }
    auto kernel = attention_fwd_kernel<D, BF16>;
    EMMY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    kernel<<<(unsigned)ctas, kAttThreads, S::kTotal, stream>>>(mq, mk, mv, out, p);
    return launch_status("attention_fwd_kernel");
}

}  // namespace emmy

namespace emmy {
// attention_f32.cu
int attention_cuda_cores(int dtype, bool causal, const void* Q, const void* K, const void* V, void* O, int64_t units, int64_t seq_q,
                         int64_t seq_k, int64_t d, float scale, cudaStream_t s);
}  // namespace emmy

static int attention_entry(int dtype, int flags, const void* Q, const void* K, const void* V, void* const* O, int n_dst, int64_t units,
                           int64_t seq_q, int64_t seq_k, int64_t d, float scale, void* cuda_stream) {
    using namespace emmy;
    if (dtype != EMMYB200_F16 && dtype != EMMYB200_BF16 && dtype != EMMYB200_F32) return fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: dtype %d (f32, f16 and bf16 only)", dtype);
    if (flags & ~(EMMYB200_ATT_CAUSAL | EMMYB200_ATT_DST_MULTICAST | EMMYB200_ATT_FORM_ONE_TILE | EMMYB200_ATT_FORM_TWO_TILES)) return fail(EMMYB200_ERR_ARG, "attention_fwd: unknown flags 0x%x", flags);
    const bool causal = flags & EMMYB200_ATT_CAUSAL;
    const bool multicast = flags & EMMYB200_ATT_DST_MULTICAST;
    const int form = flags & (EMMYB200_ATT_FORM_ONE_TILE | EMMYB200_ATT_FORM_TWO_TILES);
    if (form == (EMMYB200_ATT_FORM_ONE_TILE | EMMYB200_ATT_FORM_TWO_TILES)) return fail(EMMYB200_ERR_ARG, "attention_fwd: one form flag at most");
    if (multicast && n_dst != 1) return fail(EMMYB200_ERR_ARG, "attention_fwd: a multicast destination is a single address");
    if (n_dst < 1 || n_dst > kMaxDst) return fail(EMMYB200_ERR_ARG, "attention_fwd: %d destinations (1 to %d)", n_dst, kMaxDst);
    if (units < 0 || seq_q < 0 || seq_k < 0) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: negative extent");
    if (units == 0 || seq_q == 0) return EMMYB200_OK;
    if (seq_k == 0) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: seq_k = 0 (softmax over no keys)");
    const bool cuda_cores = dtype == EMMYB200_F32 || (d != 64 && d != 128);        // fp32 arithmetic, or a head size the tensor-core kernels lack
    if (cuda_cores && (d % 32 != 0 || d < 32 || d > 128)) return fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: head dim %lld (a multiple of 32 up to 128)", (long long)d);
    if (cuda_cores && (n_dst != 1 || multicast || form != 0))
        return fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: f32 buffers and head sizes other than 64 / 128 have one destination and one kernel form");
    if (seq_q >= (1ll << 31) || seq_k >= (1ll << 31) || units >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "attention_fwd: extents must be below 2^31");
    if (Q == nullptr || K == nullptr || V == nullptr || O == nullptr) return fail(EMMYB200_ERR_ARG, "attention_fwd: null buffer");
    for (int i = 0; i < n_dst; ++i) {
        if (O[i] == nullptr) return fail(EMMYB200_ERR_ARG, "attention_fwd: null buffer");
        if (!aligned(O[i], 16)) return fail(EMMYB200_ERR_ALIGN, "attention_fwd: buffers must be 16-byte aligned");
    }
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16)) return fail(EMMYB200_ERR_ALIGN, "attention_fwd: buffers must be 16-byte aligned");
    if (!(scale == scale) || scale == 0.0f) return fail(EMMYB200_ERR_ARG, "attention_fwd: scale must be a non-zero number");
    int rc = check_sm100();
    if (rc != EMMYB200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    if (cuda_cores) return attention_cuda_cores(dtype, causal, Q, K, V, O[0], units, seq_q, seq_k, d, scale, s);
    const bool bf16 = dtype == EMMYB200_BF16;
    if (d == 128) return bf16 ? launch_attention<128, true>(Q, K, V, O, n_dst, causal, multicast, form, units, seq_q, seq_k, scale, s)
                              : launch_attention<128, false>(Q, K, V, O, n_dst, causal, multicast, form, units, seq_q, seq_k, scale, s);
    return bf16 ? launch_attention<64, true>(Q, K, V, O, n_dst, causal, multicast, form, units, seq_q, seq_k, scale, s)
                : launch_attention<64, false>(Q, K, V, O, n_dst, causal, multicast, form, units, seq_q, seq_k, scale, s);
}

extern "C" int emmyb200_attention_fwd(int dtype, int flags, const void* Q, const void* K, const void* V, void* O, int64_t units,
                                      int64_t seq_q, int64_t seq_k, int64_t d, float scale, void* cuda_stream) {
    void* dst[1] = {O};
    if (flags & EMMYB200_ATT_DST_MULTICAST) return emmy::fail(EMMYB200_ERR_ARG, "attention_fwd: the multicast flag belongs to emmyb200_attention_fwd_allgather");
    return attention_entry(dtype, flags, Q, K, V, dst, 1, units, seq_q, seq_k, d, scale, cuda_stream);
}

extern "C" int emmyb200_attention_fwd_allgather(int dtype, int flags, const void* Q, const void* K, const void* V, void* const* O_dst,
                                                int n_dst, int64_t units, int64_t seq_q, int64_t seq_k, int64_t d, float scale,
                                                void* cuda_stream) {
    if (O_dst == nullptr) return emmy::fail(EMMYB200_ERR_ARG, "attention_fwd_allgather: null destination list");
    return attention_entry(dtype, flags, Q, K, V, O_dst, n_dst, units, seq_q, seq_k, d, scale, cuda_stream);
}
