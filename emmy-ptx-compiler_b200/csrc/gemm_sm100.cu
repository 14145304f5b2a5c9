// Dense contraction C[M,N] = epilogue(A[M,K] . B), fp16 / bf16 operands, fp32 accumulation.
//
// The reference builds this from per-warp m16n8k16 `mma.sync` cells fed through registers by
// `ldmatrix` / `cp.async` (emmyptx/mma.py:65-242, emmyptx/kernel.py:735-755) inside a rotated K loop
// (emmyptx/loops.py:231-264), converts with `cvt.rn` and stores two elements at a time, and
// refuses fused store epilogues (emmyptx/mma.py:201-203). This file is the sm_100a form:
//
//   * persistent CTAs, one per SM, walking 128 x BN output tiles in an order that keeps a band
//     of A row-blocks hot in L2;
//   * warp 0 (one thread) streams 128x64 A tiles and 64xBN B tiles into a ring of
//     128-byte-swizzled shared-memory stages with TMA, out-of-range parts zero-filled, so
//     ragged M, N, K need no guards in the main loop;
//   * warp 1 (one thread) issues tcgen05.mma 128 x BN x 16 from shared-memory descriptors into
//     one of two accumulator buffers in tensor memory, and releases stages / publishes
//     accumulators with tcgen05.commit;
//   * warps 2-5 drain the other accumulator buffer (tcgen05.ld), apply the epilogue on the fp32
//     values, round once to the output type, stage 128 x 64 pieces in swizzled shared memory and
//     hand them to TMA stores, overlapping the next tile's main loop. A store goes to every
//     destination tensor of the launch: the local C, and -- when the rows of C are sharded over
//     several GPUs -- the same rows of each peer's C over NVLink, which is the all-gather of the
//     output done by the kernel that produces it.
//
// B may be row-major K x N (an "MN-major" operand: TMA boxes of 64 N-elements per K row, and
// the MMA told to transpose) or row-major N x K (K-major, like A).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace emmy {

constexpr int kBM = 128, kBK = 64, kUmmaK = 16;
constexpr int kGemmThreads = 192;          // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue

template <int BN>
struct GemmSmem {
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (BN == 256) ? 4 : (BN == 192 ? 5 : 6);
    static constexpr int kOutBytes = kBM * 64 * 2;                                // one 128 x 64 output piece
    static constexpr int kOutOffset = kStages * kStageBytes;
    static constexpr int kBarOffset = kOutOffset + 2 * kOutBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kTotal = kBarOffset + kBarrierBytes + 1024;              // + alignment slack
};

constexpr int kMaxDst = 8;

struct GemmParams {
    int M, N, K;
    int m_blocks, n_blocks;
    int batch;              // independent products (planes of A and C; B has `batch` planes or one shared plane)
    int b_shared;           // 1: every product reads plane 0 of B
    int n_dst;              // destinations of every output piece (1 = the local C only)
    int epilogue;           // EMMYB200_EPI_*
    const void* bias;       // per-column addend of the output type, or null
    unsigned long long mc_base;     // != 0: C as a multicast address (stores go out through multimem.st, once, to every GPU)
    long long ldc, stride_c;        // of C, in elements (multicast mode only; the TMA path has them in its tensor maps)
    unsigned long long wait_limit_ns;       // after which a pipeline wait gives up
    uint32_t* status;
};

struct OutMaps {
    CUtensorMap m[kMaxDst];
};

__device__ uint32_t g_gemm_status;

// Tile order: bands of 16 row-blocks, column-blocks inside a band, row-blocks fastest, so CTAs that
// run together share B column-blocks and a small set of A row-blocks.
__device__ __forceinline__ void tile_coords(int t, int m_blocks, int n_blocks, int& mb, int& nb) {
    constexpr int kBand = 16;       // measured best of 2..64 at 8192^3 (1356 TFLOP/s at 2 or 64, 1473 at 16)
    const int per_band = kBand * n_blocks;
    const int band = t / per_band;
    const int first = band * kBand;
    const int rows = min(kBand, m_blocks - first);
    const int within = t - band * per_band;
    mb = first + within % rows;
    nb = within / rows;
}

// x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715 x^3): algebraically the tanh form of GELU, with no
// cancellation for large negative x. ex2 / rcp approximations: relative error around 1e-6, far
// below the one rounding to a 16-bit type that follows.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float u = 0.7978845608f * fmaf(0.044715f * x * x, x, x);
    const float e = ptx::ex2_approx(-2.8853900818f * u);       // exp(-2u) = 2^(-2 log2(e) u)
    return x * ptx::rcp_approx(1.0f + e);
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
    else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool BF16>
__device__ __forceinline__ float unpack1(uint16_t h) {
    if constexpr (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&h));
    else return __half2float(*reinterpret_cast<const __half*>(&h));
}

constexpr int kOutPieceBytes = kBM * 64 * 2;       // one 128 x 128-byte output piece in shared memory

// The epilogue of one 128 x BN accumulator (this CTA's rows row0 .., columns col0 ..): tensor memory -> registers
// (bias, activation, one rounding) -> swizzled 128-byte-wide pieces in shared memory -> TMA stores to every
// destination, or multimem.st to a multicast destination. Run by the four epilogue warps together (named barrier 1);
// `release` hands the accumulator buffer back once its last column has been read.
template <int BN, bool BF16, bool F32, typename Release>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, const OutMaps& out, uint32_t t_row, uint32_t out_smem,
                                                  uint32_t& piece, int row0, int col0, int plane, int row_in_tile, int epi_thread,
                                                  bool issuer, Release release) {
    constexpr int kPiece = F32 ? 32 : 64;                 // columns of one 128-byte-wide output piece
#pragma unroll 1
    for (int c = 0; c < BN; c += kPiece, ++piece) {
        const uint32_t stage = out_smem + (piece & 1) * kOutPieceBytes;
        // the stores that last read this staging buffer (two pieces ago) must be done with it
        if (issuer) ptx::tma_store_wait_read<1>();
        ptx::named_barrier(1, 128);
        const uint32_t row_smem = stage + row_in_tile * 128;
        if constexpr (F32) {
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(t_row + c, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = __uint_as_float(r[4 * q + j]);
                if (p.bias != nullptr) {
                    const int col = col0 + c + 4 * q;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (col + j < p.N) v[j] += __ldg(reinterpret_cast<const float*>(p.bias) + col + j);
                }
                if (p.epilogue == EMMYB200_EPI_GELU_TANH) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = gelu_tanh_fast(v[j]);
                } else if (p.epilogue == EMMYB200_EPI_RELU) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = fmaxf(v[j], 0.0f);
                }
                const uint32_t slot = (uint32_t)q ^ (uint32_t)(row_in_tile & 7);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_smem + slot * 16), "r"(__float_as_uint(v[0])),
                             "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3]))
                             : "memory");
            }
        }
#pragma unroll
        for (int h = 0; h < (F32 ? 0 : 2); ++h) {
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(t_row + c + 32 * h, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[8 * q + j]);
                if (p.bias != nullptr) {                // eight columns' worth, the same for every row
                    const int col = col0 + c + 32 * h + 8 * q;
                    if (col + 8 <= p.N) {
                        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias) + col));
                        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 b2 = unpack2<BF16>(w[j]);
                            v[2 * j] += b2.x;
                            v[2 * j + 1] += b2.y;
                        }
                    } else {
                        for (int j = 0; j < 8 && col + j < p.N; ++j) v[j] += unpack1<BF16>(reinterpret_cast<const uint16_t*>(p.bias)[col + j]);
                    }
                }
                if (p.epilogue == EMMYB200_EPI_GELU_TANH) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh_fast(v[j]);
                } else if (p.epilogue == EMMYB200_EPI_RELU) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.0f);
                }
                // 16-byte slot (4h + q) of the row, at its 128-byte-swizzle position
                const uint32_t slot = (uint32_t)(4 * h + q) ^ (uint32_t)(row_in_tile & 7);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_smem + slot * 16),
                             "r"(pack2<BF16>(v[0], v[1])), "r"(pack2<BF16>(v[2], v[3])),
                             "r"(pack2<BF16>(v[4], v[5])), "r"(pack2<BF16>(v[6], v[7]))
                             : "memory");
            }
        }
        if (c + kPiece >= BN) {                          // accumulator fully read: hand it back
            ptx::tc_fence_before_sync();
            __syncwarp();
            release();
        }
        ptx::fence_proxy_async_smem();
        ptx::named_barrier(1, 128);
        if (p.mc_base != 0) {
            if constexpr (!F32) {
                // 128 threads copy the 128 x 128-byte piece: 8 threads per row, 16 rows per pass, so every
                // multicast store instruction of a warp covers four full 128-byte rows
                const int tt = epi_thread, s16 = tt & 7;
                const int col = col0 + c + s16 * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = (tt >> 3) + 16 * i;
                    const int grow = row0 + r;
                    if (grow < p.M && col < p.N) {
                        uint32_t w0, w1, w2, w3;
                        ptx::ld_shared_16B(stage + r * 128 + ((s16 ^ (r & 7)) << 4), w0, w1, w2, w3);
                        const long long elem = (long long)plane * p.stride_c + (long long)grow * p.ldc + col;
                        ptx::multimem_st_16B(p.mc_base + (unsigned long long)elem * 2ull, w0, w1, w2, w3);
                    }
                }
            }
        } else {
            if (issuer && col0 + c < p.N) {
                for (int d = 0; d < p.n_dst; ++d) ptx::tma_store_3d(&out.m[d], stage, col0 + c, row0, plane);
            }
            if (issuer) ptx::tma_store_commit();
        }
    }
}

// F32: fp32-accurate products on the bf16 tensor-core path. Each fp32 operand arrives as three bf16 planes
// x = x1 + x2 + x3 (8 mantissa bits each, made by split3_kernel); the k-loop runs six times over K, one pass per
// pair (a_i, b_j) with i + j <= 4, smallest terms first, all into the same fp32 accumulator; the three dropped
// pairs are below 2^-24 of the product. The output is stored as fp32 (32-column pieces instead of 64).
constexpr uint32_t kSplitPlaneA = 0x001012, kSplitPlaneB = 0x010210;      // pair p -> plane of A / of B, 4 bits each

// OUT32: the output (and the bias) is fp32; on its own (16-bit operands, one pass) it is the reference's store of an
// accumulator fragment to an f32 buffer, plain or with red.add into a zeroed C (emmyptx/mma.py:205-242).
template <int BN, bool BF16, bool B_NK, bool F32 = false, bool OUT32 = F32>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ OutMaps out, GemmParams p) {
    using S = GemmSmem<BN>;
    constexpr int kStages = S::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t out_smem = smem_base + S::kOutOffset;
    const uint32_t bar_base = smem_base + S::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
    auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + S::kBarOffset + 8 * (2 * kStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* epi_ok = tmem_slot + 2;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.K + kBK - 1) / kBK;
    const int k_total = F32 ? 6 * k_blocks : k_blocks;          // k-blocks the accumulator of one tile receives
    const int plane_tiles = p.m_blocks * p.n_blocks;
    const int tiles = plane_tiles * p.batch;
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int s = 0; s < 2; ++s) { ptx::mbar_init(acc_full_bar(s), 1); ptx::mbar_init(acc_empty_bar(s), 4); }
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&map_a);
        ptx::prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                int mb, nb;
                const int plane = t / plane_tiles;
                tile_coords(t - plane * plane_tiles, p.m_blocks, p.n_blocks, mb, nb);
                const int b_plane = p.b_shared ? 0 : plane;
                for (int kq = 0; kq < k_total; ++kq, ++it) {
                    int kb = kq, a_plane = plane, bb_plane = b_plane;
                    if constexpr (F32) {
                        const int pair = kq / k_blocks;
                        kb = kq - pair * k_blocks;
                        a_plane = plane * 3 + (int)((kSplitPlaneA >> (4 * pair)) & 15u);
                        bb_plane = b_plane * 3 + (int)((kSplitPlaneB >> (4 * pair)) & 15u);
                    }
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = bounded_wait(wctx, empty_bar(s), ph ^ 1, 0x01010000u | s))) break;
                    const uint32_t a_dst = smem_base + s * S::kStageBytes;
                    const uint32_t b_dst = a_dst + S::kABytes;
                    ptx::mbar_arrive_expect_tx(full_bar(s), S::kStageBytes);
                    ptx::tma_load_3d(a_dst, &map_a, full_bar(s), kb * kBK, mb * kBM, a_plane);
                    if constexpr (B_NK) {
                        ptx::tma_load_3d(b_dst, &map_b, full_bar(s), kb * kBK, nb * BN, bb_plane);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            ptx::tma_load_3d(b_dst + j * (kBK * 128), &map_b, full_bar(s), nb * BN + j * 64, kb * kBK, bb_plane);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer -----------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::mma_idesc_f16(BF16, false, !B_NK, kBM, BN);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++acc_it) {
                const int as = acc_it & 1;
                const uint32_t aph = (acc_it >> 1) & 1;
                if (!(ok = bounded_wait(wctx, acc_empty_bar(as), aph ^ 1, 0x01020000u | as))) break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (int kb = 0; kb < k_total; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = bounded_wait(wctx, full_bar(s), ph, 0x01030000u | s))) break;
                    ptx::tc_fence_after_sync();
                    const uint32_t a_src = smem_base + s * S::kStageBytes;
                    const uint32_t b_src = a_src + S::kABytes;
#pragma unroll
                    for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
                        const uint64_t a_desc = ptx::smem_desc_sw128(a_src + kk * (kUmmaK * 2), 16, 1024);
                        const uint64_t b_desc = B_NK ? ptx::smem_desc_sw128(b_src + kk * (kUmmaK * 2), 16, 1024)
                                                     : ptx::smem_desc_sw128(b_src + kk * (kUmmaK * 128), kBK * 128, 1024);
                        ptx::mma_ss(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0);
                    }
                    ptx::mma_commit(empty_bar(s));
                }
                if (ok) ptx::mma_commit(acc_full_bar(as));
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: 4 warps, warp w owns tensor-memory lanes 32 (w % 4) .. +32 -----------------
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const bool issuer = threadIdx.x == 64;                   // first epilogue thread: owns the TMA stores
        uint32_t acc_it = 0, piece = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++acc_it) {
            int mb, nb;
            const int plane = t / plane_tiles;
            tile_coords(t - plane * plane_tiles, p.m_blocks, p.n_blocks, mb, nb);
            const int as = acc_it & 1;
            const uint32_t aph = (acc_it >> 1) & 1;
            // One thread waits; the outcome reaches the four warps through shared memory, so they all
            // take the same path into the named barriers below.
            if (issuer) *epi_ok = bounded_wait(wctx, acc_full_bar(as), aph, 0x01040000u | as) ? 1u : 0u;
            ptx::named_barrier(1, 128);
            ok = *epi_ok != 0;
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN;
            drain_accumulator<BN, BF16, OUT32>(p, out, t_row, out_smem, piece, mb * kBM, nb * BN, plane, row_in_tile, (int)threadIdx.x - 64, issuer,
                                             [&] { if (lane == 0) ptx::mbar_arrive(acc_empty_bar(as)); });
        }
        if (issuer) ptx::tma_store_wait<0>();
        if (p.mc_base != 0) __threadfence_system();
    }

    // ---- teardown -------------------------------------------------------------------------------
    if (*abort_flag) {                          // give copies still in flight time to land
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

// ---- host -----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                       uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(EMMYB200_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EMMYB200_ERR_ARG, "cuTensorMapEncodeTiled (2-D %llu x %llu, ld %llu) failed: %d",
                                       (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, (int)r);
    return EMMYB200_OK;
}

int make_tensor_map_3d(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols) {
    return make_tensor_map_3d_strided(out, base, planes, rows, cols, cols, rows * cols, box_rows, box_cols);
}

int make_tensor_map_3d_strided(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols, uint64_t ld,
                               uint64_t plane_stride, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(EMMYB200_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {cols, rows, planes};
    if (planes == 1) plane_stride = rows * ld;                  // unused, but must be a valid stride
    cuuint64_t strides[2] = {ld * 2, plane_stride * 2};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EMMYB200_ERR_ARG, "cuTensorMapEncodeTiled (3-D) failed: %d", (int)r);
    return EMMYB200_OK;
}

// The fp32 output of the split-precision GEMM: 32-column (128-byte) boxes.
int make_tensor_map_3d_f32(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols, uint64_t ld,
                           uint64_t plane_stride, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(EMMYB200_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {cols, rows, planes};
    if (planes == 1) plane_stride = rows * ld;
    cuuint64_t strides[2] = {ld * 4, plane_stride * 4};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(EMMYB200_ERR_ARG, "cuTensorMapEncodeTiled (3-D fp32) failed: %d", (int)r);
    return EMMYB200_OK;
}

int check_sm100() {
    int dev = 0, major = 0;
    EMMY_CUDA(cudaGetDevice(&dev));
    EMMY_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(EMMYB200_ERR_DEVICE, "device %d has compute capability %d.x; these kernels are sm_100a only", dev, major);
    return EMMYB200_OK;
}

// One CTA whose first thread waits, through the same bounded_wait as every pipeline role, on an mbarrier that nothing
// ever arrives on. The wait runs out after `limit_ns`, records its code and raises the abort flag; the other threads
// see the flag and the kernel returns. This is the give-up path of the real kernels, made to happen on purpose without
// a fault, a trap or an endless loop.
__global__ void __launch_bounds__(64) wait_expiry_kernel(uint32_t* status, unsigned long long limit_ns, uint32_t* saw_abort) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::mbar_fence_init();
    }
    __syncthreads();
    const WaitCtx ctx{&abort_flag, status, limit_ns};
    bool ok = true;
    if (threadIdx.x == 0) ok = bounded_wait(ctx, ptx::smem_u32(&bar), 0, 0x7e570001u);
    __syncthreads();
    if (threadIdx.x == 32 && saw_abort != nullptr) *saw_abort = abort_flag;     // another warp sees the flag, as the other roles do
    (void)ok;
}

__device__ uint32_t g_selftest_saw_abort;

int gemm_peek_status(uint32_t* out) {
    EMMY_CUDA(cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(uint32_t)));
    return EMMYB200_OK;
}

int gemm_read_status(uint32_t* out) {
    uint32_t zero = 0;
    EMMY_CUDA(cudaDeviceSynchronize());
    EMMY_CUDA(cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(uint32_t)));
    if (*out) EMMY_CUDA(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(uint32_t)));
    return EMMYB200_OK;
}

struct GemmCall {
    int dtype, epilogue, flags;
    const void* A; const void* B; const void* bias;
    void* const* C; int n_dst;      // with EMMYB200_GEMM_DST_MULTICAST: C[0] is a multicast address, n_dst = 1
    int64_t batch, M, N, K, lda, ldb, ldc, stride_a, stride_b, stride_c;
    bool b_shared_split = false;    // split-precision path: one B for every product (stride_b then is the split-plane stride)
};

template <int BN, bool BF16, bool B_NK, bool F32 = false, bool OUT32 = F32>
static int launch_gemm(const GemmCall& g, cudaStream_t stream) {
    using S = GemmSmem<BN>;
    CUtensorMap map_a, map_b;
    OutMaps out;
    const bool b_shared = g.stride_b == 0 || g.b_shared_split;
    constexpr uint64_t kSplit = F32 ? 3 : 1;                    // operand planes per product (see split3_kernel)
    int rc = make_tensor_map_3d_strided(&map_a, g.A, (uint64_t)g.batch * kSplit, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda,
                                        (uint64_t)g.stride_a, kBM, kBK);
    if (rc != EMMYB200_OK) return rc;
    const uint64_t b_planes = (b_shared ? 1 : (uint64_t)g.batch) * kSplit;
    rc = B_NK ? make_tensor_map_3d_strided(&map_b, g.B, b_planes, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, (uint64_t)g.stride_b, BN, kBK)
              : make_tensor_map_3d_strided(&map_b, g.B, b_planes, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, (uint64_t)g.stride_b, kBK, 64);
    if (rc != EMMYB200_OK) return rc;
    for (int d = 0; d < kMaxDst; ++d) {
        if (g.flags & EMMYB200_GEMM_DST_MULTICAST) { out.m[d] = map_a; continue; }      // unused: stores go through multimem.st
        rc = OUT32 ? make_tensor_map_3d_f32(&out.m[d], g.C[d < g.n_dst ? d : 0], (uint64_t)g.batch, (uint64_t)g.M, (uint64_t)g.N,
                                          (uint64_t)g.ldc, (uint64_t)g.stride_c, kBM, 32)
                 : make_tensor_map_3d_strided(&out.m[d], g.C[d < g.n_dst ? d : 0], (uint64_t)g.batch, (uint64_t)g.M, (uint64_t)g.N,
                                              (uint64_t)g.ldc, (uint64_t)g.stride_c, kBM, 64);
        if (rc != EMMYB200_OK) return rc;
    }
    auto kernel = gemm_tcgen05_kernel<BN, BF16, B_NK, F32, OUT32>;
    EMMY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    GemmParams p;
    p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
    p.m_blocks = (int)((g.M + kBM - 1) / kBM);
    p.n_blocks = (int)((g.N + BN - 1) / BN);
    p.batch = (int)g.batch;
    p.b_shared = b_shared ? 1 : 0;
    p.n_dst = g.n_dst;
    p.epilogue = g.epilogue;
    p.bias = g.bias;
    const bool multicast = g.flags & EMMYB200_GEMM_DST_MULTICAST;
    p.mc_base = multicast ? (unsigned long long)(uintptr_t)g.C[0] : 0ull;
    p.ldc = g.ldc;
    p.stride_c = g.stride_c;
    p.wait_limit_ns = wait_limit_ns();
    EMMY_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p.status), g_gemm_status));
    const int64_t tiles = (int64_t)p.m_blocks * p.n_blocks * g.batch;
    if (tiles >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "gemm: %lld output tiles exceed the scheduler's range", (long long)tiles);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kernel<<<grid, kGemmThreads, S::kTotal, stream>>>(map_a, map_b, out, p);
    return launch_status("gemm_tcgen05_kernel");
}

template <bool BF16, bool B_NK>
static int pick_tile(const GemmCall& g, cudaStream_t stream) {
    // 128 x 256 tiles: with both operands read from shared memory by one CTA, the 128 x 128 shape is bound by
    // shared-memory bandwidth (measured 0.6-0.7x the throughput at every size from 2048^3 to 16384^3), which
    // costs more than the emptier last wave of the wide tile. Narrow outputs keep the narrow tile.
    if (g.flags & EMMYB200_GEMM_OUT_F32) {
        if (g.N > 128) return launch_gemm<256, BF16, B_NK, false, true>(g, stream);
        return launch_gemm<128, BF16, B_NK, false, true>(g, stream);
    }
    if (g.N > 128) return launch_gemm<256, BF16, B_NK>(g, stream);
    return launch_gemm<128, BF16, B_NK>(g, stream);
}

static int gemm_entry(const GemmCall& g, void* cuda_stream) {
    if (g.dtype != EMMYB200_F16 && g.dtype != EMMYB200_BF16) return fail(EMMYB200_ERR_UNSUPPORTED, "gemm: dtype %d (f16 and bf16 only)", g.dtype);
    if (g.epilogue != EMMYB200_EPI_NONE && g.epilogue != EMMYB200_EPI_GELU_TANH && g.epilogue != EMMYB200_EPI_RELU)
        return fail(EMMYB200_ERR_ARG, "gemm: unknown epilogue %d", g.epilogue);
    if (g.flags & ~(EMMYB200_GEMM_B_NK | EMMYB200_GEMM_DST_MULTICAST | EMMYB200_GEMM_OUT_F32)) return fail(EMMYB200_ERR_ARG, "gemm: unknown flags 0x%x", g.flags);
    const bool out_f32 = g.flags & EMMYB200_GEMM_OUT_F32;
    if (out_f32 && ((g.flags & EMMYB200_GEMM_DST_MULTICAST) || g.n_dst != 1)) return fail(EMMYB200_ERR_UNSUPPORTED, "gemm: an fp32 output has one plain destination");
    if (g.flags & EMMYB200_GEMM_DST_MULTICAST) {
        if (g.n_dst != 1) return fail(EMMYB200_ERR_ARG, "gemm: a multicast destination is a single address");
        if (g.N % 8 != 0) return fail(EMMYB200_ERR_SHAPE, "gemm: multicast stores move 8 columns at a time (N = %lld)", (long long)g.N);
    }
    if (g.n_dst < 1 || g.n_dst > kMaxDst) return fail(EMMYB200_ERR_ARG, "gemm: %d destinations (1 to %d)", g.n_dst, kMaxDst);
    if (g.M < 0 || g.N < 0 || g.K < 0 || g.batch < 0) return fail(EMMYB200_ERR_SHAPE, "gemm: negative extent");
    if (g.M == 0 || g.N == 0 || g.batch == 0) return EMMYB200_OK;
    if (g.K == 0) return fail(EMMYB200_ERR_SHAPE, "gemm: K = 0 (the caller zeroes C, emmyptx/mma.py:77-79 starts accumulators at 0)");
    if (g.M >= (1ll << 31) || g.N >= (1ll << 31) || g.K >= (1ll << 31) || g.batch >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "gemm: extents must be below 2^31");
    if (g.A == nullptr || g.B == nullptr || g.C == nullptr) return fail(EMMYB200_ERR_ARG, "gemm: null buffer");
    for (int d = 0; d < g.n_dst; ++d) {
        if (g.C[d] == nullptr) return fail(EMMYB200_ERR_ARG, "gemm: null output buffer");
        if (!aligned(g.C[d], 16)) return fail(EMMYB200_ERR_ALIGN, "gemm: buffers must be 16-byte aligned");
    }
    const bool b_nk = g.flags & EMMYB200_GEMM_B_NK;
    if (g.lda < g.K || g.ldc < g.N || g.ldb < (b_nk ? g.K : g.N)) return fail(EMMYB200_ERR_SHAPE, "gemm: leading dimension smaller than the row");
    if (((g.lda | g.ldb) & 7) || (g.ldc & (out_f32 ? 3 : 7))) return fail(EMMYB200_ERR_ALIGN, "gemm: leading dimensions must be multiples of 16 bytes (8 16-bit or 4 fp32 elements)");
    if (g.batch > 1) {
        if (((g.stride_a | g.stride_b) & 7) || (g.stride_c & (out_f32 ? 3 : 7))) return fail(EMMYB200_ERR_ALIGN, "gemm: plane strides must be multiples of 8 elements (16 bytes)");
        if (g.stride_a < g.M * g.lda || g.stride_c < g.M * g.ldc || (g.stride_b != 0 && g.stride_b < (b_nk ? g.N : g.K) * g.ldb))
            return fail(EMMYB200_ERR_SHAPE, "gemm: plane stride smaller than a plane");
    }
    if (!aligned(g.A, 16) || !aligned(g.B, 16)) return fail(EMMYB200_ERR_ALIGN, "gemm: buffers must be 16-byte aligned");
    if (g.bias != nullptr && !aligned(g.bias, 16)) return fail(EMMYB200_ERR_ALIGN, "gemm: bias must be 16-byte aligned");
    int rc = check_sm100();
    if (rc != EMMYB200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    const bool bf16 = g.dtype == EMMYB200_BF16;
    if (bf16) return b_nk ? pick_tile<true, true>(g, s) : pick_tile<true, false>(g, s);
    return b_nk ? pick_tile<false, true>(g, s) : pick_tile<false, false>(g, s);
}

// ---- fp32-accurate products: operands split into three bf16 planes --------------------------------------------------
// src: `planes` matrices of rows x cols fp32 (leading dimension ld, plane_stride apart). dst: for every matrix three
// bf16 planes of rows x pitch (pitch a multiple of 8, columns beyond cols zero): x1 = bf16(x), x2 = bf16(x - x1),
// x3 = bf16(x - x1 - x2). A finite x beyond the largest bf16 (3.39e38) takes that value as x1, so the planes stay
// finite; a non-finite x keeps its value in x1 and zeros in x2, x3 (the product passes then meet inf * 0: an
// infinite operand gives NaN where a scalar fp32 loop gives +-inf, which the header states).
__global__ void __launch_bounds__(256) split3_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t planes,
                                                     int64_t rows, int64_t cols, int64_t ld, int64_t plane_stride, int64_t pitch) {
    const int64_t groups_per_row = pitch / 8;
    const int64_t total = planes * rows * groups_per_row;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t c0 = (i % groups_per_row) * 8;
        const int64_t r = (i / groups_per_row) % rows;
        const int64_t pl = i / (groups_per_row * rows);
        const float* in = src + pl * plane_stride + r * ld + c0;
        __align__(16) __nv_bfloat16 h[3][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float x = c0 + j < cols ? __ldg(in + j) : 0.0f;
            __nv_bfloat16 h1 = __float2bfloat16_rn(x);
            float f1 = __bfloat162float(h1);
            if (fabsf(f1) > 3.3895314e38f && fabsf(x) <= 3.4028235e38f) {      // rounded up to inf: clamp to the largest bf16
                f1 = copysignf(3.3895314e38f, x);
                h1 = __float2bfloat16_rn(f1);
            }
            const bool finite = fabsf(f1) <= 3.3895314e38f;
            const float r1 = finite ? x - f1 : 0.0f;
            const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
            const float r2 = r1 - __bfloat162float(h2);
            h[0][j] = h1; h[1][j] = h2; h[2][j] = __float2bfloat16_rn(r2);
        }
#pragma unroll
        for (int sidx = 0; sidx < 3; ++sidx) {
            __nv_bfloat16* out = dst + ((pl * 3 + sidx) * rows + r) * pitch + c0;
            *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(h[sidx]);
        }
    }
}

static int64_t pad8(int64_t v) { return (v + 7) / 8 * 8; }

struct SplitPlan {
    int64_t a_pitch, b_rows, b_cols, b_pitch, b_planes;
    size_t a_bytes, b_bytes;
};

static SplitPlan plan_split3(int flags, int64_t batch, int64_t M, int64_t N, int64_t K, bool b_shared) {
    SplitPlan p;
    const bool b_nk = flags & EMMYB200_GEMM_B_NK;
    p.a_pitch = pad8(K);
    p.b_rows = b_nk ? N : K;
    p.b_cols = b_nk ? K : N;
    p.b_pitch = pad8(p.b_cols);
    p.b_planes = b_shared ? 1 : batch;
    p.a_bytes = ((size_t)batch * 3 * M * p.a_pitch * 2 + 255) / 256 * 256;
    p.b_bytes = ((size_t)p.b_planes * 3 * p.b_rows * p.b_pitch * 2 + 255) / 256 * 256;
    return p;
}

}  // namespace emmy

extern "C" int64_t emmyb200_gemm_f32_workspace_bytes(int flags, int64_t batch, int64_t M, int64_t N, int64_t K, int b_shared) {
    using namespace emmy;
    if ((flags & ~EMMYB200_GEMM_B_NK) || batch < 0 || M < 0 || N < 0 || K < 1) return -1;
    if (batch == 0 || M == 0 || N == 0) return 0;
    const SplitPlan p = plan_split3(flags, batch, M, N, K, b_shared != 0);
    return (int64_t)(p.a_bytes + p.b_bytes);
}

extern "C" int emmyb200_gemm_f32(int epilogue, int flags, const float* A, const float* B, const float* bias, float* C, int64_t batch,
                                 int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t stride_a,
                                 int64_t stride_b, int64_t stride_c, void* workspace, int64_t workspace_bytes, void* cuda_stream) {
    using namespace emmy;
    if (epilogue != EMMYB200_EPI_NONE && epilogue != EMMYB200_EPI_GELU_TANH && epilogue != EMMYB200_EPI_RELU)
        return fail(EMMYB200_ERR_ARG, "gemm_f32: unknown epilogue %d", epilogue);
    if (flags & ~EMMYB200_GEMM_B_NK) return fail(EMMYB200_ERR_ARG, "gemm_f32: unknown flags 0x%x", flags);
    if (M < 0 || N < 0 || K < 0 || batch < 0) return fail(EMMYB200_ERR_SHAPE, "gemm_f32: negative extent");
    if (M == 0 || N == 0 || batch == 0) return EMMYB200_OK;
    if (K == 0) return fail(EMMYB200_ERR_SHAPE, "gemm_f32: K = 0");
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31) || batch * 3 >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "gemm_f32: extents must be below 2^31");
    if (A == nullptr || B == nullptr || C == nullptr) return fail(EMMYB200_ERR_ARG, "gemm_f32: null buffer");
    const bool b_nk = flags & EMMYB200_GEMM_B_NK;
    if (lda < K || ldc < N || ldb < (b_nk ? K : N)) return fail(EMMYB200_ERR_SHAPE, "gemm_f32: leading dimension smaller than the row");
    if (!aligned(A, 4) || !aligned(B, 4) || (bias != nullptr && !aligned(bias, 4))) return fail(EMMYB200_ERR_ALIGN, "gemm_f32: operands must be 4-byte aligned");
    if (!aligned(C, 16) || (ldc & 3) || (batch > 1 && (stride_c & 3)))
        return fail(EMMYB200_ERR_ALIGN, "gemm_f32: C must be 16-byte aligned with a leading dimension (and plane stride) that is a multiple of 4 elements");
    const bool b_shared = stride_b == 0 || batch == 1;
    if (batch > 1 && (stride_a < M * lda || stride_c < M * ldc || (!b_shared && stride_b < (b_nk ? N : K) * ldb)))
        return fail(EMMYB200_ERR_SHAPE, "gemm_f32: plane stride smaller than a plane");
    const SplitPlan sp = plan_split3(flags, batch, M, N, K, b_shared);
    if (workspace == nullptr || workspace_bytes < (int64_t)(sp.a_bytes + sp.b_bytes))
        return fail(EMMYB200_ERR_ARG, "gemm_f32: the split operands need %lld bytes of workspace", (long long)(sp.a_bytes + sp.b_bytes));
    if (!aligned(workspace, 256)) return fail(EMMYB200_ERR_ALIGN, "gemm_f32: the workspace must be 256-byte aligned");
    int rc = check_sm100();
    if (rc != EMMYB200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    __nv_bfloat16* a3 = static_cast<__nv_bfloat16*>(workspace);
    __nv_bfloat16* b3 = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(workspace) + sp.a_bytes);
    const int64_t cap = (int64_t)sm_count() * 16;
    auto blocks = [&](int64_t groups) { const int64_t b = (groups + 255) / 256; return (unsigned)(b < cap ? b : cap); };
    split3_kernel<<<blocks(batch * M * sp.a_pitch / 8), 256, 0, s>>>(A, a3, batch, M, K, lda, stride_a, sp.a_pitch);
    rc = launch_status("split3_kernel");
    if (rc != EMMYB200_OK) return rc;
    split3_kernel<<<blocks(sp.b_planes * sp.b_rows * sp.b_pitch / 8), 256, 0, s>>>(B, b3, sp.b_planes, sp.b_rows, sp.b_cols, ldb, stride_b, sp.b_pitch);
    rc = launch_status("split3_kernel");
    if (rc != EMMYB200_OK) return rc;
    void* dst[1] = {C};
    GemmCall g{EMMYB200_BF16, epilogue, flags, a3, b3, bias, dst, 1, batch, M, N, K, sp.a_pitch, sp.b_pitch, ldc,
               M * sp.a_pitch, sp.b_rows * sp.b_pitch, stride_c};
    g.b_shared_split = b_shared;
    if (N > 128) return b_nk ? launch_gemm<256, true, true, true>(g, s) : launch_gemm<256, true, false, true>(g, s);
    return b_nk ? launch_gemm<128, true, true, true>(g, s) : launch_gemm<128, true, false, true>(g, s);
}

extern "C" int emmyb200_selftest_wait_expiry(uint64_t limit_ns, void* cuda_stream) {
    using namespace emmy;
    if (limit_ns < 1000ull || limit_ns > 1000000000ull) return fail(EMMYB200_ERR_ARG, "selftest_wait_expiry: limit between 1 us and 1 s");
    int rc = check_sm100();
    if (rc != EMMYB200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    uint32_t* status = nullptr;
    uint32_t* saw = nullptr;
    EMMY_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_gemm_status));
    EMMY_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&saw), g_selftest_saw_abort));
    EMMY_CUDA(cudaMemsetAsync(saw, 0, sizeof(uint32_t), s));
    wait_expiry_kernel<<<1, 64, 0, s>>>(status, limit_ns, saw);
    rc = launch_status("wait_expiry_kernel");
    if (rc != EMMYB200_OK) return rc;
    EMMY_CUDA(cudaStreamSynchronize(s));
    uint32_t word = 0, flag = 0;
    rc = gemm_peek_status(&word);
    if (rc != EMMYB200_OK) return rc;
    EMMY_CUDA(cudaMemcpyFromSymbol(&flag, g_selftest_saw_abort, sizeof(uint32_t)));
    if (word == 0 || flag == 0) return fail(EMMYB200_ERR_DEVICE, "selftest_wait_expiry: the wait did not give up (status 0x%08x, abort flag %u)", word, flag);
    return fail(EMMYB200_ERR_TIMEOUT, "a bounded device-side wait expired: status 0x%08x", word);
}

extern "C" int emmyb200_gemm(int dtype, int epilogue, int flags, const void* A, const void* B, void* C, int64_t M,
                             int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, void* cuda_stream) {
    void* dst[1] = {C};
    if (flags & EMMYB200_GEMM_DST_MULTICAST) return emmy::fail(EMMYB200_ERR_ARG, "gemm: the multicast flag belongs to emmyb200_gemm_allgather");
    const emmy::GemmCall g{dtype, epilogue, flags, A, B, nullptr, dst, 1, 1, M, N, K, lda, ldb, ldc, 0, 0, 0};
    return emmy::gemm_entry(g, cuda_stream);
}

extern "C" int emmyb200_gemm_allgather(int dtype, int epilogue, int flags, const void* A, const void* B, void* const* C_dst,
                                       int n_dst, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                       void* cuda_stream) {
    if (C_dst == nullptr) return emmy::fail(EMMYB200_ERR_ARG, "gemm_allgather: null destination list");
    const emmy::GemmCall g{dtype, epilogue, flags, A, B, nullptr, C_dst, n_dst, 1, M, N, K, lda, ldb, ldc, 0, 0, 0};
    return emmy::gemm_entry(g, cuda_stream);
}

extern "C" int emmyb200_gemm_batched(int dtype, int epilogue, int flags, const void* A, const void* B, const void* bias, void* C,
                                     int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                     int64_t stride_a, int64_t stride_b, int64_t stride_c, void* cuda_stream) {
    if (flags & EMMYB200_GEMM_DST_MULTICAST) return emmy::fail(EMMYB200_ERR_ARG, "gemm: the multicast flag belongs to emmyb200_gemm_allgather");
    void* dst[1] = {C};
    const emmy::GemmCall g{dtype, epilogue, flags, A, B, bias, dst, 1, batch, M, N, K, lda, ldb, ldc, stride_a, stride_b, stride_c};
    return emmy::gemm_entry(g, cuda_stream);
}
