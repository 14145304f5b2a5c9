// int32 index-math gather: y[i] = (x[(i*mul + add) mod n] div d) xor (i >> shift).
//
// The reference emits this as one thread per output cell: `mul.lo.s32, add, and (n-1)`, a 4-byte
// gathered `ld.global.s32`, `div.s32`, `shr.s32`, `xor`, a 4-byte store (emmyptx/intmath.py:87-117
// for the integer stream, emmyptx/kernel.py:632-677 / :714-733 for the accesses). With mul in the
// thousands every gathered word costs a whole 32-byte DRAM sector.
//
// Tiled kernel. When gcd(mul, n) = 1 the index map is a bijection with inverse
//     i = inv * (j - add) mod n,   inv = mul^-1 mod n.
// Write j' = (j - add) mod n = mul*u + v with 0 <= v < mul (u = j' / mul). Then
//     source  j = (mul*u + v + add) mod n      : consecutive in v for a fixed u,
//     target  i = (u + inv*v) mod n            : consecutive in u for a fixed v.
// So x, seen as rows of `mul` words, is transposed into y, seen as rows that start at
// inv*v mod n: a CTA takes a TU x TV block of (u, v), reads TU runs of TV consecutive source
// words, turns them in shared memory, and writes TV runs of TU consecutive target words.
// Both sides move whole sectors; neighbouring blocks share the ragged sector at a run's end
// through L2. The order in which cells are produced is not observable, so results are
// bit-identical to the one-thread-per-cell form.
//
// Direct kernel. Everything else (gcd != 1, mul too small for runs, tiny n): one cell per
// thread with the exact 64-bit index.
#include "common.cuh"

namespace emmy {

struct DivConst {      // floor(m / d) for 0 <= m < 2^31 is (m * magic) >> (32 + hi_shift); d == 1 is the identity
    uint32_t magic;
    int hi_shift;
    int32_t d;
};

static DivConst make_div(int32_t d) {
    int L = 0;
    while ((1ll << L) < d) ++L;
    DivConst c;
    c.d = d;
    if (d == 1) { c.magic = 0; c.hi_shift = 0; return c; }
    const int shift = 31 + L;                                   // >= 32 for d >= 2
    c.magic = (uint32_t)(((1ull << shift) / (uint64_t)d) + 1);
    c.hi_shift = shift - 32;
    return c;
}

// Floor (torch `//`) or truncating (PTX `div.s32`) division by the positive constant.
// Floor: floor(x/d) = ~floor(~x/d) for x < 0, so the sign is folded in with one xor on each side.
template <bool TRUNC, bool DIV1>
__device__ __forceinline__ int32_t div_const(int32_t x, DivConst c) {
    if constexpr (DIV1) return x;
    if constexpr (TRUNC) {
        if (x == INT32_MIN) return x / c.d;
        const uint32_t m = (uint32_t)(x < 0 ? -x : x);
        const uint32_t q = __umulhi(m, c.magic) >> c.hi_shift;
        return x < 0 ? -(int32_t)q : (int32_t)q;
    } else {
        const int32_t sign = x >> 31;
        const uint32_t q = __umulhi((uint32_t)(x ^ sign), c.magic) >> c.hi_shift;
        return (int32_t)q ^ sign;
    }
}

struct GatherParams {
    const int32_t* x;
    int32_t* y;
    uint32_t n;         // cells
    uint32_t mul;       // reduced mod n
    uint32_t add;       // reduced mod n
    uint32_t inv;       // mul^-1 mod n (tiled kernel only)
    uint32_t rows;      // number of u values: (n - 1) / mul + 1
    uint32_t v_blocks;  // ceil(mul / TV)
    int shift;
    DivConst dc;
};

constexpr int kGatherThreads = 256;
// Block of the (u, v) grid one CTA turns: 128 target-run words by 32 source-run words. Measured best on B200
// among 32..512 x 32..256 (taller blocks lengthen the write runs; narrow ones keep many CTAs in flight).
constexpr int kTileU = 128, kTileV = 32;
constexpr int kMinRun = 128;      // shortest matrix side the tiled kernel is used for

// One CTA per (u-block, v-block), v fastest. All index arithmetic is 32-bit: n < 2^31, so a sum of two
// residues never wraps a uint32.
template <int TU, int TV, int NT, bool POW2, bool TRUNC, bool DIV1>
__global__ void __launch_bounds__(NT) gather_tiled_kernel(GatherParams p) {
    extern __shared__ int32_t tile_raw[];
    int32_t (*tile)[TV + 1] = reinterpret_cast<int32_t (*)[TV + 1]>(tile_raw);
    const uint32_t vb = blockIdx.x % p.v_blocks, ub = blockIdx.x / p.v_blocks;
    const uint32_t u0 = ub * TU, v0 = vb * TV;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n = p.n;
    auto mod_n = [&](uint64_t a) { return POW2 ? (uint32_t)(a & (n - 1)) : (uint32_t)(a % n); };
    const uint32_t rows_here = min((uint32_t)TU, p.rows - u0);      // u0 < rows by construction of the grid
    const uint32_t cols_here = min((uint32_t)TV, p.mul - v0);       // v0 < mul likewise
    const uint64_t last_row = (uint64_t)p.mul * (p.rows - 1);

    // Read: warp per source run (fixed u), lanes along v.
    constexpr int kWarps = NT / 32;
    const bool interior = rows_here == TU && cols_here == TV && u0 + TU < p.rows;
    uint32_t j_base = mod_n((uint64_t)p.mul * (u0 + warp) + v0 + p.add);            // source index of (u0 + warp, v0)
    const uint32_t step = mod_n((uint64_t)p.mul * kWarps);
    if (interior) {
        // Full block away from the matrix's short last row: every load is issued before the first
        // shared-memory store, so a warp keeps TU/8 * TV/32 independent loads in flight.
        int32_t vals[TU / kWarps][TV / 32];
        if constexpr (POW2) {
            // n divides 2^32: the running index may wrap a uint32 freely and is reduced by one mask per load
            const uint32_t j0 = j_base + lane;
#pragma unroll
            for (int k = 0; k < TU / kWarps; ++k)
#pragma unroll
                for (int c = 0; c < TV / 32; ++c) vals[k][c] = __ldg(p.x + ((j0 + (uint32_t)k * step + 32u * c) & (n - 1)));
        } else {
#pragma unroll
            for (int k = 0; k < TU / kWarps; ++k) {
#pragma unroll
                for (int c = 0; c < TV / 32; ++c) {
                    uint32_t j = j_base + lane + 32 * c;
                    if (j >= n) j -= n;
                    vals[k][c] = __ldg(p.x + j);
                }
                j_base += step;
                if (j_base >= n) j_base -= n;
            }
        }
#pragma unroll
        for (int k = 0; k < TU / kWarps; ++k)
#pragma unroll
            for (int c = 0; c < TV / 32; ++c) tile[warp + kWarps * k][lane + 32 * c] = vals[k][c];
    } else {
        // Edge blocks: per-element bounds. The last row of the whole matrix is short.
        for (uint32_t r = warp; r < rows_here; r += kWarps) {
            uint32_t limit = cols_here;
            if (u0 + r == p.rows - 1) limit = min(limit, (uint32_t)(n - last_row > v0 ? n - last_row - v0 : 0));
            for (uint32_t c = lane; c < TV; c += 32) {
                if (c < limit) {
                    uint32_t j = j_base + c;
                    if (j >= n) j -= n;
                    tile[r][c] = __ldg(p.x + j);
                }
            }
            j_base += step;
            if (j_base >= n) j_base -= n;
        }
    }
    __syncthreads();
    // Write: warp per target run (fixed v), lanes along u.
    if (interior) {
#pragma unroll
        for (int k = 0; k < TV / kWarps; ++k) {
            const uint32_t c = warp + kWarps * k;
            uint32_t i_base = mod_n((uint64_t)p.inv * (v0 + c)) + u0 + lane;
#pragma unroll
            for (int r = 0; r < TU / 32; ++r) {
                uint32_t i = i_base + 32 * r;
                if constexpr (POW2) i &= n - 1;
                else if (i >= n) i -= n;
                p.y[i] = div_const<TRUNC, DIV1>(tile[lane + 32 * r][c], p.dc) ^ (int32_t)(i >> p.shift);
            }
        }
        return;
    }
    for (uint32_t c = warp; c < cols_here; c += kWarps) {
        const uint32_t v = v0 + c;
        uint32_t i_base = mod_n((uint64_t)p.inv * v) + u0;
        if (i_base >= n) i_base -= n;
        // rows of this column: all of them, except that the matrix's last row may end before v
        uint32_t limit = rows_here;
        if (u0 + rows_here == p.rows && last_row + v >= n) limit -= 1;
        for (uint32_t r = lane; r < TU; r += 32) {
            if (r < limit) {
                uint32_t i = i_base + r;
                if (i >= n) i -= n;
                p.y[i] = div_const<TRUNC, DIV1>(tile[r][c], p.dc) ^ (int32_t)(i >> p.shift);
            }
        }
    }
}

template <int TU, int TV, int NT = kGatherThreads>
static int launch_tiled(GatherParams p, bool pow2, bool trunc, cudaStream_t s) {
    p.v_blocks = (p.mul + TV - 1) / TV;
    const uint64_t blocks = (uint64_t)p.v_blocks * ((p.rows + TU - 1) / TU);
    if (blocks >= (1ull << 31)) return -1;
    void (*k)(GatherParams);
    if (p.dc.d == 1) k = pow2 ? gather_tiled_kernel<TU, TV, NT, true, false, true> : gather_tiled_kernel<TU, TV, NT, false, false, true>;
    else k = pow2 ? (trunc ? gather_tiled_kernel<TU, TV, NT, true, true, false> : gather_tiled_kernel<TU, TV, NT, true, false, false>)
                  : (trunc ? gather_tiled_kernel<TU, TV, NT, false, true, false> : gather_tiled_kernel<TU, TV, NT, false, false, false>);
    const int smem = TU * (TV + 1) * 4;
    EMMY_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    k<<<(unsigned)blocks, NT, smem, s>>>(p);
    return launch_status("gather_tiled_kernel");
}

template <bool TRUNC>
__global__ void __launch_bounds__(kGatherThreads) gather_direct_kernel(GatherParams p) {
    const uint64_t n = p.n;
    const uint64_t stride = (uint64_t)gridDim.x * kGatherThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kGatherThreads + threadIdx.x; i < n; i += stride) {
        const uint64_t j = (i * p.mul + p.add) % n;
        const int32_t g = __ldg(p.x + j);
        p.y[i] = (p.dc.d == 1 ? g : div_const<TRUNC, false>(g, p.dc)) ^ (int32_t)((uint32_t)i >> p.shift);
    }
}

// mul^-1 mod n by the extended Euclidean algorithm; 0 when gcd(mul, n) != 1.
static uint32_t mod_inverse(uint64_t a, uint64_t n) {
    int64_t t = 0, nt = 1;
    int64_t r = (int64_t)n, nr = (int64_t)(a % n);
    while (nr != 0) {
        int64_t q = r / nr;
        int64_t tmp = t - q * nt; t = nt; nt = tmp;
        tmp = r - q * nr; r = nr; nr = tmp;
    }
    if (r != 1) return 0;
    if (t < 0) t += (int64_t)n;
    return (uint32_t)t;
}

}  // namespace emmy

extern "C" int emmyb200_index_gather_i32(const int32_t* x, int32_t* y, int64_t n, int64_t mul, int64_t add,
                                         int32_t d, int32_t shift, int32_t flags, void* cuda_stream) {
    using namespace emmy;
    if (n == 0) return EMMYB200_OK;
    if (n < 0 || n >= (1ll << 31)) return fail(EMMYB200_ERR_SHAPE, "index_gather: n = %lld outside [0, 2^31)", (long long)n);
    if (x == nullptr || y == nullptr) return fail(EMMYB200_ERR_ARG, "index_gather: null buffer");
    if (mul < 0 || add < 0) return fail(EMMYB200_ERR_ARG, "index_gather: mul and add must be non-negative");
    if (d < 1) return fail(EMMYB200_ERR_ARG, "index_gather: divisor %d must be >= 1", d);
    if (shift < 0 || shift > 31) return fail(EMMYB200_ERR_ARG, "index_gather: shift %d outside [0, 31]", shift);
    if (flags & ~EMMYB200_GATHER_TRUNC) return fail(EMMYB200_ERR_ARG, "index_gather: unknown flags 0x%x", flags);
    if (!aligned(x, 4) || !aligned(y, 4)) return fail(EMMYB200_ERR_ALIGN, "index_gather: buffers must be 4-byte aligned");
    {
        const char* xb = (const char*)x; const char* yb = (const char*)y;
        if (xb < yb + n * 4 && yb < xb + n * 4) return fail(EMMYB200_ERR_ARG, "index_gather: x and y overlap");
    }
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    GatherParams p;
    p.x = x; p.y = y; p.n = (uint32_t)n;
    p.mul = (uint32_t)(mul % n); p.add = (uint32_t)(add % n);
    p.shift = shift; p.dc = make_div(d);
    const bool trunc = flags & EMMYB200_GATHER_TRUNC;
    p.inv = p.mul ? mod_inverse(p.mul, (uint64_t)n) : 0;
    p.rows = p.mul ? (uint32_t)((n - 1) / p.mul + 1) : 0;
    const bool tiled = p.inv != 0 && p.mul >= kMinRun && p.rows >= kMinRun;
    if (tiled) {
        const bool pow2 = (n & (n - 1)) == 0;
        const int rc = launch_tiled<kTileU, kTileV>(p, pow2, trunc, s);
        if (rc != -1) return rc;
    }
    int64_t want = (n + kGatherThreads - 1) / kGatherThreads;
    int64_t cap = (int64_t)sm_count() * 16;
    unsigned blocks = (unsigned)(want > cap ? cap : want);
    if (trunc) gather_direct_kernel<true><<<blocks, kGatherThreads, 0, s>>>(p);
    else gather_direct_kernel<false><<<blocks, kGatherThreads, 0, s>>>(p);
    return launch_status("gather_direct_kernel");
}
