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

struct DivConst {      // floor(m / d) for 0 <= m < 2^31 is (m * magic) >> shift
    uint32_t magic;
    int shift;
    int32_t d;
};

static DivConst make_div(int32_t d) {
    int L = 0;
    while ((1ll << L) < d) ++L;
    DivConst c;
    c.shift = 31 + L;
    c.magic = (uint32_t)(((1ull << c.shift) / (uint64_t)d) + 1);
    c.d = d;
    return c;
}

// Floor (torch `//`) or truncating (PTX `div.s32`) division by the positive constant.
template <bool TRUNC>
__device__ __forceinline__ int32_t div_const(int32_t x, DivConst c) {
    if constexpr (TRUNC) {
        if (x == INT32_MIN) return x / c.d;
        uint32_t m = (uint32_t)(x < 0 ? -x : x);
        uint32_t q = (uint32_t)(((uint64_t)m * c.magic) >> c.shift);
        return x < 0 ? -(int32_t)q : (int32_t)q;
    } else {
        uint32_t m = (uint32_t)(x < 0 ? ~x : x);              // floor(x/d) = ~floor(~x/d) for x < 0
        uint32_t q = (uint32_t)(((uint64_t)m * c.magic) >> c.shift);
        return x < 0 ? ~(int32_t)q : (int32_t)q;
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

constexpr int TU = 64, TV = 64, kGatherThreads = 256;

template <bool POW2, bool TRUNC>
__global__ void __launch_bounds__(kGatherThreads) gather_tiled_kernel(GatherParams p) {
    __shared__ int32_t tile[TU][TV + 1];
    const uint32_t vb = blockIdx.x % p.v_blocks, ub = blockIdx.x / p.v_blocks;
    const uint32_t u0 = ub * TU, v0 = vb * TV;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t n = p.n;

    // Read: warp per source run (fixed u), lanes along v.
#pragma unroll 4
    for (int r = warp; r < TU; r += kGatherThreads / 32) {
        const uint32_t u = u0 + r;
        const uint64_t row = (uint64_t)p.mul * u;              // j' of v = 0
#pragma unroll
        for (int c = lane; c < TV; c += 32) {
            const uint32_t v = v0 + c;
            const uint64_t jp = row + v;
            if (u < p.rows && v < p.mul && jp < n) {
                uint64_t j = jp + p.add;
                if (j >= n) j -= n;
                tile[r][c] = __ldg(p.x + j);
            }
        }
    }
    __syncthreads();
    // Write: warp per target run (fixed v), lanes along u.
#pragma unroll 4
    for (int c = warp; c < TV; c += kGatherThreads / 32) {
        const uint32_t v = v0 + c;
        const uint64_t iv = POW2 ? (((uint64_t)p.inv * v) & (n - 1)) : (((uint64_t)p.inv * v) % n);
#pragma unroll
        for (int r = lane; r < TU; r += 32) {
            const uint32_t u = u0 + r;
            const uint64_t jp = (uint64_t)p.mul * u + v;
            if (u < p.rows && v < p.mul && jp < n) {
                uint64_t i = iv + u;
                if (i >= n) i -= n;
                p.y[i] = div_const<TRUNC>(tile[r][c], p.dc) ^ (int32_t)((uint32_t)i >> p.shift);
            }
        }
    }
}

template <bool TRUNC>
__global__ void __launch_bounds__(kGatherThreads) gather_direct_kernel(GatherParams p) {
    const uint64_t n = p.n;
    const uint64_t stride = (uint64_t)gridDim.x * kGatherThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kGatherThreads + threadIdx.x; i < n; i += stride) {
        const uint64_t j = (i * p.mul + p.add) % n;
        p.y[i] = div_const<TRUNC>(__ldg(p.x + j), p.dc) ^ (int32_t)((uint32_t)i >> p.shift);
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
    const bool tiled = p.inv != 0 && p.mul >= TV && p.rows >= TU;
    if (tiled) {
        p.v_blocks = (p.mul + TV - 1) / TV;
        const uint64_t blocks = (uint64_t)p.v_blocks * ((p.rows + TU - 1) / TU);
        if (blocks < (1ull << 31)) {
            const bool pow2 = (n & (n - 1)) == 0;
            auto k = pow2 ? (trunc ? gather_tiled_kernel<true, true> : gather_tiled_kernel<true, false>)
                          : (trunc ? gather_tiled_kernel<false, true> : gather_tiled_kernel<false, false>);
            k<<<(unsigned)blocks, kGatherThreads, 0, s>>>(p);
            return launch_status("gather_tiled_kernel");
        }
    }
    int64_t want = (n + kGatherThreads - 1) / kGatherThreads;
    int64_t cap = (int64_t)sm_count() * 16;
    unsigned blocks = (unsigned)(want > cap ? cap : want);
    if (trunc) gather_direct_kernel<true><<<blocks, kGatherThreads, 0, s>>>(p);
    else gather_direct_kernel<false><<<blocks, kGatherThreads, 0, s>>>(p);
    return launch_status("gather_direct_kernel");
}
