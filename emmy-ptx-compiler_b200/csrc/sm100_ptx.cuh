// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels are built from:
// mbarrier, TMA tile loads (cp.async.bulk.tensor, one CTA as the destination), tensor memory
// allocation, tcgen05.mma / commit / ld, and the descriptors they take. No policy lives here.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace emmy {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier -----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One poll. The hardware may hold the thread for up to the hinted time (it returns at once when the phase completes),
// so a waiting warp spends its time suspended rather than spinning through issue slots.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}

// A test without waiting.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA ------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// One box of a 2-D tensor into this CTA's shared memory; completion is counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// One box of shared memory out to a 2-D tensor (elements outside the tensor are dropped); completion is
// tracked per thread in bulk groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most N of this thread's groups are still reading their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------
// Whole-warp calls. `dst_smem` receives the base address (lane 0, column c of the allocation).
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor for 128-byte-swizzled operand tiles (what a TMA box with
// CU_TENSOR_MAP_SWIZZLE_128B writes): start address, leading and stride byte offsets in 16-byte
// units, descriptor version 1 (bits 46-47), layout type 2 = SWIZZLE_128B (bits 61-63).
//   K-major operand  (rows of 64 K-elements): rows 128 B apart, groups of 8 rows `sbo` apart.
//   MN-major operand (rows of 64 M/N-elements, one row per K index): groups of 8 K-rows `sbo`
//   apart, the next 64 M/N-elements `lbo` apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: D format fp32 (bits 4-5 = 1), A and B format
// (bits 7-9, 10-12: 0 = f16, 1 = bf16), A / B major (bits 15, 16: 0 = K-major, 1 = MN-major),
// N >> 3 (bits 17-22), M >> 4 (bits 24-28).
__host__ __device__ constexpr uint32_t mma_idesc_f16(bool bf16, bool a_mn_major, bool b_mn_major, int m, int n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
           ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- MMA ------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// The same with the descriptors given as (low, high) words: the high word of a 128-byte-swizzle descriptor is a
// constant and the low word is the start address / 16 plus constants, so a k-step costs the issuing thread one add.
__device__ __forceinline__ void mma_ss_words(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ts_words(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// High word of smem_desc_sw128 (stride offset, descriptor version, swizzle mode) and its low word for an address.
__host__ __device__ constexpr uint32_t smem_desc_sw128_hi(uint32_t sbo_bytes) { return ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ uint32_t smem_desc_sw128_lo(uint32_t addr, uint32_t lbo_bytes) { return ((addr & 0x3FFFF) >> 4) | (((lbo_bytes >> 4) & 0x3FFF) << 16); }

// The barrier gets one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- tensor memory <-> registers ------------------------------------------------------------
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
// One 16-byte store to a multicast address: the NVSwitch delivers it to the same offset of every GPU bound to the
// multicast object (the storing GPU included). Only multimem.* instructions may touch such an address.
__device__ __forceinline__ void multimem_st_16B(uint64_t mc_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(a)),
                 "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
                 : "memory");
}
__device__ __forceinline__ void ld_shared_16B(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Moves registers between the warps of a CTA: every warp of a warpgroup (four consecutive warps) executes the same one.
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace ptx

// ---- bounded waits ----------------------------------------------------------------------------
// Every pipeline wait in the tensor-core kernels goes through this. It polls the barrier; every
// 256 polls it looks at the CTA's abort flag and at the wall clock, and after `limit_ns` (a launch
// parameter: wait_limit_ns() on the host, 2 s unless emmyb200_set_wait_limit_ns changed it) it
// records `code` in the device status word, raises the abort flag and gives up. Callers leave their
// role loop on `false`, and the kernel then tears down normally (tensor memory is released, nothing
// traps).
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;

struct WaitCtx {
    volatile uint32_t* abort_flag;   // shared memory
    uint32_t* status_word;           // global memory
    uint64_t limit_ns;
};

// The limit the next launches get (host side, process-wide).
uint64_t wait_limit_ns();

// The polling loop behind the immediate test.
__device__ __forceinline__ bool bounded_wait_slow(volatile uint32_t* abort_flag, uint32_t* status_word, uint64_t limit_ns, uint32_t bar,
                                               uint32_t parity, uint32_t code) {
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((spin & 15u) == 0) {
            if (*abort_flag) return false;
            uint64_t now = ptx::global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) {
                atomicCAS(status_word, 0u, code);
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// One immediate test of the barrier (the common case in a running pipeline: the phase has long completed), then the
// polling loop.
__device__ __forceinline__ bool bounded_wait(const WaitCtx& ctx, uint32_t bar, uint32_t parity, uint32_t code) {
    if (ptx::mbar_test_wait(bar, parity)) return true;
    return bounded_wait_slow(ctx.abort_flag, ctx.status_word, ctx.limit_ns, bar, parity, code);
}

// The same for a thread whose wake-up latency matters more than the issue slots its polling takes (a lone MMA-issuing
// thread): it polls without suspending; every 64 polls it looks at the abort flag and the clock. A thread parked in
// try_wait resumes noticeably later than the phase completes: with the issuing thread of the two-tile attention kernel
// polling instead, that kernel gained 9-14 %; for whole warps (softmax, producer) the polling costs more than it saves.
__device__ __forceinline__ bool bounded_spin(const WaitCtx& ctx, uint32_t bar, uint32_t parity, uint32_t code) {
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (ptx::mbar_test_wait(bar, parity)) return true;
        if ((spin & 63u) == 0) {
            if (*ctx.abort_flag) return false;
            uint64_t now = ptx::global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > ctx.limit_ns) {
                atomicCAS(ctx.status_word, 0u, code);
                *ctx.abort_flag = 1;
                return false;
            }
        }
    }
}

// ---- TMA descriptors (host) -------------------------------------------------------------------
// 2-D row-major tensor [rows, cols] of 16-bit elements, row pitch `ld` elements, read in boxes of
// box_rows x box_cols with the 128-byte swizzle; out-of-range elements read as zero.
int make_tensor_map_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                       uint32_t box_rows, uint32_t box_cols);
// 3-D [planes, rows, cols], contiguous, boxes of 1 x box_rows x box_cols.
int make_tensor_map_3d(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols);
// The same with a row pitch `ld` and a plane pitch `plane_stride` (both in elements).
int make_tensor_map_3d_strided(CUtensorMap* out, const void* base, uint64_t planes, uint64_t rows, uint64_t cols, uint64_t ld,
                               uint64_t plane_stride, uint32_t box_rows, uint32_t box_cols);

}  // namespace emmy
