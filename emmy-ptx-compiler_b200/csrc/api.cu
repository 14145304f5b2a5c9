// Library-wide pieces of the C ABI: version, per-thread error text, device queries, and the
// device status word that bounded waits report into.
#include <atomic>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace emmy {

char* last_error_buffer() {
    static thread_local char buf[512] = "";
    return buf;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static std::atomic<uint64_t> g_wait_limit_ns{kDefaultWaitLimitNs};

uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

// Implemented next to the kernels that own a status word.
int gemm_read_status(uint32_t* out);
int attention_read_status(uint32_t* out);

}  // namespace emmy

extern "C" int emmyb200_version(void) { return 100; }

extern "C" const char* emmyb200_last_error(void) { return emmy::last_error_buffer(); }

extern "C" int emmyb200_device_status(uint32_t* status_out) {
    using namespace emmy;
    if (status_out == nullptr) return fail(EMMYB200_ERR_ARG, "device_status: null output");
    uint32_t a = 0, b = 0;
    int rc = gemm_read_status(&a);
    if (rc != EMMYB200_OK) return rc;
    rc = attention_read_status(&b);
    if (rc != EMMYB200_OK) return rc;
    *status_out = a ? a : b;
    if (*status_out != 0) {
        const uint32_t w = *status_out;
        const char* kernel = (w >> 24) == 1 ? "gemm" : ((w >> 24) == 2 ? "attention" : ((w >> 24) == 0x7e ? "wait self-test" : "unknown"));
        return fail(EMMYB200_ERR_TIMEOUT, "a bounded device-side wait expired: status 0x%08x (%s kernel, wait site %u, stage %u)", w, kernel,
                    (w >> 16) & 0xffu, w & 0xffffu);
    }
    return EMMYB200_OK;
}

extern "C" int emmyb200_set_wait_limit_ns(uint64_t limit_ns) {
    using namespace emmy;
    if (limit_ns == 0) limit_ns = kDefaultWaitLimitNs;
    if (limit_ns < 1000ull || limit_ns > 60000000000ull) return fail(EMMYB200_ERR_ARG, "set_wait_limit_ns: between 1 us and 60 s (0 restores the default of 2 s)");
    g_wait_limit_ns.store(limit_ns, std::memory_order_relaxed);
    return EMMYB200_OK;
}
