// Library-wide pieces of the C ABI: version, per-thread error text, device queries, and the
// device status word that bounded waits report into.
#include <mutex>

#include "common.cuh"

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
    return EMMYB200_OK;
}
