// placeholder until the attention kernel lands
#include "common.cuh"
namespace emmy { int attention_read_status(uint32_t* out) { *out = 0; return EMMYB200_OK; } }
extern "C" int emmyb200_attention_fwd(int, const void*, const void*, const void*, void*, int64_t, int64_t, int64_t, int64_t, float, void*) {
    return emmy::fail(EMMYB200_ERR_UNSUPPORTED, "attention_fwd: not built yet");
}
