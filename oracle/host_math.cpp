// Host build of the library's fp32 transcendentals, for the CPU test-suite. TEST INFRASTRUCTURE ONLY.
// The same header the CUDA kernels include, compiled by g++ with contraction off: bit-identical to the device.
#include "../emmy-ptx-compiler_b200/csrc/emmy_math.cuh"

extern "C" void emmy_host_apply(int op, const float* x, float* y, long n) {
    for (long i = 0; i < n; ++i) {
        float v = x[i];
        switch (op) {
            case 0: y[i] = emmy_exp_sin_tanh(v); break;
            case 1: y[i] = emmy_expf(v); break;
            case 2: y[i] = emmy_sinf(v); break;
            case 3: y[i] = emmy_cosf(v); break;
            case 4: y[i] = emmy_tanhf(v); break;
            case 6: y[i] = emmy_sigmoidf(v); break;
            case 7: y[i] = emmy_siluf(v); break;
            case 8: y[i] = emmy_reluf(v); break;
            default: y[i] = emmy_gelu_tanhf(v); break;
        }
    }
}
