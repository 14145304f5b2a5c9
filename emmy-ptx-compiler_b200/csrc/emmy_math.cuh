// fp32 transcendental functions of the elementwise op table (exp, sin, cos, tanh), written
// once for host and device.
//
// They replace the instruction sequences the reference prints for the same ops
// (emmyptx/ops.py:49-77 `_exp`, :139-148 `_tanh`, :172-180 `_sincos`), with a tighter budget:
// every function here is within 2 ulp of the correctly rounded result over the whole fp32
// range (the reference targets rtol/atol 1e-5, tools/torch_cases/__init__.py:18).
//
// Only IEEE-754 operations are used (fma, add, mul, integer bit moves), and every multiply-add
// that must be fused or must NOT be fused is spelled out, so a host build of this header
// (g++ -ffp-contract=off) gives the same bits as the device build and the accuracy can be
// checked exhaustively on a CPU. The one exception is the reciprocal inside tanh (see emmy_rcp):
// the device form can differ from the host's in the last bit, and is checked exhaustively on
// the device instead.
#pragma once
#include <stdint.h>
#include <math.h>
#include <string.h>

#if defined(__CUDACC__)
#define EMMY_HD __host__ __device__ __forceinline__
#define EMMY_HD_NOINLINE static __host__ __device__ __noinline__
#else
#define EMMY_HD static inline
#define EMMY_HD_NOINLINE static
#endif

// ---- constants (float literals round-trip exactly) --------------------------------------
#define EMMY_MAGIC 12582912.0f             // 1.5 * 2^23: adding it rounds to the nearest integer
#define EMMY_LOG2E 1.442695022e+00f
#define EMMY_LN2_HI 6.931471825e-01f       // ln2 = HI + LO to about 2^-49
#define EMMY_LN2_LO -1.904654212e-09f
#define EMMY_2OPI 6.366197467e-01f
#define EMMY_PIO2_1 1.570796371e+00f       // pi/2 = P1 + P2 + P3 to about 2^-73
#define EMMY_PIO2_2 -4.371138829e-08f
#define EMMY_PIO2_3 -1.715124510e-15f
// exp(r) = 1 + r + r^2 Q(r) on |r| <= ln2/2, weighted minimax, relative error 3.5e-9
#define EMMY_EXPQ_0 4.999999404e-01f
#define EMMY_EXPQ_1 1.666650921e-01f
#define EMMY_EXPQ_2 4.166852683e-02f
#define EMMY_EXPQ_3 8.370134979e-03f
#define EMMY_EXPQ_4 1.381166046e-03f
// sin(r) = r + r^3 S(r^2), cos(r) = 1 - r^2/2 + r^4 C(r^2) on |r| <= pi/4
#define EMMY_SINS_0 -1.666665375e-01f
#define EMMY_SINS_1 8.332112804e-03f
#define EMMY_SINS_2 -1.950873993e-04f
#define EMMY_COSC_0 4.166664556e-02f
#define EMMY_COSC_1 -1.388725126e-03f
#define EMMY_COSC_2 2.442567893e-05f
// tanh(a) = a + a^3 T(a^2) on 0 <= a <= 0.65
#define EMMY_TANH_SMALL 0.65f
#define EMMY_TANHT_0 -3.333325982e-01f
#define EMMY_TANHT_1 1.333083063e-01f
#define EMMY_TANHT_2 -5.368801951e-02f
#define EMMY_TANHT_3 2.046941034e-02f
#define EMMY_TANHT_4 -5.515154451e-03f
// Largest |x| the three-constant reduction of sin/cos is used for; beyond it the full 2/pi
// expansion takes over.
#define EMMY_TRIG_FAST_MAX 65536.0f

// ---- bit moves and unfused arithmetic ----------------------------------------------------
EMMY_HD int32_t emmy_f2i(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_int(f);
#else
    int32_t i; memcpy(&i, &f, 4); return i;
#endif
}
EMMY_HD float emmy_i2f(int32_t i) {
#if defined(__CUDA_ARCH__)
    return __int_as_float(i);
#else
    float f; memcpy(&f, &i, 4); return f;
#endif
}
EMMY_HD float emmy_mul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
EMMY_HD float emmy_add(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}
// 1/a for a in [2, 2^30] (tanh's denominator). Host: the correctly rounded quotient. Device: the hardware
// reciprocal refined by one Newton step, which is the same value except, rarely, in the last bit.
EMMY_HD float emmy_rcp(float a) {
#if defined(__CUDA_ARCH__)
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return fmaf(r, fmaf(-a, r, 1.0f), r);
#else
    return 1.0f / a;
#endif
}

// ---- exp ----------------------------------------------------------------------------------
// x = n ln2 + r, |r| <= ln2/2 (ln2 in two parts, each product fused, so r is exact to about
// 2^-49 n); e^r = 1 + r (1 + r Q(r)).
EMMY_HD float emmy_exp_poly(float x, int32_t* n_out) {
    float t = fmaf(x, EMMY_LOG2E, EMMY_MAGIC);
    float n = emmy_add(t, -EMMY_MAGIC);
    float r = fmaf(n, -EMMY_LN2_HI, x);
    r = fmaf(n, -EMMY_LN2_LO, r);
    float q = EMMY_EXPQ_4;
    q = fmaf(q, r, EMMY_EXPQ_3);
    q = fmaf(q, r, EMMY_EXPQ_2);
    q = fmaf(q, r, EMMY_EXPQ_1);
    q = fmaf(q, r, EMMY_EXPQ_0);
    float u = fmaf(q, r, 1.0f);
    *n_out = emmy_f2i(t) - emmy_f2i(EMMY_MAGIC);
    return fmaf(u, r, 1.0f);
}

// |x| <= 86: the result is a normal number, so 2^n is added straight into the exponent field.
EMMY_HD float emmy_exp_core(float x) {
    int32_t n;
    float p = emmy_exp_poly(x, &n);
    return emmy_i2f(emmy_f2i(p) + (n << 23));
}

// Everything else: NaN passes through, the argument is clamped to where the result saturates
// (e^-104 rounds to 0, e^89 overflows), and 2^n is applied as two exact powers of two, so a
// subnormal result is rounded once.
EMMY_HD_NOINLINE float emmy_exp_edge(float x) {
    if (x != x) return emmy_add(x, x);
    float xc = fminf(fmaxf(x, -104.0f), 89.0f);
    int32_t n;
    float p = emmy_exp_poly(xc, &n);
    int32_t n1 = n >> 1, n2 = n - n1;
    float s1 = emmy_i2f((n1 + 127) << 23), s2 = emmy_i2f((n2 + 127) << 23);
    return emmy_mul(emmy_mul(p, s1), s2);
}

EMMY_HD float emmy_expf(float x) {
    if (fabsf(x) <= 86.0f) return emmy_exp_core(x);
    return emmy_exp_edge(x);
}

// ---- tanh ---------------------------------------------------------------------------------
// Small |x|: odd polynomial (the exponential form cancels there). Otherwise
// tanh(a) = 1 - 2 / (e^{2a} + 1), with a clamped at 10 where the result has long been 1.
EMMY_HD float emmy_tanhf(float x) {
    float a = fabsf(x);
    float z = emmy_mul(a, a);
    float t = EMMY_TANHT_4;
    t = fmaf(t, z, EMMY_TANHT_3);
    t = fmaf(t, z, EMMY_TANHT_2);
    t = fmaf(t, z, EMMY_TANHT_1);
    t = fmaf(t, z, EMMY_TANHT_0);
    float small = fmaf(emmy_mul(a, z), t, a);
    float e = emmy_exp_core(emmy_mul(2.0f, fminf(a, 10.0f)));
    float big = fmaf(-2.0f, emmy_rcp(emmy_add(e, 1.0f)), 1.0f);
    float y = (a < EMMY_TANH_SMALL) ? small : big;
    y = (a != a) ? a : y;                                    // fminf drops a NaN: put it back
    return copysignf(y, x);
}

// ---- sin / cos ----------------------------------------------------------------------------
// The reduced argument r in [-pi/4, pi/4] and the quadrant of x, for |x| beyond the range of
// the three-constant reduction: the product of the 24-bit significand with the 128 bits of
// 2/pi that can still matter (those above contribute multiples of 4 quadrants), as an integer;
// the two bits above the binary point are the quadrant, the next 62 the fraction.
EMMY_HD_NOINLINE float emmy_trig_reduce_large(float x, int32_t* quadrant) {
    const uint32_t two_over_pi[8] = {0xa2f9836eu, 0x4e441529u, 0xfc2757d1u, 0xf534ddc0u,
                                     0xdb629599u, 0x3c439041u, 0xfe5163abu, 0xdebbc561u};
    int32_t bits = emmy_f2i(x) & 0x7fffffff;
    int32_t e = (bits >> 23) - 150;                          // |x| = m * 2^e
    uint64_t m = (uint64_t)((bits & 0x7fffff) | 0x800000);
    int32_t j0 = e >= 2 ? (e - 2) >> 5 : 0;                  // first word of 2/pi that matters
    uint32_t out[5];
    uint64_t carry = 0;
    for (int i = 3; i >= 0; --i) {                           // 128-bit window times m
        uint64_t t = m * two_over_pi[j0 + i] + carry;
        out[3 - i] = (uint32_t)t;
        carry = t >> 32;
    }
    out[4] = (uint32_t)carry;
    int32_t s = e - 32 * (j0 + 4);                           // weight of the product's bit 0
    int32_t pos = -s - 62;                                   // 64 bits from here: quadrant, fraction
    int32_t wi = pos >> 5, sh = pos & 31;
    uint64_t lo = (uint64_t)out[wi] | ((uint64_t)out[wi + 1] << 32);
    uint64_t v = lo >> sh;
    if (sh) v |= (uint64_t)out[wi + 2] << (64 - sh);
    int32_t q = (int32_t)(v >> 62);
    int64_t frac = (int64_t)(v & 0x3fffffffffffffffull);
    if (frac >= (int64_t)1 << 61) { frac -= (int64_t)1 << 62; q += 1; }
    double r = (double)frac * (1.5707963267948966 / 4611686018427387904.0);   // * (pi/2) / 2^62
    if (x < 0.0f) { r = -r; q = -q; }
    *quadrant = q;
    return (float)r;
}

EMMY_HD float emmy_trig_reduce(float x, int32_t* quadrant) {
    if (fabsf(x) <= EMMY_TRIG_FAST_MAX) {
        float t = fmaf(x, EMMY_2OPI, EMMY_MAGIC);
        float k = emmy_add(t, -EMMY_MAGIC);
        float r = fmaf(k, -EMMY_PIO2_1, x);
        r = fmaf(k, -EMMY_PIO2_2, r);
        r = fmaf(k, -EMMY_PIO2_3, r);
        *quadrant = emmy_f2i(t);                             // the low bits are k mod 4
        return r;
    }
    if (!(fabsf(x) < INFINITY)) { *quadrant = 0; return emmy_add(x, -x); }   // inf, NaN -> NaN
    return emmy_trig_reduce_large(x, quadrant);
}

EMMY_HD float emmy_sincos_kernel(float r, int32_t q) {       // sin(r + q pi/2)
    float z = emmy_mul(r, r);
    float sp = fmaf(EMMY_SINS_2, z, EMMY_SINS_1);
    sp = fmaf(sp, z, EMMY_SINS_0);
    float s = fmaf(emmy_mul(r, z), sp, r);
    float cp = fmaf(EMMY_COSC_2, z, EMMY_COSC_1);
    cp = fmaf(cp, z, EMMY_COSC_0);
    cp = fmaf(cp, z, -0.5f);
    float c = fmaf(cp, z, 1.0f);
    float y = (q & 1) ? c : s;
    return (q & 2) ? -y : y;
}

EMMY_HD float emmy_sinf(float x) {
    int32_t q;
    float r = emmy_trig_reduce(x, &q);
    float y = emmy_sincos_kernel(r, q);
    return (x == 0.0f) ? x : y;                              // sin(-0) = -0
}

EMMY_HD float emmy_cosf(float x) {
    int32_t q;
    float r = emmy_trig_reduce(x, &q);
    return emmy_sincos_kernel(r, q + 1);
}

// ---- sigmoid, SiLU, ReLU -------------------------------------------------------------------
// 1 / (1 + e^-x): the exponential above, one add and the refined reciprocal; |x| > 86 is handled apart (1 above,
// e^x below -- where 1 + e^-x would overflow -- and NaN passed through). About 2 ulp; the reference's class for these
// cases is rtol = atol = 1e-5 (tools/torch_cases/pointwise.py:17, 23).
EMMY_HD float emmy_sigmoidf(float x) {
    if (fabsf(x) <= 86.0f) return emmy_rcp(emmy_add(1.0f, emmy_exp_core(-x)));
    if (x != x) return emmy_add(x, x);
    return x > 0.0f ? 1.0f : emmy_expf(x);
}
EMMY_HD float emmy_siluf(float x) { return emmy_mul(x, emmy_sigmoidf(x)); }
EMMY_HD float emmy_reluf(float x) { return x < 0.0f ? 0.0f : x; }       // NaN stays NaN

// ---- GELU, tanh form ------------------------------------------------------------------------
// 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), each step rounded to fp32 in the order torch's
// kernel takes them (the composition the reference's case `p_gelu_tanh` traces,
// tools/torch_cases/pointwise.py:21).
EMMY_HD float emmy_gelu_tanhf(float x) {
    float x3 = emmy_mul(emmy_mul(x, x), x);
    float inner = emmy_mul(0.7978845608028654f, emmy_add(x, emmy_mul(0.044715f, x3)));
    return emmy_mul(emmy_mul(0.5f, x), emmy_add(1.0f, emmy_tanhf(inner)));
}

// ---- the fused expression of the streaming kernel ------------------------------------------
// y = exp(x) + sin(x) * tanh(x): product and sum are rounded separately (torch evaluates the
// three ops one after the other). Inside the fused form the exponential is computed once: with
// E = e^x and w = E^2 = e^{2x}, tanh(|x|) = |w - 1| / (w + 1) for |x| >= 0.65 (the odd polynomial
// below that, as in emmy_tanhf), which saves the second exponential of the stand-alone tanh. w - 1
// and w + 1 are each one fused multiply-add of E with itself; w carries about 2 ulp of relative
// error from E, which the quotient damps by 2w / (w + 1)^2 <= 0.34: the composite stays within the
// <= 5 ulp of its largest term that its tests hold it to (measured over every float with
// 2^-20 <= |x| <= 40: 4.05). sin and tanh are both odd, so the product is taken on |x|.
#define EMMY_FUSED_MAX 40.0f      // beyond it e^{2x} leaves the normal range: the three functions are called as they are
EMMY_HD float emmy_tanh_mag_from_exp(float a, float e) {      // a = |x|, e = e^x (either sign of x)
    float z = emmy_mul(a, a);
    float t = EMMY_TANHT_4;
    t = fmaf(t, z, EMMY_TANHT_3);
    t = fmaf(t, z, EMMY_TANHT_2);
    t = fmaf(t, z, EMMY_TANHT_1);
    t = fmaf(t, z, EMMY_TANHT_0);
    float small = fmaf(emmy_mul(a, z), t, a);
    float big = emmy_mul(fabsf(fmaf(e, e, -1.0f)), emmy_rcp(fmaf(e, e, 1.0f)));
    return (a < EMMY_TANH_SMALL) ? small : big;
}

// On the device the fused form takes its two exponentials from the special-function unit instead of the
// polynomial (which occupies the FP32 pipe this kernel is bound by): with t = fl(x log2 e) and
// r = x - t ln2 (two fused multiply-adds, exact to about 2^-49 t), e^x = 2^t e^r = ex2(t) (1 + r) and
// e^-|x| = ex2(-|t|) (1 -+ r); r is below 2^-18, so the first-order factor is exact to 2^-37. `ex2.approx` is
// good to 2^-22, so E carries up to about 2.5 ulp. tanh(|x|) = (1 - w) / (1 + w) with w = e^{-2|x|} <= 1 -- the
// form whose numerator loses the least (relative error of w times w / (1 - w)) -- with the reciprocal taken
// unrefined, above |x| = 0.125; below it the three-term series a - a^3/3 + 2 a^5/15 (truncation 2e-7 relative
// at the boundary). Both inaccuracies sit where sin(x) tanh(x) ~ x^2 is small against e^x ~ 1, so they vanish
// in the sum: the composite is held to the same bound in ulps of its largest term as before. The host build
// keeps the polynomial form above (no special-function unit there); the two agree to that bound, not bit for bit.
#define EMMY_FUSED_TANH_SERIES 0.125f
#if defined(__CUDACC__)
__device__ __forceinline__ float emmy_ex2_approx(float t) {
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(t));
    return p;
}
__device__ __forceinline__ float emmy_rcp_approx(float a) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}
// (e^x, tanh|x|) for |x| <= EMMY_FUSED_MAX from the quantities above; a = |x|.
__device__ __forceinline__ void emmy_exp_tanh_mufu(float x, float a, float* e_out, float* tanh_out) {
    const float t = emmy_mul(x, EMMY_LOG2E);
    float r = fmaf(t, -EMMY_LN2_HI, x);
    r = fmaf(t, -EMMY_LN2_LO, r);
    const float p = emmy_ex2_approx(t), pn = emmy_ex2_approx(-fabsf(t));
    *e_out = fmaf(p, r, p);
    const float en = fmaf(pn, x > 0.0f ? -r : r, pn);                  // e^-|x|
    const float big = emmy_mul(fmaf(-en, en, 1.0f), emmy_rcp_approx(fmaf(en, en, 1.0f)));
    const float z = emmy_mul(a, a);
    const float small = fmaf(emmy_mul(a, z), fmaf(z, 0.13333333f, -0.33333334f), a);
    *tanh_out = a < EMMY_FUSED_TANH_SERIES ? small : big;
}
#endif

EMMY_HD float emmy_exp_sin_tanh(float x) {
    float a = fabsf(x);
    if (a <= EMMY_FUSED_MAX) {
        int32_t q;
        float r = emmy_trig_reduce(a, &q);
        float s = emmy_sincos_kernel(r, q);
#if defined(__CUDA_ARCH__)
        float e, th;
        emmy_exp_tanh_mufu(x, a, &e, &th);
        return emmy_add(e, emmy_mul(s, th));
#else
        float e = emmy_exp_core(x);
        return emmy_add(e, emmy_mul(s, emmy_tanh_mag_from_exp(a, e)));
#endif
    }
    return emmy_add(emmy_expf(x), emmy_mul(emmy_sinf(x), emmy_tanhf(x)));
}
