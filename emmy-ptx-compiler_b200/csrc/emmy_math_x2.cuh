// Two-at-a-time form of y = exp(x) + sin(x) * tanh(x) for the streaming kernel (device only).
//
// Same algorithms and constants as emmy_math.cuh, evaluated on pairs with the packed fp32 instructions of
// sm_100 (fma / add / mul .f32x2: one issue slot for two elements; each lane rounds exactly like the scalar
// instruction). The caller guarantees |x| <= 86 for both elements, which selects the straight-line path of
// every function: no overflow handling in exp, the three-constant reduction in sin, no NaN. Results are
// bit-identical to the scalar device functions.
#pragma once
#include <cuda_runtime.h>

#include "../../include/emmyb200.h"
#include "emmy_math.cuh"

namespace emmy {

__device__ __forceinline__ float2 f2(float c) { return make_float2(c, c); }
// Packed ops spelled in PTX with an explicit rounding mode: `.rn` forms are never contracted into an fma
// by the assembler, which keeps product-then-sum sequences bit-identical to the scalar code.
__device__ __forceinline__ uint64_t as_u64(float2 v) { return *reinterpret_cast<uint64_t*>(&v); }
__device__ __forceinline__ float2 as_f2(uint64_t v) { return *reinterpret_cast<float2*>(&v); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(as_u64(a)), "l"(as_u64(b)), "l"(as_u64(c)));
    return as_f2(d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(as_u64(a)), "l"(as_u64(b)));
    return as_f2(d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(as_u64(a)), "l"(as_u64(b)));
    return as_f2(d);
}

// exp of both lanes, |x| <= 86: the polynomial on pairs, then 2^n added into each exponent field.
// bits(t) = bits(MAGIC) + n and bits(MAGIC) << 23 == 0 (mod 2^32), so bits(t) << 23 is n << 23.
__device__ __forceinline__ float2 exp_core2(float2 x) {
    const float2 t = fma2(x, f2(EMMY_LOG2E), f2(EMMY_MAGIC));
    const float2 n = add2(t, f2(-EMMY_MAGIC));
    float2 r = fma2(n, f2(-EMMY_LN2_HI), x);
    r = fma2(n, f2(-EMMY_LN2_LO), r);
    float2 q = fma2(f2(EMMY_EXPQ_4), r, f2(EMMY_EXPQ_3));
    q = fma2(q, r, f2(EMMY_EXPQ_2));
    q = fma2(q, r, f2(EMMY_EXPQ_1));
    q = fma2(q, r, f2(EMMY_EXPQ_0));
    const float2 u = fma2(q, r, f2(1.0f));
    const float2 p = fma2(u, r, f2(1.0f));
    float2 e;
    e.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
    e.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
    return e;
}

// tanh of the magnitudes a = |x| (the caller applies the sign, or lets it cancel).
__device__ __forceinline__ float2 tanh_mag2(float2 a) {
    const float2 z = mul2(a, a);
    float2 t = fma2(f2(EMMY_TANHT_4), z, f2(EMMY_TANHT_3));
    t = fma2(t, z, f2(EMMY_TANHT_2));
    t = fma2(t, z, f2(EMMY_TANHT_1));
    t = fma2(t, z, f2(EMMY_TANHT_0));
    const float2 small = fma2(mul2(a, z), t, a);
    const float2 m = make_float2(fminf(a.x, 10.0f), fminf(a.y, 10.0f));
    const float2 e = exp_core2(add2(m, m));
    const float2 d = add2(e, f2(1.0f));
    const float2 rc = make_float2(emmy_rcp(d.x), emmy_rcp(d.y));
    const float2 big = fma2(f2(-2.0f), rc, f2(1.0f));
    return make_float2(a.x < EMMY_TANH_SMALL ? small.x : big.x, a.y < EMMY_TANH_SMALL ? small.y : big.y);
}

__device__ __forceinline__ float2 tanh2(float2 x) {
    const float2 y = tanh_mag2(make_float2(fabsf(x.x), fabsf(x.y)));
    return make_float2(copysignf(y.x, x.x), copysignf(y.y, x.y));
}

__device__ __forceinline__ float sin_select(float s, float c, int q, float x) {
    const float y = (q & 1) ? c : s;
    const float signed_y = __int_as_float(__float_as_int(y) ^ ((q << 30) & 0x80000000));
    return (x == 0.0f) ? x : signed_y;
}

// NONNEG: the caller passes x >= 0 and does not care about the sign of a zero result.
template <bool COS, bool NONNEG = false>
__device__ __forceinline__ float2 sincos2(float2 x) {         // |x| <= 65536
    const float2 t = fma2(x, f2(EMMY_2OPI), f2(EMMY_MAGIC));
    const float2 k = add2(t, f2(-EMMY_MAGIC));
    float2 r = fma2(k, f2(-EMMY_PIO2_1), x);
    r = fma2(k, f2(-EMMY_PIO2_2), r);
    r = fma2(k, f2(-EMMY_PIO2_3), r);
    const float2 z = mul2(r, r);
    float2 sp = fma2(f2(EMMY_SINS_2), z, f2(EMMY_SINS_1));
    sp = fma2(sp, z, f2(EMMY_SINS_0));
    const float2 s = fma2(mul2(r, z), sp, r);
    float2 cp = fma2(f2(EMMY_COSC_2), z, f2(EMMY_COSC_1));
    cp = fma2(cp, z, f2(EMMY_COSC_0));
    cp = fma2(cp, z, f2(-0.5f));
    const float2 c = fma2(cp, z, f2(1.0f));
    if constexpr (COS) {                                      // cos(x) = sin(x + pi/2): one quadrant on
        const int qx = __float_as_int(t.x) + 1, qy = __float_as_int(t.y) + 1;
        return make_float2(sin_select((qx & 1) ? c.x : s.x, 0.0f, qx & ~1, 1.0f), sin_select((qy & 1) ? c.y : s.y, 0.0f, qy & ~1, 1.0f));
    }
    if constexpr (NONNEG) return make_float2(sin_select(s.x, c.x, __float_as_int(t.x), 1.0f), sin_select(s.y, c.y, __float_as_int(t.y), 1.0f));
    return make_float2(sin_select(s.x, c.x, __float_as_int(t.x), x.x), sin_select(s.y, c.y, __float_as_int(t.y), x.y));
}
__device__ __forceinline__ float2 sin2(float2 x) { return sincos2<false>(x); }
__device__ __forceinline__ float2 cos2(float2 x) { return sincos2<true>(x); }

// |tanh| of both lanes from a = |x| and e = e^x, as emmy_tanh_mag_from_exp: the odd polynomial below 0.65, else
// |e^2 - 1| / (e^2 + 1), each a fused multiply-add -- the fused expression's exponential serves tanh too.
__device__ __forceinline__ float2 tanh_mag_from_exp2(float2 a, float2 e) {
    const float2 z = mul2(a, a);
    float2 t = fma2(f2(EMMY_TANHT_4), z, f2(EMMY_TANHT_3));
    t = fma2(t, z, f2(EMMY_TANHT_2));
    t = fma2(t, z, f2(EMMY_TANHT_1));
    t = fma2(t, z, f2(EMMY_TANHT_0));
    const float2 small = fma2(mul2(a, z), t, a);
    const float2 num = fma2(e, e, f2(-1.0f)), den = fma2(e, e, f2(1.0f));
    const float2 big = mul2(make_float2(fabsf(num.x), fabsf(num.y)), make_float2(emmy_rcp(den.x), emmy_rcp(den.y)));
    return make_float2(a.x < EMMY_TANH_SMALL ? small.x : big.x, a.y < EMMY_TANH_SMALL ? small.y : big.y);
}

// exp(x) + sin(x) * tanh(x) on a pair, product and sum rounded separately as in the scalar form. sin and
// tanh are both odd, so their product is taken on |x|: the two sign transfers cancel exactly.
__device__ __forceinline__ float2 exp_sin_tanh2(float2 x) {
    const float2 a = make_float2(fabsf(x.x), fabsf(x.y));
    const float2 s = sincos2<false, true>(a);
    // the exponentials from the special-function unit, step for step as emmy_exp_tanh_mufu
    const float2 tt = mul2(x, f2(EMMY_LOG2E));
    float2 r = fma2(tt, f2(-EMMY_LN2_HI), x);
    r = fma2(tt, f2(-EMMY_LN2_LO), r);
    const float2 p = make_float2(emmy_ex2_approx(tt.x), emmy_ex2_approx(tt.y));
    const float2 pn = make_float2(emmy_ex2_approx(-fabsf(tt.x)), emmy_ex2_approx(-fabsf(tt.y)));
    const float2 e = fma2(p, r, p);
    const float2 en = fma2(pn, make_float2(x.x > 0.0f ? -r.x : r.x, x.y > 0.0f ? -r.y : r.y), pn);
    const float2 nen = make_float2(-en.x, -en.y);
    const float2 num = fma2(nen, en, f2(1.0f)), den = fma2(en, en, f2(1.0f));
    const float2 big = mul2(num, make_float2(emmy_rcp_approx(den.x), emmy_rcp_approx(den.y)));
    const float2 z = mul2(a, a);
    const float2 small = fma2(mul2(a, z), fma2(z, f2(0.13333333f), f2(-0.33333334f)), a);
    const float2 t = make_float2(a.x < EMMY_FUSED_TANH_SERIES ? small.x : big.x, a.y < EMMY_FUSED_TANH_SERIES ? small.y : big.y);
    // scalar product and sum: a packed mul feeding a packed add was observed to be fused into one fma
    return make_float2(__fadd_rn(e.x, __fmul_rn(s.x, t.x)), __fadd_rn(e.y, __fmul_rn(s.y, t.y)));
}

// sigmoid and SiLU of both lanes, |x| <= 86 (bit-identical to emmy_sigmoidf / emmy_siluf there).
__device__ __forceinline__ float2 sigmoid2(float2 x) {
    const float2 e = exp_core2(make_float2(-x.x, -x.y));
    const float2 d = add2(f2(1.0f), e);
    return make_float2(emmy_rcp(d.x), emmy_rcp(d.y));
}
__device__ __forceinline__ float2 silu2(float2 x) {
    const float2 sg = sigmoid2(x);
    return make_float2(__fmul_rn(x.x, sg.x), __fmul_rn(x.y, sg.y));
}
// tanh-form GELU of both lanes, each step rounded as in emmy_gelu_tanhf (scalar products and sums where a packed
// multiply would feed a packed add: the assembler fuses those).
__device__ __forceinline__ float2 gelu_tanh2(float2 x) {
    const float x3x = __fmul_rn(__fmul_rn(x.x, x.x), x.x), x3y = __fmul_rn(__fmul_rn(x.y, x.y), x.y);
    const float ix = __fmul_rn(0.7978845608028654f, __fadd_rn(x.x, __fmul_rn(0.044715f, x3x)));
    const float iy = __fmul_rn(0.7978845608028654f, __fadd_rn(x.y, __fmul_rn(0.044715f, x3y)));
    const float2 t = tanh2(make_float2(ix, iy));
    return make_float2(__fmul_rn(__fmul_rn(0.5f, x.x), __fadd_rn(1.0f, t.x)), __fmul_rn(__fmul_rn(0.5f, x.y), __fadd_rn(1.0f, t.y)));
}

// Largest |x| (of all lanes) for which the packed form of each op is valid; NaN fails every bound.
template <int OP> struct PackedOp { static constexpr bool kHas = false; };
template <> struct PackedOp<EMMYB200_OP_EXP_SIN_TANH> {
    static constexpr bool kHas = true;
    static constexpr float kBound = EMMY_FUSED_MAX;
    static __device__ __forceinline__ float2 apply(float2 x) { return exp_sin_tanh2(x); }
};
template <> struct PackedOp<EMMYB200_OP_EXP> {
    static constexpr bool kHas = true;
    static constexpr float kBound = 86.0f;
    static __device__ __forceinline__ float2 apply(float2 x) { return exp_core2(x); }
};
template <> struct PackedOp<EMMYB200_OP_SIN> {
    static constexpr bool kHas = true;
    static constexpr float kBound = EMMY_TRIG_FAST_MAX;
    static __device__ __forceinline__ float2 apply(float2 x) { return sin2(x); }
};
template <> struct PackedOp<EMMYB200_OP_COS> {
    static constexpr bool kHas = true;
    static constexpr float kBound = EMMY_TRIG_FAST_MAX;
    static __device__ __forceinline__ float2 apply(float2 x) { return cos2(x); }
};
template <> struct PackedOp<EMMYB200_OP_SIGMOID> {
    static constexpr bool kHas = true;
    static constexpr float kBound = 86.0f;
    static __device__ __forceinline__ float2 apply(float2 x) { return sigmoid2(x); }
};
template <> struct PackedOp<EMMYB200_OP_SILU> {
    static constexpr bool kHas = true;
    static constexpr float kBound = 86.0f;
    static __device__ __forceinline__ float2 apply(float2 x) { return silu2(x); }
};
template <> struct PackedOp<EMMYB200_OP_GELU_TANH> {
    static constexpr bool kHas = true;
    static constexpr float kBound = 1.0e12f;           // beyond it x^3 overflows: the scalar function is called
    static __device__ __forceinline__ float2 apply(float2 x) { return gelu_tanh2(x); }
};
template <> struct PackedOp<EMMYB200_OP_TANH> {
    static constexpr bool kHas = true;
    static constexpr float kBound = 3.0e38f;
    static __device__ __forceinline__ float2 apply(float2 x) { return tanh2(x); }
};

}  // namespace emmy
