// Elementwise programs compiled at first use: the cell program of a one-axis `Tile` becomes the body of a
// kernel specialised to it, as the reference prints the instructions of each `Assign` into the kernel it is
// compiling (emmyptx/kernel.py:766-784, emmyptx/ops.py:212-290).
//
// The program (include/emmyb200.h, emmyb200_pw_program) is turned into CUDA C++ text: one straight-line
// `cell()` function over named registers, inside a fixed streaming shell (128-bit accesses, two vectors in
// flight per thread, grid capped at a multiple of the SM count). The text is compiled for sm_100a by NVRTC,
// loaded through the runtime's library interface, and cached under the program's shape: op sequence, operand
// wiring, dtypes, how each input is broadcast and which vector accesses the buffers allow. Constants and
// broadcast extents are kernel arguments, so changing a scalar parameter does not compile again.
//
// Every op is spelled exactly as in the interpreter of pointwise_program.cu (explicit round-to-nearest
// intrinsics, the functions of emmy_math.cuh, which travels inside this library as text), so the two forms give
// the same bits (the sign and payload of a NaN aside); the interpreters remain the form used when NVRTC cannot be
// loaded. Integer programs (32-bit two's complement values in i32 / i64 buffers) are compiled the same way.
#include <ctype.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "pointwise_jit.h"

namespace emmy {

static const char kMathHeader[] =
#include "emmy_math_text.inc"
    ;

static const char kStdintStub[] =
    "#pragma once\n"
    "typedef signed char int8_t; typedef unsigned char uint8_t; typedef short int16_t; typedef unsigned short uint16_t;\n"
    "typedef int int32_t; typedef unsigned int uint32_t; typedef long long int64_t; typedef unsigned long long uint64_t;\n";
static const char kEmptyStub[] = "#pragma once\n";
static const char kMathStub[] = "#pragma once\n#ifndef INFINITY\n#define INFINITY (__int_as_float(0x7f800000))\n#endif\n";

// ---- NVRTC, looked up at run time so that the library loads where the compiler is not installed ------------
struct Nvrtc {
    void* handle = nullptr;
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
    const char* (*GetErrorString)(nvrtcResult) = nullptr;
    bool ok = false;
};

static const Nvrtc& nvrtc() {
    static Nvrtc n = [] {
        Nvrtc r;
        const char* env = getenv("EMMYB200_NVRTC");
        // the toolkit this library was built with first, so that logf / erff / powf are the same device functions
        const char* names[] = {env, "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.12", "libnvrtc.so"};
        for (const char* name : names) {
            if (name == nullptr || *name == 0) continue;
            r.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (r.handle != nullptr) break;
        }
        if (r.handle == nullptr) return r;
        auto sym = [&](const char* s) { return dlsym(r.handle, s); };
        r.CreateProgram = reinterpret_cast<decltype(r.CreateProgram)>(sym("nvrtcCreateProgram"));
        r.CompileProgram = reinterpret_cast<decltype(r.CompileProgram)>(sym("nvrtcCompileProgram"));
        r.GetCUBINSize = reinterpret_cast<decltype(r.GetCUBINSize)>(sym("nvrtcGetCUBINSize"));
        r.GetCUBIN = reinterpret_cast<decltype(r.GetCUBIN)>(sym("nvrtcGetCUBIN"));
        r.GetProgramLogSize = reinterpret_cast<decltype(r.GetProgramLogSize)>(sym("nvrtcGetProgramLogSize"));
        r.GetProgramLog = reinterpret_cast<decltype(r.GetProgramLog)>(sym("nvrtcGetProgramLog"));
        r.DestroyProgram = reinterpret_cast<decltype(r.DestroyProgram)>(sym("nvrtcDestroyProgram"));
        r.GetErrorString = reinterpret_cast<decltype(r.GetErrorString)>(sym("nvrtcGetErrorString"));
        r.ok = r.CreateProgram && r.CompileProgram && r.GetCUBINSize && r.GetCUBIN && r.GetProgramLogSize &&
               r.GetProgramLog && r.DestroyProgram && r.GetErrorString;
        return r;
    }();
    return n;
}

static std::atomic<int> g_jit_enabled{-1};        // -1: not decided yet (the environment is read once)

static bool jit_enabled() {
    int v = g_jit_enabled.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* env = getenv("EMMYB200_PW_JIT");
        v = (env != nullptr && env[0] == '0') ? 0 : 1;
        g_jit_enabled.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

// ---- program -> CUDA C++ -----------------------------------------------------------------------------------
// One expression per op, written with the same intrinsics as the interpreter's pw_apply() so that the two forms
// agree bit for bit. A, B, C stand for the operands.
static const char* op_expr(int op) {
    switch (op) {
        case EMMYB200_PW_ADD: return "__fadd_rn(A, B)";
        case EMMYB200_PW_SUB: return "__fsub_rn(A, B)";
        case EMMYB200_PW_MUL: return "__fmul_rn(A, B)";
        case EMMYB200_PW_DIV: return "__fdiv_rn(A, B)";
        case EMMYB200_PW_MAX: return "fmaxf(A, B)";
        case EMMYB200_PW_MIN: return "fminf(A, B)";
        case EMMYB200_PW_RELU: return "fmaxf(A, 0.0f)";
        case EMMYB200_PW_SQUARE: return "__fmul_rn(A, A)";
        case EMMYB200_PW_COPY: return "A";
        case EMMYB200_PW_NEG: return "(-A)";
        case EMMYB200_PW_ABS: return "fabsf(A)";
        case EMMYB200_PW_RCP: return "__frcp_rn(A)";
        case EMMYB200_PW_SQRT: return "__fsqrt_rn(A)";
        case EMMYB200_PW_RSQRT: return "__frcp_rn(__fsqrt_rn(A))";
        case EMMYB200_PW_EXP: return "emmy_expf(A)";
        case EMMYB200_PW_LOG: return "logf(A)";
        case EMMYB200_PW_SIGMOID: return "__frcp_rn(__fadd_rn(1.0f, emmy_expf(-A)))";
        case EMMYB200_PW_TANH: return "emmy_tanhf(A)";
        case EMMYB200_PW_ERF: return "erff(A)";
        case EMMYB200_PW_SIN: return "emmy_sinf(A)";
        case EMMYB200_PW_COS: return "emmy_cosf(A)";
        case EMMYB200_PW_POW: return "powf(A, B)";
        case EMMYB200_PW_EQ: return "(A == B ? 1.0f : 0.0f)";
        case EMMYB200_PW_NE: return "(A != B ? 1.0f : 0.0f)";
        case EMMYB200_PW_GT: return "(A > B ? 1.0f : 0.0f)";
        case EMMYB200_PW_LT: return "(A < B ? 1.0f : 0.0f)";
        case EMMYB200_PW_GE: return "(A >= B ? 1.0f : 0.0f)";
        case EMMYB200_PW_LE: return "(A <= B ? 1.0f : 0.0f)";
        case EMMYB200_PW_WHERE: return "(A != 0.0f ? B : C)";
        case EMMYB200_PW_AND: return "((A != 0.0f && B != 0.0f) ? 1.0f : 0.0f)";
        case EMMYB200_PW_OR: return "((A != 0.0f || B != 0.0f) ? 1.0f : 0.0f)";
        case EMMYB200_PW_NOT: return "(A == 0.0f ? 1.0f : 0.0f)";
        case EMMYB200_PW_FLOORDIV: return "floorf(__fdiv_rn(A, B))";
        case EMMYB200_PW_MOD: return "__fsub_rn(A, __fmul_rn(B, floorf(__fdiv_rn(A, B))))";
        default: return "A";
    }
}

static const char* op_expr_int(int op) {
    switch (op) {
        case EMMYB200_PW_ADD: return "(int)((unsigned)A + (unsigned)B)";
        case EMMYB200_PW_SUB: return "(int)((unsigned)A - (unsigned)B)";
        case EMMYB200_PW_MUL: return "(int)((unsigned)A * (unsigned)B)";
        case EMMYB200_PW_MAX: return "max(A, B)";
        case EMMYB200_PW_MIN: return "min(A, B)";
        case EMMYB200_PW_RELU: return "max(A, 0)";
        case EMMYB200_PW_SQUARE: return "(int)((unsigned)A * (unsigned)A)";
        case EMMYB200_PW_NEG: return "(int)(0u - (unsigned)A)";
        case EMMYB200_PW_ABS: return "(A < 0 ? (int)(0u - (unsigned)A) : A)";
        case EMMYB200_PW_EQ: return "(int)(A == B)";
        case EMMYB200_PW_NE: return "(int)(A != B)";
        case EMMYB200_PW_GT: return "(int)(A > B)";
        case EMMYB200_PW_LT: return "(int)(A < B)";
        case EMMYB200_PW_GE: return "(int)(A >= B)";
        case EMMYB200_PW_LE: return "(int)(A <= B)";
        case EMMYB200_PW_WHERE: return "(A != 0 ? B : C)";
        case EMMYB200_PW_AND: return "(A & B)";
        case EMMYB200_PW_OR: return "(A | B)";
        case EMMYB200_PW_NOT: return "(~A)";
        case EMMYB200_PW_XOR: return "(A ^ B)";
        case EMMYB200_PW_SHL: return "(int)((unsigned)A << ((unsigned)B & 31u))";
        case EMMYB200_PW_SHR: return "(A >> ((unsigned)B & 31u))";
        case EMMYB200_PW_DIV:
        case EMMYB200_PW_FLOORDIV: return "pw_i_div(A, B, T)";
        case EMMYB200_PW_MOD: return "pw_i_mod(A, B, T)";
        default: return "A";                                    // COPY, and ops the s32 table does not have
    }
}

static std::string operand_text(int o, bool ints) {
    char buf[24];
    if (o >= EMMYB200_PW_MAX_SLOTS) snprintf(buf, sizeof buf, ints ? "(int)c.v[%d]" : "c.v[%d]", o - EMMYB200_PW_MAX_SLOTS);
    else snprintf(buf, sizeof buf, "s%d", o);
    return buf;
}

static std::string expand(const char* pattern, const emmyb200_pw_step& st, bool ints) {
    std::string out;
    for (const char* p = pattern; *p; ++p) {
        // an operand letter (or T, the step's rounding flag) stands alone: no op spelling has such an identifier
        const bool alone = (p == pattern || !(isalnum((unsigned char)p[-1]) || p[-1] == '_')) && !(isalnum((unsigned char)p[1]) || p[1] == '_');
        if (alone && *p == 'A') out += operand_text(st.a, ints);
        else if (alone && *p == 'B') out += operand_text(st.b, ints);
        else if (alone && *p == 'C') out += operand_text(st.c, ints);
        else if (alone && *p == 'T') out += st.reserved[0] ? "1" : "0";
        else out += *p;
    }
    return out;
}

// The fixed part of every generated kernel. PW_N_IN, PW_VEC, PW_G, PW_DT0..3, PW_BC0..3 and PW_OUT_DT are defined
// in front of it; dtype codes are those of include/emmyb200.h (0 f32, 1 f16, 2 bf16, 5 u8).
static const char kIntOps[] = R"SHELL(// 32-bit two's complement ops of integer programs (the s32 table, emmyptx/ops.py:294-309): wrap-around arithmetic,
// `//` and `%` toward minus infinity unless T is 1 (toward zero, the reference's div.s32 / rem.s32).
__device__ __forceinline__ int pw_i_div(int a, int b, int trunc) {
    if (b == 0) return 0;
    if (b == -1) return (int)(0u - (unsigned)a);                 // INT_MIN / -1 wraps
    int q = a / b;
    if (!trunc && (a % b != 0) && ((a < 0) != (b < 0))) --q;
    return q;
}
__device__ __forceinline__ int pw_i_mod(int a, int b, int trunc) {
    if (b == 0 || b == -1) return 0;
    int r = a % b;
    if (!trunc && r != 0 && ((r < 0) != (b < 0))) r += b;
    return r;
}
)SHELL";

// Loads of the float programs: values are fp32, 16-bit buffers are widened, byte buffers are 0 / 1.
static const char kFloatLoads[] = R"SHELL(
// PW_G elements per thread and access group: 4 (128-bit accesses of fp32), or 8 when a 16-bit or byte buffer takes
// part (128-bit accesses of those; two per group for an fp32 buffer). PW_VEC 0: scalar accesses, groups of 4.
template <int DT> __device__ __forceinline__ float pw_ld1(const void* p, i64 i) {
    if (DT == 0) return reinterpret_cast<const float*>(p)[i];
    if (DT == 5) return reinterpret_cast<const unsigned char*>(p)[i] ? 1.0f : 0.0f;
    const unsigned short h = reinterpret_cast<const unsigned short*>(p)[i];
    if (DT == 1) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
    return __uint_as_float((unsigned)h << 16);
}
__device__ __forceinline__ float pw_half_lo(unsigned w) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((unsigned short)(w & 0xffffu))); return f; }
__device__ __forceinline__ float pw_half_hi(unsigned w) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((unsigned short)(w >> 16))); return f; }
template <int DT> __device__ __forceinline__ PwVec pw_ldv(const void* p, i64 g) {
    PwVec r;
    if (DT == 0) {
#pragma unroll
        for (int q = 0; q < PW_G / 4; ++q) {
            const float4 t = __ldcs(reinterpret_cast<const float4*>(p) + g * (PW_G / 4) + q);
            r.v[4 * q] = t.x; r.v[4 * q + 1] = t.y; r.v[4 * q + 2] = t.z; r.v[4 * q + 3] = t.w;
        }
    } else if (DT == 5) {
        unsigned w[PW_G / 4];
#if PW_G == 4
        w[0] = __ldcs(reinterpret_cast<const unsigned*>(p) + g);
#else
        const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p) + g);
        w[0] = raw.x; w[1] = raw.y;
#endif
#pragma unroll
        for (int k = 0; k < PW_G; ++k) r.v[k] = ((w[k / 4] >> (8 * (k % 4))) & 0xffu) ? 1.0f : 0.0f;
    } else {
        unsigned w[PW_G / 2];
#if PW_G == 4
        const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p) + g);
        w[0] = raw.x; w[1] = raw.y;
#else
        const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p) + g);
        w[0] = raw.x; w[1] = raw.y; w[2] = raw.z; w[3] = raw.w;
#endif
#pragma unroll
        for (int q = 0; q < PW_G / 2; ++q) {
            if (DT == 1) { r.v[2 * q] = pw_half_lo(w[q]); r.v[2 * q + 1] = pw_half_hi(w[q]); }
            else { r.v[2 * q] = __uint_as_float(w[q] << 16); r.v[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u); }
        }
    }
    return r;
}
)SHELL";

static const char kFloatStores[] = R"SHELL(
__device__ __forceinline__ void pw_st1(void* p, i64 i, float v) {
#if PW_OUT_DT == 0
    reinterpret_cast<float*>(p)[i] = v;
#elif PW_OUT_DT == 1
    unsigned short h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(v)); reinterpret_cast<unsigned short*>(p)[i] = h;
#elif PW_OUT_DT == 5
    reinterpret_cast<unsigned char*>(p)[i] = v != 0.0f ? 1 : 0;          // a bool output: 1 where the value is non-zero
#else
    unsigned short h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(v)); reinterpret_cast<unsigned short*>(p)[i] = h;
#endif
}
__device__ __forceinline__ unsigned pw_pack4b(float a, float b, float c, float d) {     // four bool bytes
    return (a != 0.0f ? 1u : 0u) | (b != 0.0f ? 0x100u : 0u) | (c != 0.0f ? 0x10000u : 0u) | (d != 0.0f ? 0x1000000u : 0u);
}
__device__ __forceinline__ unsigned pw_pack2(float lo, float hi) {      // two values rounded to the 16-bit output type
    unsigned w;
#if PW_OUT_DT == 1
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
#else
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
#endif
    return w;
}
__device__ __forceinline__ void pw_stv(void* p, i64 g, const PwVec& y) {       // group g of PW_G elements, aligned
#if PW_OUT_DT == 0
#pragma unroll
    for (int q = 0; q < PW_G / 4; ++q)
        __stcs(reinterpret_cast<float4*>(p) + g * (PW_G / 4) + q, make_float4(y.v[4 * q], y.v[4 * q + 1], y.v[4 * q + 2], y.v[4 * q + 3]));
#elif PW_OUT_DT == 5 && PW_G == 4
    __stcs(reinterpret_cast<unsigned*>(p) + g, pw_pack4b(y.v[0], y.v[1], y.v[2], y.v[3]));
#elif PW_OUT_DT == 5
    __stcs(reinterpret_cast<uint2*>(p) + g, make_uint2(pw_pack4b(y.v[0], y.v[1], y.v[2], y.v[3]), pw_pack4b(y.v[4], y.v[5], y.v[6], y.v[7])));
#elif PW_G == 4
    __stcs(reinterpret_cast<uint2*>(p) + g, make_uint2(pw_pack2(y.v[0], y.v[1]), pw_pack2(y.v[2], y.v[3])));
#else
    __stcs(reinterpret_cast<uint4*>(p) + g, make_uint4(pw_pack2(y.v[0], y.v[1]), pw_pack2(y.v[2], y.v[3]), pw_pack2(y.v[4], y.v[5]), pw_pack2(y.v[6], y.v[7])));
#endif
}
__device__ __forceinline__ void pw_out(void* p, i64 g, i64 n, const PwVec& y) {
#if PW_VEC
    pw_stv(p, g, y);
#else
    const i64 i = g * PW_G;
#pragma unroll
    for (int k = 0; k < PW_G; ++k)
        if (i + k < n) pw_st1(p, i + k, y.v[k]);
#endif
}

)SHELL";

static const char kIntLoads[] = R"SHELL(
template <int DT> __device__ __forceinline__ int pw_ld1(const void* p, i64 i) {
    if (DT == 3) return reinterpret_cast<const int*>(p)[i];
    return (int)reinterpret_cast<const long long*>(p)[i];              // 64-bit buffers hold 32-bit values (emmyptx/kernel.py:41)
}
template <int DT> __device__ __forceinline__ PwVec pw_ldv(const void* p, i64 g) {      // PW_G is 4 for integer programs
    PwVec r;
    if (DT == 3) {
        const int4 t = __ldcs(reinterpret_cast<const int4*>(p) + g);
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const longlong2 t = __ldcs(reinterpret_cast<const longlong2*>(p) + g * 2 + q);
            r.v[2 * q] = (int)t.x; r.v[2 * q + 1] = (int)t.y;
        }
    }
    return r;
}
)SHELL";

static const char kIntStores[] = R"SHELL(
__device__ __forceinline__ void pw_st1(void* p, i64 i, int v) {
#if PW_OUT_DT == 3
    reinterpret_cast<int*>(p)[i] = v;
#else
    reinterpret_cast<long long*>(p)[i] = (long long)v;
#endif
}
__device__ __forceinline__ void pw_stv(void* p, i64 g, const PwVec& y) {
#if PW_OUT_DT == 3
    __stcs(reinterpret_cast<int4*>(p) + g, make_int4(y.v[0], y.v[1], y.v[2], y.v[3]));
#else
    __stcs(reinterpret_cast<longlong2*>(p) + g * 2, make_longlong2((long long)y.v[0], (long long)y.v[1]));
    __stcs(reinterpret_cast<longlong2*>(p) + g * 2 + 1, make_longlong2((long long)y.v[2], (long long)y.v[3]));
#endif
}
__device__ __forceinline__ void pw_out(void* p, i64 g, i64 n, const PwVec& y) {
#if PW_VEC
    pw_stv(p, g, y);
#else
    const i64 i = g * PW_G;
#pragma unroll
    for (int k = 0; k < PW_G; ++k)
        if (i + k < n) pw_st1(p, i + k, y.v[k]);
#endif
}

)SHELL";

// Shared by both kinds of program (PW_T is float or int): broadcast indexing and how an input is read.
static const char kInputs[] = R"SHELL(
// Element of a broadcast input that output element i reads: (i / div) % mod, a zero extent skipping its step.
__device__ __forceinline__ i64 pw_index(i64 i, i64 n, i64 div, i64 mod) {
    if (n <= 0x7fffffffLL) {                       // the usual case: 32-bit division
        unsigned j = (unsigned)i;
        if (div > 0) j = div > 0x7fffffffLL ? 0u : j / (unsigned)div;
        if (mod > 0 && mod <= 0x7fffffffLL) j %= (unsigned)mod;
        return (i64)j;
    }
    if (div > 0) i /= div;
    if (mod > 0) i %= mod;
    return i;
}
template <int DT, int BC> __device__ __forceinline__ PwVec pw_in(const void* p, i64 g, i64 n, i64 div, i64 mod) {
#if PW_VEC
    if (BC == 2) return pw_ldv<DT>(p, pw_index(g * PW_G, n, 0, mod) / PW_G);      // a row vector, group by group
#endif
    if (BC) {
        const i64 i = g * PW_G;
        PwVec r;
#pragma unroll
        for (int k = 0; k < PW_G; ++k) r.v[k] = i + k < n ? pw_ld1<DT>(p, pw_index(i + k, n, div, mod)) : (PW_T)0;
        return r;
    }
#if PW_VEC
    return pw_ldv<DT>(p, g);
#else
    const i64 i = g * PW_G;
    PwVec r;
#pragma unroll
    for (int k = 0; k < PW_G; ++k) r.v[k] = i + k < n ? pw_ld1<DT>(p, i + k) : (PW_T)0;
    return r;
#endif
}
)SHELL";

static const char kKernel[] = R"SHELL(
#define PW_THREADS 256
#define PW_UNROLL 2
// The inputs of one trip (PW_UNROLL groups, `stride` groups apart, from group g0): every load is issued before any use.
__device__ __forceinline__ void pw_trip(PwVec* x0, PwVec* x1, PwVec* x2, PwVec* x3, const void* p0, const void* p1, const void* p2, const void* p3,
                                        i64 g0, i64 stride, i64 groups, i64 n, const PwBcast& bc) {
#pragma unroll
    for (int u = 0; u < PW_UNROLL; ++u) {
        const i64 g = g0 + u * stride;
#pragma unroll
        for (int k = 0; k < PW_G; ++k) x0[u].v[k] = x1[u].v[k] = x2[u].v[k] = x3[u].v[k] = (PW_T)0;
        if (g < groups) {
            x0[u] = pw_in<PW_DT0, PW_BC0>(p0, g, n, bc.div[0], bc.mod[0]);
#if PW_N_IN > 1
            x1[u] = pw_in<PW_DT1, PW_BC1>(p1, g, n, bc.div[1], bc.mod[1]);
#endif
#if PW_N_IN > 2
            x2[u] = pw_in<PW_DT2, PW_BC2>(p2, g, n, bc.div[2], bc.mod[2]);
#endif
#if PW_N_IN > 3
            x3[u] = pw_in<PW_DT3, PW_BC3>(p3, g, n, bc.div[3], bc.mod[3]);
#endif
        }
    }
}
extern "C" __global__ void __launch_bounds__(PW_THREADS) pw_jit_kernel(const void* p0, const void* p1, const void* p2, const void* p3,
                                                                       void* out, i64 n, PwConsts c, PwBcast bc) {
    const i64 groups = PW_VEC ? n / PW_G : (n + PW_G - 1) / PW_G;
    const i64 stride = (i64)gridDim.x * PW_THREADS;
    i64 g0 = (i64)blockIdx.x * PW_THREADS + threadIdx.x;
    PwVec x0[PW_UNROLL], x1[PW_UNROLL], x2[PW_UNROLL], x3[PW_UNROLL];
#if PW_AHEAD
    // Programs of a few cheap steps: the next trip's inputs are requested before this trip's stores go out, so loads and
    // stores of a thread overlap (measured at 2^26 elements: abs 94 -> 87 us, add 138 -> 132). Programs with a
    // transcendental step keep the plain loop below: the doubled register set costs them more than the overlap gives
    // (two-input SiLU gate 126 -> 142 us, 16-bit erf-GELU 81 -> 88).
    pw_trip(x0, x1, x2, x3, p0, p1, p2, p3, g0, stride, groups, n, bc);
    for (; g0 < groups; g0 += stride * PW_UNROLL) {
        PwVec a0[PW_UNROLL], a1[PW_UNROLL], a2[PW_UNROLL], a3[PW_UNROLL];
        pw_trip(a0, a1, a2, a3, p0, p1, p2, p3, g0 + stride * PW_UNROLL, stride, groups, n, bc);
#else
    for (; g0 < groups; g0 += stride * PW_UNROLL) {
        pw_trip(x0, x1, x2, x3, p0, p1, p2, p3, g0, stride, groups, n, bc);
#endif
#pragma unroll
        for (int u = 0; u < PW_UNROLL; ++u) {
            const i64 g = g0 + u * stride;
            if (g < groups) {
                PwVec y;
#pragma unroll
                for (int k = 0; k < PW_G; ++k) y.v[k] = pw_cell(x0[u].v[k], x1[u].v[k], x2[u].v[k], x3[u].v[k], c);
                pw_out(out, g, n, y);
            }
        }
#if PW_AHEAD
#pragma unroll
        for (int u = 0; u < PW_UNROLL; ++u) { x0[u] = a0[u]; x1[u] = a1[u]; x2[u] = a2[u]; x3[u] = a3[u]; }
#endif
    }
#if PW_VEC
    // the last n % PW_G elements of the vector form: one thread each, scalar accesses
    const int tail = (int)(n % PW_G);
    if (blockIdx.x == 0 && (int)threadIdx.x < tail) {
        const i64 i = n - tail + threadIdx.x;
        PW_T v0 = (PW_T)0, v1 = (PW_T)0, v2 = (PW_T)0, v3 = (PW_T)0;
        v0 = pw_ld1<PW_DT0>(p0, PW_BC0 ? pw_index(i, n, bc.div[0], bc.mod[0]) : i);
#if PW_N_IN > 1
        v1 = pw_ld1<PW_DT1>(p1, PW_BC1 ? pw_index(i, n, bc.div[1], bc.mod[1]) : i);
#endif
#if PW_N_IN > 2
        v2 = pw_ld1<PW_DT2>(p2, PW_BC2 ? pw_index(i, n, bc.div[2], bc.mod[2]) : i);
#endif
#if PW_N_IN > 3
        v3 = pw_ld1<PW_DT3>(p3, PW_BC3 ? pw_index(i, n, bc.div[3], bc.mod[3]) : i);
#endif
        pw_st1(out, i, pw_cell(v0, v1, v2, v3, c));
    }
#endif
}
)SHELL";

// The kernel of an indexed program (emmyb200_pointwise_indexed): one cell per thread and trip. The cell number is
// split into the digits of the tile's axes (outermost first, last fastest, emmyptx/kernel.py:587-626); input k reads
// element offset + sum coef * digit of its buffer, or IS a digit; the value goes to element out_offset + sum out_coef *
// digit. PW_NAXES and PW_KIND0..3 (0 buffer, 1 digit) are defined in front of it. 32-bit index arithmetic whenever the
// cell count and every buffer extent fit (the host says so through `narrow`).
static const char kIndexedKernel[] = R"SHELL(
struct PwIndexArg { i64 extent[6]; i64 in_offset[4]; i64 in_coef[4][6]; i64 out_offset; i64 out_coef[6]; int in_axis[4]; int narrow;
                    int pad; i64 in_rot[4][6]; i64 in_index_mod[4]; i64 in_index_mult[4]; };
template <int DT> __device__ __forceinline__ i64 pw_ldi(const void* p, i64 i) {       // an index taken from an i32 / i64 buffer
    return DT == 3 ? (i64)reinterpret_cast<const int*>(p)[i] : (i64)reinterpret_cast<const long long*>(p)[i];
}
template <typename I> __device__ __forceinline__ void pw_ix_cell(const void* p0, const void* p1, const void* p2, const void* p3, void* out, I i,
                                                               const PwConsts& c, const PwIndexArg& m) {
    I d[PW_NAXES > 0 ? PW_NAXES : 1];
    I rem = i;
#pragma unroll
    for (int a = PW_NAXES - 1; a >= 0; --a) {
        const I e = (I)m.extent[a];
        const I q = rem / e;
        d[a] = rem - q * e;
        rem = q;
    }
    I at[4], to = (I)m.out_offset;
#pragma unroll
    for (int k = 0; k < 4; ++k) at[k] = (I)m.in_offset[k];
#pragma unroll
    for (int a = 0; a < PW_NAXES; ++a) {
#if PW_SPECIAL
        const I e = (I)m.extent[a];                     // a rotated axis enters input k's map as (digit + rot) mod extent
#pragma unroll
        for (int k = 0; k < PW_N_IN; ++k) {
            I dk = d[a] + (I)m.in_rot[k][a];
            dk -= dk >= e ? e : (I)0;
            at[k] += (I)m.in_coef[k][a] * dk;
        }
#else
#pragma unroll
        for (int k = 0; k < PW_N_IN; ++k) at[k] += (I)m.in_coef[k][a] * d[a];
#endif
        to += (I)m.out_coef[a] * d[a];
    }
    PW_T v0 = (PW_T)0, v1 = (PW_T)0, v2 = (PW_T)0, v3 = (PW_T)0;
#if PW_SPECIAL
    PW_GATHER                                           // generated: index sources first, then the buffers they address
#else
    v0 = PW_KIND0 ? (PW_T)d[m.in_axis[0]] : pw_ld1<PW_DT0>(p0, (i64)at[0]);
#if PW_N_IN > 1
    v1 = PW_KIND1 ? (PW_T)d[m.in_axis[1]] : pw_ld1<PW_DT1>(p1, (i64)at[1]);
#endif
#if PW_N_IN > 2
    v2 = PW_KIND2 ? (PW_T)d[m.in_axis[2]] : pw_ld1<PW_DT2>(p2, (i64)at[2]);
#endif
#if PW_N_IN > 3
    v3 = PW_KIND3 ? (PW_T)d[m.in_axis[3]] : pw_ld1<PW_DT3>(p3, (i64)at[3]);
#endif
#endif
    pw_st1(out, (i64)to, pw_cell(v0, v1, v2, v3, c));
}
// Four consecutive cells of the innermost axis per thread and trip (PW_INNER 4: the axis' extent is a multiple of 4): the
// digits are worked out once per group, and an input (PW_IVECk) or the output (PW_OVEC) whose map advances by one
// element per cell from a 4-aligned start is moved with one vector access.
#if PW_INNER == 4
template <int DT, int VEC, int KIND> __device__ __forceinline__ PwVec pw_ix_in(const void* p, i64 at, i64 step, int axis_is_last, PW_T digit) {
    PwVec r;
    if (KIND) {
#pragma unroll
        for (int j = 0; j < 4; ++j) r.v[j] = digit + (PW_T)(axis_is_last ? j : 0);
        return r;
    }
    if (VEC) return pw_ldv<DT>(p, at >> 2);
#pragma unroll
    for (int j = 0; j < 4; ++j) r.v[j] = pw_ld1<DT>(p, at + j * step);
    return r;
}
template <typename I> __device__ __forceinline__ void pw_ix_group(const void* p0, const void* p1, const void* p2, const void* p3, void* out, I gi,
                                                                const PwConsts& c, const PwIndexArg& m) {
    I d[PW_NAXES > 0 ? PW_NAXES : 1];
    I rem = gi;
#pragma unroll
    for (int a = PW_NAXES - 1; a >= 0; --a) {
        const I e = a == PW_NAXES - 1 ? (I)(m.extent[a] >> 2) : (I)m.extent[a];
        const I q = rem / e;
        d[a] = rem - q * e;
        rem = q;
    }
    d[PW_NAXES - 1] *= 4;
    I at[4], to = (I)m.out_offset;
#pragma unroll
    for (int k = 0; k < 4; ++k) at[k] = (I)m.in_offset[k];
#pragma unroll
    for (int a = 0; a < PW_NAXES; ++a) {
#pragma unroll
        for (int k = 0; k < PW_N_IN; ++k) at[k] += (I)m.in_coef[k][a] * d[a];
        to += (I)m.out_coef[a] * d[a];
    }
    PwVec v0, v1, v2, v3;
#pragma unroll
    for (int j = 0; j < 4; ++j) v0.v[j] = v1.v[j] = v2.v[j] = v3.v[j] = (PW_T)0;
    v0 = pw_ix_in<PW_DT0, PW_IVEC0, PW_KIND0>(p0, (i64)at[0], m.in_coef[0][PW_NAXES - 1], m.in_axis[0] == PW_NAXES - 1, (PW_T)d[m.in_axis[0]]);
#if PW_N_IN > 1
    v1 = pw_ix_in<PW_DT1, PW_IVEC1, PW_KIND1>(p1, (i64)at[1], m.in_coef[1][PW_NAXES - 1], m.in_axis[1] == PW_NAXES - 1, (PW_T)d[m.in_axis[1]]);
#endif
#if PW_N_IN > 2
    v2 = pw_ix_in<PW_DT2, PW_IVEC2, PW_KIND2>(p2, (i64)at[2], m.in_coef[2][PW_NAXES - 1], m.in_axis[2] == PW_NAXES - 1, (PW_T)d[m.in_axis[2]]);
#endif
#if PW_N_IN > 3
    v3 = pw_ix_in<PW_DT3, PW_IVEC3, PW_KIND3>(p3, (i64)at[3], m.in_coef[3][PW_NAXES - 1], m.in_axis[3] == PW_NAXES - 1, (PW_T)d[m.in_axis[3]]);
#endif
    PwVec y;
#pragma unroll
    for (int j = 0; j < 4; ++j) y.v[j] = pw_cell(v0.v[j], v1.v[j], v2.v[j], v3.v[j], c);
#if PW_OVEC
    pw_stv(out, (i64)to >> 2, y);
#else
#pragma unroll
    for (int j = 0; j < 4; ++j) pw_st1(out, (i64)to + j * m.out_coef[PW_NAXES - 1], y.v[j]);
#endif
}
#endif
// A transposition (PW_TRANSPOSE 1): the one buffer input is contiguous along axis PW_RAXIS, the output along another axis
// PW_WAXIS (one of the two is the innermost axis). A CTA moves PW_TT x PW_TT tiles (64, or 32 when an axis is shorter than
// 64) of those two axes through shared memory (rows padded by one word), reading with the lanes along PW_RAXIS and writing
// with the lanes along PW_WAXIS, so both sides are coalesced, in runs of PW_TT elements; the other axes count tiles.
// PW_TIN is the index of the buffer input among the inputs.
#if PW_TRANSPOSE
template <typename I> __device__ __forceinline__ void pw_ix_tiles(const void* p0, const void* p1, const void* p2, const void* p3, void* out,
                                                                const PwConsts& c, const PwIndexArg& m, PW_T (*tile)[PW_TT + 1]) {
    const void* src = PW_TIN == 0 ? p0 : (PW_TIN == 1 ? p1 : (PW_TIN == 2 ? p2 : p3));
    const I er = (I)m.extent[PW_RAXIS], ew = (I)m.extent[PW_WAXIS];
    const I tiles_r = (er + PW_TT - 1) / PW_TT, tiles_w = (ew + PW_TT - 1) / PW_TT;
    I batch = 1;
#pragma unroll
    for (int a = 0; a < PW_NAXES; ++a)
        if (a != PW_RAXIS && a != PW_WAXIS) batch *= (I)m.extent[a];
    const i64 work = (i64)batch * tiles_r * tiles_w;
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
    I d[PW_NAXES > 0 ? PW_NAXES : 1];
    I at = 0, to = 0, r0 = 0, w0 = 0;
    // where tile w starts: the digits of the other axes, the bases of both maps, the tile's corner
    auto origin = [&](i64 w) {
        I rem = (I)w;
        const I tw = rem % tiles_w; rem /= tiles_w;
        const I tr = rem % tiles_r; rem /= tiles_r;
#pragma unroll
        for (int a = PW_NAXES - 1; a >= 0; --a) {
            if (a == PW_RAXIS || a == PW_WAXIS) { d[a] = 0; continue; }
            const I e = (I)m.extent[a];
            const I q = rem / e;
            d[a] = rem - q * e;
            rem = q;
        }
        at = (I)m.in_offset[PW_TIN];
        to = (I)m.out_offset;
#pragma unroll
        for (int a = 0; a < PW_NAXES; ++a) {
            at += (I)m.in_coef[PW_TIN][a] * d[a];
            to += (I)m.out_coef[a] * d[a];
        }
        r0 = tr * PW_TT;
        w0 = tw * PW_TT;
    };
    PW_T got[PW_TT / 8][PW_TT / 32];
    auto fetch = [&]() {                                        // every load of a tile is issued before anything uses one
#pragma unroll
        for (int k = 0; k < PW_TT / 8; ++k)
#pragma unroll
            for (int q = 0; q < PW_TT / 32; ++q) {
                const I r = r0 + x + 32 * q, v = w0 + y + 8 * k;
                got[k][q] = (r < er && v < ew) ? pw_ld1<PW_TDT>(src, (i64)(at + r + (I)m.in_coef[PW_TIN][PW_WAXIS] * v)) : (PW_T)0;
            }
    };
    i64 w = blockIdx.x;
    if (w < work) { origin(w); fetch(); }
    for (; w < work; w += gridDim.x) {
        __syncthreads();                                        // the previous tile has been read out
#pragma unroll
        for (int k = 0; k < PW_TT / 8; ++k)
#pragma unroll
            for (int q = 0; q < PW_TT / 32; ++q) tile[y + 8 * k][x + 32 * q] = got[k][q];
        __syncthreads();
        // this tile's corner and bases for the store phase; then the next tile's loads go out and fly during the stores
        const I s_to = to, s_r0 = r0, s_w0 = w0;
        I sd[PW_NAXES > 0 ? PW_NAXES : 1];
#pragma unroll
        for (int a = 0; a < PW_NAXES; ++a) sd[a] = d[a];
        if (w + gridDim.x < work) { origin(w + gridDim.x); fetch(); }
#pragma unroll
        for (int kq = 0; kq < (PW_TT / 8) * (PW_TT / 32); ++kq) {
            const int k = kq / (PW_TT / 32), q = kq % (PW_TT / 32);
            const I v = s_w0 + x + 32 * q, r = s_r0 + y + 8 * k;
            if (r < er && v < ew) {
                sd[PW_RAXIS] = r;
                sd[PW_WAXIS] = v;
                const PW_T val = tile[x + 32 * q][y + 8 * k];
                const PW_T v0 = PW_KIND0 ? (PW_T)sd[m.in_axis[0]] : val;
                const PW_T v1 = PW_N_IN > 1 ? (PW_KIND1 ? (PW_T)sd[m.in_axis[1]] : val) : (PW_T)0;
                const PW_T v2 = PW_N_IN > 2 ? (PW_KIND2 ? (PW_T)sd[m.in_axis[2]] : val) : (PW_T)0;
                const PW_T v3 = PW_N_IN > 3 ? (PW_KIND3 ? (PW_T)sd[m.in_axis[3]] : val) : (PW_T)0;
                pw_st1(out, (i64)(s_to + (I)m.out_coef[PW_RAXIS] * r + v), pw_cell(v0, v1, v2, v3, c));
            }
        }
    }
}
#endif
extern "C" __global__ void __launch_bounds__(256) pw_ix_kernel(const void* p0, const void* p1, const void* p2, const void* p3, void* out, i64 n,
                                                               PwConsts c, PwIndexArg m) {
#if PW_TRANSPOSE
    __shared__ PW_T tile[PW_TT][PW_TT + 1];
    if (m.narrow) pw_ix_tiles<int>(p0, p1, p2, p3, out, c, m, tile);
    else pw_ix_tiles<i64>(p0, p1, p2, p3, out, c, m, tile);
    return;
#endif
    const i64 stride = (i64)gridDim.x * 256;
#if PW_INNER == 4
    for (i64 g = (i64)blockIdx.x * 256 + threadIdx.x; g < (n >> 2); g += stride) {
        if (m.narrow) pw_ix_group<int>(p0, p1, p2, p3, out, (int)g, c, m);
        else pw_ix_group<i64>(p0, p1, p2, p3, out, g, c, m);
    }
#else
    for (i64 i = (i64)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        if (m.narrow) pw_ix_cell<int>(p0, p1, p2, p3, out, (int)i, c, m);
        else pw_ix_cell<i64>(p0, p1, p2, p3, out, i, c, m);
    }
#endif
}
)SHELL";

// The kernel of emmyb200_contract_indexed: one output cell per thread and trip; the cell's value is the sum over up to
// three nested reduction axes of A[...] * B[...], both addressed by affine maps of the tile's and the loops' digits,
// folded in loop order with one fused multiply-add per term (as the reference forms an FMA from the multiply feeding
// the Accum, emmyptx/kernel.py:786-797). CT_NLOOPS, PW_NAXES, PW_DT0 (A), PW_DT1 (B) and PW_OUT_DT are defined in front.
static const char kContractionKernel[] = R"SHELL(
struct CtArg { i64 extent[6]; i64 loop_extent[3]; i64 a_offset; i64 a_coef[6]; i64 a_loop[3]; i64 b_offset; i64 b_coef[6]; i64 b_loop[3];
               i64 out_offset; i64 out_coef[6]; int narrow; int pad; };
template <typename I> __device__ __forceinline__ void ct_cell(const void* a, const void* b, void* out, I i, const CtArg& m) {
    I rem = i, at = (I)m.a_offset, bt = (I)m.b_offset, to = (I)m.out_offset;
#pragma unroll
    for (int ax = PW_NAXES - 1; ax >= 0; --ax) {
        const I e = (I)m.extent[ax];
        const I q = rem / e;
        const I d = rem - q * e;
        rem = q;
        at += (I)m.a_coef[ax] * d;
        bt += (I)m.b_coef[ax] * d;
        to += (I)m.out_coef[ax] * d;
    }
    const I n0 = (I)m.loop_extent[0], n1 = CT_NLOOPS > 1 ? (I)m.loop_extent[1] : (I)1, n2 = CT_NLOOPS > 2 ? (I)m.loop_extent[2] : (I)1;
    const I a0 = (I)m.a_loop[0], a1 = CT_NLOOPS > 1 ? (I)m.a_loop[1] : (I)0, a2 = CT_NLOOPS > 2 ? (I)m.a_loop[2] : (I)0;
    const I b0 = (I)m.b_loop[0], b1 = CT_NLOOPS > 1 ? (I)m.b_loop[1] : (I)0, b2 = CT_NLOOPS > 2 ? (I)m.b_loop[2] : (I)0;
    float acc = 0.0f;
    for (I l0 = 0; l0 < n0; ++l0)
        for (I l1 = 0; l1 < n1; ++l1) {
            const I ar = at + a0 * l0 + a1 * l1, br = bt + b0 * l0 + b1 * l1;
            for (I l2 = 0; l2 < n2; ++l2)
                acc = fmaf(pw_ld1<PW_DT0>(a, (i64)(ar + a2 * l2)), pw_ld1<PW_DT1>(b, (i64)(br + b2 * l2)), acc);
        }
    pw_st1(out, (i64)to, acc);
}
extern "C" __global__ void __launch_bounds__(256) ct_kernel(const void* a, const void* b, void* out, i64 n, CtArg m) {
    const i64 stride = (i64)gridDim.x * 256;
    for (i64 i = (i64)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        if (m.narrow) ct_cell<int>(a, b, out, (int)i, m);
        else ct_cell<i64>(a, b, out, i, m);
    }
}
)SHELL";

static bool float_program(const emmyb200_pw_program& p) {          // computed in fp32; a byte output holds value != 0
    return p.out_dtype == EMMYB200_F32 || p.out_dtype == EMMYB200_F16 || p.out_dtype == EMMYB200_BF16 || p.out_dtype == EMMYB200_U8;
}

// How input k is read: 0 element i; 1 a broadcast input gathered element by element; 2 a row vector whose length is a
// multiple of the access group (a bias over the last axis): vector accesses at the wrapped position. `base_aligned`
// says whether the buffer itself allows those accesses.
static int broadcast_mode(const emmyb200_pw_program& p, int k, int group, bool base_aligned) {
    if ((p.in_div[k] | p.in_mod[k]) == 0) return 0;
    const int per = group == 8 ? 8 : 4;
    return (group != 0 && base_aligned && p.in_div[k] == 0 && p.in_mod[k] % per == 0) ? 2 : 1;
}

struct IndexedForm {        // how the indexed kernel walks the tile (chosen on the host from extents, maps and alignment)
    int inner = 1;          // cells of the innermost axis per thread: 1 or 4
    int ivec[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};      // input k is read with one vector access per group
    int ovec = 0;           // the output is written with one vector access per group
    int special = 0;        // 1: some map rotates an axis or takes an index from data: the one-cell form with spelled-out loads
    int transpose = 0;      // 1: square tiles of (taxis, innermost axis) through shared memory
    int ttile = 32;         // their side: 64 when both axes are at least that long
    int taxis = 0, tin = 0; // the axis (other than the innermost) the transposition is against; which input the buffer is
    int swapped = 0;        // 0: the input is contiguous along taxis, the output along the innermost axis; 1: the other way round
};

static std::string program_source(const emmyb200_pw_program& p, int group, const int* modes, const emmyb200_pw_index_map* map = nullptr,
                                  const IndexedForm* form = nullptr) {
    const bool ints = !float_program(p);
    const char* type = ints ? "int" : "float";
    std::string s;
    char line[200];
    snprintf(line, sizeof line, "#define PW_N_IN %d\n#define PW_VEC %d\n#define PW_G %d\n#define PW_OUT_DT %d\n#define PW_T %s\n", p.n_inputs,
             group ? 1 : 0, group == 8 && !ints ? 8 : 4, p.out_dtype, type);
    s += line;
    bool heavy = false;                 // a step that costs tens of instructions: such programs do not request inputs a trip ahead
    for (int i = 0; i < p.n_steps && !ints; ++i) {
        const int op = p.steps[i].op;
        heavy = heavy || op == EMMYB200_PW_EXP || op == EMMYB200_PW_LOG || op == EMMYB200_PW_SIGMOID || op == EMMYB200_PW_TANH || op == EMMYB200_PW_ERF ||
                op == EMMYB200_PW_SIN || op == EMMYB200_PW_COS || op == EMMYB200_PW_POW;
    }
    s += heavy || ints ? "#define PW_AHEAD 0\n" : "#define PW_AHEAD 1\n";
    for (int k = 0; k < EMMYB200_PW_MAX_INPUTS; ++k) {
        const bool used = k < p.n_inputs;
        snprintf(line, sizeof line, "#define PW_DT%d %d\n#define PW_BC%d %d\n", k, used ? p.in_dtype[k] : (ints ? EMMYB200_I32 : EMMYB200_F32), k, used ? modes[k] : 0);
        s += line;
    }
    if (map != nullptr) {
        snprintf(line, sizeof line, "#define PW_NAXES %d\n#define PW_KIND0 %d\n#define PW_KIND1 %d\n#define PW_KIND2 %d\n#define PW_KIND3 %d\n", map->n_axes,
                 map->in_kind[0] == 1, map->in_kind[1] == 1, map->in_kind[2] == 1, map->in_kind[3] == 1);
        s += line;
        const IndexedForm plain;
        const IndexedForm& f = form != nullptr ? *form : plain;
        snprintf(line, sizeof line, "#define PW_INNER %d\n#define PW_IVEC0 %d\n#define PW_IVEC1 %d\n#define PW_IVEC2 %d\n#define PW_IVEC3 %d\n#define PW_OVEC %d\n",
                 f.inner, f.ivec[0], f.ivec[1], f.ivec[2], f.ivec[3], f.ovec);
        s += line;
        snprintf(line, sizeof line, "#define PW_TT %d\n", f.ttile);
        s += line;
        snprintf(line, sizeof line, "#define PW_TRANSPOSE %d\n#define PW_RAXIS %d\n#define PW_WAXIS %d\n#define PW_TIN %d\n#define PW_TDT %d\n", f.transpose,
                 f.swapped ? map->n_axes - 1 : f.taxis, f.swapped ? f.taxis : map->n_axes - 1, f.tin, p.in_dtype[f.tin]);
        s += line;
        snprintf(line, sizeof line, "#define PW_SPECIAL %d\n", f.special);
        s += line;
        if (f.special) {                        // the loads of the one-cell form, spelled out: index sources, then everything else
            s += "#define PW_GATHER";
            for (int pass = 0; pass < 2; ++pass)
                for (int k = 0; k < p.n_inputs; ++k) {
                    const int kind = map->in_kind[k];
                    if ((kind == 3) != (pass == 0)) continue;
                    const std::string K = std::to_string(k), DT = std::to_string(p.in_dtype[k]);
                    if (kind == 3) {
                        s += " i64 x" + K + " = pw_ldi<" + DT + ">(p" + K + ", (i64)at[" + K + "]);";
                        if (map->in_index_abs[k]) s += " x" + K + " = x" + K + " < 0 ? -x" + K + " : x" + K + ";";
                        s += " x" + K + " %= m.in_index_mod[" + K + "]; if (x" + K + " < 0) x" + K + " += m.in_index_mod[" + K + "];";
                    } else if (kind == 2) {
                        s += " v" + K + " = pw_ld1<" + DT + ">(p" + K + ", (i64)at[" + K + "] + m.in_index_mult[" + K + "] * x" + std::to_string(map->in_index_of[k]) + ");";
                    } else if (kind == 1) {
                        s += " v" + K + " = (PW_T)d[m.in_axis[" + K + "]];";
                    } else if (kind == 4) {
                        s += " { i64 g = (i64)at[" + K + "]; g = g < 0 ? 0 : (g >= m.in_index_mod[" + K + "] ? m.in_index_mod[" + K + "] - 1 : g); v" + K +
                             " = pw_ld1<" + DT + ">(p" + K + ", g); }";
                    } else {
                        s += " v" + K + " = pw_ld1<" + DT + ">(p" + K + ", (i64)at[" + K + "]);";
                    }
                }
            s += "\n";
        }
    }
    if (!ints) s += "#include \"emmy_math.cuh\"\n";
    s += "typedef long long i64;\n"
         "struct PwConsts { float v[16]; };\n"
         "struct PwBcast { i64 div[4]; i64 mod[4]; };\n"
         "struct PwVec { PW_T v[PW_G]; };\n";
    if (ints) s += kIntOps;
    snprintf(line, sizeof line, "__device__ __forceinline__ %s pw_cell(%s i0, %s i1, %s i2, %s i3, const PwConsts& c) {\n    %s s0 = i0, s1 = i1, s2 = i2, s3 = i3",
             type, type, type, type, type, type);
    s += line;
    for (int k = EMMYB200_PW_MAX_INPUTS; k < EMMYB200_PW_MAX_SLOTS; ++k) {
        snprintf(line, sizeof line, ", s%d = 0", k);
        s += line;
    }
    s += ";\n";
    for (int i = 0; i < p.n_steps; ++i) {
        const emmyb200_pw_step& st = p.steps[i];
        snprintf(line, sizeof line, "    s%d = ", st.dst);
        s += line;
        s += expand(ints ? op_expr_int(st.op) : op_expr(st.op), st, ints);
        s += ";\n";
    }
    snprintf(line, sizeof line, "    return s%d;\n}\n", p.out_slot);
    s += line;
    s += ints ? kIntLoads : kFloatLoads;
    if (map == nullptr) s += kInputs;
    s += ints ? kIntStores : kFloatStores;
    s += map == nullptr ? kKernel : kIndexedKernel;
    return s;
}

// Everything the generated text depends on, and nothing else: the cache key.
static std::string program_key(const emmyb200_pw_program& p, int group, const int* modes) {
    std::string k;
    auto put = [&](int v) { k.push_back((char)(v & 0xff)); };
    put(p.n_inputs); put(p.n_steps); put(p.out_slot); put(p.out_dtype); put(group);
    for (int i = 0; i < p.n_inputs; ++i) { put(p.in_dtype[i]); put(modes[i]); }
    for (int i = 0; i < p.n_steps; ++i) { put(p.steps[i].op); put(p.steps[i].dst); put(p.steps[i].a); put(p.steps[i].b); put(p.steps[i].c); put(p.steps[i].reserved[0]); }
    return k;
}

// Source text -> device code for sm_100a. No device is needed for this step.
static int compile_source(const std::string& src, std::vector<char>* cubin) {
    const Nvrtc& rt = nvrtc();
    if (!rt.ok) return fail(EMMYB200_ERR_UNSUPPORTED, "pointwise_program: NVRTC is not available (%s)", rt.handle ? "symbols missing" : "libnvrtc.so.12 not found");
    const char* header_text[] = {kMathHeader, kStdintStub, kMathStub, kEmptyStub};
    const char* header_name[] = {"emmy_math.cuh", "stdint.h", "math.h", "string.h"};
    nvrtcProgram prog = nullptr;
    nvrtcResult r = rt.CreateProgram(&prog, src.c_str(), "pw_jit_kernel.cu", 4, header_text, header_name);
    if (r != NVRTC_SUCCESS) return fail(EMMYB200_ERR_DEVICE, "nvrtcCreateProgram: %s", rt.GetErrorString(r));
    const char* options[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
    r = rt.CompileProgram(prog, 3, options);
    if (r != NVRTC_SUCCESS) {
        size_t n = 0;
        rt.GetProgramLogSize(prog, &n);
        std::string log(n, '\0');
        if (n > 1) rt.GetProgramLog(prog, &log[0]);
        rt.DestroyProgram(&prog);
        return fail(EMMYB200_ERR_DEVICE, "pointwise_program: NVRTC (%s): %.400s", rt.GetErrorString(r), log.c_str());
    }
    size_t bytes = 0;
    r = rt.GetCUBINSize(prog, &bytes);
    if (r == NVRTC_SUCCESS && bytes > 0) {
        cubin->resize(bytes);
        r = rt.GetCUBIN(prog, cubin->data());
    }
    rt.DestroyProgram(&prog);
    if (r != NVRTC_SUCCESS || bytes == 0) return fail(EMMYB200_ERR_DEVICE, "pointwise_program: NVRTC produced no device code (%s)", rt.GetErrorString(r));
    return EMMYB200_OK;
}

struct JitKernel {
    cudaLibrary_t library = nullptr;
    cudaKernel_t kernel = nullptr;
    int ctas_per_sm = 8;            // 256-thread CTAs resident per SM (the kernel's registers decide), asked once at load
};

// Grid-stride kernels are sized to what is resident at once: a grid larger than that runs a thin last wave.
static void ask_residency(JitKernel* k) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reinterpret_cast<const void*>(k->kernel), 256, 0) == cudaSuccess && per_sm >= 1)
        k->ctas_per_sm = per_sm;
    else
        cudaGetLastError();         // an older runtime that does not take kernel handles here: keep the default
}

static std::mutex g_jit_mutex;
static std::map<std::string, JitKernel>& jit_cache() {
    static std::map<std::string, JitKernel>* m = new std::map<std::string, JitKernel>();      // never destroyed: the runtime may be gone first
    return *m;
}
static std::atomic<long long> g_jit_compiles{0};

struct PwConstsArg { float v[16]; };
struct PwBcastArg { long long div[4]; long long mod[4]; };

int pw_jit_launch(const emmyb200_pw_program& prog, const void* const* inputs, void* out, int64_t n, int group, cudaStream_t stream) {
    if (!jit_enabled() || !nvrtc().ok) return kPwJitUnavailable;
    JitKernel k;
    int modes[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};
    for (int i = 0; i < prog.n_inputs; ++i) {
        const int dt = prog.in_dtype[i];
        const int es = dt == EMMYB200_I64 ? 8 : (dt == EMMYB200_F32 || dt == EMMYB200_I32 ? 4 : (dt == EMMYB200_U8 ? 1 : 2));
        modes[i] = broadcast_mode(prog, i, group, aligned(inputs[i], (size_t)(group == 8 ? 8 : 4) * es));
    }
    {
        std::lock_guard<std::mutex> lock(g_jit_mutex);
        const std::string key = program_key(prog, group, modes);
        auto it = jit_cache().find(key);
        if (it == jit_cache().end()) {
            std::vector<char> cubin;
            int rc = compile_source(program_source(prog, group, modes), &cubin);
            if (rc != EMMYB200_OK) return rc;
            cudaError_t e = cudaLibraryLoadData(&k.library, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
            if (e != cudaSuccess) return cuda_fail(e, "cudaLibraryLoadData (specialised elementwise kernel)");
            e = cudaLibraryGetKernel(&k.kernel, k.library, "pw_jit_kernel");
            if (e != cudaSuccess) { cudaLibraryUnload(k.library); return cuda_fail(e, "cudaLibraryGetKernel (specialised elementwise kernel)"); }
            ask_residency(&k);
            g_jit_compiles.fetch_add(1);
            it = jit_cache().emplace(key, k).first;
        }
        k = it->second;
    }
    const void* p[EMMYB200_PW_MAX_INPUTS] = {nullptr, nullptr, nullptr, nullptr};
    PwConstsArg c;
    PwBcastArg bc;
    for (int i = 0; i < EMMYB200_PW_MAX_CONSTS; ++i) c.v[i] = prog.consts[i];
    for (int i = 0; i < EMMYB200_PW_MAX_INPUTS; ++i) {
        if (i < prog.n_inputs) p[i] = inputs[i];
        bc.div[i] = i < prog.n_inputs ? prog.in_div[i] : 0;
        bc.mod[i] = i < prog.n_inputs ? prog.in_mod[i] : 0;
    }
    long long count = n;
    void* args[] = {&p[0], &p[1], &p[2], &p[3], &out, &count, &c, &bc};
    const int per = group == 8 ? 8 : 4;
    const int64_t groups = (n + per - 1) / per;
    const int64_t want = (groups + 256 * 2 - 1) / (256 * 2);
    const int64_t cap = (int64_t)sm_count() * k.ctas_per_sm;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(k.kernel), dim3(blocks), dim3(256), args, 0, stream);
    if (e != cudaSuccess) return cuda_fail(e, "launch of the specialised elementwise kernel");
    return EMMYB200_OK;
}

static int check_program(const emmyb200_pw_program* prog, const char* who, const emmyb200_pw_index_map* map = nullptr) {
    if (prog == nullptr) return fail(EMMYB200_ERR_ARG, "%s: null program", who);
    if (prog->n_inputs < 1 || prog->n_inputs > EMMYB200_PW_MAX_INPUTS || prog->n_steps < 0 || prog->n_steps > EMMYB200_PW_MAX_STEPS ||
        prog->out_slot < 0 || prog->out_slot >= EMMYB200_PW_MAX_SLOTS)
        return fail(EMMYB200_ERR_ARG, "%s: not a program (inputs, steps or output slot out of range)", who);
    const bool ints = prog->out_dtype == EMMYB200_I32 || prog->out_dtype == EMMYB200_I64;
    if (!float_program(*prog) && !ints) return fail(EMMYB200_ERR_UNSUPPORTED, "%s: output dtype %d", who, prog->out_dtype);
    if (map != nullptr && prog->out_dtype == EMMYB200_U8) return fail(EMMYB200_ERR_UNSUPPORTED, "%s: indexed programs write f32 / f16 / bf16 / i32 / i64", who);
    for (int k = 0; k < prog->n_inputs; ++k) {
        const int d = prog->in_dtype[k];
        const bool index_source = map != nullptr && map->in_kind[k] == 3;          // read as an integer, never as a program value
        const bool ok = (ints || index_source) ? (d == EMMYB200_I32 || d == EMMYB200_I64)
                                               : (d == EMMYB200_F32 || d == EMMYB200_F16 || d == EMMYB200_BF16 || d == EMMYB200_U8);
        if (!ok) return fail(EMMYB200_ERR_UNSUPPORTED, "%s: input %d has dtype %d (%s program)", who, k, d, ints ? "an integer" : "a float");
    }
    for (int i = 0; i < prog->n_steps; ++i) {
        const emmyb200_pw_step& st = prog->steps[i];
        if (st.op >= EMMYB200_PW_OP_COUNT || st.dst >= EMMYB200_PW_MAX_SLOTS) return fail(EMMYB200_ERR_ARG, "%s: bad step %d", who, i);
        for (int o : {st.a, st.b, st.c})
            if (o >= EMMYB200_PW_MAX_SLOTS + EMMYB200_PW_MAX_CONSTS) return fail(EMMYB200_ERR_ARG, "%s: bad operand in step %d", who, i);
    }
    return EMMYB200_OK;
}

struct PwIndexArgHost { long long extent[6]; long long in_offset[4]; long long in_coef[4][6]; long long out_offset; long long out_coef[6]; int in_axis[4]; int narrow;
                        int pad; long long in_rot[4][6]; long long in_index_mod[4]; long long in_index_mult[4]; };

}  // namespace emmy

extern "C" int emmyb200_pointwise_indexed(const emmyb200_pw_program* prog, const emmyb200_pw_index_map* map, const void* const* inputs, void* out,
                                          void* cuda_stream) {
    using namespace emmy;
    if (map == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: null index map");
    int rc = check_program(prog, "pointwise_indexed", map);
    if (rc != EMMYB200_OK) return rc;
    if (map->n_axes < 1 || map->n_axes > EMMYB200_PW_MAX_AXES) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: %d axes (1 to %d)", map->n_axes, EMMYB200_PW_MAX_AXES);
    int64_t n = 1;
    bool narrow = true;
    for (int a = 0; a < map->n_axes; ++a) {
        if (map->extent[a] < 0) return fail(EMMYB200_ERR_SHAPE, "pointwise_indexed: negative extent");
        if (map->extent[a] != 0 && n > ((int64_t)1 << 40)) return fail(EMMYB200_ERR_SHAPE, "pointwise_indexed: too many cells");
        n *= map->extent[a];
    }
    if (n == 0) return EMMYB200_OK;
    if (n > 0x7fffffffLL) narrow = false;
    // the largest and smallest element every map reaches: for the 32-bit choice, and so that a negative index is refused
    auto range_ok = [&](int64_t off, const int64_t* coef, const char* what) -> int {
        int64_t lo = off, hi = off;
        for (int a = 0; a < map->n_axes; ++a) {
            const int64_t span = coef[a] * (map->extent[a] - 1);
            if (span < 0) lo += span; else hi += span;
        }
        if (lo < 0) return fail(EMMYB200_ERR_SHAPE, "pointwise_indexed: %s reaches element %lld", what, (long long)lo);
        if (hi > 0x7fffffffLL) narrow = false;
        for (int a = 0; a < map->n_axes; ++a)
            if (coef[a] > 0x7fffffffLL || coef[a] < -0x7fffffffLL) narrow = false;
        return EMMYB200_OK;
    };
    if (inputs == nullptr || out == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: null buffer");
    bool special = false;
    for (int k = 0; k < prog->n_inputs; ++k) {
        const int kind = map->in_kind[k];
        if (kind < 0 || kind > 4) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: input %d has kind %d", k, kind);
        if (kind == 1) {
            if (map->in_axis[k] < 0 || map->in_axis[k] >= map->n_axes) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: input %d names axis %d", k, map->in_axis[k]);
            continue;
        }
        if (inputs[k] == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: null buffer");
        if (kind == 4) {                // a guarded read: the index is clamped into the buffer, the map may leave it
            if (map->in_index_mod[k] < 1) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: guarded input %d needs its buffer's element count", k);
            narrow = false;
            special = true;
            continue;
        }
        if ((rc = range_ok(map->in_offset[k], map->in_coef[k], "an input map")) != EMMYB200_OK) return rc;
        for (int a = 0; a < map->n_axes; ++a) {
            if (map->in_rot[k][a] < 0 || (map->in_rot[k][a] != 0 && map->in_rot[k][a] >= map->extent[a]))
                return fail(EMMYB200_ERR_ARG, "pointwise_indexed: input %d rotates axis %d by %lld (0 to extent - 1)", k, a, (long long)map->in_rot[k][a]);
            special = special || map->in_rot[k][a] != 0;
        }
        if (kind == 3) {
            if (map->in_index_mod[k] < 1) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: index source %d needs a modulus (it is what bounds the index)", k);
            special = true;
        }
        if (kind == 2) {
            const int src = map->in_index_of[k];
            if (src < 0 || src >= prog->n_inputs || map->in_kind[src] != 3) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: input %d takes its index from input %d, which is no index source", k, src);
            if (map->in_index_mult[k] < 0) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: negative index multiplier");
            if (map->in_offset[k] + map->in_index_mult[k] * (map->in_index_mod[src] - 1) > 0x7fffffffLL) narrow = false;
            special = true;
        }
    }
    for (int st = 0; st < prog->n_steps; ++st)
        for (int o : {prog->steps[st].a, prog->steps[st].b, prog->steps[st].c})
            if (o < prog->n_inputs && map->in_kind[o] == 3) return fail(EMMYB200_ERR_ARG, "pointwise_indexed: step %d reads index source %d as a value", st, o);
    if ((rc = range_ok(map->out_offset, map->out_coef, "the output map")) != EMMYB200_OK) return rc;
    if (!nvrtc().ok) return fail(EMMYB200_ERR_UNSUPPORTED, "pointwise_indexed: needs the run-time compiler (libnvrtc.so.12 not found)");
    emmyb200_pw_index_map key_map = *map;
    for (int k = prog->n_inputs; k < EMMYB200_PW_MAX_INPUTS; ++k) key_map.in_kind[k] = 0;
    // groups of four cells along the innermost axis when its extent allows; vector accesses for the maps that advance by
    // one element per cell from a start that is 4-aligned in every group (offset and the other coefficients multiples of
    // 4, the buffer aligned for four elements)
    IndexedForm form;
    const int last = map->n_axes - 1;
    auto elem_size = [](int dt) { return dt == EMMYB200_I64 ? 8 : (dt == EMMYB200_F32 || dt == EMMYB200_I32 ? 4 : (dt == EMMYB200_U8 ? 1 : 2)); };
    auto vector_ok = [&](int64_t off, const int64_t* coef, const void* base, int dt) {
        if (coef[last] != 1 || (off & 3) || !aligned(base, (size_t)4 * elem_size(dt))) return false;
        for (int a = 0; a < last; ++a)
            if (coef[a] & 3) return false;
        return true;
    };
    // a transposition: one buffer input, contiguous along some other axis than the innermost, the output contiguous along
    // the innermost axis, both axes long enough for 32 x 32 tiles
    {
        int buffers = 0, which = 0;
        for (int k = 0; k < prog->n_inputs; ++k)
            if (map->in_kind[k] != 1) { ++buffers; which = k; }
        if (buffers == 1 && last >= 1 && map->extent[last] >= 32) {
            const bool out_inner = map->out_coef[last] == 1 && map->in_coef[which][last] != 1;         // reads stride along the innermost axis
            const bool in_inner = map->in_coef[which][last] == 1 && map->out_coef[last] != 1;          // writes do
            for (int a = 0; a < last && (out_inner || in_inner); ++a)
                if ((out_inner ? map->in_coef[which][a] : map->out_coef[a]) == 1 && map->extent[a] >= 32) {
                    form.transpose = 1; form.taxis = a; form.tin = which; form.swapped = in_inner ? 1 : 0;
                    form.ttile = map->extent[a] >= 64 && map->extent[last] >= 64 ? 64 : 32;
                    break;
                }
        }
    }
    form.special = special ? 1 : 0;
    if (special) form.transpose = 0;
    if (!special && !form.transpose && map->extent[last] % 4 == 0) {
        form.inner = 4;
        for (int k = 0; k < prog->n_inputs; ++k)
            form.ivec[k] = map->in_kind[k] == 0 && vector_ok(map->in_offset[k], map->in_coef[k], inputs[k], prog->in_dtype[k]) ? 1 : 0;
        form.ovec = vector_ok(map->out_offset, map->out_coef, out, prog->out_dtype) ? 1 : 0;
    }
    JitKernel kern;
    {
        std::lock_guard<std::mutex> lock(g_jit_mutex);
        const int modes[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};
        std::string key = program_key(*prog, 0, modes);
        key.push_back('x');
        key.push_back((char)map->n_axes);
        for (int k = 0; k < EMMYB200_PW_MAX_INPUTS; ++k) { key.push_back((char)key_map.in_kind[k]); key.push_back((char)form.ivec[k]); }
        key.push_back((char)form.inner);
        key.push_back((char)form.ovec);
        key.push_back((char)form.transpose);
        key.push_back((char)form.taxis);
        key.push_back((char)form.ttile);
        key.push_back((char)form.swapped);
        key.push_back((char)form.tin);
        key.push_back((char)form.special);
        for (int k = 0; k < prog->n_inputs; ++k) { key.push_back((char)map->in_index_of[k]); key.push_back((char)(map->in_index_abs[k] != 0)); }
        auto it = jit_cache().find(key);
        if (it == jit_cache().end()) {
            std::vector<char> cubin;
            rc = compile_source(program_source(*prog, 0, modes, &key_map, &form), &cubin);
            if (rc != EMMYB200_OK) return rc;
            cudaError_t e = cudaLibraryLoadData(&kern.library, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
            if (e != cudaSuccess) return cuda_fail(e, "cudaLibraryLoadData (indexed elementwise kernel)");
            e = cudaLibraryGetKernel(&kern.kernel, kern.library, "pw_ix_kernel");
            if (e != cudaSuccess) { cudaLibraryUnload(kern.library); return cuda_fail(e, "cudaLibraryGetKernel (indexed elementwise kernel)"); }
            g_jit_compiles.fetch_add(1);
            it = jit_cache().emplace(key, kern).first;
        }
        kern = it->second;
    }
    const void* p[EMMYB200_PW_MAX_INPUTS] = {nullptr, nullptr, nullptr, nullptr};
    PwConstsArg c;
    PwIndexArgHost m;
    memset(&m, 0, sizeof m);
    for (int i = 0; i < EMMYB200_PW_MAX_CONSTS; ++i) c.v[i] = prog->consts[i];
    for (int a = 0; a < EMMYB200_PW_MAX_AXES; ++a) {
        m.extent[a] = a < map->n_axes ? map->extent[a] : 1;
        m.out_coef[a] = a < map->n_axes ? map->out_coef[a] : 0;
    }
    m.out_offset = map->out_offset;
    for (int k = 0; k < prog->n_inputs; ++k) {
        p[k] = map->in_kind[k] != 1 ? inputs[k] : nullptr;
        m.in_offset[k] = map->in_offset[k];
        m.in_axis[k] = map->in_kind[k] == 1 ? map->in_axis[k] : 0;
        for (int a = 0; a < map->n_axes; ++a) {
            m.in_coef[k][a] = map->in_kind[k] != 1 ? map->in_coef[k][a] : 0;
            m.in_rot[k][a] = map->in_kind[k] != 1 ? map->in_rot[k][a] : 0;
        }
        m.in_index_mod[k] = map->in_index_mod[k];
        m.in_index_mult[k] = map->in_index_mult[k];
    }
    m.narrow = narrow ? 1 : 0;
    long long count = n;
    void* args[] = {&p[0], &p[1], &p[2], &p[3], &out, &count, &c, &m};
    int64_t want = (n / form.inner + 255) / 256;
    if (form.transpose) {
        want = ((map->extent[form.taxis] + form.ttile - 1) / form.ttile) * ((map->extent[last] + form.ttile - 1) / form.ttile);
        for (int a = 0; a < last; ++a)
            if (a != form.taxis) want *= map->extent[a];
    }
    const int64_t cap = (int64_t)sm_count() * 16;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(kern.kernel), dim3(blocks), dim3(256), args, 0, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return cuda_fail(e, "launch of the indexed elementwise kernel");
    return EMMYB200_OK;
}

namespace emmy {

struct CtArgHost { long long extent[6]; long long loop_extent[3]; long long a_offset; long long a_coef[6]; long long a_loop[3]; long long b_offset;
                   long long b_coef[6]; long long b_loop[3]; long long out_offset; long long out_coef[6]; int narrow; int pad; };

static std::string contraction_source(const emmyb200_contraction_map& m) {
    char line[256];
    snprintf(line, sizeof line,
             "#define PW_N_IN 2\n#define PW_VEC 0\n#define PW_G 4\n#define PW_T float\n#define PW_OUT_DT %d\n#define PW_DT0 %d\n#define PW_DT1 %d\n"
             "#define PW_NAXES %d\n#define CT_NLOOPS %d\n",
             m.out_dtype, m.a_dtype, m.b_dtype, m.n_axes, m.n_loops);
    std::string s = line;
    s += "typedef long long i64;\nstruct PwVec { PW_T v[PW_G]; };\n";
    s += kFloatLoads;
    s += kFloatStores;
    s += kContractionKernel;
    return s;
}

static int check_contraction(const emmyb200_contraction_map* m, const char* who) {
    if (m == nullptr) return fail(EMMYB200_ERR_ARG, "%s: null map", who);
    if (m->n_axes < 1 || m->n_axes > EMMYB200_PW_MAX_AXES || m->n_loops < 1 || m->n_loops > EMMYB200_CT_MAX_LOOPS)
        return fail(EMMYB200_ERR_ARG, "%s: %d tile axes (1 to %d), %d reduction axes (1 to %d)", who, m->n_axes, EMMYB200_PW_MAX_AXES, m->n_loops, EMMYB200_CT_MAX_LOOPS);
    auto float_ok = [](int d) { return d == EMMYB200_F32 || d == EMMYB200_F16 || d == EMMYB200_BF16; };
    if (!float_ok(m->a_dtype) || !float_ok(m->b_dtype) || !float_ok(m->out_dtype)) return fail(EMMYB200_ERR_UNSUPPORTED, "%s: f32 / f16 / bf16 buffers", who);
    return EMMYB200_OK;
}

}  // namespace emmy

extern "C" int emmyb200_contract_indexed(const emmyb200_contraction_map* map, const void* A, const void* B, void* out, void* cuda_stream) {
    using namespace emmy;
    int rc = check_contraction(map, "contract_indexed");
    if (rc != EMMYB200_OK) return rc;
    int64_t n = 1, terms = 1;
    for (int a = 0; a < map->n_axes; ++a) {
        if (map->extent[a] < 0 || (map->extent[a] != 0 && n > ((int64_t)1 << 40))) return fail(EMMYB200_ERR_SHAPE, "contract_indexed: bad extent");
        n *= map->extent[a];
    }
    for (int l = 0; l < map->n_loops; ++l) {
        if (map->loop_extent[l] < 1 || terms > ((int64_t)1 << 40)) return fail(EMMYB200_ERR_SHAPE, "contract_indexed: a reduction axis has %lld terms", (long long)map->loop_extent[l]);
        terms *= map->loop_extent[l];
    }
    if (n == 0) return EMMYB200_OK;
    if (A == nullptr || B == nullptr || out == nullptr) return fail(EMMYB200_ERR_ARG, "contract_indexed: null buffer");
    bool narrow = n <= 0x7fffffffLL;
    auto range_ok = [&](int64_t off, const int64_t* coef, const int64_t* loop, const char* what) -> int {
        int64_t lo = off, hi = off;
        for (int a = 0; a < map->n_axes; ++a) {
            const int64_t span = coef[a] * (map->extent[a] - 1);
            if (span < 0) lo += span; else hi += span;
        }
        for (int l = 0; loop != nullptr && l < map->n_loops; ++l) {
            const int64_t span = loop[l] * (map->loop_extent[l] - 1);
            if (span < 0) lo += span; else hi += span;
        }
        if (lo < 0) return fail(EMMYB200_ERR_SHAPE, "contract_indexed: %s reaches element %lld", what, (long long)lo);
        if (hi > 0x7fffffffLL) narrow = false;
        return EMMYB200_OK;
    };
    if ((rc = range_ok(map->a_offset, map->a_coef, map->a_loop_coef, "the map of A")) != EMMYB200_OK) return rc;
    if ((rc = range_ok(map->b_offset, map->b_coef, map->b_loop_coef, "the map of B")) != EMMYB200_OK) return rc;
    if ((rc = range_ok(map->out_offset, map->out_coef, nullptr, "the output map")) != EMMYB200_OK) return rc;
    if (!nvrtc().ok) return fail(EMMYB200_ERR_UNSUPPORTED, "contract_indexed: needs the run-time compiler (libnvrtc.so.12 not found)");
    JitKernel kern;
    {
        std::lock_guard<std::mutex> lock(g_jit_mutex);
        std::string key = "ct";
        for (int v : {map->n_axes, map->n_loops, map->a_dtype, map->b_dtype, map->out_dtype}) key.push_back((char)v);
        auto it = jit_cache().find(key);
        if (it == jit_cache().end()) {
            std::vector<char> cubin;
            rc = compile_source(contraction_source(*map), &cubin);
            if (rc != EMMYB200_OK) return rc;
            cudaError_t e = cudaLibraryLoadData(&kern.library, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
            if (e != cudaSuccess) return cuda_fail(e, "cudaLibraryLoadData (indexed contraction kernel)");
            e = cudaLibraryGetKernel(&kern.kernel, kern.library, "ct_kernel");
            if (e != cudaSuccess) { cudaLibraryUnload(kern.library); return cuda_fail(e, "cudaLibraryGetKernel (indexed contraction kernel)"); }
            g_jit_compiles.fetch_add(1);
            it = jit_cache().emplace(key, kern).first;
        }
        kern = it->second;
    }
    CtArgHost m;
    memset(&m, 0, sizeof m);
    for (int a = 0; a < EMMYB200_PW_MAX_AXES; ++a) {
        const bool live = a < map->n_axes;
        m.extent[a] = live ? map->extent[a] : 1;
        m.a_coef[a] = live ? map->a_coef[a] : 0;
        m.b_coef[a] = live ? map->b_coef[a] : 0;
        m.out_coef[a] = live ? map->out_coef[a] : 0;
    }
    for (int l = 0; l < EMMYB200_CT_MAX_LOOPS; ++l) {
        const bool live = l < map->n_loops;
        m.loop_extent[l] = live ? map->loop_extent[l] : 1;
        m.a_loop[l] = live ? map->a_loop_coef[l] : 0;
        m.b_loop[l] = live ? map->b_loop_coef[l] : 0;
    }
    m.a_offset = map->a_offset; m.b_offset = map->b_offset; m.out_offset = map->out_offset;
    m.narrow = narrow ? 1 : 0;
    long long count = n;
    void* args[] = {&A, &B, &out, &count, &m};
    const int64_t want = (n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(kern.kernel), dim3(blocks), dim3(256), args, 0, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return cuda_fail(e, "launch of the indexed contraction kernel");
    return EMMYB200_OK;
}

extern "C" int emmyb200_contract_indexed_compile(const emmyb200_contraction_map* map, int64_t* code_bytes) {
    using namespace emmy;
    int rc = check_contraction(map, "contract_indexed_compile");
    if (rc != EMMYB200_OK) return rc;
    std::vector<char> cubin;
    rc = compile_source(contraction_source(*map), &cubin);
    if (rc == EMMYB200_OK && code_bytes != nullptr) *code_bytes = (int64_t)cubin.size();
    return rc;
}

extern "C" int emmyb200_pointwise_indexed_compile(const emmyb200_pw_program* prog, const emmyb200_pw_index_map* map, int64_t* code_bytes) {
    using namespace emmy;
    if (map == nullptr || map->n_axes < 1 || map->n_axes > EMMYB200_PW_MAX_AXES) return fail(EMMYB200_ERR_ARG, "pointwise_indexed_compile: bad index map");
    int rc = check_program(prog, "pointwise_indexed_compile", map);
    if (rc != EMMYB200_OK) return rc;
    emmyb200_pw_index_map key_map = *map;
    bool special = false;
    for (int k = 0; k < EMMYB200_PW_MAX_INPUTS; ++k) {
        key_map.in_kind[k] = k < prog->n_inputs ? map->in_kind[k] : 0;
        if (k < prog->n_inputs && (map->in_kind[k] == 2 || map->in_kind[k] == 3 || map->in_kind[k] == 4)) special = true;
        if (k < prog->n_inputs && map->in_kind[k] == 2 && (map->in_index_of[k] < 0 || map->in_index_of[k] >= prog->n_inputs || map->in_kind[map->in_index_of[k]] != 3))
            return fail(EMMYB200_ERR_ARG, "pointwise_indexed_compile: input %d takes its index from no index source", k);
        for (int a = 0; k < prog->n_inputs && a < map->n_axes; ++a) special = special || map->in_rot[k][a] != 0;
    }
    if (special) {
        IndexedForm form;
        form.special = 1;
        const int modes0[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};
        std::vector<char> code;
        rc = compile_source(program_source(*prog, 0, modes0, &key_map, &form), &code);
        if (rc == EMMYB200_OK && code_bytes != nullptr) *code_bytes = (int64_t)code.size();
        return rc;
    }
    const int modes[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};
    std::vector<char> cubin;
    rc = compile_source(program_source(*prog, 0, modes, &key_map), &cubin);
    if (rc != EMMYB200_OK) return rc;
    if (map->extent[map->n_axes - 1] % 4 == 0) {          // the grouped form, every buffer taken as vector-accessible
        IndexedForm form;
        form.inner = 4;
        form.ovec = 1;
        for (int k = 0; k < prog->n_inputs; ++k) form.ivec[k] = key_map.in_kind[k] == 0 ? 1 : 0;
        std::vector<char> grouped;
        rc = compile_source(program_source(*prog, 0, modes, &key_map, &form), &grouped);
        if (rc != EMMYB200_OK) return rc;
    }
    for (int variant = 0; variant < 4 && map->n_axes >= 2; ++variant) {    // the tiled transposition, axis 0 against the innermost axis
        IndexedForm form;
        form.transpose = 1;
        form.ttile = variant & 1 ? 64 : 32;
        form.swapped = variant >> 1;
        for (int k = 0; k < prog->n_inputs; ++k)
            if (key_map.in_kind[k] == 0) form.tin = k;
        std::vector<char> tiled;
        rc = compile_source(program_source(*prog, 0, modes, &key_map, &form), &tiled);
        if (rc != EMMYB200_OK) return rc;
    }
    if (code_bytes != nullptr) *code_bytes = (int64_t)cubin.size();
    return EMMYB200_OK;
}

extern "C" int emmyb200_set_pointwise_jit(int enabled) {
    const bool before = emmy::jit_enabled();
    emmy::g_jit_enabled.store(enabled ? 1 : 0, std::memory_order_relaxed);
    return before ? 1 : 0;
}

extern "C" int emmyb200_pointwise_jit_state(int64_t* kernels_compiled) {
    if (kernels_compiled != nullptr) *kernels_compiled = emmy::g_jit_compiles.load();
    if (!emmy::jit_enabled()) return 0;
    return emmy::nvrtc().ok ? 1 : -1;
}

extern "C" int64_t emmyb200_pointwise_program_source(const emmyb200_pw_program* prog, int group, char* text, int64_t capacity) {
    using namespace emmy;
    if (prog == nullptr || prog->n_inputs < 1 || prog->n_inputs > EMMYB200_PW_MAX_INPUTS || prog->n_steps < 0 ||
        prog->n_steps > EMMYB200_PW_MAX_STEPS || prog->out_slot < 0 || prog->out_slot >= EMMYB200_PW_MAX_SLOTS)
        return fail(EMMYB200_ERR_ARG, "pointwise_program_source: not a program (inputs, steps or output slot out of range)");
    if (!float_program(*prog) && prog->out_dtype != EMMYB200_I32 && prog->out_dtype != EMMYB200_I64)
        return fail(EMMYB200_ERR_UNSUPPORTED, "pointwise_program_source: output dtype %d", prog->out_dtype);
    if (!float_program(*prog) && group == 8) return fail(EMMYB200_ERR_ARG, "pointwise_program_source: integer programs use groups of 4");
    for (int i = 0; i < prog->n_steps; ++i) {
        const emmyb200_pw_step& st = prog->steps[i];
        if (st.op >= EMMYB200_PW_OP_COUNT || st.dst >= EMMYB200_PW_MAX_SLOTS) return fail(EMMYB200_ERR_ARG, "pointwise_program_source: bad step %d", i);
        for (int o : {st.a, st.b, st.c})
            if (o >= EMMYB200_PW_MAX_SLOTS + EMMYB200_PW_MAX_CONSTS) return fail(EMMYB200_ERR_ARG, "pointwise_program_source: bad operand in step %d", i);
    }
    if (group != 0 && group != 4 && group != 8) return fail(EMMYB200_ERR_ARG, "pointwise_program_source: group %d (0, 4 or 8)", group);
    int modes[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};
    for (int i = 0; i < prog->n_inputs; ++i) modes[i] = broadcast_mode(*prog, i, group, true);
    const std::string s = program_source(*prog, group, modes);
    if (text != nullptr && capacity > 0) {
        const size_t m = (size_t)capacity - 1 < s.size() ? (size_t)capacity - 1 : s.size();
        memcpy(text, s.data(), m);
        text[m] = 0;
    }
    return (int64_t)s.size() + 1;
}

extern "C" int emmyb200_pointwise_program_compile(const emmyb200_pw_program* prog, int group, int64_t* code_bytes) {
    using namespace emmy;
    const int64_t need = emmyb200_pointwise_program_source(prog, group, nullptr, 0);
    if (need < 0) return (int)need;
    std::vector<char> cubin;
    int modes[EMMYB200_PW_MAX_INPUTS] = {0, 0, 0, 0};
    for (int i = 0; i < prog->n_inputs; ++i) modes[i] = broadcast_mode(*prog, i, group, true);
    const int rc = compile_source(program_source(*prog, group, modes), &cubin);
    if (rc == EMMYB200_OK && code_bytes != nullptr) *code_bytes = (int64_t)cubin.size();
    return rc;
}
