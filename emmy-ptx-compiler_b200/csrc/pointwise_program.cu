// General elementwise kernel: y[i] = f(x0[i], x1[i], ...) for a straight-line program of ops from the
// reference's elementwise table (emmyptx/ops.py:212-290, `lower_op`).
//
// The reference prints the instructions of each `Assign` into the kernel it is compiling
// (emmyptx/kernel.py:766-784). Here the cell program travels as data: up to 48 steps `dst = op(a, b, c)` over
// 16 value slots, operands being slots or constants. A program is normally compiled into a kernel of its own at
// first use (pointwise_jit.cu); this file holds the entry point and the interpreters that run a program when the
// run-time compiler is not there. One CTA-wide interpreter
// loop runs it -- the control flow is the same for every thread, so there is no divergence -- with the slots
// held per thread as float4 (four elements at a time, 128-bit global accesses, 16-bit inputs and outputs
// widened / rounded once at the ends, as emmyptx/kernel.py:693-712 does).
// exp, sin, cos and tanh are the library's own <= 2 ulp functions; log, erf, pow, sqrt and the divisions use
// CUDA's device math functions (1-2 ulp), well inside the reference's 1e-5 class for these ops.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "emmy_math.cuh"
#include "pointwise_jit.h"

namespace emmy {

constexpr int kPwThreads = 256;
constexpr int kPwSlots = EMMYB200_PW_MAX_SLOTS;
constexpr int kPwUnroll = 2;

// One scalar op; `op` is uniform across the CTA, so the switch never diverges.
__device__ __forceinline__ float pw_apply(int op, float a, float b, float c) {
    switch (op) {
        case EMMYB200_PW_ADD: return __fadd_rn(a, b);
        case EMMYB200_PW_SUB: return __fsub_rn(a, b);
        case EMMYB200_PW_MUL: return __fmul_rn(a, b);
        case EMMYB200_PW_DIV: return __fdiv_rn(a, b);
        case EMMYB200_PW_MAX: return fmaxf(a, b);
        case EMMYB200_PW_MIN: return fminf(a, b);
        case EMMYB200_PW_RELU: return fmaxf(a, 0.0f);
        case EMMYB200_PW_SQUARE: return __fmul_rn(a, a);
        case EMMYB200_PW_COPY: return a;
        case EMMYB200_PW_NEG: return -a;
        case EMMYB200_PW_ABS: return fabsf(a);
        case EMMYB200_PW_RCP: return __frcp_rn(a);
        case EMMYB200_PW_SQRT: return __fsqrt_rn(a);
        case EMMYB200_PW_RSQRT: return __frcp_rn(__fsqrt_rn(a));       // as the reference: sqrt.rn then rcp.rn (ops.py:249-252)
        case EMMYB200_PW_EXP: return emmy_expf(a);
        case EMMYB200_PW_LOG: return logf(a);
        case EMMYB200_PW_SIGMOID: return __frcp_rn(__fadd_rn(1.0f, emmy_expf(-a)));
        case EMMYB200_PW_TANH: return emmy_tanhf(a);
        case EMMYB200_PW_ERF: return erff(a);
        case EMMYB200_PW_SIN: return emmy_sinf(a);
        case EMMYB200_PW_COS: return emmy_cosf(a);
        case EMMYB200_PW_POW: return powf(a, b);
        case EMMYB200_PW_EQ: return a == b ? 1.0f : 0.0f;
        case EMMYB200_PW_NE: return a != b ? 1.0f : 0.0f;
        case EMMYB200_PW_GT: return a > b ? 1.0f : 0.0f;
        case EMMYB200_PW_LT: return a < b ? 1.0f : 0.0f;
        case EMMYB200_PW_GE: return a >= b ? 1.0f : 0.0f;
        case EMMYB200_PW_LE: return a <= b ? 1.0f : 0.0f;
        case EMMYB200_PW_WHERE: return a != 0.0f ? b : c;
        case EMMYB200_PW_AND: return (a != 0.0f && b != 0.0f) ? 1.0f : 0.0f;
        case EMMYB200_PW_OR: return (a != 0.0f || b != 0.0f) ? 1.0f : 0.0f;
        case EMMYB200_PW_NOT: return a == 0.0f ? 1.0f : 0.0f;
        case EMMYB200_PW_FLOORDIV: return floorf(__fdiv_rn(a, b));
        case EMMYB200_PW_MOD: return __fsub_rn(a, __fmul_rn(b, floorf(__fdiv_rn(a, b))));
        default: return a;
    }
}

template <typename T>
__device__ __forceinline__ float4 pw_load4(const void* base, int64_t v) {
    if constexpr (sizeof(T) == 4) {
        return __ldcs(reinterpret_cast<const float4*>(base) + v);
    } else {
        const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(base) + v);
        if constexpr (std::is_same<T, __half>::value) {
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            return make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            return make_float4(lo.x, lo.y, hi.x, hi.y);
        }
    }
}

__device__ __forceinline__ float pw_load1(const void* base, int dtype, int64_t i) {
    if (dtype == EMMYB200_F32) return reinterpret_cast<const float*>(base)[i];
    if (dtype == EMMYB200_U8) return reinterpret_cast<const uint8_t*>(base)[i] ? 1.0f : 0.0f;
    if (dtype == EMMYB200_F16) return __half2float(reinterpret_cast<const __half*>(base)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}

__device__ __forceinline__ void pw_store1(void* base, int dtype, int64_t i, float v) {
    if (dtype == EMMYB200_F32) reinterpret_cast<float*>(base)[i] = v;
    else if (dtype == EMMYB200_F16) reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
    else if (dtype == EMMYB200_U8) reinterpret_cast<uint8_t*>(base)[i] = v != 0.0f ? 1 : 0;          // a bool output
    else reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
}

// Index of the element input k supplies for output element i.
__device__ __forceinline__ int64_t pw_index(const emmyb200_pw_program& prog, int k, int64_t i) {
    if (prog.in_div[k] > 0) i /= prog.in_div[k];
    if (prog.in_mod[k] > 0) i %= prog.in_mod[k];
    return i;
}

struct PwArgs {
    const void* in[EMMYB200_PW_MAX_INPUTS];
    void* out;
    int64_t n;
};

// VEC: all buffers are aligned for 128-bit (fp32) / 64-bit (16-bit types) accesses of four elements.
// FAST: no step writes an input's slot, so inputs and forwarded results may stay in registers (see below).
constexpr uint8_t kPwStore = 1;       // step.reserved[1]: the result must also go to its slot
template <bool VEC, bool FAST>
__global__ void __launch_bounds__(kPwThreads, 3) pointwise_program_kernel(const __grid_constant__ emmyb200_pw_program prog, PwArgs args) {
    // Per-thread value slots, indexed by the program: they live in local memory, i.e. in L1 for the few slots a
    // program touches, and do not cap the number of resident threads the way a shared-memory file would. L1 traffic
    // is what bounds a naive interpreter (every step reads two or three slots and writes one), so values bypass the
    // slot file wherever the program's shape allows: the inputs stay in registers (picked by a uniform switch), the
    // result of a step is forwarded to the next step in registers, and a result is written to its slot only when a
    // later step (other than the next) or the output needs it -- the host marks those steps (kPwStore). A chain of
    // unary / binary ops, the usual shape of an activation function, then touches no local memory at all.
    float4 slots[kPwSlots][kPwUnroll];
    float4 in0[kPwUnroll], in1[kPwUnroll], in2[kPwUnroll], in3[kPwUnroll], acc[kPwUnroll];
    const int tid = threadIdx.x;
    const int64_t groups = VEC ? args.n / 4 : (args.n + 3) / 4;
    const int64_t stride = (int64_t)gridDim.x * kPwThreads;
    for (int64_t g0 = (int64_t)blockIdx.x * kPwThreads + tid; g0 < groups; g0 += stride * kPwUnroll) {
        // kPwUnroll groups of four elements per thread and trip: more bytes in flight, one dispatch per step for all
        for (int k = 0; k < prog.n_inputs; ++k) {
#pragma unroll
            for (int u = 0; u < kPwUnroll; ++u) {
                const int64_t g = g0 + u * stride;
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (g < groups && (prog.in_div[k] | prog.in_mod[k]) != 0) {     // a broadcast input: four gathered loads
                    const int64_t i = g * 4;
                    v.x = pw_load1(args.in[k], prog.in_dtype[k], pw_index(prog, k, i));
                    v.y = i + 1 < args.n ? pw_load1(args.in[k], prog.in_dtype[k], pw_index(prog, k, i + 1)) : 0.0f;
                    v.z = i + 2 < args.n ? pw_load1(args.in[k], prog.in_dtype[k], pw_index(prog, k, i + 2)) : 0.0f;
                    v.w = i + 3 < args.n ? pw_load1(args.in[k], prog.in_dtype[k], pw_index(prog, k, i + 3)) : 0.0f;
                } else if (g < groups) {
                    if constexpr (VEC) {
                        const int dt = prog.in_dtype[k];
                        if (dt == EMMYB200_U8) {
                            const uchar4 m = __ldcs(reinterpret_cast<const uchar4*>(args.in[k]) + g);
                            v = make_float4(m.x ? 1.0f : 0.0f, m.y ? 1.0f : 0.0f, m.z ? 1.0f : 0.0f, m.w ? 1.0f : 0.0f);
                        } else {
                            v = dt == EMMYB200_F32 ? pw_load4<float>(args.in[k], g)
                              : dt == EMMYB200_F16 ? pw_load4<__half>(args.in[k], g) : pw_load4<__nv_bfloat16>(args.in[k], g);
                        }
                    } else {
                        const int64_t i = g * 4;
                        v.x = pw_load1(args.in[k], prog.in_dtype[k], i);
                        v.y = i + 1 < args.n ? pw_load1(args.in[k], prog.in_dtype[k], i + 1) : 0.0f;
                        v.z = i + 2 < args.n ? pw_load1(args.in[k], prog.in_dtype[k], i + 2) : 0.0f;
                        v.w = i + 3 < args.n ? pw_load1(args.in[k], prog.in_dtype[k], i + 3) : 0.0f;
                    }
                }
                if (k == 0) in0[u] = v;
                else if (k == 1) in1[u] = v;
                else if (k == 2) in2[u] = v;
                else in3[u] = v;
                if (!FAST) slots[k][u] = v;
            }
        }
        int prev_dst = -1;
        for (int s = 0; s < prog.n_steps; ++s) {
            const emmyb200_pw_step st = prog.steps[s];
#pragma unroll
            for (int u = 0; u < kPwUnroll; ++u) {
                auto operand = [&](int o) {
                    if (o >= kPwSlots) { const float c = prog.consts[o - kPwSlots]; return make_float4(c, c, c, c); }
                    if (FAST) {
                        if (o == prev_dst) return acc[u];
                        if (o < prog.n_inputs) return o == 0 ? in0[u] : (o == 1 ? in1[u] : (o == 2 ? in2[u] : in3[u]));
                    }
                    return slots[o][u];
                };
                const float4 a = operand(st.a), b = operand(st.b), c = operand(st.c);
                float4 r;
                r.x = pw_apply(st.op, a.x, b.x, c.x);
                r.y = pw_apply(st.op, a.y, b.y, c.y);
                r.z = pw_apply(st.op, a.z, b.z, c.z);
                r.w = pw_apply(st.op, a.w, b.w, c.w);
                if (!FAST || (st.reserved[1] & kPwStore)) slots[st.dst][u] = r;
                acc[u] = r;
            }
            prev_dst = st.dst;
        }
#pragma unroll
        for (int u = 0; u < kPwUnroll; ++u) {
            const int64_t g = g0 + u * stride;
            if (g >= groups) continue;
            const int os = prog.out_slot;
            const float4 y = !FAST ? slots[os][u]
                                   : (os == prev_dst ? acc[u] : (os < prog.n_inputs ? (os == 0 ? in0[u] : (os == 1 ? in1[u] : (os == 2 ? in2[u] : in3[u]))) : slots[os][u]));
            if constexpr (VEC) {
                if (prog.out_dtype == EMMYB200_F32) {
                    __stcs(reinterpret_cast<float4*>(args.out) + g, y);
                } else if (prog.out_dtype == EMMYB200_F16) {
                    const __half2 lo = __floats2half2_rn(y.x, y.y), hi = __floats2half2_rn(y.z, y.w);
                    __stcs(reinterpret_cast<uint2*>(args.out) + g, make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi)));
                } else if (prog.out_dtype == EMMYB200_U8) {
                    const uint32_t w = (y.x != 0.0f ? 1u : 0u) | (y.y != 0.0f ? 0x100u : 0u) | (y.z != 0.0f ? 0x10000u : 0u) | (y.w != 0.0f ? 0x1000000u : 0u);
                    __stcs(reinterpret_cast<uint32_t*>(args.out) + g, w);
                } else {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                    __stcs(reinterpret_cast<uint2*>(args.out) + g, make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi)));
                }
            } else {
                const int64_t i = g * 4;
                pw_store1(args.out, prog.out_dtype, i, y.x);
                if (i + 1 < args.n) pw_store1(args.out, prog.out_dtype, i + 1, y.y);
                if (i + 2 < args.n) pw_store1(args.out, prog.out_dtype, i + 2, y.z);
                if (i + 3 < args.n) pw_store1(args.out, prog.out_dtype, i + 3, y.w);
            }
        }
    }
    // the last n % 4 elements of the vector form: one thread, scalar accesses
    if constexpr (VEC) {
        const int tail = (int)(args.n & 3);
        if (blockIdx.x == 0 && tid < tail) {
            const int64_t i = (args.n & ~(int64_t)3) + tid;
            float regs[kPwSlots];
            for (int k = 0; k < prog.n_inputs; ++k) regs[k] = pw_load1(args.in[k], prog.in_dtype[k], pw_index(prog, k, i));
            for (int s = 0; s < prog.n_steps; ++s) {
                const emmyb200_pw_step st = prog.steps[s];
                auto operand = [&](int o) { return o >= kPwSlots ? prog.consts[o - kPwSlots] : regs[o]; };
                regs[st.dst] = pw_apply(st.op, operand(st.a), operand(st.b), operand(st.c));
            }
            pw_store1(args.out, prog.out_dtype, i, regs[prog.out_slot]);
        }
    }
}

// ---- integer programs: 32-bit two's complement values, one element per thread and trip ----------------------------
__device__ __forceinline__ int pw_apply_int(int op, int a, int b, int c, int trunc) {
    const unsigned ua = (unsigned)a, ub = (unsigned)b;
    switch (op) {
        case EMMYB200_PW_ADD: return (int)(ua + ub);
        case EMMYB200_PW_SUB: return (int)(ua - ub);
        case EMMYB200_PW_MUL: return (int)(ua * ub);
        case EMMYB200_PW_MAX: return max(a, b);
        case EMMYB200_PW_MIN: return min(a, b);
        case EMMYB200_PW_RELU: return max(a, 0);
        case EMMYB200_PW_SQUARE: return (int)(ua * ua);
        case EMMYB200_PW_NEG: return (int)(0u - ua);
        case EMMYB200_PW_ABS: return a < 0 ? (int)(0u - ua) : a;
        case EMMYB200_PW_EQ: return a == b;
        case EMMYB200_PW_NE: return a != b;
        case EMMYB200_PW_GT: return a > b;
        case EMMYB200_PW_LT: return a < b;
        case EMMYB200_PW_GE: return a >= b;
        case EMMYB200_PW_LE: return a <= b;
        case EMMYB200_PW_WHERE: return a != 0 ? b : c;
        case EMMYB200_PW_AND: return a & b;
        case EMMYB200_PW_OR: return a | b;
        case EMMYB200_PW_NOT: return ~a;
        case EMMYB200_PW_XOR: return a ^ b;
        case EMMYB200_PW_SHL: return (int)(ua << (ub & 31u));
        case EMMYB200_PW_SHR: return a >> (ub & 31u);
        case EMMYB200_PW_DIV:
        case EMMYB200_PW_FLOORDIV: {
            if (b == 0) return 0;
            if (b == -1) return (int)(0u - ua);                 // INT_MIN / -1 wraps
            int q = a / b;
            if (!trunc && (a % b != 0) && ((a < 0) != (b < 0))) --q;
            return q;
        }
        case EMMYB200_PW_MOD: {
            if (b == 0 || b == -1) return 0;
            int r = a % b;
            if (!trunc && r != 0 && ((r < 0) != (b < 0))) r += b;
            return r;
        }
        default: return a;                                      // COPY
    }
}

__device__ __forceinline__ int pw_load_int(const void* base, int dtype, int64_t i) {
    return dtype == EMMYB200_I32 ? reinterpret_cast<const int*>(base)[i] : (int)reinterpret_cast<const long long*>(base)[i];
}

__global__ void __launch_bounds__(kPwThreads) pointwise_program_int_kernel(const __grid_constant__ emmyb200_pw_program prog, PwArgs args) {
    const int64_t stride = (int64_t)gridDim.x * kPwThreads;
    for (int64_t i = (int64_t)blockIdx.x * kPwThreads + threadIdx.x; i < args.n; i += stride) {
        int regs[kPwSlots];
        for (int k = 0; k < prog.n_inputs; ++k) regs[k] = pw_load_int(args.in[k], prog.in_dtype[k], pw_index(prog, k, i));
        for (int s = 0; s < prog.n_steps; ++s) {
            const emmyb200_pw_step st = prog.steps[s];
            auto operand = [&](int o) { return o >= kPwSlots ? (int)prog.consts[o - kPwSlots] : regs[o]; };
            regs[st.dst] = pw_apply_int(st.op, operand(st.a), operand(st.b), operand(st.c), st.reserved[0]);
        }
        const int y = regs[prog.out_slot];
        if (prog.out_dtype == EMMYB200_I32) reinterpret_cast<int*>(args.out)[i] = y;
        else reinterpret_cast<long long*>(args.out)[i] = (long long)y;
    }
}

static int elem_size(int dtype) {
    return dtype == EMMYB200_F32 || dtype == EMMYB200_I32 ? 4 : (dtype == EMMYB200_I64 ? 8 : (dtype == EMMYB200_U8 ? 1 : 2));
}

}  // namespace emmy

extern "C" int emmyb200_pointwise_program(const emmyb200_pw_program* prog, const void* const* inputs, void* out, int64_t n,
                                          void* cuda_stream) {
    using namespace emmy;
    if (prog == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise_program: null program");
    if (prog->n_inputs < 1 || prog->n_inputs > EMMYB200_PW_MAX_INPUTS) return fail(EMMYB200_ERR_ARG, "pointwise_program: %d inputs (1 to %d)", prog->n_inputs, EMMYB200_PW_MAX_INPUTS);
    if (prog->n_steps < 0 || prog->n_steps > EMMYB200_PW_MAX_STEPS) return fail(EMMYB200_ERR_ARG, "pointwise_program: %d steps (0 to %d)", prog->n_steps, EMMYB200_PW_MAX_STEPS);
    if (prog->out_slot < 0 || prog->out_slot >= kPwSlots) return fail(EMMYB200_ERR_ARG, "pointwise_program: output slot %d", prog->out_slot);
    const bool int_program = prog->out_dtype == EMMYB200_I32 || prog->out_dtype == EMMYB200_I64;
    auto float_ok = [](int d) { return d == EMMYB200_F32 || d == EMMYB200_F16 || d == EMMYB200_BF16; };
    auto int_ok = [](int d) { return d == EMMYB200_I32 || d == EMMYB200_I64; };
    if (!int_program && !float_ok(prog->out_dtype) && prog->out_dtype != EMMYB200_U8)
        return fail(EMMYB200_ERR_UNSUPPORTED, "pointwise_program: output dtype %d", prog->out_dtype);
    for (int k = 0; k < prog->n_inputs; ++k) {
        const int d = prog->in_dtype[k];
        if (int_program ? !int_ok(d) : !(float_ok(d) || d == EMMYB200_U8))
            return fail(EMMYB200_ERR_UNSUPPORTED, "pointwise_program: input %d has dtype %d (%s program)", k, d, int_program ? "an integer" : "a float");
    }
    for (int s = 0; s < prog->n_steps; ++s) {
        const emmyb200_pw_step& st = prog->steps[s];
        if (st.op >= EMMYB200_PW_OP_COUNT) return fail(EMMYB200_ERR_ARG, "pointwise_program: step %d has unknown op %d", s, st.op);
        if (st.dst >= kPwSlots) return fail(EMMYB200_ERR_ARG, "pointwise_program: step %d writes slot %d", s, st.dst);
        for (int o : {st.a, st.b, st.c})
            if (o >= kPwSlots + EMMYB200_PW_MAX_CONSTS) return fail(EMMYB200_ERR_ARG, "pointwise_program: step %d reads operand %d", s, o);
    }
    if (n < 0) return fail(EMMYB200_ERR_SHAPE, "pointwise_program: n = %lld is negative", (long long)n);
    if (n == 0) return EMMYB200_OK;
    if (inputs == nullptr || out == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise_program: null buffer");
    PwArgs args;
    bool vec = aligned(out, 4 * elem_size(prog->out_dtype));
    if (!aligned(out, elem_size(prog->out_dtype))) return fail(EMMYB200_ERR_ALIGN, "pointwise_program: misaligned output");
    for (int k = 0; k < EMMYB200_PW_MAX_INPUTS; ++k) args.in[k] = nullptr;
    for (int k = 0; k < prog->n_inputs; ++k) {
        if (inputs[k] == nullptr) return fail(EMMYB200_ERR_ARG, "pointwise_program: null buffer");
        if (!aligned(inputs[k], elem_size(prog->in_dtype[k]))) return fail(EMMYB200_ERR_ALIGN, "pointwise_program: misaligned input %d", k);
        if (prog->in_div[k] < 0 || prog->in_mod[k] < 0) return fail(EMMYB200_ERR_ARG, "pointwise_program: negative broadcast extent for input %d", k);
        if ((prog->in_div[k] | prog->in_mod[k]) == 0) vec = vec && aligned(inputs[k], 4 * elem_size(prog->in_dtype[k]));
        args.in[k] = inputs[k];
    }
    args.out = out;
    args.n = n;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    const int64_t groups = (n + 3) / 4;
    const int64_t want = (groups + kPwThreads * kPwUnroll - 1) / (kPwThreads * kPwUnroll);
    const int64_t cap = (int64_t)sm_count() * 8;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    // A program runs as a kernel compiled for it (pointwise_jit.cu); the interpreters below take over where
    // that form is switched off or the run-time compiler is missing.
    {
        // groups of 8 elements when a 16-bit or byte buffer takes part and every buffer is aligned for it
        bool narrow = elem_size(prog->out_dtype) < 4, vec8 = aligned(out, 8 * elem_size(prog->out_dtype));
        for (int k = 0; k < prog->n_inputs; ++k) {
            if ((prog->in_div[k] | prog->in_mod[k]) != 0) continue;
            narrow = narrow || elem_size(prog->in_dtype[k]) < 4;
            vec8 = vec8 && aligned(inputs[k], 8 * elem_size(prog->in_dtype[k]));
        }
        const int rc = pw_jit_launch(*prog, args.in, out, n, vec ? (narrow && vec8 ? 8 : 4) : 0, s);
        if (rc != kPwJitUnavailable) return rc;
    }
    if (int_program) {
        const int64_t want_i = (n + kPwThreads - 1) / kPwThreads;
        pointwise_program_int_kernel<<<(unsigned)(want_i < cap ? want_i : cap), kPwThreads, 0, s>>>(*prog, args);
        return launch_status("pointwise_program_int_kernel");
    }
    // Which results must reach the slot file: those read by a step other than the next one before they are overwritten,
    // or (the last definition of the output slot, unless it is the last step) by the store. Inputs stay in registers
    // as long as no step writes their slots.
    emmyb200_pw_program marked = *prog;
    bool fast = true;
    for (int i = 0; i < marked.n_steps; ++i) {
        const int dst = marked.steps[i].dst;
        if (dst < marked.n_inputs) fast = false;
        bool needed = false;
        for (int j = i + 1; j < marked.n_steps; ++j) {
            const emmyb200_pw_step& later = marked.steps[j];
            if (j > i + 1 && (later.a == dst || later.b == dst || later.c == dst)) needed = true;
            if (later.dst == dst) { if (j == i + 1) {} break; }
            if (j == marked.n_steps - 1 && dst == marked.out_slot) needed = true;
        }
        marked.steps[i].reserved[1] = needed ? kPwStore : 0;
    }
    if (vec) {
        if (fast) pointwise_program_kernel<true, true><<<blocks, kPwThreads, 0, s>>>(marked, args);
        else pointwise_program_kernel<true, false><<<blocks, kPwThreads, 0, s>>>(marked, args);
    } else {
        if (fast) pointwise_program_kernel<false, true><<<blocks, kPwThreads, 0, s>>>(marked, args);
        else pointwise_program_kernel<false, false><<<blocks, kPwThreads, 0, s>>>(marked, args);
    }
    return launch_status("pointwise_program_kernel");
}
