/* emmyb200 -- C ABI of the sm_100a kernel library that stands in for the PTX entry points
 * emmyptx prints.
 *
 * In the reference a compiled kernel is a `.visible .entry <name>(.param .u64 buf, ...)` in PTX
 * text (emmyptx/kernel.py:130-155, parameters in meta.json's `arg_order`, :166-183), loaded and
 * launched with the CUDA driver API (tools/run_local.py:64-72, :100-102). Here the kernels are
 * precompiled; each entry point below takes the same caller-owned device buffers (plain
 * pointers, never retained), the extents the reference bakes into the PTX as constants, and
 * the CUDA stream to launch on (the reference always uses the NULL stream). Calls are
 * asynchronous: they enqueue work and return.
 *
 * Status: 0 = ok; < 0 = the arguments were rejected before anything was launched;
 * > 0 = the cudaError_t of a failed runtime call. `emmyb200_last_error()` gives the text
 * for the calling host thread. Nothing in the library traps, and every device-side wait is
 * bounded: a pipeline wait that gives up records where in a status word that
 * `emmyb200_device_status()` reads back (the reference's only device-side error path is a
 * `trap`, emmyptx/kernel.py:685-691).
 */
#ifndef EMMYB200_H
#define EMMYB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EMMYB200_OK 0
#define EMMYB200_ERR_ARG (-1)         /* null pointer, bad enum */
#define EMMYB200_ERR_SHAPE (-2)       /* extent the kernel family does not cover */
#define EMMYB200_ERR_ALIGN (-3)       /* pointer or leading dimension not aligned as required */
#define EMMYB200_ERR_UNSUPPORTED (-4) /* valid request, no kernel variant for it */
#define EMMYB200_ERR_DEVICE (-5)      /* not an sm_100 device */
#define EMMYB200_ERR_TIMEOUT (-6)     /* a bounded device-side wait expired (see device_status) */

/* Element types of buffers, named as in emmyptx/kernel.py:34-35 (`ELEM`). */
#define EMMYB200_F32 0
#define EMMYB200_F16 1
#define EMMYB200_BF16 2
#define EMMYB200_I32 3
#define EMMYB200_I64 4   /* integer programs only: computed in 32 bits, as the reference does (emmyptx/kernel.py:41) */
#define EMMYB200_U8 5    /* a bool / byte buffer of a float program: an input reads as 0 or 1, an output holds value != 0 */

int emmyb200_version(void);

/* Text of the last non-zero status on this host thread (never NULL). */
const char* emmyb200_last_error(void);

/* Unary fp32 ops of the elementwise table, emmyptx/ops.py:212-290 (`lower_op`), applied to a
 * flat array the way a one-axis `Tile` does (emmyptx/kernel.py:551-585): y[i] = op(x[i]).
 * EXP_SIN_TANH is the fused expression exp(x) + sin(x) * tanh(x). Each function is within
 * 2 ulp of the correctly rounded value for every fp32 input. x and y may be the same buffer. */
#define EMMYB200_OP_EXP_SIN_TANH 0
#define EMMYB200_OP_EXP 1
#define EMMYB200_OP_SIN 2
#define EMMYB200_OP_COS 3
#define EMMYB200_OP_TANH 4
#define EMMYB200_OP_GELU_TANH 5
#define EMMYB200_OP_SIGMOID 6     /* 1 / (1 + exp(-x)); tools/torch_cases/pointwise.py:17 */
#define EMMYB200_OP_SILU 7        /* x * sigmoid(x); pointwise.py:23 */
#define EMMYB200_OP_RELU 8        /* pointwise.py:19 */
int emmyb200_pointwise_f32(int op, const float* x, float* y, int64_t n, void* cuda_stream);

/* Any other straight-line elementwise expression over up to 4 same-sized inputs: the cell program of a
 * one-axis `Tile` (emmyptx/kernel.py:766-784 `visit_Assign` calling emmyptx/ops.py:212 `lower_op` once per
 * statement) handed over as data. Values are fp32 (the reference's only compute type, emmyptx/kernel.py:31-38);
 * f16 / bf16 buffers are widened on load and rounded once on store. A step computes
 * slot[dst] = op(operand a, b, c); an operand < EMMYB200_PW_MAX_SLOTS names a slot, otherwise constant
 * consts[operand - EMMYB200_PW_MAX_SLOTS]. Inputs arrive in slots 0 .. n_inputs-1; `out_slot` is stored.
 * Float programs may also read U8 buffers (bool masks, as 0 / 1). A program whose output is I32 or I64 is an integer
 * program (the s32 table of emmyptx/ops.py:294-309 and emmyptx/intmath.py): every buffer is I32 or I64, values are
 * 32-bit two's complement, AND / OR / NOT / XOR are bitwise, SHL / SHR shift (SHR arithmetically), constants are
 * the integers held in `consts`, and FLOORDIV / MOD round toward minus infinity unless the step's reserved[0] is 1
 * (toward zero, the reference's div.s32 / rem.s32). */
#define EMMYB200_PW_MAX_SLOTS 16
#define EMMYB200_PW_MAX_CONSTS 16
#define EMMYB200_PW_MAX_STEPS 48
#define EMMYB200_PW_MAX_INPUTS 4
enum {
    EMMYB200_PW_ADD, EMMYB200_PW_SUB, EMMYB200_PW_MUL, EMMYB200_PW_DIV, EMMYB200_PW_MAX, EMMYB200_PW_MIN,
    EMMYB200_PW_RELU, EMMYB200_PW_SQUARE, EMMYB200_PW_COPY, EMMYB200_PW_NEG, EMMYB200_PW_ABS, EMMYB200_PW_RCP,
    EMMYB200_PW_SQRT, EMMYB200_PW_RSQRT, EMMYB200_PW_EXP, EMMYB200_PW_LOG, EMMYB200_PW_SIGMOID, EMMYB200_PW_TANH,
    EMMYB200_PW_ERF, EMMYB200_PW_SIN, EMMYB200_PW_COS, EMMYB200_PW_POW, EMMYB200_PW_EQ, EMMYB200_PW_NE,
    EMMYB200_PW_GT, EMMYB200_PW_LT, EMMYB200_PW_GE, EMMYB200_PW_LE, EMMYB200_PW_WHERE, EMMYB200_PW_AND,
    EMMYB200_PW_OR, EMMYB200_PW_NOT, EMMYB200_PW_FLOORDIV, EMMYB200_PW_MOD, EMMYB200_PW_XOR, EMMYB200_PW_SHL,
    EMMYB200_PW_SHR, EMMYB200_PW_OP_COUNT
};
typedef struct {
    uint8_t op, dst, a, b, c, reserved[3];
} emmyb200_pw_step;
typedef struct {
    int32_t n_inputs, n_steps, out_slot, out_dtype;
    int32_t in_dtype[EMMYB200_PW_MAX_INPUTS];
    float consts[EMMYB200_PW_MAX_CONSTS];
    emmyb200_pw_step steps[EMMYB200_PW_MAX_STEPS];
    /* Broadcast inputs: element i of the output reads element (i / in_div[k]) % in_mod[k] of input k (0 = that
     * step is skipped; both 0: element i, the default). in_mod = cols gives a row vector broadcast over a
     * [rows, cols] output (a bias, batch-norm statistics); in_div = cols a column vector (an outer product). */
    int64_t in_div[EMMYB200_PW_MAX_INPUTS];
    int64_t in_mod[EMMYB200_PW_MAX_INPUTS];
} emmyb200_pw_program;
int emmyb200_pointwise_program(const emmyb200_pw_program* program, const void* const* inputs, void* out,
                               int64_t n, void* cuda_stream);

/* How programs run. By default each distinct program shape (op sequence, operand wiring, dtypes, which inputs
 * are broadcast, vector or scalar accesses) is compiled once, at its first launch, into a kernel of its own -- the
 * counterpart of the reference printing the ops into the entry it compiles (emmyptx/kernel.py:766-784) -- by the
 * toolkit's run-time compiler (libnvrtc.so.12, looked up when first needed; EMMYB200_NVRTC names another file).
 * Constants and broadcast extents are launch arguments and do not compile again. The first launch of a shape takes
 * the compile time (a fraction of a second) and cannot be part of a stream capture. With the compiler missing, or
 * after emmyb200_set_pointwise_jit(0) (or EMMYB200_PW_JIT=0 in the environment), programs run on precompiled
 * interpreter kernels with the same results bit for bit (the sign and payload of a NaN aside), at a fraction of the
 * bandwidth.
 *   emmyb200_set_pointwise_jit      returns the previous setting (1 compiled, 0 interpreter).
 *   emmyb200_pointwise_jit_state    1 compiled form in use, 0 switched off, -1 wanted but the compiler could not be
 *                                   loaded; *kernels_compiled (may be NULL) counts the compilations so far.
 *   emmyb200_pointwise_program_source   the CUDA C++ text of the kernel for `program`; group = elements per thread and
 *                                   access: 4 (128-bit accesses of fp32 / i32), 8 (128-bit accesses of 16-bit types; float programs only), 0
 *                                   (scalar accesses, for unaligned buffers); returns the size needed including the
 *                                   terminator, or a negative status.
 *   emmyb200_pointwise_program_compile  compiles that text for sm_100a without launching (no device needed);
 *                                   *code_bytes (may be NULL) receives the size of the device code. */
int emmyb200_set_pointwise_jit(int enabled);
int emmyb200_pointwise_jit_state(int64_t* kernels_compiled);
int64_t emmyb200_pointwise_program_source(const emmyb200_pw_program* program, int group, char* text, int64_t capacity);
int emmyb200_pointwise_program_compile(const emmyb200_pw_program* program, int group, int64_t* code_bytes);

/* The same cell programs with index maps: a one-cell-per-element Tile whose Loads and Write address their buffers by
 * affine functions of the tile's axis variables -- the reference's data-movement cases (tools/torch_cases/shapes.py:6-19:
 * transpose, permute, slices, flip, repeat, expand, stack) and masks made from the axis variables themselves (tril:
 * shapes.py:19). The cell number is split into the digits of the axes (outermost first, last fastest, as
 * emmyptx/kernel.py:587-626 decodes `gid`); input k is element in_offset[k] + sum_a in_coef[k][a] * digit[a] of its
 * buffer (in_kind 0), or the value of digit in_axis[k] itself with no buffer behind it (in_kind 1; inputs[k] unused; kinds 2
 * and 3, below, address a buffer through an index read from another one); the
 * result is stored at out_offset + sum_a out_coef[a] * digit[a]. The program's in_div / in_mod are ignored. Nothing
 * here can check an index against a buffer's size: the caller does (the facade checks every map's range against the
 * tensor shapes); a map that reaches a negative element is refused. Always a compiled kernel (see above); without the
 * run-time compiler the call answers EMMYB200_ERR_UNSUPPORTED. The kernel takes one of three forms: 32 x 32
 * shared-memory tiles when the one buffer input is contiguous along another axis than the innermost and the output
 * along the innermost (a transposition: both sides coalesced); groups of four cells with 128-bit accesses where a map
 * advances one element per cell from a 4-aligned start (slices, flips, concatenations); one cell per thread otherwise. */
#define EMMYB200_PW_MAX_AXES 6
typedef struct {
    int32_t n_axes, reserved;
    int64_t extent[EMMYB200_PW_MAX_AXES];
    int32_t in_kind[EMMYB200_PW_MAX_INPUTS];
    int32_t in_axis[EMMYB200_PW_MAX_INPUTS];
    int64_t in_offset[EMMYB200_PW_MAX_INPUTS];
    int64_t in_coef[EMMYB200_PW_MAX_INPUTS][EMMYB200_PW_MAX_AXES];
    int64_t out_offset;
    int64_t out_coef[EMMYB200_PW_MAX_AXES];
    /* Rotations (torch.roll, shapes.py:16): the digit of axis a enters input k's map as (digit + in_rot[k][a]) mod extent[a];
     * 0 <= in_rot < extent. */
    int64_t in_rot[EMMYB200_PW_MAX_INPUTS][EMMYB200_PW_MAX_AXES];
    /* Indices taken from data (embedding, gather: shapes.py:20-24). An input of in_kind 3 is an index source: an I32 / I64
     * buffer read through its own affine map, made non-negative (in_index_abs) and reduced modulo in_index_mod (required:
     * the modulus is what bounds the index; the remainder is the non-negative one); no step may read it as a value. An
     * input of in_kind 2 is a buffer whose element index is its affine map plus in_index_mult[k] times the value of index
     * source in_index_of[k].
     * An input of in_kind 4 is a guarded read (a Load inside a `Cond` on the axis variables, emmyptx/kernel.py:825-840: the
     * two halves of a concatenation, a padded border): its affine index is clamped into [0, in_index_mod[k]) -- the
     * buffer's element count -- so the map may leave the buffer in cells whose value the program does not select. */
    int32_t in_index_of[EMMYB200_PW_MAX_INPUTS];
    int32_t in_index_abs[EMMYB200_PW_MAX_INPUTS];
    int64_t in_index_mod[EMMYB200_PW_MAX_INPUTS];
    int64_t in_index_mult[EMMYB200_PW_MAX_INPUTS];
} emmyb200_pw_index_map;
int emmyb200_pointwise_indexed(const emmyb200_pw_program* program, const emmyb200_pw_index_map* map,
                               const void* const* inputs, void* out, void* cuda_stream);
/* Compiles the kernel of an indexed program for sm_100a without launching it (no device needed). */
int emmyb200_pointwise_indexed_compile(const emmyb200_pw_program* program, const emmyb200_pw_index_map* map, int64_t* code_bytes);

/* Contractions over nested loops with affine maps: a one-cell-per-output Tile whose body is up to three nested Loops
 * folding A[...] * B[...] into an accumulator (emmyptx/kernel.py:786-797, emmyptx/loops.py:70-90) -- the reference's
 * convolutions (tools/torch_cases/conv.py:6-7) and any other sum of products that is not a plain matrix product. The
 * output cell's digits (as for emmyb200_pointwise_indexed) and the loops' counters address A and B through affine maps;
 * terms are folded in loop order, one fused multiply-add each, in fp32; the result is rounded once to out_dtype and
 * stored through the output map. One cell per thread, on the CUDA cores: sized for the reference's cases (48 to 72
 * terms per output), not a tensor-core convolution. Always a kernel compiled at first use. */
#define EMMYB200_CT_MAX_LOOPS 3
typedef struct {
    int32_t n_axes, n_loops;
    int64_t extent[EMMYB200_PW_MAX_AXES];           /* tile axes, outermost first */
    int64_t loop_extent[EMMYB200_CT_MAX_LOOPS];     /* reduction axes, outermost first */
    int64_t a_offset, a_coef[EMMYB200_PW_MAX_AXES], a_loop_coef[EMMYB200_CT_MAX_LOOPS];
    int64_t b_offset, b_coef[EMMYB200_PW_MAX_AXES], b_loop_coef[EMMYB200_CT_MAX_LOOPS];
    int64_t out_offset, out_coef[EMMYB200_PW_MAX_AXES];
    int32_t a_dtype, b_dtype, out_dtype, reserved;  /* EMMYB200_F32 / F16 / BF16 */
} emmyb200_contraction_map;
int emmyb200_contract_indexed(const emmyb200_contraction_map* map, const void* A, const void* B, void* out, void* cuda_stream);
int emmyb200_contract_indexed_compile(const emmyb200_contraction_map* map, int64_t* code_bytes);

/* The int32 index-math gather
 *     y[i] = (x[(i * mul + add) mod n] div d) xor (i >> shift),   0 <= i < n,
 * i.e. the s32 instruction stream of emmyptx/intmath.py:36-38, :87-117 and
 * emmyptx/ops.py:294-309 around one gathered load (emmyptx/kernel.py:632-677).
 * The index is the mathematical (i * mul + add) mod n, which for a power-of-two n equals
 * the wrapped-int32 value the reference masks with n - 1. `div` rounds toward minus infinity
 * (torch's `//`, tools/torch_cases/dtypes.py:17-19) unless EMMYB200_GATHER_TRUNC is set, which
 * gives the reference PTX's `div.s32` (toward zero). Requires n >= 1, n < 2^31, 0 <= mul,
 * 0 <= add, d >= 1, 0 <= shift <= 31; x and y must not overlap. */
#define EMMYB200_GATHER_TRUNC 1
int emmyb200_index_gather_i32(const int32_t* x, int32_t* y, int64_t n, int64_t mul, int64_t add,
                              int32_t d, int32_t shift, int32_t flags, void* cuda_stream);

/* C[M,N] = epilogue(A[M,K] . B) with fp32 accumulation and one rounding to the output type,
 * replacing the RegFragment / LdmatrixLoad / MmaSyncPtx / RegStore statement family
 * (emmyptx/mma.py:65-242). A is row-major with leading dimension lda. B is row-major K x N
 * (ldb >= N) or, with EMMYB200_GEMM_B_NK, row-major N x K (`b_trans`, emmyptx/mma.py:112-113;
 * ldb >= K). dtype (F16 or BF16) is the type of A, B and C. Epilogues: NONE, or GELU_TANH =
 * 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) on the fp32 accumulator -- the fusion the
 * reference refuses (emmyptx/mma.py:201-203). Any M, N, K >= 1; pointers 16-byte aligned and
 * leading dimensions multiples of 8 elements. */
#define EMMYB200_EPI_NONE 0
#define EMMYB200_EPI_GELU_TANH 1
#define EMMYB200_EPI_RELU 2
#define EMMYB200_GEMM_B_NK 1
#define EMMYB200_GEMM_DST_MULTICAST 2   /* emmyb200_gemm_allgather only, see there */
#define EMMYB200_GEMM_OUT_F32 4         /* C (and the bias of emmyb200_gemm_batched) is fp32: the accumulator stored without
                                         * narrowing, which is also what the reference's split-K store (red.add.f32 into a
                                         * zeroed f32 C, emmyptx/mma.py:205-242) adds up to; C is overwritten, ldc and
                                         * stride_c count fp32 elements (multiples of 4); one destination */
int emmyb200_gemm(int dtype, int epilogue, int flags, const void* A, const void* B, void* C,
                  int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                  void* cuda_stream);

/* `batch` independent products with one launch (the reference's batched and broadcast matmul cases,
 * tools/torch_cases/matmul.py:11-12, :31): plane b of A (stride_a elements apart) times plane b of B
 * (stride_b apart; stride_b = 0 shares one B) into plane b of C (stride_c apart). `bias`, if not NULL, holds N
 * values of the output type added to every row of the fp32 accumulator before the epilogue function
 * (F.linear's bias, matmul.py:13-14); epilogues NONE, GELU_TANH, RELU. Other rules as emmyb200_gemm. */
int emmyb200_gemm_batched(int dtype, int epilogue, int flags, const void* A, const void* B, const void* bias,
                          void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                          int64_t ldb, int64_t ldc, int64_t stride_a, int64_t stride_b, int64_t stride_c,
                          void* cuda_stream);

/* fp32 in, fp32 out, fp32-accurate: the reference's float32 matmul cases (tools/torch_cases/matmul.py:10-16: mm, bmm,
 * broadcast, F.linear with bias, einsum), which it lowers to scalar FMA loops (emmyptx/kernel.py:786-797). Here each
 * operand is split into three bf16 planes (x = x1 + x2 + x3, 24 mantissa bits together) in `workspace`, and the six
 * products a_i b_j with i + j <= 4 run on the bf16 tensor-core path into one fp32 accumulator; the dropped terms
 * are below 2^-24 of a product, and the accumulator truncates once per 16-deep block, so the error is bounded by
 * about 2^-23 (8 + K / 16) sum_k |a_k b_k| (measured: 1e-7 .. 8e-7 of that sum for operands of random sign). Arguments as emmyb200_gemm_batched with float buffers (`bias`: N floats or NULL);
 * lda / ldb / strides of A and B are unrestricted, C must be 16-byte aligned with ldc (and stride_c) a multiple
 * of 4. `workspace`: emmyb200_gemm_f32_workspace_bytes(flags, batch, M, N, K, b_shared) bytes, 256-byte aligned
 * (b_shared = 1 when stride_b is 0 or batch is 1). Non-finite operands: an infinite element of A or B makes every
 * output element it contributes to NaN (the split meets inf * 0), where the reference's scalar fp32 loop gives +-inf;
 * NaN operands give NaN as there. Finite operands of any magnitude are handled (values beyond the bf16 range are
 * carried by the lower planes). No counterpart for the split itself in the reference. */
int64_t emmyb200_gemm_f32_workspace_bytes(int flags, int64_t batch, int64_t M, int64_t N, int64_t K, int b_shared);
int emmyb200_gemm_f32(int epilogue, int flags, const float* A, const float* B, const float* bias, float* C,
                      int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                      int64_t stride_a, int64_t stride_b, int64_t stride_c, void* workspace, int64_t workspace_bytes,
                      void* cuda_stream);

/* The same GEMM on one GPU's row shard of A, with every output piece stored to n_dst destination buffers
 * (1..8): C_dst[0] is this GPU's own C shard, the others are the addresses, valid on this GPU, of where the
 * same rows live in each peer's copy of the full C (peer-mapped device memory). Run by every GPU of a group
 * on its own rows, it leaves the complete C on all of them: the kernel's own TMA stores over NVLink take the
 * place of a separate all-gather. All destinations share ldc and alignment rules. The caller synchronises
 * the group before reading rows written by peers. With EMMYB200_GEMM_DST_MULTICAST, n_dst is 1 and C_dst[0] is the
 * address of this GPU's rows inside an NVSwitch multicast mapping of C (N a multiple of 8): every piece is then
 * stored once with multimem.st and the switch delivers it to all GPUs of the group, this one included, so the
 * GPU's outgoing NVLink traffic is its own shard instead of one copy per peer. No counterpart in the reference,
 * which is single-GPU (tools/run_local.py:51-57); it serves the row-sharded configuration of the benchmark. */
int emmyb200_gemm_allgather(int dtype, int epilogue, int flags, const void* A, const void* B, void* const* C_dst,
                            int n_dst, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                            void* cuda_stream);

/* O = softmax(Q K^T * scale) V per (batch, head) unit, fp32 softmax, non-causal: what the
 * reference emits as generic fused statements (dot-product Loops + Accum, WarpShuffle /
 * TreeHalve row reductions, `_exp`: emmyptx/kernel.py:786-797, :856-900, emmyptx/ops.py:49-77).
 * Q, O: [units, seq_q, d]; K, V: [units, seq_k, d]; contiguous, any seq_q, seq_k >= 1. dtype F16 or BF16 with d = 128
 * or 64 runs on the tensor cores (the benchmark configuration). dtype F32 -- the reference's own attention cases,
 * tools/torch_cases/fused.py:21-22, 31-36, models.py:17-19 -- and 16-bit buffers with another head size (d a
 * multiple of 32 up to 128) run on a CUDA-core kernel that keeps every product and sum in fp32, as the reference's
 * lowering does; it has one form, one destination and at most 65535 units. EMMYB200_ATT_CAUSAL: query i attends to keys 0..i only (the lower-triangular
 * mask of tools/torch_cases/models.py:17-19, fused.py:31-36). Two kernel forms exist -- one 128-query tile per
 * CTA with two CTAs sharing an SM, or two tiles per persistent CTA -- and the library picks by size (two tiles per CTA
 * when a unit has at least eight key tiles and there is a pair of query tiles for every SM: what was measured faster); EMMYB200_ATT_FORM_ONE_TILE / _TWO_TILES force one (tuning and tests; results agree within the
 * rounding of P). */
#define EMMYB200_ATT_CAUSAL 1
#define EMMYB200_ATT_DST_MULTICAST 2    /* emmyb200_attention_fwd_allgather only, see there */
#define EMMYB200_ATT_FORM_ONE_TILE 4
#define EMMYB200_ATT_FORM_TWO_TILES 8
int emmyb200_attention_fwd(int dtype, int flags, const void* Q, const void* K, const void* V, void* O,
                           int64_t units, int64_t seq_q, int64_t seq_k, int64_t d, float scale,
                           void* cuda_stream);

/* The same attention on one GPU's share of the units, every output tile stored to n_dst destinations
 * (1..8): O_dst[0] is this GPU's own slice of O, the others the addresses, valid on this GPU, of the same
 * slice inside each peer's full O. No counterpart in the reference (single GPU); it serves the
 * (batch x head)-sharded configuration. The caller synchronises the group before reading peers' units.
 * EMMYB200_ATT_DST_MULTICAST: n_dst = 1 and O_dst[0] is the multicast address of the slice (as for the GEMM). */
int emmyb200_attention_fwd_allgather(int dtype, int flags, const void* Q, const void* K, const void* V,
                                     void* const* O_dst, int n_dst, int64_t units, int64_t seq_q,
                                     int64_t seq_k, int64_t d, float scale, void* cuda_stream);

/* Reductions over the last axis of a contiguous fp32 [rows, cols] array and the normalisations built on them:
 * the kernels the reference assembles from per-thread `Accum` loops, `WarpShuffle` butterflies and `TreeHalve`
 * shared-memory trees (emmyptx/kernel.py:786-797, :856-900) for the cases of tools/torch_cases/reductions.py:6-19
 * and fused.py:6-13. Ops below EMMYB200_ROW_SOFTMAX store one value per row (y: float[rows]; ARGMAX:
 * int64_t[rows], first index of the maximum, NaN counting as the largest, as torch); the others store
 * y: float[rows, cols]. VAR and STD are the unbiased estimates (torch's default). LAYER_NORM is
 * (x - mean) / sqrt(biased var + eps) * weight + bias and RMS_NORM x / sqrt(mean(x^2) + eps) * weight, `weight`
 * and `bias` being float[cols] or NULL; NORMALIZE is x / max(||x||_2, eps); DOT needs `weight` (the vector). Other ops
 * take NULL for both.
 * Rows of more than 65536 elements are reduced in pieces by several thread blocks, which needs
 * emmyb200_rowwise_workspace_bytes(op, rows, cols) bytes of 256-byte-aligned device memory (contents
 * irrelevant before, undefined after; 0 for shorter rows, -1 for arguments the call would reject); results do
 * not depend on the order in which blocks finish. rows >= 0, 1 <= cols < 2^31. */
#define EMMYB200_ROW_SUM 0
#define EMMYB200_ROW_MEAN 1
#define EMMYB200_ROW_AMAX 2
#define EMMYB200_ROW_AMIN 3
#define EMMYB200_ROW_PROD 4
#define EMMYB200_ROW_VAR 5
#define EMMYB200_ROW_STD 6
#define EMMYB200_ROW_NORM2 7
#define EMMYB200_ROW_LOGSUMEXP 8
#define EMMYB200_ROW_ARGMAX 9
#define EMMYB200_ROW_COSINE 11   /* y[r] = x[r] . w[r] / max(||x[r]|| ||w[r]||, eps), `weight` a second float[rows, cols] (fused.py:16) */
#define EMMYB200_ROW_DOT 10      /* y[r] = sum_c x[r, c] * weight[c]: a matrix-vector product (tools/torch_cases/matmul.py:22) */
#define EMMYB200_ROW_SOFTMAX 16
#define EMMYB200_ROW_LOG_SOFTMAX 17
#define EMMYB200_ROW_LAYER_NORM 18
#define EMMYB200_ROW_RMS_NORM 19
#define EMMYB200_ROW_NORMALIZE 20
int64_t emmyb200_rowwise_workspace_bytes(int op, int64_t rows, int64_t cols);
int emmyb200_rowwise_f32(int op, const float* x, const float* weight, const float* bias, void* y, int64_t rows,
                         int64_t cols, float eps, void* workspace, int64_t workspace_bytes, void* cuda_stream);

/* The same reductions over the middle axis of a contiguous fp32 [outer, rows, cols] array (outer = 1: over dim 0 of a
 * matrix, tools/torch_cases/reductions.py:9, fused.py:7; a sum over several axes is a row pass followed by this
 * one, reductions.py:10). Ops: the reducing ones (y: float[outer, cols]; ARGMAX: int64_t[outer, cols], the row
 * index) and SOFTMAX, LOG_SOFTMAX, NORMALIZE (y: float[outer, rows, cols]). Tall arrays are cut into row slices
 * handled by different thread blocks, and mapping ops keep per-column statistics: both need
 * emmyb200_colwise_workspace_bytes(op, outer, rows, cols) bytes of 256-byte-aligned device memory (possibly 0;
 * -1 for arguments the call would reject). outer <= 65535, 1 <= rows, cols < 2^31. */
int64_t emmyb200_colwise_workspace_bytes(int op, int64_t outer, int64_t rows, int64_t cols);
int emmyb200_colwise_f32(int op, const float* x, void* y, int64_t outer, int64_t rows, int64_t cols, float eps,
                         void* workspace, int64_t workspace_bytes, void* cuda_stream);

/* y[r, c] = x[r, 0] + ... + x[r, c] over a contiguous fp32 [rows, cols] array (torch.cumsum(x, -1),
 * tools/torch_cases/reductions.py:18). x and y may be the same buffer. */
int emmyb200_cumsum_f32(const float* x, float* y, int64_t rows, int64_t cols, void* cuda_stream);

/* emmyb200_rowwise_f32 without a workspace argument and without any allocation: the scratch memory of long rows is
 * a fixed array inside the library's device image (emmyb200_rowwise_static_capacity() bytes per device). Shapes
 * whose emmyb200_rowwise_workspace_bytes() exceeds the capacity are rejected with EMMYB200_ERR_SHAPE; all others
 * behave exactly as emmyb200_rowwise_f32. Calls on one device share the array, so they must be ordered (one
 * stream, or events between streams). These two entry points have no counterpart in the reference, whose kernels
 * never use scratch memory beyond their own shared memory. */
int64_t emmyb200_rowwise_static_capacity(void);
int emmyb200_rowwise_f32_static(int op, const float* x, const float* weight, const float* bias, void* y, int64_t rows,
                                int64_t cols, float eps, void* cuda_stream);

/* Launches the kernel a handle names, from raw device pointers: the counterpart of `cuLaunchKernel` on the PTX entry
 * the reference prints (tools/run_local.py:94-102 builds one pointer per parameter of meta.json's `arg_order`,
 * emmyptx/kernel.py:166-183 declares buffers as `.param .u64` and scalars as `.param .f32 / .s32`). `handle_json` is the
 * text compile.py / compile_kernel printed; `params[i]` points at the value of the i-th name in the handle's
 * `arg_order`: at a device pointer (a `void*`) for a buffer, at a float or an int32_t for a scalar argument; n_params
 * must equal the length of `arg_order`. `workspace`: emmyb200_launch_workspace_bytes(handle_json) bytes of
 * 256-byte-aligned device memory (0 for most kernels: NULL then). The handle's shapes are the ones the kernel was
 * compiled for, as the reference bakes them into its PTX; nothing is retained; the call is asynchronous. */
int64_t emmyb200_launch_workspace_bytes(const char* handle_json);
int emmyb200_launch(const char* handle_json, void* const* params, int n_params, void* workspace, int64_t workspace_bytes,
                    void* cuda_stream);

/* Reads (and clears) the device status word of the current device into *status_out: 0 if no bounded wait has
 * expired since the last call, else a code naming kernel (bits 24-31: 1 GEMM, 2 attention), wait site (16-23)
 * and pipeline stage (0-15). Returns EMMYB200_OK with a zero word and EMMYB200_ERR_TIMEOUT with a non-zero one
 * (the outputs of the launches since the last clean read are then not to be trusted; the device and the library
 * stay usable). Synchronises the device. This replaces the reference's only device-side error path, a `trap`
 * that kills the context (emmyptx/kernel.py:685-691). */
int emmyb200_device_status(uint32_t* status_out);

/* The time after which a device-side pipeline wait gives up, for the launches that follow (process-wide; default
 * 2 s; 0 restores the default; 1 us .. 60 s). A watchdog setting: a healthy launch never waits anywhere near it.
 * No counterpart in the reference. */
int emmyb200_set_wait_limit_ns(uint64_t limit_ns);

/* Self-test of the give-up path: launches one small CTA whose first thread waits, through the same bounded wait as
 * every pipeline role of the tensor-core kernels, on a barrier that nothing arrives on, with `limit_ns` (1 us .. 1 s)
 * as the limit; waits for the stream; and returns EMMYB200_ERR_TIMEOUT when -- as it must -- the wait expired, set the
 * status word and raised the CTA's abort flag (EMMYB200_ERR_DEVICE if it did not). The status word stays set until
 * emmyb200_device_status reads it. Nothing faults or traps; the device stays usable. No counterpart in the
 * reference. */
int emmyb200_selftest_wait_expiry(uint64_t limit_ns, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* EMMYB200_H */
