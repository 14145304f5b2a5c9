"""ctypes binding of libemmyb200.so, the sm_100a kernel library.

The reference reaches its kernels through the CUDA driver API (`tools/run_local.py:64-72` loads
PTX, `:100-102` launches it). Here the kernels are precompiled, so the binding is one
`ctypes.CDLL` and typed entry points; device memory and streams are torch's. There is no CPU
path: without the library, or without a CUDA device, every call raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libemmyb200.so"

F32, F16, BF16, I32 = 0, 1, 2, 3
OP_EXP_SIN_TANH, OP_EXP, OP_SIN, OP_COS, OP_TANH, OP_GELU_TANH = range(6)
POINTWISE_OPS = {"exp_sin_tanh": OP_EXP_SIN_TANH, "exp": OP_EXP, "sin": OP_SIN, "cos": OP_COS,
                 "tanh": OP_TANH, "gelu_tanh": OP_GELU_TANH, "sigmoid": 6, "silu": 7, "relu": 8}
PW_MAX_SLOTS, PW_MAX_CONSTS, PW_MAX_STEPS, PW_MAX_INPUTS = 16, 16, 48, 4
PW_OPS = {name: i for i, name in enumerate(
    ["add", "subtract", "multiply", "divide", "maximum", "minimum", "relu", "square", "copy", "negative", "abs", "reciprocal",
     "sqrt", "rsqrt", "exp", "log", "sigmoid", "tanh", "erf", "sin", "cos", "pow", "equal", "not_equal", "greater", "less",
     "greater_equal", "less_equal", "where", "bitwise_and", "bitwise_or", "bitwise_not", "floor_divide", "mod"])}
PW_OPS.update(bitwise_xor=len(PW_OPS), left_shift=len(PW_OPS) + 1, right_shift=len(PW_OPS) + 2)
PW_OPS.update(exp_fast=PW_OPS["exp"], remainder=PW_OPS["mod"])
I64, U8 = 4, 5
DTYPE_CODES = {"f32": F32, "f16": F16, "bf16": BF16, "i32": I32, "i64": I64, "int": I32, "bool": U8, "u8": U8}


class PwStep(ctypes.Structure):
    _fields_ = [("op", ctypes.c_uint8), ("dst", ctypes.c_uint8), ("a", ctypes.c_uint8), ("b", ctypes.c_uint8),
                ("c", ctypes.c_uint8), ("reserved", ctypes.c_uint8 * 3)]


PW_MAX_AXES = 6


class PwIndexMap(ctypes.Structure):
    _fields_ = [("n_axes", ctypes.c_int32), ("reserved", ctypes.c_int32), ("extent", ctypes.c_int64 * PW_MAX_AXES),
                ("in_kind", ctypes.c_int32 * PW_MAX_INPUTS), ("in_axis", ctypes.c_int32 * PW_MAX_INPUTS),
                ("in_offset", ctypes.c_int64 * PW_MAX_INPUTS), ("in_coef", (ctypes.c_int64 * PW_MAX_AXES) * PW_MAX_INPUTS),
                ("out_offset", ctypes.c_int64), ("out_coef", ctypes.c_int64 * PW_MAX_AXES),
                ("in_rot", (ctypes.c_int64 * PW_MAX_AXES) * PW_MAX_INPUTS), ("in_index_of", ctypes.c_int32 * PW_MAX_INPUTS),
                ("in_index_abs", ctypes.c_int32 * PW_MAX_INPUTS), ("in_index_mod", ctypes.c_int64 * PW_MAX_INPUTS),
                ("in_index_mult", ctypes.c_int64 * PW_MAX_INPUTS)]


CT_MAX_LOOPS = 3


class ContractionMap(ctypes.Structure):
    _fields_ = [("n_axes", ctypes.c_int32), ("n_loops", ctypes.c_int32), ("extent", ctypes.c_int64 * PW_MAX_AXES),
                ("loop_extent", ctypes.c_int64 * CT_MAX_LOOPS),
                ("a_offset", ctypes.c_int64), ("a_coef", ctypes.c_int64 * PW_MAX_AXES), ("a_loop_coef", ctypes.c_int64 * CT_MAX_LOOPS),
                ("b_offset", ctypes.c_int64), ("b_coef", ctypes.c_int64 * PW_MAX_AXES), ("b_loop_coef", ctypes.c_int64 * CT_MAX_LOOPS),
                ("out_offset", ctypes.c_int64), ("out_coef", ctypes.c_int64 * PW_MAX_AXES),
                ("a_dtype", ctypes.c_int32), ("b_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class PwProgram(ctypes.Structure):
    _fields_ = [("n_inputs", ctypes.c_int32), ("n_steps", ctypes.c_int32), ("out_slot", ctypes.c_int32),
                ("out_dtype", ctypes.c_int32), ("in_dtype", ctypes.c_int32 * PW_MAX_INPUTS),
                ("consts", ctypes.c_float * PW_MAX_CONSTS), ("steps", PwStep * PW_MAX_STEPS),
                ("in_div", ctypes.c_int64 * PW_MAX_INPUTS), ("in_mod", ctypes.c_int64 * PW_MAX_INPUTS)]


EPI_NONE, EPI_GELU_TANH, EPI_RELU = 0, 1, 2
EPILOGUES = {None: EPI_NONE, "none": EPI_NONE, "gelu_tanh": EPI_GELU_TANH, "relu": EPI_RELU}
GEMM_B_NK = 1
GEMM_DST_MULTICAST = 2
ATT_CAUSAL = 1
ATT_DST_MULTICAST = 2
ATT_FORMS = {None: 0, "one_tile": 4, "two_tiles": 8}
GATHER_TRUNC = 1
ROW_OPS = {"sum": 0, "mean": 1, "amax": 2, "amin": 3, "prod": 4, "var": 5, "std": 6, "norm2": 7, "logsumexp": 8, "argmax": 9, "dot": 10, "cosine": 11,
           "softmax": 16, "log_softmax": 17, "layer_norm": 18, "rms_norm": 19, "normalize": 20}
ROW_MAP_FIRST = 16            # ops from here on write [rows, cols]

_SIGNATURES = {
    "emmyb200_version": (ctypes.c_int, []),
    "emmyb200_last_error": (ctypes.c_char_p, []),
    "emmyb200_pointwise_f32": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                              ctypes.c_void_p]),
    "emmyb200_pointwise_program": (ctypes.c_int, [ctypes.POINTER(PwProgram), ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p,
                                                  ctypes.c_int64, ctypes.c_void_p]),
    "emmyb200_set_pointwise_jit": (ctypes.c_int, [ctypes.c_int]),
    "emmyb200_pointwise_jit_state": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int64)]),
    "emmyb200_pointwise_program_source": (ctypes.c_int64, [ctypes.POINTER(PwProgram), ctypes.c_int, ctypes.c_char_p, ctypes.c_int64]),
    "emmyb200_pointwise_program_compile": (ctypes.c_int, [ctypes.POINTER(PwProgram), ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]),
    "emmyb200_pointwise_indexed": (ctypes.c_int, [ctypes.POINTER(PwProgram), ctypes.POINTER(PwIndexMap), ctypes.POINTER(ctypes.c_void_p),
                                                  ctypes.c_void_p, ctypes.c_void_p]),
    "emmyb200_pointwise_indexed_compile": (ctypes.c_int, [ctypes.POINTER(PwProgram), ctypes.POINTER(PwIndexMap), ctypes.POINTER(ctypes.c_int64)]),
    "emmyb200_contract_indexed": (ctypes.c_int, [ctypes.POINTER(ContractionMap), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "emmyb200_contract_indexed_compile": (ctypes.c_int, [ctypes.POINTER(ContractionMap), ctypes.POINTER(ctypes.c_int64)]),
    "emmyb200_index_gather_i32": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                                 ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                 ctypes.c_void_p]),
    "emmyb200_gemm": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                     ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]),
    "emmyb200_gemm_batched": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int64] * 10 + [ctypes.c_void_p]),
    "emmyb200_gemm_f32_workspace_bytes": (ctypes.c_int64, [ctypes.c_int] + [ctypes.c_int64] * 4 + [ctypes.c_int]),
    "emmyb200_gemm_f32": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
                          + [ctypes.c_int64] * 10 + [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
    "emmyb200_gemm_allgather": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]),
    "emmyb200_attention_fwd": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                              ctypes.c_int64, ctypes.c_float, ctypes.c_void_p]),
    "emmyb200_attention_fwd_allgather": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                        ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int64,
                                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_float,
                                                        ctypes.c_void_p]),
    "emmyb200_rowwise_workspace_bytes": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64]),
    "emmyb200_rowwise_f32": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_void_p]),
    "emmyb200_colwise_workspace_bytes": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]),
    "emmyb200_colwise_f32": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                            ctypes.c_float, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
    "emmyb200_cumsum_f32": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]),
    "emmyb200_rowwise_static_capacity": (ctypes.c_int64, []),
    "emmyb200_rowwise_f32_static": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                   ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p]),
    "emmyb200_launch_workspace_bytes": (ctypes.c_int64, [ctypes.c_char_p]),
    "emmyb200_launch": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_void_p]),
    "emmyb200_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32)]),
    "emmyb200_set_wait_limit_ns": (ctypes.c_int, [ctypes.c_uint64]),
    "emmyb200_selftest_wait_expiry": (ctypes.c_int, [ctypes.c_uint64, ctypes.c_void_p]),
}
ERR_TIMEOUT = -6
EXPORTS = tuple(_SIGNATURES)


class KernelError(RuntimeError):
    """A non-zero status from the library (the reference raises RuntimeError for driver errors,
    tools/run_local.py:44-48)."""

    def __init__(self, status: int, message: str) -> None:
        super().__init__(f"emmyb200 status {status}: {message}")
        self.status = status


_lib = None


def library() -> ctypes.CDLL:
    """The loaded library. Raises if it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python {LIB_PATH.parent.parent / 'build.py'}`")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise KernelError(status, library().emmyb200_last_error().decode())


def _stream(stream) -> int:
    import torch
    return (torch.cuda.current_stream() if stream is None else stream).cuda_stream


def _need_cuda(*tensors, strided: bool = False) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("emmyb200 kernels take CUDA tensors only (there is no CPU path)")
        if not strided and not t.is_contiguous():
            raise RuntimeError("emmyb200 kernels take contiguous tensors")


def dtype_code(t) -> int:
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32}[t.dtype]


def pointwise(op: str, x, out=None, stream=None):
    """out[i] = op(x[i]) for a float32 CUDA tensor; `op` is a key of POINTWISE_OPS."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.float32:
        raise TypeError("pointwise: float32 only")
    out = torch.empty_like(x) if out is None else out
    _need_cuda(out)
    check(library().emmyb200_pointwise_f32(POINTWISE_OPS[op], x.data_ptr(), out.data_ptr(), x.numel(), _stream(stream)))
    return out


def make_program(program: dict) -> PwProgram:
    """The C struct for a program in the form the matcher emits: {"in_dtypes": [...], "out_dtype": ..., "out_slot": k,
    "consts": [...], "steps": [[op name, dst, a, b, c], ...]} (operands >= PW_MAX_SLOTS name constants). An integer
    program (output i32 / i64) may carry "int_div": "trunc" to round `//` and `%` toward zero."""
    p = PwProgram()
    p.n_inputs, p.n_steps = len(program["in_dtypes"]), len(program["steps"])
    p.out_slot, p.out_dtype = program["out_slot"], DTYPE_CODES[program["out_dtype"]]
    for i, d in enumerate(program["in_dtypes"]):
        p.in_dtype[i] = DTYPE_CODES[d]
        p.in_div[i] = program.get("in_div", [0] * PW_MAX_INPUTS)[i]            # broadcast inputs: element (i // div) % mod
        p.in_mod[i] = program.get("in_mod", [0] * PW_MAX_INPUTS)[i]
    for i, c in enumerate(program["consts"]):
        p.consts[i] = c
    for i, (op, dst, a, b, c) in enumerate(program["steps"]):
        p.steps[i].op, p.steps[i].dst, p.steps[i].a, p.steps[i].b, p.steps[i].c = PW_OPS[op], dst, a, b, c
        p.steps[i].reserved[0] = 1 if program.get("int_div") == "trunc" else 0
    return p


def pointwise_program(program: dict, inputs: list, out, stream=None):
    """out[i] = program(inputs[0][i], inputs[1][i], ...): the general elementwise kernel."""
    _need_cuda(out, *inputs)
    arr = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
    prog = make_program(program)
    check(library().emmyb200_pointwise_program(ctypes.byref(prog), arr, out.data_ptr(), out.numel(), _stream(stream)))
    return out


def make_index_map(index_map: dict) -> PwIndexMap:
    """The C struct for {"extents": [...], "inputs": [{"offset": o, "coef": [...]} | {"axis": a}, ...], "out": {"offset": o,
    "coef": [...]}}: input k reads element offset + sum coef[a] * digit[a] of its buffer, or is the digit of axis a. A buffer
    input may carry "rot" (rotations), "index_mod" / "index_abs" (an index source), "index_of" / "index_mult" (addressed
    through one) or "clamp" (a guarded read: the index is clamped into [0, clamp))."""
    m = PwIndexMap()
    if not 1 <= len(index_map["extents"]) <= PW_MAX_AXES or len(index_map["inputs"]) > PW_MAX_INPUTS:
        raise ValueError(f"an index map has 1 to {PW_MAX_AXES} axes and at most {PW_MAX_INPUTS} inputs")
    m.n_axes = len(index_map["extents"])
    for a, e in enumerate(index_map["extents"]):
        m.extent[a] = e
    for k, src in enumerate(index_map["inputs"]):
        if "axis" in src:
            m.in_kind[k], m.in_axis[k] = 1, src["axis"]
        else:
            m.in_offset[k] = src["offset"]
            for a, c in enumerate(src["coef"]):
                m.in_coef[k][a] = c
            for a, r in enumerate(src.get("rot", [])):              # rotation of axis a: (digit + r) mod extent
                m.in_rot[k][a] = r
            if "index_mod" in src:                                  # an index source: |value| (if abs) mod index_mod
                m.in_kind[k], m.in_index_mod[k], m.in_index_abs[k] = 3, src["index_mod"], 1 if src.get("index_abs") else 0
            elif "index_of" in src:                                 # addressed through index source index_of
                m.in_kind[k], m.in_index_of[k], m.in_index_mult[k] = 2, src["index_of"], src["index_mult"]
            elif "clamp" in src:                                    # a guarded read: the index is clamped into [0, clamp)
                m.in_kind[k], m.in_index_mod[k] = 4, src["clamp"]
    m.out_offset = index_map["out"]["offset"]
    for a, c in enumerate(index_map["out"]["coef"]):
        m.out_coef[a] = c
    return m


def pointwise_indexed(program: dict, index_map: dict, inputs: list, out, stream=None):
    """One value per cell of a tile with the given axis extents; input k is an element of inputs[k] chosen by an affine
    map of the cell's axis digits (or a digit itself: inputs[k] is then None), the value is stored through the output
    map. Index ranges are checked against the tensors here: the C entry point cannot."""
    import math
    ext = index_map["extents"]
    def reach(m):
        lo = hi = m["offset"]
        for c, e in zip(m["coef"], ext):
            lo, hi = lo + min(0, c * (e - 1)), hi + max(0, c * (e - 1))
        return lo, hi
    real = [t for t in inputs if t is not None]
    _need_cuda(out, *real)
    if math.prod(ext) > 0:
        for k, src in enumerate(index_map["inputs"]):
            if "clamp" in src:                                      # a guarded read: clamped into the buffer by the kernel
                if not 1 <= src["clamp"] <= inputs[k].numel():
                    raise IndexError(f"pointwise_indexed: input {k} is clamped to {src['clamp']} elements of {inputs[k].numel()}")
            elif "axis" not in src:
                lo, hi = reach(src)
                if "index_of" in src:                               # plus the largest row the index source can name
                    hi += src["index_mult"] * (index_map["inputs"][src["index_of"]]["index_mod"] - 1)
                if lo < 0 or hi >= inputs[k].numel():
                    raise IndexError(f"pointwise_indexed: input {k} is read at elements {lo}..{hi} of {inputs[k].numel()}")
        lo, hi = reach(index_map["out"])
        if lo < 0 or hi >= out.numel():
            raise IndexError(f"pointwise_indexed: the output is written at elements {lo}..{hi} of {out.numel()}")
    arr = (ctypes.c_void_p * len(inputs))(*[None if t is None else t.data_ptr() for t in inputs])
    prog, m = make_program(program), make_index_map(index_map)
    check(library().emmyb200_pointwise_indexed(ctypes.byref(prog), ctypes.byref(m), arr, out.data_ptr(), _stream(stream)))
    return out


def indexed_compile(program: dict, index_map: dict) -> int:
    """Compile an indexed program's kernel for sm_100a without launching it (works without a GPU)."""
    prog, m = make_program(program), make_index_map(index_map)
    n = ctypes.c_int64(0)
    check(library().emmyb200_pointwise_indexed_compile(ctypes.byref(prog), ctypes.byref(m), ctypes.byref(n)))
    return n.value


def make_contraction_map(cmap: dict) -> ContractionMap:
    """The C struct for {"extents": [...], "loops": [...], "a": {"offset", "coef", "loop_coef", "dtype"}, "b": {...},
    "out": {"offset", "coef", "dtype"}}: out[cell] = sum over the loops of A[a-map] * B[b-map]."""
    if not 1 <= len(cmap["extents"]) <= PW_MAX_AXES or not 1 <= len(cmap["loops"]) <= CT_MAX_LOOPS:
        raise ValueError(f"a contraction has 1 to {PW_MAX_AXES} tile axes and 1 to {CT_MAX_LOOPS} reduction axes")
    m = ContractionMap()
    m.n_axes, m.n_loops = len(cmap["extents"]), len(cmap["loops"])
    for a, e in enumerate(cmap["extents"]):
        m.extent[a] = e
    for l, e in enumerate(cmap["loops"]):
        m.loop_extent[l] = e
    for side in ("a", "b"):
        src = cmap[side]
        setattr(m, f"{side}_offset", src["offset"])
        setattr(m, f"{side}_dtype", DTYPE_CODES[src["dtype"]])
        for a, c in enumerate(src["coef"]):
            getattr(m, f"{side}_coef")[a] = c
        for l, c in enumerate(src["loop_coef"]):
            getattr(m, f"{side}_loop_coef")[l] = c
    m.out_offset, m.out_dtype = cmap["out"]["offset"], DTYPE_CODES[cmap["out"]["dtype"]]
    for a, c in enumerate(cmap["out"]["coef"]):
        m.out_coef[a] = c
    return m


def contract_indexed(cmap: dict, a, b, out, stream=None):
    """out[cell] = sum over the map's reduction axes of a[...] * b[...] (fp32 fused multiply-adds in loop order), the
    cell's digits and the loop counters addressing a and b through affine maps. Index ranges are checked against the
    tensors here."""
    _need_cuda(a, b, out)
    ext, loops = cmap["extents"], cmap["loops"]

    def reach(src, with_loops=True):
        lo = hi = src["offset"]
        terms = list(zip(src["coef"], ext)) + (list(zip(src["loop_coef"], loops)) if with_loops else [])
        for c, e in terms:
            lo, hi = lo + min(0, c * (e - 1)), hi + max(0, c * (e - 1))
        return lo, hi
    for name, t, src, wl in (("a", a, cmap["a"], True), ("b", b, cmap["b"], True), ("out", out, cmap["out"], False)):
        if 0 in ext:
            break                                   # an empty tile addresses nothing
        lo, hi = reach(src, wl)
        if lo < 0 or hi >= t.numel():
            raise IndexError(f"contract_indexed: {name} is addressed at elements {lo}..{hi} of {t.numel()}")
    m = make_contraction_map(cmap)
    check(library().emmyb200_contract_indexed(ctypes.byref(m), a.data_ptr(), b.data_ptr(), out.data_ptr(), _stream(stream)))
    return out


def contraction_compile(cmap: dict) -> int:
    """Compile an indexed contraction's kernel for sm_100a without launching it (works without a GPU)."""
    m = make_contraction_map(cmap)
    n = ctypes.c_int64(0)
    check(library().emmyb200_contract_indexed_compile(ctypes.byref(m), ctypes.byref(n)))
    return n.value


def set_pointwise_jit(enabled: bool) -> bool:
    """Float programs as kernels compiled at first use (True, the default) or on the interpreter kernel; returns the
    previous setting."""
    return bool(library().emmyb200_set_pointwise_jit(1 if enabled else 0))


def pointwise_jit_state() -> tuple[int, int]:
    """(state, kernels compiled so far): state 1 = compiled form in use, 0 = switched off, -1 = the run-time compiler
    could not be loaded (programs run on the interpreter)."""
    n = ctypes.c_int64(0)
    return library().emmyb200_pointwise_jit_state(ctypes.byref(n)), n.value


def program_source(program: dict, group: int = 4) -> str:
    """The CUDA C++ text of the kernel a float program is compiled to; `group` = elements per thread and access group
    (4, 8, or 0 for scalar accesses)."""
    prog = make_program(program)
    need = library().emmyb200_pointwise_program_source(ctypes.byref(prog), int(group), None, 0)
    if need < 0:
        check(int(need))
    buf = ctypes.create_string_buffer(need)
    library().emmyb200_pointwise_program_source(ctypes.byref(prog), int(group), buf, need)
    return buf.value.decode()


def program_compile(program: dict, group: int = 4) -> int:
    """Compile a float program's kernel for sm_100a without launching it (works without a GPU); returns the size of
    the device code."""
    prog = make_program(program)
    n = ctypes.c_int64(0)
    check(library().emmyb200_pointwise_program_compile(ctypes.byref(prog), int(group), ctypes.byref(n)))
    return n.value


def index_gather(x, mul: int, add: int, div: int, shift: int, trunc: bool = False, out=None, stream=None):
    """out[i] = (x[(i*mul + add) mod n] // div) ^ (i >> shift) for an int32 CUDA tensor."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.int32:
        raise TypeError("index_gather: int32 only")
    out = torch.empty_like(x) if out is None else out
    _need_cuda(out)
    check(library().emmyb200_index_gather_i32(x.data_ptr(), out.data_ptr(), x.numel(), mul, add, div, shift,
                                              GATHER_TRUNC if trunc else 0, _stream(stream)))
    return out


GEMM_OUT_F32 = 4


def _out_flag(a, out, out_f32: bool) -> int:
    """The fp32-output flag of the 16-bit GEMM: asked for, or implied by the output tensor's dtype."""
    import torch
    if out is not None and out.dtype == torch.float32:
        return GEMM_OUT_F32
    if out is not None and out.dtype != a.dtype:
        raise TypeError("gemm: the output has the operands' dtype or float32")
    return GEMM_OUT_F32 if out_f32 else 0


def gemm(a, b, epilogue: str | None = None, b_is_nk: bool = False, out=None, stream=None, out_f32: bool = False):
    """out = epilogue(a @ b) (or a @ b.T when `b_is_nk`), fp16 / bf16, fp32 accumulation. `out_f32` (or a float32 `out`):
    the accumulator is stored as fp32 instead of being rounded to the operands' type."""
    import torch
    _need_cuda(a, b)
    if a.dtype != b.dtype or a.dim() != 2 or b.dim() != 2:
        raise TypeError("gemm: two 2-D tensors of one 16-bit dtype")
    m, k = a.shape
    n = b.shape[0] if b_is_nk else b.shape[1]
    if (b.shape[1] if b_is_nk else b.shape[0]) != k:
        raise ValueError(f"gemm: inner extents differ: {tuple(a.shape)} x {tuple(b.shape)}")
    flag = _out_flag(a, out, out_f32)
    out = torch.empty((m, n), dtype=torch.float32 if flag else a.dtype, device=a.device) if out is None else out
    _need_cuda(out)
    check(library().emmyb200_gemm(dtype_code(a), EPILOGUES[epilogue], (GEMM_B_NK if b_is_nk else 0) | flag, a.data_ptr(),
                                  b.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), b.stride(0), out.stride(0),
                                  _stream(stream)))
    return out


def gemm_batched(a, b, bias=None, epilogue: str | None = None, b_is_nk: bool = False, out=None, stream=None, out_f32: bool = False):
    """out[i] = epilogue(a[i] @ b[i] + bias) for 3-D a; b is 3-D (one plane per product) or 2-D (shared by all). With
    `out_f32` (or a float32 `out`) the output and the bias are float32."""
    import torch
    _need_cuda(a, b)
    if a.dim() != 3 or b.dim() not in (2, 3) or a.dtype != b.dtype:
        raise TypeError("gemm_batched: a is 3-D, b 2-D or 3-D, one 16-bit dtype")
    batch, m, k = a.shape
    n = b.shape[-2] if b_is_nk else b.shape[-1]
    if (b.shape[-1] if b_is_nk else b.shape[-2]) != k or (b.dim() == 3 and b.shape[0] != batch):
        raise ValueError(f"gemm_batched: shapes do not agree: {tuple(a.shape)} x {tuple(b.shape)}")
    flag = _out_flag(a, out, out_f32)
    out = torch.empty((batch, m, n), dtype=torch.float32 if flag else a.dtype, device=a.device) if out is None else out
    _need_cuda(out)
    if bias is not None:
        _need_cuda(bias)
        if bias.dtype != out.dtype or bias.numel() != n:
            raise ValueError("gemm_batched: bias holds N values of the output's dtype")
    check(library().emmyb200_gemm_batched(dtype_code(a), EPILOGUES[epilogue], (GEMM_B_NK if b_is_nk else 0) | flag, a.data_ptr(),
                                          b.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), batch, m, n, k,
                                          a.stride(1), b.stride(-2), out.stride(1), a.stride(0), b.stride(0) if b.dim() == 3 else 0,
                                          out.stride(0), _stream(stream)))
    return out


class HostGemm:
    """epilogue(A @ B) with A, B and C in pinned host memory: B is copied to the device once per call, A in row chunks
    on a copy stream, and each chunk's product is copied back on a third stream while the next chunk is on its way
    in and being multiplied, so that a call costs about as long as the larger of its host-to-device copies and its
    arithmetic instead of their sum. Device buffers are allocated once, in the constructor."""

    def __init__(self, m: int, n: int, k: int, dtype, device, epilogue: str | None = None, chunks: int = 8, overlap_calls: bool = True):
        """`overlap_calls`: the copy-in of a call starts as soon as the previous call's last product has been computed,
        while that call's last rows are still on their way back to the host (the host link carries both directions at
        once); the host inputs must then be ready when the call is made, not merely ordered after earlier work on `stream`."""
        import torch
        while chunks > 1 and (m % chunks or (m // chunks) % 128):
            chunks -= 1                                                        # whole row blocks per chunk
        self.m, self.n, self.k, self.epilogue, self.chunks, self.rows = m, n, k, epilogue, chunks, m // chunks
        self.overlap_calls, self.called = overlap_calls, False
        self.a = torch.empty(m, k, dtype=dtype, device=device)
        self.b = torch.empty(k, n, dtype=dtype, device=device)
        self.c = torch.empty(m, n, dtype=dtype, device=device)
        self.copy_in, self.copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.ev_in = [torch.cuda.Event() for _ in range(chunks + 1)]
        self.ev_done = [torch.cuda.Event() for _ in range(chunks)]

    def __call__(self, a_host, b_host, c_host, stream=None):
        """Enqueue the whole call; `c_host` is complete when `stream` (default: the current one) has caught up."""
        import torch
        main = torch.cuda.current_stream() if stream is None else stream
        if self.overlap_calls and self.called:
            self.copy_in.wait_event(self.ev_done[-1])                          # the previous call's products have read A and B
        else:
            self.copy_in.wait_stream(main)                                     # the buffers may still be in use by earlier work
        self.copy_out.wait_stream(main)
        self.called = True
        with torch.cuda.stream(self.copy_in):
            self.b.copy_(b_host, non_blocking=True)
            self.ev_in[0].record()
            for i in range(self.chunks):
                rows = slice(i * self.rows, (i + 1) * self.rows)
                self.a[rows].copy_(a_host[rows], non_blocking=True)
                self.ev_in[i + 1].record()
        main.wait_event(self.ev_in[0])
        for i in range(self.chunks):
            rows = slice(i * self.rows, (i + 1) * self.rows)
            main.wait_event(self.ev_in[i + 1])
            gemm(self.a[rows], self.b, epilogue=self.epilogue, out=self.c[rows], stream=main)
            self.ev_done[i].record(main)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(self.ev_done[i])
                c_host[rows].copy_(self.c[rows], non_blocking=True)
        main.wait_stream(self.copy_out)
        return c_host


def gemm_f32(a, b, bias=None, epilogue: str | None = None, b_is_nk: bool = False, out=None, workspace=None, stream=None):
    """float32 matmul with float32 accuracy on the tensor cores. a: [M, K] or [batch, M, K]; b: [K, N] ([N, K] with
    b_is_nk), shared by every product, or [batch, K, N]; bias: [N] or None. Last axes must be contiguous."""
    import torch
    _need_cuda(a, b, strided=True)              # row-pitched views are fine: the split reads element by element
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError("gemm_f32: float32 operands")
    squeeze = a.dim() == 2
    a3 = a.unsqueeze(0) if squeeze else a
    if a3.dim() != 3 or b.dim() not in (2, 3) or a3.stride(-1) != 1 or b.stride(-1) != 1:
        raise TypeError("gemm_f32: [batch,] M x K and [batch,] K x N operands with contiguous last axes")
    batch, m, k = a3.shape
    n = b.shape[-2] if b_is_nk else b.shape[-1]
    if (b.shape[-1] if b_is_nk else b.shape[-2]) != k or (b.dim() == 3 and b.shape[0] != batch):
        raise ValueError("gemm_f32: operand shapes do not agree")
    if out is None:
        out = torch.empty((batch, m, n), dtype=torch.float32, device=a.device)
        if squeeze:
            out = out[0]
    _need_cuda(out, strided=True)
    o3 = out.unsqueeze(0) if out.dim() == 2 else out
    stride_b = b.stride(0) if b.dim() == 3 and batch > 1 else 0
    lib = library()
    flags = GEMM_B_NK if b_is_nk else 0
    need = lib.emmyb200_gemm_f32_workspace_bytes(flags, batch, m, n, k, 1 if stride_b == 0 else 0)
    if need > 0 and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
        if stream is not None:
            # a workspace made here is dropped on return while the kernels on `stream` still read it: tell the caching
            # allocator, so that the block is not handed to other work before that stream has passed this point
            workspace.record_stream(stream)
    if bias is not None:
        _need_cuda(bias)
        if bias.dtype != torch.float32 or bias.numel() != n or not bias.is_contiguous():
            raise TypeError("gemm_f32: bias is a contiguous float32 vector of N elements")
    check(lib.emmyb200_gemm_f32(EPILOGUES[epilogue], flags, a3.data_ptr(), b.data_ptr(), bias.data_ptr() if bias is not None else None,
                                o3.data_ptr(), batch, m, n, k, a3.stride(1), b.stride(-2), o3.stride(1),
                                a3.stride(0) if batch > 1 else 0, stride_b, o3.stride(0) if batch > 1 else 0,
                                workspace.data_ptr() if workspace is not None else None,
                                workspace.numel() if workspace is not None else 0, _stream(stream)))
    return out


def gemm_allgather(a, b, dst_ptrs: list[int], ldc: int, epilogue: str | None = None, b_is_nk: bool = False, multicast: bool = False,
                   stream=None):
    """epilogue(a @ b) for this rank's rows of A, every output piece stored to each address in `dst_ptrs`
    (this rank's shard first, then where the same rows live in each peer's full C). With `multicast`, `dst_ptrs` is the
    one address of the shard inside a multicast mapping of C, and the switch replicates every store."""
    _need_cuda(a, b)
    m, k = a.shape
    n = b.shape[0] if b_is_nk else b.shape[1]
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    check(library().emmyb200_gemm_allgather(dtype_code(a), EPILOGUES[epilogue],
                                            (GEMM_B_NK if b_is_nk else 0) | (GEMM_DST_MULTICAST if multicast else 0), a.data_ptr(),
                                            b.data_ptr(), arr, len(dst_ptrs), m, n, k, a.stride(0), b.stride(0), ldc,
                                            _stream(stream)))


def attention(q, k, v, scale: float | None = None, causal: bool = False, out=None, stream=None, form: str | None = None):
    """softmax(q k^T * scale) v over the last two axes; leading axes are independent units. `causal`: query i sees
    keys 0..i only. `form`: "one_tile" / "two_tiles" forces a kernel form (default: the library's choice)."""
    import torch
    _need_cuda(q, k, v)
    d = q.shape[-1]
    units = q.numel() // (q.shape[-2] * d)
    out = torch.empty_like(q) if out is None else out
    _need_cuda(out)
    scale = d ** -0.5 if scale is None else scale
    check(library().emmyb200_attention_fwd(dtype_code(q), (ATT_CAUSAL if causal else 0) | ATT_FORMS[form], q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), units,
                                           q.shape[-2], k.shape[-2], d, scale, _stream(stream)))
    return out


def attention_allgather(q, k, v, dst_ptrs: list[int], scale: float | None = None, causal: bool = False, multicast: bool = False,
                        stream=None, form: str | None = None):
    """attention() on this rank's units, every output tile stored to each address in `dst_ptrs` (this rank's slice of
    O first, then the same slice inside each peer's full O; with `multicast`, the slice's one multicast address)."""
    _need_cuda(q, k, v)
    d = q.shape[-1]
    units = q.numel() // (q.shape[-2] * d)
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    scale = d ** -0.5 if scale is None else scale
    check(library().emmyb200_attention_fwd_allgather(dtype_code(q), (ATT_CAUSAL if causal else 0) | (ATT_DST_MULTICAST if multicast else 0) | ATT_FORMS[form],
                                                     q.data_ptr(), k.data_ptr(), v.data_ptr(), arr, len(dst_ptrs),
                                                     units, q.shape[-2], k.shape[-2], d, scale, _stream(stream)))


def rowwise(op: str, x, weight=None, bias=None, eps: float = 0.0, out=None, workspace=None, stream=None):
    """Reduce (or normalise) the last axis of a contiguous float32 CUDA tensor; `op` is a key of ROW_OPS. Reducing ops
    return x.shape[:-1] (int64 for argmax), the others x.shape. Long rows need workspace memory, taken from torch's
    allocator unless a uint8 tensor is passed."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() < 1:
        raise TypeError("rowwise: a contiguous float32 tensor with at least one axis")
    code = ROW_OPS[op]
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if out is None:
        out = (torch.empty_like(x) if code >= ROW_MAP_FIRST else
               torch.empty(x.shape[:-1], dtype=torch.int64 if op == "argmax" else torch.float32, device=x.device))
    _need_cuda(out)
    for t in (weight, bias):
        if t is not None:
            _need_cuda(t)
            want = x.numel() if op == "cosine" else cols               # cosine: the second matrix, same shape as x
            if t.dtype != torch.float32 or t.numel() != want or not t.is_contiguous():
                raise TypeError("rowwise: weight / bias are contiguous float32 vectors of the row length (cosine: a second array like x)")
    lib = library()
    need = lib.emmyb200_rowwise_workspace_bytes(code, rows, cols)
    if need > 0 and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib.emmyb200_rowwise_f32(code, x.data_ptr(), weight.data_ptr() if weight is not None else None,
                                   bias.data_ptr() if bias is not None else None, out.data_ptr(), rows, cols, eps,
                                   workspace.data_ptr() if workspace is not None else None,
                                   workspace.numel() if workspace is not None else 0, _stream(stream)))
    return out


COL_OPS = ("sum", "mean", "amax", "amin", "prod", "var", "std", "norm2", "logsumexp", "argmax", "softmax", "log_softmax", "normalize")


def colwise(op: str, x, eps: float = 0.0, out=None, workspace=None, stream=None):
    """Reduce (or normalise) axis -2 of a contiguous float32 CUDA tensor of 2 or more axes: a [rows, cols] matrix over
    dim 0, a [..., rows, cols] stack plane by plane. `op` is one of COL_OPS."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() < 2:
        raise TypeError("colwise: a contiguous float32 tensor with at least two axes")
    if op not in COL_OPS:
        raise KeyError(op)
    code = ROW_OPS[op]
    rows, cols = x.shape[-2], x.shape[-1]
    outer = x.numel() // (rows * cols) if rows * cols else 0
    if out is None:
        out = (torch.empty_like(x) if code >= ROW_MAP_FIRST else
               torch.empty((*x.shape[:-2], cols), dtype=torch.int64 if op == "argmax" else torch.float32, device=x.device))
    _need_cuda(out)
    lib = library()
    need = lib.emmyb200_colwise_workspace_bytes(code, outer, rows, cols)
    if need > 0 and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib.emmyb200_colwise_f32(code, x.data_ptr(), out.data_ptr(), outer, rows, cols, eps,
                                   workspace.data_ptr() if workspace is not None else None,
                                   workspace.numel() if workspace is not None else 0, _stream(stream)))
    return out


def cumsum(x, out=None, stream=None):
    """Running sum along the last axis of a contiguous float32 CUDA tensor."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() < 1:
        raise TypeError("cumsum: a contiguous float32 tensor with at least one axis")
    out = torch.empty_like(x) if out is None else out
    _need_cuda(out)
    cols = x.shape[-1]
    check(library().emmyb200_cumsum_f32(x.data_ptr(), out.data_ptr(), x.numel() // cols if cols else 0, cols, _stream(stream)))
    return out


def device_status() -> int:
    """Reads and clears the device status word (non-zero: a bounded device-side wait expired). Does not raise on an
    expired wait: `check_device()` does."""
    word = ctypes.c_uint32(0)
    rc = library().emmyb200_device_status(ctypes.byref(word))
    if rc not in (0, ERR_TIMEOUT):
        check(rc)
    return word.value


def check_device() -> None:
    """Raises KernelError (status EMMYB200_ERR_TIMEOUT) if a bounded device-side wait expired since the last read."""
    word = ctypes.c_uint32(0)
    check(library().emmyb200_device_status(ctypes.byref(word)))
