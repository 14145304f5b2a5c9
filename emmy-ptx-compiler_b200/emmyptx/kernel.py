"""Kernel IR -> kernel handle: the builder API of the reference, bound to precompiled sm_100a kernels.

Same surface as the reference's `emmyptx/kernel.py`: `KernelCompiler(graph, kernel, launch, target, level)
.compile()` (`kernel.py:88, 130`), `compile_kernel(graph, kernel, launch, target)` (`:903-920`) and
`CompileError` (`:61`). The reference returns PTX text for one `.visible .entry`; this returns the text of
a *kernel handle*, a small JSON object naming the entry, the kernel variant in `libemmyb200.so` that
computes it, the variant's parameters and the launch descriptor's `arg_order`. `emmyptx.run_local.run_kernel`
takes that text where the reference's runner takes PTX. An IR no variant computes raises `CompileError`, as
unsupported IR does in the reference; nothing falls back to another implementation.
"""
from __future__ import annotations

import json
import math

from .match import tensor_table, Unmatched, match_kernel
from .ops import OpError

TARGET = "sm_100a"
HANDLE_VERSION = 1


class CompileError(NotImplementedError):
    pass


class KernelCompiler:
    error = CompileError

    def __init__(self, graph, kernel, launch: dict, target: str = TARGET, level: int = 2, int_div: str = "floor") -> None:
        """`level` is accepted for compatibility (the kernels are prebuilt at one optimisation level).
        `int_div`: 'floor' gives integer `//` and `%` torch's rounding, the semantics the reference's cases are
        checked against; 'trunc' reproduces the reference's PTX (`div.s32` / `rem.s32`)."""
        if target not in (TARGET, "sm_100"):           # "sm_100" is what a runner derives from the device's compute capability
            raise CompileError(f"target {target!r}: these kernels are built for {TARGET} only")
        if level not in (0, 1, 2):
            raise CompileError(f"optimization level {level!r} is not 0, 1 or 2")
        if int_div not in ("floor", "trunc"):
            raise CompileError(f"int_div {int_div!r} is not 'floor' or 'trunc'")
        if "arg_order" not in launch:
            raise CompileError("the launch descriptor has no arg_order")
        self.graph, self.kernel, self.launch = graph, kernel, launch
        self.target, self.level, self.int_div = target, level, int_div

    def match(self) -> dict:
        """The kernel variant and its parameters, as a dict."""
        # as the reference: an f64 buffer is refused rather than silently computed in f32 (emmyptx/kernel.py:185-187)
        for name, (_, dtype) in tensor_table(self.graph).items():
            if dtype == "f64" and name in self.launch["arg_order"]:
                raise CompileError(f"buffer {name!r} is f64: these kernels compute in f32, which would silently lose the f64 precision")
        try:
            m = match_kernel(self.graph, self.kernel, self.launch, self.int_div)
        except (Unmatched, OpError) as e:
            raise CompileError(f"{self.kernel.name}: {e}") from None
        names = set(self.launch["arg_order"])
        for b in (*m["inputs"], *m["outputs"]):
            if b not in names:
                raise CompileError(f"{self.kernel.name}: buffer {b!r} is not in the launch's arg_order")
        return m

    def compile(self) -> str:
        m = self.match()
        handle = {
            "emmyb200_handle": HANDLE_VERSION,
            "entry": self.kernel.name,
            "target": self.target,
            "variant": m["variant"],
            "params": m["params"],
            "inputs": m["inputs"],
            "outputs": m["outputs"],
            "arg_order": list(self.launch["arg_order"]),
            # kept for the record; the library sizes its own grids
            "grid": list(self.launch.get("grid", [])), "block": list(self.launch.get("block", [])),
            "smem_bytes": int(self.launch.get("smem_bytes", 0)),
            "lib": "libemmyb200.so",
        }
        return json.dumps(handle, indent=1) + "\n"


def compile_kernel(graph, kernel, launch: dict, target: str = TARGET) -> str:
    """The handle for `kernel`. (The reference retries at lower optimisation levels when a transformation
    trips or the PTX grows past the runner's size limit, `kernel.py:903-920`; a handle has neither problem.)"""
    return KernelCompiler(graph, kernel, launch, target).compile()


def algorithmic_work(handle: dict) -> tuple[float, str]:
    """(work, unit) one launch of the handle's kernel performs: bytes moved for streaming kernels (each
    element read once and written once), floating-point operations for contractions."""
    p, v = handle["params"], handle["variant"]
    if v in ("pointwise_f32", "index_gather_i32"):
        return 8.0 * p["n"], "B"
    if v == "pointwise_program":
        size = {"f32": 4, "f16": 2, "bf16": 2, "i32": 4, "int": 4, "i64": 8, "bool": 1, "u8": 1}
        prog, n = p["program"], p["n"]
        div, mod = prog.get("in_div", [0] * 4), prog.get("in_mod", [0] * 4)
        read = sum(size[d] * (mod[k] or (n // div[k] if div[k] else n)) for k, d in enumerate(prog["in_dtypes"]))      # broadcast inputs are small
        return float(read + n * size[prog["out_dtype"]]), "B"
    if v == "pointwise_indexed":
        size = {"f32": 4, "f16": 2, "bf16": 2, "i32": 4, "int": 4, "i64": 8, "bool": 1, "u8": 1}
        prog, n, im = p["program"], p["n"], p["index_map"]
        read = 0
        for d, src in zip(prog["in_dtypes"], im["inputs"]):
            if "axis" in src:
                continue                                    # an axis digit: no memory behind it
            distinct = 1
            for c, e in zip(src["coef"], im["extents"]):    # elements the map can reach: axes it ignores repeat them
                distinct *= e if c else 1
            read += size[d] * distinct
        return float(read + n * size[prog["out_dtype"]]), "B"
    if v == "contract_indexed":
        return 2.0 * p["n"] * p["terms"], "flop"
    if v == "gemm":
        return 2.0 * p["m"] * p["n"] * p["k"], "flop"
    if v == "gemm_f32":
        return 2.0 * p["batch"] * p["m"] * p["n"] * p["k"], "flop"
    if v == "gemm_batched":
        return 2.0 * p["batch"] * p["m"] * p["n"] * p["k"], "flop"
    if v == "attention_fwd":
        sq, sk = p["seq_q"], p["seq_k"]
        pairs = sq * sk
        if p.get("causal"):                       # query i meets keys 0 .. min(i, sk - 1)
            full = max(0, sq - sk)
            tri = min(sq, sk)
            pairs = tri * (tri + 1) // 2 + full * sk
        return 4.0 * p["units"] * pairs * p["d"], "flop"
    if v == "rowwise_f32":
        is_map = p["op"] in ("softmax", "log_softmax", "layer_norm", "rms_norm", "normalize")
        return 4.0 * p["rows"] * (p["cols"] * (2 if is_map else 1) + (0 if is_map else 1)), "B"
    if v == "colwise_f32":
        is_map = p["op"] in ("softmax", "log_softmax", "normalize")
        n = p["outer"] * p["rows"] * p["cols"]
        return 4.0 * (n * (2 if is_map else 1) + (0 if is_map else p["outer"] * p["cols"])), "B"
    raise CompileError(f"unknown variant {v!r}")
