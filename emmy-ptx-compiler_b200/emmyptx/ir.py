"""Stand-in Kernel IR node classes, and builders for the benchmark configurations.

The reference never imports IR classes: it dispatches on `type(node).__name__` and reads attributes
(`emmyptx/kernel.py:313, 487`; `emmyptx/loops.py:51-63`), and gets the real objects from the tracer
package `emmy-ml` through `emmy.compiler.graph.Graph.from_dict` (`compile.py:15, 43`). This module
provides classes with the same names and attributes, so a kernel can be described, serialised to
`<kernel>.ir.json` and compiled without the tracer; objects from the real tracer are accepted just the
same, because the matcher here is duck-typed in the same way.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any

_NODES: dict[str, type] = {}


def _node(cls):
    cls = dataclass(cls)
    _NODES[cls.__name__] = cls
    return cls


# ---- graph ------------------------------------------------------------------------------------------
@_node
class Dim:
    value: int

    def as_static(self) -> int:
        return int(self.value)


@_node
class DType:
    name: str


@_node
class TensorInfo:
    name: str
    shape: list
    dtype: Any


@_node
class Node:
    op: Any
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)


@_node
class InputOp:
    name: str = "input"


@_node
class Graph:
    nodes: dict

    def to_dict(self) -> dict:
        return to_jsonable(self)

    @staticmethod
    def from_dict(d: dict) -> "Graph":
        return from_jsonable(d)


def tensor(name: str, shape, dtype: str) -> TensorInfo:
    return TensorInfo(name, [Dim(int(s)) for s in shape], DType(dtype))


# ---- expressions ---------------------------------------------------------------------------------------
class _Expr:
    def free_vars(self) -> set:
        out = set()
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            for item in (v if isinstance(v, (list, tuple)) else [v]):
                if isinstance(item, _Expr):
                    out |= item.free_vars()
        return out


@_node
class Literal(_Expr):
    value: Any
    dtype: Any = None


@_node
class Var(_Expr):
    name: str

    def free_vars(self) -> set:
        return {self.name}


@_node
class BinaryExpr(_Expr):
    op: str
    left: Any
    right: Any


@_node
class TernaryExpr(_Expr):
    cond: Any
    if_true: Any
    if_false: Any


@_node
class CastExpr(_Expr):
    dtype: str
    expr: Any


@_node
class FuncCallExpr(_Expr):
    name: str
    args: list


# ---- statements ------------------------------------------------------------------------------------------
class _Stmt:
    def pretty(self) -> list:
        """Lines describing the statement, the first one its headline: the tracer's nodes have this method and
        the reference's tensor-core lowering names a statement by it in diagnostics (emmyptx/mma.py:67, 83, 184,
        200; emmyptx/kernel.py:479)."""
        shown = ", ".join(f"{f.name}={getattr(self, f.name)!r}" for f in dataclasses.fields(self)
                          if isinstance(getattr(self, f.name), (str, int, bool)))
        return [f"{type(self).__name__}({shown})"]


@_node
class Op:
    name: str
    identity: Any = None


@_node
class Axis:
    name: str
    extent: Any


@_node
class KernelOp:
    name: str
    body: list


@_node
class Tile:
    axes: list
    body: list
    aux_threads: int = 0
    block_threads: int = 0
    raster_group: int = 0
    raster_axes: Any = None
    raster_orient: str = "m"


@_node
class Load:
    names: list
    input: str
    index: list


@_node
class Write:
    output: str
    index: list
    values: list
    atomic: bool = False
    swizzle: str = "NONE"


@_node
class Assign:
    name: str
    op: Any
    args: list
    dtype: Any = None


@_node
class Let:
    name: str
    value: Any
    dtype: Any = None


@_node
class Branch:
    select: Any             # the predicate (an expression of axis variables and earlier values); unused in the last branch
    value: Any              # a value name or a number


@_node
class Select:
    """`name = v0 when p0, v1 when p1, ..., v_last otherwise` (emmyptx/kernel.py:812-822)."""
    name: str
    branches: list


@_node
class Cond:
    """`if cond: body else: else_body` on an expression of the axis variables (emmyptx/kernel.py:825-840)."""
    cond: Any
    body: list
    else_body: list


@_node
class Loop:
    axis: Any
    body: list
    unroll: bool = False
    seed: bool = True


@_node
class Accum:
    name: str
    base: Any
    value: str
    op: Any


@_node
class Init:
    name: str
    identity: Any = 0.0


@_node
class Smem:
    name: str
    dtype: str
    extents: list
    align: int = 16


@_node
class RegFragment(_Stmt):
    name: str
    role: str
    dtype: Any
    shape: tuple = (16, 8, 16)
    count: int = 1
    nregs: Any = None


@_node
class LdmatrixLoad(_Stmt):
    frag: str
    role: str
    src_buffer: str
    src_index: list
    ldm: int = 0
    staged: bool = False
    b_trans: bool = False
    pair_frag: Any = None
    swizzle: str = "NONE"
    fragment_layout: str = "m16n8k16"
    byte_slab: bool = False
    scale_buffer: Any = None
    gmem_guard: Any = None
    k_zero: Any = None


@_node
class MmaSyncPtx(_Stmt):
    c_frag: str
    a_frag: str
    b_frag: str
    shape: tuple = (16, 8, 16)
    ab_dtype: str = "f16"
    c_dtype: str = "f32"
    b_row_major: bool = False
    sfa_frag: Any = None


@_node
class RegStore(_Stmt):
    frag: str
    dst_buffer: str
    dst_index: list
    ldm: int = 0
    row_dim: Any = None
    col_dim: Any = None
    m_guard: Any = None
    n_guard: Any = None
    atomic: bool = False
    epilogue: Any = None
    bias: Any = None
    extra_frags: Any = None
    swizzle: str = "NONE"
    fragment_layout: str = "m16n8k16"
    volta_interleaved: bool = False


@_node
class WarpShuffle:
    state: list
    state_b: list
    combine_states: list
    length: int = 32


# ---- (de)serialisation ----------------------------------------------------------------------------------
def to_jsonable(x):
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
        d = {"__node__": type(x).__name__}
        for f in dataclasses.fields(x):
            d[f.name] = to_jsonable(getattr(x, f.name))
        return d
    if isinstance(x, dict):
        return {k: to_jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [to_jsonable(v) for v in x]
    return x


def from_jsonable(x):
    if isinstance(x, dict) and "__node__" in x:
        cls = _NODES[x["__node__"]]
        return cls(**{k: from_jsonable(v) for k, v in x.items() if k != "__node__"})
    if isinstance(x, dict):
        return {k: from_jsonable(v) for k, v in x.items()}
    if isinstance(x, list):
        return [from_jsonable(v) for v in x]
    return x


# ---- builders: the five benchmark configurations as Kernel IR --------------------------------------------
def _graph(kernel: KernelOp, inputs: list[TensorInfo], outputs: list[TensorInfo]) -> Graph:
    nodes = {t.name: Node(InputOp(), [], [t]) for t in inputs}
    nodes[kernel.name] = Node(kernel, [t.name for t in inputs], outputs)
    return Graph(nodes)


def _launch(kernel: KernelOp, arg_names: list[str], cells: int, block: int = 256, smem: int = 0) -> dict:
    return {"entry": kernel.name, "arg_order": arg_names, "grid": [-(-cells // block), 1, 1], "block": [block, 1, 1],
            "smem_bytes": smem}


def pointwise_kernel(n: int, expr: str = "exp_sin_tanh", name: str = "k_pointwise"):
    """y = op(x) over a one-axis tile. `exp_sin_tanh` is exp(x) + sin(x) * tanh(x), the statement list the
    tracer produces for that torch expression: one Load, four Assigns through the op table, one Write."""
    a0 = Axis("a0", Dim(n))
    body = [Load(["v0"], "x", [Var("a0")])]
    if expr == "exp_sin_tanh":
        body += [Assign("v1", Op("exp"), ["v0"]), Assign("v2", Op("sin"), ["v0"]), Assign("v3", Op("tanh"), ["v0"]),
                 Assign("v4", Op("multiply"), ["v2", "v3"]), Assign("v5", Op("add"), ["v1", "v4"])]
        out = "v5"
    elif expr == "gelu_tanh":
        body += [Assign("c0", Op("multiply"), ["v0", "v0"]), Assign("c1", Op("multiply"), ["c0", "v0"]),
                 Assign("c2", Op("multiply"), ["c1", 0.044715]), Assign("c3", Op("add"), ["v0", "c2"]),
                 Assign("c4", Op("multiply"), ["c3", 0.7978845608028654]), Assign("c5", Op("tanh"), ["c4"]),
                 Assign("c6", Op("add"), ["c5", 1.0]), Assign("c7", Op("multiply"), ["v0", 0.5]),
                 Assign("c8", Op("multiply"), ["c7", "c6"])]
        out = "c8"
    else:
        body += [Assign("v1", Op(expr), ["v0"])]
        out = "v1"
    body.append(Write("y", [Var("a0")], [out]))
    k = KernelOp(name, [Tile([a0], body)])
    g = _graph(k, [tensor("x", [n], "f32")], [tensor("y", [n], "f32")])
    return g, k, _launch(k, ["x", "y"], n)


def elementwise_kernel(n: int, inputs: dict, steps: list, out_dtype: str = "f32", name: str = "k_elementwise",
                       scalars: dict | None = None):
    """A general elementwise kernel: `inputs` maps buffer name -> dtype (each of n elements); `steps` is a list of
    (value name, op name, args) with args naming earlier values, the loaded inputs (by buffer name) or numbers;
    the last step's value is written to `out`. `scalars` maps the names of by-value parameters to 'f32' / 's32':
    they follow the buffers in `arg_order`, are described in the launch's `args` (emmyptx/kernel.py:166-178) and
    may be named by the steps like any value."""
    a0 = Axis("a0", Dim(n))
    body = [Load([b], b, [Var("a0")]) for b in inputs]
    body += [Assign(v, Op(op), list(args)) for v, op, args in steps]
    body.append(Write("out", [Var("a0")], [steps[-1][0]]))
    k = KernelOp(name, [Tile([a0], body)])
    g = _graph(k, [tensor(b, [n], dt) for b, dt in inputs.items()], [tensor("out", [n], out_dtype)])
    launch = _launch(k, [*inputs, "out", *(scalars or {})], n)
    if scalars:
        launch["args"] = ([{"name": b, "dtype": dt, "shape": [n]} for b, dt in inputs.items()] + [{"name": "out", "dtype": out_dtype, "shape": [n], "output": True}]
                          + [{"name": s, "dtype": dt, "shape": [], "scalar": True} for s, dt in scalars.items()])
    return g, k, launch


def broadcast_kernel(rows: int, cols: int, loads: list, steps: list, inputs: dict, name: str = "k_bcast"):
    """An elementwise kernel over a [rows, cols] tile whose inputs may be smaller than the tile: `loads` is a list of
    (value, buffer, axis names) -- a buffer indexed by ("r0", "c0") is the matrix, by ("c0",) a row vector, by ("r0",) a
    column vector -- `inputs` maps buffer -> shape (fp32), `steps` as in elementwise_kernel. The reference's broadcast cases:
    f_batch_norm_eval, m_outer, s_expand, p_bcast_rowcol (tools/torch_cases/fused.py:18-20, matmul.py:23, shapes.py:19,
    pointwise.py:56)."""
    r0, c0 = Axis("r0", Dim(rows)), Axis("c0", Dim(cols))
    body = [Load([v], buf, [Var(a) for a in axes]) for v, buf, axes in loads]
    body += [Assign(v, Op(op), list(args)) for v, op, args in steps]
    body.append(Write("out", [Var("r0"), Var("c0")], [steps[-1][0]]))
    k = KernelOp(name, [Tile([r0, c0], body)])
    g = _graph(k, [tensor(nm, shp, "f32") for nm, shp in inputs.items()], [tensor("out", [rows, cols], "f32")])
    return g, k, _launch(k, [*inputs, "out"], rows * cols)


def int_elementwise_kernel(n: int, steps: list, in_dtype: str = "i32", out_dtype: str = "i32", inputs=("a",), name: str = "k_int"):
    """An integer cell program: integer-typed Assigns over the s32 op table (emmyptx/ops.py:294-309) on i32 / i64 buffers of
    n elements each; `steps` as in elementwise_kernel."""
    a0 = Axis("a0", Dim(n))
    body = [Load([b], b, [Var("a0")]) for b in inputs]
    body += [Assign(v, Op(op), list(args), DType("int")) for v, op, args in steps]
    body.append(Write("out", [Var("a0")], [steps[-1][0]]))
    k = KernelOp(name, [Tile([a0], body)])
    g = _graph(k, [tensor(b, [n], in_dtype) for b in inputs], [tensor("out", [n], out_dtype)])
    return g, k, _launch(k, [*inputs, "out"], n)


def index_gather_kernel(n: int, mul: int = 7919, add: int = 13, div: int = 3, shift: int = 2, name: str = "k_gather"):
    """y[i] = (x[(i*mul + add) % n] // div) ^ (i >> shift), int32."""
    a0 = Axis("a0", Dim(n))
    i = Var("a0")
    idx = BinaryExpr("%", BinaryExpr("+", BinaryExpr("*", i, Literal(mul, "int")), Literal(add, "int")), Literal(n, "int"))
    body = [Load(["g"], "x", [idx]),
            Assign("q", Op("floor_divide"), ["g", div], "int"),
            Let("s", BinaryExpr(">>", i, Literal(shift, "int")), "int"),
            Assign("r", Op("bitwise_xor"), ["q", "s"], "int"),
            Write("y", [i], ["r"])]
    k = KernelOp(name, [Tile([a0], body)])
    g = _graph(k, [tensor("x", [n], "i32")], [tensor("y", [n], "i32")])
    return g, k, _launch(k, ["x", "y"], n)


def matmul_f32_kernel(m: int, n: int, k: int, batch: int = 1, b_trans: bool = False, b_batched: bool = True, bias: bool = False,
                      relu: bool = False, name: str = "k_mm_f32", a_trans: bool = False):
    """A float32 product the way the reference lowers it without tensor-core statements: one tile cell per output
    element, a loop over K folding a * b into an accumulator (emmyptx/kernel.py:786-797; the fma is formed from the
    multiply feeding the Accum), then the optional bias and ReLU, then the store."""
    axes = ([Axis("b0", Dim(batch))] if batch > 1 else []) + [Axis("m0", Dim(m)), Axis("n0", Dim(n))]
    lead = [Var("b0")] if batch > 1 else []
    b_lead = lead if (b_batched and batch > 1) else []
    b_index = b_lead + ([Var("n0"), Var("k0")] if b_trans else [Var("k0"), Var("n0")])
    a_index = lead + ([Var("k0"), Var("m0")] if a_trans else [Var("m0"), Var("k0")])           # a.t() @ b reads A[k, m]
    body = [Loop(Axis("k0", Dim(k)), [Load(["a"], "A", a_index), Load(["b"], "B", b_index),
                                      Assign("p", Op("multiply"), ["a", "b"]), Accum("acc", None, "p", Op("add"))])]
    out = "acc"
    ins = [tensor("A", ([batch] if batch > 1 else []) + ([k, m] if a_trans else [m, k]), "f32"),
           tensor("B", ([batch] if b_lead else []) + ([n, k] if b_trans else [k, n]), "f32")]
    if bias:
        ins.append(tensor("bias", [n], "f32"))
        body += [Load(["bv"], "bias", [Var("n0")]), Assign("s", Op("add"), [out, "bv"])]
        out = "s"
    if relu:
        body.append(Assign("r", Op("relu"), [out]))
        out = "r"
    body.append(Write("C", lead + [Var("m0"), Var("n0")], [out]))
    kern = KernelOp(name, [Tile(axes, body)])
    g = _graph(kern, ins, [tensor("C", ([batch] if batch > 1 else []) + [m, n], "f32")])
    return g, kern, _launch(kern, [t.name for t in ins] + ["C"], batch * m * n)


def colwise_kernel(op: str, rows: int, cols: int, eps: float = 1e-12, name: str = "k_colwise"):
    """The same statement shapes for a reduction over dim 0 of X[rows, cols]: one tile cell per column, the loop walks
    the rows (tools/torch_cases/reductions.py:9 `x.sum(0)`, fused.py:7 `softmax(x, 0)`)."""
    g, kern, launch = rowwise_kernel(op, cols, rows, eps, name)          # cells = columns, loop length = rows

    def swap(stmts):
        for s in stmts:
            if isinstance(s, (Load, Write)) and len(s.index) == 2:
                s.index = [s.index[1], s.index[0]]
            if isinstance(s, Loop):
                swap(s.body)
    swap(kern.body[0].body)
    is_map = op in ("softmax", "log_softmax", "normalize")
    g = _graph(kern, [tensor("X", [rows, cols], "f32")], [tensor("Y", [rows, cols] if is_map else [cols], "f32")])
    return g, kern, launch


def rowwise_kernel(op: str, rows: int, cols: int, eps: float = 1e-5, name: str = "k_rowwise", lanes: bool = False):
    """A reduction over the last axis of X[rows, cols] (or a normalisation built on one) in the statement shapes the
    reference lowers (emmyptx/kernel.py:786-797 `Accum` inside a `Loop`): one tile cell -- one thread of the reference's
    kernel -- per row, a loop per pass over the row. `lanes=True` appends a `WarpShuffle` after every loop (:856-866): the
    form a schedule with one warp per row ends its loops with; with one thread per row the reference's butterfly would
    add up 32 different rows, so that form is only for exercising the matcher, never compiled for its result."""
    r0, c0 = Axis("r0", Dim(rows)), Axis("c0", Dim(cols))
    ld = lambda: Load(["x"], "X", [Var("r0"), Var("c0")])
    shuffle = lambda st, o: [WarpShuffle([st], [st + "_b"], [Assign(st, Op(o), [st, st + "_b"])], 32)] if lanes else []
    fold = lambda st, o, pre=(): [Loop(c0, [ld(), *pre, Accum(st, None, pre[-1].name if pre else "x", Op(o))]), *shuffle(st, o)]
    inputs, body, out, is_map = [tensor("X", [rows, cols], "f32")], [], None, False
    if op in ("sum", "mean", "amax", "amin", "prod"):
        body = fold("acc", {"sum": "add", "mean": "add", "amax": "maximum", "amin": "minimum", "prod": "multiply"}[op])
        out = "acc"
        if op == "mean":
            body.append(Assign("m", Op("multiply"), ["acc", 1.0 / cols]))
            out = "m"
    elif op == "norm2":
        body = fold("acc", "add", [Assign("sq", Op("multiply"), ["x", "x"])]) + [Assign("n", Op("sqrt"), ["acc"])]
        out = "n"
    elif op == "dot":                                   # a matrix-vector product: the vector is the second input
        inputs.append(tensor("W", [cols], "f32"))
        body = [Loop(c0, [ld(), Load(["w"], "W", [Var("c0")]), Assign("p", Op("multiply"), ["x", "w"]), Accum("acc", None, "p", Op("add"))]),
                *shuffle("acc", "add")]
        out = "acc"
    elif op in ("var", "std", "layer_norm"):
        body = fold("acc", "add") + [Assign("mean", Op("multiply"), ["acc", 1.0 / cols])]
        body += fold("acc2", "add", [Assign("d", Op("subtract"), ["x", "mean"]), Assign("d2", Op("multiply"), ["d", "d"])])
        body.append(Assign("var", Op("multiply"), ["acc2", 1.0 / (cols if op == "layer_norm" else cols - 1)]))
        out = "var"
        if op == "std":
            body.append(Assign("sd", Op("sqrt"), ["var"]))
            out = "sd"
        if op == "layer_norm":
            inputs += [tensor("W", [cols], "f32"), tensor("B", [cols], "f32")]
            body += [Assign("ve", Op("add"), ["var", float(eps)]), Assign("rs", Op("rsqrt"), ["ve"]),
                     Loop(c0, [ld(), Load(["w"], "W", [Var("c0")]), Load(["b"], "B", [Var("c0")]),
                               Assign("d", Op("subtract"), ["x", "mean"]), Assign("n", Op("multiply"), ["d", "rs"]),
                               Assign("s", Op("multiply"), ["n", "w"]), Assign("o", Op("add"), ["s", "b"]),
                               Write("Y", [Var("r0"), Var("c0")], ["o"])])]
            is_map = True
    elif op in ("logsumexp", "softmax", "log_softmax"):
        body = fold("mx", "maximum")
        body += fold("se", "add", [Assign("d", Op("subtract"), ["x", "mx"]), Assign("e", Op("exp"), ["d"])])
        if op == "logsumexp":
            body += [Assign("l", Op("log"), ["se"]), Assign("o", Op("add"), ["l", "mx"])]
            out = "o"
        else:
            tail = ([Assign("o", Op("divide"), ["e", "se"])] if op == "softmax" else
                    [Assign("l", Op("log"), ["se"]), Assign("o", Op("subtract"), ["d", "l"])])
            body.append(Loop(c0, [ld(), Assign("d", Op("subtract"), ["x", "mx"]), Assign("e", Op("exp"), ["d"]), *tail,
                                  Write("Y", [Var("r0"), Var("c0")], ["o"])]))
            is_map = True
    elif op in ("rms_norm", "normalize"):
        body = fold("acc", "add", [Assign("sq", Op("multiply"), ["x", "x"])])
        if op == "rms_norm":
            inputs.append(tensor("W", [cols], "f32"))
            body += [Assign("ms", Op("multiply"), ["acc", 1.0 / cols]), Assign("ve", Op("add"), ["ms", float(eps)]),
                     Assign("rs", Op("rsqrt"), ["ve"]),
                     Loop(c0, [ld(), Load(["w"], "W", [Var("c0")]), Assign("n", Op("multiply"), ["x", "rs"]),
                               Assign("o", Op("multiply"), ["n", "w"]), Write("Y", [Var("r0"), Var("c0")], ["o"])])]
        else:
            body += [Assign("nrm", Op("sqrt"), ["acc"]), Assign("den", Op("maximum"), ["nrm", float(eps)]),
                     Loop(c0, [ld(), Assign("o", Op("divide"), ["x", "den"]), Write("Y", [Var("r0"), Var("c0")], ["o"])])]
        is_map = True
    else:
        raise KeyError(op)
    if not is_map:
        body.append(Write("Y", [Var("r0")], [out]))
    kern = KernelOp(name, [Tile([r0], body)])
    g = _graph(kern, inputs, [tensor("Y", [rows, cols] if is_map else [rows], "f32")])
    return g, kern, _launch(kern, [t.name for t in inputs] + ["Y"], rows * 32 if lanes else rows)


def gemm_kernel(m: int, n: int, k: int, dtype: str = "f16", epilogue: str | None = None, b_trans: bool = False,
                name: str = "k_gemm", batch: tuple = (), b_batched: bool = True, bias: bool = False,
                out_dtype: str | None = None, split_k: int = 1):
    """C = A B on mma.sync cells, as the tracer schedules a 16-bit matmul: accumulator / operand fragments, a K
    loop of fragment loads straight from global memory and MMAs, a fragment store (optionally with a fused
    epilogue, which the reference rejects, emmyptx/mma.py:201-203). One warp per 16x8 cell: the tile's axes are
    (batch,) row cell, column cell and the 32 lanes of the warp, so that the thread-to-cell map of
    emmyptx/kernel.py:551-626 hands every warp one cell and `mma.sync` runs warp-wide. Ragged extents carry the
    guards of emmyptx/mma.py:128-151, 217-242 (clamped rows / columns, zero K tail, predicated stores). The
    reference's compiler accepts this IR as it stands (without epilogue and bias); the tile sizes of the tracer's
    real schedule are unknown and do not matter to the matcher. `out_dtype="f32"` stores the accumulator without
    narrowing; `split_k` > 1 adds a tile axis that cuts the K loop into that many parts, each cell adding its partial
    sum into a zeroed f32 C (`atomic`: red.add.f32, emmyptx/mma.py:205-242)."""
    out_dtype = out_dtype or dtype
    k_cells = -(-k // 16)
    if split_k > 1 and (out_dtype != "f32" or k_cells % split_k):
        raise ValueError("split_k needs an f32 output and a K loop it divides")
    am, an = Axis("m0", Dim(-(-m // 16))), Axis("n0", Dim(-(-n // 8)))
    kk = Axis("k0", Dim(k_cells // split_k))
    lit = lambda v: Literal(int(v), "int")
    row, col = BinaryExpr("*", Var("m0"), lit(16)), BinaryExpr("*", Var("n0"), lit(8))
    kcell = Var("k0") if split_k == 1 else BinaryExpr("+", BinaryExpr("*", Var("s0"), lit(k_cells // split_k)), Var("k0"))
    kof = BinaryExpr("*", kcell, lit(16))
    lead = list(batch)
    bvar = [Var("b0")] if lead else []
    b_index = (bvar if b_batched else []) + ([col, kof] if b_trans else [kof, col])
    rag_m, rag_n, rag_k = m % 16 != 0, n % 8 != 0, k % 16 != 0
    a_load = LdmatrixLoad("_a", "a", "A", bvar + [row, kof], gmem_guard=(row, lit(m)) if rag_m else None,
                          k_zero=(kof, lit(k)) if rag_k else None)
    b_load = LdmatrixLoad("_b", "b", "B", b_index, b_trans=b_trans, gmem_guard=(col, lit(n)) if rag_n else None,
                          k_zero=(kof, lit(k)) if rag_k else None)
    body = [RegFragment("_c", "c", DType("f32")), RegFragment("_a", "a", DType(dtype)), RegFragment("_b", "b", DType(dtype)),
            Loop(kk, [a_load, b_load, MmaSyncPtx("_c", "_a", "_b", ab_dtype=dtype)]),
            RegStore("_c", "C", bvar + [row, col], epilogue=epilogue, bias="bias" if bias else None, atomic=split_k > 1,
                     m_guard=(row, lit(m)) if rag_m else None, n_guard=(col, lit(n)) if rag_n else None)]
    axes = (([Axis("b0", Dim(math.prod(lead)))] if lead else []) + ([Axis("s0", Dim(split_k))] if split_k > 1 else []) +
            [am, an, Axis("lane0", Dim(32))])
    kern = KernelOp(name, [Tile(axes, body)])
    bshape = [n, k] if b_trans else [k, n]
    flat = [math.prod(lead)] if lead else []
    ins = [tensor("A", flat + [m, k], dtype), tensor("B", (flat if b_batched else []) + bshape, dtype)]
    if bias:
        ins.append(tensor("bias", [n], out_dtype))
    g = _graph(kern, ins, [tensor("C", flat + [m, n], out_dtype)])
    cells = math.prod(lead or [1]) * split_k * am.extent.value * an.extent.value * 32
    return g, kern, _launch(kern, [t.name for t in ins] + ["C"], cells, block=128)


def attention_kernel(units_shape: list[int], seq_q: int, seq_k: int, d: int, dtype: str = "bf16", scale: float | None = None,
                     name: str = "k_sdpa", causal: bool = False, mask: str | None = None):
    """softmax(Q K^T * scale) V as fused statements: two MMA groups with a scaled, optionally masked exponential and
    two row reductions between them, written per (query, key) pair -- the tile's last axis counts queries, the loop
    keys. Only what the matcher reads is spelled out, and the softmax works on fragment names directly, which the
    reference's compiler has no statement for (its tracer stages S through shared memory): this IR is NOT accepted
    by the reference, unlike every other builder here. `causal` adds the lower-triangular mask the way
    `masked_fill(~tril, -inf)` lowers: `less_equal(key, query)` feeding a `where`. `mask` selects other masks
    ("upper", "band", "padding") that the matcher must refuse."""
    scale = d ** -0.5 if scale is None else scale
    kind = mask or ("causal" if causal else None)
    masks = {
        None: [],
        "causal": [Assign("keep", Op("less_equal"), [Var("j0"), Var("q0")])],
        "upper": [Assign("keep", Op("greater_equal"), [Var("j0"), Var("q0")])],
        "band": [Assign("lo", Op("subtract"), [Var("q0"), 16]), Assign("k1", Op("less_equal"), [Var("j0"), Var("q0")]),
                 Assign("k2", Op("greater"), [Var("j0"), "lo"]), Assign("keep", Op("multiply"), ["k1", "k2"])],
        "padding": [Assign("keep", Op("less"), [Var("j0"), seq_k - 8])],
    }[kind]
    fill = [Assign("t0", Op("where"), ["keep", "t0", float("-inf")])] if masks else []
    u = 1
    for s in units_shape:
        u *= s
    ax = [Axis("u0", Dim(u)), Axis("q0", Dim(seq_q))]
    body = [RegFragment("_s", "c", DType("f32")), RegFragment("_o", "c", DType("f32")),
            RegFragment("_q", "a", DType(dtype)), RegFragment("_k", "b", DType(dtype)), RegFragment("_v", "b", DType(dtype)),
            Loop(Axis("j0", Dim(seq_k)), [
                LdmatrixLoad("_q", "a", "Q", [Var("u0"), Var("q0"), Literal(0, "int")]),
                LdmatrixLoad("_k", "b", "K", [Var("u0"), Var("j0"), Literal(0, "int")], b_trans=True),
                MmaSyncPtx("_s", "_q", "_k", ab_dtype=dtype),
                Assign("t0", Op("multiply"), ["_s", scale]), *masks, *fill,
                WarpShuffle(["mx"], ["mx_b"], [Assign("mx", Op("maximum"), ["mx", "mx_b"])], 4),
                Assign("t1", Op("subtract"), ["t0", "mx"]), Assign("p", Op("exp"), ["t1"]),
                WarpShuffle(["sm"], ["sm_b"], [Assign("sm", Op("add"), ["sm", "sm_b"])], 4),
                LdmatrixLoad("_v", "b", "V", [Var("u0"), Var("j0"), Literal(0, "int")]),
                MmaSyncPtx("_o", "p", "_v", ab_dtype=dtype)]),
            Assign("o", Op("divide"), ["_o", "sm"]),
            RegStore("_o", "O", [Var("u0"), Var("q0"), Literal(0, "int")])]
    kern = KernelOp(name, [Tile(ax, body)])
    shp = list(units_shape)
    g = _graph(kern, [tensor("Q", shp + [seq_q, d], dtype), tensor("K", shp + [seq_k, d], dtype),
                      tensor("V", shp + [seq_k, d], dtype)], [tensor("O", shp + [seq_q, d], dtype)])
    return g, kern, _launch(kern, ["Q", "K", "V", "O"], u * -(-seq_q // 16) * 32, block=128)


def attention_scalar_kernel(units_shape: list[int], seq_q: int, seq_k: int, d: int, dtype: str = "f32", scale: float | None = None,
                            causal: bool = False, mask: str | None = None, name: str = "k_sdpa_f32"):
    """softmax(Q K^T * scale) V on float32 buffers the way the reference lowers a fused expression without tensor-core
    statements (tools/torch_cases/fused.py:21-22, 31-36; models.py:17-19): one tile cell per output element, dot
    products as a `Loop` folding q * k with an `Accum` (emmyptx/kernel.py:786-797; every loop seeds the accumulators
    directly inside it, emmyptx/loops.py:92-102), a first pass over the keys for the row maximum and a second one for
    the sum of exponentials and the weighted sum of V. Only statements the reference's compiler has are used, so it
    compiles this kernel too. `causal` / `mask` as in attention_kernel."""
    scale = d ** -0.5 if scale is None else scale
    kind = mask or ("causal" if causal else None)
    add, mx = Op("add", 0.0), Op("maximum", float("-inf"))

    def keep(j):
        return {None: [],
                "causal": [Assign("keep", Op("less_equal"), [j, "q0"])],        # axis variables are names like any other
                "upper": [Assign("keep", Op("greater_equal"), [j, "q0"])],
                "padding": [Assign("keep", Op("less"), [j, seq_k - 8])]}[kind]

    def scores(j, k, out):
        dot = Loop(Axis(k, Dim(d)), [Load(["qv"], "Q", [Var("u0"), Var("q0"), Var(k)]), Load(["kv"], "K", [Var("u0"), Var(j), Var(k)]),
                                    Assign("pr", Op("multiply"), ["qv", "kv"]), Accum("dot_" + out, None, "pr", add)])
        fill = [Assign(out, Op("where"), ["keep", out, float("-inf")])] if kind else []
        return [dot, Assign(out, Op("multiply"), ["dot_" + out, scale]), *keep(j), *fill]

    u = 1
    for s in units_shape:
        u *= s
    body = [Loop(Axis("j0", Dim(seq_k)), [*scores("j0", "k0", "t"), Accum("mx", None, "t", mx)]),
            Loop(Axis("j1", Dim(seq_k)), [*scores("j1", "k1", "t2"), Assign("dl", Op("subtract"), ["t2", "mx"]), Assign("e", Op("exp"), ["dl"]),
                                          Accum("den", None, "e", add), Load(["vv"], "V", [Var("u0"), Var("j1"), Var("c0")]),
                                          Assign("pv", Op("multiply"), ["e", "vv"]), Accum("num", None, "pv", add)]),
            Assign("o", Op("divide"), ["num", "den"]),
            Write("O", [Var("u0"), Var("q0"), Var("c0")], ["o"])]
    kern = KernelOp(name, [Tile([Axis("u0", Dim(u)), Axis("q0", Dim(seq_q)), Axis("c0", Dim(d))], body)])
    g = _graph(kern, [tensor("Q", [u, seq_q, d], dtype), tensor("K", [u, seq_k, d], dtype), tensor("V", [u, seq_k, d], dtype)],
               [tensor("O", [u, seq_q, d], dtype)])
    return g, kern, _launch(kern, ["Q", "K", "V", "O"], u * seq_q * d)


def layout_kernel(case: str, name: str | None = None):
    """The reference's data-movement cases (tools/torch_cases/shapes.py:6-19) as one-cell-per-element tiles whose Loads and
    Write index their buffers with expressions of the axis variables -- what a tracer hands over for a transpose, a
    slice or a flip -- plus masks made of the axis variables themselves (tril) and a concatenation written slice by
    slice (`s_cat_a`, `s_cat_b`: two kernels over one output), and the two pooling cases of tools/torch_cases/conv.py:8-9 with
    their windows spelled out as shifted loads. Returns (graph, kernel, launch)."""
    lit = lambda v: Literal(int(v), "int")
    add = lambda a, b: BinaryExpr("+", a, b)
    mul = lambda a, b: BinaryExpr("*", a, b)
    sub = lambda a, b: BinaryExpr("-", a, b)
    A = lambda nm, n: Axis(nm, Dim(n))
    cases = {
        # name: (axes, inputs {buffer: shape}, loads [(value, buffer, index)], assigns, out shape, out index, value)
        "s_transpose": ([A("i0", 96), A("j0", 64)], {"X": [64, 96]}, [("x", "X", [Var("j0"), Var("i0")])], [], [96, 64], [Var("i0"), Var("j0")], "x"),
        "s_permute": ([A("a0", 32), A("b0", 8), A("c0", 16)], {"X": [8, 16, 32]}, [("x", "X", [Var("b0"), Var("c0"), Var("a0")])],
                      [Assign("y", Op("multiply"), ["x", 2.0])], [32, 8, 16], [Var("a0"), Var("b0"), Var("c0")], "y"),
        "s_slice": ([A("r0", 64), A("c0", 40)], {"X": [64, 128]}, [("x", "X", [Var("r0"), add(Var("c0"), lit(10))])],
                    [Assign("y", Op("multiply"), ["x", 2.0])], [64, 40], [Var("r0"), Var("c0")], "y"),
        "s_strided_slice": ([A("i0", 512)], {"X": [1024]}, [("x", "X", [mul(Var("i0"), lit(2))])], [Assign("y", Op("add"), ["x", 1.0])],
                            [512], [Var("i0")], "y"),
        "s_flip": ([A("r0", 64), A("c0", 128)], {"X": [64, 128]}, [("x", "X", [Var("r0"), sub(lit(127), Var("c0"))])], [], [64, 128],
                   [Var("r0"), Var("c0")], "x"),
        "s_repeat": ([A("t0", 2), A("r0", 32), A("c0", 64)], {"X": [32, 64]}, [("x", "X", [Var("r0"), Var("c0")])],
                     [Assign("y", Op("add"), ["x", 0.0])], [64, 64], [add(mul(Var("t0"), lit(32)), Var("r0")), Var("c0")], "y"),
        "s_stack": ([A("s0", 2), A("r0", 32), A("c0", 64)], {"A": [32, 64], "B": [32, 64]},
                    [("a", "A", [Var("r0"), Var("c0")]), ("b", "B", [Var("r0"), Var("c0")])],
                    [Assign("first", Op("equal"), ["s0", 0.0]), Assign("y", Op("where"), ["first", "a", "b"])], [2, 32, 64],
                    [Var("s0"), Var("r0"), Var("c0")], "y"),
        "s_tril": ([A("r0", 64), A("c0", 64)], {"X": [64, 64]}, [("x", "X", [Var("r0"), Var("c0")])],
                   [Assign("keep", Op("less_equal"), ["c0", "r0"]), Assign("y", Op("where"), ["keep", "x", 0.0])], [64, 64],
                   [Var("r0"), Var("c0")], "y"),
        "s_cat_a": ([A("r0", 32), A("c0", 64)], {"A": [32, 64]}, [("a", "A", [Var("r0"), Var("c0")])], [], [32, 112], [Var("r0"), Var("c0")], "a"),
        "s_cat_b": ([A("r0", 32), A("c0", 48)], {"B": [32, 48]}, [("b", "B", [Var("r0"), Var("c0")])], [], [32, 112],
                    [Var("r0"), add(Var("c0"), lit(64))], "b"),
        # pooling windows spelled out (tools/torch_cases/conv.py:8-9): a handful of shifted loads folded by the Assign chain
        "c_avg_pool1d": ([A("c0", 16), A("i0", 32)], {"X": [16, 128]},
                         [(f"x{t}", "X", [Var("c0"), add(mul(Var("i0"), lit(4)), lit(t))]) for t in range(4)],
                         [Assign("s0_", Op("add"), ["x0", "x1"]), Assign("s1_", Op("add"), ["x2", "x3"]), Assign("s2_", Op("add"), ["s0_", "s1_"]),
                          Assign("y", Op("multiply"), ["s2_", 0.25])], [16, 32], [Var("c0"), Var("i0")], "y"),
        "c_max_pool2d": ([A("c0", 8), A("i0", 16), A("j0", 16)], {"X": [8, 32, 32]},
                         [(f"x{di}{dj}", "X", [Var("c0"), add(mul(Var("i0"), lit(2)), lit(di)), add(mul(Var("j0"), lit(2)), lit(dj))])
                          for di in range(2) for dj in range(2)],
                         [Assign("m0_", Op("maximum"), ["x00", "x01"]), Assign("m1_", Op("maximum"), ["x10", "x11"]),
                          Assign("y", Op("maximum"), ["m0_", "m1_"])], [8, 16, 16], [Var("c0"), Var("i0"), Var("j0")], "y"),
        # the same mask as s_tril spelled as a Select on the axis variables (emmyptx/kernel.py:812-822), and a window of
        # columns kept through a Let of a compound predicate (`F.pad`-like masking; emmyptx/kernel.py:344-369)
        "s_tril_select": ([A("r0", 64), A("c0", 64)], {"X": [64, 64]}, [("x", "X", [Var("r0"), Var("c0")])],
                          [Select("y", [Branch(BinaryExpr("<=", Var("c0"), Var("r0")), "x"), Branch(None, 0.0)])], [64, 64],
                          [Var("r0"), Var("c0")], "y"),
        "s_window_let": ([A("r0", 64), A("c0", 128)], {"X": [64, 128]}, [("x", "X", [Var("r0"), Var("c0")])],
                         [Let("inside", BinaryExpr("&&", BinaryExpr(">=", Var("c0"), lit(3)), BinaryExpr("<", Var("c0"), lit(120)))),
                          Assign("m", Op("where"), ["inside", "x", 0.0]), Assign("y", Op("multiply"), ["m", 2.0])], [64, 128],
                         [Var("r0"), Var("c0")], "y"),
        # torch.cat([a, b], -1) (shapes.py:13) as one kernel: a Cond on the column picks the source (emmyptx/kernel.py:825-840)
        "s_cat_cond": ([A("r0", 32), A("c0", 112)], {"A": [32, 64], "B": [32, 48]}, [],
                       [Cond(BinaryExpr("<", Var("c0"), lit(64)),
                             [Load(["a"], "A", [Var("r0"), Var("c0")]), Write("out", [Var("r0"), Var("c0")], ["a"])],
                             [Load(["b"], "B", [Var("r0"), sub(Var("c0"), lit(64))]), Write("out", [Var("r0"), Var("c0")], ["b"])])],
                       [32, 112], None, None),
        # F.pad(x, (3, 3)) as a Cond: inside the window the shifted element, zero in the border
        "s_pad_cond": ([A("r0", 8), A("c0", 70)], {"X": [8, 64]}, [],
                       [Cond(BinaryExpr("&&", BinaryExpr(">=", Var("c0"), lit(3)), BinaryExpr("<", Var("c0"), lit(67))),
                             [Load(["x"], "X", [Var("r0"), sub(Var("c0"), lit(3))]), Write("out", [Var("r0"), Var("c0")], ["x"])],
                             [Write("out", [Var("r0"), Var("c0")], [0.0])])],
                       [8, 70], None, None),
        # a rotation: the index wraps around along one axis
        "s_roll": ([A("r0", 64), A("c0", 128)], {"X": [64, 128]}, [("x", "X", [Var("r0"), BinaryExpr("%", add(Var("c0"), lit(125)), lit(128))])], [],
                   [64, 128], [Var("r0"), Var("c0")], "x"),
    }
    if case in ("s_embedding", "s_gather"):
        # an index read from an integer buffer, made non-negative and reduced (`idx.abs() % n`, shapes.py:20-24), then used as
        # a coordinate of the second Load
        emb = case == "s_embedding"
        axes = [A("i0", 64), A("j0", 32)] if emb else [A("r0", 32), A("k0", 8)]
        idx_index = [Var("i0")] if emb else [Var("r0"), Var("k0")]
        src_index = [Var("m"), Var("j0")] if emb else [Var("r0"), Var("m")]
        body = [Load(["t"], "IDX", idx_index), Assign("a", Op("abs"), ["t"], DType("int")),
                Assign("m", Op("mod"), ["a", 100 if emb else 64], DType("int")), Load(["v"], "SRC", src_index),
                Write("out", [Var(axes[0].name), Var(axes[1].name)], ["v"])]
        kern = KernelOp(name or f"k_{case}", [Tile(axes, body)])
        g = _graph(kern, [tensor("IDX", [64] if emb else [32, 8], "i64"), tensor("SRC", [100, 32] if emb else [32, 64], "f32")],
                   [tensor("out", [64, 32] if emb else [32, 8], "f32")])
        return g, kern, _launch(kern, ["IDX", "SRC", "out"], axes[0].extent.value * axes[1].extent.value)
    axes, ins, loads, assigns, out_shape, out_index, value = cases[case]
    body = [Load([v], buf, idx) for v, buf, idx in loads] + list(assigns) + ([Write("out", out_index, [value])] if out_index is not None else [])
    kern = KernelOp(name or f"k_{case}", [Tile(axes, body)])
    cells = 1
    for a in axes:
        cells *= a.extent.value
    g = _graph(kern, [tensor(b, shp, "f32") for b, shp in ins.items()], [tensor("out", out_shape, "f32")])
    return g, kern, _launch(kern, [*ins, "out"], cells)


def conv_kernel(case: str = "c_conv1d", name: str | None = None):
    """The reference's convolution cases (tools/torch_cases/conv.py:6-7) as scalar loops: one tile cell per output element,
    nested Loops over the input channels and the taps folding w * x into an accumulator (emmyptx/kernel.py:786-797;
    every Loop seeds the accumulators directly inside it, emmyptx/loops.py:92-102, so only the innermost body holds the
    Accum and the accumulator is carried across the outer trips by `seed=False` on the inner Loops)."""
    lit = lambda v: Literal(int(v), "int")
    add = lambda a, b: BinaryExpr("+", a, b)
    if case == "c_conv1d":              # x [1, 16, 128], w [32, 16, 3] -> [1, 32, 126]
        axes = [Axis("o0", Dim(32)), Axis("i0", Dim(126))]
        inner = [Load(["wv"], "W", [Var("o0"), Var("c0"), Var("t0")]), Load(["xv"], "X", [Var("c0"), add(Var("i0"), Var("t0"))]),
                 Assign("p", Op("multiply"), ["wv", "xv"]), Accum("acc", None, "p", Op("add", 0.0))]
        body = [Init("acc", 0.0), Loop(Axis("c0", Dim(16)), [Loop(Axis("t0", Dim(3)), inner, seed=False)], seed=False),
                Write("out", [Var("o0"), Var("i0")], ["acc"])]
        ins, out_shape = [tensor("X", [16, 128], "f32"), tensor("W", [32, 16, 3], "f32")], [32, 126]
    elif case == "c_conv2d":            # x [1, 8, 32, 32], w [16, 8, 3, 3] -> [1, 16, 30, 30]
        axes = [Axis("o0", Dim(16)), Axis("i0", Dim(30)), Axis("j0", Dim(30))]
        inner = [Load(["wv"], "W", [Var("o0"), Var("c0"), Var("u0"), Var("v0")]),
                 Load(["xv"], "X", [Var("c0"), add(Var("i0"), Var("u0")), add(Var("j0"), Var("v0"))]),
                 Assign("p", Op("multiply"), ["wv", "xv"]), Accum("acc", None, "p", Op("add", 0.0))]
        body = [Init("acc", 0.0),
                Loop(Axis("c0", Dim(8)), [Loop(Axis("u0", Dim(3)), [Loop(Axis("v0", Dim(3)), inner, seed=False)], seed=False)], seed=False),
                Write("out", [Var("o0"), Var("i0"), Var("j0")], ["acc"])]
        ins, out_shape = [tensor("X", [8, 32, 32], "f32"), tensor("W", [16, 8, 3, 3], "f32")], [16, 30, 30]
    else:
        raise KeyError(case)
    kern = KernelOp(name or f"k_{case}", [Tile(axes, body)])
    cells = 1
    for a in axes:
        cells *= a.extent.value
    g = _graph(kern, ins, [tensor("out", out_shape, "f32")])
    return g, kern, _launch(kern, ["X", "W", "out"], cells)


def rename_buffers(built, mapping: dict):
    """(graph, kernel, launch) with buffers renamed old -> new everywhere they are named: tensor and node names, Load
    and Write targets, the launch's argument order. The builders above use fixed names (A, B, C, X, Y ...); a problem
    of several kernels passes buffers on by name (tools/run_local.py:90-91, 132-133), so its kernels need names of
    their own."""
    graph, kernel, launch = built

    def swap(x):
        if isinstance(x, str):
            return mapping.get(x, x)
        if isinstance(x, list):
            return [swap(v) for v in x]
        if isinstance(x, dict):
            return {swap(k) if k != "__node__" else k: (v if k == "__node__" else swap(v)) for k, v in x.items()}
        return x
    value_names = {n for s in _walk_statements(kernel.body) for n in (getattr(s, "names", None) or [getattr(s, "name", None)]) if isinstance(n, str)}
    clash = value_names & (set(mapping) | set(mapping.values()))
    if clash:
        raise ValueError(f"{sorted(clash)} name values inside the kernel: not buffers, or new names that would shadow them")
    g2 = from_jsonable(swap(to_jsonable(graph)))
    k2 = next(n.op for n in g2.nodes.values() if type(n.op).__name__ == "KernelOp")
    return g2, k2, swap(launch)


def _walk_statements(body):
    for s in body:
        yield s
        sub = getattr(s, "body", None)
        if isinstance(sub, list):
            yield from _walk_statements(sub)

