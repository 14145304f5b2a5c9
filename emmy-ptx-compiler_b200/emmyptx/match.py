"""Kernel IR -> precompiled sm_100a kernel variant.

Where the reference's `KernelCompiler` prints PTX statement by statement, the replacement ships a fixed set
of hand-written kernels. This module decides which of them computes a given `KernelOp`, and with which
parameters -- or that none does, which is a `CompileError` (there is no generic fallback and no CPU path).

Streaming kernels are recognised by behaviour, not by spelling: the cell program (Load / Let / Assign /
Write under one `Tile`, the statements of `emmyptx/kernel.py:632-822`) is run on a handful of probe cells
in float64 / exact integers over synthetic buffer contents, and compared with what each kernel variant
computes for the same cells. Two programs that mean the same thing match the same kernel, however the
tracer happened to arrange them. Contractions are recognised by their tensor-core statements
(`RegFragment` / `LdmatrixLoad` / `MmaSyncPtx` / `RegStore`, `emmyptx/mma.py`), whose buffers, layout flags
and epilogue give the GEMM's parameters; the tile sizes the tracer chose are irrelevant here. Row reductions
(`Loop` / `Accum` under a tile over the rows) are recognised by behaviour too, a few probe rows at a time.
"""
from __future__ import annotations

import math

import numpy as np

from .ops import FLOAT_OPS, INT_OPS, INT_OPS_TRUNC, MOVE_OPS, OpError, Program, lower_int_op, lower_op

INT_DTYPES = {"int", "i32", "i64", "int32", "int64", "u32", "u8", "i8"}      # emmyptx/kernel.py:41
_FUNC_ALIASES = {"fmax": "maximum", "fmin": "minimum", "fabs": "abs"}       # emmyptx/kernel.py:55


class Unmatched(Exception):
    """The IR is well-formed but no kernel variant computes it."""


def children(stmt) -> list:
    out = []
    for attr in ("body", "else_body", "combine_states"):
        sub = getattr(stmt, attr, None)
        if sub is not None and not isinstance(sub, (str, bytes)):
            out.append(sub)
    return out


def walk(body):
    """Every statement in `body`, nested ones included (emmyptx/loops.py:51-56)."""
    for s in body:
        yield s
        for sub in children(s):
            yield from walk(sub)


def _kind(x) -> str:
    return type(x).__name__


def _dtype_name(dt):
    return None if dt is None else getattr(dt, "name", dt)


def tensor_table(graph) -> dict:
    """name -> (shape, dtype) for every tensor the graph knows (emmyptx/kernel.py:122-125)."""
    out = {}
    for node in graph.nodes.values():
        for t in node.outputs:
            out[t.name] = (tuple(int(d.as_static()) for d in t.shape) or (1,), _dtype_name(t.dtype))
    return out


# ---- probe buffers: contents as a pure function of the element index -------------------------------------
def _hash(idx: np.ndarray, salt: int) -> np.ndarray:
    h = (idx.astype(np.uint64) + np.uint64(salt)) * np.uint64(0x9E3779B97F4A7C15)
    h ^= h >> np.uint64(29)
    h *= np.uint64(0xBF58476D1CE4E5B9)
    h ^= h >> np.uint64(32)
    return h


def probe_values(name: str, dtype: str, idx: np.ndarray) -> np.ndarray:
    salt = sum(ord(c) * 131 ** i for i, c in enumerate(name)) % (2**31)
    h = _hash(idx, salt)
    if dtype in ("i32", "i64"):
        return (h % np.uint64(2**31 + 1)).astype(np.int64) - 2**30
    return (h % np.uint64(2**24)).astype(np.float64) / 2**24 * 8.0 - 4.0


# ---- the cell interpreter -----------------------------------------------------------------------------------
class CellInterpreter:
    """Runs a pointwise cell program on `cells` (flat cell ids) with numpy arrays as values."""

    def __init__(self, tensors: dict, cells: np.ndarray, int_ops: dict) -> None:
        self.tensors, self.cells, self.int_ops = tensors, cells, int_ops
        self.env: dict = {}
        self.loads: list = []       # (buffer, flat index array)
        self.writes: list = []      # (buffer, flat index array, [value arrays])
        self.program = Program()

    def lookup(self, name):
        if isinstance(name, bool):
            return np.full(self.cells.shape, float(name))
        if isinstance(name, int):
            return np.full(self.cells.shape, name, dtype=np.int64)
        if isinstance(name, float):
            return np.full(self.cells.shape, name, dtype=np.float64)
        if name not in self.env:
            raise Unmatched(f"use of undefined name {name!r}")
        return self.env[name]

    @staticmethod
    def _is_int(v) -> bool:
        return np.asarray(v).dtype.kind in "iub"

    def expr(self, e):
        k = _kind(e)
        if k == "Literal":
            if isinstance(e.value, bool):
                return np.full(self.cells.shape, e.value)
            dt = _dtype_name(e.dtype)
            if dt in INT_DTYPES or (dt is None and isinstance(e.value, int)):
                return np.full(self.cells.shape, int(e.value), dtype=np.int64)
            return np.full(self.cells.shape, float(e.value), dtype=np.float64)
        if k == "Var":
            return self.lookup(e.name)
        if k == "BinaryExpr":
            return self.binary(e.op, self.expr(e.left), self.expr(e.right))
        if k == "TernaryExpr":
            return np.where(self.truthy(self.expr(e.cond)), self.expr(e.if_true), self.expr(e.if_false))
        if k == "CastExpr":
            v = self.expr(e.expr)
            return np.trunc(v).astype(np.int64) if e.dtype in INT_DTYPES else np.asarray(v, dtype=np.float64)
        if k == "FuncCallExpr":
            name = _FUNC_ALIASES.get(e.name, e.name)
            if name not in FLOAT_OPS:
                raise OpError(f"elementwise op {name!r} is not supported")
            return FLOAT_OPS[name][1](*[np.asarray(self.expr(a), dtype=np.float64) for a in e.args])
        if k == "FlatIndex":
            return self.flat_index(e.buffer, e.index)
        raise Unmatched(f"unsupported expression {k}")

    @staticmethod
    def truthy(v):
        return np.asarray(v) != 0

    def binary(self, op, a, b):
        if op in ("&&", "||"):
            return (self.truthy(a) & self.truthy(b)) if op == "&&" else (self.truthy(a) | self.truthy(b))
        cmp = {"<": np.less, "<=": np.less_equal, ">": np.greater, ">=": np.greater_equal, "==": np.equal, "!=": np.not_equal}
        if op in cmp:
            return cmp[op](a, b)
        if not (self._is_int(a) and self._is_int(b)):
            f = {"+": np.add, "-": np.subtract, "*": np.multiply, "/": np.divide, "max": np.maximum, "min": np.minimum}
            if op not in f:
                raise Unmatched(f"float operator {op!r} is not supported")
            return f[op](np.asarray(a, np.float64), np.asarray(b, np.float64))
        a, b = np.asarray(a, np.int64), np.asarray(b, np.int64)
        # Index arithmetic is exact (no int32 wrap): for the power-of-two moduli the reference's masks
        # assume, the wrapped and the exact value agree (emmyptx/intmath.py:108-116, :231-233).
        if op in ("/", "//"):
            q = np.abs(a) // np.abs(b)
            return np.where((a < 0) != (b < 0), -q, q)
        if op == "%":
            return np.mod(a, b) if np.all(b > 0) else a - b * np.trunc(a / b).astype(np.int64)
        f = {"+": np.add, "-": np.subtract, "*": np.multiply, "<<": np.left_shift, ">>": np.right_shift, "&": np.bitwise_and,
             "|": np.bitwise_or, "^": np.bitwise_xor, "max": np.maximum, "min": np.minimum}
        if op not in f:
            raise Unmatched(f"integer operator {op!r} is not supported")
        return f[op](a, b)

    def flat_index(self, buffer: str, index) -> np.ndarray:
        """Row-major element offset (emmyptx/kernel.py:410-421)."""
        index = list(index)
        if buffer not in self.tensors:
            raise Unmatched(f"unknown buffer {buffer!r}")
        shape = self.tensors[buffer][0]
        if len(shape) != len(index):
            shape = (1,) * len(index)
        flat = np.zeros(self.cells.shape, dtype=np.int64)
        for dim, e in enumerate(index):
            flat = flat * shape[dim] + np.asarray(self.expr(e), dtype=np.int64)
        return flat

    def run(self, stmts) -> None:
        for s in stmts:
            k = _kind(s)
            if k == "Load":
                flat = self.flat_index(s.input, s.index)
                dtype = self.tensors[s.input][1]
                for j, name in enumerate(s.names):
                    self.env[name] = probe_values(s.input, dtype, flat + j)
                self.loads.append((s.input, flat, len(s.names)))
            elif k == "Let":
                v = self.expr(s.value)
                dt = _dtype_name(s.dtype)
                if dt is not None:
                    v = np.trunc(v).astype(np.int64) if dt in INT_DTYPES else np.asarray(v, np.float64)
                self.env[s.name] = v
            elif k == "Assign":
                is_int = _dtype_name(s.dtype) in INT_DTYPES
                args = [self.lookup(a) for a in s.args]
                if is_int:
                    lower_int_op(self.program, s.op.name, list(s.args), s.name)
                    self.env[s.name] = self.int_ops[s.op.name][1](*[np.asarray(a, np.int64) for a in args])
                else:
                    lower_op(self.program, s.op.name, list(s.args), s.name)
                    self.env[s.name] = FLOAT_OPS[s.op.name][1](*[np.asarray(a, np.float64) for a in args])
            elif k == "Write":
                if getattr(s, "atomic", False):
                    raise Unmatched("atomic writes belong to split-K schedules, which have no variant")
                self.writes.append((s.output, self.flat_index(s.output, s.index), [self.lookup(v) for v in s.values]))
            else:
                raise Unmatched(f"statement {k} inside a streaming tile has no kernel variant")


# ---- variants -------------------------------------------------------------------------------------------------
POINTWISE_F64 = {
    "exp_sin_tanh": lambda x: np.exp(x) + np.sin(x) * np.tanh(x),
    "exp": np.exp, "sin": np.sin, "cos": np.cos, "tanh": np.tanh,
    "gelu_tanh": lambda x: 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x**3))),
    "sigmoid": lambda x: 1.0 / (1.0 + np.exp(-x)), "silu": lambda x: x / (1.0 + np.exp(-x)), "relu": lambda x: np.maximum(x, 0.0),
}


def _int_literals(kernel) -> set:
    """Every integer constant spelled in the kernel: Literals in expressions and numeric Assign arguments."""
    found = set()

    def visit(x):
        if _kind(x) == "Literal" and isinstance(x.value, int) and not isinstance(x.value, bool):
            found.add(int(x.value))
        for attr in ("left", "right", "cond", "if_true", "if_false", "expr", "value"):
            sub = getattr(x, attr, None)
            if sub is not None and not isinstance(sub, (str, int, float, bool)):
                visit(sub)
        for attr in ("args", "index"):
            for sub in getattr(x, attr, None) or []:
                if isinstance(sub, int) and not isinstance(sub, bool):
                    found.add(sub)
                elif not isinstance(sub, (str, float, bool)):
                    visit(sub)

    for s in walk(kernel.body):
        visit(s)
    return found


PW_SLOTS, PW_CONSTS, PW_STEPS, PW_INPUTS = 16, 16, 48, 4
PW_OP_NAMES = {"add", "subtract", "multiply", "divide", "maximum", "minimum", "relu", "square", "copy", "negative", "abs",
               "reciprocal", "sqrt", "rsqrt", "exp", "exp_fast", "log", "sigmoid", "tanh", "erf", "sin", "cos", "pow", "equal",
               "not_equal", "greater", "less", "greater_equal", "less_equal", "where", "bitwise_and", "bitwise_or",
               "bitwise_not", "floor_divide", "mod", "remainder", *MOVE_OPS}


def scalar_args(launch: dict) -> dict:
    """name -> 'f32' | 's32' for the launch's scalar parameters (passed by value: emmyptx/kernel.py:171-178)."""
    return {a["name"]: ("f32" if a.get("dtype", "f32") == "f32" else "s32") for a in launch.get("args", []) if a.get("scalar")}


def build_program(tile, tensors: dict, out_name: str, out_value_name, integer: bool = False, scalars: dict | None = None) -> dict:
    """The tile's cell program as data for the general elementwise kernel: inputs in slots 0.., one slot per live
    value (slots are reused once a value is dead), numeric operands in the constant table. `integer`: an s32 program
    (every Assign integer-typed, ops from the integer table, constants whole numbers). A scalar parameter of the
    launch gets a constant slot of its own, filled with its value when the kernel is launched (`scalar_consts`)."""
    scalars = scalars or {}
    scalar_slot: dict = {}
    stmts = list(tile.body)
    inputs, slot_of = [], {}
    for s in stmts:
        if _kind(s) == "Load":
            if s.input not in inputs:
                inputs.append(s.input)
            slot_of[s.names[0]] = inputs.index(s.input)
    if len(inputs) > PW_INPUTS:
        raise Unmatched(f"{len(inputs)} input buffers: the general elementwise kernel takes {PW_INPUTS}")
    assigns = [s for s in stmts if _kind(s) == "Assign"]
    if any(_kind(s) not in ("Load", "Assign", "Write") for s in stmts):
        raise Unmatched("the general elementwise kernel runs Load / Assign / Write programs")
    last_use = {}
    for i, s in enumerate(assigns):
        for a in s.args:
            if isinstance(a, str):
                last_use[a] = i
    last_use[out_value_name] = len(assigns)
    free = [k for k in range(PW_SLOTS - 1, len(inputs) - 1, -1)]
    consts, steps = [], []
    for i, s in enumerate(assigns):
        if (_dtype_name(s.dtype) in INT_DTYPES) != integer:
            raise Unmatched("a cell program mixing integer and float Assigns has no kernel")
        if integer and s.op.name not in INT_OPS:
            raise OpError(f"integer elementwise op {s.op.name!r} is not supported")
        if not integer and s.op.name not in PW_OP_NAMES:
            raise OpError(f"elementwise op {s.op.name!r} is not supported")
        ops = []
        for a in s.args:
            if isinstance(a, str) and a in scalars and a not in slot_of:
                if a not in scalar_slot:
                    consts.append(("scalar", a))                    # a placeholder no literal can equal
                    scalar_slot[a] = len(consts) - 1
                    if len(consts) > PW_CONSTS:
                        raise Unmatched(f"more than {PW_CONSTS} distinct constants")
                ops.append(PW_SLOTS + scalar_slot[a])
            elif isinstance(a, str):
                if a not in slot_of:
                    raise Unmatched(f"use of undefined name {a!r}")
                ops.append(slot_of[a])
            else:
                v = float(a)
                if integer and (v != int(v) or abs(v) >= 2**24):
                    raise Unmatched(f"integer constant {a!r} does not fit the program's constant table")
                if v not in consts:
                    consts.append(v)
                if len(consts) > PW_CONSTS:
                    raise Unmatched(f"more than {PW_CONSTS} distinct constants")
                ops.append(PW_SLOTS + consts.index(v))
        for a in set(x for x in s.args if isinstance(x, str) and x in slot_of):          # operands that die here free their slots
            if last_use.get(a) == i and slot_of[a] >= len(inputs):
                free.append(slot_of[a])
        if not free:
            raise Unmatched(f"more than {PW_SLOTS} live values")
        dst = free.pop()
        slot_of[s.name] = dst
        steps.append(["copy" if s.op.name in MOVE_OPS else s.op.name, dst, *(ops + [0, 0])[:3]])
        if s.name not in last_use:                                      # never read: its slot is free again at once
            free.append(dst)
    if len(steps) > PW_STEPS:
        raise Unmatched(f"{len(steps)} steps: the general elementwise kernel takes {PW_STEPS}")
    prog = {"inputs": inputs, "in_dtypes": [tensors[b][1] for b in inputs], "out_dtype": tensors[out_name][1],
            "out_slot": slot_of[out_value_name], "consts": [0.0 if isinstance(c, tuple) else c for c in consts], "steps": steps}
    if scalar_slot:
        prog["scalar_consts"] = [[name, idx, scalars[name]] for name, idx in scalar_slot.items()]
    return prog


class Load:
    """A synthetic Load the indexed matcher puts in front of a cell program (one per source of a value)."""

    def __init__(self, name: str, source: str) -> None:
        self.names, self.input, self.index = [name], source, []


class _Body:
    def __init__(self, body: list) -> None:
        self.body = body


def _fit_affine(idx: np.ndarray, digits: list, what: str):
    """offset and one coefficient per axis such that idx = offset + sum coef * digit on every probe cell, or Unmatched.
    The probe cells contain cell 0 and, for every axis longer than 1, the cell whose only non-zero digit is a 1 there."""
    zero = np.all([d == 0 for d in digits], axis=0) if digits else np.ones(idx.shape, bool)
    off = int(idx[zero][0])
    coef = []
    for a, d in enumerate(digits):
        unit = (d == 1) & np.all([dd == 0 for b, dd in enumerate(digits) if b != a], axis=0)
        coef.append(int(idx[unit][0]) - off if unit.any() else 0)
    want = off + sum(c * d for c, d in zip(coef, digits)) if digits else np.full(idx.shape, off)
    if not np.array_equal(np.asarray(idx, np.int64), np.asarray(want, np.int64)):
        raise Unmatched(f"{what} is not an affine function of the tile's axis variables")
    return off, coef


def _fit_rotated(idx: np.ndarray, digits: list, extents: list, what: str):
    """offset, coefficients and one rotation per axis such that idx = offset + sum coef * ((digit + rot) mod extent) on every
    probe cell (torch.roll along one or more axes), or Unmatched. Needs the probe cells to hold, for every axis, all cells
    whose other digits are zero."""
    coef, rot = [], []
    for a, (d, e) in enumerate(zip(digits, extents)):
        line = np.all([dd == 0 for b, dd in enumerate(digits) if b != a], axis=0)
        order = np.argsort(d[line])
        if e == 1:
            coef.append(0), rot.append(0)
            continue
        if line.sum() != e:
            raise Unmatched(f"{what} is not an affine function of the tile's axis variables")
        values = np.asarray(idx[line][order], np.int64)
        steps = np.diff(values)
        vals, counts = np.unique(steps, return_counts=True)
        c = int(vals[np.argmax(counts)])
        wraps = np.nonzero(steps != c)[0]
        if len(wraps) == 0:
            coef.append(c), rot.append(0)
        elif len(wraps) == 1 and int(steps[wraps[0]]) == -c * (e - 1):
            coef.append(c), rot.append(e - 1 - int(wraps[0]))
        else:
            raise Unmatched(f"{what} is neither affine nor a rotation along axis {a}")
    zero = np.all([d == 0 for d in digits], axis=0)
    off = int(idx[zero][0]) - sum(c * r for c, r in zip(coef, rot))
    want = off + sum(c * ((d + r) % e) for c, r, d, e in zip(coef, rot, digits, extents))
    if not np.array_equal(np.asarray(idx, np.int64), np.asarray(want, np.int64)):
        raise Unmatched(f"{what} is neither affine nor a rotation of the tile's axis variables")
    return off, coef, rot


def _index_chain(tile, name: str):
    """`name` as (load statement, abs?, modulus): the value of an integer Load, optionally through `abs`, then reduced by a
    positive literal modulus -- the only form of a data-dependent coordinate that is bounded by construction."""
    defs = {s.name: s for s in tile.body if _kind(s) == "Assign"}
    loads = {s.names[0]: s for s in tile.body if _kind(s) == "Load"}
    st = defs.get(name)
    if st is None or st.op.name not in ("mod", "remainder") or len(st.args) != 2 or _dtype_name(st.dtype) not in INT_DTYPES:
        raise Unmatched("a coordinate taken from data must be reduced by a literal modulus")
    src, mod = st.args
    if isinstance(mod, bool) or not isinstance(mod, (int, float)) or mod != int(mod) or mod < 1 or not isinstance(src, str):
        raise Unmatched("a coordinate taken from data must be reduced by a positive literal modulus")
    use_abs = False
    if src in defs:
        if defs[src].op.name != "abs" or _dtype_name(defs[src].dtype) not in INT_DTYPES or not isinstance(defs[src].args[0], str):
            raise Unmatched("between the integer Load and the modulus only `abs` is understood")
        use_abs, src = True, defs[src].args[0]
    if src not in loads:
        raise Unmatched("a coordinate taken from data starts at a Load")
    return loads[src], use_abs, int(mod), {name, st.args[0]} if use_abs else {name}


def _reach(off: int, coef: list, extents: list):
    lo = hi = off
    for c, e in zip(coef, extents):
        lo, hi = lo + min(0, c * (e - 1)), hi + max(0, c * (e - 1))
    return lo, hi


def match_indexed(graph, kernel, launch: dict, int_div: str = "floor") -> dict:
    """A one-cell-per-element Tile whose Loads and Write address their buffers by affine functions of the axis variables,
    and whose Assigns may use the axis variables as values: the reference's data-movement cases (transpose, permute,
    slices, flip, stack, a concatenation written slice by slice: tools/torch_cases/shapes.py:6-17) and masks made from
    indices (tril, :19). Every index expression is run on probe cells, fitted, checked on all of them and checked against
    the buffers' sizes over the whole tile; the Assign chain becomes a cell program as for any elementwise kernel."""
    tensors = tensor_table(graph)
    tiles = [s for s in kernel.body if _kind(s) == "Tile"]
    if len(kernel.body) != 1 or len(tiles) != 1:
        raise Unmatched("a streaming kernel is one Tile")
    tile = tiles[0]
    if len(tile.axes) > 6:
        raise Unmatched("more than 6 tile axes")
    extents = [int(a.extent.as_static()) for a in tile.axes]
    names = [a.name for a in tile.axes]
    n = math.prod(extents)
    if n > 2**31 - 1 or n < 1:
        raise Unmatched(f"a tile of {n} cells has no indexed variant")
    if any(_kind(s) not in ("Load", "Assign", "Write") for s in tile.body):
        raise Unmatched("the indexed elementwise kernel runs Load / Assign / Write programs")
    strides = [math.prod(extents[a + 1:]) for a in range(len(extents))]
    rng = np.random.default_rng(0)
    lines = [np.arange(e) * st for st, e in zip(strides, extents) if 1 < e <= 4096]      # every cell of each axis' line through cell 0
    cells = np.unique(np.concatenate([np.arange(min(n, 64)), rng.integers(0, n, 200), [n - 1],
                                      [st for st, e in zip(strides, extents) if e > 1], *lines])).astype(np.int64)
    it = CellInterpreter(tensors, cells, INT_OPS_TRUNC if int_div == "trunc" else INT_OPS)
    digits = [(cells // st) % e for st, e in zip(strides, extents)]
    for nm, d in zip(names, digits):
        it.env[nm] = d
    it.run(tile.body)
    loads = [s for s in tile.body if _kind(s) == "Load"]
    writes = [s for s in tile.body if _kind(s) == "Write"]
    if len(writes) != 1 or len(it.writes) != 1 or len(it.writes[0][2]) != 1 or _kind(tile.body[-1]) != "Write":
        raise Unmatched("indexed kernels end in one Write of one value per cell")
    if any(cnt != 1 for _, _, cnt in it.loads) or len(it.loads) != len(loads):
        raise Unmatched("indexed kernels read one element per Load")
    out_name, out_idx, _ = it.writes[0]
    out_dtype = tensors[out_name][1]
    integer = out_dtype in ("i32", "i64", "int")
    ok_in = ("i32", "i64", "int") if integer else ("f32", "f16", "bf16", "bool", "u8")
    if not integer and out_dtype not in ("f32", "f16", "bf16"):
        raise Unmatched(f"no indexed variant writes {out_dtype}")
    # the sources of values, in program order: one per Load, one per axis variable an Assign uses as a value
    body, sources, synthetic = [], [], dict(tensors)
    # Loads whose index uses a value that is not an axis variable: a coordinate taken from data
    axis_names = set(names)
    indirect, hidden, index_loads = {}, set(), {}
    for k, s in enumerate(loads):
        free = set()
        for e in s.index:
            free |= e.free_vars() if hasattr(e, "free_vars") else set()
        extra = sorted(free - axis_names)
        if not extra:
            continue
        if len(extra) != 1:
            raise Unmatched("a Load takes at most one coordinate from data")
        src_load, use_abs, mod, chain = _index_chain(tile, extra[0])
        saved = it.env[extra[0]]
        it.env[extra[0]] = np.zeros(cells.shape, np.int64)
        base = it.flat_index(s.input, s.index)
        it.env[extra[0]] = np.ones(cells.shape, np.int64)
        mult = np.unique(it.flat_index(s.input, s.index) - base)
        it.env[extra[0]] = saved
        if len(mult) != 1 or int(mult[0]) < 0:
            raise Unmatched("the coordinate taken from data does not enter the index linearly")
        indirect[k] = (base, int(mult[0]), src_load, use_abs, mod)
        hidden |= chain
        index_loads[id(src_load)] = (use_abs, mod)
    for k, (s, (buf, idx, _)) in enumerate(zip(loads, it.loads)):
        is_source = id(s) in index_loads
        if is_source:
            if tensors[buf][1] not in ("i32", "i64", "int"):
                raise Unmatched("an index is read from an integer buffer")
        elif tensors[buf][1] not in ok_in:
            raise Unmatched(f"input {buf!r} of dtype {tensors[buf][1]} in {'an integer' if integer else 'a float'} program")
        rot = None
        fit_on = indirect[k][0] if k in indirect else idx
        try:
            off, coef = _fit_affine(fit_on, digits, f"the index of {buf!r}")
        except Unmatched:
            if k in indirect or is_source:
                raise
            off, coef, rot = _fit_rotated(fit_on, digits, extents, f"the index of {buf!r}")
        lo, hi = _reach(off, coef, extents)
        if k in indirect:
            hi += indirect[k][1] * (indirect[k][4] - 1)
        guarded = bool(getattr(s, "guarded", False))            # hoisted out of a Cond: the kernel clamps the index
        if guarded and (rot is not None or k in indirect or is_source):
            raise Unmatched("a Load inside a Cond is addressed by a plain affine index")
        if not guarded and (lo < 0 or hi >= math.prod(tensors[buf][0])):
            raise Unmatched(f"the index of {buf!r} leaves the buffer (elements {lo}..{hi} of {math.prod(tensors[buf][0])})")
        name = f"__in{k}"
        synthetic[name] = (tensors[buf][0], tensors[buf][1])
        src = {"buffer": buf, "offset": off, "coef": coef}
        if guarded and (lo < 0 or hi >= math.prod(tensors[buf][0])):
            src["clamp"] = math.prod(tensors[buf][0])
        if rot is not None and any(rot):
            src["rot"] = rot
        if is_source:
            src["index_mod"], src["index_abs"] = index_loads[id(s)][1], index_loads[id(s)][0]
        if k in indirect:
            src["index_of_load"], src["index_mult"] = indirect[k][2], indirect[k][1]
        sources.append(src)
        if not is_source:
            body.append(Load(s.names[0], name))
    if index_loads:
        used = {a for st in tile.body if _kind(st) == "Assign" and st.name not in hidden for a in st.args if isinstance(a, str)}
        used |= {v for w in tile.body if _kind(w) == "Write" for v in w.values if isinstance(v, str)}
        for s in loads:
            if id(s) in index_loads and (s.names[0] in used or hidden & used):
                raise Unmatched("a value read as an index is not also a value of the program")
    used_axes = [nm for nm in names if any(_kind(s) == "Assign" and nm in [a for a in s.args if isinstance(a, str)] for s in tile.body)]
    for nm in used_axes:
        synthetic[f"__axis_{nm}"] = ((n,), "i32" if integer else "f32")
        sources.append({"axis": names.index(nm)})
        body.append(Load(nm, f"__axis_{nm}"))
    if not sources:
        raise Unmatched("an indexed kernel reads something")
    body += [s for s in tile.body if _kind(s) != "Load" and not (_kind(s) == "Assign" and s.name in hidden)]
    off, coef = _fit_affine(out_idx, digits, "the index of the Write")
    lo, hi = _reach(off, coef, extents)
    if lo < 0 or hi >= math.prod(tensors[out_name][0]):
        raise Unmatched(f"the Write leaves its buffer (elements {lo}..{hi} of {math.prod(tensors[out_name][0])})")
    order = sorted((abs(c), e) for c, e in zip(coef, extents) if e > 1)         # no two cells may write one element
    span = 0
    for c, e in order:
        if c <= span:
            raise Unmatched("two cells write the same element")
        span += c * (e - 1)
    scalars = scalar_args(launch)
    prog = build_program(_Body(body), synthetic, out_name, writes[0].values[0], integer=integer, scalars=scalars)
    if integer:
        prog["int_div"] = int_div
    by_name = {f"__in{k}": sources[k] for k in range(len(loads))}
    by_name.update({f"__axis_{nm}": sources[len(loads) + j] for j, nm in enumerate(used_axes)})
    ordered = [by_name[nm] for nm in prog["inputs"]]
    # index sources ride along as extra inputs that no step reads
    for k, s in enumerate(loads):
        if id(s) in index_loads:
            ordered.append(sources[k])
            prog["in_dtypes"].append(tensors[s.input][1])
    if len(ordered) > PW_INPUTS:
        raise Unmatched(f"{len(ordered)} sources: the indexed elementwise kernel takes {PW_INPUTS}")
    for src in ordered:
        if "index_of_load" in src:
            target = sources[next(k for k, ld in enumerate(loads) if ld is src.pop("index_of_load"))]
            src["index_of"] = next(j for j, o in enumerate(ordered) if o is target)
    index_map = {"extents": extents, "inputs": ordered, "out": {"offset": off, "coef": coef}}
    return {"variant": "pointwise_indexed", "inputs": [src["buffer"] for src in ordered if "buffer" in src], "outputs": [out_name],
            "params": {"n": n, "program": {k: v for k, v in prog.items() if k != "inputs"}, "index_map": index_map}}


# ---- Let and Select as Assigns ---------------------------------------------------------------------------------
_EXPR_OPS = {"+": "add", "-": "subtract", "*": "multiply", "/": "divide", "<": "less", "<=": "less_equal", ">": "greater",
             ">=": "greater_equal", "==": "equal", "!=": "not_equal", "&&": "bitwise_and", "||": "bitwise_or"}


class _Op:
    def __init__(self, name: str) -> None:
        self.name, self.identity = name, None


class Assign:
    """A synthetic Assign (what the desugaring below writes in place of a Let or a Select)."""

    def __init__(self, name: str, op: str, args: list) -> None:
        self.name, self.op, self.args, self.dtype = name, _Op(op), args, None


class _Var:
    def __init__(self, name: str) -> None:
        self.name = name

    def free_vars(self) -> set:
        return {self.name}


_Var.__name__ = "Var"


def guarded_load(names: list, buffer: str, index: list):
    """A Load hoisted out of a Cond: it runs in every cell, so the kernel clamps its index into the buffer."""
    ld = object.__new__(Load)
    ld.names, ld.input, ld.index, ld.guarded = names, buffer, index, True
    return ld


class Write:
    def __init__(self, output: str, index: list, values: list) -> None:
        self.output, self.index, self.values, self.atomic = output, index, values, False


def merged_write(output: str, index: list, values: list):
    return Write(output, index, values)


def desugar_float_body(body: list) -> list:
    """The statement list with every float `Let` (name = expression) and `Select` (name = v0 when p0, ... ,
    emmyptx/kernel.py:812-822) rewritten as Assigns over the op table, so that the cell-program builders see
    Load / Assign / Write only. Expressions may use axis variables, earlier values, literals, arithmetic, comparisons,
    `&&` / `||` (masks are 1.0 / 0.0, as the reference's comparisons are: emmyptx/ops.py:116-120), the ternary and calls of
    ops by name. Integer expressions (shifts, `//`, `%`, casts to int) are not rewritten: Unmatched.
    A `Cond` on such an expression (emmyptx/kernel.py:825-840) is flattened: the Loads of both arms run in every cell as
    guarded Loads (the kernel clamps their indices into the buffers), values are renamed per arm, and what both arms
    define or write to the same element is merged with `where` on the predicate -- the two halves of a concatenation, a
    padded border. Arms that write different elements (or only one of which writes) have no kernel variant."""
    out, counter = [], [0]

    def fresh() -> str:
        counter[0] += 1
        return f"__e{counter[0]}"

    def operand(e):
        k = _kind(e)
        if isinstance(e, (int, float)) and not isinstance(e, bool):
            return float(e)
        if isinstance(e, bool):
            return 1.0 if e else 0.0
        if isinstance(e, str):
            return e
        if k == "Literal":
            return (1.0 if e.value else 0.0) if isinstance(e.value, bool) else float(e.value)
        if k == "Var":
            return e.name
        if k == "BinaryExpr":
            if e.op not in _EXPR_OPS:
                raise Unmatched(f"operator {e.op!r} in a float expression has no elementwise op")
            name = fresh()
            out.append(Assign(name, _EXPR_OPS[e.op], [operand(e.left), operand(e.right)]))
            return name
        if k == "TernaryExpr":
            name = fresh()
            out.append(Assign(name, "where", [operand(e.cond), operand(e.if_true), operand(e.if_false)]))
            return name
        if k == "CastExpr":
            if e.dtype in INT_DTYPES:
                raise Unmatched("a cast to an integer inside a float expression")
            return operand(e.expr)
        if k == "FuncCallExpr":
            name = fresh()
            out.append(Assign(name, _FUNC_ALIASES.get(e.name, e.name), [operand(a) for a in e.args]))
            return name
        raise Unmatched(f"unsupported expression {k}")

    def same_expr(a, b) -> bool:
        if _kind(a) != _kind(b):
            return False
        if not hasattr(a, "__dict__"):
            return a == b
        fields = [f for f in vars(a) if not f.startswith("_")]
        return all(same_expr(getattr(a, f), getattr(b, f, None)) if not isinstance(getattr(a, f), (list, tuple)) else
                   (isinstance(getattr(b, f, None), (list, tuple)) and len(getattr(a, f)) == len(getattr(b, f)) and
                    all(same_expr(x, y) for x, y in zip(getattr(a, f), getattr(b, f)))) for f in fields)

    def rename_expr(e, names: dict):
        """The expression with value names replaced (axis variables and untouched names stay)."""
        k = _kind(e)
        if isinstance(e, str):
            return names.get(e, e)
        if k == "Var":
            return _Var(names.get(e.name, e.name))
        if k in ("BinaryExpr", "TernaryExpr", "CastExpr", "FuncCallExpr"):
            copy = object.__new__(type(e))
            for f, v in vars(e).items():
                setattr(copy, f, [rename_expr(x, names) for x in v] if isinstance(v, (list, tuple)) else
                        (rename_expr(v, names) if hasattr(v, "__dict__") else v))
            return copy
        return e

    def branch(stmts, tag: str):
        """One arm of a Cond, flattened: Loads become guarded Loads of renamed values, Assigns / Lets / Selects are renamed,
        Writes are collected. Returns (statements, {original name: renamed}, writes)."""
        names, flat, writes = {}, [], []
        for t in stmts:
            k = _kind(t)
            if k == "Load":
                for nm in t.names:
                    names[nm] = f"{nm}__{tag}"
                flat.append(guarded_load([names[nm] for nm in t.names], t.input, [rename_expr(e, names) for e in t.index]))
            elif k == "Assign":
                args = [names.get(a, a) if isinstance(a, str) else a for a in t.args]
                names[t.name] = f"{t.name}__{tag}"
                a2 = Assign(names[t.name], t.op.name, args)
                a2.dtype = t.dtype
                flat.append(a2)
            elif k == "Write":
                writes.append((t.output, list(t.index), [names.get(v, v) if isinstance(v, str) else v for v in t.values], bool(getattr(t, "atomic", False))))
            else:
                raise Unmatched(f"statement {k} inside a Cond has no kernel variant")
        return flat, names, writes

    for s in body:
        k = _kind(s)
        if k == "Cond":
            counter[0] += 1
            pred = operand(s.cond)
            then_flat, then_names, then_writes = branch(list(s.body), f"t{counter[0]}")
            else_flat, else_names, else_writes = branch(list(getattr(s, "else_body", None) or []), f"e{counter[0]}")
            out.extend(then_flat)
            out.extend(else_flat)
            for nm in then_names:                                       # a value both arms define lives on after the Cond
                if nm in else_names:
                    out.append(Assign(nm, "where", [pred, then_names[nm], else_names[nm]]))
            if len(then_writes) != len(else_writes):
                raise Unmatched("the two arms of a Cond must write the same elements (a cell that writes nothing has no kernel variant)")
            for (o1, i1, v1, at1), (o2, i2, v2, at2) in zip(then_writes, else_writes):
                if o1 != o2 or at1 or at2 or len(v1) != 1 or len(v2) != 1 or len(i1) != len(i2) or not all(same_expr(x, y) for x, y in zip(i1, i2)):
                    raise Unmatched("the two arms of a Cond must write the same elements")
                name = fresh()
                out.append(Assign(name, "where", [pred, v1[0], v2[0]]))
                out.append(merged_write(o1, i1, [name]))
        elif k == "Let":
            if _dtype_name(getattr(s, "dtype", None)) in INT_DTYPES:
                raise Unmatched("an integer Let in a float cell program")
            out.append(Assign(s.name, "copy", [operand(s.value)]))
        elif k == "Select":
            branches = list(s.branches)
            if not branches:
                raise Unmatched("a Select without branches")
            result = operand(branches[-1].value)
            for b in reversed(branches[:-1]):
                pred = operand(b.select)
                name = fresh()
                out.append(Assign(name, "where", [pred, operand(b.value), result]))
                result = name
            out.append(Assign(s.name, "copy", [result]))
        else:
            out.append(s)
    return out


class Tile:
    """A Tile with another body (the matchers tell statements by class name, hence the name)."""

    def __init__(self, tile, body: list) -> None:
        self.axes, self.body = tile.axes, body


class KernelOp:
    def __init__(self, kernel, body: list) -> None:
        self.name, self.body = kernel.name, body


def match_streaming(graph, kernel, launch: dict, int_div: str = "floor") -> dict:
    try:
        return _match_streaming(graph, kernel, launch, int_div)
    except Unmatched as first:
        # not element i of every buffer (or a broadcast of it): Loads and the Write may still be affine in the axis variables
        try:
            return match_indexed(graph, kernel, launch, int_div)
        except (Unmatched, OpError):
            pass
        # float Lets and Selects spelled out as Assigns, then the same two matchers
        tiles = [s for s in kernel.body if _kind(s) == "Tile"]
        if len(kernel.body) == 1 and len(tiles) == 1 and any(_kind(s) in ("Let", "Select", "Cond") for s in tiles[0].body):
            try:
                plain = KernelOp(kernel, [Tile(tiles[0], desugar_float_body(tiles[0].body))])
                try:
                    return _match_streaming(graph, plain, launch, int_div)
                except Unmatched:
                    return match_indexed(graph, plain, launch, int_div)
            except (Unmatched, OpError):
                pass
        raise first from None


def _match_streaming(graph, kernel, launch: dict, int_div: str = "floor") -> dict:
    tensors = tensor_table(graph)
    tiles = [s for s in kernel.body if _kind(s) == "Tile"]
    if len(kernel.body) != 1 or len(tiles) != 1:
        raise Unmatched("a streaming kernel is one Tile")
    tile = tiles[0]
    n = math.prod(int(a.extent.as_static()) for a in tile.axes)
    if n > 2**31 - 1:
        raise Unmatched(f"a tile of {n} cells needs 64-bit indexing")           # emmyptx/kernel.py:556-557
    rng = np.random.default_rng(0)
    cells = np.unique(np.concatenate([np.arange(min(n, 96)), rng.integers(0, n, 160), [n - 1]])).astype(np.int64)
    it = CellInterpreter(tensors, cells, INT_OPS_TRUNC if int_div == "trunc" else INT_OPS)
    scalars = scalar_args(launch)
    for k, (name, ty) in enumerate(scalars.items()):        # a value no fixed-function variant's expression contains
        it.env[name] = np.full(cells.shape, 1.3719 + 0.2113 * k) if ty == "f32" else np.full(cells.shape, 5 + 3 * k, dtype=np.int64)
    used_scalars = {a for st in tile.body if _kind(st) == "Assign" for a in st.args if isinstance(a, str) and a in scalars}
    # axis variables: last axis fastest (emmyptx/kernel.py:587-626, without rasterisation)
    rem = cells.copy()
    for a in reversed(tile.axes):
        e = int(a.extent.as_static())
        it.env[a.name] = rem % e
        rem = rem // e
    it.run(tile.body)
    if len(it.writes) != 1 or len(it.writes[0][2]) != 1:
        raise Unmatched("streaming variants write one value per cell to one buffer")
    out_name, out_idx, (value,) = it.writes[0]
    if not np.array_equal(out_idx, cells) or math.prod(tensors[out_name][0]) != n:
        raise Unmatched("streaming variants write cell i to element i")
    buffers = {b for b, _, _ in it.loads}
    if any(cnt != 1 for _, _, cnt in it.loads):
        raise Unmatched("streaming variants read one element per load")
    float_types = ("f32", "f16", "bf16")
    int_types = ("i32", "i64", "int")
    identity = all(np.array_equal(i, cells) for _, i, _ in it.loads) and all(math.prod(tensors[b][0]) == n for b in buffers)
    # Broadcast reads: element (i // div) % mod of a smaller buffer (a row vector over a matrix, a column vector, ...).
    # The divisors tried are the products of the output's trailing extents.
    out_shape = tensors[out_name][0]
    divisors = sorted({math.prod(out_shape[j:]) for j in range(len(out_shape) + 1)})
    pattern = {}
    for b, i, _ in it.loads:
        size = math.prod(tensors[b][0])
        found = next(((d if d > 1 else 0, 0 if (d == 1 and size == n) else size) for d in divisors
                      if np.array_equal(i, (cells // d) % size)), None)
        if found is None or pattern.setdefault(b, found) != found:
            pattern = None
            break
    broadcast = pattern is not None and not identity
    if (identity or broadcast) and tensors[out_name][1] in int_types and all(tensors[b][1] in int_types for b in buffers) and buffers:
        # an integer expression of element i of every buffer: the s32 program kernel (the gather is the other integer kernel)
        prog = build_program(tile, tensors, out_name, tile.body[-1].values[0] if _kind(tile.body[-1]) == "Write" else None, integer=True, scalars=scalars)
        prog["int_div"] = int_div
        if broadcast:
            prog["in_div"], prog["in_mod"] = [pattern[b][0] for b in prog["inputs"]], [pattern[b][1] for b in prog["inputs"]]
        return {"variant": "pointwise_program", "params": {"n": n, "program": {k: v for k, v in prog.items() if k != "inputs"}},
                "inputs": prog["inputs"], "outputs": [out_name]}
    # a bool / byte output holds 1 where the program's value is non-zero (a comparison stored as it is: `x > y`)
    general = (tensors[out_name][1] in float_types + ("bool", "u8") and all(tensors[b][1] in float_types + ("bool", "u8") for b in buffers)
               and (identity or broadcast) and bool(buffers))
    if general and (used_scalars or broadcast or not (len(buffers) == 1 and tensors[next(iter(buffers))][1] == "f32" and tensors[out_name][1] == "f32")):
        prog = build_program(tile, tensors, out_name, tile.body[-1].values[0] if _kind(tile.body[-1]) == "Write" else None, scalars=scalars)
        if broadcast:
            prog["in_div"], prog["in_mod"] = [pattern[b][0] for b in prog["inputs"]], [pattern[b][1] for b in prog["inputs"]]
        return {"variant": "pointwise_program", "params": {"n": n, "program": {k: v for k, v in prog.items() if k != "inputs"}},
                "inputs": prog["inputs"], "outputs": [out_name]}
    if used_scalars:
        raise Unmatched("scalar parameters are taken by elementwise programs over float or integer buffers only")
    if len(buffers) != 1:
        raise Unmatched("streaming variants read one input buffer")
    (src,) = buffers
    src_shape, src_dtype = tensors[src]
    out_dtype = tensors[out_name][1]
    idx = it.loads[0][1]
    if any(not np.array_equal(i, idx) for _, i, _ in it.loads):
        raise Unmatched("streaming variants read one element per cell")
    if src_dtype == "f32" and out_dtype == "f32":
        if not np.array_equal(idx, cells) or math.prod(src_shape) != n:
            raise Unmatched("float streaming variants read element i for cell i")
        x = probe_values(src, "f32", cells)
        got = np.asarray(value, dtype=np.float64)
        for op, f in POINTWISE_F64.items():
            if np.allclose(got, f(x), rtol=1e-9, atol=1e-12):
                return {"variant": "pointwise_f32", "params": {"op": op, "n": n}, "inputs": [src], "outputs": [out_name]}
        # not one of the specialised expressions: the general elementwise kernel runs the program as data
        prog = build_program(tile, tensors, out_name, tile.body[-1].values[0])
        return {"variant": "pointwise_program", "params": {"n": n, "program": {k: v for k, v in prog.items() if k != "inputs"}},
                "inputs": prog["inputs"], "outputs": [out_name]}
    if src_dtype == "i32" and out_dtype == "i32":
        size = math.prod(src_shape)
        if size != n:
            raise Unmatched("the index gather reads a buffer as large as the tile")
        add = int(idx[cells == 0][0]) % size if 0 in cells else None
        mul = (int(idx[cells == 1][0]) - add) % size if n > 1 else 0
        if add is None or not np.array_equal(idx, (cells * mul + add) % size):
            raise Unmatched("the gather index is not (i * mul + add) mod n")
        g = probe_values(src, "i32", idx)
        lits = sorted(_int_literals(kernel))
        divs = [d for d in lits if d >= 1] or [1]
        shifts = [s for s in lits if 0 <= s <= 31] + [0]
        got = np.asarray(value, dtype=np.int64)
        div = INT_OPS_TRUNC["floor_divide"][1] if int_div == "trunc" else INT_OPS["floor_divide"][1]
        for d in divs:
            for sh in dict.fromkeys(shifts):
                if np.array_equal(got, np.bitwise_xor(div(g, np.int64(d)), cells >> sh)):
                    return {"variant": "index_gather_i32", "inputs": [src], "outputs": [out_name],
                            "params": {"n": n, "mul": mul, "add": add, "div": d, "shift": sh, "trunc": int_div == "trunc"}}
        raise Unmatched("the integer expression is not (x[idx] div d) xor (i >> s)")
    raise Unmatched(f"no streaming variant for {src_dtype} -> {out_dtype}")


def _epilogue_name(ep):
    if ep is None:
        return None
    name = getattr(ep, "name", ep)
    name = str(name).lower()
    if name in ("none", ""):
        return None
    if name in ("gelu_tanh", "gelu"):
        return "gelu_tanh"
    if name == "relu":
        return "relu"
    raise Unmatched(f"store epilogue {name!r} has no fused variant (have: gelu_tanh, relu)")


def _attention_scale(stmts, mmas, d: int) -> float:
    """The factor on the scores: the literal of the one `multiply` whose other operand is the accumulator fragment of
    the first MMA group (S = Q K^T); 1 when nothing scales the scores. Two candidates (a separately folded log2(e),
    say) are ambiguous, and a scale that is not a literal cannot be passed to the kernel: both match nothing."""
    s_frag = mmas[0].c_frag
    cands = []
    for st in stmts:
        if _kind(st) == "Assign" and st.op.name == "multiply" and s_frag in [a for a in st.args if isinstance(a, str)]:
            lits = [float(a) for a in st.args if isinstance(a, (int, float)) and not isinstance(a, bool)]
            cands += lits
    if len(cands) > 1:
        raise Unmatched(f"more than one constant multiplies the scores ({cands}): which is the softmax scale is ambiguous")
    if cands:
        return cands[0]
    if any(_kind(st) == "Assign" and st.op.name in ("multiply", "divide") and s_frag in [a for a in st.args if isinstance(a, str)]
           for st in stmts):
        raise Unmatched("the scores are scaled by something other than a literal")
    return 1.0


def _attention_mask(kernel, stmts, seq_q: int, seq_k: int) -> bool:
    """False for an unmasked softmax, True for the lower-triangular (causal) mask, `Unmatched` for any other mask.
    A mask is a `where` that fills -inf (tools/torch_cases/fused.py:31-36; models.py:17-19). Its condition is run on
    probe (query, key) index pairs -- the tile's last axis must count queries and the loop's axis keys, one each --
    and only `key <= query` kept / `key > query` filled is the causal variant; a padding, banded or upper-triangular
    mask is some other function of the pair and is refused."""
    neg_inf = lambda a: isinstance(a, float) and a == float("-inf")
    fills = [st for st in stmts if _kind(st) == "Assign" and st.op.name == "where" and any(neg_inf(a) for a in st.args)]
    if not fills:
        return False
    if len(fills) > 1:
        raise Unmatched("more than one masking `where`")
    tiles = [st for st in kernel.body if _kind(st) == "Tile"]
    loops = [st for st in stmts if _kind(st) in ("Loop", "StridedLoop") and fills[0] in list(walk(st.body))]
    if len(tiles) != 1 or not loops:
        raise Unmatched("a masked softmax is one Tile with the mask inside the key loop")
    q_axis, k_axis = tiles[0].axes[-1], loops[-1].axis
    if int(q_axis.extent.as_static()) != seq_q or int(k_axis.extent.as_static()) != seq_k:
        raise Unmatched("the mask's indices do not count single queries and keys: it cannot be checked")
    qs = np.unique(np.clip([0, 1, 2, 7, 8, 15, 16, 17, seq_q // 2, seq_q - 2, seq_q - 1], 0, seq_q - 1))
    ks = np.unique(np.clip([0, 1, 2, 7, 8, 15, 16, 17, seq_k // 2, seq_k - 2, seq_k - 1], 0, seq_k - 1))
    qq, kk = (g.reshape(-1).astype(np.int64) for g in np.meshgrid(qs, ks, indexing="ij"))
    it = CellInterpreter({}, qq, INT_OPS)
    it.env[q_axis.name], it.env[k_axis.name] = qq, kk

    def value(a):
        return it.expr(a) if hasattr(a, "free_vars") or _kind(a) in ("Var", "Literal", "BinaryExpr") else it.lookup(a)

    for st in walk(loops[-1].body):
        if st is fills[0]:
            break
        if _kind(st) == "Let":
            try:
                it.env[st.name] = it.expr(st.value)
            except Unmatched:
                pass
        elif _kind(st) == "Assign" and st.op.name in FLOAT_OPS:
            try:
                it.env[st.name] = FLOAT_OPS[st.op.name][1](*[np.asarray(value(a), np.float64) for a in st.args])
            except Unmatched:                      # depends on data, not on the indices alone
                pass
    cond, if_true, if_false = fills[0].args
    try:
        c = np.asarray(value(cond), np.float64) != 0
    except Unmatched:
        raise Unmatched("the mask's condition is not a function of the query and key indices alone") from None
    keep = c if neg_inf(if_false) else ~c
    if np.array_equal(keep, kk <= qq):
        return True
    raise Unmatched("a masked softmax other than the lower-triangular one (key <= query) has no variant")


def _k_covered_once(kernel, a_load, k: int) -> None:
    """The K offsets at which the kernel's cells read A -- the last index of the `a` fragment load over every value of
    the tile and loop variables it depends on -- are 0, 16, 32, ... up to K, each exactly once. That holds for one loop
    over K and for a split-K schedule (a tile axis times a shorter loop); a kernel that skips or repeats part of K is
    some other computation."""
    expr = a_load.src_index[-1]
    extents = {}
    for s in walk(kernel.body):
        kind = _kind(s)
        if kind == "Tile":
            extents.update({a.name: int(a.extent.as_static()) for a in s.axes})
        elif kind in ("Loop", "StridedLoop"):
            extents[s.axis.name] = int(s.axis.extent.as_static())
    names = sorted(expr.free_vars()) if hasattr(expr, "free_vars") else []
    if any(nm not in extents for nm in names):
        raise Unmatched("the K index of the A fragment depends on something other than tile and loop variables")
    total = math.prod(extents[nm] for nm in names) if names else 1
    if total > 1 << 20:
        raise Unmatched("the K index of the A fragment ranges over too many cells to check")
    grids = np.meshgrid(*[np.arange(extents[nm], dtype=np.int64) for nm in names], indexing="ij") if names else []
    it = CellInterpreter({}, np.zeros(total, dtype=np.int64), INT_OPS)
    for nm, g in zip(names, grids):
        it.env[nm] = g.reshape(-1)
    offs = np.sort(np.asarray(it.expr(expr), dtype=np.int64).reshape(-1))
    want = np.arange(0, -(-k // 16) * 16, 16, dtype=np.int64)
    if offs.shape != want.shape or not np.array_equal(offs, want):
        raise Unmatched("the cells' K offsets do not cover K exactly once")


def match_contraction(graph, kernel, launch: dict) -> dict:
    tensors = tensor_table(graph)
    stmts = list(walk(kernel.body))
    loads = [s for s in stmts if _kind(s) == "LdmatrixLoad"]
    mmas = [s for s in stmts if _kind(s) == "MmaSyncPtx"]
    stores = [s for s in stmts if _kind(s) == "RegStore"]
    for m in mmas:
        if tuple(m.shape) != (16, 8, 16) or m.c_dtype != "f32" or m.ab_dtype not in ("f16", "bf16") or m.sfa_frag is not None:
            raise Unmatched("only f16 / bf16 operands with f32 accumulators are supported")      # emmyptx/mma.py:185-187
    if len(stores) != 1:
        raise Unmatched("a contraction kernel stores one output")
    srcs = list(dict.fromkeys(s.src_buffer for s in loads))
    out = stores[0].dst_buffer
    for b in (*srcs, out):
        if b not in tensors:
            raise Unmatched(f"unknown buffer {b!r}")
    dtype = mmas[0].ab_dtype
    out_f32 = tensors[out][1] == "f32"
    if any(tensors[b][1] != dtype for b in srcs) or (tensors[out][1] != dtype and not out_f32):
        raise Unmatched("operands have the MMA's 16-bit dtype, the output that dtype or f32")
    if stores[0].atomic and not out_f32:
        raise Unmatched("an atomic (split-K) store adds into an f32 buffer")          # emmyptx/mma.py:205-207
    has_softmax = any(_kind(s) == "Assign" and s.op.name in ("exp", "exp_fast") for s in stmts)
    if len(srcs) == 3 and has_softmax:
        q, k, v = (tensors[b][0] for b in srcs)
        o = tensors[out][0]
        if not (len(q) >= 2 and q[:-2] == k[:-2] == v[:-2] == o[:-2] and k == v and q == o and q[-1] == k[-1]):
            raise Unmatched(f"attention shapes do not agree: {q}, {k}, {v} -> {o}")
        if out_f32 or stores[0].atomic:
            raise Unmatched("tensor-core attention stores the operands' 16-bit dtype")
        d = q[-1]
        if d % 32 or not 32 <= d <= 128:
            raise Unmatched(f"attention head dim {d} has no variant (multiples of 32 up to 128)")
        scale, causal = _attention_scale(stmts, mmas, d), _attention_mask(kernel, stmts, q[-2], k[-2])
        return {"variant": "attention_fwd", "inputs": srcs, "outputs": [out],
                "params": {"dtype": dtype, "units": math.prod(q[:-2]), "seq_q": q[-2], "seq_k": k[-2], "d": d, "scale": scale,
                           "causal": causal}}
    if len(srcs) != 2:
        raise Unmatched("a GEMM reads two operand buffers")
    a_loads = [s for s in loads if s.role == "a"]
    b_loads = [s for s in loads if s.role == "b"]
    if not a_loads or not b_loads:
        raise Unmatched("a GEMM loads an `a` and a `b` fragment")
    a_name, b_name = a_loads[0].src_buffer, b_loads[0].src_buffer
    b_trans = bool(b_loads[0].b_trans)
    (a_shape, _), (b_shape, _), (c_shape, _) = tensors[a_name], tensors[b_name], tensors[out]
    # leading axes of A are independent products (bmm); B carries the same leading axes or none (broadcast)
    if len(a_shape) < 2 or len(b_shape) < 2 or len(c_shape) != len(a_shape):
        raise Unmatched(f"GEMM shapes do not agree: {a_shape} x {b_shape} -> {c_shape}")
    lead = a_shape[:-2]
    if b_shape[:-2] not in ((), lead) or c_shape[:-2] != lead:
        raise Unmatched(f"batched GEMM: leading axes {lead} / {b_shape[:-2]} / {c_shape[:-2]} do not line up")
    m, k = a_shape[-2:]
    n = b_shape[-2] if b_trans else b_shape[-1]
    if (b_shape[-1] if b_trans else b_shape[-2]) != k or c_shape[-2:] != (m, n):
        raise Unmatched(f"GEMM shapes do not agree: {a_shape} x {b_shape} -> {c_shape}")
    if k % 8 or n % 8:
        raise Unmatched("row pitches must be multiples of 8 elements (16-byte TMA strides)")
    _k_covered_once(kernel, a_loads[0], k)
    bias = getattr(stores[0], "bias", None)
    inputs = [a_name, b_name]
    if bias is not None:
        if bias not in tensors or math.prod(tensors[bias][0]) != n or tensors[bias][1] != tensors[out][1]:
            raise Unmatched(f"bias {bias!r} must hold N = {n} values of the output's dtype {tensors[out][1]}")
        inputs.append(bias)
    params = {"dtype": dtype, "m": m, "n": n, "k": k, "b_trans": b_trans, "epilogue": _epilogue_name(stores[0].epilogue)}
    if out_f32:
        # The accumulator stored as it is. A split-K schedule (several cells adding partial sums into a zeroed C with
        # red.add.f32) computes the same C; here one kernel covers K and overwrites C.
        params["out_f32"] = True
        if stores[0].atomic and stores[0].epilogue is not None:
            raise Unmatched("an epilogue cannot be applied to partial sums")
    if lead or bias is not None:
        params.update(batch=math.prod(lead), b_shared=len(b_shape) == 2, bias=bias is not None)
        return {"variant": "gemm_batched", "inputs": inputs, "outputs": [out], "params": params}
    return {"variant": "gemm", "inputs": inputs, "outputs": [out], "params": params}


# ---- row reductions and normalisations --------------------------------------------------------------------------
_ACCUM = {"add": np.sum, "maximum": np.max, "minimum": np.min, "multiply": np.prod}


def _softmax64(x):
    e = np.exp(x - x.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def _moments(x):
    m = x.mean(-1, keepdims=True)
    return m, ((x - m) ** 2).sum(-1, keepdims=True)


# op -> f(x, w, b, eps) in float64; reducing ops return [rows, 1]
ROWWISE_F64 = {
    "sum": lambda x, w, b, e: x.sum(-1, keepdims=True),
    "mean": lambda x, w, b, e: x.mean(-1, keepdims=True),
    "amax": lambda x, w, b, e: x.max(-1, keepdims=True),
    "amin": lambda x, w, b, e: x.min(-1, keepdims=True),
    "prod": lambda x, w, b, e: x.prod(-1, keepdims=True),
    "var": lambda x, w, b, e: _moments(x)[1] / (x.shape[-1] - 1),
    "std": lambda x, w, b, e: np.sqrt(_moments(x)[1] / (x.shape[-1] - 1)),
    "norm2": lambda x, w, b, e: np.sqrt((x * x).sum(-1, keepdims=True)),
    "dot": lambda x, w, b, e: (x * w).sum(-1, keepdims=True),
    "logsumexp": lambda x, w, b, e: np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1, keepdims=True)) + x.max(-1, keepdims=True),
    "softmax": lambda x, w, b, e: _softmax64(x),
    "log_softmax": lambda x, w, b, e: np.log(_softmax64(x)),
    "layer_norm": lambda x, w, b, e: (x - _moments(x)[0]) / np.sqrt(_moments(x)[1] / x.shape[-1] + e) * w + b,
    "rms_norm": lambda x, w, b, e: x / np.sqrt((x * x).mean(-1, keepdims=True) + e) * w,
    "normalize": lambda x, w, b, e: x / np.maximum(np.sqrt((x * x).sum(-1, keepdims=True)), e),
}
ROWWISE_MAPS = ("softmax", "log_softmax", "layer_norm", "rms_norm", "normalize")


class RowInterpreter(CellInterpreter):
    """Runs a row-reduction kernel on a few probe rows, every value a [rows, cols] float64 array (row-level
    values are constant along a row). A `Loop` over the row's columns runs its body once on whole rows; an `Accum`
    (emmyptx/kernel.py:786-797) reduces along the row; the `WarpShuffle` / `TreeHalve` that merge the lanes' partial
    states (:856-900) change nothing once a row is reduced whole, and are skipped."""

    def __init__(self, tensors: dict, rows: np.ndarray, cols: int) -> None:
        super().__init__(tensors, np.zeros((len(rows), cols), dtype=np.int64), INT_OPS)
        self.cols = cols

    def run(self, stmts) -> None:
        for s in stmts:
            k = _kind(s)
            if k in ("Loop", "StridedLoop"):
                if int(s.axis.extent.as_static()) != self.cols:
                    raise Unmatched("a row kernel loops over the whole row")
                self.env[s.axis.name] = np.broadcast_to(np.arange(self.cols, dtype=np.int64), self.cells.shape)
                self.run(s.body)
            elif k == "Accum":
                if s.op.name not in _ACCUM:
                    raise Unmatched(f"no row reduction folds with {s.op.name!r}")
                red = _ACCUM[s.op.name](np.asarray(self.lookup(s.value), np.float64), axis=1, keepdims=True)
                base = s.base if s.base is not None else (s.name if s.name in self.env else None)
                if base is not None:
                    red = FLOAT_OPS[s.op.name][1](np.asarray(self.lookup(base), np.float64)[:, :1], red)
                self.env[s.name] = np.broadcast_to(red, self.cells.shape)
            elif k in ("WarpShuffle", "TreeHalve", "Sync", "Smem", "Init"):
                continue
            elif k == "Assign":
                args = [np.asarray(self.lookup(a), np.float64) for a in s.args]
                if s.op.name not in FLOAT_OPS:
                    raise OpError(f"elementwise op {s.op.name!r} is not supported")
                self.env[s.name] = np.broadcast_to(FLOAT_OPS[s.op.name][1](*args), self.cells.shape)
            else:
                super().run([s])


def match_rowwise(graph, kernel, launch: dict) -> dict:
    tensors = tensor_table(graph)
    tiles = [s for s in kernel.body if _kind(s) == "Tile"]
    if len(kernel.body) != 1 or len(tiles) != 1:
        raise Unmatched("a row kernel is one Tile")
    tile = tiles[0]
    loops = [s for s in walk(tile.body) if _kind(s) in ("Loop", "StridedLoop")]
    cols = int(loops[0].axis.extent.as_static())
    rows = math.prod(int(a.extent.as_static()) for a in tile.axes)
    probe = np.unique([0, rows // 2, rows - 1]).astype(np.int64)
    it = RowInterpreter(tensors, probe, cols)
    rem = np.broadcast_to(probe[:, None], it.cells.shape).copy()
    for a in reversed(tile.axes):
        e = int(a.extent.as_static())
        it.env[a.name] = rem % e
        rem = rem // e
    it.run(tile.body)
    if len(it.writes) != 1 or len(it.writes[0][2]) != 1:
        raise Unmatched("row kernels write one value to one buffer")
    out_name, out_idx, (value,) = it.writes[0]
    # The input is read either as X[cell, k] (a reduction over the last axis) or as X[k, cell] (over dim 0), k being the
    # loop variable; vectors read as V[k] are weight and bias, in load order (last-axis form only).
    along_last = probe[:, None] * cols + np.arange(cols)[None, :]
    along_first = np.arange(cols)[None, :] * rows + probe[:, None]
    big = [(b, i) for b, i, _ in it.loads if math.prod(tensors[b][0]) == rows * cols]
    if not big:
        raise Unmatched("a reduction kernel reads one buffer of cells x loop-length elements")
    over_dim0 = rows > 1 and all(np.array_equal(i, along_first) for _, i in big)
    element = along_first if over_dim0 else along_last
    src = [b for b, i in big if np.array_equal(i, element)]
    vecs = list(dict.fromkeys(b for b, i, _ in it.loads if math.prod(tensors[b][0]) == cols and b not in src
                              and np.array_equal(i, np.broadcast_to(np.arange(cols), i.shape))))
    if len(set(src)) != 1 or len(set(b for b, _, _ in it.loads)) != 1 + len(vecs) or len(vecs) > 2 or (vecs and over_dim0):
        raise Unmatched("a reduction kernel reads one buffer and, over the last axis, at most a weight and a bias vector")
    if any(tensors[b][1] != "f32" for b in (src[0], out_name, *vecs)):
        raise Unmatched("reduction kernels are float32")
    x = probe_values(src[0], "f32", element)
    w = probe_values(vecs[0], "f32", np.arange(cols))[None, :] if vecs else np.ones((1, cols))
    b = probe_values(vecs[1], "f32", np.arange(cols))[None, :] if len(vecs) > 1 else np.zeros((1, cols))
    is_map = math.prod(tensors[out_name][0]) == rows * cols and cols > 1
    want_idx = element if is_map else np.broadcast_to(probe[:, None], element.shape)
    if not np.array_equal(out_idx, want_idx):
        raise Unmatched("a reduction kernel writes one value per cell, or one per element in the input's layout")
    got = np.asarray(value, np.float64)
    literals = sorted({float(a) for s in walk(tile.body) if _kind(s) == "Assign" for a in s.args
                       if isinstance(a, float) and 0.0 < a < 1e-2}, reverse=True)
    for op, f in ROWWISE_F64.items():
        if (op in ROWWISE_MAPS) != is_map or (vecs and op not in ("layer_norm", "rms_norm", "dot")) or (len(vecs) > 1 and op != "layer_norm"):
            continue
        if (op == "dot") != (len(vecs) == 1 and not is_map):
            continue
        if over_dim0 and op in ("layer_norm", "rms_norm", "dot"):
            continue
        for eps in (literals + [0.0] if op in ("layer_norm", "rms_norm", "normalize") else [0.0]):
            with np.errstate(all="ignore"):
                ref = np.broadcast_to(f(x, w, b, eps), got.shape)
            if np.allclose(got, ref, rtol=1e-9, atol=1e-12):
                if over_dim0:
                    return {"variant": "colwise_f32", "inputs": [src[0]], "outputs": [out_name],
                            "params": {"op": op, "outer": 1, "rows": cols, "cols": rows, "eps": eps}}
                return {"variant": "rowwise_f32", "inputs": [src[0], *vecs], "outputs": [out_name],
                        "params": {"op": op, "rows": rows, "cols": cols, "eps": eps, "weight": len(vecs) > 0, "bias": len(vecs) > 1}}
    raise Unmatched("the row program is none of the reductions or normalisations the library has")


def match_dot(graph, kernel, launch: dict) -> dict:
    """A float32 matrix product written as scalar loops (one tile cell per output element, a `Loop` over K folding
    a[m, k] * b[k, n] with an `Accum`; tools/torch_cases/matmul.py:10-14): recognised by running a few output cells
    and comparing with the product of the probe buffers. Batched A, a B shared by the batch or one per product, B as
    K x N or N x K, an optional bias vector and ReLU are told apart by the buffers' index patterns and the values."""
    tensors = tensor_table(graph)
    tiles = [s for s in kernel.body if _kind(s) == "Tile"]
    if len(kernel.body) != 1 or len(tiles) != 1:
        raise Unmatched("a product kernel is one Tile")
    tile = tiles[0]
    loops = [s for s in walk(tile.body) if _kind(s) in ("Loop", "StridedLoop")]
    if len(loops) != 1:
        raise Unmatched("a product kernel has one loop over K")
    k = int(loops[0].axis.extent.as_static())
    cells = math.prod(int(a.extent.as_static()) for a in tile.axes)
    # every cell of a small output, else the corners and 62 random cells: enough of them that some pre-activation is
    # negative, which is what tells a ReLU store from a plain one by value
    probe = (np.arange(cells) if cells <= 64 else
             np.unique(np.concatenate([[0, cells - 1], np.random.default_rng(0).integers(0, cells, 62)]))).astype(np.int64)
    it = RowInterpreter(tensors, probe, k)
    rem = np.broadcast_to(probe[:, None], it.cells.shape).copy()
    for a in reversed(tile.axes):
        e = int(a.extent.as_static())
        it.env[a.name] = rem % e
        rem = rem // e
    it.run(tile.body)
    if len(it.writes) != 1 or len(it.writes[0][2]) != 1:
        raise Unmatched("product kernels write one value to one buffer")
    out_name, out_idx, (value,) = it.writes[0]
    shape = tensors[out_name][0]
    if len(shape) < 2 or math.prod(shape) != cells or not np.array_equal(out_idx[:, 0], probe):
        raise Unmatched("a product kernel writes C[..., m, n], one cell each")
    m, n = shape[-2], shape[-1]
    batch = cells // (m * n)
    bt, mi, ni = probe // (m * n), (probe // n) % m, probe % n
    kk = np.arange(k)[None, :]
    a_idx = (bt[:, None] * m + mi[:, None]) * k + kk
    b_forms = {("kn", False): (bt[:, None] * k + kk) * n + ni[:, None], ("kn", True): kk * n + ni[:, None] + 0 * bt[:, None],
               ("nk", False): (bt[:, None] * n + ni[:, None]) * k + kk, ("nk", True): ni[:, None] * k + kk + 0 * bt[:, None]}
    names = list(dict.fromkeys(b for b, _, _ in it.loads))
    a_name = next((b for b, i, _ in it.loads if math.prod(tensors[b][0]) == batch * m * k and np.array_equal(i, a_idx)), None)
    b_name = layout = shared = b_idx = None
    for bname, i, _ in it.loads:
        if bname == a_name:
            continue
        for (lay, sh), idx in b_forms.items():
            if math.prod(tensors[bname][0]) == (1 if sh else batch) * k * n and np.array_equal(i, idx):
                b_name, layout, shared, b_idx = bname, lay, sh or batch == 1, idx
                break
        if b_name:
            break
    if a_name is None or b_name is None:
        raise Unmatched("the loop does not read a[m, k] and b[k, n] (or b[n, k])")
    bias = [bn for bn in names if bn not in (a_name, b_name)]
    if len(bias) > 1 or (bias and math.prod(tensors[bias[0]][0]) != n):
        raise Unmatched("besides the two operands a product kernel reads at most a bias vector of N elements")
    if any(tensors[t][1] != "f32" for t in (a_name, b_name, out_name, *bias)):
        raise Unmatched("scalar-loop products are float32 (16-bit ones use the tensor-core statements)")
    av, bv = probe_values(a_name, "f32", a_idx), probe_values(b_name, "f32", b_idx)
    ref = (av * bv).sum(-1)
    if bias:
        ref = ref + probe_values(bias[0], "f32", ni)
    got = np.asarray(value, np.float64)[:, 0]
    # The epilogue is read off the IR -- a `relu`, or a `maximum` against a literal 0, between the fold and the store --
    # and the values confirm it. Values alone cannot decide when no probed pre-activation is negative (tiny outputs):
    # then the statement list must be one of the forms known here, or nothing matches.
    after = [s for s in tile.body if _kind(s) == "Assign"]
    is_zero = lambda a: isinstance(a, (int, float)) and not isinstance(a, bool) and float(a) == 0.0
    relu_stmts = [s for s in after if s.op.name == "relu" or (s.op.name == "maximum" and any(is_zero(a) for a in s.args))]
    known_forms = all(s in relu_stmts or s.op.name in ("add", "multiply", "copy") for s in after)
    decisive = bool((ref < 0).any())
    if not decisive and not known_forms:
        raise Unmatched("no probed pre-activation is negative and the statements after the fold are not a known epilogue")
    epilogue = "relu" if relu_stmts else None
    want = np.maximum(ref, 0.0) if epilogue == "relu" else ref
    if np.allclose(got, want, rtol=1e-9, atol=1e-12):
        return {"variant": "gemm_f32", "inputs": [a_name, b_name, *bias], "outputs": [out_name],
                "params": {"batch": batch, "m": m, "n": n, "k": k, "b_trans": layout == "nk", "b_shared": bool(shared),
                           "bias": bool(bias), "epilogue": epilogue}}
    if decisive and not relu_stmts and np.allclose(got, np.maximum(ref, 0.0), rtol=1e-9, atol=1e-12):
        # a ReLU spelled some other way (a `where` on the sign, say): the values are unambiguous
        return {"variant": "gemm_f32", "inputs": [a_name, b_name, *bias], "outputs": [out_name],
                "params": {"batch": batch, "m": m, "n": n, "k": k, "b_trans": layout == "nk", "b_shared": bool(shared),
                           "bias": bool(bias), "epilogue": "relu"}}
    raise Unmatched("the loop is not a plain product (optionally plus a bias vector, optionally through ReLU)")


class NestInterpreter(RowInterpreter):
    """Runs a kernel whose loops nest (a dot product per key inside a loop over the keys) on a few probe cells. The
    innermost loops run once on whole vectors, as in RowInterpreter; a loop that contains another runs iteration by
    iteration, its own `Accum`s folding one value per trip. Every loop seeds the accumulators directly inside it with
    the op's identity (emmyptx/loops.py:92-102). Loads are recorded at their first execution only."""

    def __init__(self, tensors: dict, cells: np.ndarray, cols: int) -> None:
        super().__init__(tensors, cells, cols)
        self.vector = False                 # inside an innermost loop
        self.first_loads: dict = {}         # id(statement) -> (buffer, flat index at the first execution)

    def _value(self, a):
        return self.expr(a) if hasattr(a, "free_vars") or _kind(a) in ("Var", "Literal", "BinaryExpr") else self.lookup(a)

    def run(self, stmts) -> None:
        for s in stmts:
            k = _kind(s)
            if k in ("Loop", "StridedLoop"):
                extent = int(s.axis.extent.as_static())
                if getattr(s, "seed", True):
                    for a in s.body:
                        if _kind(a) == "Accum":
                            ident = getattr(a.op, "identity", None)
                            self.env[a.name] = np.full(self.cells.shape, 0.0 if ident is None else float(ident))
                if any(_kind(x) in ("Loop", "StridedLoop") for x in walk(s.body)):
                    for i in range(extent):
                        self.env[s.axis.name] = np.full(self.cells.shape, i, dtype=np.int64)
                        self.run(s.body)
                else:
                    if extent != self.cols:
                        raise Unmatched("the innermost loops of a fused attention run over the head dimension")
                    self.env[s.axis.name] = np.broadcast_to(np.arange(self.cols, dtype=np.int64), self.cells.shape)
                    self.vector = True
                    try:
                        self.run(s.body)
                    finally:
                        self.vector = False
            elif k == "Accum":
                if s.op.name not in _ACCUM:
                    raise Unmatched(f"no reduction folds with {s.op.name!r}")
                value = np.asarray(self.lookup(s.value), np.float64)
                base = np.asarray(self.lookup(s.base if s.base is not None else s.name), np.float64)
                if self.vector:
                    value, base = _ACCUM[s.op.name](value, axis=1, keepdims=True), base[:, :1]
                self.env[s.name] = np.broadcast_to(FLOAT_OPS[s.op.name][1](base, value), self.cells.shape)
            elif k == "Load":
                n_before = len(self.loads)
                CellInterpreter.run(self, [s])
                buf, flat, _ = self.loads.pop()
                assert len(self.loads) == n_before
                self.first_loads.setdefault(id(s), (buf, flat))
            elif k == "Assign":
                if s.op.name not in FLOAT_OPS:
                    raise OpError(f"elementwise op {s.op.name!r} is not supported")
                with np.errstate(all="ignore"):
                    self.env[s.name] = np.broadcast_to(FLOAT_OPS[s.op.name][1](*[np.asarray(self._value(a), np.float64) for a in s.args]),
                                                       self.cells.shape)
            elif k in ("WarpShuffle", "TreeHalve", "Sync", "Smem", "Init"):
                continue
            else:
                CellInterpreter.run(self, [s])


def match_attention_scalar(graph, kernel, launch: dict) -> dict:
    """softmax(Q K^T * scale) V written as scalar loops on float buffers (the reference's own attention cases:
    tools/torch_cases/fused.py:21-22, 31-36; models.py:17-19): recognised by running a few output cells and comparing
    them with the attention of the probe buffers, unmasked and lower-triangular, for every literal that could be the
    scale. Anything else the loops might compute -- another mask, a bias on the scores -- matches nothing."""
    tensors = tensor_table(graph)
    tiles = [s for s in kernel.body if _kind(s) == "Tile"]
    if len(kernel.body) != 1 or len(tiles) != 1:
        raise Unmatched("a fused attention kernel is one Tile")
    tile = tiles[0]
    writes = [s for s in walk(tile.body) if _kind(s) == "Write"]
    if len(writes) != 1 or writes[0].output not in tensors:
        raise Unmatched("a fused attention kernel writes one buffer")
    out_name = writes[0].output
    o_shape, o_dtype = tensors[out_name]
    if len(o_shape) < 2:
        raise Unmatched("attention output is [..., queries, d]")
    seq_q, d = int(o_shape[-2]), int(o_shape[-1])
    units = math.prod(o_shape[:-2])
    cells = math.prod(int(a.extent.as_static()) for a in tile.axes)
    if cells != units * seq_q * d:
        raise Unmatched("one tile cell per output element")
    if o_dtype not in ("f32", "f16", "bf16"):
        raise Unmatched("attention buffers are float")
    if d % 32 or not 32 <= d <= 128:
        raise Unmatched(f"attention head dim {d} has no variant (multiples of 32 up to 128)")
    rng = np.random.default_rng(1)
    rows = np.unique([0, 1, seq_q // 2, seq_q - 1])
    probe = np.unique([(int(rng.integers(0, units)) * seq_q + int(r)) * d + int(rng.integers(0, d)) for r in rows for _ in range(2)]).astype(np.int64)
    it = NestInterpreter(tensors, probe, d)
    rem = np.broadcast_to(probe[:, None], it.cells.shape).copy()
    for a in reversed(tile.axes):
        e = int(a.extent.as_static())
        it.env[a.name] = rem % e
        rem = rem // e
    it.run(tile.body)
    if len(it.writes) != 1 or len(it.writes[0][2]) != 1 or not np.array_equal(it.writes[0][1][:, 0], probe):
        raise Unmatched("a fused attention kernel writes O[unit, query, column], one cell each")
    got = np.asarray(it.writes[0][2][0], np.float64)[:, 0]
    un, qi, ci = probe // (seq_q * d), (probe // d) % seq_q, probe % d
    kk = np.arange(d)[None, :]
    loads = list(it.first_loads.values())
    q_idx = (un[:, None] * seq_q + qi[:, None]) * d + kk
    q_name = next((b for b, i in loads if tuple(tensors[b][0][-2:]) == (seq_q, d) and math.prod(tensors[b][0]) == units * seq_q * d
                   and np.array_equal(i, q_idx)), None)
    others = [(b, i) for b, i in loads if b != q_name]
    if q_name is None or not others:
        raise Unmatched("the loops do not read q[unit, query, :]")
    seq_k = int(tensors[others[0][0]][0][-2])
    k_idx0 = (un[:, None] * seq_k) * d + kk                      # key 0, all columns: the first trip of the key loop
    v_idx0 = np.broadcast_to((un[:, None] * seq_k) * d + ci[:, None], k_idx0.shape)
    fits = lambda b: len(tensors[b][0]) >= 2 and tuple(tensors[b][0][-2:]) == (seq_k, d) and math.prod(tensors[b][0]) == units * seq_k * d
    k_name = next((b for b, i in others if fits(b) and np.array_equal(i, k_idx0)), None)
    v_name = next((b for b, i in others if fits(b) and b != k_name and np.array_equal(i, v_idx0)), None)
    if k_name is None or v_name is None or {b for b, _ in loads} != {q_name, k_name, v_name}:
        raise Unmatched("the loops do not read k[unit, key, :] and v[unit, key, column] besides q")
    if len({tensors[b][1] for b in (q_name, k_name, v_name, out_name)}) != 1:
        raise Unmatched("q, k, v and the output share one dtype")
    dt = tensors[q_name][1]
    jj = np.arange(seq_k)
    qv = probe_values(q_name, dt, q_idx)                                                                    # [P, d]
    kv = probe_values(k_name, dt, ((un[:, None, None] * seq_k + jj[None, :, None]) * d + kk[None, :, :]))     # [P, seq_k, d]
    vv = probe_values(v_name, dt, (un[:, None] * seq_k + jj[None, :]) * d + ci[:, None])                    # [P, seq_k]
    dots = np.einsum("pd,pjd->pj", qv, kv)
    literals = {float(a) for s in walk(tile.body) if _kind(s) == "Assign" and s.op.name in ("multiply", "divide")
                for a in s.args if isinstance(a, (int, float)) and not isinstance(a, bool) and np.isfinite(a) and a != 0}
    scales = sorted(literals | {1.0 / x for x in literals} | {1.0})
    for causal in (False, True):
        for scale in scales:
            t = dots * scale
            if causal:
                t = np.where(jj[None, :] <= qi[:, None], t, -np.inf)
            ref = (_softmax64(t) * vv).sum(-1)
            if np.allclose(got, ref, rtol=1e-9, atol=1e-12):
                return {"variant": "attention_fwd", "inputs": [q_name, k_name, v_name], "outputs": [out_name],
                        "params": {"dtype": dt, "units": units, "seq_q": seq_q, "seq_k": seq_k, "d": d, "scale": scale, "causal": causal}}
    raise Unmatched("the loops are not softmax(q k^T * scale) v, unmasked or with the lower-triangular mask")


def match_loop_contraction(graph, kernel, launch: dict) -> dict:
    """A Tile with one cell per output element whose nested Loops fold `a[...] * b[...]` into one accumulator with `add`:
    the reference's convolution cases written as scalar loops (tools/torch_cases/conv.py:6-7 lowered as in
    emmyptx/kernel.py:786-797). The statement shape is checked structurally -- a chain of up to three Loops, the
    innermost holding Load, Load, Assign multiply, Accum add and nothing else; the accumulator seeded with zero exactly
    once -- and the three index expressions are run on probe values of the tile's and the loops' variables, fitted as
    affine maps, verified on every probe and checked against the buffers' sizes over the whole iteration space."""
    tensors = tensor_table(graph)
    tiles = [s for s in kernel.body if _kind(s) == "Tile"]
    if len(kernel.body) != 1 or len(tiles) != 1:
        raise Unmatched("a loop contraction is one Tile")
    tile = tiles[0]
    if not 1 <= len(tile.axes) <= 6:
        raise Unmatched("1 to 6 tile axes")
    body = [s for s in tile.body if _kind(s) not in ("Sync",)]
    inits = [s for s in body if _kind(s) == "Init"]
    rest = [s for s in body if _kind(s) != "Init"]
    if len(rest) != 2 or _kind(rest[0]) not in ("Loop",) or _kind(rest[1]) != "Write" or len(inits) > 1 or (inits and body[0] is not inits[0]):
        raise Unmatched("a loop contraction is [Init,] Loop, Write")
    chain, node = [], rest[0]
    while True:
        chain.append(node)
        if len(node.body) == 1 and _kind(node.body[0]) == "Loop":
            node = node.body[0]
            continue
        break
    if len(chain) > 3:
        raise Unmatched("more than 3 nested reduction loops")
    inner = chain[-1].body
    if [_kind(s) for s in inner] != ["Load", "Load", "Assign", "Accum"]:
        raise Unmatched("the innermost loop is Load, Load, Assign multiply, Accum add")
    la, lb, mul, acc = inner
    if len(la.names) != 1 or len(lb.names) != 1 or mul.op.name != "multiply" or sorted(map(str, mul.args)) != sorted([la.names[0], lb.names[0]]) \
            or la.names[0] == lb.names[0]:
        raise Unmatched("the product is of the two loaded values")
    ident = getattr(acc.op, "identity", None)
    if acc.op.name != "add" or acc.value != mul.name or acc.base not in (None, acc.name) or (ident is not None and float(ident) != 0.0):
        raise Unmatched("the accumulator folds the product with add")
    # seeded with zero exactly once: by an Init in front when the innermost Loop does not seed, else by a lone seeding Loop
    inner_seeds = bool(getattr(chain[-1], "seed", True))
    if inner_seeds and len(chain) > 1:
        raise Unmatched("the innermost loop would reset the accumulator on every outer trip")
    if not inner_seeds and not (inits and inits[0].name == acc.name and float(inits[0].identity) == 0.0):
        raise Unmatched("the accumulator is not seeded with zero")
    write = rest[1]
    if list(write.values) != [acc.name] or write.output not in tensors:
        raise Unmatched("the Write stores the accumulator")
    extents = [int(a.extent.as_static()) for a in tile.axes]
    loops = [int(lp.axis.extent.as_static()) for lp in chain]
    names = [a.name for a in tile.axes] + [lp.axis.name for lp in chain]
    if len(set(names)) != len(names) or min(extents + loops) < 1:
        raise Unmatched("axis names are distinct and extents positive")
    n = math.prod(extents)
    if n > 2**31 - 1:
        raise Unmatched(f"a tile of {n} cells has no contraction variant")
    for nm in (la.input, lb.input):
        if nm not in tensors or tensors[nm][1] not in ("f32", "f16", "bf16"):
            raise Unmatched("contraction inputs are float buffers")
    out_name = write.output
    if tensors[out_name][1] not in ("f32", "f16", "bf16"):
        raise Unmatched("the contraction writes a float buffer")
    # probe points of the joint iteration space: the origin, every unit vector, the far corner and random points
    all_ext = extents + loops
    rng = np.random.default_rng(2)
    pts = [np.zeros(len(all_ext), np.int64), np.asarray(all_ext, np.int64) - 1]
    pts += [np.eye(len(all_ext), dtype=np.int64)[a] for a, e in enumerate(all_ext) if e > 1]
    pts += [rng.integers(0, all_ext) for _ in range(200)]
    pts = np.unique(np.stack(pts), axis=0)
    digits = [pts[:, a] for a in range(len(all_ext))]
    it = CellInterpreter(tensors, np.arange(len(pts), dtype=np.int64), INT_OPS)
    for nm, d in zip(names, digits):
        it.env[nm] = d
    fits = {}
    for key, buf, index in (("a", la.input, la.index), ("b", lb.input, lb.index), ("out", out_name, write.index)):
        free = set()
        for e in index:
            free |= e.free_vars() if hasattr(e, "free_vars") else set()
        if free - set(names) or (key == "out" and free - set(names[:len(extents)])):
            raise Unmatched(f"the index of {buf!r} uses something other than the axis variables")
        off, coef = _fit_affine(it.flat_index(buf, index), digits, f"the index of {buf!r}")
        lo, hi = _reach(off, coef, all_ext)
        if lo < 0 or hi >= math.prod(tensors[buf][0]):
            raise Unmatched(f"the index of {buf!r} leaves the buffer (elements {lo}..{hi} of {math.prod(tensors[buf][0])})")
        fits[key] = (off, coef)
    o_off, o_coef = fits["out"]
    order = sorted((abs(c), e) for c, e in zip(o_coef[:len(extents)], extents) if e > 1)       # no two cells may write one element
    span = 0
    for c, e in order:
        if c <= span:
            raise Unmatched("two cells write the same element")
        span += c * (e - 1)
    na = len(extents)
    side = lambda key, buf: {"buffer": buf, "offset": fits[key][0], "coef": fits[key][1][:na], "loop_coef": fits[key][1][na:], "dtype": tensors[buf][1]}
    cmap = {"extents": extents, "loops": loops, "a": side("a", la.input), "b": side("b", lb.input),
            "out": {"offset": o_off, "coef": o_coef[:na], "dtype": tensors[out_name][1]}}
    return {"variant": "contract_indexed", "inputs": [la.input, lb.input], "outputs": [out_name], "params": {"n": n, "terms": math.prod(loops), "map": cmap}}


def match_kernel(graph, kernel, launch: dict, int_div: str = "floor") -> dict:
    kinds = {_kind(s) for s in walk(kernel.body)}
    if "MmaSyncPtx" in kinds:
        return match_contraction(graph, kernel, launch)
    if "Accum" in kinds:
        loops = [s for s in walk(kernel.body) if _kind(s) in ("Loop", "StridedLoop")]
        if any(_kind(x) in ("Loop", "StridedLoop") for lp in loops for x in walk(lp.body)):
            try:
                return match_attention_scalar(graph, kernel, launch)        # loops that nest: a dot product per key
            except Unmatched as first:
                try:
                    return match_loop_contraction(graph, kernel, launch)    # or a sum of products over several axes
                except Unmatched as second:
                    raise Unmatched(f"{first}; {second}") from None
        try:
            return match_dot(graph, kernel, launch)
        except Unmatched:
            pass
        try:
            return match_rowwise(graph, kernel, launch)
        except Unmatched as first:
            try:
                return match_loop_contraction(graph, kernel, launch)        # a product with other strides: a.t() @ b
            except Unmatched:
                raise first from None
    return match_streaming(graph, kernel, launch, int_div)
