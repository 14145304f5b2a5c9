"""Elementwise op table: one IR op name -> what computes it on the device.

Mirror of the reference's `emmyptx/ops.py`: there `lower_op(em, name, args, dst)` prints the PTX
instructions of `dst = name(*args)` into an Emitter (`ops.py:212-290`) and `lower_int_op` does the same for
s32 values (`:301-309`); an unknown name raises `OpError` (`:29`, `:290`, `:309`). Here nothing is printed:
`em` is a `Program`, the straight-line scalar program of one tile cell, and lowering an op appends one
step to it. The matcher (`emmyptx/match.py`) then recognises whole programs and binds them to a
precompiled sm_100a kernel; the numeric meaning of each step (float64 / exact integers, as the
reference's checker evaluates cases, `tools/check_torch.py:194-237`) lives in `FLOAT_OPS` / `INT_OPS`.
"""
from __future__ import annotations

import math

import numpy as np


class OpError(NotImplementedError):
    pass


def _erf(x):
    return np.vectorize(math.erf, otypes=[np.float64])(x)


def _wrap32(v):
    return ((np.asarray(v, dtype=np.int64) + 2**31) % 2**32) - 2**31


def _floor_div_int(a, b):
    return _wrap32(np.floor_divide(a, b))


def _trunc_div_int(a, b):
    q = np.abs(a) // np.abs(b)
    return _wrap32(np.where((a < 0) != (b < 0), -q, q))


# Names the reference lowers as a plain register move (emmyptx/ops.py:236-237: the value is already fp32 in a register,
# the narrowing or widening happened at the load or happens at the store).
MOVE_OPS = ("pad", "from_f8e4m3", "from_f8e5m2", "to_f8e4m3", "to_f8e5m2")

# name -> (arity, float64 meaning). Comparisons give 1.0 / 0.0 masks (the reference's convention, ops.py:116-120).
FLOAT_OPS = {
    "add": (2, np.add), "subtract": (2, np.subtract), "multiply": (2, np.multiply), "divide": (2, np.divide),
    "maximum": (2, np.maximum), "minimum": (2, np.minimum), "relu": (1, lambda a: np.maximum(a, 0.0)),
    "square": (1, np.square), "copy": (1, lambda a: a), "negative": (1, np.negative), "abs": (1, np.abs),
    "reciprocal": (1, np.reciprocal), "sqrt": (1, np.sqrt), "rsqrt": (1, lambda a: 1.0 / np.sqrt(a)),
    "exp": (1, np.exp), "exp_fast": (1, np.exp), "log": (1, np.log), "sigmoid": (1, lambda a: 1.0 / (1.0 + np.exp(-a))),
    "tanh": (1, np.tanh), "erf": (1, _erf), "sin": (1, np.sin), "cos": (1, np.cos), "pow": (2, np.power),
    "equal": (2, lambda a, b: (a == b) * 1.0), "not_equal": (2, lambda a, b: (a != b) * 1.0),
    "greater": (2, lambda a, b: (a > b) * 1.0), "less": (2, lambda a, b: (a < b) * 1.0),
    "greater_equal": (2, lambda a, b: (a >= b) * 1.0), "less_equal": (2, lambda a, b: (a <= b) * 1.0),
    "where": (3, lambda c, a, b: np.where(c != 0, a, b)),
    "floor_divide": (2, lambda a, b: np.floor(a / b)), "mod": (2, lambda a, b: a - b * np.floor(a / b)),
    "remainder": (2, lambda a, b: a - b * np.floor(a / b)),
    # logical and / or / not of 1.0 / 0.0 masks (emmyptx/ops.py:274-279)
    "bitwise_and": (2, lambda a, b: ((a != 0) & (b != 0)) * 1.0), "bitwise_or": (2, lambda a, b: ((a != 0) | (b != 0)) * 1.0),
    "bitwise_not": (1, lambda a: (a == 0) * 1.0),
}
FLOAT_OPS.update({name: FLOAT_OPS["copy"] for name in MOVE_OPS})

# Integer ops work on wrapped int32 values. `floor_divide` / `mod` follow torch (round toward minus
# infinity), the semantics the reference's cases are checked against (tools/torch_cases/dtypes.py:17-19);
# the reference's own PTX truncates (ops.py:294-297), which `INT_OPS_TRUNC` reproduces.
INT_OPS = {
    "add": (2, lambda a, b: _wrap32(a + b)), "subtract": (2, lambda a, b: _wrap32(a - b)),
    "multiply": (2, lambda a, b: _wrap32(a * b)), "floor_divide": (2, _floor_div_int), "divide": (2, _floor_div_int),
    "mod": (2, lambda a, b: _wrap32(np.mod(a, b))), "remainder": (2, lambda a, b: _wrap32(np.mod(a, b))),
    "maximum": (2, np.maximum), "minimum": (2, np.minimum), "bitwise_and": (2, np.bitwise_and),
    "bitwise_or": (2, np.bitwise_or), "bitwise_xor": (2, np.bitwise_xor),
    "left_shift": (2, lambda a, b: _wrap32(a << b)), "right_shift": (2, lambda a, b: a >> b),
    "copy": (1, lambda a: a), "abs": (1, lambda a: _wrap32(np.abs(a))),
}
INT_OPS_TRUNC = dict(INT_OPS, floor_divide=(2, _trunc_div_int), divide=(2, _trunc_div_int),
                     mod=(2, lambda a, b: _wrap32(a - b * _trunc_div_int(a, b))),
                     remainder=(2, lambda a, b: _wrap32(a - b * _trunc_div_int(a, b))))


class Program(list):
    """Steps `(dst, kind, name, args)` of one cell's scalar program, in order; kind is 'f32' or 's32'."""


def lower_op(em: Program, name: str, args: list, dst) -> None:
    """Append `dst = name(*args)` for an f32 elementwise op."""
    if name not in FLOAT_OPS:
        raise OpError(f"elementwise op {name!r} is not supported")
    if len(args) != FLOAT_OPS[name][0]:
        raise OpError(f"elementwise op {name!r} takes {FLOAT_OPS[name][0]} arguments, got {len(args)}")
    em.append((dst, "f32", name, list(args)))


def lower_int_op(em: Program, name: str, args: list, dst) -> None:
    """Append `dst = name(*args)` for an s32 elementwise op."""
    if name not in INT_OPS:
        raise OpError(f"integer elementwise op {name!r} is not supported")
    em.append((dst, "s32", name, list(args)))
