"""The oracle proper: each configuration's expression evaluated by torch / numpy on CPU.

float64 is the truth the reference's harness compares against (`tools/check_torch.py:194-237`);
the float32 evaluations are the reference's "CPU path" that `bench.py` times.
"""
from __future__ import annotations

import numpy as np


# ---- C1: y = exp(x) + sin(x) * tanh(x) ---------------------------------------------------------
def c1_f64(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float64)
    return np.exp(x) + np.sin(x) * np.tanh(x)


def c1_f32_torch(x):
    """The same expression as torch evaluates it in fp32 (three ops, each rounded)."""
    import torch
    return torch.exp(x) + torch.sin(x) * torch.tanh(x)


UNARY_F64 = {
    "exp": np.exp, "sin": np.sin, "cos": np.cos, "tanh": np.tanh,
    "gelu_tanh": lambda x: 0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x**3))),
    "exp_sin_tanh": lambda x: np.exp(x) + np.sin(x) * np.tanh(x),
    "sigmoid": lambda x: 1.0 / (1.0 + np.exp(-x)), "silu": lambda x: x / (1.0 + np.exp(-x)), "relu": lambda x: np.maximum(x, 0.0),
}


def ulp32(ref64: np.ndarray) -> np.ndarray:
    """Size of one fp32 ulp at |ref| (the spacing of floats at the rounded reference)."""
    r = np.abs(ref64.astype(np.float32)).astype(np.float64)
    r = np.minimum(r, float(np.finfo(np.float32).max))
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(r > 0, r, 1.0)))
    e = np.where(r > 0, e, -149.0)
    return np.exp2(np.maximum(e - 23.0, -149.0))


def ulp_error(got32: np.ndarray, ref64: np.ndarray) -> np.ndarray:
    return np.abs(got32.astype(np.float64) - ref64) / ulp32(ref64)


def c1_condition_ulp(got32: np.ndarray, x32: np.ndarray) -> np.ndarray:
    """Error of the composite in ulps of its largest term: |y - y64| / ulp32(max(|e^x|, |sin tanh|, |y|)).
    exp(x) + sin(x) tanh(x) cancels near x = -3.18, where even a per-op correctly rounded fp32
    evaluation is thousands of output-ulps off; measured against the largest term, a <= 2 ulp
    implementation of each function stays below about 2 + 2 + 1."""
    x = x32.astype(np.float64)
    e, st = np.exp(x), np.sin(x) * np.tanh(x)
    y = e + st
    scale = np.maximum(np.maximum(np.abs(e), np.abs(st)), np.abs(y))
    return np.abs(got32.astype(np.float64) - y) / ulp32(scale)


# ---- C2: y[i] = (x[(i*mul + add) mod n] // d) ^ (i >> shift) -----------------------------------------
def c2_reference(x: np.ndarray, mul: int = 7919, add: int = 13, d: int = 3, shift: int = 2, trunc: bool = False) -> np.ndarray:
    """Exact (int64) index arithmetic; floor division as torch's `//` (`tools/torch_cases/dtypes.py:17-19`),
    or truncating division as the reference's `div.s32` (`emmyptx/ops.py:294-297`) with `trunc`."""
    n = x.shape[0]
    i = np.arange(n, dtype=np.int64)
    g = x[(i * mul + add) % n].astype(np.int64)
    q = np.where(g < 0, -((-g) // d), g // d) if trunc else g // d
    return (q ^ (i >> shift)).astype(np.int32)


def c2_torch(x, mul: int = 7919, add: int = 13, d: int = 3, shift: int = 2):
    """The torch CPU evaluation that `bench.py` times (int64 index, floor division)."""
    import torch
    n = x.shape[0]
    i = torch.arange(n, dtype=torch.int64)
    g = x[(i * mul + add) % n]
    return torch.bitwise_xor(torch.div(g, d, rounding_mode="floor"), (i >> shift).to(torch.int32))


# ---- C3 / C4: GEMM (+ tanh-GELU), fp32 accumulation, one rounding to the output type ----------------
def gemm_reference(a, b, epilogue: str | None = None, b_is_nk: bool = False, double: bool = False):
    """fp32 (or fp64) product of the already-rounded inputs; epilogue on the unrounded accumulator
    (compute-dtype rule of `emmyptx/kernel.py:31-38`: values are f32 until the final store)."""
    import torch
    dt = torch.float64 if double else torch.float32
    bb = b.to(dt)
    c = a.to(dt) @ (bb.t() if b_is_nk else bb)
    if epilogue == "gelu_tanh":
        c = torch.nn.functional.gelu(c, approximate="tanh")
    return c


def gemm_tolerance_ok(got, ref, rel: float = 1e-2):
    """|c - ref| <= rel |ref| + rel std(ref): relative 1e-2 with an absolute floor scaled to the
    output's spread. Returns (ok, worst ratio to the bound)."""
    import torch
    ref = ref.to(torch.float64)
    err = (got.to(torch.float64) - ref).abs()
    bound = rel * ref.abs() + rel * ref.std()
    ratio = float((err / bound).max())
    return ratio <= 1.0, ratio


# ---- C5: attention forward ----------------------------------------------------------------------------
def attention_reference(q, k, v, scale: float | None = None, double: bool = False, causal: bool = False):
    """softmax(q k^T * scale) v per unit, fp32 (or fp64) throughout, on the already-rounded inputs. `causal`: scores of
    keys after the query are filled with -inf (tools/torch_cases/fused.py:31-36, models.py:17-19)."""
    import torch
    dt = torch.float64 if double else torch.float32
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(q.shape[-2], k.shape[-2], dtype=torch.bool).tril(), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v)


# ---- row reductions and normalisations (tools/torch_cases/reductions.py:6-19, fused.py:6-13) ----------------------
def rowwise_reference(op: str, x, weight=None, bias=None, eps: float = 0.0):
    """float64 torch evaluation of one row op on float32 data, as tools/check_torch.py:194-237 defines truth."""
    import torch
    import torch.nn.functional as F
    x = x.double()
    w = None if weight is None else weight.double()
    b = None if bias is None else bias.double()
    n = x.shape[-1]
    if op == "sum": return x.sum(-1)
    if op == "mean": return x.mean(-1)
    if op == "amax": return x.amax(-1)
    if op == "amin": return x.amin(-1)
    if op == "prod": return x.prod(-1)
    if op == "var": return x.var(-1)
    if op == "std": return x.std(-1)
    if op == "norm2": return torch.linalg.vector_norm(x, dim=-1)
    if op == "logsumexp": return torch.logsumexp(x, -1)
    if op == "argmax": return x.argmax(-1)
    if op == "dot": return x @ w
    if op == "cosine": return F.cosine_similarity(x, w, dim=-1, eps=eps)
    if op == "softmax": return torch.softmax(x, -1)
    if op == "log_softmax": return torch.log_softmax(x, -1)
    if op == "layer_norm": return F.layer_norm(x, (n,), w, b, eps)
    if op == "rms_norm":
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return y if w is None else y * w
    if op == "normalize": return F.normalize(x, dim=-1, eps=eps)
    raise KeyError(op)


def colwise_reference(op: str, x, eps: float = 0.0):
    """The same ops over axis -2 (dim 0 of a matrix; tools/torch_cases/reductions.py:9, fused.py:7), float64."""
    import torch
    y = rowwise_reference(op, x.transpose(-1, -2), eps=eps)
    return y.transpose(-1, -2) if y.dim() == x.dim() else y


def cumsum_reference(x):
    """torch.cumsum(x, -1) in float64 (tools/torch_cases/reductions.py:18)."""
    import torch
    return torch.cumsum(x.double(), -1)


# ---- the reference harness's comparison -----------------------------------------------------------------
def compare(got: np.ndarray, ref: np.ndarray, rtol: float, atol: float) -> dict:
    """`tools/check_torch.py:260-278`: isclose with equal NaNs, plus the vacuity check (an all-zero
    output against a non-zero reference fails)."""
    g, r = got.reshape(ref.shape).astype(np.float64), ref.astype(np.float64)
    close = np.isclose(g, r, rtol=rtol, atol=atol, equal_nan=True)
    vacuous = bool(np.all(g == 0)) and not bool(np.all(r == 0))
    with np.errstate(invalid="ignore"):
        err = np.where((g == r) | (np.isnan(g) & np.isnan(r)), 0.0, np.abs(g - r))
    return dict(ok=bool(close.all()) and not vacuous, off=int((~close).sum()), max_err=float(np.nanmax(err, initial=0.0)),
                vacuous=vacuous)
