"""Seeded synthetic inputs with the shapes and value distributions of the five configurations.

Seeds follow the reference's runner: argument i of a kernel is drawn from
`np.random.default_rng(i)` (`tools/run_local.py:86-87`, `tools/check_torch.py:186-191`).
"""
from __future__ import annotations

import numpy as np


def to_bf16_bits(values) -> np.ndarray:
    """fp32 -> bf16 bit patterns, round to nearest even (as `tools/run_local.py:31-37`)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(raw) -> np.ndarray:
    """bf16 bit patterns -> fp32 (as `tools/run_local.py:40-41`)."""
    return (np.asarray(raw).astype(np.uint32) << 16).view(np.float32)


def c1_input(n: int = 2**20, seed: int = 0) -> np.ndarray:
    """x ~ Uniform[-4, 4], float32."""
    return np.random.default_rng(seed).uniform(-4.0, 4.0, n).astype(np.float32)


def c2_input(n: int = 2**26, seed: int = 0) -> np.ndarray:
    """x ~ Uniform int32 [-2^30, 2^30]."""
    return np.random.default_rng(seed).integers(-2**30, 2**30, n, dtype=np.int32, endpoint=True)


def gemm_inputs(m: int, n: int, k: int, dtype: str, b_is_nk: bool = False, scaled: bool = True, batch: tuple = ()):
    """A[m,k], B[k,n] (or [n,k]) ~ N(0,1)/sqrt(k), rounded to `dtype` ('f16' or 'bf16'); `scaled=False` gives
    the plain N(0,1) operands of the reference's own matmul cases (tools/torch_cases/matmul.py:27-32), `batch`
    leading axes on both. Returns torch CPU tensors of that dtype."""
    import torch
    scale = np.float32(1.0 / np.sqrt(k)) if scaled else np.float32(1.0)
    lead = tuple(batch)
    a = np.random.default_rng(0).standard_normal(lead + (m, k), dtype=np.float32) * scale
    b = np.random.default_rng(1).standard_normal(lead + ((n, k) if b_is_nk else (k, n)), dtype=np.float32) * scale
    td = torch.float16 if dtype == "f16" else torch.bfloat16
    return torch.from_numpy(a).to(td), torch.from_numpy(b).to(td)


def attention_inputs_f32(units: int, seq_q: int, seq_k: int, d: int):
    """Q[units,seq_q,d], K, V[units,seq_k,d] ~ N(0,1) as float32 numpy arrays, argument i seeded with i, the way the
    reference's runner fills graph inputs (tools/run_local.py:86-87)."""
    return tuple(np.random.default_rng(seed).standard_normal((units, s, d)).astype(np.float32)
                 for seed, s in ((0, seq_q), (1, seq_k), (2, seq_k)))


def attention_inputs(units: int, seq_q: int, seq_k: int, d: int, dtype: str = "bf16"):
    """Q[units,seq_q,d], K, V[units,seq_k,d] ~ N(0,1), rounded to `dtype`; torch CPU tensors."""
    import torch
    td = torch.float16 if dtype == "f16" else torch.bfloat16
    out = []
    for seed, s in ((0, seq_q), (1, seq_k), (2, seq_k)):
        x = np.random.default_rng(seed).standard_normal((units, s, d), dtype=np.float32)
        out.append(torch.from_numpy(x).to(td))
    return tuple(out)


def layout_buffers(tensors: dict, arg_order: list) -> dict:
    """Buffers for a data-movement kernel: float argument i ~ N(0, 1) seeded with i (tools/run_local.py:86-87), integer
    (index) arguments uniform in [-1000, 1000); the output starts as zeros (:92-93)."""
    bufs = {}
    for i, name in enumerate(arg_order):
        shape = tensors[name]["shape"]
        if name == "out":
            bufs[name] = np.zeros(shape, np.float32)
        elif tensors[name].get("dtype") == "i64":               # an index buffer: either sign, beyond the table's size
            bufs[name] = np.random.default_rng(i).integers(-1000, 1000, shape).astype(np.int64)
        else:
            bufs[name] = np.random.default_rng(i).standard_normal(shape).astype(np.float32)
    return bufs


def seeded_buffers(tensors: dict, arg_order: list) -> dict:
    """Buffers for a kernel whose last argument is its output: argument i ~ N(0, 1) seeded with i (tools/run_local.py:86-87),
    the output zeroed (:92-93)."""
    bufs = {}
    for i, name in enumerate(arg_order):
        shape = tensors[name]["shape"]
        bufs[name] = np.zeros(shape, np.float32) if i == len(arg_order) - 1 else np.random.default_rng(i).standard_normal(shape).astype(np.float32)
    return bufs


LAYOUT_EXPECTED = {     # what each data-movement case computes, on the buffers of layout_buffers (numpy, exact)
    "s_transpose": lambda b: b["X"].T, "s_permute": lambda b: b["X"].transpose(2, 0, 1) * np.float32(2), "s_slice": lambda b: b["X"][:, 10:50] * np.float32(2),
    "s_strided_slice": lambda b: b["X"][::2] + np.float32(1), "s_flip": lambda b: b["X"][:, ::-1], "s_stack": lambda b: np.stack([b["A"], b["B"]]),
    "s_cat_cond": lambda b: np.concatenate([b["A"], b["B"]], -1), "s_pad_cond": lambda b: np.pad(b["X"], ((0, 0), (3, 3))),
    "s_tril": lambda b: np.tril(b["X"]), "s_tril_select": lambda b: np.tril(b["X"]),
    "s_window_let": lambda b: np.where((np.arange(128) >= 3) & (np.arange(128) < 120), b["X"], np.float32(0)) * np.float32(2), "s_repeat": lambda b: np.tile(b["X"], (2, 1)),
    "s_roll": lambda b: np.roll(b["X"], 3, -1), "s_embedding": lambda b: b["SRC"][np.abs(b["IDX"]) % 100],
    "s_gather": lambda b: np.take_along_axis(b["SRC"], np.abs(b["IDX"]) % 64, 1),
    "c_avg_pool1d": lambda b: ((b["X"][:, 0::4] + b["X"][:, 1::4]) + (b["X"][:, 2::4] + b["X"][:, 3::4])) * np.float32(0.25),
    "c_max_pool2d": lambda b: b["X"].reshape(8, 16, 2, 16, 2).max(axis=(2, 4)),
    "s_cat_a": lambda b: np.concatenate([b["A"], np.zeros((32, 48), np.float32)], -1),
    "s_cat_b": lambda b: np.concatenate([np.zeros((32, 64), np.float32), b["B"]], -1),
}


def conv_expected(case: str, b: dict) -> np.ndarray:
    """The reference's convolution cases (tools/torch_cases/conv.py:6-7: stride 1, no padding, no bias, batch 1) in
    float64 on the buffers of layout_buffers: out[o, i...] = sum over c and the taps of W[o, c, t...] * X[c, i + t...]."""
    x, w = b["X"].astype(np.float64), b["W"].astype(np.float64)
    taps = w.shape[2:]
    win = np.lib.stride_tricks.sliding_window_view(x, taps, axis=tuple(range(1, x.ndim)))      # [c, i..., t...]
    if case == "c_conv1d":
        return np.einsum("oct,cit->oi", w, win)
    return np.einsum("ocuv,cijuv->oij", w, win)


def reduce_expected(name: str, b: dict) -> np.ndarray:
    """What the seeded row / column / fp32-product kernels compute (tools/torch_cases/reductions.py, fused.py, matmul.py),
    in float64 on the buffers of seeded_buffers. `row_<op>` reduces the last axis of X, `col_<op>` the first."""
    f = lambda k: b[k].astype(np.float64)
    if name == "m_mm":
        return f("A") @ f("B")
    if name == "m_bmm":
        return np.einsum("bmk,bkn->bmn", f("A"), f("B"))
    if name == "m_linear_bias_relu":
        return np.maximum(f("A") @ f("B").T + f("bias"), 0.0)
    if name == "m_transpose_lhs":
        return f("A").T @ f("B")
    kind, op = name.split("_", 1)
    x = f("X") if kind == "row" else f("X").T                 # reduce the last axis either way
    mx = x.max(-1, keepdims=True)
    lse = np.log(np.exp(x - mx).sum(-1, keepdims=True)) + mx
    n = x.shape[-1]
    mean = x.mean(-1, keepdims=True)
    var_b = ((x - mean) ** 2).mean(-1, keepdims=True)
    out = {
        "sum": lambda: x.sum(-1), "mean": lambda: x.mean(-1), "amax": lambda: x.max(-1), "amin": lambda: x.min(-1), "prod": lambda: x.prod(-1),
        "norm2": lambda: np.sqrt((x * x).sum(-1)), "var": lambda: x.var(-1, ddof=1), "std": lambda: x.std(-1, ddof=1), "logsumexp": lambda: lse[..., 0],
        "softmax": lambda: np.exp(x - lse), "log_softmax": lambda: x - lse,
        "layer_norm": lambda: (x - mean) / np.sqrt(var_b + 1e-5) * f("W") + f("B"),
        "rms_norm": lambda: x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * f("W"),
        "normalize": lambda: x / np.maximum(np.sqrt((x * x).sum(-1, keepdims=True)), 1e-12),
        "dot": lambda: x @ f("W"),
    }[op]()
    return out if kind == "row" or out.ndim == 1 else out.T

