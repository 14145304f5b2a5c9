"""Row reductions and normalisations against the float64 oracle, on the reference's own cases
(tools/torch_cases/reductions.py:6-19, fused.py:6-13) at its tolerance classes (tools/torch_cases/__init__.py:16-21),
then over row lengths that exercise every thread-group width, every cluster size, the unaligned path and the split
(multi-block) path.

Tolerances: ROUND (1e-6) for extrema, exact for argmax, RED (1e-4) for sums of a few thousand terms; for longer
rows the absolute floor grows with sqrt(cols) (the rounding of a sum of cols terms of unit size).
"""
import numpy as np
import pytest

from oracle import reference

pytestmark = pytest.mark.gpu

REDUCING = ["sum", "mean", "amax", "amin", "prod", "var", "std", "norm2", "logsumexp", "argmax", "dot", "cosine"]
MAPPING = ["softmax", "log_softmax", "layer_norm", "rms_norm", "normalize"]


def _data(op, rows, cols, seed=0):
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    if op == "prod" and cols <= 4096:
        x = 1 + x * 0.01                                   # keeps the product in range, as r_prod does
    elif op == "prod":
        # Long rows: fp32 products of numbers near 1 drift systematically (torch's own float32 prod is 3e-4 off at
        # 2^18 terms), so the factors are powers of two and signs, whose product is exact in any order.
        u = torch.rand(rows, cols, generator=g)
        x = torch.ones(rows, cols)
        x[u < 1e-4] = 2.0
        x[(u >= 1e-4) & (u < 2e-4)] = 0.5
        x[u > 0.99] = -1.0
    w = torch.randn(cols, generator=g) if op in ("layer_norm", "rms_norm", "dot") else None
    if op == "cosine":
        w = torch.randn(rows, cols, generator=g)
    b = torch.randn(cols, generator=g) if op == "layer_norm" else None
    eps = {"layer_norm": 1e-5, "rms_norm": 1e-6, "normalize": 1e-12, "cosine": 1e-8}.get(op, 0.0)
    return x, w, b, eps


def _run(op, x, w, b, eps, cuda, **kw):
    import torch
    from emmyptx import runtime
    dev = lambda t: None if t is None else t.to(cuda)
    y = runtime.rowwise(op, dev(x), dev(w), dev(b), eps, **kw)
    torch.cuda.synchronize()
    return y.cpu()


def _check(op, got, ref, cols, rtol=1e-4, atol=1e-4):
    if op == "argmax":
        assert np.array_equal(got.numpy(), ref.numpy())
        return
    if op in ("amax", "amin"):
        rtol = atol = 1e-6
    elif op in ("sum", "dot", "norm2", "logsumexp", "log_softmax"):
        atol = atol + 1e-6 * cols ** 0.5
    res = reference.compare(got.numpy(), ref.numpy(), rtol, atol)
    assert res["ok"], (op, cols, res)


# ---- the reference's cases ------------------------------------------------------------------------------------
@pytest.mark.parametrize("op,rows,cols,rtol,atol", [
    ("sum", 1, 8192, 1e-4, 1e-4),            # r_sum
    ("sum", 1, 1 << 20, 1e-3, 1e-2),         # r_big_sum_default
    ("mean", 128, 300, 1e-4, 1e-4),          # r_mean_rows
    ("amax", 96, 200, 1e-6, 1e-6), ("amin", 96, 200, 1e-6, 1e-6),      # r_amax_amin
    ("prod", 64, 32, 1e-4, 1e-4),            # r_prod
    ("var", 64, 512, 1e-4, 1e-4), ("std", 64, 512, 1e-4, 1e-4),        # r_var_std
    ("norm2", 64, 512, 1e-4, 1e-4),          # r_vector_norm
    ("logsumexp", 64, 512, 1e-4, 1e-4),      # r_logsumexp
    ("argmax", 64, 512, 0, 0),               # r_argmax, r_max_with_idx
    ("cosine", 64, 256, 1e-4, 1e-5),         # f_cosine_sim
    ("dot", 256, 128, 1e-3, 1e-3),           # m_matvec (tools/torch_cases/matmul.py:22), the matmul class
    ("softmax", 64, 1000, 1e-3, 1e-5),       # f_softmax
    ("log_softmax", 48, 256, 1e-3, 1e-4),    # f_log_softmax
    ("layer_norm", 64, 768, 1e-3, 1e-4),     # f_layer_norm_affine
    ("rms_norm", 32, 512, 1e-3, 1e-4),       # f_rms_norm
    ("normalize", 64, 256, 1e-4, 1e-5),      # f_normalize
])
def test_reference_cases(op, rows, cols, rtol, atol, cuda):
    x, w, b, eps = _data(op, rows, cols)
    got = _run(op, x, w, b, eps, cuda)
    ref = reference.rowwise_reference(op, x, w, b, eps)
    if op == "argmax":
        assert np.array_equal(got.numpy(), ref.numpy())
    else:
        res = reference.compare(got.numpy(), ref.numpy(), rtol, atol)
        assert res["ok"], res


# ---- every group width, ragged and unaligned rows ----------------------------------------------------------------
@pytest.mark.parametrize("cols", [1, 3, 4, 5, 31, 64, 127, 256, 257, 500, 1000, 1024, 1028, 2048, 3000, 4096, 4099, 8192,      # one CTA or less per row
                                  8196, 16384, 20001, 32768, 40000, 65536])                             # clusters of 2, 4, 8
@pytest.mark.parametrize("op", REDUCING + MAPPING)
def test_cached_rows(op, cols, cuda):
    rows = 37 if cols <= 8192 else 11
    x, w, b, eps = _data(op, rows, cols, seed=cols)
    got = _run(op, x, w, b, eps, cuda)
    _check(op, got, reference.rowwise_reference(op, x, w, b, eps), cols)


@pytest.mark.parametrize("rows,cols", [(1, 65540), (3, 80001), (2, 1 << 18), (150, 70000), (1, (1 << 22) + 4), (700, 66000)])
@pytest.mark.parametrize("op", REDUCING + MAPPING)
def test_split_rows(op, rows, cols, cuda):
    x, w, b, eps = _data(op, rows, cols, seed=rows)
    got = _run(op, x, w, b, eps, cuda)
    _check(op, got, reference.rowwise_reference(op, x, w, b, eps), cols)


@pytest.mark.parametrize("op", ["sum", "var", "logsumexp", "argmax", "softmax", "layer_norm"])
def test_views_that_start_off_a_16_byte_boundary(op, cuda):
    import torch
    from emmyptx import runtime
    for rows, cols in ((9, 516), (2, 40000), (2, 70001)):
        x, w, b, eps = _data(op, rows, cols, seed=3)
        flat = torch.zeros(rows * cols + 1, device=cuda)
        flat[1:] = x.reshape(-1).to(cuda)
        a = runtime.rowwise(op, flat[1:].view(rows, cols), None if w is None else w.to(cuda), None if b is None else b.to(cuda), eps)
        torch.cuda.synchronize()
        _check(op, a.cpu(), reference.rowwise_reference(op, x, w, b, eps), cols)


def test_leading_axes_are_rows(cuda):
    import torch
    x = torch.randn(4, 6, 50, generator=torch.Generator().manual_seed(1))
    got = _run("softmax", x, None, None, 0.0, cuda)
    assert got.shape == x.shape
    _check("softmax", got, reference.rowwise_reference("softmax", x), 50)
    assert _run("amax", x, None, None, 0.0, cuda).shape == (4, 6)


# ---- special values: torch's float32 result is the expectation (NaN placement, infinities, ties) -------------------------
@pytest.mark.parametrize("cols", [40, 5000, 70000])
def test_nan_inf_and_ties(cols, cuda):
    import torch
    g = torch.Generator().manual_seed(5)
    x = torch.randn(8, cols, generator=g)
    x[1, cols // 2] = float("nan")
    x[2, 7] = float("inf")
    x[3, cols - 1] = float("-inf")
    x[4] = float("-inf")
    x[5, 3] = x[5, cols - 2] = 9.0                       # a tie: the first index wins
    x[6, 11] = float("nan"); x[6, 2] = float("inf")      # NaN outranks +inf
    x[7] = 2.5
    for op in ("amax", "amin", "argmax", "logsumexp", "softmax", "log_softmax", "sum"):
        got = _run(op, x, None, None, 0.0, cuda).numpy()
        want = reference.rowwise_reference(op, x.float()).numpy() if op != "argmax" else x.argmax(-1).numpy()
        if op == "argmax":
            assert np.array_equal(got, want), op
        else:
            assert np.array_equal(np.isnan(got), np.isnan(want)), op
            assert np.allclose(got, want, rtol=1e-4, atol=1e-5, equal_nan=True), op


def test_split_result_does_not_depend_on_block_order(cuda):
    """The pieces of a long row are merged in index order by whichever block finishes last: repeated launches agree
    bit for bit."""
    import torch
    from emmyptx import runtime
    x = torch.randn(3, 1 << 21, generator=torch.Generator().manual_seed(2)).to(cuda)
    for op in ("sum", "var", "logsumexp"):
        first = runtime.rowwise(op, x).clone()
        for _ in range(5):
            assert torch.equal(runtime.rowwise(op, x), first)


def test_properties_at_size(cuda):
    """Size-independent checks on 256 MiB: softmax rows sum to one and are invariant to a shift of the row; the
    sum is linear; layer-normalised rows have zero mean and unit variance."""
    import torch
    from emmyptx import runtime
    x = torch.randn(65536, 1024, device=cuda, generator=torch.Generator(device=cuda).manual_seed(0))
    p = runtime.rowwise("softmax", x)
    assert (runtime.rowwise("sum", p) - 1).abs().max().item() <= 1e-5
    q = runtime.rowwise("softmax", x + 3.0)
    assert (p - q).abs().max().item() <= 1e-6
    s = runtime.rowwise("sum", x)
    assert (runtime.rowwise("sum", x * 2.0) - 2.0 * s).abs().max().item() == 0.0
    z = runtime.rowwise("layer_norm", x, eps=0.0)
    assert runtime.rowwise("mean", z).abs().max().item() <= 1e-6
    assert (runtime.rowwise("var", z) * (1023 / 1024) - 1).abs().max().item() <= 1e-5


def test_workspace_contract(cuda, lib):
    import torch
    from emmyptx import runtime
    assert lib.emmyb200_rowwise_workspace_bytes(0, 100, 65536) == 0
    need = lib.emmyb200_rowwise_workspace_bytes(0, 4, 1 << 20)
    assert need > 0 and need % 256 == 0
    assert lib.emmyb200_rowwise_workspace_bytes(99, 4, 8) == -1
    x = torch.randn(4, 1 << 20, device=cuda)
    y = torch.empty(4, device=cuda)
    f = lib.emmyb200_rowwise_f32
    assert f(0, x.data_ptr(), None, None, y.data_ptr(), 4, 1 << 20, 0.0, None, 0, None) == -1
    assert b"workspace" in lib.emmyb200_last_error()
    ws = torch.full((need,), 0xAB, dtype=torch.uint8, device=cuda)           # contents do not matter
    assert f(0, x.data_ptr(), None, None, y.data_ptr(), 4, 1 << 20, 0.0, ws.data_ptr(), need, None) == 0
    torch.cuda.synchronize()
    assert torch.allclose(y, x.double().sum(-1).float(), rtol=1e-4, atol=1e-2)
    assert torch.equal(runtime.rowwise("sum", x, workspace=ws), y)          # and it can be reused


def test_rejects_bad_arguments(cuda, lib):
    import torch
    x = torch.zeros(64, device=cuda)
    p = x.data_ptr()
    f = lib.emmyb200_rowwise_f32
    assert f(11, p, None, None, p, 8, 8, 0.0, None, 0, None) == -1            # unknown op
    assert f(0, None, None, None, p, 8, 8, 0.0, None, 0, None) == -1
    assert f(0, p, p, None, p, 8, 8, 0.0, None, 0, None) == -1                # a weight for a plain sum
    assert f(19, p, p, p, p, 8, 8, 0.0, None, 0, None) == -1                  # rms_norm has no bias
    assert f(0, p, None, None, p, 8, 0, 0.0, None, 0, None) == -2             # empty rows
    assert f(0, p, None, None, p, 0, 8, 0.0, None, 0, None) == 0              # no rows: nothing to do
    assert f(0, p, None, None, p, -1, 8, 0.0, None, 0, None) == -1
