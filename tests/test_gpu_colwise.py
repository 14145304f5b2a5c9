"""Reductions over the middle axis (dim 0 of a matrix), the normalisations over it, and cumsum, against the float64
oracle: the reference's cases r_sum_dim0, r_sum_multi_dim, r_cumsum (tools/torch_cases/reductions.py:9-10, :18) and
f_softmax_dim0 (fused.py:7) at its tolerances, then shapes that exercise one and many row slices, ragged and
unaligned columns, stacks of planes, and special values.

Tolerances as for the row kernels: ROUND (1e-6) for extrema, exact for argmax, RED (1e-4) with an absolute floor that
grows with sqrt(length) for long sums.
"""
import numpy as np
import pytest

from oracle import reference

pytestmark = pytest.mark.gpu

OPS = ["sum", "mean", "amax", "amin", "prod", "var", "std", "norm2", "logsumexp", "argmax", "softmax", "log_softmax", "normalize"]


def _data(op, shape, seed=0):
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    if op == "prod":
        rows = shape[-2]
        if rows <= 4096:
            x = 1 + x * 0.01
        else:                                     # exact factors for long products (see the row-kernel tests)
            u = torch.rand(*shape, generator=g)
            x = torch.ones(*shape)
            x[u < 1e-4] = 2.0
            x[(u >= 1e-4) & (u < 2e-4)] = 0.5
            x[u > 0.99] = -1.0
    return x


def _check(op, got, ref, n):
    if op == "argmax":
        assert np.array_equal(got.numpy(), ref.numpy())
        return
    rtol = atol = 1e-4
    if op in ("amax", "amin"):
        rtol = atol = 1e-6
    elif op in ("sum", "norm2", "logsumexp", "log_softmax"):
        atol = atol + 1e-6 * n ** 0.5
    res = reference.compare(got.numpy(), ref.numpy(), rtol, atol)
    assert res["ok"], (op, n, res)


def _run(op, x, cuda, eps=0.0):
    import torch
    from emmyptx import runtime
    y = runtime.colwise(op, x.to(cuda), eps)
    torch.cuda.synchronize()
    return y.cpu()


def test_reference_cases(cuda):
    import torch
    from emmyptx import runtime
    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 64, generator=g)                                   # r_sum_dim0
    assert reference.compare(_run("sum", x, cuda).numpy(), x.double().sum(0).numpy(), 1e-4, 1e-4)["ok"]
    assert reference.compare(_run("softmax", x, cuda).numpy(), torch.softmax(x.double(), 0).numpy(), 1e-3, 1e-5)["ok"]   # f_softmax_dim0
    x = torch.randn(8, 32, 64, generator=g)                                 # r_sum_multi_dim: x.sum((0, 2))
    inner = runtime.rowwise("sum", x.to(cuda))                              # [8, 32]
    got = runtime.colwise("sum", inner).cpu()                               # [32]
    assert reference.compare(got.numpy(), x.double().sum((0, 2)).numpy(), 1e-4, 1e-4)["ok"]
    x = torch.randn(32, 256, generator=g)                                   # r_cumsum
    got = runtime.cumsum(x.to(cuda)).cpu()
    assert reference.compare(got.numpy(), reference.cumsum_reference(x).numpy(), 1e-4, 1e-4)["ok"]


@pytest.mark.parametrize("shape", [(1, 1), (7, 5), (256, 64), (1000, 130), (100000, 4), (5, 100000), (4096, 1024), (70001, 33),
                                   (3, 50, 20), (2, 3, 9000, 8)])
@pytest.mark.parametrize("op", OPS)
def test_shapes(op, shape, cuda):
    x = _data(op, shape, seed=len(shape) + shape[-1])
    eps = 1e-12 if op == "normalize" else 0.0
    got = _run(op, x, cuda, eps)
    ref = reference.colwise_reference(op, x, eps)
    assert got.shape == ref.shape
    _check(op, got, ref, shape[-2])


@pytest.mark.parametrize("op", ["sum", "var", "argmax", "softmax"])
def test_views_that_start_off_a_16_byte_boundary(op, cuda):
    import torch
    from emmyptx import runtime
    rows, cols = 3000, 36
    x = _data(op, (rows, cols), seed=3)
    flat = torch.zeros(rows * cols + 1, device=cuda)
    flat[1:] = x.reshape(-1).to(cuda)
    got = runtime.colwise(op, flat[1:].view(rows, cols)).cpu()
    _check(op, got, reference.colwise_reference(op, x), rows)


@pytest.mark.parametrize("rows", [9, 20000])
def test_nan_inf_and_ties(rows, cuda):
    import torch
    x = torch.randn(rows, 8, generator=torch.Generator().manual_seed(5))
    x[rows // 2, 1] = float("nan")
    x[3, 2] = float("inf")
    x[rows - 1, 3] = float("-inf")
    x[:, 4] = float("-inf")
    x[2, 5] = x[rows - 2, 5] = 9.0
    x[7, 6] = float("nan"); x[1, 6] = float("inf")
    x[:, 7] = 2.5
    for op in ("amax", "amin", "argmax", "logsumexp", "softmax", "log_softmax", "sum"):
        got = _run(op, x, cuda).numpy()
        want = reference.colwise_reference(op, x).numpy() if op != "argmax" else x.argmax(0).numpy()
        if op == "argmax":
            assert np.array_equal(got, want), op
        else:
            assert np.array_equal(np.isnan(got), np.isnan(want)), op
            assert np.allclose(got, want, rtol=1e-4, atol=1e-5, equal_nan=True), op


def test_sliced_result_does_not_depend_on_block_order(cuda):
    import torch
    from emmyptx import runtime
    x = torch.randn(1 << 20, 16, generator=torch.Generator().manual_seed(2)).to(cuda)
    for op in ("sum", "var", "logsumexp"):
        first = runtime.colwise(op, x).clone()
        for _ in range(5):
            assert torch.equal(runtime.colwise(op, x), first)


@pytest.mark.parametrize("cols", [1, 3, 4, 255, 256, 1000, 2048, 2052, 5000, 100000])
def test_cumsum(cols, cuda):
    import torch
    from emmyptx import runtime
    for rows in (1, 37):
        x = torch.randn(rows, cols, generator=torch.Generator().manual_seed(cols))
        got = runtime.cumsum(x.to(cuda)).cpu()
        res = reference.compare(got.numpy(), reference.cumsum_reference(x).numpy(), 1e-4, 1e-4 + 2e-6 * cols ** 0.5)
        assert res["ok"], (rows, cols, res)
    xd = x.to(cuda)
    expect = runtime.cumsum(xd).clone()
    runtime.cumsum(xd, out=xd)                                              # in place
    assert torch.equal(xd, expect)
    flat = torch.zeros(rows * cols + 1, device=cuda)                        # a view off the 16-byte grid
    flat[1:] = x.reshape(-1).to(cuda)
    off = runtime.cumsum(flat[1:].view(rows, cols)).cpu()                  # scalar accesses, other slab size: other rounding
    assert reference.compare(off.numpy(), reference.cumsum_reference(x).numpy(), 1e-4, 1e-4 + 2e-6 * cols ** 0.5)["ok"]


def test_cumsum_of_integers_is_exact(cuda):
    """Small integers sum exactly in fp32 whatever the order: the scan's bookkeeping (slab carries, lane offsets) is
    checked bit for bit on long rows."""
    import torch
    from emmyptx import runtime
    x = torch.randint(-3, 4, (5, 300001), generator=torch.Generator().manual_seed(1)).float()
    got = runtime.cumsum(x.to(cuda)).cpu()
    assert torch.equal(got, torch.cumsum(x.double(), -1).float())


def test_rejects_bad_arguments(cuda, lib):
    import torch
    x = torch.zeros(64, device=cuda)
    p = x.data_ptr()
    f = lib.emmyb200_colwise_f32
    assert f(18, p, p, 1, 8, 8, 0.0, None, 0, None) == -1                 # layer_norm is a row op only
    assert f(0, None, p, 1, 8, 8, 0.0, None, 0, None) == -1
    assert f(0, p, p, 1, 0, 8, 0.0, None, 0, None) == -2                  # nothing to reduce
    assert f(0, p, p, 0, 8, 8, 0.0, None, 0, None) == 0
    assert f(16, p, p, 1, 8, 8, 0.0, None, 0, None) == -1                 # softmax needs workspace for its statistics
    assert b"workspace" in lib.emmyb200_last_error()
    assert lib.emmyb200_colwise_workspace_bytes(0, 1, 8, 8) == 0
    assert lib.emmyb200_colwise_workspace_bytes(0, 1, 1 << 20, 8) > 0
    assert lib.emmyb200_colwise_workspace_bytes(18, 1, 8, 8) == -1
    g = lib.emmyb200_cumsum_f32
    assert g(None, p, 2, 4, None) == -1
    assert g(p, p, 0, 4, None) == 0
    assert g(p, p, -1, 4, None) == -1
