"""fp32 streaming transcendental kernels against the float64 oracle (C1 and the single ops).

Tolerance: each function within 2 ulp of the correctly rounded float64 value (the bound the
library documents; the reference's own class for these ops is rtol = atol = 1e-5,
tools/torch_cases/__init__.py:18, which is checked too). The composite exp + sin*tanh cancels
near x = -3.18, so it is held to 5 ulp of its largest term (2 + 2 from the factors and the sum's
own roundings) and to the reference's 1e-5 class.
"""
import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu


def _run(op, x_np, cuda):
    import torch
    from emmyptx import runtime
    x = torch.from_numpy(x_np).to(cuda)
    y = runtime.pointwise(op, x)
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("op", ["exp", "sin", "cos", "tanh"])
def test_unary_within_2ulp_uniform(op, cuda):
    x = inputs.c1_input(2**20)
    got = _run(op, x, cuda)
    ref = reference.UNARY_F64[op](x.astype(np.float64))
    assert reference.ulp_error(got, ref).max() <= 2.0
    assert reference.compare(got, ref, 1e-5, 1e-5)["ok"]


@pytest.mark.parametrize("op", ["exp", "sin", "cos", "tanh"])
def test_unary_within_2ulp_wide_range(op, cuda):
    """Every binade, both signs, plus zeros, infinities and NaN."""
    rng = np.random.default_rng(7)
    bits = rng.integers(0, 2**32, 2**21, dtype=np.uint64).astype(np.uint32)
    x = np.concatenate([bits.view(np.float32), np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 88.7, -103.9, 1e5, 65536.0,
                                                          -65537.0, 3.4e38], np.float32)])
    got = _run(op, x, cuda)
    with np.errstate(all="ignore"):
        ref = reference.UNARY_F64[op](x.astype(np.float64))
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)
    ref32 = ref.astype(np.float32)
    inf = np.isinf(ref32) & ~nan
    assert np.array_equal(got[inf], ref32[inf])
    fin = ~nan & ~inf
    assert reference.ulp_error(got[fin], ref[fin]).max() <= 2.0


def test_c1_composite(cuda):
    x = inputs.c1_input(2**20)
    got = _run("exp_sin_tanh", x, cuda)
    ref = reference.c1_f64(x)
    assert reference.compare(got, ref, 1e-5, 1e-5)["ok"]
    assert reference.c1_condition_ulp(got, x).max() <= 5.0
    # and no worse than torch's own fp32 evaluation, measured the same way
    import torch
    t32 = reference.c1_f32_torch(torch.from_numpy(x)).numpy()
    assert reference.c1_condition_ulp(got, x).max() <= reference.c1_condition_ulp(t32, x).max() + 3.0


@pytest.mark.parametrize("op", ["sigmoid", "silu", "relu"])
def test_activation_ops(op, cuda):
    """p_sigmoid, p_silu, p_relu (tools/torch_cases/pointwise.py:17-23) as streaming ops: the reference's class
    (rtol = atol = 1e-5), a few ulp on normal results, NaN and infinities as torch gives them, and the packed path
    (aligned buffer) bit-identical to the scalar one (a view 4 bytes into the allocation)."""
    import torch
    from emmyptx import runtime
    x = np.concatenate([inputs.c1_input(2**18) * 5, np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 87.0, -87.0, -100.0, 1e30], np.float32)])
    got = _run(op, x, cuda)
    with np.errstate(all="ignore"):
        ref = reference.UNARY_F64[op](x.astype(np.float64))
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    fin = np.isfinite(ref) & (np.abs(ref) > 1e-30)
    assert reference.compare(got[fin], ref[fin], 1e-5, 1e-5)["ok"]
    assert reference.ulp_error(got[fin], ref[fin]).max() <= 4.0
    xd = torch.from_numpy(np.concatenate([[0.0], x]).astype(np.float32)).to(cuda)
    shifted = torch.zeros_like(xd)
    runtime.pointwise(op, xd[1:], out=shifted[1:])
    torch.cuda.synchronize()
    assert np.array_equal(shifted[1:].cpu().numpy(), got, equal_nan=True)


def test_gelu_tanh(cuda):
    x = (np.random.default_rng(0).standard_normal(2**18) * 3).astype(np.float32)
    got = _run("gelu_tanh", x, cuda)
    ref = reference.UNARY_F64["gelu_tanh"](x.astype(np.float64))
    assert reference.compare(got, ref, 1e-5, 1e-5)["ok"]


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 1025, 2**16 + 7])
def test_ragged_sizes_and_unaligned_views(n, cuda):
    import torch
    from emmyptx import runtime
    x = inputs.c1_input(n + 1)
    ref = reference.c1_f64(x)
    got = _run("exp_sin_tanh", x[:n].copy(), cuda)
    assert got.shape == (n,)
    if n:
        assert reference.compare(got, ref[:n], 1e-5, 1e-5)["ok"]
        # a view that starts 4 bytes into the allocation takes the scalar kernel
        xd = torch.from_numpy(x).to(cuda)
        out = torch.zeros(n + 1, dtype=torch.float32, device=cuda)
        runtime.pointwise("exp_sin_tanh", xd[1:], out=out[1:])
        torch.cuda.synchronize()
        assert np.array_equal(out[1:].cpu().numpy(), _run("exp_sin_tanh", x[1:].copy(), cuda))
        assert out[0].item() == 0.0


def test_in_place(cuda):
    import torch
    from emmyptx import runtime
    x = inputs.c1_input(2**16)
    xd = torch.from_numpy(x).to(cuda)
    expect = runtime.pointwise("exp_sin_tanh", xd).clone()
    runtime.pointwise("exp_sin_tanh", xd, out=xd)
    torch.cuda.synchronize()
    assert torch.equal(xd, expect)


def test_rejects_bad_arguments(cuda, lib):
    import torch
    from emmyptx import runtime
    x = torch.zeros(8, dtype=torch.float32, device=cuda)
    assert lib.emmyb200_pointwise_f32(99, x.data_ptr(), x.data_ptr(), 8, None) == -1
    assert b"unknown op" in lib.emmyb200_last_error()
    assert lib.emmyb200_pointwise_f32(0, None, x.data_ptr(), 8, None) == -1
    with pytest.raises(RuntimeError):
        runtime.pointwise("exp", torch.zeros(8))          # a CPU tensor: there is no CPU path
