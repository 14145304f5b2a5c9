"""Every fp32 input through the shipped kernels, on the device: exp, sin, cos, tanh within 2 ulp of float64.

The streaming kernels pick between a packed straight-line path and the general scalar path per vector; this
test covers both by pushing all 2^32 bit patterns through `emmyb200_pointwise_f32` and comparing with torch's
float64 functions evaluated on the same device (the checker here is float64 arithmetic, not the CPU oracle: the
CPU oracle covers sampled inputs in test_gpu_pointwise.py and the host build of the same math is checked
exhaustively by oracle/ulp_exhaustive.cpp).
"""
import pytest

pytestmark = pytest.mark.gpu

CHUNK = 2**27
FLT_MAX = 3.4028234663852886e38


def _worst_ulp(op, ref_fn, cuda):
    import torch
    from emmyptx import runtime
    worst = torch.zeros((), dtype=torch.float64, device=cuda)
    bad = 0
    base = torch.arange(CHUNK, dtype=torch.int64, device=cuda)
    for start in range(0, 2**32, CHUNK):
        bits = (base + start).to(torch.int32) if start < 2**31 else (base + (start - 2**32)).to(torch.int32)
        x = bits.view(torch.float32)
        y = runtime.pointwise(op, x)
        x64 = x.double()
        ref = ref_fn(x64)
        nan = torch.isnan(ref)
        bad += int((torch.isnan(y) != nan).sum())
        over = ref.abs() > FLT_MAX                              # rounds to +-inf (or is inf)
        bad += int((over & ~nan & (y.double().abs() < FLT_MAX)).sum())
        bad += int((over & ~nan & (torch.sign(y.double()) != torch.sign(ref))).sum())
        ok = ~nan & ~over
        ref32 = ref.float()
        e = torch.frexp(ref32.abs()).exponent.to(torch.int64)
        ulp = torch.ldexp(torch.ones_like(ref), (e - 24).clamp(min=-149))
        err = torch.where(ok, (y.double() - ref).abs() / ulp, torch.zeros_like(ref))
        worst = torch.maximum(worst, err.max())
        del x64, ref, err, ulp, ref32
    return float(worst), bad


@pytest.mark.parametrize("op", ["exp", "tanh", "sin", "cos"])
def test_all_inputs_within_two_ulp(op, cuda):
    import torch
    worst, bad = _worst_ulp(op, getattr(torch, op), cuda)
    print(f"{op}: worst error over all 2^32 inputs = {worst:.4f} ulp")
    assert bad == 0
    assert worst <= 2.0


def test_fused_expression_over_its_whole_fast_range(cuda):
    """exp(x) + sin(x) * tanh(x) on every float with 2^-20 <= |x| <= 40 -- the range the fused form (exponentials from
    the special-function unit, tanh from e^{-2|x|}) serves -- against float64 on the same device: within 5 ulp of the
    largest term (the sum cancels near x = -3.18, so output-ulps say nothing there) and far inside the reference's
    class for this case, rtol = atol = 1e-5 (tools/torch_cases/pointwise.py:8-57)."""
    import torch
    from emmyptx import runtime
    lo = torch.tensor(2.0 ** -20, dtype=torch.float32).view(torch.int32).item()
    hi = torch.tensor(40.0, dtype=torch.float32).view(torch.int32).item()
    chunk = 2 ** 26
    worst, worst_class = 0.0, 0.0
    for sign in (0, -2 ** 31):
        for start in range(lo, hi + 1, chunk):
            n = min(chunk, hi + 1 - start)
            x = (torch.arange(n, dtype=torch.int64, device=cuda) + start + sign).to(torch.int32).view(torch.float32)
            y = runtime.pointwise("exp_sin_tanh", x).double()
            xd = x.double()
            e, st = torch.exp(xd), torch.sin(xd) * torch.tanh(xd)
            ref = e + st
            scale = torch.maximum(torch.maximum(e.abs(), st.abs()), ref.abs()).float()
            ulp = torch.ldexp(torch.ones_like(ref), (torch.frexp(scale).exponent.to(torch.int64) - 24).clamp(min=-149))
            worst = max(worst, float(((y - ref).abs() / ulp).max()))
            worst_class = max(worst_class, float(((y - ref).abs() / (1e-5 * ref.abs() + 1e-5)).max()))
    print(f"fused expression: worst {worst:.3f} ulp of the largest term; {worst_class:.4f} of the rtol = atol = 1e-5 class")
    assert worst <= 5.0
    assert worst_class <= 0.1

