"""float32 matmul (three-way bf16 split on the tensor cores) against float64: the reference's float32 matmul cases
(tools/torch_cases/matmul.py:10-16) at its MM class (rtol = atol = 1e-3), and at a float32-level bound that a plain
bf16 or tf32 product would miss by orders of magnitude:

    |c - ref| <= 1.5 * 2^-23 * (8 + K / 16) * (|a| . |b|)

The K / 16 term is the tensor core's accumulator, which truncates (rather than rounds) once per 16-deep product
block; measured on all-positive operands the error is about K / 16 * 2^-24 of the sum (cuBLAS's FMA chain: about
2^-20 whatever K), and with random signs 1e-7 .. 8e-7 of |a| . |b|.
"""
import numpy as np
import pytest

from oracle import reference

pytestmark = pytest.mark.gpu


def _rand(shape, seed):
    import torch
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def _check(got, a, b, bias=None, b_is_nk=False, post=None, reference_class=True):
    import torch
    a64, b64 = a.double(), b.double()
    if b_is_nk:
        b64 = b64.transpose(-1, -2)
    ref = a64 @ b64
    mag = a64.abs() @ b64.abs()
    if bias is not None:
        ref = ref + bias.double()
        mag = mag + bias.double().abs()
    err = (got.double() - (post(ref) if post else ref)).abs()
    bound = 1.5 * 2.0 ** -23 * (8 + a.shape[-1] / 16)
    worst = float((err / (bound * mag + 1e-30)).max())
    assert worst <= 1.0, f"worst error {worst:.2f}x the float32 bound"
    if reference_class:          # rtol = atol = 1e-3 against the result itself: only meaningful without heavy cancellation
        assert reference.compare(got.numpy(), (post(ref) if post else ref).numpy(), 1e-3, 1e-3)["ok"]


def test_reference_cases(cuda):
    import torch
    from emmyptx import runtime
    a, b = _rand((128, 96), 0), _rand((96, 80), 1)                            # m_mm, m_einsum
    _check(runtime.gemm_f32(a.to(cuda), b.to(cuda)).cpu(), a, b)
    a, b = _rand((4, 64, 32), 2), _rand((4, 32, 48), 3)                       # m_bmm
    _check(runtime.gemm_f32(a.to(cuda), b.to(cuda)).cpu(), a, b)
    b = _rand((32, 48), 4)                                                    # m_bcast_matmul
    _check(runtime.gemm_f32(a.to(cuda), b.to(cuda)).cpu(), a, b)
    x, w, bias = _rand((64, 128), 5), _rand((96, 128), 6), _rand((96,), 7)    # m_linear_bias
    _check(runtime.gemm_f32(x.to(cuda), w.to(cuda), bias=bias.to(cuda), b_is_nk=True).cpu(), x, w, bias, b_is_nk=True)
    x, w1 = _rand((32, 128), 8), _rand((256, 128), 9)                         # t_module_mlp's first layer with its activation
    got = runtime.gemm_f32(x.to(cuda), w1.to(cuda), b_is_nk=True, epilogue="relu").cpu()
    _check(got, x, w1, b_is_nk=True, post=lambda r: r.clamp_min(0))


@pytest.mark.parametrize("m,n,k", [(1, 4, 1), (5, 8, 3), (100, 72, 200), (129, 260, 65), (256, 256, 256), (300, 1000, 777), (1024, 132, 4096)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_shapes(m, n, k, b_is_nk, cuda):
    from emmyptx import runtime
    a = _rand((m, k), m + k)
    b = _rand((n, k) if b_is_nk else (k, n), n + k)
    _check(runtime.gemm_f32(a.to(cuda), b.to(cuda), b_is_nk=b_is_nk).cpu(), a, b, b_is_nk=b_is_nk)


def test_float32_accuracy_where_16_bit_products_fail(cuda):
    """Operands with 24 significant bits and a wide range of magnitudes: the result must carry float32 accuracy
    (a single bf16 product is wrong in the third digit, tf32 in the fourth)."""
    import torch
    from emmyptx import runtime
    g = torch.Generator().manual_seed(11)
    a = torch.randn(512, 2048, generator=g) * torch.exp2(torch.randint(-20, 20, (512, 2048), generator=g).float())
    b = torch.randn(2048, 384, generator=g) * torch.exp2(torch.randint(-20, 20, (2048, 384), generator=g).float())
    got = runtime.gemm_f32(a.to(cuda), b.to(cuda)).cpu()
    _check(got, a, b, reference_class=False)
    plain = (a.bfloat16().float() @ b.bfloat16().float())
    ref = a.double() @ b.double()
    mag = a.double().abs() @ b.double().abs()
    assert float(((plain.double() - ref).abs() / mag).max()) > 1e-3          # what one bf16 pass would have given
    assert float(((got.double() - ref).abs() / mag).max()) < 3e-5


def test_views_and_strides(cuda):
    """A and B may be any row-pitched views (the split reads them element-wise); C needs a pitch that is a multiple of 4."""
    import torch
    from emmyptx import runtime
    big_a, big_b = _rand((70, 203), 1).to(cuda), _rand((150, 97), 2).to(cuda)
    a, b = big_a[3:67, 5:135], big_b[10:140, 1:93]                               # 64 x 130 and 130 x 92, odd offsets and pitches
    out = torch.zeros(64, 100, device=cuda)
    runtime.gemm_f32(a, b, out=out[:, :92])
    torch.cuda.synchronize()
    _check(out[:, :92].cpu(), a.cpu(), b.cpu())
    assert float(out[:, 92:].abs().max()) == 0.0


def test_large_against_sampled_float64(cuda):
    import torch
    from emmyptx import runtime
    a = torch.randn(4096, 4096, device=cuda, generator=torch.Generator(device=cuda).manual_seed(0))
    b = torch.randn(4096, 4096, device=cuda, generator=torch.Generator(device=cuda).manual_seed(1))
    got = runtime.gemm_f32(a, b)
    rows = torch.arange(0, 4096, 97, device=cuda)
    ref = a[rows].double() @ b.double()
    mag = a[rows].double().abs() @ b.double().abs()
    assert float(((got[rows].double() - ref).abs() / mag).max()) < 4e-6
    assert runtime.device_status() == 0


def test_rejects_bad_arguments(cuda, lib):
    import torch
    x = torch.zeros(4096, device=cuda)
    p = x.data_ptr()
    f = lib.emmyb200_gemm_f32
    need = lib.emmyb200_gemm_f32_workspace_bytes(0, 1, 16, 16, 16, 1)
    assert need > 0 and need % 256 == 0
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    args = lambda **kw: [kw.get("epi", 0), kw.get("flags", 0), p, p, None, p, 1, 16, 16, kw.get("k", 16), 16, 16, kw.get("ldc", 16), 0, 0, 0,
                         kw.get("ws", ws.data_ptr()), kw.get("wsb", need), None]
    assert f(*args()) == 0
    assert f(*args(epi=9)) == -1
    assert f(*args(flags=4)) == -1
    assert f(*args(k=0)) == -2
    assert f(*args(ldc=18)) == -3                       # C pitch must be a multiple of 4 floats
    assert f(*args(ws=None)) == -1 and b"workspace" in lib.emmyb200_last_error()
    assert f(*args(wsb=need - 1)) == -1
    torch.cuda.synchronize()
