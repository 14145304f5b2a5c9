"""tcgen05 GEMM (C3, C4 and the ragged shapes of tools/torch_cases/matmul.py) against the oracle.

Tolerance (stated by the task for fp16/bf16 GEMMs): |c - ref| <= 1e-2 |ref| + 1e-2 std(ref) with
ref the fp32-accumulated product of the same rounded inputs. The reference's own classes for
tensor-core matmuls (rtol 2e-2 / atol 1e-1 for f16, 5e-2 / 5e-1 for bf16, matmul.py:5-7) are
looser and are implied.
"""
import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu


def _gemm(a, b, cuda, **kw):
    import torch
    from emmyptx import runtime
    c = runtime.gemm(a.to(cuda), b.to(cuda), **kw)
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    return c.cpu()


SHAPES = [
    (128, 256, 64), (128, 256, 256), (256, 512, 512), (512, 512, 512),          # m_f16_mm_staged / m_bf16_mm sizes
    (256, 256, 256),                                                             # m_f16_mm
    (100, 200, 72), (100, 72, 200),                                              # m_f16_mm_odd: ragged M, N, K
    (1, 8, 8), (129, 264, 8), (300, 1000, 136), (64, 512, 256),                  # tiny and tail-heavy
    (1024, 1024, 1024), (2048, 512, 1024),                                       # x14_matmul_2048-like
]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_gemm_matches_oracle(m, n, k, dtype, cuda):
    a, b = inputs.gemm_inputs(m, n, k, dtype)
    got = _gemm(a, b, cuda)
    ok, ratio = reference.gemm_tolerance_ok(got, reference.gemm_reference(a, b))
    assert ok, f"worst error {ratio:.2f}x the bound"
    assert got.abs().sum() > 0


@pytest.mark.parametrize("m,n,k", [(256, 512, 512), (100, 200, 72), (64, 512, 256), (1024, 1024, 1024)])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_gemm_b_stored_n_by_k(m, n, k, dtype, cuda):
    """F.linear's weight layout (m_f16_linear, matmul.py:32)."""
    a, b = inputs.gemm_inputs(m, n, k, dtype, b_is_nk=True)
    got = _gemm(a, b, cuda, b_is_nk=True)
    ok, ratio = reference.gemm_tolerance_ok(got, reference.gemm_reference(a, b, b_is_nk=True))
    assert ok, f"worst error {ratio:.2f}x the bound"


@pytest.mark.parametrize("m,n,k", [(256, 512, 512), (100, 200, 72), (1024, 2048, 1024)])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_gemm_gelu_epilogue(m, n, k, dtype, cuda):
    import torch
    a, b = inputs.gemm_inputs(m, n, k, dtype)
    a = a * 8                                  # spread the pre-activation over GELU's curved part
    got = _gemm(a, b, cuda, epilogue="gelu_tanh")
    ok, ratio = reference.gemm_tolerance_ok(got, reference.gemm_reference(a, b, "gelu_tanh"))
    assert ok, f"worst error {ratio:.2f}x the bound"


def test_gemm_unnormalised_randn_reference_tolerance(cuda):
    """The reference's own case m_f16_mm_staged: randn inputs, rtol 2e-2 / atol 1e-1 vs float64."""
    import torch
    a = torch.from_numpy(np.random.default_rng(0).standard_normal((512, 512)).astype(np.float16))
    b = torch.from_numpy(np.random.default_rng(1).standard_normal((512, 512)).astype(np.float16))
    got = _gemm(a, b, cuda)
    ref = reference.gemm_reference(a, b, double=True)
    assert reference.compare(got.float().numpy(), ref.numpy(), 2e-2, 1e-1)["ok"]


def test_c3_full_size(cuda):
    a, b = inputs.gemm_inputs(4096, 4096, 4096, "f16")
    got = _gemm(a, b, cuda)
    ok, ratio = reference.gemm_tolerance_ok(got, reference.gemm_reference(a, b))
    assert ok, f"worst error {ratio:.2f}x the bound"


def test_c4_full_size_sampled_rows(cuda):
    """Configuration 4 at its own size: M = N = K = 16384, bf16, tanh-GELU fused into the store. The GPU computes the
    whole product; the oracle checks a seeded sample of 256 whole rows plus the rows at the edges of 128-row output
    tiles, of the 16-row-block bands the tile order walks, and of the matrix (fp32 product of the same rounded
    operands, GELU on the fp32 value, one rounding to bf16 by the kernel only; comparison and vacuity check as
    tools/check_torch.py:260-278 with the task's rule |c - ref| <= 1e-2 |ref| + 1e-2 std(ref))."""
    import torch
    from emmyptx import runtime
    s = 16384
    a, b = inputs.gemm_inputs(s, s, s, "bf16")
    c = runtime.gemm(a.to(cuda), b.to(cuda), epilogue="gelu_tanh")
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    edges = [0, 1, 127, 128, 129, 2047, 2048, 8191, 8192, 16255, 16256, s - 2, s - 1]
    rows = sorted(set(edges) | set(np.random.default_rng(4).integers(0, s, 256).tolist()))
    ref = reference.gemm_reference(a[rows], b, "gelu_tanh")
    got = c[rows].cpu()
    ok, ratio = reference.gemm_tolerance_ok(got, ref)
    assert ok, f"worst error {ratio:.2f}x the bound"
    assert not reference.compare(got.float().numpy(), ref.numpy(), 1e-2, 1e-2 * float(ref.std()))["vacuous"]
    # every column block of every sampled row was written (no tile skipped): no element kept the fill value
    fill = torch.full((8, s), float("nan"), dtype=torch.bfloat16, device=cuda)
    runtime.gemm(a[:8].to(cuda), b.to(cuda), epilogue="gelu_tanh", out=fill)
    assert not torch.isnan(fill).any()
    # size-independent property: the rows of a row-permuted A give the permuted rows of C bit for bit
    perm = torch.from_numpy(np.random.default_rng(6).permutation(s)[:1024])
    sub = runtime.gemm(a[perm].to(cuda).contiguous(), b.to(cuda), epilogue="gelu_tanh")
    assert torch.equal(sub, c[perm.to(cuda)])


def test_linearity_at_size(cuda):
    """Size-independent property at a large size: (2A) B = 2 (A B) exactly (scaling by 2 is exact
    in bf16, whose exponent range keeps these outputs normal), and rows of a row-permuted A give
    the permuted rows of C bit for bit."""
    import torch
    a, b = inputs.gemm_inputs(4096, 2048, 2048, "bf16")
    c1 = _gemm(a, b, cuda)
    c2 = _gemm(a * 2, b, cuda)
    assert torch.equal(c1 * 2, c2)
    perm = torch.from_numpy(np.random.default_rng(5).permutation(4096))
    assert torch.equal(_gemm(a[perm].contiguous(), b, cuda), c1[perm])


def test_leading_dimensions(cuda):
    """Row pitches larger than the rows (views into wider allocations)."""
    import torch
    from emmyptx import runtime
    a, b = inputs.gemm_inputs(200, 136, 264, "bf16")
    A = torch.zeros(200, 512, dtype=torch.bfloat16, device=cuda); A[:, :264] = a.to(cuda)
    B = torch.zeros(264, 256, dtype=torch.bfloat16, device=cuda); B[:, :136] = b.to(cuda)
    C = torch.full((200, 144), 7.0, dtype=torch.bfloat16, device=cuda)
    runtime.check(runtime.library().emmyb200_gemm(runtime.BF16, 0, 0, A.data_ptr(), B.data_ptr(), C.data_ptr(), 200, 136, 264,
                                                  512, 256, 144, None))
    torch.cuda.synchronize()
    ok, ratio = reference.gemm_tolerance_ok(C[:, :136].cpu(), reference.gemm_reference(a, b))
    assert ok, ratio
    assert torch.all(C[:, 136:] == 7.0)        # nothing written past N


def test_rejects_bad_arguments(cuda, lib):
    import torch
    x = torch.zeros(64 * 64, dtype=torch.float16, device=cuda)
    p = x.data_ptr()
    g = lib.emmyb200_gemm
    assert g(0, 0, 0, p, p, p, 64, 64, 64, 64, 64, 64, None) == -4          # f32 operands
    assert g(1, 7, 0, p, p, p, 64, 64, 64, 64, 64, 64, None) == -1          # epilogue
    assert g(1, 0, 0, p, p, p, 64, 64, 64, 60, 64, 64, None) == -2          # lda < K
    assert g(1, 0, 0, p, p, p, 60, 60, 60, 60, 60, 60, None) == -3          # pitches not multiples of 8
    assert g(1, 0, 0, p + 2, p, p, 64, 64, 64, 64, 64, 64, None) == -3      # misaligned pointer
    assert g(1, 0, 0, p, p, p, 0, 64, 64, 64, 64, 64, None) == 0            # empty
    assert g(1, 0, 0, p, p, p, 64, 64, 0, 64, 64, 64, None) == -2           # K = 0


@pytest.mark.parametrize("batch,m,n,k,shared", [(4, 128, 96, 64, False),      # m_f16_bmm (matmul.py:31)
                                                 (4, 64, 48, 32, True),        # m_bcast_matmul's shape, 16-bit
                                                 (3, 100, 72, 200, False), (5, 300, 264, 136, True)])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_batched_and_broadcast(batch, m, n, k, shared, dtype, cuda):
    import torch
    from emmyptx import runtime
    td = torch.float16 if dtype == "f16" else torch.bfloat16
    a = torch.from_numpy(np.random.default_rng(0).standard_normal((batch, m, k)).astype(np.float32) / k**0.5).to(td)
    b = torch.from_numpy(np.random.default_rng(1).standard_normal((k, n) if shared else (batch, k, n)).astype(np.float32) / k**0.5).to(td)
    got = runtime.gemm_batched(a.to(cuda), b.to(cuda)).cpu()
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    ref = torch.matmul(a.float(), b.float())
    ok, ratio = reference.gemm_tolerance_ok(got, ref)
    assert ok, f"worst error {ratio:.2f}x the bound"


@pytest.mark.parametrize("epilogue", [None, "relu", "gelu_tanh"])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_bias_and_relu_epilogue(epilogue, dtype, cuda):
    """F.linear(x, w, b) with the weight stored N x K (m_linear_bias / m_f16_linear shapes), bias added to the fp32
    accumulator, then the activation, one rounding."""
    import torch
    from emmyptx import runtime
    td = torch.float16 if dtype == "f16" else torch.bfloat16
    m, n, k = 64, 520, 256
    x = torch.from_numpy(np.random.default_rng(0).standard_normal((1, m, k)).astype(np.float32)).to(td)
    w = torch.from_numpy(np.random.default_rng(1).standard_normal((n, k)).astype(np.float32) / k**0.5).to(td)
    bias = torch.from_numpy(np.random.default_rng(2).standard_normal(n).astype(np.float32)).to(td)
    got = runtime.gemm_batched(x.to(cuda), w.to(cuda), bias=bias.to(cuda), epilogue=epilogue, b_is_nk=True).cpu()[0]
    ref = x[0].float() @ w.float().t() + bias.float()
    if epilogue == "relu":
        ref = torch.relu(ref)
    elif epilogue == "gelu_tanh":
        ref = torch.nn.functional.gelu(ref, approximate="tanh")
    ok, ratio = reference.gemm_tolerance_ok(got, ref)
    assert ok, f"worst error {ratio:.2f}x the bound"
    if epilogue == "relu":
        assert (got >= 0).all()


def test_host_buffer_call_overlaps_copies_and_matches_the_device_call(cuda):
    """runtime.HostGemm: pinned host A, B in, C out, in row chunks on three streams; same bits as one device call."""
    import torch
    from emmyptx import runtime
    m, n, k = 1024, 384, 256
    a, b = inputs.gemm_inputs(m, n, k, "bf16")
    a_h, b_h = a.pin_memory(), b.pin_memory()
    c_h = torch.zeros(m, n, dtype=torch.bfloat16).pin_memory()
    call = runtime.HostGemm(m, n, k, torch.bfloat16, cuda, epilogue="gelu_tanh", chunks=4)
    assert call.chunks == 4 and call.rows == 256
    for _ in range(2):                                   # twice: the second call must wait for the first one's buffers
        call(a_h, b_h, c_h)
    torch.cuda.synchronize()
    expect = runtime.gemm(a.to(cuda), b.to(cuda), epilogue="gelu_tanh").cpu()
    assert torch.equal(c_h, expect)
    # back-to-back calls on different host buffers: the second call's copy-in overlaps the first one's copy-back
    a2, b2 = (x.flip(0).contiguous().pin_memory() for x in (a, b))
    c2 = torch.zeros(m, n, dtype=torch.bfloat16).pin_memory()
    for overlap in (True, False):
        call = runtime.HostGemm(m, n, k, torch.bfloat16, cuda, epilogue="gelu_tanh", chunks=4, overlap_calls=overlap)
        c_h.zero_(), c2.zero_()
        call(a_h, b_h, c_h)
        call(a2, b2, c2)
        call(a_h, b_h, c_h)
        torch.cuda.synchronize()
        assert torch.equal(c_h, expect)
        assert torch.equal(c2, runtime.gemm(a2.to(cuda), b2.to(cuda), epilogue="gelu_tanh").cpu())
    assert runtime.HostGemm(300, 64, 64, torch.bfloat16, cuda, chunks=8).chunks == 1     # no whole-block split: one chunk


# ---- fp32 output: the accumulator stored without narrowing (and what a split-K schedule adds up to) -----------------
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 512), (100, 200, 72), (100, 72, 200), (1, 8, 8), (300, 1000, 136), (1024, 1024, 1024)])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_f32_output(m, n, k, dtype, b_is_nk, cuda):
    """emmyptx/mma.py:205-242 stores an accumulator fragment to an f32 buffer as it is, or adds it with red.add.f32. The
    result is the fp32-accumulated product of the 16-bit operands, unrounded: the bound is that of fp32 accumulation
    (a few 2^-24 of sum |a b|), far inside the task's 16-bit tolerance."""
    import torch
    a, b = inputs.gemm_inputs(m, n, k, dtype, b_is_nk=b_is_nk)
    got = _gemm(a, b, cuda, b_is_nk=b_is_nk, out_f32=True)
    assert got.dtype == torch.float32
    bb = b.double().t() if b_is_nk else b.double()
    ref = a.double() @ bb
    scale = a.double().abs() @ bb.abs()
    assert float(((got.double() - ref).abs() / (scale * 2.0 ** -21 + 1e-30)).max()) <= 1.0
    # the 16-bit output of the same product is this value rounded once
    narrow = _gemm(a, b, cuda, b_is_nk=b_is_nk)
    assert torch.equal(narrow, got.to(narrow.dtype))


def test_f32_output_batched_with_f32_bias_and_epilogues(cuda):
    import torch
    from emmyptx import runtime
    rng = np.random.default_rng(4)
    a = torch.from_numpy(rng.standard_normal((3, 100, 136)).astype(np.float32) / 12).to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((3, 136, 264)).astype(np.float32) / 12).to(torch.bfloat16)
    bias = torch.from_numpy(rng.standard_normal(264).astype(np.float32))
    for epilogue in (None, "relu", "gelu_tanh"):
        got = runtime.gemm_batched(a.to(cuda), b.to(cuda), bias=bias.to(cuda), epilogue=epilogue, out_f32=True).cpu()
        assert got.dtype == torch.float32 and runtime.device_status() == 0
        ref = torch.matmul(a.double(), b.double()) + bias.double()
        ref = torch.relu(ref) if epilogue == "relu" else (torch.nn.functional.gelu(ref, approximate="tanh") if epilogue else ref)
        tol = 2e-3 if epilogue == "gelu_tanh" else 1e-5            # the fused GELU uses the hardware exponential
        assert torch.allclose(got.double(), ref, rtol=tol, atol=tol), (epilogue, float((got.double() - ref).abs().max()))
    with pytest.raises(ValueError, match="output's dtype"):
        runtime.gemm_batched(a.to(cuda), b.to(cuda), bias=bias.to(torch.bfloat16).to(cuda), out_f32=True)


def test_f32_output_argument_checks(cuda, lib):
    import torch
    x = torch.zeros(256 * 256, dtype=torch.float32, device=cuda)
    p = x.data_ptr()
    assert lib.emmyb200_gemm(1, 0, 4, p, p, p, 64, 64, 64, 64, 64, 64, None) == 0
    assert lib.emmyb200_gemm(1, 0, 4, p, p, p, 64, 62, 64, 64, 64, 62, None) == -3          # ldc must be a multiple of 4 fp32 elements
    assert lib.emmyb200_gemm(1, 0, 4, p, p, p, 64, 60, 64, 64, 60, 60, None) == -3          # ldb (16-bit) must still be a multiple of 8
    assert lib.emmyb200_gemm(1, 0, 4, p, p, p, 64, 60, 64, 64, 64, 60, None) == 0           # ldc = 60 fp32 elements is 16-byte aligned
    assert lib.emmyb200_gemm(1, 0, 4 | 2, p, p, p, 64, 64, 64, 64, 64, 64, None) < 0        # no multicast destination in fp32
    torch.cuda.synchronize()

