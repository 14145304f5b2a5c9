"""Attention forward (C5 and the shapes of the reference's f_sdpa / f_sdpa_f16 / x16_attn_512 cases)
against the fp32 oracle.

Tolerance: |o - ref| <= 1e-2 |ref| + 1e-2 std(ref), ref = fp32 softmax(QK^T/sqrt(d))V of the same rounded
inputs (the reference's class for attention is MM, rtol = atol = 1e-3 on fp32 buffers, and HALF 1e-2 for
16-bit ones: tools/torch_cases/__init__.py:20-21, fused.py:21-28).
"""
import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu


FORMS = ["one_tile", "two_tiles"]     # both kernel forms, forced; the default choice is exercised by the other tests


def _attn(q, k, v, cuda, **kw):
    import torch
    from emmyptx import runtime
    o = runtime.attention(q.to(cuda), k.to(cuda), v.to(cuda), **kw)
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    return o.cpu()


@pytest.mark.parametrize("units,sq,sk,d", [
    (2, 128, 128, 128), (3, 256, 384, 128), (2, 512, 512, 128),       # x16_attn_512-like
    (2, 100, 200, 128), (1, 1, 1, 128), (2, 129, 257, 128), (1, 300, 77, 128),   # ragged
    (4, 256, 256, 64), (2, 130, 190, 64),                              # f_sdpa_f16 head size
    (1, 2048, 2048, 128),
])
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("form", FORMS)
def test_attention_matches_oracle(units, sq, sk, d, dtype, form, cuda):
    q, k, v = inputs.attention_inputs(units, sq, sk, d, dtype)
    got = _attn(q, k, v, cuda, form=form)
    ref = reference.attention_reference(q, k, v)
    ok, ratio = reference.gemm_tolerance_ok(got, ref)
    assert ok, f"worst error {ratio:.2f}x the bound"


@pytest.mark.parametrize("form", FORMS)
def test_large_logits_and_scale(form, cuda):
    """Scores spread over hundreds of log2 units: the running max must be raised (and the accumulator
    rescaled) many times; in the two-tile form, whose exponentials are taken against the maximum of the earlier
    tiles, the jump at key 512 also takes the overflow guard (reference raised, tile done again)."""
    import torch
    q, k, v = inputs.attention_inputs(2, 256, 1024, 128, "bf16")
    k = k.clone()
    k[:, 512:] *= 3                       # later keys dominate
    got = _attn(q * 2, k, v, cuda, scale=1.0, form=form)
    ref = reference.attention_reference(q * 2, k, v, scale=1.0)
    ok, ratio = reference.gemm_tolerance_ok(got, ref)
    assert ok, f"worst error {ratio:.2f}x the bound"


@pytest.mark.parametrize("form", FORMS)
def test_c5_sampled_units(form, cuda):
    """Full sequence length of C5 (4096) on a few (batch, head) units; every unit is independent."""
    q, k, v = inputs.attention_inputs(3, 4096, 4096, 128, "bf16")
    got = _attn(q, k, v, cuda, form=form)
    ref = reference.attention_reference(q, k, v)
    ok, ratio = reference.gemm_tolerance_ok(got, ref)
    assert ok, f"worst error {ratio:.2f}x the bound"


def test_c5_full_size_sampled_rows(cuda):
    """Configuration 5 at its own size: 256 (batch, head) units of 4096 x 128, bf16. The GPU computes all of O; the
    oracle checks seeded query rows (tile edges included) of a seeded sample of units spread over the whole grid,
    fp32 softmax(q k^T / sqrt(d)) v of the same rounded operands."""
    import torch
    from emmyptx import runtime
    units, s, d = 256, 4096, 128
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(units, s, d, generator=g).to(torch.bfloat16) for _ in range(3))
    o = runtime.attention(q.to(cuda), k.to(cuda), v.to(cuda))
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    worst = 0.0
    for u in sorted({0, 1, 147, 148, 255} | set(np.random.default_rng(12).integers(0, units, 7).tolist())):
        rows = sorted({0, 127, 128, 255, 256, s - 129, s - 128, s - 1} | set(np.random.default_rng(u).integers(0, s, 56).tolist()))
        ref = reference.attention_reference(q[u][rows], k[u], v[u])
        ok, ratio = reference.gemm_tolerance_ok(o[u][rows].cpu(), ref)
        worst = max(worst, ratio)
    assert worst <= 1.0, f"worst error {worst:.2f}x the bound"


def test_rows_sum_property(cuda):
    """Size-independent property: with V = all ones every output element is exactly 1 up to rounding
    (softmax rows sum to 1), and permuting the keys together with the values leaves O unchanged up to
    summation order."""
    import torch
    q, k, v = inputs.attention_inputs(2, 512, 1024, 128, "bf16")
    ones = torch.ones_like(v)
    got = _attn(q, k, ones, cuda)
    assert (got.float() - 1).abs().max() <= 2 ** -7
    perm = torch.from_numpy(np.random.default_rng(9).permutation(1024))
    a = _attn(q, k, v, cuda)
    b = _attn(q, k[:, perm].contiguous(), v[:, perm].contiguous(), cuda)
    assert (a.float() - b.float()).abs().max() <= 1e-2 * a.float().std() + 1e-2 * a.float().abs().max()


@pytest.mark.parametrize("units,s,d", [(2, 256, 128), (3, 300, 128), (2, 64, 32 * 2), (1, 1000, 128), (2, 129, 64),
                                       (80, 512, 64),      # more pairs of tiles than SMs: a second, partial round of the deal
                                       (60, 768, 128)])    # 180 pairs of three lengths
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("form", FORMS)
def test_causal(units, s, d, dtype, form, cuda):
    """t_causal_sdpa / f_masked_attn_manual (tools/torch_cases/models.py:17-19, fused.py:31-36): lower-triangular mask.

    The absolute floor of the bound is taken per query row (1e-2 of the row's rms) rather than over the whole
    output: early rows average a handful of values and are O(1) while late rows average thousands and are small,
    so one global std would hold the early rows' 16-bit probabilities to a tighter class than 1e-2."""
    import torch
    q, k, v = inputs.attention_inputs(units, s, s, d, dtype)
    got = _attn(q, k, v, cuda, causal=True, form=form)
    scores = torch.matmul(q.double(), k.double().transpose(-1, -2)) * d ** -0.5
    mask = torch.ones(s, s, dtype=torch.bool).tril()
    ref = torch.matmul(torch.softmax(scores.masked_fill(~mask, float("-inf")), -1), v.double())
    bound = 1e-2 * ref.abs() + 1e-2 * ref.pow(2).mean(-1, keepdim=True).sqrt()
    ratio = float(((got.double() - ref).abs() / bound).max())
    assert ratio <= 1.0, f"worst error {ratio:.2f}x the bound"
    assert torch.equal(got[:, 0].float(), v[:, 0].float())        # the first query sees one key: O = V[0] exactly


@pytest.mark.parametrize("form", FORMS)
def test_causal_skips_tiles_past_the_diagonal(form, cuda):
    """Keys after the query must not influence the result at all: poisoning them with NaN changes nothing."""
    import torch
    q, k, v = inputs.attention_inputs(2, 384, 384, 128, "bf16")
    a = _attn(q, k, v, cuda, causal=True, form=form)
    k2, v2 = k.clone(), v.clone()
    k2[:, 256:] = float("nan")
    v2[:, 256:] = float("nan")
    b = _attn(q, k2, v2, cuda, causal=True, form=form)
    assert torch.equal(a[:, :256], b[:, :256])


def test_rejects_bad_arguments(cuda, lib):
    import torch
    x = torch.zeros(2 * 128 * 128, dtype=torch.bfloat16, device=cuda)
    p = x.data_ptr()
    f = lib.emmyb200_attention_fwd
    assert f(2, 0, p, p, p, p, 2, 128, 128, 80, 0.1, None) == -4      # head dim: multiples of 32 up to 128
    assert f(2, 0, p, p, p, p, 2, 128, 128, 160, 0.1, None) == -4
    assert f(3, 0, p, p, p, p, 2, 128, 128, 128, 0.1, None) == -4     # an integer dtype
    assert f(0, 4, p, p, p, p, 2, 128, 128, 128, 0.1, None) == -4     # f32 has one kernel form
    assert f(2, 8, p, p, p, p, 2, 128, 128, 32, 0.1, None) == -4      # and so has a head size off the tensor-core kernels
    assert f(2, 0, p, p, p, p, 2, 128, 0, 128, 0.1, None) == -2       # no keys
    assert f(2, 0, p, p, p, p, 0, 128, 128, 128, 0.1, None) == 0      # no units
    assert f(2, 16, p, p, p, p, 2, 128, 128, 128, 0.1, None) == -1    # unknown flag
    assert f(2, 12, p, p, p, p, 2, 128, 128, 128, 0.1, None) == -1    # both form flags
    assert f(2, 0, None, p, p, p, 2, 128, 128, 128, 0.1, None) == -1


# ---- fp32 buffers, and head sizes the tensor-core kernels do not take: the CUDA-core kernel ------------------------
def _attn_ref64(q, k, v, scale, causal):
    import torch
    s = torch.matmul(q.double(), k.double().transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(q.shape[-2], k.shape[-2], dtype=torch.bool).tril(), float("-inf"))
    return torch.matmul(torch.softmax(s, -1), v.double())


@pytest.mark.parametrize("units,sq,sk,d,causal,scale", [
    (2, 64, 64, 32, False, None),            # f_sdpa: q, k, v = randn(1, 2, 64, 32)            (tools/torch_cases/fused.py:21-22)
    (4, 128, 128, 64, True, None),           # t_causal_sdpa: randn(1, 4, 128, 64), is_causal   (models.py:17-19)
    (1, 64, 64, 32, True, 0.17677669),       # f_masked_attn_manual: mask above the diagonal   (fused.py:31-36)
    (3, 77, 130, 96, False, None), (2, 33, 200, 128, False, 0.3), (2, 200, 200, 128, True, None), (1, 1, 1, 32, False, None),
    (5, 300, 45, 64, False, None),
])
def test_f32_attention_in_fp32_arithmetic(units, sq, sk, d, causal, scale, cuda):
    """The reference's own attention cases are fp32 with d = 32 or 64; its tolerance class for them is MM (rtol = atol
    = 1e-3). The kernel keeps every product in fp32, so the bound here is two orders tighter."""
    import torch
    g = torch.Generator().manual_seed(units * 1000 + sq)
    q = torch.randn(units, sq, d, generator=g)
    k, v = torch.randn(units, sk, d, generator=g), torch.randn(units, sk, d, generator=g)
    sc = d ** -0.5 if scale is None else scale
    got = _attn(q, k, v, cuda, causal=causal, scale=sc)
    assert got.dtype == torch.float32
    ref = _attn_ref64(q, k, v, sc, causal)
    assert torch.allclose(got.double(), ref, rtol=1e-5, atol=1e-5), float((got.double() - ref).abs().max())
    if causal:
        assert torch.allclose(got[:, 0], v[:, 0], rtol=1e-6, atol=0)          # the first query sees one key


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("units,sq,sk,d,causal", [(2, 100, 100, 32, False), (3, 130, 130, 96, True), (1, 64, 257, 32, False)])
def test_16_bit_attention_with_other_head_sizes(units, sq, sk, d, causal, dtype, cuda):
    q, k, v = inputs.attention_inputs(units, sq, sk, d, dtype)
    got = _attn(q, k, v, cuda, causal=causal)
    ref = _attn_ref64(q, k, v, d ** -0.5, causal)
    bound = 1e-2 * ref.abs() + 1e-2 * ref.pow(2).mean(-1, keepdim=True).sqrt()
    assert float(((got.double() - ref).abs() / bound).max()) <= 1.0


def test_f32_attention_large_scores(cuda):
    """Scores hundreds of log2 units apart: the running maximum is raised many times and nothing overflows. Scores of
    magnitude 1000 carry an absolute fp32 error of 1e-3, which is the relative error of a probability: the bound is
    that of the arithmetic, not of the kernel."""
    import torch
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(2, 96, 64, generator=g) * 4, torch.randn(2, 500, 64, generator=g) * 4, torch.randn(2, 500, 64, generator=g)
    k[:, 250:] *= 3
    got = _attn(q, k, v, cuda, scale=1.0)
    ref = _attn_ref64(q, k, v, 1.0, False)
    assert torch.isfinite(got).all() and torch.allclose(got.double(), ref, rtol=5e-3, atol=5e-3), float((got.double() - ref).abs().max())


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("causal", [False, True])
def test_every_output_tile_goes_to_every_destination(form, causal, cuda):
    """The store path of the sharded configuration on one GPU: two destinations, both local buffers. Each must hold exactly
    what the single-destination call writes, in both kernel forms (the multicast form of the same path needs a second GPU
    and is covered by the two-GPU tests)."""
    import torch
    from emmyptx import runtime
    q, k, v = (t.to(cuda) for t in inputs.attention_inputs(3, 700, 900 if not causal else 700, 128, "bf16"))
    plain = runtime.attention(q, k, v, causal=causal, form=form)
    o1, o2 = torch.zeros_like(q), torch.zeros_like(q)
    runtime.attention_allgather(q, k, v, [o1.data_ptr(), o2.data_ptr()], causal=causal, form=form)
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    assert torch.equal(o1, plain) and torch.equal(o2, plain)

