"""The oracle pinned against the reference's own output (CPU only).

tests/golden/golden.npz holds what the reference's PTX computes for the streaming configurations and for its
tensor-core matmul cases (its own compiler's output, executed by oracle/ptx_interp.py; make_golden.py). The float64
oracle must agree with it within the reference's tolerance class for transcendental ops (rtol = atol = 1e-5,
tools/torch_cases/__init__.py:18) and for 16-bit matmuls (tools/torch_cases/matmul.py:7); the integer oracle, in
its truncating mode, bit for bit.
"""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import inputs, ptx_interp, reference

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "golden.npz")


@pytest.mark.parametrize("case,op", [("c1_exp_sin_tanh_n4096", "exp_sin_tanh"), ("p_exp_n4096", "exp"),
                                     ("p_tanh_n4096", "tanh"), ("p_sin_n4096", "sin")])
def test_float_oracle_agrees_with_reference_output(golden, case, op):
    x = inputs.c1_input(4096)
    ref = reference.UNARY_F64[op](x.astype(np.float64))
    res = reference.compare(golden[f"{case}.y"], ref, 1e-5, 1e-5)
    assert res["ok"], res


def test_c1_at_full_size(golden):
    x = inputs.c1_input(2**20)
    keep = golden["c1_exp_sin_tanh_n1048576.index"]
    assert reference.compare(golden["c1_exp_sin_tanh_n1048576.y"], reference.c1_f64(x)[keep], 1e-5, 1e-5)["ok"]


def test_integer_oracle_matches_reference_output_bit_for_bit(golden):
    x = inputs.c2_input(2**16)
    assert np.array_equal(golden["c2_gather_n65536.y"], reference.c2_reference(x, trunc=True))
    x = inputs.c2_input(2**20)
    keep = golden["c2_gather_n1048576.index"]
    assert np.array_equal(golden["c2_gather_n1048576.y"], reference.c2_reference(x, trunc=True)[keep])


def test_reference_truncates_where_torch_floors(golden):
    """The documented divergence (tools/torch_cases/dtypes.py:17-19): the floor-mode oracle (torch's //) differs
    from the reference's PTX exactly where the gathered value is negative and not a multiple of 3."""
    x = inputs.c2_input(2**16)
    floor, trunc = reference.c2_reference(x), golden["c2_gather_n65536.y"]
    i = np.arange(2**16, dtype=np.int64)
    g = x[(i * 7919 + 13) % 2**16].astype(np.int64)
    assert np.array_equal(floor != trunc, (g < 0) & (g % 3 != 0))
    assert np.array_equal(reference.c2_torch(__import__("torch").from_numpy(x)).numpy(), floor)


def test_interpreter_runs_the_committed_ptx():
    """The fixture is reproducible from the committed PTX text."""
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())["c2_gather_n65536"]
    x = inputs.c2_input(2**16)
    y = np.zeros_like(x)
    ptx_interp.run_entry((GOLDEN / "c2_gather_n65536.ref.ptx").read_text(), {"x": x, "y": y}, info["launch"]["grid"][0],
                         info["launch"]["block"][0])
    assert np.array_equal(y, np.load(GOLDEN / "golden.npz")["c2_gather_n65536.y"])


def test_bf16_rounding_matches_torch():
    """Round-to-nearest-even of the fp32 bits (tools/run_local.py:31-37) is what torch's .bfloat16() does."""
    import torch
    v = np.random.default_rng(0).standard_normal(10000).astype(np.float32)
    bits = inputs.to_bf16_bits(v)
    assert np.array_equal(bits, torch.from_numpy(v).bfloat16().view(torch.uint16).numpy())
    assert np.array_equal(inputs.from_bf16_bits(bits), torch.from_numpy(v).bfloat16().float().numpy())


def test_condition_aware_ulp_metric_on_torch_fp32():
    """torch's own fp32 evaluation of C1 is thousands of raw output-ulps off where the sum cancels, and about 2
    when measured at the largest term: the metric the GPU test uses is meaningful."""
    import torch
    x = inputs.c1_input(2**20)
    t32 = reference.c1_f32_torch(torch.from_numpy(x)).numpy()
    assert reference.ulp_error(t32, reference.c1_f64(x)).max() > 100
    assert reference.c1_condition_ulp(t32, x).max() < 3.0


HALF_MM, BF16_MM = dict(rtol=2e-2, atol=1e-1), dict(rtol=5e-2, atol=5e-1)      # tools/torch_cases/matmul.py:7


def _golden_gemm(golden, case):
    import torch
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]["gemm"]
    a, b = inputs.gemm_inputs(info["m"], info["n"], info["k"], info["dtype"], info["b_trans"], scaled=False,
                              batch=tuple(info["batch"]))
    bb = b.double().transpose(-1, -2) if info["b_trans"] else b.double()
    ref = (a.double() @ bb).reshape(-1, info["n"]).numpy()
    td = torch.float16 if info["dtype"] == "f16" else torch.bfloat16
    got = torch.from_numpy(golden[f"{case}.c"].view(np.int16)).view(td).double().numpy()
    if f"{case}.rows" in golden.files:
        ref = ref[golden[f"{case}.rows"]]
    return got, ref, (HALF_MM if info["dtype"] == "f16" else BF16_MM), td


@pytest.mark.parametrize("case", ["m_f16_mm_32x16x32", "m_f16_mm_odd", "m_f16_mm", "m_bf16_mm", "m_f16_linear", "m_f16_bmm"])
def test_gemm_oracle_agrees_with_the_reference_kernel(golden, case):
    """The reference's mma.sync kernel (fragments, K loop, converted store; emmyptx/mma.py:65-242) for its own matmul
    cases, executed from its PTX text, against the float64 product of the same rounded operands: inside the
    reference's tolerance class, and -- the kernel accumulating in fp32 and rounding once -- within one rounding of
    the output type of the float64 value almost everywhere."""
    import torch
    got, ref, tol, td = _golden_gemm(golden, case)
    res = reference.compare(got, ref, **tol)
    assert res["ok"], res
    once = torch.from_numpy(ref).to(td).double().numpy()
    assert np.mean(got == once) > 0.98          # the rest differ by the fp32 accumulation's last bit before rounding


def test_interpreter_reproduces_the_gemm_fixture():
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())["m_f16_mm_32x16x32"]
    import torch
    a, b = inputs.gemm_inputs(32, 16, 32, "f16", scaled=False)
    bufs = {"A": a.view(torch.int16).numpy().copy(), "B": b.view(torch.int16).numpy().copy(), "C": np.zeros((32, 16), np.int16)}
    ptx_interp.run_entry((GOLDEN / "m_f16_mm_32x16x32.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
    assert np.array_equal(bufs["C"].view(np.uint16), np.load(GOLDEN / "golden.npz")["m_f16_mm_32x16x32.c"])



ATTENTION_CASES = ["f_sdpa", "t_causal_sdpa", "f_masked_attn_manual"]


def _attention_case(case):
    import torch
    a = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]["attention"]
    units = int(np.prod(a["units"]))
    q, k, v = (torch.from_numpy(x) for x in inputs.attention_inputs_f32(units, a["seq_q"], a["seq_k"], a["d"]))
    return a, q, k, v


@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_attention_oracle_agrees_with_the_reference_kernel(golden, case):
    """The reference's own attention cases (fp32 q, k, v; tools/torch_cases/fused.py:21-22, 31-36, models.py:17-19),
    its compiler's PTX for the scalar-loop kernel executed on the CPU, against the oracle's float64 attention: inside
    the reference's class for them (MM: rtol = atol = 1e-3) and, both being fp32 evaluations, two orders tighter."""
    a, q, k, v = _attention_case(case)
    ref = reference.attention_reference(q, k, v, scale=a["scale"], double=True, causal=a["causal"]).numpy()
    got = golden[f"{case}.o"].astype(np.float64)
    assert reference.compare(got, ref, rtol=1e-3, atol=1e-3)["ok"]
    assert np.allclose(got, ref, rtol=1e-5, atol=2e-6), float(np.abs(got - ref).max())


def test_interpreter_reproduces_the_attention_fixture():
    """Run-time loops with static trip counts (emmyptx/loops.py:231-264) are followed by the interpreter."""
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())["f_sdpa"]
    q, k, v = inputs.attention_inputs_f32(2, 64, 64, 32)
    bufs = {"Q": q.copy(), "K": k.copy(), "V": v.copy(), "O": np.zeros((2, 64, 32), np.float32)}
    ptx_interp.run_entry((GOLDEN / "f_sdpa.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
    assert np.array_equal(bufs["O"], np.load(GOLDEN / "golden.npz")["f_sdpa.o"])


@pytest.mark.parametrize("case", ["m_f16_mm_f32out", "m_bf16_mm_splitk4"])
def test_f32_output_gemm_fixture(golden, case):
    """The accumulator stored to an f32 buffer, and the split-K form of the same product (red.add.f32 into a zeroed C):
    both are the float64 product to within fp32 accumulation."""
    g = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]["gemm"]
    a, b = inputs.gemm_inputs(g["m"], g["n"], g["k"], g["dtype"], g["b_trans"], scaled=False)
    ref = (a.double() @ b.double()).numpy()
    scale = (a.double().abs() @ b.double().abs()).numpy() * 2.0 ** -21
    assert np.all(np.abs(golden[f"{case}.c32"].astype(np.float64) - ref) <= scale)


@pytest.mark.parametrize("case", ["s_transpose", "s_permute", "s_slice", "s_strided_slice", "s_flip", "s_stack", "s_tril", "s_cat_a", "s_cat_b",
                                  "s_roll", "s_embedding", "s_gather", "c_avg_pool1d", "c_max_pool2d", "s_tril_select", "s_window_let", "s_cat_cond", "s_pad_cond"])
def test_layout_fixture_is_what_numpy_computes(golden, case):
    """The reference's PTX for the data-movement kernels, executed on the CPU, moves exactly the elements the torch
    expression of the case moves (tools/torch_cases/shapes.py:6-19)."""
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]
    bufs = inputs.layout_buffers(info["tensors"], info["launch"]["arg_order"])
    assert np.array_equal(golden[f"{case}.out"], np.ascontiguousarray(inputs.LAYOUT_EXPECTED[case](bufs)).astype(np.float32))


@pytest.mark.parametrize("case", ["c_conv1d", "c_conv2d"])
def test_convolution_fixture_is_the_float64_convolution(golden, case):
    """The reference's PTX for its convolution cases (tools/torch_cases/conv.py:6-7), executed on the CPU, against the
    float64 sum of the same products: within fp32 accumulation of 48 and 72 terms (the reference's own bar for this
    category is its matmul tolerance class, tools/torch_cases/conv.py:6-7)."""
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]
    bufs = inputs.layout_buffers(info["tensors"], info["launch"]["arg_order"])
    ref = inputs.conv_expected(case, bufs)
    assert golden[f"{case}.out"].shape == ref.shape
    assert np.abs(golden[f"{case}.out"].astype(np.float64) - ref).max() < 2e-5


SEEDED = [f"row_{op}" for op in ("sum", "mean", "amax", "amin", "prod", "norm2", "var", "std", "logsumexp", "softmax", "log_softmax", "layer_norm",
                                 "rms_norm", "normalize", "dot")] + ["col_sum", "col_amax", "col_softmax", "m_mm", "m_bmm", "m_linear_bias_relu", "m_transpose_lhs"]


@pytest.mark.parametrize("case", SEEDED)
def test_reduction_and_f32_product_fixtures(golden, case):
    """The reference's PTX for the row / column reductions and normalisations (one thread per row: a loop per pass) and for
    the float32 products written as scalar loops, executed on the CPU: the float64 value of the same expression, to within
    fp32 accumulation (1e-5 of the result's scale, the reference's own class for these cases; 1e-4 for the 96- to 128-term
    dot products)."""
    info = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]
    bufs = inputs.seeded_buffers(info["tensors"], info["launch"]["arg_order"])
    ref = inputs.reduce_expected(case, bufs)
    got = golden[f"{case}.out"].astype(np.float64)
    assert got.shape == ref.shape
    tol = 1e-4 if case.startswith("m_") or case == "row_dot" else 1e-5
    assert np.all(np.abs(got - ref) <= tol * np.maximum(1.0, np.abs(ref).max())), (case, np.abs(got - ref).max())


@pytest.mark.parametrize("case", ["att16_bf16_causal_d64", "att16_f16_d128"])
def test_16_bit_attention_fixture(golden, case):
    """The reference's PTX for the scalar-loop attention on 16-bit buffers, executed on the CPU: the float64 attention of the
    same rounded operands to within one rounding to the output type."""
    import torch
    a = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]["attention"]
    units = int(np.prod(a["units"]))
    q, k, v = inputs.attention_inputs(units, a["seq_q"], a["seq_k"], a["d"], a["dtype"])
    ref = reference.attention_reference(q, k, v, scale=a["scale"], double=True, causal=a["causal"]).numpy()
    unit = (2.0 ** -8 if a["dtype"] == "bf16" else 2.0 ** -11) * max(1.0, float(np.abs(ref).max()))
    assert np.abs(golden[f"{case}.o"].astype(np.float64) - ref).max() <= unit

