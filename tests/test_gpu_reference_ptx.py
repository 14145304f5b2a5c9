"""Kernel against kernel: the reference's own PTX (tests/golden/*.ref.ptx, printed by the reference's compiler)
JIT-loaded on this GPU through the driver API, as the reference's runner does (tools/run_local.py:64-72,
:100-102), next to the sm_100a kernels on the same device buffers.

The reference text targets sm_89; the driver JITs it forward. The two streaming kernels are straight-line code
with in-range addresses by construction (grid * block == n, indices masked to n - 1). The tensor-core kernels
(`mma.sync` on fragments read from global memory, emmyptx/mma.py:65-242) are the guard-free ones of the fixture
set: whole m16n8k16 cells only, every address inside its buffer (checked when the fixtures are generated,
tests/golden/make_reference_ptx.py).
"""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def run_ptx(ptx: str, entry: str, ptrs: list, grid: int, block: int) -> None:
    from emmyptx.ptx_driver import PtxModule
    with PtxModule(ptx) as m:
        m.launch(m.function(entry), ptrs, grid, block)
        m.synchronize()


@pytest.fixture(scope="module")
def manifest():
    return json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())


def _reference_kernel(case, manifest, x_dev, cuda):
    import torch
    torch.cuda.synchronize()
    info = manifest[case]
    y = torch.zeros_like(x_dev)                      # outputs start zeroed (tools/run_local.py:92-93)
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [x_dev.data_ptr(), y.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    return y


def test_gather_bit_exact_against_the_reference_kernel(manifest, cuda):
    import torch
    from emmyptx import runtime
    x = torch.from_numpy(inputs.c2_input(2**20)).to(cuda)
    theirs = _reference_kernel("c2_gather_n1048576", manifest, x, cuda)
    ours = runtime.index_gather(x, 7919, 13, 3, 2, trunc=True)
    assert torch.equal(ours, theirs)
    # and the CPU interpreter of the same PTX agrees with the GPU's execution of it
    g = np.load(GOLDEN / "golden.npz")
    assert np.array_equal(theirs.cpu().numpy()[g["c2_gather_n1048576.index"]], g["c2_gather_n1048576.y"])


def test_pointwise_against_the_reference_kernel(manifest, cuda):
    import torch
    from emmyptx import runtime
    x_np = inputs.c1_input(2**20)
    x = torch.from_numpy(x_np).to(cuda)
    theirs = _reference_kernel("c1_exp_sin_tanh_n1048576", manifest, x, cuda).cpu().numpy()
    ours = runtime.pointwise("exp_sin_tanh", x).cpu().numpy()
    ref = reference.c1_f64(x_np)
    assert reference.compare(theirs, ref, 1e-5, 1e-5)["ok"]          # the reference meets its own class here
    assert reference.compare(ours, theirs, 1e-5, 1e-5)["ok"]         # and the two kernels agree within it
    # ours is the tighter of the two against float64, in the class's own measure (|err| / (1e-5 |ref| + 1e-5)) and in
    # ulps of the largest term (the fused form's exponentials come from the special-function unit: up to 2.5 ulp on a
    # large e^x, so the largest absolute error alone is no longer below the reference's)
    share = lambda y: (np.abs(y - ref) / (1e-5 * np.abs(ref) + 1e-5)).max()
    assert share(ours) <= share(theirs) and share(ours) <= 0.05
    assert reference.c1_condition_ulp(ours, x_np).max() <= min(5.0, reference.c1_condition_ulp(theirs, x_np).max())


HALF_MM, BF16_MM = dict(rtol=2e-2, atol=1e-1), dict(rtol=5e-2, atol=5e-1)      # tools/torch_cases/matmul.py:7


@pytest.mark.parametrize("case", ["m_f16_mm", "m_bf16_mm", "m_f16_linear", "m_f16_bmm"])
def test_gemm_against_the_reference_kernel(manifest, cuda, case):
    """The reference's own matmul cases (tools/torch_cases/matmul.py:27-32): its mma.sync kernel and the tcgen05 kernel
    on the same device buffers. Both must sit inside the reference's tolerance class of the float64 product; the two
    kernels accumulate in fp32 and round once, so they agree to one unit of the output type; and ours is no further
    from float64 than theirs. The CPU execution of the same PTX (the golden vectors) agrees with the GPU's."""
    import torch
    from emmyptx import runtime
    info = manifest[case]
    g = info["gemm"]
    assert g["device"]
    a, b = inputs.gemm_inputs(g["m"], g["n"], g["k"], g["dtype"], g["b_trans"], scaled=False, batch=tuple(g["batch"]))
    a_d, b_d = a.to(cuda), b.to(cuda)
    theirs = torch.zeros(*g["batch"], g["m"], g["n"], dtype=a.dtype, device=cuda)
    torch.cuda.synchronize()
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [a_d.data_ptr(), b_d.data_ptr(), theirs.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    if g["batch"]:
        ours = runtime.gemm_batched(a_d, b_d)
    else:
        ours = runtime.gemm(a_d, b_d, b_is_nk=g["b_trans"])
    torch.cuda.synchronize()
    bb = b.double().transpose(-1, -2) if g["b_trans"] else b.double()
    ref = (a.double() @ bb).numpy()
    tol = HALF_MM if g["dtype"] == "f16" else BF16_MM
    theirs_np, ours_np = theirs.cpu().double().numpy(), ours.cpu().double().numpy()
    assert reference.compare(theirs_np, ref, **tol)["ok"]
    assert reference.compare(ours_np, ref, **tol)["ok"]
    # kernel against kernel: identical after rounding except where the fp32 sums differ in their last bits
    assert np.mean(theirs_np == ours_np) > 0.98
    spacing = np.abs(ref) * (2.0 ** -10 if g["dtype"] == "f16" else 2.0 ** -7) + 1e-3
    assert np.all(np.abs(theirs_np - ours_np) <= 2 * spacing)
    assert np.abs(ours_np - ref).mean() <= np.abs(theirs_np - ref).mean() * 1.02
    gold = np.load(GOLDEN / "golden.npz")
    cpu = torch.from_numpy(gold[f"{case}.c"].view(np.int16)).view(a.dtype).double().numpy()
    on_gpu, space = theirs_np.reshape(-1, g["n"]), spacing.reshape(-1, g["n"])
    if f"{case}.rows" in gold.files:
        on_gpu, space = on_gpu[gold[f"{case}.rows"]], space[gold[f"{case}.rows"]]
    assert np.mean(cpu == on_gpu) > 0.98 and np.all(np.abs(cpu - on_gpu) <= 2 * space)



@pytest.mark.parametrize("case", ["f_sdpa", "t_causal_sdpa", "f_masked_attn_manual"])
def test_attention_against_the_reference_kernel(manifest, cuda, case):
    """The reference's own attention cases (fp32 q, k, v): the PTX its compiler prints for the scalar-loop kernel and
    the CUDA-core attention kernel of this library on the same device buffers. Nested loops with static trip counts, no
    barriers, every index a tile or loop variable with the buffer's own extent (checked when the fixture is generated).
    Both sit inside the reference's class (MM, 1e-3) of the float64 attention, agree with each other to fp32 rounding,
    and the CPU execution of the same PTX (the golden vector) agrees with the GPU's."""
    import torch
    from emmyptx import runtime
    info = manifest[case]
    a = info["attention"]
    units = int(np.prod(a["units"]))
    q, k, v = (torch.from_numpy(x).to(cuda) for x in inputs.attention_inputs_f32(units, a["seq_q"], a["seq_k"], a["d"]))
    theirs = torch.zeros(units, a["seq_q"], a["d"], device=cuda)
    torch.cuda.synchronize()
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [q.data_ptr(), k.data_ptr(), v.data_ptr(), theirs.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    ours = runtime.attention(q, k, v, scale=a["scale"], causal=a["causal"])
    torch.cuda.synchronize()
    ref = reference.attention_reference(q.cpu(), k.cpu(), v.cpu(), scale=a["scale"], double=True, causal=a["causal"]).numpy()
    theirs_np, ours_np = theirs.cpu().double().numpy(), ours.cpu().double().numpy()
    assert reference.compare(theirs_np, ref, rtol=1e-3, atol=1e-3)["ok"]
    assert reference.compare(ours_np, ref, rtol=1e-3, atol=1e-3)["ok"]
    assert np.allclose(ours_np, theirs_np, rtol=1e-5, atol=4e-6), float(np.abs(ours_np - theirs_np).max())
    assert np.abs(ours_np - ref).max() <= 2 * np.abs(theirs_np - ref).max() + 1e-6
    cpu = np.load(GOLDEN / "golden.npz")[f"{case}.o"].astype(np.float64)
    assert np.allclose(cpu, theirs_np, rtol=1e-5, atol=4e-6)          # ex2.approx and the division differ in the last bits


@pytest.mark.parametrize("case", ["c3_f16_mm_4096", "c4_bf16_mm_16384"])
def test_benchmark_size_products_against_the_reference_kernel(manifest, cuda, case):
    """Configurations 3 and 4 at their own sizes (4096^3 fp16; 16384^3 bf16): the reference's tensor-core lowering of the same
    IR (one warp per m16n8k16 cell, fragments read from global memory, emmyptx/mma.py:128-180) and `gemm_tcgen05_kernel` on
    the same device buffers. Both accumulate in fp32 and round once, so the outputs agree to one unit of the output type
    (the k order differs), and most elements are identical. Configuration 4's tanh-GELU cannot be part of the reference's
    store, so the fused epilogue is checked against the same GELU applied to this library's own unfused product."""
    import torch
    from emmyptx import runtime
    info = manifest[case]
    g = info["gemm"]
    td = torch.float16 if g["dtype"] == "f16" else torch.bfloat16
    gen = torch.Generator(device=cuda)
    gen.manual_seed(5)
    a = (torch.randn(g["m"], g["k"], device=cuda, generator=gen) / g["k"] ** 0.5).to(td)
    b = (torch.randn(g["k"], g["n"], device=cuda, generator=gen) / g["k"] ** 0.5).to(td)
    theirs = torch.zeros(g["m"], g["n"], device=cuda, dtype=td)
    torch.cuda.synchronize()
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [a.data_ptr(), b.data_ptr(), theirs.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    ours = runtime.gemm(a, b)
    torch.cuda.synchronize()
    unit = 2.0 ** (-8 if g["dtype"] == "bf16" else -11)
    rows = torch.randperm(g["m"], device=cuda, generator=gen)[:1024]                 # a sample of whole rows keeps the fp32 copies small
    o, t = ours[rows].float(), theirs[rows].float()
    assert bool(((o - t).abs() <= unit * t.abs() + 1e-3 * unit).all())
    assert float((ours[rows] == theirs[rows]).float().mean()) > 0.9
    ref = (a[rows[:64]].double() @ b.double())
    assert bool(((ours[rows[:64]].double() - ref).abs() <= unit * ref.abs() + 1e-3).all())
    if case.startswith("c4"):
        del theirs
        fused = runtime.gemm(a, b, epilogue="gelu_tanh")
        torch.cuda.synchronize()
        want = torch.nn.functional.gelu(ours[rows].float(), approximate="tanh")
        # the fused epilogue sees the fp32 accumulator, the comparison its bf16 rounding: two roundings apart at most
        assert bool(((fused[rows].float() - want).abs() <= 2 * unit * want.abs() + 2 * unit * 0.05).all())
    assert runtime.device_status() == 0


@pytest.mark.parametrize("case", ["att16_bf16_s1024_d128", "att16_bf16_causal_s1024_d128", "att16_bf16_s4096_d128"])
def test_both_attention_forms_against_the_reference_kernel(manifest, cuda, case):
    """Eight key tiles per unit and more (the last case is one unit of configuration 5: 4096 x 4096 x 128): long enough for
    `attention_fwd_pair_kernel` (two query tiles per CTA), which the library would pick here only with more units, so both
    forms are forced in turn and compared with the reference's scalar-loop
    kernel for the same IR on the same device buffers (a few seconds of CUDA-core work). Both forms inside the reference's
    bf16 class of the float64 attention and within two units of bf16 of the reference's kernel."""
    import torch
    from emmyptx import runtime
    info = manifest[case]
    a = info["attention"]
    units = int(np.prod(a["units"]))
    q, k, v = (t.to(cuda) for t in inputs.attention_inputs(units, a["seq_q"], a["seq_k"], a["d"], a["dtype"]))
    theirs = torch.zeros_like(q)
    torch.cuda.synchronize()
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [q.data_ptr(), k.data_ptr(), v.data_ptr(), theirs.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    torch.cuda.synchronize()
    ref = reference.attention_reference(q.cpu(), k.cpu(), v.cpu(), scale=None, double=True, causal=a["causal"]).numpy()
    theirs_np = theirs.cpu().double().numpy()
    assert reference.compare(theirs_np, ref, rtol=5e-2, atol=5e-1)["ok"]
    unit = 2.0 ** -8 * max(1.0, float(np.abs(ref).max()))
    for form in ("one_tile", "two_tiles"):
        ours = runtime.attention(q, k, v, causal=a["causal"], form=form)
        torch.cuda.synchronize()
        ours_np = ours.cpu().double().numpy()
        assert reference.compare(ours_np, ref, rtol=5e-2, atol=5e-1)["ok"], form
        assert np.abs(ours_np - theirs_np).max() <= 2 * unit, (form, float(np.abs(ours_np - theirs_np).max()))
    assert runtime.device_status() == 0


@pytest.mark.parametrize("case", ["att16_bf16_causal_d64", "att16_f16_d128"])
def test_tensor_core_attention_against_the_reference_kernel(manifest, cuda, case):
    """16-bit q, k, v at the head sizes the tensor-core kernels take: the reference's PTX for the scalar-loop kernel on
    16-bit buffers (every product and sum in fp32, one rounding at the store) and `attention_fwd_kernel` (tcgen05; P rounded
    to 16 bits before the second product) on the same device buffers. Both inside the reference's 16-bit matmul class of the
    float64 attention (HALF_MM / BF16_MM, tools/torch_cases/matmul.py:7), kernel against kernel within two units of the
    output type at the result's scale, and the CPU execution of the PTX agreeing with the GPU's to one unit."""
    import torch
    from emmyptx import ir, runtime
    from emmyptx.kernel import compile_kernel
    info = manifest[case]
    a = info["attention"]
    units = int(np.prod(a["units"]))
    handle = json.loads(compile_kernel(*ir.attention_scalar_kernel(a["units"], a["seq_q"], a["seq_k"], a["d"], a["dtype"], a["scale"], a["causal"], name=case)))
    assert handle["variant"] == "attention_fwd" and handle["params"]["dtype"] == a["dtype"] and handle["params"]["causal"] == a["causal"]
    q, k, v = (t.to(cuda) for t in inputs.attention_inputs(units, a["seq_q"], a["seq_k"], a["d"], a["dtype"]))
    theirs = torch.zeros_like(q)
    torch.cuda.synchronize()
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [q.data_ptr(), k.data_ptr(), v.data_ptr(), theirs.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    ours = runtime.attention(q, k, v, scale=handle["params"]["scale"], causal=a["causal"])
    torch.cuda.synchronize()
    ref = reference.attention_reference(q.cpu(), k.cpu(), v.cpu(), scale=handle["params"]["scale"], double=True, causal=a["causal"]).numpy()
    tol = dict(rtol=5e-2, atol=5e-1) if a["dtype"] == "bf16" else dict(rtol=2e-2, atol=1e-1)
    theirs_np, ours_np = theirs.cpu().double().numpy(), ours.cpu().double().numpy()
    assert reference.compare(theirs_np, ref, **tol)["ok"]
    assert reference.compare(ours_np, ref, **tol)["ok"]
    unit = (2.0 ** -8 if a["dtype"] == "bf16" else 2.0 ** -11) * max(1.0, float(np.abs(ref).max()))
    assert np.abs(ours_np - theirs_np).max() <= 2 * unit, float(np.abs(ours_np - theirs_np).max())
    cpu = np.load(GOLDEN / "golden.npz")[f"{case}.o"].astype(np.float64)
    assert np.abs(cpu - theirs_np).max() <= unit


@pytest.mark.parametrize("case", ["m_f16_mm_f32out", "m_bf16_mm_splitk4"])
def test_f32_output_gemm_against_the_reference_kernel(manifest, cuda, case):
    """The reference's store of an accumulator fragment to an f32 buffer, plain and as the split-K form (four cells per
    output cell adding partial sums into a zeroed C with red.add.f32, emmyptx/mma.py:239-240), next to the tcgen05 kernel's
    fp32 output on the same buffers: both are fp32 accumulations of the same products and agree to a few 2^-24 of
    sum |a b|; the CPU execution of the same PTX agrees likewise."""
    import torch
    from emmyptx import runtime
    info = manifest[case]
    g = info["gemm"]
    assert g["device"] and g["out_f32"]
    a, b = inputs.gemm_inputs(g["m"], g["n"], g["k"], g["dtype"], g["b_trans"], scaled=False)
    a_d, b_d = a.to(cuda), b.to(cuda)
    theirs = torch.zeros(g["m"], g["n"], dtype=torch.float32, device=cuda)       # zeroed: the split-K cells add into it
    torch.cuda.synchronize()
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [a_d.data_ptr(), b_d.data_ptr(), theirs.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    ours = runtime.gemm(a_d, b_d, out_f32=True)
    torch.cuda.synchronize()
    ref = (a.double() @ b.double()).numpy()
    scale = (a.double().abs() @ b.double().abs()).numpy() * 2.0 ** -21
    theirs_np, ours_np = theirs.cpu().double().numpy(), ours.cpu().double().numpy()
    assert np.all(np.abs(theirs_np - ref) <= scale) and np.all(np.abs(ours_np - ref) <= scale)
    assert np.all(np.abs(theirs_np - ours_np) <= scale)
    cpu = np.load(GOLDEN / "golden.npz")[f"{case}.c32"].astype(np.float64)
    assert np.all(np.abs(cpu - theirs_np) <= scale)

