"""The stand-in Kernel IR is IR the reference's own compiler accepts (CPU only; needs a checkout of the reference).

The facade's matchers are exercised on IR made by the builders of `emmyptx/ir.py`. This test feeds the same objects
to the reference's `compile_kernel` (emmyptx/kernel.py:903): every builder whose statements the reference supports
must compile to PTX there, so the matchers see IR of the form the reference consumes, not a private dialect. Two
builders are outside the reference's statement set by design and must be refused by it: a tensor-core store with a
fused epilogue (emmyptx/mma.py:201-203 -- the fusion is what the sm_100a GEMM adds), and the 16-bit attention kernel,
whose softmax between the two MMA groups is written on fragment names directly (the reference has no statement that turns
an accumulator fragment into an operand fragment; its tracer goes through shared memory). The checkout is looked up
in $EMMYPTX_REFERENCE, else in a directory `reference` next to the repository; without one the test is skipped.
"""
import importlib
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = Path(os.environ.get("EMMYPTX_REFERENCE", ROOT.parent / "reference"))


@pytest.fixture(scope="module")
def reference_compile():
    if not (REF / "emmyptx" / "kernel.py").exists():
        pytest.skip("no checkout of the reference")
    # the facade package has the same name; load the reference's under its own name from its own path
    saved_path, saved_mods = list(sys.path), {k: v for k, v in sys.modules.items() if k == "emmyptx" or k.startswith("emmyptx.")}
    for k in saved_mods:
        del sys.modules[k]
    sys.path.insert(0, str(REF))
    try:
        mod = importlib.import_module("emmyptx.kernel")
        assert Path(mod.__file__).resolve().is_relative_to(REF.resolve())
        yield mod
    finally:
        for k in [k for k in sys.modules if k == "emmyptx" or k.startswith("emmyptx.")]:
            del sys.modules[k]
        sys.modules.update(saved_mods)
        sys.path[:] = saved_path


def _ir():
    spec = importlib.util.spec_from_file_location("standin_ir_for_reference", ROOT / "emmy-ptx-compiler_b200" / "emmyptx" / "ir.py")
    ir = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = ir
    spec.loader.exec_module(ir)
    return ir


ROW_OPS = ["sum", "mean", "amax", "amin", "prod", "var", "std", "norm2", "dot", "logsumexp", "softmax", "log_softmax",
           "layer_norm", "rms_norm", "normalize"]


def accepted_cases(ir):
    yield "c1", ir.pointwise_kernel(4096, "exp_sin_tanh")
    yield "gelu", ir.pointwise_kernel(4096, "gelu_tanh")
    yield "c2", ir.index_gather_kernel(2**16)
    yield "where", ir.elementwise_kernel(1024, {"x": "f32", "m": "bool"}, [("nx", "negative", ["x"]), ("y", "where", ["m", "x", "nx"])])
    yield "m_f16_mm", ir.gemm_kernel(256, 256, 256, "f16")
    yield "m_bf16_mm", ir.gemm_kernel(512, 512, 512, "bf16")
    yield "m_f16_mm_odd", ir.gemm_kernel(100, 72, 200, "f16")
    yield "m_f16_linear", ir.gemm_kernel(64, 512, 256, "f16", None, True)
    yield "m_f16_bmm", ir.gemm_kernel(128, 96, 64, "f16", batch=(4,))
    yield "m_f16_bcast", ir.gemm_kernel(128, 96, 64, "f16", batch=(4,), b_batched=False)
    yield "m_f16_mm_f32out", ir.gemm_kernel(128, 128, 256, "f16", out_dtype="f32")
    yield "m_bf16_mm_splitk4", ir.gemm_kernel(128, 128, 256, "bf16", out_dtype="f32", split_k=4)
    yield "c3", ir.gemm_kernel(4096, 4096, 4096, "f16")
    yield "c4_without_epilogue", ir.gemm_kernel(16384, 16384, 16384, "bf16")
    yield "m_mm", ir.matmul_f32_kernel(128, 80, 96)
    yield "m_bmm", ir.matmul_f32_kernel(64, 48, 32, batch=4)
    yield "m_linear_bias_relu", ir.matmul_f32_kernel(64, 96, 128, b_trans=True, bias=True, relu=True)
    yield "f_sdpa", ir.attention_scalar_kernel([1, 2], 64, 64, 32)
    yield "t_causal_sdpa", ir.attention_scalar_kernel([1, 4], 128, 128, 64, causal=True)
    yield "f_masked_attn_manual", ir.attention_scalar_kernel([1], 64, 64, 32, scale=0.17677669, causal=True)
    for case in ("s_transpose", "s_permute", "s_slice", "s_strided_slice", "s_flip", "s_repeat", "s_stack", "s_tril", "s_cat_a", "s_cat_b", "s_roll",
                 "s_embedding", "s_gather", "c_avg_pool1d", "c_max_pool2d", "s_tril_select", "s_window_let", "s_cat_cond", "s_pad_cond"):
        yield case, ir.layout_kernel(case)
    for case in ("c_conv1d", "c_conv2d"):
        yield case, ir.conv_kernel(case)
    for op in ROW_OPS:
        yield f"row_{op}", ir.rowwise_kernel(op, 64, 256)
    for op in ("sum", "amax", "softmax"):
        yield f"col_{op}", ir.colwise_kernel(op, 256, 64)


def test_reference_compiles_the_builders_ir(reference_compile):
    ir = _ir()
    for name, (graph, kernel, launch) in accepted_cases(ir):
        ptx = reference_compile.compile_kernel(graph, kernel, launch, target="sm_89")
        assert f".visible .entry {kernel.name}(" in ptx, name
        if "MmaSyncPtx" in {type(s).__name__ for s in _walk(kernel.body)}:
            assert "mma.sync.aligned.m16n8k16.row.col.f32" in ptx, name


def test_reference_output_is_the_committed_fixture(reference_compile):
    """The committed PTX fixtures are what the reference prints today for the same IR."""
    ir = _ir()
    golden = ROOT / "tests" / "golden"
    for name, built in (("m_f16_mm", ir.gemm_kernel(256, 256, 256, "f16", name="m_f16_mm")),
                        ("m_f16_linear", ir.gemm_kernel(64, 512, 256, "f16", None, True, name="m_f16_linear")),
                        ("c2_gather_n65536", ir.index_gather_kernel(2**16, name="c2_gather_n65536")),
                        ("t_causal_sdpa", ir.attention_scalar_kernel([1, 4], 128, 128, 64, causal=True, name="t_causal_sdpa"))):
        assert reference_compile.compile_kernel(*built, target="sm_89") == (golden / f"{name}.ref.ptx").read_text(), name


def test_reference_refuses_what_lies_outside_its_statement_set(reference_compile):
    ir = _ir()
    with pytest.raises(reference_compile.CompileError, match="epilogue"):
        reference_compile.compile_kernel(*ir.gemm_kernel(256, 256, 256, "bf16", "gelu_tanh"), target="sm_89")
    with pytest.raises(reference_compile.CompileError):
        reference_compile.compile_kernel(*ir.attention_kernel([2], 128, 128, 64, "f16"), target="sm_89")


def _walk(body):
    for s in body:
        yield s
        for attr in ("body",):
            sub = getattr(s, attr, None)
            if isinstance(sub, list):
                yield from _walk(sub)
