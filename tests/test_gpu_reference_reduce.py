"""Row / column reductions and normalisations and the float32 products, kernel against kernel: the reference compiler's own
PTX for the same IR (one thread per row with a loop per pass; one thread per output element with a loop over K), committed
as text fixtures, is JIT-loaded on this GPU and run on the same seeded buffers as this library's kernels
(`emmyb200_rowwise_f32`, `emmyb200_colwise_f32`, `emmyb200_gemm_f32`, `emmyb200_contract_indexed`). Both must sit inside the
reference's tolerance class of the float64 value (tools/torch_cases/__init__.py:17-21: RED / TRANS 1e-5 scaled to the
result, MM 1e-3), agree with each other to that class, and the CPU execution of the PTX (the golden vectors) must agree
with the GPU's."""
import json
from pathlib import Path

import numpy as np
import pytest

from emmyptx import ir, run_local
from emmyptx.kernel import compile_kernel
from oracle import inputs

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
ROWS = ["sum", "mean", "amax", "amin", "prod", "norm2", "var", "std", "logsumexp", "softmax", "log_softmax", "layer_norm", "rms_norm",
        "normalize", "dot"]
BUILD = {f"row_{op}": (lambda op=op: ir.rowwise_kernel(op, 64, 256, name=f"row_{op}")) for op in ROWS}
BUILD.update({f"col_{op}": (lambda op=op: ir.colwise_kernel(op, 256, 64, name=f"col_{op}")) for op in ("sum", "amax", "softmax")})
BUILD.update({
    "m_mm": lambda: ir.matmul_f32_kernel(128, 80, 96, name="m_mm"),
    "m_bmm": lambda: ir.matmul_f32_kernel(64, 48, 32, batch=4, name="m_bmm"),
    "m_linear_bias_relu": lambda: ir.matmul_f32_kernel(64, 96, 128, b_trans=True, bias=True, relu=True, name="m_linear_bias_relu"),
    "m_transpose_lhs": lambda: ir.matmul_f32_kernel(128, 80, 96, a_trans=True, name="m_transpose_lhs"),
})
VARIANT = {"m_mm": "gemm_f32", "m_bmm": "gemm_f32", "m_linear_bias_relu": "gemm_f32", "m_transpose_lhs": "contract_indexed"}


@pytest.mark.parametrize("case", sorted(BUILD))
def test_against_the_reference_kernel(case, cuda):
    import torch
    from emmyptx.ptx_driver import PtxModule
    manifest = json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())[case]
    graph, kernel, launch = BUILD[case]()
    assert launch == manifest["launch"]                                   # the fixture was made from this IR
    handle = json.loads(compile_kernel(graph, kernel, launch))
    assert handle["variant"] == VARIANT.get(case, "rowwise_f32" if case.startswith("row_") else "colwise_f32")
    host = inputs.seeded_buffers(manifest["tensors"], launch["arg_order"])
    result = launch["arg_order"][-1]
    ref = inputs.reduce_expected(case, host)
    scale = max(1.0, float(np.abs(ref).max()))
    tol = (1e-3 if case.startswith("m_") else 1e-5) * scale

    dev = {nm: torch.from_numpy(a).to(cuda) for nm, a in host.items()}
    run_local.init()
    run_local.launch(handle, dev)
    torch.cuda.synchronize()
    ours = dev[result].cpu().numpy().astype(np.float64)

    theirs_t = torch.zeros_like(dev[result])
    ptrs = [dev[nm].data_ptr() if nm != result else theirs_t.data_ptr() for nm in launch["arg_order"]]
    with PtxModule((GOLDEN / f"{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(case), ptrs, launch["grid"][0], launch["block"][0])
        m.synchronize()
    theirs = theirs_t.cpu().numpy().astype(np.float64)

    assert ours.shape == ref.shape
    assert np.abs(theirs - ref).max() <= tol, "the reference's kernel meets its own class"
    assert np.abs(ours - ref).max() <= tol
    assert np.abs(ours - theirs).max() <= tol
    # the CPU execution of the same PTX (exp / log through numpy instead of the GPU's approximations: a looser match there)
    golden = np.load(GOLDEN / "golden.npz")[f"{case}.out"].astype(np.float64)
    assert np.abs(golden - theirs).max() <= 1e-5 * scale
