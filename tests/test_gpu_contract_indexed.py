"""Nested-loop sums of products through `emmyb200_contract_indexed`: the reference's convolution cases
(tools/torch_cases/conv.py:6-7) written as scalar loops, from IR to result through the facade, against the float64
convolution, against torch's own convolution on this GPU and -- bit for bit, since both fold fp32 fused multiply-adds in
the same loop order -- against the reference compiler's PTX for the same IR (golden vector from the CPU, and JIT-loaded
on this GPU next to ours)."""
import json
from pathlib import Path

import numpy as np
import pytest

from emmyptx import ir, run_local
from emmyptx.kernel import compile_kernel
from oracle import inputs

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
MM = dict(rtol=1e-3, atol=1e-3)           # the reference's bar for this category (tools/torch_cases/__init__.py:20)


@pytest.mark.parametrize("case", ["c_conv1d", "c_conv2d"])
def test_convolution_case_matches_the_reference_kernel(case, cuda):
    import torch
    import torch.nn.functional as F
    from emmyptx.ptx_driver import PtxModule
    g, k, launch = ir.conv_kernel(case, name=case)
    handle = json.loads(compile_kernel(g, k, launch))
    assert handle["variant"] == "contract_indexed"
    tensors = {t.name: {"shape": [d.as_static() for d in t.shape], "dtype": t.dtype.name} for nd in g.nodes.values() for t in nd.outputs}
    host = inputs.layout_buffers(tensors, launch["arg_order"])
    dev = {nm: torch.from_numpy(a).to(cuda) for nm, a in host.items()}
    run_local.init()
    run_local.launch(handle, dev)
    torch.cuda.synchronize()
    got = dev["out"].cpu().numpy()
    ref = inputs.conv_expected(case, host)
    assert np.abs(got.astype(np.float64) - ref).max() < 2e-5
    conv = F.conv1d if case == "c_conv1d" else F.conv2d
    assert np.allclose(got, conv(dev["X"][None], dev["W"])[0].cpu().numpy(), **MM)
    # the reference's PTX for the same IR: the CPU-interpreted golden vector, and the same text on this GPU
    assert np.array_equal(np.load(GOLDEN / "golden.npz")[f"{case}.out"], got)
    theirs = torch.zeros_like(dev["out"])
    ptrs = [dev[nm].data_ptr() if nm != "out" else theirs.data_ptr() for nm in launch["arg_order"]]
    with PtxModule((GOLDEN / f"{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(case), ptrs, launch["grid"][0], launch["block"][0])
        m.synchronize()
    assert torch.equal(theirs, dev["out"])


def test_contractions_directly(cuda):
    """16-bit buffers, a strided and dilated 1-d convolution with a flipped kernel (negative coefficient), one reduction
    axis (a matrix-vector product), an empty tile, and the range checks."""
    import torch
    from emmyptx import runtime as rt
    # out[o, i] = sum_{c, t} w[o, c, 2 - t] * x[c, 2 i + 3 t]: stride 2, dilation 3, taps reversed
    x = torch.randn(6, 64, device=cuda).to(torch.bfloat16)
    w = torch.randn(5, 6, 3, device=cuda).to(torch.float16)
    n_out = (64 - 3 * 2 - 1) // 2 + 1
    out = torch.zeros(5, n_out, dtype=torch.bfloat16, device=cuda)
    cm = {"extents": [5, n_out], "loops": [6, 3], "a": {"offset": 2, "coef": [18, 0], "loop_coef": [3, -1], "dtype": "f16"},
          "b": {"offset": 0, "coef": [0, 2], "loop_coef": [64, 3], "dtype": "bf16"}, "out": {"offset": 0, "coef": [n_out, 1], "dtype": "bf16"}}
    rt.contract_indexed(cm, w.reshape(-1), x.reshape(-1), out.reshape(-1))
    ref = torch.nn.functional.conv1d(x.double()[None], w.double().flip(-1), stride=2, dilation=3)[0]
    assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2)
    # one reduction axis: y = A v
    a = torch.randn(300, 517, device=cuda)
    v = torch.randn(517, device=cuda)
    y = torch.zeros(300, device=cuda)
    mv = {"extents": [300], "loops": [517], "a": {"offset": 0, "coef": [517], "loop_coef": [1], "dtype": "f32"},
          "b": {"offset": 0, "coef": [0], "loop_coef": [1], "dtype": "f32"}, "out": {"offset": 0, "coef": [1], "dtype": "f32"}}
    rt.contract_indexed(mv, a.reshape(-1), v, y)
    assert torch.allclose(y.double(), a.double() @ v.double(), rtol=1e-5, atol=1e-4)
    # an empty tile launches nothing and touches nothing
    rt.contract_indexed(dict(mv, extents=[0]), a.reshape(-1), v, y)
    # ranges are checked against the tensors before anything is launched
    with pytest.raises(IndexError):
        rt.contract_indexed(dict(mv, loops=[518]), a.reshape(-1), v, y)
    with pytest.raises(IndexError):
        rt.contract_indexed(dict(mv, out={"offset": 1, "coef": [1], "dtype": "f32"}), a.reshape(-1), v, y)
    with pytest.raises(IndexError):
        rt.contract_indexed(dict(mv, a={"offset": 0, "coef": [-517], "loop_coef": [1], "dtype": "f32"}), a.reshape(-1), v, y)
    torch.cuda.synchronize()


def test_a_larger_convolution(cuda):
    """A 64-channel 3 x 3 convolution over a 128 x 128 image (more cells than one wave of threads, int32 index path)."""
    import torch
    from emmyptx import runtime as rt
    c, o, h = 64, 32, 128
    x = torch.randn(c, h, h, device=cuda)
    w = torch.randn(o, c, 3, 3, device=cuda)
    out = torch.zeros(o, h - 2, h - 2, device=cuda)
    cm = {"extents": [o, h - 2, h - 2], "loops": [c, 3, 3], "a": {"offset": 0, "coef": [c * 9, 0, 0], "loop_coef": [9, 3, 1], "dtype": "f32"},
          "b": {"offset": 0, "coef": [0, h, 1], "loop_coef": [h * h, h, 1], "dtype": "f32"}, "out": {"offset": 0, "coef": [(h - 2) ** 2, h - 2, 1], "dtype": "f32"}}
    rt.contract_indexed(cm, w.reshape(-1), x.reshape(-1), out.reshape(-1))
    torch.cuda.synchronize()
    ref = torch.nn.functional.conv2d(x.double()[None], w.double())[0]
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=5e-4)


def test_transposed_lhs_product(cuda):
    """m_transpose_lhs (tools/torch_cases/matmul.py:20): a.t() @ b with a stored [k, m]. The float32 GEMM reads A row-major,
    so the facade serves this product with the indexed contraction (one reduction axis, A walked with stride m)."""
    import torch
    g, k, launch = ir.matmul_f32_kernel(128, 80, 96, a_trans=True, name="m_transpose_lhs")
    handle = json.loads(compile_kernel(g, k, launch))
    assert handle["variant"] == "contract_indexed" and handle["params"]["map"]["a"]["loop_coef"] == [128]
    a, b = torch.randn(96, 128, device=cuda), torch.randn(96, 80, device=cuda)
    out = torch.zeros(128, 80, device=cuda)
    run_local.init()
    run_local.launch(handle, {"A": a, "B": b, "C": out})
    torch.cuda.synchronize()
    assert torch.allclose(out.double(), a.double().T @ b.double(), **MM)
    assert torch.allclose(out.double(), a.double().T @ b.double(), rtol=1e-5, atol=1e-4)

