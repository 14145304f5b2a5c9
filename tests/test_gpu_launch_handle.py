"""emmyb200_launch: a kernel handle launched from raw device pointers, the way the reference's runner launches a PTX
entry (tools/run_local.py:80-102: one pointer per parameter of `arg_order`, buffers as device pointers, scalars by
value). The test plays a runner that holds nothing but addresses: it compiles IR to handle text, passes the text and
a ctypes parameter array through the C ABI, and checks the buffers against the oracle."""
import ctypes
import json

import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu


def launch(lib, text: str, values: list, stream=None) -> int:
    """values: per arg_order entry a torch CUDA tensor (passed as its device pointer) or a ctypes scalar."""
    import torch
    holders = [ctypes.c_void_p(v.data_ptr()) if isinstance(v, torch.Tensor) else v for v in values]
    params = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.byref(h), ctypes.c_void_p) for h in holders])
    need = lib.emmyb200_launch_workspace_bytes(text.encode())
    assert need >= 0
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda") if need else None
    rc = lib.emmyb200_launch(text.encode(), params, len(holders), ws.data_ptr() if ws is not None else None, need, stream)
    torch.cuda.synchronize()
    return rc


def handle_text(built) -> str:
    from emmyptx.kernel import compile_kernel
    return compile_kernel(*built)


def test_streaming_and_gather_handles(cuda, lib):
    import torch
    from emmyptx import ir
    x = inputs.c1_input(2**16)
    xd, yd = torch.from_numpy(x).to(cuda), torch.zeros(2**16, device=cuda)
    assert launch(lib, handle_text(ir.pointwise_kernel(2**16)), [xd, yd]) == 0
    assert reference.compare(yd.cpu().numpy(), reference.c1_f64(x), 1e-5, 1e-5)["ok"]
    xi = inputs.c2_input(2**20)
    xid, yid = torch.from_numpy(xi).to(cuda), torch.zeros(2**20, dtype=torch.int32, device=cuda)
    assert launch(lib, handle_text(ir.index_gather_kernel(2**20)), [xid, yid]) == 0
    assert np.array_equal(yid.cpu().numpy(), reference.c2_reference(xi))


def test_indexed_handles(cuda, lib):
    """Data-movement kernels (tools/torch_cases/shapes.py:6-19): the handle carries the index map, the runner only pointers."""
    import torch
    from emmyptx import ir
    x = torch.randn(64, 64, device=cuda)
    out = torch.zeros(64, 64, device=cuda)
    assert launch(lib, handle_text(ir.layout_kernel("s_tril")), [x, out]) == 0
    assert torch.equal(out, torch.tril(x))
    a, b = torch.randn(32, 64, device=cuda), torch.randn(32, 64, device=cuda)
    stacked = torch.zeros(2, 32, 64, device=cuda)
    assert launch(lib, handle_text(ir.layout_kernel("s_stack")), [a, b, stacked]) == 0
    assert torch.equal(stacked, torch.stack([a, b]))
    x = torch.randn(64, 96, device=cuda)
    t = torch.zeros(96, 64, device=cuda)
    assert launch(lib, handle_text(ir.layout_kernel("s_transpose")), [x, t]) == 0
    assert torch.equal(t, x.t().contiguous())
    x = torch.randn(64, 128, device=cuda)                               # a negative coefficient in the handle's map
    f = torch.zeros(64, 128, device=cuda)
    assert launch(lib, handle_text(ir.layout_kernel("s_flip")), [x, f]) == 0
    assert torch.equal(f, x.flip(-1))


def test_scalar_parameters_are_passed_by_value(cuda, lib):
    """out = (x * alpha + y) * 2 with alpha a `.param .f32`-style argument: the same handle, two values."""
    import torch
    from emmyptx import ir
    n = 5000
    built = ir.elementwise_kernel(n, {"x": "f32", "y": "f32"}, [("ax", "multiply", ["x", "alpha"]), ("s", "add", ["ax", "y"]),
                                                                ("o", "multiply", ["s", 2.0])], scalars={"alpha": "f32"})
    text = handle_text(built)
    assert json.loads(text)["arg_order"] == ["x", "y", "out", "alpha"]
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(n, generator=g), torch.randn(n, generator=g)
    out = torch.zeros(n, device=cuda)
    for alpha in (0.5, -3.25):
        assert launch(lib, text, [x.to(cuda), y.to(cuda), out, ctypes.c_float(alpha)]) == 0
        ref = (x.double() * alpha + y.double()) * 2
        assert reference.compare(out.cpu().numpy(), ref.numpy(), 1e-6, 1e-6)["ok"]
    # an integer scalar in an integer program
    built = ir.elementwise_kernel(n, {"a": "i32"}, [("t", "multiply", ["a", "k"]), ("o", "add", ["t", 7])], out_dtype="i32", scalars={"k": "s32"})
    for st in built[1].body[0].body:
        if type(st).__name__ == "Assign":
            st.dtype = "i32"
    a = torch.randint(-1000, 1000, (n,), dtype=torch.int32)
    oi = torch.zeros(n, dtype=torch.int32, device=cuda)
    assert launch(lib, handle_text(built), [a.to(cuda), oi, ctypes.c_int32(-11)]) == 0
    assert torch.equal(oi.cpu(), a * -11 + 7)


def test_contraction_handles(cuda, lib):
    import torch
    from emmyptx import ir
    a, b = inputs.gemm_inputs(300, 520, 264, "bf16")
    c = torch.zeros(300, 520, dtype=torch.bfloat16, device=cuda)
    assert launch(lib, handle_text(ir.gemm_kernel(300, 520, 264, "bf16", "gelu_tanh")), [a.to(cuda), b.to(cuda), c]) == 0
    ok, ratio = reference.gemm_tolerance_ok(c.cpu(), reference.gemm_reference(a, b, "gelu_tanh"))
    assert ok, ratio
    a, b = inputs.gemm_inputs(64, 512, 256, "f16", b_is_nk=True)
    bias = torch.randn(512).half()
    c = torch.zeros(64, 512, dtype=torch.float16, device=cuda)
    text = handle_text(ir.gemm_kernel(64, 512, 256, "f16", "relu", True, bias=True, name="k_linear"))
    assert launch(lib, text, [a.to(cuda), b.to(cuda), bias.to(cuda), c]) == 0
    ref = torch.relu(a.float() @ b.float().t() + bias.float())
    ok, ratio = reference.gemm_tolerance_ok(c.cpu(), ref)
    assert ok, ratio
    a, b = inputs.gemm_inputs(128, 96, 256, "f16")                      # split-K IR: one kernel with an fp32 output
    c32 = torch.zeros(128, 96, dtype=torch.float32, device=cuda)
    assert launch(lib, handle_text(ir.gemm_kernel(128, 96, 256, "f16", out_dtype="f32", split_k=4)), [a.to(cuda), b.to(cuda), c32]) == 0
    assert torch.allclose(c32.cpu().double(), a.double() @ b.double(), rtol=1e-5, atol=1e-6)
    q, k, v = inputs.attention_inputs(3, 200, 328, 128, "bf16")
    o = torch.zeros_like(q, device=cuda)
    assert launch(lib, handle_text(ir.attention_kernel([3], 200, 328, 128, "bf16")), [q.to(cuda), k.to(cuda), v.to(cuda), o]) == 0
    ok, ratio = reference.gemm_tolerance_ok(o.cpu(), reference.attention_reference(q, k, v))
    assert ok, ratio


def test_handles_that_need_a_workspace(cuda, lib):
    import torch
    from emmyptx import ir
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4, 200000, generator=g)                         # rows beyond 65536 columns: split path, scratch memory
    y = torch.zeros_like(x, device=cuda)
    text = handle_text(ir.rowwise_kernel("softmax", 4, 200000))
    assert lib.emmyb200_launch_workspace_bytes(text.encode()) > 0
    assert launch(lib, text, [x.to(cuda), y]) == 0
    assert reference.compare(y.cpu().numpy(), reference.rowwise_reference("softmax", x).numpy(), 1e-3, 1e-5)["ok"]
    a, b = torch.randn(96, 200, generator=g), torch.randn(200, 136, generator=g)
    c = torch.zeros(96, 136, device=cuda)
    text = handle_text(ir.matmul_f32_kernel(96, 136, 200))
    assert lib.emmyb200_launch_workspace_bytes(text.encode()) > 0
    assert launch(lib, text, [a.to(cuda), b.to(cuda), c]) == 0
    assert reference.compare(c.cpu().numpy(), (a.double() @ b.double()).numpy(), 1e-3, 1e-3)["ok"]


def test_launch_rejects_what_it_cannot_run(cuda, lib):
    import torch
    from emmyptx import ir
    text = handle_text(ir.pointwise_kernel(64))
    x = torch.zeros(64, device=cuda)
    assert launch(lib, text, [x]) == -1                               # one parameter short
    assert b"arg_order" in lib.emmyb200_last_error()
    assert lib.emmyb200_launch(b"not json", None, 0, None, 0, None) == -1
    broken = json.loads(text)
    broken["variant"] = "frobnicate"
    assert launch(lib, json.dumps(broken), [x, x]) == -4


def test_contraction_handle(cuda, lib):
    """A convolution written as scalar loops (tools/torch_cases/conv.py:7): the handle carries the three affine maps, the
    runner passes X, W and out in the launch's argument order."""
    import torch
    from emmyptx import ir
    built = ir.conv_kernel("c_conv2d")
    assert built[2]["arg_order"] == ["X", "W", "out"]
    x = torch.randn(8, 32, 32, device=cuda)
    w = torch.randn(16, 8, 3, 3, device=cuda)
    out = torch.zeros(16, 30, 30, device=cuda)
    assert launch(lib, handle_text(built), [x, w, out]) == 0
    ref = torch.nn.functional.conv2d(x.double()[None], w.double())[0]
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-4)


def test_guarded_read_handle(cuda, lib):
    """torch.cat as one kernel (a Cond on the column index): the handle's index map carries the clamp of each guarded read."""
    import torch
    from emmyptx import ir
    a, b = torch.randn(32, 64, device=cuda), torch.randn(32, 48, device=cuda)
    out = torch.zeros(32, 112, device=cuda)
    assert launch(lib, handle_text(ir.layout_kernel("s_cat_cond")), [a, b, out]) == 0
    assert torch.equal(out, torch.cat([a, b], -1))


@pytest.mark.parametrize("case,value", [("sc_axpy2", 0.5), ("sc_axpy2", -3.25), ("sc_imul", -11)])
def test_scalar_parameters_against_the_reference_kernel(case, value, cuda, lib):
    """The reference's PTX for the same IR takes the scalar as a `.param .f32` / `.param .s32` in the same position of the
    argument list; this library's handle takes it through `emmyb200_launch`. Same buffers, same value: the integer
    program bit for bit, the float one to one rounding (the driver's JIT contracts the reference's multiply and add)."""
    import ctypes as ct
    from pathlib import Path
    import torch
    from emmyptx import ir
    from emmyptx.ptx_driver import PtxModule
    from elementwise_cases import SCALAR_CASES, scalar_kernel
    golden = Path(__file__).resolve().parent / "golden"
    built = scalar_kernel(ir, case)
    manifest = json.loads((golden / "reference_ptx_manifest.json").read_text())[case]
    assert built[2]["arg_order"] == manifest["launch"]["arg_order"]
    ins, _steps, out_dt, scalars, integer = SCALAR_CASES[case]
    n = 5000
    g = torch.Generator().manual_seed(0)
    bufs = [(torch.randint(-1000, 1000, (n,), dtype=torch.int32, generator=g) if integer else torch.randn(n, generator=g)).to(cuda) for _ in ins]
    tdt = torch.int32 if integer else torch.float32
    ours, theirs = torch.zeros(n, dtype=tdt, device=cuda), torch.zeros(n, dtype=tdt, device=cuda)
    scalar = ct.c_int32(value) if integer else ct.c_float(value)
    assert launch(lib, handle_text(built), [*bufs, ours, scalar]) == 0
    launch_d = built[2]
    with PtxModule((golden / f"{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(case), [*[b.data_ptr() for b in bufs], theirs.data_ptr(), scalar], launch_d["grid"][0], launch_d["block"][0])
        m.synchronize()
    torch.cuda.synchronize()
    if integer:
        assert torch.equal(ours, theirs) and torch.equal(ours.cpu(), bufs[0].cpu() * value + 7)
    else:
        assert torch.allclose(ours, theirs, rtol=1e-6, atol=1e-6)

