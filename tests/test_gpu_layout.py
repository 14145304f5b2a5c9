"""Data movement through the indexed elementwise kernel (`emmyb200_pointwise_indexed`): the reference's layout cases
(tools/torch_cases/shapes.py:6-19) written as one-cell-per-element tiles with index expressions of the axis variables,
from IR to result through the facade, bit for bit against numpy and against the reference compiler's own PTX for the same
IR (run on the CPU into the golden vectors, and on this GPU next to ours)."""
import json
from pathlib import Path

import numpy as np
import pytest

from emmyptx import ir, run_local
from emmyptx.kernel import compile_kernel
from oracle import inputs

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["s_transpose", "s_permute", "s_slice", "s_strided_slice", "s_flip", "s_repeat", "s_stack", "s_tril", "s_cat_a", "s_cat_b",
         "s_roll", "s_embedding", "s_gather", "c_avg_pool1d", "c_max_pool2d", "s_tril_select", "s_window_let", "s_cat_cond", "s_pad_cond"]


def _run(case, cuda):
    import torch
    g, k, launch = ir.layout_kernel(case, name=case)
    handle = json.loads(compile_kernel(g, k, launch))
    tensors = {t.name: {"shape": [d.as_static() for d in t.shape], "dtype": t.dtype.name} for nd in g.nodes.values() for t in nd.outputs}
    host = inputs.layout_buffers(tensors, launch["arg_order"])
    dev = {nm: torch.from_numpy(a).to(cuda) for nm, a in host.items()}
    run_local.init()
    run_local.launch(handle, dev)
    torch.cuda.synchronize()
    return handle, host, dev, launch


@pytest.mark.parametrize("case", CASES)
def test_layout_case_matches_numpy_and_the_reference_kernel(case, cuda):
    import torch
    from emmyptx.ptx_driver import PtxModule
    handle, host, dev, launch = _run(case, cuda)
    assert handle["variant"] == ("pointwise_program" if case == "s_repeat" else "pointwise_indexed")
    want = np.ascontiguousarray(inputs.LAYOUT_EXPECTED[case](host)).astype(np.float32)
    got = dev["out"].cpu().numpy()
    assert np.array_equal(got, want)
    if not (GOLDEN / f"{case}.ref.ptx").exists():
        return
    # the reference's PTX for the same IR: on the CPU (golden vector) and on this GPU, same buffers
    assert np.array_equal(np.load(GOLDEN / "golden.npz")[f"{case}.out"], want)
    theirs = torch.zeros_like(dev["out"])
    ptrs = [dev[nm].data_ptr() if nm != "out" else theirs.data_ptr() for nm in launch["arg_order"]]
    with PtxModule((GOLDEN / f"{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(case), ptrs, launch["grid"][0], launch["block"][0])
        m.synchronize()
    assert torch.equal(theirs, dev["out"])


def test_concatenation_in_two_kernels(cuda):
    """torch.cat([a, b], -1) (shapes.py:13) as two kernels over one output, each writing its slice through an output map."""
    import torch
    out = torch.zeros(32, 112, device=cuda)
    host = {}
    for case in ("s_cat_a", "s_cat_b"):
        g, k, launch = ir.layout_kernel(case)
        handle = json.loads(compile_kernel(g, k, launch))
        tensors = {t.name: {"shape": [d.as_static() for d in t.shape]} for nd in g.nodes.values() for t in nd.outputs}
        h = inputs.layout_buffers(tensors, launch["arg_order"])
        src = launch["arg_order"][0]
        host[src] = h[src]
        run_local.launch(handle, {src: torch.from_numpy(h[src]).to(cuda), "out": out})
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), np.concatenate([host["A"], host["B"]], -1))


def test_indexed_programs_directly(cuda):
    """Other dtypes, negative strides, an integer program with an axis digit as a value, index ranges checked."""
    import torch
    from emmyptx import runtime as rt
    S = rt.PW_MAX_SLOTS
    x = torch.randn(40, 24, device=cuda).to(torch.bfloat16)
    out = torch.zeros(24, 40, dtype=torch.float16, device=cuda)
    prog = {"in_dtypes": ["bf16"], "out_dtype": "f16", "out_slot": 4, "consts": [0.5], "steps": [["multiply", 4, 0, S, 0]]}
    imap = {"extents": [24, 40], "inputs": [{"offset": 39 * 24, "coef": [1, -24]}], "out": {"offset": 0, "coef": [40, 1]}}   # transpose + flip
    rt.pointwise_indexed(prog, imap, [x.reshape(-1)], out.reshape(-1))
    want = (x.float().flip(0).t() * 0.5).to(torch.float16)
    assert torch.equal(out, want)
    a = torch.arange(4 * 5 * 6, dtype=torch.int32, device=cuda)
    oi = torch.zeros(4 * 5 * 6, dtype=torch.int64, device=cuda)
    progi = {"in_dtypes": ["i32", "i32"], "out_dtype": "i64", "out_slot": 4, "consts": [100], "steps": [["multiply", 4, 1, S, 0], ["add", 4, 4, 0, 0]]}
    imapi = {"extents": [4, 5, 6], "inputs": [{"offset": 119, "coef": [-30, -6, -1]}, {"axis": 1}], "out": {"offset": 0, "coef": [30, 6, 1]}}
    rt.pointwise_indexed(progi, imapi, [a, None], oi)
    i = np.arange(120)
    assert np.array_equal(oi.cpu().numpy(), (119 - i) + 100 * ((i // 6) % 5))
    with pytest.raises(IndexError, match="input 0"):
        rt.pointwise_indexed(prog, dict(imap, inputs=[{"offset": 39 * 24 + 1, "coef": [1, -24]}]), [x.reshape(-1)], out.reshape(-1))
    with pytest.raises(IndexError, match="output"):
        rt.pointwise_indexed(prog, dict(imap, out={"offset": 1, "coef": [40, 1]}), [x.reshape(-1)], out.reshape(-1))
    m = rt.make_index_map(dict(imap, inputs=[{"offset": 0, "coef": [1, -24]}]))           # reaches a negative element: refused by the C entry too
    arr = (__import__("ctypes").c_void_p * 1)(x.data_ptr())
    p = rt.make_program(prog)
    import ctypes
    assert rt.library().emmyb200_pointwise_indexed(ctypes.byref(p), ctypes.byref(m), arr, out.data_ptr(), None) == -2
    assert rt.device_status() == 0


def test_large_transpose(cuda):
    """A transpose well beyond the reference's case: 4096 x 2048 floats, against torch."""
    import torch
    from emmyptx import runtime as rt
    x = torch.randn(4096, 2048, device=cuda)
    out = torch.empty(2048, 4096, device=cuda)
    prog = {"in_dtypes": ["f32"], "out_dtype": "f32", "out_slot": 0, "consts": [], "steps": []}
    rt.pointwise_indexed(prog, {"extents": [2048, 4096], "inputs": [{"offset": 0, "coef": [1, 2048]}], "out": {"offset": 0, "coef": [4096, 1]}},
                         [x.reshape(-1)], out.reshape(-1))
    assert torch.equal(out, x.t().contiguous())


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_batched_transposition_through_shared_memory_tiles(dtype, cuda):
    """out[b, i, j] = x[b, j, i] * (j <= i), ragged 32 x 32 tiles, a batch axis in front, an axis digit as a value: the tiled
    form of the indexed kernel (one buffer input contiguous along another axis than the innermost)."""
    import torch
    from emmyptx import runtime as rt
    S = rt.PW_MAX_SLOTS
    td = torch.float32 if dtype == "f32" else torch.bfloat16
    b, rows, cols = 3, 70, 45                                   # x: [b, cols, rows] -> out: [b, rows, cols]
    x = torch.randn(b, cols, rows, device=cuda).to(td)
    out = torch.full((b, rows, cols), 7.0, device=cuda, dtype=td)
    prog = {"in_dtypes": [dtype, "f32", "f32"], "out_dtype": dtype, "out_slot": 5, "consts": [0.0],
            "steps": [["less_equal", 4, 2, 1, 0], ["where", 5, 4, 0, S]]}
    imap = {"extents": [b, rows, cols], "inputs": [{"offset": 0, "coef": [cols * rows, 1, rows]}, {"axis": 1}, {"axis": 2}],
            "out": {"offset": 0, "coef": [rows * cols, cols, 1]}}
    rt.pointwise_indexed(prog, imap, [x.reshape(-1), None, None], out.reshape(-1))
    i = torch.arange(rows, device=cuda)[:, None]
    j = torch.arange(cols, device=cuda)[None, :]
    want = torch.where(j <= i, x.transpose(1, 2), torch.zeros((), device=cuda, dtype=td))
    assert torch.equal(out, want)
    # reversed along the transposed axis as well: a negative coefficient on the innermost axis
    imap["inputs"][0] = {"offset": (cols - 1) * rows, "coef": [cols * rows, 1, -rows]}
    rt.pointwise_indexed(prog, imap, [x.reshape(-1), None, None], out.reshape(-1))
    assert torch.equal(out, torch.where(j <= i, x.flip(1).transpose(1, 2), torch.zeros((), device=cuda, dtype=td)))


def test_rotation_and_data_dependent_rows_directly(cuda):
    """A rotation along two axes at once; an embedding with int32 indices of either sign into a bf16 table with a scale in
    the program; the range check on the largest row the modulus allows."""
    import torch
    from emmyptx import runtime as rt
    S = rt.PW_MAX_SLOTS
    x = torch.randn(37, 50, device=cuda)
    out = torch.zeros_like(x)
    ident = {"in_dtypes": ["f32"], "out_dtype": "f32", "out_slot": 0, "consts": [], "steps": []}
    rt.pointwise_indexed(ident, {"extents": [37, 50], "inputs": [{"offset": 0, "coef": [50, 1], "rot": [37 - 5, 50 - 7]}], "out": {"offset": 0, "coef": [50, 1]}},
                         [x.reshape(-1)], out.reshape(-1))
    assert torch.equal(out, torch.roll(x, (5, 7), (0, 1)))
    table = torch.randn(300, 48, device=cuda).to(torch.bfloat16)
    idx = torch.randint(-5000, 5000, (1000,), device=cuda, dtype=torch.int32)
    emb = torch.zeros(1000, 48, device=cuda, dtype=torch.bfloat16)
    prog = {"in_dtypes": ["bf16", "i32"], "out_dtype": "bf16", "out_slot": 4, "consts": [2.0], "steps": [["multiply", 4, 0, S, 0]]}
    imap = {"extents": [1000, 48], "inputs": [{"offset": 0, "coef": [0, 1], "index_of": 1, "index_mult": 48}, {"offset": 0, "coef": [1, 0], "index_mod": 300}],
            "out": {"offset": 0, "coef": [48, 1]}}
    rt.pointwise_indexed(prog, imap, [table.reshape(-1), idx], emb.reshape(-1))
    rows = torch.remainder(idx.long(), 300)                     # the non-negative remainder, no abs
    assert torch.equal(emb, (table[rows].float() * 2).to(torch.bfloat16))
    with pytest.raises(IndexError, match="input 0"):
        rt.pointwise_indexed(prog, dict(imap, inputs=[imap["inputs"][0], {"offset": 0, "coef": [1, 0], "index_mod": 301}]), [table.reshape(-1), idx], emb.reshape(-1))
    assert rt.device_status() == 0


@pytest.mark.parametrize("shape", [(96, 64), (100, 70), (257, 130), (64, 4096), (3, 65, 200), (2, 129, 64)])
def test_transpositions_either_way(shape, cuda):
    """The shared-memory tiled form with the tile laid out in output order (strided reads) and in input order (strided
    writes), 32- and 64-wide tiles, ragged edges, a leading batch axis, f32 and bf16, against torch's transpose."""
    import torch
    from emmyptx import runtime as rt
    *lead, r, c = shape
    b = lead[0] if lead else 1
    for dt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        x = torch.randn(b, r, c, device=cuda).to(dt)
        want = x.transpose(1, 2).contiguous()
        prog = {"in_dtypes": [name], "out_dtype": name, "out_slot": 0, "consts": [], "steps": []}
        # cells in output order [b, c, r]: the input is read with stride c along the innermost axis
        out = torch.zeros(b, c, r, device=cuda, dtype=dt)
        m = {"extents": [b, c, r], "inputs": [{"offset": 0, "coef": [r * c, 1, c]}], "out": {"offset": 0, "coef": [r * c, r, 1]}}
        rt.pointwise_indexed(prog, m, [x.reshape(-1)], out.reshape(-1))
        assert torch.equal(out, want)
        # cells in input order [b, r, c]: the output is written with stride r along the innermost axis
        out2 = torch.zeros(b, c, r, device=cuda, dtype=dt)
        m2 = {"extents": [b, r, c], "inputs": [{"offset": 0, "coef": [r * c, c, 1]}], "out": {"offset": 0, "coef": [r * c, 1, r]}}
        rt.pointwise_indexed(prog, m2, [x.reshape(-1)], out2.reshape(-1))
        assert torch.equal(out2, want)
    # a program on the way: 2 x + 1 while transposing, cells in input order
    x = torch.randn(r, c, device=cuda)
    S = rt.PW_MAX_SLOTS
    prog = {"in_dtypes": ["f32"], "out_dtype": "f32", "out_slot": 2, "consts": [2.0, 1.0], "steps": [["multiply", 1, 0, S, 0], ["add", 2, 1, S + 1, 0]]}
    out = torch.zeros(c, r, device=cuda)
    rt.pointwise_indexed(prog, {"extents": [r, c], "inputs": [{"offset": 0, "coef": [c, 1]}], "out": {"offset": 0, "coef": [1, r]}}, [x.reshape(-1)], out.reshape(-1))
    assert torch.equal(out, (x * 2 + 1).t().contiguous())

