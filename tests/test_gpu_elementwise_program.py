"""The general elementwise kernel on the reference's own pointwise and dtype cases
(tools/torch_cases/pointwise.py:8-57, dtypes.py:5-12): each case is written once as Kernel IR (what the tracer would
hand over: Loads, a chain of Assigns through the op table, a Write) and once as the torch expression the reference's
checker evaluates in float64 on the same seeded inputs. Tolerances are the reference's classes
(tools/torch_cases/__init__.py:17-21): ROUND 1e-6, TRANS 1e-5, HALF 1e-2.
"""
import json

import numpy as np
import pytest

from emmyptx import ir, run_local
from emmyptx.kernel import compile_kernel

pytestmark = pytest.mark.gpu
ROUND, TRANS, HALF = 1e-6, 1e-5, 1e-2


@pytest.fixture(autouse=True, params=["compiled", "interpreter"])
def program_form(request):
    """Every case runs twice: as the kernel compiled for the program at first use, and on the interpreter kernel."""
    from emmyptx import runtime
    before = runtime.set_pointwise_jit(request.param == "compiled")
    if request.param == "compiled":
        assert runtime.pointwise_jit_state()[0] == 1, "the run-time compiler was not found: float programs would silently run interpreted"
    yield request.param
    runtime.set_pointwise_jit(before)

from elementwise_cases import BCAST_CASES, BCAST_SHAPE, BOOL_IN, CASES, INT_CASES, OUT_DTYPE  # noqa: E402  (the cases as data, shared with the fixture generator)


def _expected(expr, arrays):
    import torch
    import torch.nn.functional as F
    scope = {"torch": torch, "F": F, **{k: torch.from_numpy(np.asarray(v, dtype=np.float64)) for k, v in arrays.items()}}
    return eval(expr, scope).numpy()


@pytest.mark.parametrize("case", sorted(CASES))
@pytest.mark.parametrize("n", [4096, 4099])
def test_reference_pointwise_cases(case, n, cuda):
    from oracle import reference
    inputs, steps, expr, tol = CASES[case]
    out_dtype = OUT_DTYPE.get(case, "f32")
    built = ir.elementwise_kernel(n, inputs, steps, out_dtype, name=case)
    text = compile_kernel(*built)
    args = [{"name": b, "dtype": dt, "shape": [n], "seed": i} for i, (b, dt) in enumerate(inputs.items())]
    args.append({"name": "out", "dtype": out_dtype, "shape": [n], "output": True})
    run_local.init()
    got = run_local.run_kernel(text, dict(built[2], args=args), {})["out"]
    # graph input i is default_rng(i).standard_normal rounded to the buffer's dtype (tools/run_local.py:86-87)
    arrays = {}
    for i, (b, dt) in enumerate(inputs.items()):
        host = run_local.to_device(np.random.default_rng(i).standard_normal([n]), dt)
        arrays[b] = run_local.from_device(host, dt).astype(np.float64)
    ref = _expected(expr, arrays)
    rtol, atol = tol if isinstance(tol, tuple) else (tol, tol)
    res = reference.compare(np.asarray(got, dtype=np.float64), ref, rtol, atol)
    assert res["ok"], (case, res)


@pytest.mark.parametrize("case", sorted(CASES))
def test_reference_kernel_for_the_same_ir(case, cuda, program_form):
    """Kernel against kernel: the reference compiler's PTX for the same elementwise IR (tests/golden/ew_<case>.ref.ptx,
    one thread per element) JIT-loaded on this GPU and run on the same device buffers. Both results sit inside the
    reference's class of the float64 expression, and they agree with each other inside it."""
    import torch
    from pathlib import Path
    from emmyptx.ptx_driver import PtxModule
    from oracle import reference
    if program_form != "compiled":
        pytest.skip("one comparison per case is enough")
    golden = Path(__file__).resolve().parent / "golden"
    manifest = json.loads((golden / "reference_ptx_manifest.json").read_text())[f"ew_{case}"]
    inputs, steps, expr, tol = CASES[case]
    out_dtype = OUT_DTYPE.get(case, "f32")
    n = 4096
    built = ir.elementwise_kernel(n, inputs, steps, out_dtype, name=f"ew_{case}")
    assert built[2] == manifest["launch"]                                # the fixture was made from this IR
    handle = json.loads(compile_kernel(*built))
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "bool": torch.bool}
    dev, arrays = {}, {}
    for i, (b, dt) in enumerate(inputs.items()):
        host = run_local.to_device(np.random.default_rng(i).standard_normal([n]), dt)
        arrays[b] = run_local.from_device(host, dt).astype(np.float64)
        t = torch.from_numpy(np.ascontiguousarray(host))
        dev[b] = (t.view(torch.bfloat16) if dt == "bf16" else t).to(cuda)
    ours = torch.zeros(n, dtype=tdt[out_dtype], device=cuda)
    theirs = torch.zeros(n, dtype=tdt[out_dtype], device=cuda)
    run_local.init()
    run_local.launch(handle, dict(dev, out=ours))
    launch = built[2]
    with PtxModule((golden / f"ew_{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(f"ew_{case}"), [dev[nm].data_ptr() if nm != "out" else theirs.data_ptr() for nm in launch["arg_order"]],
                 launch["grid"][0], launch["block"][0])
        m.synchronize()
    torch.cuda.synchronize()
    ref = _expected(expr, arrays)
    rtol, atol = tol if isinstance(tol, tuple) else (tol, tol)
    o, t = ours.double().cpu().numpy(), theirs.double().cpu().numpy()
    assert reference.compare(o, ref, rtol, atol)["ok"]
    res = reference.compare(t, ref, rtol, atol)
    assert res["ok"], ("the reference's kernel against float64", case, res)
    res = reference.compare(o, t, 2 * rtol, 2 * atol)
    assert res["ok"], ("kernel against kernel", case, res)


def test_program_limits_are_compile_errors():
    from emmyptx.kernel import CompileError
    steps = [(f"v{i}", "add", ["x" if i == 0 else f"v{i-1}", float(i)]) for i in range(20)]            # 20 distinct constants
    with pytest.raises(CompileError, match="constants"):
        compile_kernel(*ir.elementwise_kernel(64, {"x": "f32"}, steps))
    many = {f"x{i}": "f32" for i in range(5)}
    with pytest.raises(CompileError, match="input buffers"):
        compile_kernel(*ir.elementwise_kernel(64, many, [("a", "add", ["x0", "x1"])]))
    h = json.loads(compile_kernel(*ir.elementwise_kernel(64, {"x": "f32"}, [(f"v{i}", "add", ["x" if i == 0 else f"v{i-1}", 1.0]) for i in range(40)])))
    assert h["variant"] == "pointwise_program" and len(h["params"]["program"]["steps"]) == 40
    assert max(s[1] for s in h["params"]["program"]["steps"]) < 16           # slots are recycled


# ---- integer programs and bool inputs (tools/torch_cases/dtypes.py:11-16) -----------------------------------------
def _int_kernel(n, steps, in_dt="i32", out_dt="i32", ins=("a",)):
    return ir.int_elementwise_kernel(n, steps, in_dt, out_dt, ins)


def _run_built(built, arrays, out_dtype, n, **kw):
    import torch
    from emmyptx.kernel import KernelCompiler
    g, k, launch = built
    handle = json.loads(KernelCompiler(g, k, launch, **kw).compile())
    assert handle["variant"] == "pointwise_program"
    run_local.init()
    dev = torch.device("cuda:0")
    bufs = {name: torch.from_numpy(a).to(dev) for name, a in arrays.items()}
    bufs["out"] = torch.zeros(n, dtype=out_dtype, device=dev)
    run_local.launch(handle, bufs)
    torch.cuda.synchronize()
    return bufs["out"].cpu().numpy()


@pytest.mark.parametrize("n", [1024, 4099])
def test_integer_cases_are_bit_exact(n, cuda):
    import torch
    rng = np.random.default_rng(n)
    a = rng.integers(-8, 8, n).astype(np.int32)
    got = _run_built(_int_kernel(n, [("t", "multiply", ["a", 3]), ("u", "add", ["t", 1])]), {"a": a}, torch.int32, n)
    assert np.array_equal(got, a * 3 + 1)                                                           # d_i32_arith
    steps = [("q", "floor_divide", ["a", 3]), ("r", "mod", ["a", 3]), ("s", "multiply", ["r", 100]), ("u", "add", ["q", "s"])]
    got = _run_built(_int_kernel(n, steps), {"a": a}, torch.int32, n)
    assert np.array_equal(got, a // 3 + (a % 3) * 100)                                              # d_i32_floordiv_mod (torch floors)
    got = _run_built(_int_kernel(n, steps), {"a": a}, torch.int32, n, int_div="trunc")              # the reference's div.s32 / rem.s32
    q = np.trunc(a / 3).astype(np.int32)
    assert np.array_equal(got, q + (a - 3 * q) * 100)
    a64 = rng.integers(-4, 4, n).astype(np.int64)
    got = _run_built(_int_kernel(n, [("t", "multiply", ["a", 3]), ("u", "add", ["t", 1])], "i64", "i64"), {"a": a64}, torch.int64, n)
    assert np.array_equal(got, a64 * 3 + 1)                                                         # d_i64_arith


def test_integer_ops_wrap_and_shift_as_s32(cuda):
    import torch
    n = 2048
    rng = np.random.default_rng(3)
    a = rng.integers(-2**31, 2**31, n).astype(np.int32)
    b = rng.integers(-2**31, 2**31, n).astype(np.int32)
    a[:4] = [np.iinfo(np.int32).min, np.iinfo(np.int32).max, -1, 0]
    steps = [("m", "multiply", ["a", "b"]), ("x", "bitwise_xor", ["m", "a"]), ("s", "right_shift", ["x", 3]), ("t", "left_shift", ["b", 5]),
             ("o", "bitwise_or", ["s", "t"]), ("n", "bitwise_and", ["o", 16777215]), ("d", "subtract", ["n", "a"]), ("z", "maximum", ["d", "b"])]
    got = _run_built(_int_kernel(n, steps, ins=("a", "b")), {"a": a, "b": b}, torch.int32, n)
    a64, b64 = a.astype(np.int64), b.astype(np.int64)
    wrap = lambda v: ((v + 2**31) % 2**32 - 2**31)
    m = wrap(a64 * b64)
    x = m ^ a64
    o = (x >> 3) | wrap(b64 << 5)
    d = wrap((o & 16777215) - a64)
    assert np.array_equal(got, np.maximum(d, b64).astype(np.int32))


@pytest.mark.parametrize("n", [1024, 4099])
def test_bool_mask_input(n, cuda):
    """d_bool_in: torch.where(m, x, -x) with a bool buffer as a graph input."""
    import torch
    rng = np.random.default_rng(1)
    x = rng.standard_normal(n).astype(np.float32)
    m = rng.standard_normal(n) > 0
    built = ir.elementwise_kernel(n, {"x": "f32", "m": "bool"}, [("nx", "negative", ["x"]), ("y", "where", ["m", "x", "nx"])])
    got = _run_built(built, {"x": x, "m": m}, torch.float32, n)
    assert np.array_equal(got, np.where(m, x, -x))


@pytest.mark.parametrize("case", sorted(INT_CASES) + ["d_bool_in"])
def test_integer_and_bool_input_kernels_against_the_reference_kernel(case, cuda, program_form):
    """The reference's PTX for the same integer IR (div.s32 / rem.s32: truncating `//` and `%`, which `int_div="trunc"`
    reproduces) and for the bool-input program, on the same device buffers: bit for bit."""
    import torch
    from pathlib import Path
    from emmyptx.kernel import KernelCompiler
    from emmyptx.ptx_driver import PtxModule
    if program_form != "compiled":
        pytest.skip("one comparison per case is enough")
    golden = Path(__file__).resolve().parent / "golden"
    n = 4096
    rng = np.random.default_rng(5)
    if case == "d_bool_in":
        built = ir.elementwise_kernel(n, *BOOL_IN, name="ew_d_bool_in")
        host = {"x": rng.standard_normal(n).astype(np.float32), "m": rng.standard_normal(n) > 0}
        out_dt = torch.float32
    else:
        steps, in_dt, out_dt_name, ins = INT_CASES[case]
        built = ir.int_elementwise_kernel(n, steps, in_dt, out_dt_name, ins, name=f"ew_{case}")
        npdt = np.int64 if in_dt == "i64" else np.int32
        lo, hi = (-2**31, 2**31) if case == "int_wrap_shift" else (-8, 8)
        host = {b: rng.integers(lo, hi, n).astype(npdt) for b in ins}
        out_dt = torch.int64 if out_dt_name == "i64" else torch.int32
    manifest = json.loads((golden / "reference_ptx_manifest.json").read_text())[f"ew_{case}"]
    assert built[2] == manifest["launch"]
    handle = json.loads(KernelCompiler(*built, int_div="trunc").compile())
    dev = {b: torch.from_numpy(a).to(cuda) for b, a in host.items()}
    ours, theirs = torch.zeros(n, dtype=out_dt, device=cuda), torch.zeros(n, dtype=out_dt, device=cuda)
    run_local.init()
    run_local.launch(handle, dict(dev, out=ours))
    launch = built[2]
    with PtxModule((golden / f"ew_{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(f"ew_{case}"), [dev[nm].data_ptr() if nm != "out" else theirs.data_ptr() for nm in launch["arg_order"]],
                 launch["grid"][0], launch["block"][0])
        m.synchronize()
    torch.cuda.synchronize()
    assert torch.equal(ours, theirs)


# ---- broadcast inputs (f_batch_norm_eval, m_outer, s_expand: tools/torch_cases/fused.py:18-20, matmul.py:23, shapes.py) ----
def _tile2(rows, cols, loads, steps, ins, out_shape):
    assert list(out_shape) == [rows, cols]
    return ir.broadcast_kernel(rows, cols, loads, steps, ins)


@pytest.mark.parametrize("case", sorted(BCAST_CASES))
def test_broadcast_kernels_against_the_reference_kernel(case, cuda, program_form):
    """The reference's PTX for the same broadcast IR on the same device buffers. Ours equals numpy bit for bit (every
    operation rounded on its own, as torch evaluates the expression); the reference's kernel agrees bit for bit where there
    is one operation per element, and to one rounding (1e-6) where a multiply feeds an add: the driver's JIT contracts
    those two of its PTX into a fused multiply-add."""
    import torch
    from pathlib import Path
    from emmyptx.ptx_driver import PtxModule
    if program_form != "compiled":
        pytest.skip("one comparison per case is enough")
    golden = Path(__file__).resolve().parent / "golden"
    loads, steps, ins, expr = BCAST_CASES[case]
    rows, cols = BCAST_SHAPE
    built = ir.broadcast_kernel(rows, cols, loads, steps, ins, name=f"bc_{case}")
    manifest = json.loads((golden / "reference_ptx_manifest.json").read_text())[f"bc_{case}"]
    assert built[2] == manifest["launch"]
    handle = json.loads(compile_kernel(*built))
    assert handle["variant"] == "pointwise_program"
    host = {nm: np.random.default_rng(i).standard_normal(shp).astype(np.float32) for i, (nm, shp) in enumerate(ins.items())}
    dev = {nm: torch.from_numpy(a).to(cuda) for nm, a in host.items()}
    ours, theirs = torch.zeros(rows, cols, device=cuda), torch.zeros(rows, cols, device=cuda)
    run_local.init()
    run_local.launch(handle, dict(dev, out=ours))
    launch = built[2]
    with PtxModule((golden / f"bc_{case}.ref.ptx").read_text()) as m:
        m.launch(m.function(f"bc_{case}"), [dev[nm].data_ptr() if nm != "out" else theirs.data_ptr() for nm in launch["arg_order"]],
                 launch["grid"][0], launch["block"][0])
        m.synchronize()
    torch.cuda.synchronize()
    if [st[1] for st in steps][-2:] == ["multiply", "add"]:
        assert torch.allclose(ours, theirs, rtol=1e-6, atol=1e-6)
    else:
        assert torch.equal(ours, theirs)
    assert np.array_equal(ours.cpu().numpy(), eval(expr, {"np": np, **host}).astype(np.float32))


@pytest.mark.parametrize("rows,cols", [(32, 64), (33, 61), (67, 1032)])
def test_broadcast_inputs(rows, cols, cuda):
    import torch
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    m, w, b = (rng.standard_normal(cols).astype(np.float32) for _ in range(3))
    # batch norm in eval mode with the per-channel scale folded: (x - m) * w + b, three row vectors over a matrix
    built = _tile2(rows, cols, [("x", "X", ("r0", "c0")), ("m", "M", ("c0",)), ("w", "W", ("c0",)), ("b", "B", ("c0",))],
                   [("d", "subtract", ["x", "m"]), ("s", "multiply", ["d", "w"]), ("o", "add", ["s", "b"])],
                   {"X": [rows, cols], "M": [cols], "W": [cols], "B": [cols]}, [rows, cols])
    got = _run_built(built, {"X": x.reshape(-1), "M": m, "W": w, "B": b}, torch.float32, rows * cols)
    assert np.array_equal(got.reshape(rows, cols), (x - m) * w + b)
    # outer product: a column vector and a row vector
    a, v = rng.standard_normal(rows).astype(np.float32), rng.standard_normal(cols).astype(np.float32)
    built = _tile2(rows, cols, [("a", "A", ("r0",)), ("v", "V", ("c0",))], [("o", "multiply", ["a", "v"])], {"A": [rows], "V": [cols]}, [rows, cols])
    got = _run_built(built, {"A": a, "V": v}, torch.float32, rows * cols)
    assert np.array_equal(got.reshape(rows, cols), np.outer(a, v))
    # p_bcast_rowcol (tools/torch_cases/pointwise.py:56): a matrix times a row vector plus a column vector
    built = _tile2(rows, cols, [("x", "X", ("r0", "c0")), ("r", "R", ("c0",)), ("c", "C", ("r0",))], [("p", "multiply", ["x", "r"]), ("o", "add", ["p", "c"])],
                   {"X": [rows, cols], "R": [cols], "C": [rows]}, [rows, cols])
    got = _run_built(built, {"X": x.reshape(-1), "R": v, "C": a}, torch.float32, rows * cols)
    assert np.array_equal(got.reshape(rows, cols), x * v + a[:, None])
    # s_reshape (shapes.py:10): a flat buffer read as a matrix -- the same element order, so an ordinary streaming program
    built = _tile2(rows, cols, [("x", "X", ("r0", "c0"))], [("o", "add", ["x", 1.0])], {"X": [rows, cols]}, [rows, cols])
    got = _run_built(built, {"X": x.reshape(-1)}, torch.float32, rows * cols)
    assert np.array_equal(got, x.reshape(-1) + np.float32(1))
    # s_expand (shapes.py:19): one row repeated
    built = _tile2(rows, cols, [("v", "V", ("c0",))], [("o", "add", ["v", 0.0])], {"V": [cols]}, [rows, cols])
    got = _run_built(built, {"V": v}, torch.float32, rows * cols)
    assert np.array_equal(got.reshape(rows, cols), np.broadcast_to(v, (rows, cols)))


def test_compiled_and_interpreted_forms_agree_bit_for_bit(cuda):
    """One program through every float op of the table, on values that include zeros, infinities, NaN and subnormals;
    f32 / f16 / bf16 / bool inputs, aligned and unaligned views, ragged lengths. The two forms must give the same bits."""
    import torch
    from emmyptx import runtime as rt
    S = rt.PW_MAX_SLOTS
    unary = ["relu", "square", "copy", "negative", "abs", "reciprocal", "sqrt", "rsqrt", "exp", "log", "sigmoid", "tanh", "erf", "sin", "cos", "bitwise_not"]
    binary = ["add", "subtract", "multiply", "divide", "maximum", "minimum", "pow", "equal", "not_equal", "greater", "less", "greater_equal",
              "less_equal", "bitwise_and", "bitwise_or", "floor_divide", "mod"]
    g = torch.Generator(device="cpu").manual_seed(5)
    special = torch.tensor([0.0, -0.0, 1.0, -1.0, float("inf"), -float("inf"), float("nan"), 1e-40, -1e-40, 88.0, -104.0, 1e5, 3.4e38, 0.5])
    for n in (4096, 4099, 3):
        x = torch.randn(n + 4, generator=g) * 3
        x[1:1 + min(n, len(special))] = special[:min(n, len(special))]
        y = torch.randn(n + 4, generator=g)
        xs = {"f32": x.cuda(), "f16": x.half().cuda(), "bf16": x.bfloat16().cuda()}
        ys = {"f32": y.cuda(), "f16": y.half().cuda(), "bf16": y.bfloat16().cuda()}
        mask = (torch.randn(n + 4, generator=g) > 0).cuda()
        for off in (0, 1, 4):           # 128-bit accesses everywhere; none; 64-bit ones for the 16-bit buffers
            for dt_in, dt_out in (("f32", "f32"), ("f16", "bf16"), ("bf16", "f16"), ("f32", "f16")):
                tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dt_out]
                for ops, arity in ((unary, 1), (binary, 2)):
                    for op in ops:
                        prog = {"in_dtypes": [dt_in, dt_in, "bool"], "out_dtype": dt_out, "out_slot": 5, "consts": [0.75],
                                "steps": [[op, 4, 0, 1 if arity == 2 else 0, 0], ["where", 5, 2, 4, S + 0]]}
                        ins = [xs[dt_in][off:off + n], ys[dt_in][off:off + n], mask[off:off + n]]
                        outs = []
                        for compiled in (True, False):
                            rt.set_pointwise_jit(compiled)
                            out = torch.full((n + 8,), 7.0, dtype=tdt, device="cuda")
                            rt.pointwise_program(prog, ins, out[off:off + n])
                            outs.append(out.cpu())
                        # same bits, except that a NaN need only be a NaN in both (its sign and payload are not specified)
                        nan = [o.float().isnan() for o in outs]
                        assert torch.equal(nan[0], nan[1]), (op, n, off, dt_in, dt_out)
                        a, b = (o.view(torch.int16 if tdt != torch.float32 else torch.int32)[~nan[0]] for o in outs)
                        assert torch.equal(a, b), (op, n, off, dt_in, dt_out)


def test_constants_and_extents_do_not_compile_again(cuda, program_form):
    import torch
    from emmyptx import runtime as rt
    if program_form != "compiled":
        pytest.skip("only the compiled form has a cache")
    S = rt.PW_MAX_SLOTS
    x = torch.randn(5000, device="cuda")
    prog = {"in_dtypes": ["f32"], "out_dtype": "f32", "out_slot": 4, "consts": [1.5, -2.0], "steps": [["multiply", 4, 0, S, 0], ["add", 4, 4, S + 1, 0], ["tanh", 4, 4, 0, 0]]}
    out = torch.empty_like(x)
    rt.pointwise_program(prog, [x], out)
    compiled = rt.pointwise_jit_state()[1]
    for c in (0.25, 3.0):
        prog["consts"] = [c, 1.0]
        rt.pointwise_program(prog, [x], out)
        assert torch.allclose(out, torch.tanh(x * c + 1.0), atol=1e-6)
    rt.pointwise_program(prog, [x[:4096]], out[:4096])
    assert rt.pointwise_jit_state()[1] == compiled
