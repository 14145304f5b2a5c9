"""The kernel-builder API (compile.py, emmyptx.kernel) on CPU: which IR matches which kernel variant.

Mirrors how the reference is driven (compile.py:34-57; tools/check_torch.py:289 runs it as a subprocess on
<entry>.ir.json next to meta.json) with the artefact being a kernel handle instead of PTX.
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from emmyptx import ir
from emmyptx.kernel import CompileError, KernelCompiler, algorithmic_work, compile_kernel

ROOT = Path(__file__).resolve().parent.parent
COMPILE = ROOT / "emmy-ptx-compiler_b200" / "compile.py"


def handle(built, **kw):
    g, k, launch = built
    return json.loads(KernelCompiler(g, k, launch, **kw).compile() if kw else compile_kernel(g, k, launch))


def test_the_five_configurations_match_their_kernels():
    h = handle(ir.pointwise_kernel(2**20))
    assert (h["variant"], h["params"]) == ("pointwise_f32", {"op": "exp_sin_tanh", "n": 2**20})
    assert algorithmic_work(h) == (8.0 * 2**20, "B")
    h = handle(ir.index_gather_kernel(2**26))
    assert h["variant"] == "index_gather_i32"
    assert h["params"] == {"n": 2**26, "mul": 7919, "add": 13, "div": 3, "shift": 2, "trunc": False}
    assert algorithmic_work(h) == (8.0 * 2**26, "B")
    h = handle(ir.gemm_kernel(4096, 4096, 4096, "f16"))
    assert h["params"] == {"dtype": "f16", "m": 4096, "n": 4096, "k": 4096, "b_trans": False, "epilogue": None}
    assert algorithmic_work(h) == (2.0 * 4096**3, "flop")
    h = handle(ir.gemm_kernel(16384, 16384, 16384, "bf16", "gelu_tanh"))
    assert h["params"]["epilogue"] == "gelu_tanh" and h["params"]["dtype"] == "bf16"
    h = handle(ir.attention_kernel([16, 16], 4096, 4096, 128))
    assert h["variant"] == "attention_fwd" and h["params"]["units"] == 256 and h["params"]["d"] == 128
    assert abs(h["params"]["scale"] - 128 ** -0.5) < 1e-12
    assert algorithmic_work(h) == (4.0 * 256 * 4096 * 4096 * 128, "flop")
    assert h["params"]["causal"] is False
    assert handle(ir.attention_kernel([2], 512, 512, 64, "f16", causal=True))["params"]["causal"] is True


def test_matching_is_by_meaning_not_by_spelling():
    """The same expression arranged differently (operands commuted, tanh's argument named differently, the
    modulus written as a mask) lands on the same variant."""
    g, k, launch = ir.pointwise_kernel(1024)
    body = k.body[0].body
    body[4].args = ["v3", "v2"]            # tanh * sin
    body[5].args = ["v4", "v1"]            # product + exp
    assert handle((g, k, launch))["params"]["op"] == "exp_sin_tanh"
    g, k, launch = ir.index_gather_kernel(2**12)
    k.body[0].body[0].index[0].op = "&"
    k.body[0].body[0].index[0].right = ir.Literal(2**12 - 1, "int")
    assert handle((g, k, launch))["params"]["mul"] == 7919 % 2**12     # only mul mod n is observable
    assert handle(ir.pointwise_kernel(512, "gelu_tanh"))["params"]["op"] == "gelu_tanh"


def test_gather_parameters_are_recovered():
    h = handle(ir.index_gather_kernel(10**6 + 3, mul=65537, add=12345, div=5, shift=4))
    assert h["params"] == {"n": 10**6 + 3, "mul": 65537, "add": 12345, "div": 5, "shift": 4, "trunc": False}
    assert handle(ir.index_gather_kernel(2**16), int_div="trunc")["params"]["trunc"] is True


def test_layout_flags_and_ragged_shapes():
    assert handle(ir.gemm_kernel(64, 512, 256, "f16", None, True))["params"]["b_trans"] is True       # m_f16_linear
    assert handle(ir.gemm_kernel(100, 72, 200, "f16"))["params"]["m"] == 100                           # m_f16_mm_odd


def test_unsupported_ir_is_a_compile_error():
    assert handle(ir.pointwise_kernel(100, "erf"))["variant"] == "pointwise_program"     # any op-table expression compiles
    g, k, launch = ir.pointwise_kernel(100, "exp")
    k.body[0].body.insert(1, ir.Loop(ir.Axis("r0", ir.Dim(4)), []))
    with pytest.raises(CompileError, match="no kernel variant"):
        handle((g, k, launch))
    g, k, launch = ir.pointwise_kernel(100, "exp")
    k.body[0].body[1].op = ir.Op("frobnicate")
    with pytest.raises(CompileError, match="not supported"):          # OpError surfaces as CompileError
        handle((g, k, launch))
    with pytest.raises(CompileError, match="sm_100a only"):
        KernelCompiler(*ir.pointwise_kernel(64), target="sm_89")
    with pytest.raises(CompileError, match="epilogue"):
        handle(ir.gemm_kernel(64, 64, 64, "f16", "swish"))
    with pytest.raises(CompileError, match="multiples of 8"):
        handle(ir.gemm_kernel(64, 60, 64, "f16"))
    g, k, launch = ir.gemm_kernel(64, 64, 64, "f16")
    k.body[0].body[3].body[2].c_dtype = "f16"
    with pytest.raises(CompileError, match="f32 accumulators"):
        handle((g, k, launch))
    g, k, launch = ir.pointwise_kernel(64)
    launch["arg_order"] = ["x", "z"]
    with pytest.raises(CompileError, match="arg_order"):
        handle((g, k, launch))
    g, k, launch = ir.pointwise_kernel(64)
    k.body[0].body.append(ir.Write("y", [ir.Var("a0")], ["v1"], atomic=True))
    with pytest.raises(CompileError, match="atomic"):
        handle((g, k, launch))


def test_compile_py_command_line(tmp_path):
    g, k, launch = ir.index_gather_kernel(2**16, name="k_idx")
    (tmp_path / "k_idx.ir.json").write_text(json.dumps(g.to_dict()))
    (tmp_path / "meta.json").write_text(json.dumps({"kernels": [dict(launch, args=[])]}))
    r = subprocess.run([sys.executable, str(COMPILE), str(tmp_path / "k_idx.ir.json")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    h = json.loads(r.stdout)
    assert h["entry"] == "k_idx" and h["variant"] == "index_gather_i32" and h["arg_order"] == ["x", "y"]
    r = subprocess.run([sys.executable, str(COMPILE), str(tmp_path / "k_idx.ir.json"), "--int-div", "trunc", "--level", "0"],
                       capture_output=True, text=True)
    assert json.loads(r.stdout)["params"]["trunc"] is True
    # without meta.json the launch is guessed from the graph (compile.py:21-31)
    (tmp_path / "meta.json").unlink()
    r = subprocess.run([sys.executable, str(COMPILE), str(tmp_path / "k_idx.ir.json")], capture_output=True, text=True)
    assert json.loads(r.stdout)["arg_order"] == ["x", "y"]
    # unsupported IR: non-zero exit, message on stderr, nothing on stdout
    g, k, launch = ir.pointwise_kernel(64, "frobnicate", name="k_erf")
    (tmp_path / "k_erf.ir.json").write_text(json.dumps(g.to_dict()))
    r = subprocess.run([sys.executable, str(COMPILE), str(tmp_path / "k_erf.ir.json")], capture_output=True, text=True)
    assert r.returncode != 0 and "compile error" in r.stderr and r.stdout == ""
    # two kernels in one file
    g2, k2, _ = ir.pointwise_kernel(64, "exp", name="k_exp")
    g.nodes["k_exp"] = g2.nodes["k_exp"]
    (tmp_path / "two.ir.json").write_text(json.dumps(g.to_dict()))
    r = subprocess.run([sys.executable, str(COMPILE), str(tmp_path / "two.ir.json")], capture_output=True, text=True)
    assert r.returncode != 0 and "expected one KernelOp" in r.stderr


def test_ir_json_round_trip():
    g, k, _ = ir.gemm_kernel(128, 256, 64, "bf16", "gelu_tanh")
    g2 = ir.Graph.from_dict(json.loads(json.dumps(g.to_dict())))
    assert g2.to_dict() == g.to_dict()
    assert type(g2.nodes["k_gemm"].op).__name__ == "KernelOp"


def test_row_reductions_are_matched_by_behaviour():
    """Every row op the builder can spell is recognised, with its extents and epsilon; a differently arranged program
    with the same meaning (mean as a division, the variance through E[x^2] - E[x]^2) matches the same kernel."""
    from emmyptx.ir import Accum, Assign, Axis, Dim, KernelOp, Load, Loop, Op, Tile, Var, Write, _graph, _launch, tensor
    for op in ("sum", "mean", "amax", "amin", "prod", "var", "std", "norm2", "logsumexp", "dot", "softmax", "log_softmax",
               "layer_norm", "rms_norm", "normalize"):
        h = handle(ir.rowwise_kernel(op, 48, 256, eps=1e-6))
        assert h["variant"] == "rowwise_f32" and h["params"]["op"] == op, op
        assert (h["params"]["rows"], h["params"]["cols"]) == (48, 256)
    assert handle(ir.rowwise_kernel("layer_norm", 8, 64, eps=1e-3))["params"]["eps"] == 1e-3
    assert handle(ir.rowwise_kernel("layer_norm", 8, 64))["inputs"] == ["X", "W", "B"]
    assert algorithmic_work(handle(ir.rowwise_kernel("softmax", 64, 1000))) == (8.0 * 64 * 1000, "B")

    # the same programs walking dim 0 instead of the last axis go to the column kernels
    for op in ("sum", "amax", "var", "logsumexp", "softmax", "normalize"):
        h = handle(ir.colwise_kernel(op, 256, 64))
        assert h["variant"] == "colwise_f32" and h["params"]["op"] == op, op
        assert (h["params"]["outer"], h["params"]["rows"], h["params"]["cols"]) == (1, 256, 64)

    rows, cols = 10, 96
    r0, c0 = Axis("r0", Dim(rows)), Axis("c0", Dim(cols))
    ld = Load(["x"], "X", [Var("r0"), Var("c0")])
    body = [Loop(c0, [ld, Accum("s1", None, "x", Op("add")), Assign("xx", Op("square"), ["x"]), Accum("s2", None, "xx", Op("add"))]),
            Assign("m", Op("divide"), ["s1", float(cols)]), Assign("mm", Op("multiply"), ["m", "s1"]),
            Assign("num", Op("subtract"), ["s2", "mm"]), Assign("v", Op("divide"), ["num", float(cols - 1)]),
            Write("Y", [Var("r0")], ["v"])]
    k = KernelOp("k_var2", [Tile([r0], body)])
    g = _graph(k, [tensor("X", [rows, cols], "f32")], [tensor("Y", [rows], "f32")])
    assert handle((g, k, _launch(k, ["X", "Y"], rows)))["params"]["op"] == "var"
    # a reduction the library does not have is refused, not approximated
    body = [Loop(c0, [ld, Assign("a", Op("abs"), ["x"]), Accum("s", None, "a", Op("add"))]), Write("Y", [Var("r0")], ["s"])]
    k = KernelOp("k_l1", [Tile([r0], body)])
    g = _graph(k, [tensor("X", [rows, cols], "f32")], [tensor("Y", [rows], "f32")])
    with pytest.raises(CompileError):
        handle((g, k, _launch(k, ["X", "Y"], rows)))


def test_float32_products_written_as_loops_match_the_split_precision_gemm():
    """m_mm, m_bmm, m_bcast_matmul, m_linear_bias (tools/torch_cases/matmul.py:10-14) as the scalar-loop IR."""
    h = handle(ir.matmul_f32_kernel(128, 80, 96))
    assert h["variant"] == "gemm_f32" and h["params"] == {"batch": 1, "m": 128, "n": 80, "k": 96, "b_trans": False, "b_shared": True,
                                                           "bias": False, "epilogue": None}
    assert algorithmic_work(h) == (2.0 * 128 * 80 * 96, "flop")
    assert handle(ir.matmul_f32_kernel(64, 48, 32, batch=4))["params"]["b_shared"] is False
    assert handle(ir.matmul_f32_kernel(64, 48, 32, batch=4, b_batched=False))["params"]["b_shared"] is True
    p = handle(ir.matmul_f32_kernel(64, 96, 128, b_trans=True, bias=True))
    assert p["params"]["b_trans"] and p["params"]["bias"] and p["inputs"] == ["A", "B", "bias"]
    assert handle(ir.matmul_f32_kernel(32, 256, 128, b_trans=True, bias=True, relu=True))["params"]["epilogue"] == "relu"


def test_integer_and_bool_programs_match_the_program_kernel():
    """d_i32_arith / d_i32_floordiv_mod / d_bool_in (tools/torch_cases/dtypes.py:11-16): integer-typed Assigns become an
    integer program (with the division mode of the compile), a bool buffer is a legal input of a float program, and
    a program mixing integer and float Assigns is refused."""
    from emmyptx.ir import Assign, Axis, DType, Dim, KernelOp, Load, Op, Tile, Var, Write, _graph, _launch, tensor

    def int_kernel(steps, mixed=False):
        a0 = Axis("a0", Dim(1024))
        body = [Load(["a"], "a", [Var("a0")])]
        body += [Assign(v, Op(op), list(args), None if (mixed and i == 0) else DType("int")) for i, (v, op, args) in enumerate(steps)]
        body.append(Write("out", [Var("a0")], [steps[-1][0]]))
        k = KernelOp("k_int", [Tile([a0], body)])
        return _graph(k, [tensor("a", [1024], "i32")], [tensor("out", [1024], "i32")]), k, _launch(k, ["a", "out"], 1024)

    steps = [("q", "floor_divide", ["a", 3]), ("r", "mod", ["a", 3]), ("s", "multiply", ["r", 100]), ("u", "add", ["q", "s"])]
    h = handle(int_kernel(steps))
    assert h["variant"] == "pointwise_program" and h["params"]["program"]["out_dtype"] == "i32"
    assert h["params"]["program"]["int_div"] == "floor" and len(h["params"]["program"]["steps"]) == 4
    assert handle(int_kernel(steps), int_div="trunc")["params"]["program"]["int_div"] == "trunc"
    assert algorithmic_work(h) == (8.0 * 1024, "B")
    with pytest.raises(CompileError):
        handle(int_kernel(steps, mixed=True))
    with pytest.raises(CompileError):
        handle(int_kernel([("t", "multiply", ["a", 2.5])]))                 # not a whole number
    h = handle(ir.elementwise_kernel(1024, {"x": "f32", "m": "bool"}, [("nx", "negative", ["x"]), ("y", "where", ["m", "x", "nx"])]))
    assert h["params"]["program"]["in_dtypes"] == ["f32", "bool"]


def test_broadcast_reads_become_program_inputs_with_an_index_map():
    """A row vector over a matrix (bias, batch-norm statistics), a column vector (outer product): the reads are matched as
    element (i // div) % mod of the smaller buffer; an index that is affine in the axis variables goes to the indexed kernel."""
    from emmyptx.ir import Assign, Axis, BinaryExpr, Dim, KernelOp, Literal, Load, Op, Tile, Var, Write, _graph, _launch, tensor
    r0, c0 = Axis("r0", Dim(64)), Axis("c0", Dim(96))

    def build(a_index, a_shape):
        body = [Load(["a"], "A", a_index), Load(["b"], "B", [Var("c0")]), Assign("o", Op("multiply"), ["a", "b"]),
                Write("Y", [Var("r0"), Var("c0")], ["o"])]
        k = KernelOp("k_outer", [Tile([r0, c0], body)])
        return _graph(k, [tensor("A", a_shape, "f32"), tensor("B", [96], "f32")], [tensor("Y", [64, 96], "f32")]), k, _launch(k, ["A", "B", "Y"], 64 * 96)

    prog = handle(build([Var("r0")], [64]))["params"]["program"]
    assert (prog["in_div"], prog["in_mod"]) == ([96, 0], [64, 96])
    assert algorithmic_work(handle(build([Var("r0")], [64]))) == (4.0 * (64 + 96 + 64 * 96), "B")
    h = handle(build([BinaryExpr("-", Literal(63, "int"), Var("r0"))], [64]))            # a reversed read is not a broadcast:
    assert h["variant"] == "pointwise_indexed"                                         # it is an affine index map
    assert {"buffer": "A", "offset": 63, "coef": [-1, 0]} in h["params"]["index_map"]["inputs"]


def test_relu_epilogue_is_read_from_the_ir_when_no_probed_value_is_negative():
    """Outputs so small that every probed pre-activation may be positive: the ReLU must not be dropped."""
    for m, n, k in [(1, 2, 16), (2, 2, 8), (64, 48, 32)]:
        assert handle(ir.matmul_f32_kernel(m, n, k, relu=True))["params"]["epilogue"] == "relu", (m, n, k)
        assert handle(ir.matmul_f32_kernel(m, n, k, relu=False))["params"]["epilogue"] is None, (m, n, k)
    # a ReLU spelled as maximum(x, 0) is the same epilogue
    g, k_, launch = ir.matmul_f32_kernel(1, 2, 16, relu=True)
    relu = next(s for s in k_.body[0].body if type(s).__name__ == "Assign" and s.op.name == "relu")
    relu.op, relu.args = ir.Op("maximum"), [relu.args[0], 0.0]
    assert handle((g, k_, launch))["params"]["epilogue"] == "relu"


def test_attention_mask_and_scale_are_checked_not_guessed():
    """Only key <= query is the causal variant; other masks, and an ambiguous scale, match nothing."""
    for mask in ("upper", "band", "padding"):
        with pytest.raises(CompileError, match="lower-triangular"):
            handle(ir.attention_kernel([2], 256, 256, 64, "f16", mask=mask))
    g, k, launch = ir.attention_kernel([2], 256, 256, 64, "f16")
    loop = next(s for s in k.body[0].body if type(s).__name__ == "Loop")
    at = next(i for i, s in enumerate(loop.body) if type(s).__name__ == "Assign" and s.op.name == "multiply")
    loop.body.insert(at + 1, ir.Assign("t0", ir.Op("multiply"), ["_s", 1.4426950408889634]))
    with pytest.raises(CompileError, match="ambiguous"):
        handle((g, k, launch))
    # a constant that multiplies something other than the scores is not the scale
    g, k, launch = ir.attention_kernel([2], 256, 256, 64, "f16", scale=0.2)
    loop = next(s for s in k.body[0].body if type(s).__name__ == "Loop")
    loop.body.append(ir.Assign("unused", ir.Op("multiply"), ["sm", 3.0]))
    assert handle((g, k, launch))["params"]["scale"] == 0.2
    # masked_fill form: where(mask, -inf, s) with mask = key > query
    g, k, launch = ir.attention_kernel([2], 256, 256, 64, "f16", causal=True)
    loop = next(s for s in k.body[0].body if type(s).__name__ == "Loop")
    cmp = next(s for s in loop.body if type(s).__name__ == "Assign" and s.name == "keep")
    fill = next(s for s in loop.body if type(s).__name__ == "Assign" and s.op.name == "where")
    cmp.op, fill.args = ir.Op("greater"), ["keep", float("-inf"), "t0"]
    assert handle((g, k, launch))["params"]["causal"] is True


def test_scalar_parameters_become_launch_time_constants():
    """A by-value parameter of the launch (emmyptx/kernel.py:171-178) gets a constant slot that the launch fills."""
    built = ir.elementwise_kernel(256, {"x": "f32"}, [("a", "multiply", ["x", "alpha"]), ("o", "add", ["a", "beta"])], scalars={"alpha": "f32", "beta": "f32"})
    h = handle(built)
    assert h["variant"] == "pointwise_program" and h["arg_order"] == ["x", "out", "alpha", "beta"]
    prog = h["params"]["program"]
    assert sorted(prog["scalar_consts"]) == [["alpha", 0, "f32"], ["beta", 1, "f32"]]
    assert prog["steps"][0][2:4] == [0, 16] and prog["steps"][1][3] == 17
    # a scalar no step uses changes nothing
    h2 = handle(ir.elementwise_kernel(256, {"x": "f32"}, [("o", "exp", ["x"])], scalars={"unused": "f32"}))
    assert h2["variant"] == "pointwise_f32" and h2["params"]["op"] == "exp"


def test_common_activations_map_to_streaming_ops():
    """sigmoid, SiLU and ReLU however spelled land on the fixed-function streaming kernel, not on the interpreter."""
    h = handle(ir.elementwise_kernel(4096, {"x": "f32"}, [("s", "sigmoid", ["x"]), ("y", "multiply", ["x", "s"])]))
    assert (h["variant"], h["params"]["op"]) == ("pointwise_f32", "silu")
    h = handle(ir.elementwise_kernel(4096, {"x": "f32"}, [("n", "negative", ["x"]), ("e", "exp", ["n"]), ("d", "add", ["e", 1.0]), ("y", "reciprocal", ["d"])]))
    assert (h["variant"], h["params"]["op"]) == ("pointwise_f32", "sigmoid")
    h = handle(ir.elementwise_kernel(4096, {"x": "f32"}, [("y", "maximum", ["x", 0.0])]))
    assert (h["variant"], h["params"]["op"]) == ("pointwise_f32", "relu")



def test_scalar_loop_attention_is_matched_by_behaviour():
    """The reference's own attention cases are fp32 and arrive as nested scalar loops (tools/torch_cases/fused.py:21-22,
    31-36; models.py:17-19); a few output cells are run and compared with attention of the probe buffers."""
    h = handle(ir.attention_scalar_kernel([1, 2], 64, 64, 32))
    assert h["variant"] == "attention_fwd" and h["inputs"] == ["Q", "K", "V"] and h["outputs"] == ["O"]
    assert h["params"] == {"dtype": "f32", "units": 2, "seq_q": 64, "seq_k": 64, "d": 32, "scale": 32 ** -0.5, "causal": False}
    h = handle(ir.attention_scalar_kernel([1, 4], 128, 128, 64, causal=True))
    assert h["params"]["causal"] is True and h["params"]["scale"] == 0.125 and h["params"]["units"] == 4
    h = handle(ir.attention_scalar_kernel([1], 64, 64, 32, scale=0.17677669, causal=True))
    assert h["params"]["scale"] == 0.17677669 and h["params"]["causal"] is True
    h = handle(ir.attention_scalar_kernel([3], 40, 72, 96, scale=2.0))
    assert (h["params"]["seq_q"], h["params"]["seq_k"], h["params"]["d"], h["params"]["scale"]) == (40, 72, 96, 2.0)
    assert algorithmic_work(h) == (4.0 * 3 * 40 * 72 * 96, "flop")
    for mask in ("upper", "padding"):
        with pytest.raises(CompileError, match="lower-triangular"):
            handle(ir.attention_scalar_kernel([2], 64, 64, 32, mask=mask))
    with pytest.raises(CompileError, match="head dim"):
        handle(ir.attention_scalar_kernel([2], 64, 64, 48))
    # a bias on the scores is some other function: nothing matches
    g, k, launch = ir.attention_scalar_kernel([2], 64, 64, 32)
    for loop in (s for s in k.body[0].body if type(s).__name__ == "Loop"):
        at = next(i for i, s in enumerate(loop.body) if type(s).__name__ == "Assign" and s.op.name == "multiply")
        loop.body.insert(at + 1, ir.Assign(loop.body[at].name, ir.Op("add"), [loop.body[at].name, "j0" if loop.axis.name == "j0" else "j1"]))
    with pytest.raises(CompileError, match="not softmax"):
        handle((g, k, launch))


def test_f32_output_and_split_k_contractions():
    """A fragment store to an f32 buffer (emmyptx/mma.py:205-207) and its split-K form (a tile axis over parts of K, cells
    adding partial sums with red.add.f32, :239-240) are one kernel with an fp32 output; the cells' K offsets must cover K
    exactly once."""
    h = handle(ir.gemm_kernel(128, 96, 256, "bf16", out_dtype="f32"))
    assert h["variant"] == "gemm" and h["params"]["out_f32"] is True and h["params"]["k"] == 256
    h = handle(ir.gemm_kernel(128, 96, 256, "f16", out_dtype="f32", split_k=4))
    assert h["variant"] == "gemm" and h["params"]["out_f32"] is True and h["params"]["k"] == 256
    h = handle(ir.gemm_kernel(64, 96, 128, "f16", None, True, out_dtype="f32", split_k=2, batch=(3,)))
    assert h["variant"] == "gemm_batched" and h["params"]["out_f32"] is True and h["params"]["b_trans"] is True
    assert "out_f32" not in handle(ir.gemm_kernel(128, 96, 256, "bf16"))["params"]
    g, k, launch = ir.gemm_kernel(128, 96, 256, "f16", out_dtype="f32", split_k=4)
    loop = next(s for s in k.body[0].body if type(s).__name__ == "Loop")
    loop.axis = ir.Axis("k0", ir.Dim(3))                      # each part one cell short: a quarter of K is never read
    with pytest.raises(CompileError, match="cover K exactly once"):
        handle((g, k, launch))
    g, k, launch = ir.gemm_kernel(128, 96, 256, "f16")
    store = next(s for s in k.body[0].body if type(s).__name__ == "RegStore")
    store.atomic = True                                        # red.add needs an f32 buffer
    with pytest.raises(CompileError, match="f32 buffer"):
        handle((g, k, launch))


def test_layout_kernels_become_indexed_programs():
    """Loads and Writes whose indices are affine in the axis variables (tools/torch_cases/shapes.py:6-19), and masks made of
    the axis variables themselves: every index is fitted on probe cells and checked against the buffers."""
    h = handle(ir.layout_kernel("s_transpose"))
    assert h["variant"] == "pointwise_indexed" and h["inputs"] == ["X"]
    assert h["params"]["index_map"] == {"extents": [96, 64], "inputs": [{"buffer": "X", "offset": 0, "coef": [1, 96]}], "out": {"offset": 0, "coef": [64, 1]}}
    assert handle(ir.layout_kernel("s_flip"))["params"]["index_map"]["inputs"][0] == {"buffer": "X", "offset": 127, "coef": [128, -1]}
    assert handle(ir.layout_kernel("s_slice"))["params"]["index_map"]["inputs"][0] == {"buffer": "X", "offset": 10, "coef": [128, 1]}
    assert handle(ir.layout_kernel("s_cat_b"))["params"]["index_map"]["out"] == {"offset": 64, "coef": [112, 1]}
    h = handle(ir.layout_kernel("s_tril"))
    assert h["params"]["index_map"]["inputs"][1:] == [{"axis": 0}, {"axis": 1}] or h["params"]["index_map"]["inputs"][1:] == [{"axis": 1}, {"axis": 0}]
    assert [st[0] for st in h["params"]["program"]["steps"]] == ["less_equal", "where"]
    h = handle(ir.layout_kernel("s_stack"))
    assert h["inputs"] == ["A", "B"] and {"axis": 0} in h["params"]["index_map"]["inputs"]
    assert handle(ir.layout_kernel("s_repeat"))["variant"] == "pointwise_program"           # a broadcast: the vectorised kernel
    h = handle(ir.layout_kernel("s_roll"))                                                  # wraps around: a rotation of axis 1
    assert h["params"]["index_map"]["inputs"][0] == {"buffer": "X", "offset": 0, "coef": [128, 1], "rot": [0, 125]}
    h = handle(ir.layout_kernel("s_embedding"))                                             # a row taken from data
    srcs = h["params"]["index_map"]["inputs"]
    assert h["inputs"] == ["SRC", "IDX"] and h["params"]["program"]["in_dtypes"] == ["f32", "i64"]
    assert srcs[1] == {"buffer": "IDX", "offset": 0, "coef": [1, 0], "index_mod": 100, "index_abs": True}
    assert srcs[0] == {"buffer": "SRC", "offset": 0, "coef": [0, 1], "index_mult": 32, "index_of": 1}
    assert handle(ir.layout_kernel("s_gather"))["params"]["index_map"]["inputs"][0]["index_mult"] == 1
    g, k, launch = ir.layout_kernel("s_embedding")                                          # without the modulus nothing bounds the row
    body = k.body[0].body
    load = next(s for s in body if type(s).__name__ == "Load" and s.input == "SRC")
    load.index[0] = ir.Var("a")
    with pytest.raises(CompileError):
        handle((g, k, launch))
    g, k, launch = ir.layout_kernel("s_embedding")                                          # a modulus larger than the table
    next(s for s in k.body[0].body if type(s).__name__ == "Assign" and s.op.name == "mod").args[1] = 101
    with pytest.raises(CompileError):
        handle((g, k, launch))
    g, k, launch = ir.layout_kernel("s_slice")                                              # a slice that leaves its buffer
    load = next(s for s in k.body[0].body if type(s).__name__ == "Load")
    load.index[1] = ir.BinaryExpr("+", ir.Var("c0"), ir.Literal(100, "int"))
    with pytest.raises(CompileError):
        handle((g, k, launch))
    g, k, launch = ir.layout_kernel("s_transpose")                                          # two cells writing one element
    write = next(s for s in k.body[0].body if type(s).__name__ == "Write")
    write.index = [ir.Var("j0"), ir.Literal(0, "int")]
    with pytest.raises(CompileError):
        handle((g, k, launch))


def test_convolution_loops_become_an_indexed_contraction():
    """Nested Loops folding w * x into one accumulator (tools/torch_cases/conv.py:6-7 as scalar loops): the three index
    expressions are fitted over the tile's and the loops' variables and checked against the buffers."""
    h = handle(ir.conv_kernel("c_conv1d"))
    assert h["variant"] == "contract_indexed" and h["inputs"] == ["W", "X"] and h["outputs"] == ["out"]
    assert h["params"]["map"] == {"extents": [32, 126], "loops": [16, 3],
                                  "a": {"buffer": "W", "offset": 0, "coef": [48, 0], "loop_coef": [3, 1], "dtype": "f32"},
                                  "b": {"buffer": "X", "offset": 0, "coef": [0, 1], "loop_coef": [128, 1], "dtype": "f32"},
                                  "out": {"offset": 0, "coef": [126, 1], "dtype": "f32"}}
    assert algorithmic_work(h) == (2.0 * 32 * 126 * 48, "flop")
    h = handle(ir.conv_kernel("c_conv2d"))
    assert h["params"]["map"]["b"] == {"buffer": "X", "offset": 0, "coef": [0, 32, 1], "loop_coef": [1024, 32, 1], "dtype": "f32"}
    assert h["params"]["terms"] == 72 and h["params"]["n"] == 16 * 30 * 30

    def inner(k):
        lp = next(s for s in k.body[0].body if type(s).__name__ == "Loop")
        while type(lp.body[0]).__name__ == "Loop":
            lp = lp.body[0]
        return lp
    g, k, launch = ir.conv_kernel("c_conv1d")                       # a tap that runs past the row
    inner(k).body[1].index[1] = ir.BinaryExpr("+", ir.BinaryExpr("+", ir.Var("i0"), ir.Var("t0")), ir.Literal(1, "int"))
    with pytest.raises(CompileError, match="leaves the buffer"):
        handle((g, k, launch))
    g, k, launch = ir.conv_kernel("c_conv1d")                       # the innermost loop re-seeding the accumulator on every outer trip
    inner(k).seed = True
    with pytest.raises(CompileError, match="reset the accumulator"):
        handle((g, k, launch))
    g, k, launch = ir.conv_kernel("c_conv1d")                       # an accumulator nobody seeds
    k.body[0].body.pop(0)
    with pytest.raises(CompileError, match="not seeded"):
        handle((g, k, launch))
    g, k, launch = ir.conv_kernel("c_conv2d")                       # something other than a product
    inner(k).body[2].op = ir.Op("add")
    with pytest.raises(CompileError):
        handle((g, k, launch))
    g, k, launch = ir.conv_kernel("c_conv2d")                       # folding with max
    inner(k).body[3].op = ir.Op("maximum")
    with pytest.raises(CompileError):
        handle((g, k, launch))
    g, k, launch = ir.conv_kernel("c_conv1d")                       # an index that is not affine in the variables
    inner(k).body[0].index[2] = ir.BinaryExpr("*", ir.Var("t0"), ir.Var("t0"))
    with pytest.raises(CompileError):
        handle((g, k, launch))


def test_transposed_lhs_is_an_indexed_contraction_and_sm_100_is_a_target():
    h = handle(ir.matmul_f32_kernel(128, 80, 96, a_trans=True))                 # a.t() @ b: A walked with stride m
    assert h["variant"] == "contract_indexed" and h["params"]["map"]["loops"] == [96]
    assert handle(ir.matmul_f32_kernel(128, 80, 96))["variant"] == "gemm_f32"   # the row-major product keeps its kernel
    assert handle(ir.rowwise_kernel("dot", 64, 256))["variant"] == "rowwise_f32"
    # a runner passes the name it derives from the device's compute capability (tools/run_local.py:57-60)
    assert json.loads(compile_kernel(*ir.pointwise_kernel(64), target="sm_100"))["variant"] == "pointwise_f32"
    renamed = ir.rename_buffers(ir.matmul_f32_kernel(32, 256, 128, b_trans=True, bias=True), {"A": "inp", "B": "w1", "bias": "b1", "C": "h1"})
    h = handle(renamed)
    assert h["inputs"] == ["inp", "w1", "b1"] and h["outputs"] == ["h1"] and h["arg_order"] == ["inp", "w1", "b1", "h1"]
    with pytest.raises(ValueError):
        ir.rename_buffers(ir.rowwise_kernel("rms_norm", 64, 256), {"X": "x"})    # would shadow the loaded value x


def test_f64_buffers_are_refused_and_bool_outputs_are_programs():
    """d_f64_add (tools/torch_cases/dtypes.py:13): the reference refuses an f64 buffer rather than compute it in f32
    (emmyptx/kernel.py:185-187), and so does this compiler. p_cmp_bool_out (pointwise.py:50): a comparison stored to a
    bool buffer is an elementwise program with a byte output."""
    with pytest.raises(CompileError, match="is f64"):
        handle(ir.elementwise_kernel(1024, {"x": "f64"}, [("a", "multiply", ["x", 2.0]), ("b", "add", ["a", 1.0])], "f64"))
    h = handle(ir.elementwise_kernel(4096, {"x": "f32", "y": "f32"}, [("m", "greater", ["x", "y"])], "bool"))
    assert h["variant"] == "pointwise_program" and h["params"]["program"]["out_dtype"] == "bool"


def test_move_only_op_names_are_copies():
    """`pad` and the f8 conversion names are plain register moves in the reference's op table (emmyptx/ops.py:236-237);
    here they become `copy` steps of an elementwise program."""
    for name in ("pad", "from_f8e4m3", "to_f8e5m2"):
        h = handle(ir.elementwise_kernel(4096, {"x": "f16"}, [("a", name, ["x"]), ("b", "add", ["a", 1.0])], "f16"))
        assert h["variant"] == "pointwise_program" and [st[0] for st in h["params"]["program"]["steps"]] == ["copy", "add"]


def test_let_and_select_become_assigns():
    """A mask written as a Select on the axis variables (emmyptx/kernel.py:812-822) or kept in a Let of a compound predicate
    is spelled out as comparison / logical / where steps of an indexed program; integer expressions are not rewritten."""
    h = handle(ir.layout_kernel("s_tril_select"))
    assert h["variant"] == "pointwise_indexed"
    assert [st[0] for st in h["params"]["program"]["steps"]] == ["less_equal", "where", "copy"]
    assert h["params"]["index_map"]["inputs"][1:] in ([{"axis": 0}, {"axis": 1}], [{"axis": 1}, {"axis": 0}])
    h = handle(ir.layout_kernel("s_window_let"))
    assert [st[0] for st in h["params"]["program"]["steps"]] == ["greater_equal", "less", "bitwise_and", "copy", "where", "multiply"]
    g, k, launch = ir.layout_kernel("s_window_let")
    k.body[0].body[1] = ir.Let("inside", ir.BinaryExpr(">>", ir.Var("c0"), ir.Literal(2, "int")))      # a shift has no float op
    with pytest.raises(CompileError):
        handle((g, k, launch))
    assert handle(ir.index_gather_kernel(2**16))["variant"] == "index_gather_i32"                        # the integer Let of the gather is untouched


def test_cond_becomes_guarded_loads_and_a_where():
    """torch.cat as one kernel: a Cond on the column index with a Load and a Write in each arm (emmyptx/kernel.py:825-840).
    Both Loads run in every cell with their indices clamped into the buffers; the Write stores where(pred, a, b)."""
    h = handle(ir.layout_kernel("s_cat_cond"))
    assert h["variant"] == "pointwise_indexed" and h["inputs"] == ["A", "B"]
    srcs = h["params"]["index_map"]["inputs"]
    assert srcs[0] == {"buffer": "A", "offset": 0, "coef": [64, 1], "clamp": 2048}
    assert srcs[1] == {"buffer": "B", "offset": -64, "coef": [48, 1], "clamp": 1536}
    assert [st[0] for st in h["params"]["program"]["steps"]] == ["less", "where"]
    g, k, launch = ir.layout_kernel("s_cat_cond")               # one arm that writes nothing: some cells would stay unwritten
    k.body[0].body[0].else_body = []
    with pytest.raises(CompileError):
        handle((g, k, launch))
    g, k, launch = ir.layout_kernel("s_cat_cond")               # arms writing different elements
    k.body[0].body[0].else_body[1].index = [ir.Var("r0"), ir.Literal(0, "int")]
    with pytest.raises(CompileError):
        handle((g, k, launch))


def test_row_ops_match_with_and_without_a_warp_shuffle():
    """The row kernels are recognised from one thread per row (a loop per pass: the form whose reference PTX the fixtures
    hold) and from the same loops followed by a WarpShuffle (emmyptx/kernel.py:856-866: how a warp-per-row schedule ends them)."""
    for op in ("sum", "softmax", "layer_norm", "dot"):
        plain, laned = handle(ir.rowwise_kernel(op, 48, 256)), handle(ir.rowwise_kernel(op, 48, 256, lanes=True))
        assert plain["variant"] == laned["variant"] == "rowwise_f32" and plain["params"] == laned["params"]
    kinds = {type(s).__name__ for s in ir.rowwise_kernel("sum", 8, 64)[1].body[0].body}
    assert "WarpShuffle" not in kinds and "WarpShuffle" in {type(s).__name__ for s in ir.rowwise_kernel("sum", 8, 64, lanes=True)[1].body[0].body}

