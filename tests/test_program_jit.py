"""The compile-at-first-use form of elementwise programs, as far as it goes without a GPU: the CUDA C++ text a program
becomes, and that the run-time compiler turns it into sm_100a device code. The generated kernel replaces the entry the
reference prints for a one-axis Tile (emmyptx/kernel.py:766-784 calling emmyptx/ops.py:212 once per Assign)."""
import pytest

from emmyptx import runtime as rt

S = rt.PW_MAX_SLOTS
LERP = {"in_dtypes": ["f32", "f32", "f32"], "out_dtype": "f32", "out_slot": 5, "consts": [],
        "steps": [["subtract", 4, 1, 0, 0], ["multiply", 4, 4, 2, 0], ["add", 5, 0, 4, 0]]}


def test_source_spells_each_step_once_in_order(lib):
    text = rt.program_source(LERP)
    body = text[text.index("pw_cell("):text.index("return s5;")]
    lines = [ln.strip() for ln in body.splitlines() if ln.strip().startswith("s") and "=" in ln and not ln.strip().startswith("float")]
    assert lines == ["s4 = __fsub_rn(s1, s0);", "s4 = __fmul_rn(s4, s2);", "s5 = __fadd_rn(s0, s4);"]
    assert "#define PW_N_IN 3" in text and "#define PW_VEC 1" in text
    assert "#define PW_VEC 0" in rt.program_source(LERP, group=0)
    assert "#define PW_G 8" in rt.program_source(LERP, group=8)


def test_constants_are_arguments_and_broadcast_is_a_flag(lib):
    prog = {"in_dtypes": ["f16", "bool", "bf16"], "out_dtype": "bf16", "out_slot": 4, "consts": [0.5, 2.0], "in_mod": [0, 0, 7],
            "steps": [["where", 4, 1, 0, S + 1], ["pow", 4, 4, S + 0, 0], ["maximum", 4, 4, 2, 0]]}
    text = rt.program_source(prog)
    assert "s4 = (s1 != 0.0f ? s0 : c.v[1]);" in text and "s4 = powf(s4, c.v[0]);" in text
    assert "#define PW_DT0 1" in text and "#define PW_DT1 5" in text and "#define PW_DT2 2" in text
    assert "#define PW_BC2 1" in text and "#define PW_BC0 0" in text and "#define PW_OUT_DT 2" in text
    other = dict(prog, consts=[9.0, -1.0], in_mod=[0, 0, 13])
    assert rt.program_source(other) == text            # same text, so the same cached kernel
    assert "#define PW_BC2 2" in rt.program_source(dict(prog, in_mod=[0, 0, 64]))      # a row vector read with vector accesses


def test_every_float_op_compiles_for_sm100a(lib):
    if rt.pointwise_jit_state()[0] != 1:
        pytest.skip("libnvrtc is not installed here")
    names = [k for k, v in sorted(rt.PW_OPS.items(), key=lambda kv: kv[1]) if k not in ("exp_fast", "remainder")]
    steps = []
    for i, op in enumerate(names):                    # a chain, so that no step is dead code
        steps.append([op, 4 + (i % 8), 4 + ((i + 7) % 8) if i else 0, 1, 2])
    for out_dtype, vec in (("f32", 4), ("f16", 8), ("bf16", 0), ("bf16", 4), ("f32", 8)):
        prog = {"in_dtypes": ["f32", "f16", "bf16", "bool"], "out_dtype": out_dtype, "out_slot": steps[-1][1], "consts": [1.0],
                "in_div": [0, 3, 0, 0], "steps": steps}
        assert rt.program_compile(prog, vec) > 1000


def test_integer_programs_are_compiled_too(lib):
    prog = {"in_dtypes": ["i32", "i64"], "out_dtype": "i64", "out_slot": 5, "consts": [3], "int_div": "trunc",
            "steps": [["add", 4, 0, S, 0], ["floor_divide", 4, 4, 1, 0], ["left_shift", 5, 4, S, 0]]}
    text = rt.program_source(prog)
    assert "#define PW_T int" in text and "emmy_math.cuh" not in text
    assert "s4 = (int)((unsigned)s0 + (unsigned)(int)c.v[0]);" in text and "s4 = pw_i_div(s4, s1, 1);" in text
    assert "pw_i_div(s4, s1, 0)" in rt.program_source({k: v for k, v in prog.items() if k != "int_div"})
    with pytest.raises(rt.KernelError, match="groups of 4"):
        rt.program_source(prog, group=8)
    if rt.pointwise_jit_state()[0] == 1:
        names = ["add", "subtract", "multiply", "maximum", "minimum", "relu", "square", "negative", "abs", "equal", "not_equal", "greater", "less",
                 "greater_equal", "less_equal", "where", "bitwise_and", "bitwise_or", "bitwise_not", "bitwise_xor", "left_shift", "right_shift",
                 "divide", "floor_divide", "mod", "copy"]
        steps = [[op, 4 + (i % 8), 4 + ((i + 7) % 8) if i else 0, 1, 0] for i, op in enumerate(names)]
        for group in (4, 0):
            assert rt.program_compile({"in_dtypes": ["i32", "i64"], "out_dtype": "i32", "out_slot": steps[-1][1], "consts": [2], "steps": steps}, group) > 1000


def test_indexed_programs_compile_for_sm100a(lib):
    if rt.pointwise_jit_state()[0] != 1:
        pytest.skip("libnvrtc is not installed here")
    prog = {"in_dtypes": ["f32", "f32", "f32"], "out_dtype": "bf16", "out_slot": 5, "consts": [0.0], "steps": [["less_equal", 4, 2, 1, 0], ["where", 5, 4, 0, S]]}
    imap = {"extents": [64, 64], "inputs": [{"offset": 0, "coef": [64, 1]}, {"axis": 0}, {"axis": 1}], "out": {"offset": 0, "coef": [64, 1]}}
    assert rt.indexed_compile(prog, imap) > 1000
    progi = {"in_dtypes": ["i32", "i64"], "out_dtype": "i64", "out_slot": 4, "consts": [3], "steps": [["add", 4, 0, 1, 0]]}
    assert rt.indexed_compile(progi, {"extents": [4, 5, 6], "inputs": [{"offset": 119, "coef": [-30, -6, -1]}, {"axis": 2}], "out": {"offset": 0, "coef": [30, 6, 1]}}) > 1000
    with pytest.raises(ValueError):
        rt.indexed_compile(prog, dict(imap, extents=[2] * 7, out={"offset": 0, "coef": [1] * 7}, inputs=[{"offset": 0, "coef": [1] * 7}, {"axis": 0}, {"axis": 1}]))


def test_indexed_contractions_compile_for_sm100a(lib):
    """The nested-loop sum of products (convolutions written as scalar loops) as a kernel compiled on this machine."""
    cm = {"extents": [32, 126], "loops": [16, 3], "a": {"offset": 0, "coef": [48, 0], "loop_coef": [3, 1], "dtype": "f32"},
          "b": {"offset": 0, "coef": [0, 1], "loop_coef": [128, 1], "dtype": "f32"}, "out": {"offset": 0, "coef": [126, 1], "dtype": "f32"}}
    assert rt.contraction_compile(cm) > 1000
    cm3 = {"extents": [16, 30, 30], "loops": [8, 3, 3], "a": {"offset": 0, "coef": [72, 0, 0], "loop_coef": [9, 3, 1], "dtype": "bf16"},
           "b": {"offset": 0, "coef": [0, 32, 1], "loop_coef": [1024, 32, 1], "dtype": "f16"}, "out": {"offset": 0, "coef": [900, 30, 1], "dtype": "bf16"}}
    assert rt.contraction_compile(cm3) > 1000
    with pytest.raises(ValueError):
        rt.contraction_compile(dict(cm, loops=[2, 2, 2, 2]))
    with pytest.raises(rt.KernelError):
        rt.contraction_compile(dict(cm, out={"offset": 0, "coef": [126, 1], "dtype": "i32"}))


def test_bool_outputs_compile_in_every_group(lib):
    """A comparison stored to a byte buffer (1 where the value is non-zero): scalar stores, four bytes and eight bytes a group."""
    S = rt.PW_MAX_SLOTS
    prog = {"in_dtypes": ["f32", "f32"], "out_dtype": "bool", "out_slot": 2, "consts": [], "steps": [["greater", 2, 0, 1, 0]]}
    for group in (0, 4, 8):
        assert "#define PW_OUT_DT 5" in rt.program_source(prog, group)
    assert rt.program_compile(prog) > 1000


def test_guarded_reads_compile(lib):
    """Inputs whose index is clamped into the buffer (Loads hoisted out of a Cond): the one-cell form with spelled-out loads."""
    S = rt.PW_MAX_SLOTS
    prog = {"in_dtypes": ["f32", "f32", "f32"], "out_dtype": "f32", "out_slot": 3, "consts": [64.0], "steps": [["less", 3, 2, S, 0], ["where", 3, 3, 0, 1]]}
    imap = {"extents": [32, 112], "inputs": [{"offset": 0, "coef": [64, 1], "clamp": 2048}, {"offset": -64, "coef": [48, 1], "clamp": 1536}, {"axis": 1}],
            "out": {"offset": 0, "coef": [112, 1]}}
    assert rt.indexed_compile(prog, imap) > 1000

