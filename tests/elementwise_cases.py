"""The reference's pointwise and dtype cases (tools/torch_cases/pointwise.py:8-57, dtypes.py:5-12) as data: each case once as the
statement list of an elementwise kernel (what `ir.elementwise_kernel` takes: Loads of the inputs, a chain of Assigns through
the op table, a Write) and once as the torch expression the reference's checker evaluates in float64 on the same seeded
inputs. Shared by the GPU parity tests and by the script that compiles the same kernels with the reference compiler into
PTX fixtures. Tolerances are the reference's classes (tools/torch_cases/__init__.py:17-21): ROUND 1e-6, TRANS 1e-5, HALF 1e-2."""
ROUND, TRANS, HALF = 1e-6, 1e-5, 1e-2

# id -> (inputs, steps, torch expression over float64 tensors named like the inputs, tolerance)
CASES = {
    "p_abs": ({"x": "f32"}, [("a", "abs", ["x"])], "torch.abs(x)", ROUND),
    "p_neg_sub": ({"x": "f32", "y": "f32"}, [("a", "negative", ["x"]), ("b", "subtract", ["a", "y"])], "-x - y", ROUND),
    "p_div": ({"x": "f32", "y": "f32"}, [("a", "abs", ["y"]), ("b", "add", ["a", 0.5]), ("c", "divide", ["x", "b"])], "x / (y.abs() + 0.5)", ROUND),
    "p_max_min": ({"x": "f32", "y": "f32"}, [("a", "maximum", ["x", "y"]), ("b", "minimum", ["x", "y"]), ("c", "add", ["a", "b"])],
                  "torch.maximum(x, y) + torch.minimum(x, y)", ROUND),
    "p_log": ({"x": "f32"}, [("a", "abs", ["x"]), ("b", "add", ["a", 0.5]), ("c", "log", ["b"])], "torch.log(x.abs() + 0.5)", TRANS),
    "p_sqrt_rsqrt": ({"x": "f32"}, [("a", "abs", ["x"]), ("b", "sqrt", ["a"]), ("c", "add", ["a", 0.1]), ("d", "rsqrt", ["c"]), ("e", "add", ["b", "d"])],
                     "torch.sqrt(x.abs()) + torch.rsqrt(x.abs() + 0.1)", TRANS),
    "p_reciprocal": ({"x": "f32"}, [("a", "abs", ["x"]), ("b", "add", ["a", 0.5]), ("c", "reciprocal", ["b"])], "torch.reciprocal(x.abs() + 0.5)", ROUND),
    "p_sigmoid": ({"x": "f32"}, [("a", "sigmoid", ["x"])], "torch.sigmoid(x)", TRANS),
    "p_relu": ({"x": "f32"}, [("a", "relu", ["x"])], "torch.relu(x)", ROUND),
    "p_gelu_erf": ({"x": "f32"}, [("a", "multiply", ["x", 0.7071067811865476]), ("b", "erf", ["a"]), ("c", "add", ["b", 1.0]),
                                  ("d", "multiply", ["x", 0.5]), ("e", "multiply", ["d", "c"])], "F.gelu(x)", TRANS),
    "p_silu": ({"x": "f32"}, [("a", "sigmoid", ["x"]), ("b", "multiply", ["x", "a"])], "F.silu(x)", TRANS),
    "p_erf": ({"x": "f32"}, [("a", "erf", ["x"])], "torch.erf(x)", TRANS),
    "p_sin_cos": ({"x": "f32"}, [("a", "multiply", ["x", 3.0]), ("b", "sin", ["a"]), ("c", "cos", ["a"]), ("d", "add", ["b", "c"])],
                  "torch.sin(x * 3) + torch.cos(x * 3)", TRANS),
    "p_square_cube": ({"x": "f32"}, [("a", "square", ["x"]), ("b", "multiply", ["a", "x"]), ("c", "add", ["a", "b"])], "x ** 2 + x ** 3", ROUND),
    "p_pow_frac": ({"x": "f32"}, [("a", "abs", ["x"]), ("b", "add", ["a", 0.1]), ("c", "pow", ["b", 0.7])], "torch.pow(x.abs() + 0.1, 0.7)", TRANS),
    "p_clamp": ({"x": "f32"}, [("a", "maximum", ["x", -0.5]), ("b", "minimum", ["a", 0.5])], "torch.clamp(x, -0.5, 0.5)", ROUND),
    "p_where": ({"x": "f32"}, [("m", "greater", ["x", 0.0]), ("a", "multiply", ["x", 0.1]), ("b", "where", ["m", "x", "a"])],
                "torch.where(x > 0, x, x * 0.1)", ROUND),
    "p_cmp_to_float": ({"x": "f32", "y": "f32"}, [("m", "greater", ["x", "y"])], "(x > y).double()", ROUND),
    "p_lerp": ({"x": "f32", "y": "f32"}, [("a", "subtract", ["y", "x"]), ("b", "multiply", ["a", 0.3]), ("c", "add", ["x", "b"])],
               "torch.lerp(x, y, 0.3)", ROUND),
    "p_addcmul": ({"x": "f32", "y": "f32", "z": "f32"}, [("a", "multiply", ["y", "z"]), ("b", "multiply", ["a", 0.5]), ("c", "add", ["x", "b"])],
                  "torch.addcmul(x, y, z, value=0.5)", ROUND),
    "p_remainder": ({"x": "f32"}, [("a", "multiply", ["x", 5.0]), ("b", "remainder", ["a", 1.5])], "torch.remainder(x * 5, 1.5)", TRANS),
    "p_floor_divide": ({"x": "f32"}, [("a", "multiply", ["x", 5.0]), ("b", "floor_divide", ["a", 1.5])], "torch.floor_divide(x * 5, 1.5)", ROUND),
    "d_f16_add": ({"x": "f16", "y": "f16"}, [("a", "add", ["x", "y"])], "x + y", HALF),
    "d_bf16_add": ({"x": "bf16", "y": "bf16"}, [("a", "add", ["x", "y"])], "x + y", HALF),
    "d_bf16_gelu": ({"x": "bf16"}, [("a", "multiply", ["x", 0.7071067811865476]), ("b", "erf", ["a"]), ("c", "add", ["b", 1.0]),
                                    ("d", "multiply", ["x", 0.5]), ("e", "multiply", ["d", "c"])], "F.gelu(x)", HALF),
    "d_f32_to_f16": ({"x": "f32"}, [("a", "copy", ["x"])], "x", HALF),
    "d_f16_gelu": ({"x": "f16"}, [("a", "multiply", ["x", 0.7071067811865476]), ("b", "erf", ["a"]), ("c", "add", ["b", 1.0]),
                                  ("d", "multiply", ["x", 0.5]), ("e", "multiply", ["d", "c"])], "F.gelu(x)", HALF),
    # cases the reference's front end decomposes before its compiler sees them; here they are written over the op table directly
    "p_gelu_tanh": ({"x": "f32"}, [("a", "square", ["x"]), ("b", "multiply", ["a", "x"]), ("c", "multiply", ["b", 0.044715]), ("d", "add", ["x", "c"]),
                                   ("e", "multiply", ["d", 0.7978845608028654]), ("f", "tanh", ["e"]), ("g", "add", ["f", 1.0]),
                                   ("h", "multiply", ["x", 0.5]), ("i", "multiply", ["h", "g"])], "F.gelu(x, approximate='tanh')", TRANS),
    "p_softplus": ({"x": "f32"}, [("a", "exp", ["x"]), ("b", "add", ["a", 1.0]), ("c", "log", ["b"])], "F.softplus(x)", TRANS),
    "p_mish": ({"x": "f32"}, [("a", "exp", ["x"]), ("b", "add", ["a", 1.0]), ("c", "log", ["b"]), ("d", "tanh", ["c"]), ("e", "multiply", ["x", "d"])],
               "F.mish(x)", TRANS),
    "p_elu": ({"x": "f32"}, [("m", "greater", ["x", 0.0]), ("a", "exp", ["x"]), ("b", "subtract", ["a", 1.0]), ("c", "where", ["m", "x", "b"])], "F.elu(x)", TRANS),
    "p_leaky_relu": ({"x": "f32"}, [("m", "greater", ["x", 0.0]), ("a", "multiply", ["x", 0.1]), ("b", "where", ["m", "x", "a"])], "F.leaky_relu(x, 0.1)", ROUND),
    "p_hardtanh": ({"x": "f32"}, [("a", "maximum", ["x", -1.0]), ("b", "minimum", ["a", 1.0])], "F.hardtanh(x)", ROUND),
    "p_hardswish": ({"x": "f32"}, [("a", "add", ["x", 3.0]), ("b", "maximum", ["a", 0.0]), ("c", "minimum", ["b", 6.0]), ("d", "multiply", ["x", "c"]),
                                   ("e", "divide", ["d", 6.0])], "F.hardswish(x)", ROUND),
    "p_relu6": ({"x": "f32"}, [("a", "multiply", ["x", 4.0]), ("b", "maximum", ["a", 0.0]), ("c", "minimum", ["b", 6.0])], "F.relu6(x * 4)", ROUND),
    "p_log1p": ({"x": "f32"}, [("a", "abs", ["x"]), ("b", "add", ["a", 1.0]), ("c", "log", ["b"])], "torch.log1p(x.abs())", TRANS),
    "p_expm1": ({"x": "f32"}, [("a", "exp", ["x"]), ("b", "subtract", ["a", 1.0])], "torch.expm1(x)", TRANS),
    "p_floor": ({"x": "f32"}, [("a", "multiply", ["x", 3.0]), ("b", "floor_divide", ["a", 1.0])], "torch.floor(x * 3)", ROUND),
    "p_floor_ceil": ({"x": "f32"}, [("a", "multiply", ["x", 3.0]), ("b", "floor_divide", ["a", 1.0]), ("c", "multiply", ["x", -5.0]),
                                    ("d", "floor_divide", ["c", 1.0]), ("e", "subtract", ["b", "d"])], "torch.floor(x * 3) + torch.ceil(x * 5)", ROUND),
    # round half to even: floor, then one up when the fraction is above a half, or exactly a half with an odd floor
    "p_round": ({"x": "f32"}, [("a", "multiply", ["x", 3.0]), ("r", "floor_divide", ["a", 1.0]), ("d", "subtract", ["a", "r"]), ("g", "greater", ["d", 0.5]),
                               ("t", "equal", ["d", 0.5]), ("o", "remainder", ["r", 2.0]), ("u", "multiply", ["t", "o"]), ("v", "maximum", ["g", "u"]),
                               ("w", "add", ["r", "v"])], "torch.round(x * 3)", ROUND),
    "p_trunc": ({"x": "f32"}, [("a", "multiply", ["x", 3.0]), ("f", "floor_divide", ["a", 1.0]), ("n", "negative", ["a"]), ("g", "floor_divide", ["n", 1.0]),
                               ("c", "negative", ["g"]), ("m", "greater_equal", ["a", 0.0]), ("t", "where", ["m", "f", "c"])], "torch.trunc(x * 3)", ROUND),
    "p_sign": ({"x": "f32"}, [("p", "greater", ["x", 0.0]), ("n", "less", ["x", 0.0]), ("s", "subtract", ["p", "n"])], "torch.sign(x)", ROUND),
    "p_exp2_log2": ({"x": "f32"}, [("a", "multiply", ["x", 0.6931471805599453]), ("b", "exp", ["a"]), ("c", "abs", ["x"]), ("d", "add", ["c", 0.5]),
                                   ("e", "log", ["d"]), ("f", "multiply", ["e", 1.4426950408889634]), ("g", "add", ["b", "f"])],
                    "torch.exp2(x) + torch.log2(x.abs() + 0.5)", TRANS),
    # atan: |x| or its reciprocal in [0, 1], halved once more by atan(t) = 2 atan(t / (1 + sqrt(1 + t^2))), then the odd series to u^11
    "p_atan": ({"x": "f32"}, [("ax", "abs", ["x"]), ("rc", "reciprocal", ["ax"]), ("t", "minimum", ["ax", "rc"]), ("t2", "square", ["t"]), ("q", "add", ["t2", 1.0]),
                              ("sq", "sqrt", ["q"]), ("dn", "add", ["sq", 1.0]), ("u", "divide", ["t", "dn"]), ("u2", "square", ["u"]),
                              ("p5", "multiply", ["u2", -0.09090909090909091]), ("p4", "add", ["p5", 0.1111111111111111]), ("p4m", "multiply", ["p4", "u2"]),
                              ("p3", "add", ["p4m", -0.14285714285714285]), ("p3m", "multiply", ["p3", "u2"]), ("p2", "add", ["p3m", 0.2]),
                              ("p2m", "multiply", ["p2", "u2"]), ("p1", "add", ["p2m", -0.3333333333333333]), ("p1m", "multiply", ["p1", "u2"]),
                              ("p0", "add", ["p1m", 1.0]), ("at", "multiply", ["p0", "u"]), ("a2", "multiply", ["at", 2.0]),
                              ("big", "greater", ["ax", 1.0]), ("co", "subtract", [1.5707963267948966, "a2"]), ("r", "where", ["big", "co", "a2"]),
                              ("neg", "less", ["x", 0.0]), ("nr", "negative", ["r"]), ("out", "where", ["neg", "nr", "r"])], "torch.atan(x)", TRANS),
    # atan2(x, y): the angle of (y, x) -- atan of min / max of the magnitudes as in p_atan (one halving, series to u^11),
    # then pi/2 - a where |x| > |y|, pi - a where y < 0, and the sign of x
    "p_atan2": ({"x": "f32", "y": "f32"}, [("ax", "abs", ["x"]), ("ay", "abs", ["y"]), ("lo", "minimum", ["ax", "ay"]), ("hi", "maximum", ["ax", "ay"]),
                                           ("t", "divide", ["lo", "hi"]), ("t2", "square", ["t"]), ("q", "add", ["t2", 1.0]), ("sq", "sqrt", ["q"]),
                                           ("dn", "add", ["sq", 1.0]), ("u", "divide", ["t", "dn"]), ("u2", "square", ["u"]),
                                           ("p5", "multiply", ["u2", -0.09090909090909091]), ("p4", "add", ["p5", 0.1111111111111111]), ("p4m", "multiply", ["p4", "u2"]),
                                           ("p3", "add", ["p4m", -0.14285714285714285]), ("p3m", "multiply", ["p3", "u2"]), ("p2", "add", ["p3m", 0.2]),
                                           ("p2m", "multiply", ["p2", "u2"]), ("p1", "add", ["p2m", -0.3333333333333333]), ("p1m", "multiply", ["p1", "u2"]),
                                           ("p0", "add", ["p1m", 1.0]), ("at", "multiply", ["p0", "u"]), ("a2", "multiply", ["at", 2.0]),
                                           ("steep", "greater", ["ax", "ay"]), ("co", "subtract", [1.5707963267948966, "a2"]), ("r1", "where", ["steep", "co", "a2"]),
                                           ("left", "less", ["y", 0.0]), ("su", "subtract", [3.141592653589793, "r1"]), ("r2", "where", ["left", "su", "r1"]),
                                           ("neg", "less", ["x", 0.0]), ("nr", "negative", ["r2"]), ("out", "where", ["neg", "nr", "r2"])], "torch.atan2(x, y)", TRANS),
    "p_cmp_bool_out": ({"x": "f32", "y": "f32"}, [("m", "greater", ["x", "y"])], "x > y", ROUND),
    "p_pow_tensor": ({"x": "f32", "y": "f32"}, [("a", "abs", ["x"]), ("b", "add", ["a", 0.1]), ("c", "pow", ["b", "y"])], "torch.pow(x.abs() + 0.1, y)", (1e-4, 1e-5)),
    "p_masked_fill": ({"x": "f32"}, [("m", "less", ["x", 0.0]), ("a", "where", ["m", 0.0, "x"])], "x.masked_fill(x < 0, 0.0)", ROUND),
    # fmod keeps the dividend's sign: a - b * trunc(a / b)
    "p_fmod": ({"x": "f32"}, [("a", "multiply", ["x", 5.0]), ("q", "divide", ["a", 1.5]), ("f", "floor_divide", ["q", 1.0]), ("n", "negative", ["q"]),
                              ("g", "floor_divide", ["n", 1.0]), ("c", "negative", ["g"]), ("m", "greater_equal", ["q", 0.0]), ("t", "where", ["m", "f", "c"]),
                              ("p", "multiply", ["t", 1.5]), ("r", "subtract", ["a", "p"])], "torch.fmod(x * 5, 1.5)", TRANS),
}
OUT_DTYPE = {"p_cmp_bool_out": "bool", "d_f16_gelu": "f16", "d_f16_add": "f16", "d_bf16_add": "bf16", "d_bf16_gelu": "bf16", "d_f32_to_f16": "f16"}

# Integer programs (tools/torch_cases/dtypes.py:14-19) and the wrap / shift behaviour of the s32 op table:
# id -> (steps, input dtype, output dtype, input names)
INT_CASES = {
    "d_i32_arith": ([("t", "multiply", ["a", 3]), ("u", "add", ["t", 1])], "i32", "i32", ("a",)),
    "d_i32_floordiv_mod": ([("q", "floor_divide", ["a", 3]), ("r", "mod", ["a", 3]), ("s", "multiply", ["r", 100]), ("u", "add", ["q", "s"])],
                           "i32", "i32", ("a",)),
    "d_i64_arith": ([("t", "multiply", ["a", 3]), ("u", "add", ["t", 1])], "i64", "i64", ("a",)),
    "int_wrap_shift": ([("m", "multiply", ["a", "b"]), ("x", "bitwise_xor", ["m", "a"]), ("s", "right_shift", ["x", 3]), ("t", "left_shift", ["b", 5]),
                        ("o", "bitwise_or", ["s", "t"]), ("n", "bitwise_and", ["o", 16777215]), ("d", "subtract", ["n", "a"]), ("z", "maximum", ["d", "b"])],
                       "i32", "i32", ("a", "b")),
}
# d_bool_in (dtypes.py:16): a bool buffer as a graph input of a float program
BOOL_IN = ({"x": "f32", "m": "bool"}, [("nx", "negative", ["x"]), ("y", "where", ["m", "x", "nx"])])

# Broadcast inputs at [33, 61] (ragged against every access width): id -> (loads, steps, inputs {buffer: shape}, numpy expression)
BCAST_SHAPE = (33, 61)
BCAST_CASES = {
    "f_batch_norm_eval": ([("x", "X", ("r0", "c0")), ("m", "M", ("c0",)), ("w", "W", ("c0",)), ("b", "B", ("c0",))],
                          [("d", "subtract", ["x", "m"]), ("s", "multiply", ["d", "w"]), ("o", "add", ["s", "b"])],
                          {"X": [33, 61], "M": [61], "W": [61], "B": [61]}, "(X - M) * W + B"),
    "m_outer": ([("a", "A", ("r0",)), ("v", "V", ("c0",))], [("o", "multiply", ["a", "v"])], {"A": [33], "V": [61]}, "A[:, None] * V[None, :]"),
    "p_bcast_rowcol": ([("x", "X", ("r0", "c0")), ("r", "R", ("c0",)), ("c", "C", ("r0",))], [("p", "multiply", ["x", "r"]), ("o", "add", ["p", "c"])],
                       {"X": [33, 61], "R": [61], "C": [33]}, "X * R + C[:, None]"),
    "s_expand": ([("v", "V", ("c0",))], [("o", "add", ["v", 0.0])], {"V": [61]}, "np.broadcast_to(V, (33, 61)) + np.float32(0)"),
}

# By-value scalar parameters of a launch (emmyptx/kernel.py:166-183): id -> (inputs, steps, output dtype, scalars, integer program?)
SCALAR_CASES = {
    "sc_axpy2": ({"x": "f32", "y": "f32"}, [("ax", "multiply", ["x", "alpha"]), ("s", "add", ["ax", "y"]), ("o", "multiply", ["s", 2.0])], "f32",
                 {"alpha": "f32"}, False),
    "sc_imul": ({"a": "i32"}, [("t", "multiply", ["a", "k"]), ("o", "add", ["t", 7])], "i32", {"k": "s32"}, True),
}


def scalar_kernel(ir, case: str, n: int = 5000):
    """(graph, kernel, launch) of a SCALAR_CASES entry, built with the given ir module."""
    ins, steps, out_dt, scalars, integer = SCALAR_CASES[case]
    built = ir.elementwise_kernel(n, ins, steps, out_dtype=out_dt, scalars=scalars, name=case)
    if integer:
        for st in built[1].body[0].body:
            if type(st).__name__ == "Assign":
                st.dtype = "i32"
    return built

