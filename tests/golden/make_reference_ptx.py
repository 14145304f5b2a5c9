"""Generate the reference's own PTX for the two streaming configurations, for tensor-core GEMMs and for its fp32
attention cases, as fixtures.

    python tests/golden/make_reference_ptx.py <path to a checkout of the reference>

Needs the reference checkout (read-only) and nothing else: its `KernelCompiler` dispatches on class *names*, so
the stand-in IR classes of `emmy-ptx-compiler_b200/emmyptx/ir.py` drive it. The PTX text it prints is the
reference's output for these kernels; `oracle/ptx_interp.py` executes it on the CPU to produce the golden
vectors (`make_golden.py`), and the GPU tests JIT the same text on the device to compare kernel against kernel.
Targets are sm_89 (the reference's default); sm_100 devices JIT it forward.

The GEMM cases are the reference's own 16-bit matmul shapes (tools/torch_cases/matmul.py:27-32) compiled from the
stand-in contraction IR (`ir.gemm_kernel`: one warp per m16n8k16 output cell, fragments read straight from global
memory, emmyptx/mma.py:128-180). Cases marked `device` run on a GPU; they are restricted to extents with
M % 16 == N % 8 == K % 16 == 0, for which the IR carries no guards and every address the kernel forms is inside its
buffer by construction -- the script works the largest element index of every fragment load and store out of the
IR's own index expressions and stops if one is out of range. Ragged cases (clamped rows, zero-filled K tail,
predicated stores) are only ever executed by the CPU interpreter.

The layout cases (`ir.layout_kernel`: transpose, permute, slices, flip, stack, tril, a concatenation written in two
kernels; tools/torch_cases/shapes.py:6-19) are one-cell-per-element tiles whose index expressions are affine in the axis
variables; the facade's matcher checks every index range against the buffers before it accepts such a kernel, and the GPU
test runs the reference's PTX only for kernels the matcher accepted.

The attention cases are the reference's own three (tools/torch_cases/fused.py:21-22, 31-36; models.py:17-19): fp32
q, k, v, compiled from the scalar-loop stand-in IR (`ir.attention_scalar_kernel`: one cell per output element, nested
loops with static trip counts, no barriers). Every buffer index is a bare tile or loop variable whose extent equals
the buffer's extent in that position, which the script checks, and the cell count is a whole number of blocks.
"""
import importlib.util
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
if len(sys.argv) != 2:
    sys.exit(__doc__)
ref = Path(sys.argv[1])
sys.path.insert(0, str(ref))
from emmyptx.kernel import compile_kernel  # noqa: E402  (the reference's)

spec = importlib.util.spec_from_file_location("standin_ir", REPO / "emmy-ptx-compiler_b200" / "emmyptx" / "ir.py")
ir = importlib.util.module_from_spec(spec)
sys.modules["standin_ir"] = ir
spec.loader.exec_module(ir)

CASES = {
    "c1_exp_sin_tanh_n4096": ir.pointwise_kernel(4096, "exp_sin_tanh", name="c1_exp_sin_tanh_n4096"),
    "c1_exp_sin_tanh_n1048576": ir.pointwise_kernel(2**20, "exp_sin_tanh", name="c1_exp_sin_tanh_n1048576"),
    "p_exp_n4096": ir.pointwise_kernel(4096, "exp", name="p_exp_n4096"),
    "p_tanh_n4096": ir.pointwise_kernel(4096, "tanh", name="p_tanh_n4096"),
    "p_sin_n4096": ir.pointwise_kernel(4096, "sin", name="p_sin_n4096"),
    "c2_gather_n65536": ir.index_gather_kernel(2**16, name="c2_gather_n65536"),
    "c2_gather_n1048576": ir.index_gather_kernel(2**20, name="c2_gather_n1048576"),
    # full-size kernels, only ever timed on the device next to ours (no CPU golden vectors at these sizes)
    "c2_gather_n67108864": ir.index_gather_kernel(2**26, name="c2_gather_n67108864"),
    "c1_exp_sin_tanh_n268435456": ir.pointwise_kernel(2**28, "exp_sin_tanh", name="c1_exp_sin_tanh_n268435456"),
}

GEMMS = {       # name: (m, n, k, dtype, b_trans, batch, device)
    "m_f16_mm_32x16x32": (32, 16, 32, "f16", False, (), False),              # small: CPU golden vector
    "m_f16_mm_odd": (100, 72, 200, "f16", False, (), False),                 # matmul.py:28, ragged: CPU only
    "m_f16_mm": (256, 256, 256, "f16", False, (), True),                     # matmul.py:27
    "m_bf16_mm": (512, 512, 512, "bf16", False, (), True),                   # matmul.py:30
    "m_f16_linear": (64, 512, 256, "f16", True, (), True),                   # matmul.py:32, B stored N x K
    "m_f16_bmm": (128, 96, 64, "f16", False, (4,), True),                    # matmul.py:31
    "c3_f16_mm_4096": (4096, 4096, 4096, "f16", False, (), True),            # configuration 3: run on the device only
    "c4_bf16_mm_16384": (16384, 16384, 16384, "bf16", False, (), True),      # configuration 4's product (its GELU is refused as a fused store)
    "m_f16_mm_f32out": (128, 128, 256, "f16", False, (), True),              # the accumulator stored to an f32 buffer (mma.py:205-207)
    "m_bf16_mm_splitk4": (128, 128, 256, "bf16", False, (), True),           # four cells per output cell, red.add.f32 (mma.py:239-240)
}
GEMM_OUT = {"m_f16_mm_f32out": ("f32", 1), "m_bf16_mm_splitk4": ("f32", 4)}      # name: (output dtype, K splits)


ATTENTION = {   # name: (units shape, seq_q, seq_k, d, causal, scale)
    "f_sdpa": ([1, 2], 64, 64, 32, False, None),                              # fused.py:21-22
    "t_causal_sdpa": ([1, 4], 128, 128, 64, True, None),                      # models.py:17-19
    "f_masked_attn_manual": ([1], 64, 64, 32, True, 0.17677669),              # fused.py:31-36: scores above the diagonal filled
}


# The same scalar loops on 16-bit buffers (loads widened to fp32, the result rounded once at the store): what pins the
# tensor-core attention kernels, which take f16 / bf16 at head sizes 64 and 128, to a kernel the reference compiles.
ATTENTION16 = {   # name: (units shape, seq_q, seq_k, d, causal, scale, dtype)
    "att16_bf16_causal_d64": ([1, 2], 128, 128, 64, True, None, "bf16"),
    "att16_f16_d128": ([2], 128, 128, 128, False, None, "f16"),
    # long enough for the two-tile kernel (eight key tiles): run on the GPU only, next to both kernel forms
    "att16_bf16_s1024_d128": ([2], 1024, 1024, 128, False, None, "bf16"),
    "att16_bf16_causal_s1024_d128": ([2], 1024, 1024, 128, True, None, "bf16"),
    # one unit of configuration 5 (4096 x 4096 x 128, bf16)
    "att16_bf16_s4096_d128": ([1], 4096, 4096, 128, False, None, "bf16"),
}


def assert_indices_are_axes(graph, kernel) -> None:
    """Every Load / Write index of a scalar-loop kernel is a bare axis variable with the buffer's own extent."""
    shapes = {t.name: [d.as_static() for d in t.shape] for nd in graph.nodes.values() for t in nd.outputs}
    tile = kernel.body[0]
    extent = {a.name: a.extent.as_static() for a in tile.axes}
    for s in ir_walk(tile.body):
        if type(s).__name__ == "Loop":
            extent[s.axis.name] = s.axis.extent.as_static()
    cells = 1
    for a in tile.axes:
        cells *= a.extent.as_static()
    assert cells % 256 == 0
    for s in ir_walk(tile.body):
        kind = type(s).__name__
        if kind in ("Load", "Write"):
            buf, idx = (s.input, s.index) if kind == "Load" else (s.output, s.index)
            assert len(idx) == len(shapes[buf])
            for e, dim in zip(idx, shapes[buf]):
                assert type(e).__name__ == "Var" and extent[e.name] == dim, (kind, buf, e)


def _max_index(e, hi: dict) -> int:
    """Largest value of an index expression over the axis ranges `hi` (name -> largest value); the expressions the
    builder writes are sums and products of non-negative terms, so the maximum is reached at the axes' maxima."""
    kind = type(e).__name__
    if kind == "Literal":
        return int(e.value)
    if kind == "Var":
        return hi[e.name]
    if kind == "BinaryExpr" and e.op in ("+", "*"):
        a, b = _max_index(e.left, hi), _max_index(e.right, hi)
        return a + b if e.op == "+" else a * b
    raise SystemExit(f"unexpected index expression {e!r}")


def assert_in_range(graph, kernel, m, n, k) -> None:
    """Every fragment access of a guard-free GEMM stays inside its buffer: the cell's base index plus the fragment's
    own extent (16 x 16 for A, 16 x 8 for B in either storage order, 16 x 8 for C; emmyptx/mma.py:6-10)."""
    assert m % 16 == 0 and n % 8 == 0 and k % 16 == 0, "device cases carry no guards"
    shapes = {t.name: [d.as_static() for d in t.shape] for nd in graph.nodes.values() for t in nd.outputs}
    tile = kernel.body[0]
    hi = {a.name: a.extent.as_static() - 1 for a in tile.axes}
    for s in ir_walk(tile.body):
        kind = type(s).__name__
        if kind in ("Loop",):
            hi[s.axis.name] = s.axis.extent.as_static() - 1
    for s in ir_walk(tile.body):
        kind = type(s).__name__
        if kind == "LdmatrixLoad":
            assert s.gmem_guard is None and s.k_zero is None
            shape, idx = shapes[s.src_buffer], s.src_index
            span = (15, 15) if s.role == "a" else ((7, 15) if s.b_trans else (15, 7))
        elif kind == "RegStore":
            assert s.m_guard is None and s.n_guard is None
            shape, idx, span = shapes[s.dst_buffer], s.dst_index, (15, 7)
        else:
            continue
        top = [_max_index(e, hi) for e in idx]
        top[-2] += span[0]
        top[-1] += span[1]
        assert len(top) == len(shape) and all(0 <= t < d for t, d in zip(top, shape)), (kind, top, shape)


def ir_walk(body):
    for s in body:
        yield s
        sub = getattr(s, "body", None)
        if isinstance(sub, list):
            yield from ir_walk(sub)


manifest = {}
for name, (m, n, k, dtype, b_trans, batch, device) in GEMMS.items():
    out_dtype, split_k = GEMM_OUT.get(name, (None, 1))
    graph, kernel, launch = ir.gemm_kernel(m, n, k, dtype, None, b_trans, name=name, batch=batch, out_dtype=out_dtype, split_k=split_k)
    if device:
        assert_in_range(graph, kernel, m, n, k)
    CASES[name] = (graph, kernel, launch)

for name, (units, sq, sk, d, causal, scale) in ATTENTION.items():
    graph, kernel, launch = ir.attention_scalar_kernel(units, sq, sk, d, "f32", scale, causal, name=name)
    assert_indices_are_axes(graph, kernel)
    CASES[name] = (graph, kernel, launch)

for name, (units, sq, sk, d, causal, scale, dtype) in ATTENTION16.items():
    graph, kernel, launch = ir.attention_scalar_kernel(units, sq, sk, d, dtype, scale, causal, name=name)
    assert_indices_are_axes(graph, kernel)
    CASES[name] = (graph, kernel, launch)

LAYOUT = ["s_transpose", "s_permute", "s_slice", "s_strided_slice", "s_flip", "s_stack", "s_tril", "s_cat_a", "s_cat_b",      # shapes.py:6-19
          "s_roll", "s_embedding", "s_gather", "s_tril_select", "s_window_let", "s_cat_cond", "s_pad_cond",
          "c_avg_pool1d", "c_max_pool2d"]                                                                              # conv.py:8-9
for name in LAYOUT:
    graph, kernel, launch = ir.layout_kernel(name, name=name)
    assert launch["grid"][0] * launch["block"][0] >= 1
    CASES[name] = (graph, kernel, launch)

CONV = ["c_conv1d", "c_conv2d"]                                                                                         # conv.py:6-7
for name in CONV:
    CASES[name] = ir.conv_kernel(name, name=name)

# Row and column reductions / normalisations (tools/torch_cases/reductions.py, fused.py) in the one-thread-per-row form, and
# the float32 products written as scalar loops (matmul.py:9-14): compiled by the reference as they are, executed on the CPU
# into golden vectors and on the GPU next to this library's kernels.
ROWS = ["sum", "mean", "amax", "amin", "prod", "norm2", "var", "std", "logsumexp", "softmax", "log_softmax", "layer_norm", "rms_norm",
        "normalize", "dot"]
COLS = ["sum", "amax", "softmax"]
REDUCE = {}
for op in ROWS:
    REDUCE[f"row_{op}"] = ir.rowwise_kernel(op, 64, 256, name=f"row_{op}")
for op in COLS:
    REDUCE[f"col_{op}"] = ir.colwise_kernel(op, 256, 64, name=f"col_{op}")
REDUCE["m_mm"] = ir.matmul_f32_kernel(128, 80, 96, name="m_mm")
REDUCE["m_bmm"] = ir.matmul_f32_kernel(64, 48, 32, batch=4, name="m_bmm")
REDUCE["m_linear_bias_relu"] = ir.matmul_f32_kernel(64, 96, 128, b_trans=True, bias=True, relu=True, name="m_linear_bias_relu")
REDUCE["m_transpose_lhs"] = ir.matmul_f32_kernel(128, 80, 96, a_trans=True, name="m_transpose_lhs")
CASES.update(REDUCE)

# The pointwise and dtype cases as elementwise kernels (tests/elementwise_cases.py): only ever run on the GPU next to this
# library's kernels (no CPU golden vectors: the interpreter does not model every approximation these use).
sys.path.insert(0, str(HERE.parent))
import elementwise_cases  # noqa: E402

ELEMENTWISE = {}
for case, (ins, steps, _expr, _tol) in elementwise_cases.CASES.items():
    ELEMENTWISE[f"ew_{case}"] = ir.elementwise_kernel(4096, ins, steps, elementwise_cases.OUT_DTYPE.get(case, "f32"), name=f"ew_{case}")
for case, (steps, in_dt, out_dt, ins) in elementwise_cases.INT_CASES.items():
    ELEMENTWISE[f"ew_{case}"] = ir.int_elementwise_kernel(4096, steps, in_dt, out_dt, ins, name=f"ew_{case}")
for case, (loads, steps, ins, _expr) in elementwise_cases.BCAST_CASES.items():
    ELEMENTWISE[f"bc_{case}"] = ir.broadcast_kernel(*elementwise_cases.BCAST_SHAPE, loads, steps, ins, name=f"bc_{case}")
for case in elementwise_cases.SCALAR_CASES:
    ELEMENTWISE[case] = elementwise_cases.scalar_kernel(ir, case)
ELEMENTWISE["ew_d_bool_in"] = ir.elementwise_kernel(4096, *elementwise_cases.BOOL_IN, name="ew_d_bool_in")
CASES.update(ELEMENTWISE)

for name, (graph, kernel, launch) in CASES.items():
    ptx = compile_kernel(graph, kernel, launch, target="sm_89")
    (HERE / f"{name}.ref.ptx").write_text(ptx)
    manifest[name] = {"entry": kernel.name, "launch": launch, **({"gemm": dict(zip(("m", "n", "k", "dtype", "b_trans", "batch", "device"), GEMMS[name]), out_f32=name in GEMM_OUT,
                                       split_k=GEMM_OUT.get(name, (None, 1))[1])} if name in GEMMS else {}),
                      **({"attention": dict(zip(("units", "seq_q", "seq_k", "d", "causal", "scale"), ATTENTION[name]))} if name in ATTENTION else {}),
                      **({"attention": dict(zip(("units", "seq_q", "seq_k", "d", "causal", "scale", "dtype"), ATTENTION16[name]))} if name in ATTENTION16 else {}),
                      **({"layout": True} if name in LAYOUT or name in CONV else {}),
                      **({"seeded": True} if name in REDUCE else {}),
                      **({"elementwise": True} if name in ELEMENTWISE else {}),
                      "tensors": {t.name: {"shape": [d.as_static() for d in t.shape], "dtype": t.dtype.name}
                                  for n in graph.nodes.values() for t in n.outputs}}
    print(f"{name}: {len(ptx.splitlines())} lines of PTX")
(HERE / "reference_ptx_manifest.json").write_text(json.dumps(manifest, indent=1) + "\n")
