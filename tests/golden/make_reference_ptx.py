"""Generate the reference's own PTX for the two streaming configurations (and a small GEMM), as fixtures.

    python tests/golden/make_reference_ptx.py <path to a checkout of the reference>

Needs the reference checkout (read-only) and nothing else: its `KernelCompiler` dispatches on class *names*, so
the stand-in IR classes of `emmy-ptx-compiler_b200/emmyptx/ir.py` drive it. The PTX text it prints is the
reference's output for these kernels; `oracle/ptx_interp.py` executes it on the CPU to produce the golden
vectors (`make_golden.py`), and the GPU tests JIT the same text on the device to compare kernel against kernel.
Targets are sm_89 (the reference's default); sm_100 devices JIT it forward.
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

manifest = {}
for name, (graph, kernel, launch) in CASES.items():
    ptx = compile_kernel(graph, kernel, launch, target="sm_89")
    (HERE / f"{name}.ref.ptx").write_text(ptx)
    manifest[name] = {"entry": kernel.name, "launch": launch,
                      "tensors": {t.name: {"shape": [d.as_static() for d in t.shape], "dtype": t.dtype.name}
                                  for n in graph.nodes.values() for t in n.outputs}}
    print(f"{name}: {len(ptx.splitlines())} lines of PTX")
(HERE / "reference_ptx_manifest.json").write_text(json.dumps(manifest, indent=1) + "\n")
