"""Compile one Emmy Kernel IR file to a kernel handle for the sm_100a kernel library.

    python compile.py path/to/<kernel>.ir.json > out.handle.json
    python compile.py path/to/<kernel>.ir.json --target sm_100a

Same command line as the reference's compile.py (compile.py:34-57): the launch descriptor `meta.json` next
to the IR supplies the parameter order (`arg_order`); exactly one KernelOp per file; the artefact goes to
stdout, diagnostics to stderr, and the exit status says whether it compiled. The artefact is a kernel handle
(see emmyptx/kernel.py), not PTX. The IR is loaded with the tracer package's Graph when it is installed, and
with the stand-in classes of emmyptx/ir.py otherwise.
"""

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from emmyptx.kernel import TARGET, CompileError, KernelCompiler, compile_kernel  # noqa: E402

try:
    from emmy.compiler.graph import Graph
except ImportError:
    from emmyptx.ir import Graph


def find_launch(meta: dict | None, kernel, graph) -> dict:
    """The launch descriptor for `kernel` (same contract as the reference's compile.py:21-31).

    Looked up in `meta["kernels"]` by entry name; a meta file that describes a single kernel is taken to mean this
    one whatever it is called. With no usable meta the descriptor is derived from the graph: parameters are the
    kernel node's inputs followed by its outputs, 256-thread blocks, an unknown grid (0) and no dynamic shared
    memory -- the handle's own launch geometry does not depend on it.
    """
    described = (meta or {}).get("kernels", [])
    by_name = [entry for entry in described if entry.get("entry") == kernel.name]
    if by_name:
        return by_name[0]
    if len(described) == 1:
        return described[0]
    owner = [node for node in graph.nodes.values() if node.op is kernel][0]
    params = list(owner.inputs) + [tensor.name for tensor in owner.outputs]
    return {"arg_order": params, "block": [256, 1, 1], "grid": [0, 1, 1], "smem_bytes": 0}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("ir", help="a Kernel IR json file (<kernel>.ir.json)")
    ap.add_argument("--target", default=TARGET, help=f"target architecture (only {TARGET})")
    ap.add_argument("--level", type=int, choices=(0, 1, 2), help="accepted for compatibility; the kernels are prebuilt")
    ap.add_argument("--int-div", choices=("floor", "trunc"), default="floor",
                    help="integer // and %%: torch's rounding (default) or the reference PTX's truncation")
    args = ap.parse_args()

    ir_path = Path(args.ir)
    graph = Graph.from_dict(json.loads(ir_path.read_text()))
    kernels = [n.op for n in graph.nodes.values() if type(n.op).__name__ == "KernelOp"]
    if len(kernels) != 1:
        sys.exit(f"expected one KernelOp in {ir_path}, found {len(kernels)}")
    kernel = kernels[0]
    meta_path = ir_path.parent / "meta.json"
    meta = json.loads(meta_path.read_text()) if meta_path.exists() else None
    launch = find_launch(meta, kernel, graph)
    try:
        if args.level is None and args.int_div == "floor":
            text = compile_kernel(graph, kernel, launch, target=args.target)
        else:
            text = KernelCompiler(graph, kernel, launch, args.target, level=2 if args.level is None else args.level,
                                  int_div=args.int_div).compile()
    except CompileError as e:
        sys.exit(f"compile error: {e}")
    sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
