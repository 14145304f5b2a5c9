"""Golden vectors: the reference's own PTX (tests/golden/*.ref.ptx) executed on the CPU by
oracle/ptx_interp.py on the seeded inputs of oracle/inputs.py.

    python tests/golden/make_golden.py

Writes tests/golden/golden.npz: for each case the output the reference's kernel produces (`<case>.y`; for the
tensor-core GEMM cases `<case>.c`, the 16-bit output as raw bit patterns, on N(0,1) operands seeded per argument
as oracle/inputs.gemm_inputs(scaled=False) draws them; for the fp32 attention cases `<case>.o`, on the operands of
oracle/inputs.attention_inputs_f32). Integer outputs are exact; float outputs are the reference's algorithm with its three hardware
approximations evaluated correctly rounded (see ptx_interp.py). Regenerate only together with the .ref.ptx
files (make_reference_ptx.py, which needs the reference checkout).
"""
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import inputs, ptx_interp  # noqa: E402

manifest = json.loads((HERE / "reference_ptx_manifest.json").read_text())
out = {}
for name, info in manifest.items():
    if "gemm" in info:
        g = info["gemm"]
        if g["m"] > 512:
            continue                      # device-only timing case
        a, b = inputs.gemm_inputs(g["m"], g["n"], g["k"], g["dtype"], g["b_trans"], scaled=False, batch=tuple(g["batch"]))
        bufs = {"A": a.view(__import__("torch").int16).numpy().copy(), "B": b.view(__import__("torch").int16).numpy().copy(),
                "C": np.zeros(tuple(g["batch"]) + (g["m"], g["n"]), np.float32 if g.get("out_f32") else np.int16)}
        ptx_interp.run_entry((HERE / f"{name}.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
        if g.get("out_f32"):              # the fp32 accumulator itself (a zeroed C and red.add.f32 for the split-K case)
            out[f"{name}.c32"] = bufs["C"]
            print(name, bufs["C"][0, :4])
            continue
        c = bufs["C"].view(np.uint16).reshape(-1, g["n"])
        if c.shape[0] > 128:              # keep the fixture small: every fourth row of the larger cases
            keep = np.arange(0, c.shape[0], 4)
            out[f"{name}.rows"] = keep.astype(np.int64)
            c = c[keep]
        out[f"{name}.c"] = c
        print(name, c[0, :4])
        continue
    if "attention" in info:
        a = info["attention"]
        units = int(np.prod(a["units"]))
        if a["seq_k"] > 256:
            continue                                # too long for the CPU interpreter: compared on the GPU only
        if "dtype" in a:                            # 16-bit buffers as their bit patterns; the golden vector widened to fp32
            import torch
            q, k, v = (t.view(torch.uint16).numpy().copy() for t in inputs.attention_inputs(units, a["seq_q"], a["seq_k"], a["d"], a["dtype"]))
            bufs = {"Q": q, "K": k, "V": v, "O": np.zeros((units, a["seq_q"], a["d"]), np.uint16)}
            ptx_interp.run_entry((HERE / f"{name}.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
            td = torch.float16 if a["dtype"] == "f16" else torch.bfloat16
            out[f"{name}.o"] = torch.from_numpy(bufs["O"]).view(td).float().numpy()
            print(name, out[f"{name}.o"][0, 0, :4])
            continue
        q, k, v = inputs.attention_inputs_f32(units, a["seq_q"], a["seq_k"], a["d"])
        bufs = {"Q": q.copy(), "K": k.copy(), "V": v.copy(), "O": np.zeros((units, a["seq_q"], a["d"]), np.float32)}
        ptx_interp.run_entry((HERE / f"{name}.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
        out[f"{name}.o"] = bufs["O"]
        print(name, bufs["O"][0, 0, :4])
        continue
    if info.get("elementwise"):
        continue                          # run on the GPU only, next to the library's kernels
    if info.get("seeded"):
        bufs = inputs.seeded_buffers(info["tensors"], info["launch"]["arg_order"])
        ptx_interp.run_entry((HERE / f"{name}.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
        result = info["launch"]["arg_order"][-1]
        out[f"{name}.out"] = bufs[result]
        print(name, bufs[result].reshape(-1)[:4])
        continue
    if info.get("layout"):
        bufs = inputs.layout_buffers(info["tensors"], info["launch"]["arg_order"])
        ptx_interp.run_entry((HERE / f"{name}.ref.ptx").read_text(), bufs, info["launch"]["grid"][0], info["launch"]["block"][0])
        out[f"{name}.out"] = bufs["out"]
        print(name, bufs["out"].reshape(-1)[:4])
        continue
    n = info["tensors"]["x"]["shape"][0]
    if n > 2**20 or (name.startswith("c1") and n > 4096 and False):
        continue
    x = inputs.c2_input(n) if info["tensors"]["x"]["dtype"] == "i32" else inputs.c1_input(n)
    y = np.zeros_like(x)
    grid, block = info["launch"]["grid"][0], info["launch"]["block"][0]
    ptx_interp.run_entry((HERE / f"{name}.ref.ptx").read_text(), {"x": x, "y": y}, grid, block)
    if n > 65536:                         # keep the fixture small: a strided sample of the large cases
        keep = np.arange(0, n, n // 4096)
        out[f"{name}.index"] = keep.astype(np.int64)
        y = y[keep]
    out[f"{name}.y"] = y
    print(name, y[:4])
np.savez_compressed(HERE / "golden.npz", **out)
print("wrote", HERE / "golden.npz", (HERE / "golden.npz").stat().st_size, "bytes")
