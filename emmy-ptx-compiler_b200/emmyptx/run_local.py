"""Run compiled kernels on the local GPU: the counterpart of the reference's `tools/run_local.py`.

Same roles, same names: `init()` (`run_local.py:51-61`), `load(text, entry)` (`:64-72`) and
`run_kernel(text, k, produced)` (`:75-113`), where `text` is what `compile.py` printed -- PTX in the
reference, a kernel handle here -- and `k` is the kernel's entry of `meta.json`: `args` in parameter order,
each with `name`, `dtype`, `shape` and one of `seed` (input number: `default_rng(seed).standard_normal`),
`data`, `intermediate` (produced by an earlier kernel of the problem) or nothing (zeroed), and `output`.
`run_problem(pdir, target, level)` (`:116-141`) runs a problem folder -- `meta.json` (the kernels in launch order,
`rtol`, `atol`), one `<entry>.ir.json` per kernel, `expected.npz` -- compiling each kernel with this package's
`compile.py`, feeding every output forward by name and checking the ones `expected.npz` holds; `main()` is the same
command line (`python -m emmyptx.run_local <problems folder> [--only PREFIX] [--level N]`, `:144-160`).
Buffers are created the way the reference's runner creates them, live in device memory for the duration of
the call, and outputs come back as numpy arrays (bf16 widened to float32, as `from_device` does).
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

from . import runtime

ROOT = Path(__file__).resolve().parent.parent          # the folder that holds compile.py

DTYPES = {"f32": np.float32, "f16": np.float16, "f64": np.float64, "i32": np.int32, "i64": np.int64,
          "bool": np.bool_, "bf16": np.uint16}


def to_device(values, dtype: str) -> np.ndarray:
    """`values` as the host image of a `dtype` buffer; bf16 is the upper half of the fp32 bits, rounded to
    nearest even (`tools/run_local.py:31-37`)."""
    if dtype != "bf16":
        return np.asarray(values).astype(DTYPES[dtype])
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def from_device(raw: np.ndarray, dtype: str) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32) if dtype == "bf16" else raw


def init() -> str:
    """Make GPU 0 current and return its target name ('sm_100'); raises without a CUDA device."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(0)
    major, minor = torch.cuda.get_device_capability(0)
    runtime.library()
    return f"sm_{major}{minor}"


def load(text: str, entry: str) -> dict:
    """Parse a kernel handle and check that it is the one for `entry`."""
    try:
        handle = json.loads(text)
    except json.JSONDecodeError as e:
        raise RuntimeError(f"not a kernel handle: {e}") from None
    if handle.get("emmyb200_handle") != 1 or handle.get("entry") != entry:
        raise RuntimeError(f"kernel handle is for entry {handle.get('entry')!r}, asked for {entry!r}")
    return handle


def _torch_view(host: np.ndarray, dtype: str):
    import torch
    t = torch.from_numpy(host)
    return t.view(torch.bfloat16) if dtype == "bf16" else t


def run_kernel(text: str, k: dict, produced: dict) -> dict:
    """Launch one kernel of a problem; return its outputs by name."""
    import torch
    handle = load(text, k["entry"])
    dev = torch.device("cuda", torch.cuda.current_device())
    bufs, meta, scalars = {}, {}, {}
    for a in k["args"]:
        if a.get("scalar"):                     # passed by value (tools/run_local.py:82-83)
            scalars[a["name"]] = a["value"]
            continue
        shape = a["shape"] or [1]
        if "seed" in a:
            host = to_device(np.random.default_rng(a["seed"]).standard_normal(shape), a["dtype"])
        elif "data" in a:
            host = to_device(np.asarray(a["data"]).reshape(shape), a["dtype"])
        elif a.get("intermediate"):
            host = to_device(np.asarray(produced[a["name"]]).reshape(shape), a["dtype"])
        else:
            host = np.zeros(shape, DTYPES[a["dtype"]])
        bufs[a["name"]] = _torch_view(np.ascontiguousarray(host), a["dtype"]).to(dev)
        meta[a["name"]] = a
    order = [a["name"] for a in k["args"]]
    if order != handle["arg_order"]:
        raise RuntimeError(f"kernel arguments {order} do not match the handle's arg_order {handle['arg_order']}")
    launch(handle, bufs, scalars=scalars)
    torch.cuda.synchronize()
    if runtime.device_status() != 0:
        raise RuntimeError("a bounded device-side wait expired")
    outputs = {}
    for a in k["args"]:
        if a.get("output"):
            t = bufs[a["name"]]
            raw = (t.view(torch.uint16) if a["dtype"] == "bf16" else t).cpu().numpy()
            outputs[a["name"]] = from_device(raw, a["dtype"])
    return outputs


def launch(handle: dict, bufs: dict, stream=None, scalars: dict | None = None) -> None:
    """Enqueue the handle's kernel on buffers (CUDA tensors by argument name); `scalars`: the launch's by-value
    arguments by name."""
    p, v = handle["params"], handle["variant"]
    if v == "pointwise_program" and p["program"].get("scalar_consts"):
        prog = dict(p["program"], consts=list(p["program"]["consts"]))
        for name, idx, _ in prog["scalar_consts"]:
            if scalars is None or name not in scalars:
                raise RuntimeError(f"scalar argument {name!r} has no value")
            prog["consts"][idx] = float(scalars[name])
        p = dict(p, program=prog)
    ins = [bufs[n] for n in handle["inputs"]]
    out = bufs[handle["outputs"][0]]
    if v == "pointwise_f32":
        runtime.pointwise(p["op"], ins[0].reshape(-1), out=out.reshape(-1), stream=stream)
    elif v == "pointwise_program":
        runtime.pointwise_program(p["program"], [t.reshape(-1) for t in ins], out.reshape(-1), stream=stream)
    elif v == "pointwise_indexed":
        flat = iter(t.reshape(-1) for t in ins)
        tensors = [None if "axis" in src else next(flat) for src in p["index_map"]["inputs"]]
        runtime.pointwise_indexed(p["program"], p["index_map"], tensors, out.reshape(-1), stream=stream)
    elif v == "contract_indexed":
        runtime.contract_indexed(p["map"], ins[0].reshape(-1), ins[1].reshape(-1), out.reshape(-1), stream=stream)
    elif v == "index_gather_i32":
        runtime.index_gather(ins[0].reshape(-1), p["mul"], p["add"], p["div"], p["shift"], p["trunc"], out=out.reshape(-1),
                             stream=stream)
    elif v == "gemm":
        runtime.gemm(ins[0], ins[1], epilogue=p["epilogue"], b_is_nk=p["b_trans"], out=out, stream=stream)
    elif v == "gemm_batched":
        a = ins[0].reshape(p["batch"], p["m"], p["k"])
        bshape = (p["n"], p["k"]) if p["b_trans"] else (p["k"], p["n"])
        b = ins[1].reshape(bshape if p["b_shared"] else (p["batch"], *bshape))
        runtime.gemm_batched(a, b, bias=ins[2].reshape(-1) if p["bias"] else None, epilogue=p["epilogue"], b_is_nk=p["b_trans"],
                             out=out.reshape(p["batch"], p["m"], p["n"]), stream=stream)
    elif v == "attention_fwd":
        shp = (p["units"], -1, p["d"])
        runtime.attention(ins[0].reshape(shp), ins[1].reshape(shp), ins[2].reshape(shp), scale=p["scale"],
                          causal=p.get("causal", False), out=out.reshape(shp), stream=stream)
    elif v == "rowwise_f32":
        x = ins[0].reshape(p["rows"], p["cols"])
        runtime.rowwise(p["op"], x, ins[1].reshape(-1) if p["weight"] else None, ins[2].reshape(-1) if p["bias"] else None,
                        p["eps"], out=out.reshape(x.shape if p["op"] in ("softmax", "log_softmax", "layer_norm", "rms_norm", "normalize")
                                                  else (p["rows"],)), stream=stream)
    elif v == "gemm_f32":
        a = ins[0].reshape(p["batch"], p["m"], p["k"])
        bshape = (p["n"], p["k"]) if p["b_trans"] else (p["k"], p["n"])
        b = ins[1].reshape(bshape if p["b_shared"] else (p["batch"], *bshape))
        runtime.gemm_f32(a, b, bias=ins[2].reshape(-1) if p["bias"] else None, epilogue=p["epilogue"], b_is_nk=p["b_trans"],
                         out=out.reshape(p["batch"], p["m"], p["n"]), stream=stream)
    elif v == "colwise_f32":
        x = ins[0].reshape(p["outer"], p["rows"], p["cols"])
        is_map = p["op"] in ("softmax", "log_softmax", "normalize")
        runtime.colwise(p["op"], x, p["eps"], out=out.reshape(x.shape if is_map else (p["outer"], p["cols"])), stream=stream)
    else:
        raise RuntimeError(f"unknown kernel variant {v!r}")


def run_problem(pdir: Path, target: str, level: int | None = None) -> tuple[bool, str]:
    """Compile and run the kernels of one problem folder in order; (passed, one line of detail). Outputs are kept by
    name for later kernels (`intermediate` arguments) and compared with `expected.npz` where it has them."""
    pdir = Path(pdir)
    meta = json.loads((pdir / "meta.json").read_text())
    with np.load(pdir / "expected.npz") as z:
        expected = {name: z[name] for name in z.files}
    produced, lines = {}, []
    for k in meta["kernels"]:
        cmd = [sys.executable, str(ROOT / "compile.py"), str(pdir / f"{k['entry']}.ir.json"), "--target", target]
        if level is not None:
            cmd += ["--level", str(level)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            last = (done.stderr.strip().splitlines() or ["?"])[-1]
            return False, f"compile.py failed: {last}"
        try:
            outputs = run_kernel(done.stdout, k, produced)
        except RuntimeError as e:
            return False, str(e).splitlines()[0]
        produced.update(outputs)
        for name, got in outputs.items():
            if name not in expected:
                continue
            want = expected[name].astype(np.float64)
            have = np.asarray(got).reshape(want.shape).astype(np.float64)
            worst = float(np.abs(have - want).max()) if want.size else 0.0
            if not np.allclose(have, want, rtol=meta["rtol"], atol=meta["atol"]):
                return False, f"{name}: max abs err {worst:.3e} (rtol={meta['rtol']} atol={meta['atol']})"
            lines.append(f"{name}: max abs err {worst:.3e}")
    return True, "; ".join(lines)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Run every problem of a folder on the local GPU.")
    ap.add_argument("problems", type=Path, help="a problems folder")
    ap.add_argument("--only", default="", help="only problems whose name starts with this")
    ap.add_argument("--level", type=int, choices=(0, 1, 2), help="accepted for compatibility; the kernels are prebuilt")
    args = ap.parse_args(argv)
    target = init()
    found = sorted(p for p in args.problems.iterdir() if (p / "meta.json").exists() and p.name.startswith(args.only))
    passed = 0
    for p in found:
        ok, detail = run_problem(p, target, args.level)
        passed += bool(ok)
        print(f"{'PASS' if ok else 'FAIL'}  {p.name:28s} {detail}", flush=True)
    print(f"\n{passed}/{len(found)} passed on the local GPU ({target})")
    return 0 if passed == len(found) else 1


if __name__ == "__main__":
    sys.exit(main())
