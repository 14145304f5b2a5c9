"""Build the kernel library: every .cu under csrc/ -> lib/libemmyb200.so, for sm_100a only.

    python build.py [--force] [--verbose]

One nvcc process per translation unit (in parallel), then one link. Objects are rebuilt when
their source, a header they might include, or this script is newer. The library links the CUDA
runtime statically and looks the one driver entry point it needs (cuTensorMapEncodeTiled) and the
run-time compiler (libnvrtc, for elementwise programs) up at run time, so it loads on a machine without a
GPU driver and fails only when a kernel is asked for.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "lib" / "libemmyb200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v", "-I", str(OBJ)]


def _newest_header() -> float:
    deps = [*CSRC.glob("*.cuh"), *CSRC.glob("*.h"), HERE.parent / "include" / "emmyb200.h", Path(__file__)]
    return max(p.stat().st_mtime for p in deps)


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _newest_header()):
        return obj
    cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ / (src.stem + ".ptxas.log")).write_text(r.stderr)
    if r.returncode:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def _embed_math_header() -> None:
    """emmy_math.cuh as a string literal: the kernels compiled at run time (pointwise_jit.cu) include it by name."""
    text = (CSRC / "emmy_math.cuh").read_text()
    assert ')EMMYTEXT"' not in text
    inc = OBJ / "emmy_math_text.inc"
    body = 'R"EMMYTEXT(' + text + ')EMMYTEXT"\n'
    if not inc.exists() or inc.read_text() != body:
        inc.write_text(body)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    _embed_math_header()
    sources = sorted(CSRC.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), sources))
    if force or not LIB.exists() or LIB.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"link failed:\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas resource usage")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
