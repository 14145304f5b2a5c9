"""Kernel against kernel: the reference's own PTX (tests/golden/*.ref.ptx, printed by the reference's compiler)
JIT-loaded on this GPU through the driver API, as the reference's runner does (tools/run_local.py:64-72,
:100-102), next to the sm_100a kernels on the same device buffers.

The reference text targets sm_89; the driver JITs it forward. Only the two streaming kernels are run: straight
line code with in-range addresses by construction (grid * block == n, indices masked to n - 1).
"""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def run_ptx(ptx: str, entry: str, ptrs: list, grid: int, block: int) -> None:
    from emmyptx.ptx_driver import PtxModule
    with PtxModule(ptx) as m:
        m.launch(m.function(entry), ptrs, grid, block)
        m.synchronize()


@pytest.fixture(scope="module")
def manifest():
    return json.loads((GOLDEN / "reference_ptx_manifest.json").read_text())


def _reference_kernel(case, manifest, x_dev, cuda):
    import torch
    torch.cuda.synchronize()
    info = manifest[case]
    y = torch.zeros_like(x_dev)                      # outputs start zeroed (tools/run_local.py:92-93)
    run_ptx((GOLDEN / f"{case}.ref.ptx").read_text(), info["entry"], [x_dev.data_ptr(), y.data_ptr()],
            info["launch"]["grid"][0], info["launch"]["block"][0])
    return y


def test_gather_bit_exact_against_the_reference_kernel(manifest, cuda):
    import torch
    from emmyptx import runtime
    x = torch.from_numpy(inputs.c2_input(2**20)).to(cuda)
    theirs = _reference_kernel("c2_gather_n1048576", manifest, x, cuda)
    ours = runtime.index_gather(x, 7919, 13, 3, 2, trunc=True)
    assert torch.equal(ours, theirs)
    # and the CPU interpreter of the same PTX agrees with the GPU's execution of it
    g = np.load(GOLDEN / "golden.npz")
    assert np.array_equal(theirs.cpu().numpy()[g["c2_gather_n1048576.index"]], g["c2_gather_n1048576.y"])


def test_pointwise_against_the_reference_kernel(manifest, cuda):
    import torch
    from emmyptx import runtime
    x_np = inputs.c1_input(2**20)
    x = torch.from_numpy(x_np).to(cuda)
    theirs = _reference_kernel("c1_exp_sin_tanh_n1048576", manifest, x, cuda).cpu().numpy()
    ours = runtime.pointwise("exp_sin_tanh", x).cpu().numpy()
    ref = reference.c1_f64(x_np)
    assert reference.compare(theirs, ref, 1e-5, 1e-5)["ok"]          # the reference meets its own class here
    assert reference.compare(ours, theirs, 1e-5, 1e-5)["ok"]         # and the two kernels agree within it
    # ours is the tighter of the two against float64
    assert np.abs(ours - ref).max() <= np.abs(theirs - ref).max()
    assert reference.c1_condition_ulp(ours, x_np).max() <= reference.c1_condition_ulp(theirs, x_np).max()
