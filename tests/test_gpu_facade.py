"""End to end through the reference-facing API, the way the reference's harness drives it
(tools/check_torch.py:281-295): IR file + meta.json -> `compile.py` as a subprocess -> the artefact text ->
`run_local.run_kernel(text, k, produced)` -> compare with the float64 oracle on the same seeded inputs.
Also: the kernels against the committed golden vectors (the reference's own output)."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from emmyptx import ir, run_local
from oracle import inputs, reference

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
COMPILE = ROOT / "emmy-ptx-compiler_b200" / "compile.py"
GOLDEN = Path(__file__).resolve().parent / "golden"


def compile_and_run(tmp_path, built, args, extra=()):
    g, k, launch = built
    (tmp_path / f"{k.name}.ir.json").write_text(json.dumps(g.to_dict()))
    entry = dict(launch, args=args)
    (tmp_path / "meta.json").write_text(json.dumps({"kernels": [entry]}))
    r = subprocess.run([sys.executable, str(COMPILE), str(tmp_path / f"{k.name}.ir.json"), *extra], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert run_local.init() == "sm_100"
    return run_local.run_kernel(r.stdout, entry, {})


def seeded(seed, shape, dtype="f32"):
    """Graph input number `seed` as the reference's runner makes it (tools/run_local.py:86-87)."""
    return run_local.to_device(np.random.default_rng(seed).standard_normal(shape), dtype)


def test_pointwise_through_the_facade(tmp_path, cuda):
    n = 50_000
    out = compile_and_run(tmp_path, ir.pointwise_kernel(n), [
        {"name": "x", "dtype": "f32", "shape": [n], "seed": 0}, {"name": "y", "dtype": "f32", "shape": [n], "output": True}])
    x = seeded(0, [n])
    assert reference.compare(out["y"], reference.c1_f64(x), 1e-5, 1e-5)["ok"]


def test_gather_through_the_facade_both_division_modes(tmp_path, cuda):
    n = 2**18
    x = inputs.c2_input(n)
    args = [{"name": "x", "dtype": "i32", "shape": [n], "data": x.tolist()}, {"name": "y", "dtype": "i32", "shape": [n], "output": True}]
    out = compile_and_run(tmp_path, ir.index_gather_kernel(n), args)
    assert np.array_equal(out["y"], reference.c2_reference(x))
    out = compile_and_run(tmp_path, ir.index_gather_kernel(n), args, extra=("--int-div", "trunc"))
    assert np.array_equal(out["y"], reference.c2_reference(x, trunc=True))


@pytest.mark.parametrize("dtype,epilogue,b_trans,tol", [("f16", None, False, (2e-2, 1e-1)), ("bf16", None, False, (5e-2, 5e-1)),
                                                         ("f16", None, True, (2e-2, 1e-1)), ("bf16", "gelu_tanh", False, (5e-2, 5e-1))])
def test_gemm_through_the_facade_reference_tolerances(tmp_path, cuda, dtype, epilogue, b_trans, tol):
    """Un-normalised randn operands and the reference's tensor-core tolerances (tools/torch_cases/matmul.py:5-7)."""
    import torch
    m, n, k = 256, 512, 512
    bshape = [n, k] if b_trans else [k, n]
    out = compile_and_run(tmp_path, ir.gemm_kernel(m, n, k, dtype, epilogue, b_trans), [
        {"name": "A", "dtype": dtype, "shape": [m, k], "seed": 0}, {"name": "B", "dtype": dtype, "shape": bshape, "seed": 1},
        {"name": "C", "dtype": dtype, "shape": [m, n], "output": True}])
    td = torch.float16 if dtype == "f16" else torch.bfloat16
    a = torch.from_numpy(np.random.default_rng(0).standard_normal((m, k)).astype(np.float32)).to(td)
    b = torch.from_numpy(np.random.default_rng(1).standard_normal(bshape).astype(np.float32)).to(td)
    ref = reference.gemm_reference(a, b, epilogue, b_is_nk=b_trans, double=True).numpy()
    res = reference.compare(np.asarray(out["C"], dtype=np.float64), ref, *tol)
    assert res["ok"], res


def test_attention_through_the_facade(tmp_path, cuda):
    import torch
    shp = [2, 3, 256, 128]
    out = compile_and_run(tmp_path, ir.attention_kernel([2, 3], 256, 256, 128, "bf16"), [
        {"name": n, "dtype": "bf16", "shape": shp, "seed": i} for i, n in enumerate("QKV")] +
        [{"name": "O", "dtype": "bf16", "shape": shp, "output": True}])
    q, k, v = (torch.from_numpy(np.random.default_rng(i).standard_normal(shp).astype(np.float32)).bfloat16() for i in range(3))
    ref = reference.attention_reference(q, k, v, double=True).numpy()
    assert reference.compare(out["O"].reshape(shp).astype(np.float64), ref, 1e-2, 1e-2)["ok"]       # HALF class


def test_causal_attention_through_the_facade(tmp_path, cuda):
    import torch
    shp = [4, 200, 64]
    out = compile_and_run(tmp_path, ir.attention_kernel([4], 200, 200, 64, "f16", causal=True), [
        {"name": n, "dtype": "f16", "shape": shp, "seed": i} for i, n in enumerate("QKV")] +
        [{"name": "O", "dtype": "f16", "shape": shp, "output": True}])
    q, k, v = (torch.from_numpy(np.random.default_rng(i).standard_normal(shp).astype(np.float32)).half().double() for i in range(3))
    scores = (q @ k.transpose(-1, -2)) * 64 ** -0.5
    scores = scores.masked_fill(~torch.ones(200, 200, dtype=torch.bool).tril(), float("-inf"))
    ref = (torch.softmax(scores, -1) @ v).numpy()
    assert reference.compare(out["O"].reshape(shp).astype(np.float64), ref, 1e-2, 1e-2)["ok"]       # HALF class


@pytest.mark.parametrize("op,rows,cols,rtol,atol", [
    ("mean", 128, 300, 1e-4, 1e-4), ("var", 64, 512, 1e-4, 1e-4), ("logsumexp", 64, 512, 1e-4, 1e-4),
    ("softmax", 64, 1000, 1e-3, 1e-5), ("layer_norm", 64, 768, 1e-3, 1e-4), ("rms_norm", 32, 512, 1e-3, 1e-4)])
def test_row_kernels_through_the_facade(tmp_path, cuda, op, rows, cols, rtol, atol):
    """r_mean_rows, r_var_std, r_logsumexp, f_softmax, f_layer_norm_affine, f_rms_norm (tools/torch_cases/reductions.py,
    fused.py) at the reference's tolerances."""
    import torch
    built = ir.rowwise_kernel(op, rows, cols, eps=1e-5)
    names = [t for t in built[2]["arg_order"] if t != "Y"]
    shapes = {"X": [rows, cols], "W": [cols], "B": [cols]}
    is_map = op in ("softmax", "layer_norm", "rms_norm")
    out = compile_and_run(tmp_path, built, [{"name": n, "dtype": "f32", "shape": shapes[n], "seed": i} for i, n in enumerate(names)] +
                          [{"name": "Y", "dtype": "f32", "shape": [rows, cols] if is_map else [rows], "output": True}])
    t = {n: torch.from_numpy(seeded(i, shapes[n])) for i, n in enumerate(names)}
    ref = reference.rowwise_reference(op, t["X"], t.get("W"), t.get("B"), 1e-5).numpy()
    assert reference.compare(out["Y"], ref, rtol, atol)["ok"]


@pytest.mark.parametrize("op,rtol,atol", [("sum", 1e-4, 1e-4), ("softmax", 1e-3, 1e-5)])
def test_dim0_kernels_through_the_facade(tmp_path, cuda, op, rtol, atol):
    """r_sum_dim0 and f_softmax_dim0 (tools/torch_cases/reductions.py:9, fused.py:7)."""
    import torch
    rows, cols = 256, 64
    out_shape = [rows, cols] if op == "softmax" else [cols]
    out = compile_and_run(tmp_path, ir.colwise_kernel(op, rows, cols), [
        {"name": "X", "dtype": "f32", "shape": [rows, cols], "seed": 0}, {"name": "Y", "dtype": "f32", "shape": out_shape, "output": True}])
    x = torch.from_numpy(seeded(0, [rows, cols]))
    assert reference.compare(out["Y"], reference.colwise_reference(op, x).numpy(), rtol, atol)["ok"]


@pytest.mark.parametrize("kw", [dict(m=128, n=80, k=96), dict(m=64, n=48, k=32, batch=4), dict(m=64, n=48, k=32, batch=4, b_batched=False),
                                dict(m=64, n=96, k=128, b_trans=True, bias=True)])
def test_float32_matmul_through_the_facade(tmp_path, cuda, kw):
    """m_mm, m_bmm, m_bcast_matmul, m_linear_bias at the reference's MM class (rtol = atol = 1e-3)."""
    import torch
    built = ir.matmul_f32_kernel(**kw)
    tensors = {t.name: [int(d.as_static()) for d in t.shape] for node in built[0].nodes.values() for t in node.outputs}
    names = [nm for nm in built[2]["arg_order"] if nm != "C"]
    out = compile_and_run(tmp_path, built, [{"name": nm, "dtype": "f32", "shape": tensors[nm], "seed": i} for i, nm in enumerate(names)] +
                          [{"name": "C", "dtype": "f32", "shape": tensors["C"], "output": True}])
    t = {nm: torch.from_numpy(seeded(i, tensors[nm])).double() for i, nm in enumerate(names)}
    b = t["B"].transpose(-1, -2) if kw.get("b_trans") else t["B"]
    ref = t["A"] @ b + (t["bias"] if "bias" in t else 0.0)
    assert reference.compare(out["C"].reshape(ref.shape), ref.numpy(), 1e-3, 1e-3)["ok"]


def test_kernels_against_the_reference_golden_vectors(cuda):
    """golden.npz is the reference's own PTX executed on these inputs. Integer kernel in the reference's
    (truncating) mode: bit for bit. Float kernels: within the reference's tolerance class of each other."""
    import torch
    from emmyptx import runtime
    g = np.load(GOLDEN / "golden.npz")
    x = inputs.c2_input(2**16)
    y = runtime.index_gather(torch.from_numpy(x).to(cuda), 7919, 13, 3, 2, trunc=True).cpu().numpy()
    assert np.array_equal(y, g["c2_gather_n65536.y"])
    x = inputs.c2_input(2**20)
    y = runtime.index_gather(torch.from_numpy(x).to(cuda), 7919, 13, 3, 2, trunc=True).cpu().numpy()
    assert np.array_equal(y[g["c2_gather_n1048576.index"]], g["c2_gather_n1048576.y"])
    xf = inputs.c1_input(4096)
    for case, op in (("c1_exp_sin_tanh_n4096", "exp_sin_tanh"), ("p_exp_n4096", "exp"), ("p_tanh_n4096", "tanh"), ("p_sin_n4096", "sin")):
        y = runtime.pointwise(op, torch.from_numpy(xf).to(cuda)).cpu().numpy()
        assert reference.compare(y, g[f"{case}.y"], 1e-5, 1e-5)["ok"], case


def test_handle_for_another_entry_is_refused(cuda):
    from emmyptx.kernel import compile_kernel
    text = compile_kernel(*ir.pointwise_kernel(64))
    with pytest.raises(RuntimeError, match="asked for"):
        run_local.load(text, "some_other_entry")
    with pytest.raises(RuntimeError, match="not a kernel handle"):
        run_local.load(".version 8.0", "k_pointwise")


def test_batched_matmul_and_linear_bias_through_the_facade(tmp_path, cuda):
    """m_f16_bmm (tools/torch_cases/matmul.py:31) and a 16-bit F.linear with bias and ReLU: randn operands, the
    reference's tensor-core tolerance (rtol 2e-2, atol 1e-1) against float64."""
    import torch
    out = compile_and_run(tmp_path, ir.gemm_kernel(128, 96, 64, "f16", batch=(4,)), [
        {"name": "A", "dtype": "f16", "shape": [4, 128, 64], "seed": 0}, {"name": "B", "dtype": "f16", "shape": [4, 64, 96], "seed": 1},
        {"name": "C", "dtype": "f16", "shape": [4, 128, 96], "output": True}])
    a = torch.from_numpy(seeded(0, [4, 128, 64], "f16")).double()
    b = torch.from_numpy(seeded(1, [4, 64, 96], "f16")).double()
    assert reference.compare(np.asarray(out["C"], np.float64).reshape(4, 128, 96), torch.bmm(a, b).numpy(), 2e-2, 1e-1)["ok"]

    out = compile_and_run(tmp_path, ir.gemm_kernel(64, 512, 256, "f16", "relu", True, bias=True, name="k_linear"), [
        {"name": "A", "dtype": "f16", "shape": [64, 256], "seed": 0}, {"name": "B", "dtype": "f16", "shape": [512, 256], "seed": 1},
        {"name": "bias", "dtype": "f16", "shape": [512], "seed": 2}, {"name": "C", "dtype": "f16", "shape": [64, 512], "output": True}])
    x, w, bias = (torch.from_numpy(seeded(i, shp, "f16")).double() for i, shp in enumerate(([64, 256], [512, 256], [512])))
    ref = torch.relu(torch.nn.functional.linear(x, w, bias)).numpy()
    assert reference.compare(np.asarray(out["C"], np.float64).reshape(64, 512), ref, 2e-2, 1e-1)["ok"]


def test_split_k_and_fp32_attention_through_the_facade(tmp_path, cuda):
    """A split-K contraction (f32 C, red.add.f32 in the reference, emmyptx/mma.py:239-240) and the reference's fp32
    attention cases (tools/torch_cases/fused.py:21-22; models.py:17-19) from IR file to result."""
    import torch
    out = compile_and_run(tmp_path, ir.gemm_kernel(128, 96, 256, "bf16", out_dtype="f32", split_k=4, name="k_splitk"), [
        {"name": "A", "dtype": "bf16", "shape": [128, 256], "seed": 0}, {"name": "B", "dtype": "bf16", "shape": [256, 96], "seed": 1},
        {"name": "C", "dtype": "f32", "shape": [128, 96], "output": True}])
    a = torch.from_numpy(run_local.from_device(seeded(0, [128, 256], "bf16"), "bf16")).double()
    b = torch.from_numpy(run_local.from_device(seeded(1, [256, 96], "bf16"), "bf16")).double()
    assert np.allclose(np.asarray(out["C"], np.float64).reshape(128, 96), (a @ b).numpy(), rtol=1e-5, atol=1e-4)

    for name, units, s, d, causal in (("f_sdpa", [1, 2], 64, 32, False), ("t_causal_sdpa", [1, 4], 128, 64, True)):
        u = int(np.prod(units))
        out = compile_and_run(tmp_path, ir.attention_scalar_kernel(units, s, s, d, causal=causal, name=name), [
            *[{"name": nm, "dtype": "f32", "shape": [u, s, d], "seed": i} for i, nm in enumerate("QKV")],
            {"name": "O", "dtype": "f32", "shape": [u, s, d], "output": True}])
        q, k, v = (torch.from_numpy(np.asarray(seeded(i, [u, s, d]), np.float32)) for i in range(3))
        ref = reference.attention_reference(q, k, v, double=True, causal=causal).numpy()
        assert reference.compare(np.asarray(out["O"], np.float64).reshape(u, s, d), ref, 1e-3, 1e-3)["ok"]       # MM class
        assert np.allclose(np.asarray(out["O"], np.float64).reshape(u, s, d), ref, rtol=1e-5, atol=1e-5)

