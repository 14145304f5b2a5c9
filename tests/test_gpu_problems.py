"""Problems of several kernels through `run_local.run_problem`: the reference's runner compiles the kernels of a problem
folder one by one, launches them in order and hands every output on by name (tools/run_local.py:116-141). The
problems here have the shape of its composite cases -- a module MLP (tools/torch_cases/models.py:22-26), a Llama-style
feed-forward sublayer (:8-16), a soft-target cross-entropy (fused.py:19-20), addmm (matmul.py:16-17) -- cut into kernels this library has
(float32 products with bias, row normalisations, elementwise programs, row reductions), with seeded inputs, weights
passed as `data`, and torch in float64 as the expected result at the reference's matmul tolerance class."""
import json

import numpy as np
import pytest

from emmyptx import ir, run_local

pytestmark = pytest.mark.gpu
MM = dict(rtol=1e-3, atol=1e-3)           # tools/torch_cases/__init__.py:20


def _arg(name, dtype, shape, **how):
    return dict(name=name, dtype=dtype, shape=list(shape), **how)


def _write_problem(folder, kernels, expected, tol):
    """kernels: [(built, args)], args in the launch's argument order."""
    folder.mkdir(parents=True)
    described = []
    for (graph, kernel, launch), args in kernels:
        assert [a["name"] for a in args] == launch["arg_order"]
        (folder / f"{kernel.name}.ir.json").write_text(json.dumps(graph.to_dict()))
        described.append(dict(launch, args=args))
    (folder / "meta.json").write_text(json.dumps({"kernels": described, **tol}))
    np.savez(folder / "expected.npz", **expected)
    return folder


def _seeded(seed, shape):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def _mlp(folder):
    import torch
    x = _seeded(0, (32, 128))
    rng = np.random.default_rng(10)
    w1, b1 = (rng.standard_normal((256, 128)) / np.sqrt(128)).astype(np.float32), (rng.standard_normal(256) * 0.1).astype(np.float32)
    w2, b2 = (rng.standard_normal((64, 256)) / 16).astype(np.float32), (rng.standard_normal(64) * 0.1).astype(np.float32)
    fc1 = ir.rename_buffers(ir.matmul_f32_kernel(32, 256, 128, b_trans=True, bias=True, name="k_fc1"), {"A": "inp", "B": "w1", "bias": "b1", "C": "h1"})
    act = ir.rename_buffers(ir.elementwise_kernel(32 * 256, {"h1": "f32"}, [("a", "multiply", ["h1", 0.7071067811865476]), ("b", "erf", ["a"]), ("c", "add", ["b", 1.0]),
                                                                            ("d", "multiply", ["h1", 0.5]), ("e", "multiply", ["d", "c"])], name="k_gelu"), {"out": "h2"})
    fc2 = ir.rename_buffers(ir.matmul_f32_kernel(32, 64, 256, b_trans=True, bias=True, name="k_fc2"), {"A": "h2", "B": "w2", "bias": "b2", "C": "y"})
    kernels = [
        (fc1, [_arg("inp", "f32", (32, 128), seed=0), _arg("w1", "f32", (256, 128), data=w1.tolist()), _arg("b1", "f32", (256,), data=b1.tolist()),
               _arg("h1", "f32", (32, 256), output=True)]),
        (act, [_arg("h1", "f32", (32 * 256,), intermediate=True), _arg("h2", "f32", (32 * 256,), output=True)]),
        (fc2, [_arg("h2", "f32", (32, 256), intermediate=True), _arg("w2", "f32", (64, 256), data=w2.tolist()), _arg("b2", "f32", (64,), data=b2.tolist()),
               _arg("y", "f32", (32, 64), output=True)]),
    ]
    t = lambda a: torch.from_numpy(a).double()
    h1 = t(x) @ t(w1).T + t(b1)
    y = torch.nn.functional.gelu(h1) @ t(w2).T + t(b2)
    return _write_problem(folder, kernels, {"h1": h1.numpy(), "y": y.numpy()}, MM)


def _swiglu(folder):
    import torch
    x, g = _seeded(0, (64, 256)), _seeded(1, (256,))
    w1, w3, w2 = _seeded(2, (256, 512)), _seeded(3, (256, 512)), _seeded(4, (512, 256))
    norm = ir.rename_buffers(ir.rowwise_kernel("rms_norm", 64, 256, eps=1e-6, name="k_norm"), {"X": "inp", "W": "g", "Y": "h"})
    up1 = ir.rename_buffers(ir.matmul_f32_kernel(64, 512, 256, name="k_up1"), {"A": "h", "B": "w1", "C": "u1"})
    up3 = ir.rename_buffers(ir.matmul_f32_kernel(64, 512, 256, name="k_up3"), {"A": "h", "B": "w3", "C": "u3"})
    gate = ir.rename_buffers(ir.elementwise_kernel(64 * 512, {"u1": "f32", "u3": "f32"}, [("a", "multiply", ["u1", 0.0625]), ("s", "sigmoid", ["a"]), ("t", "multiply", ["a", "s"]),
                                                                                        ("b", "multiply", ["u3", 0.0625]), ("c", "multiply", ["t", "b"])], name="k_gate"), {"out": "act"})
    down = ir.rename_buffers(ir.matmul_f32_kernel(64, 256, 512, name="k_down"), {"A": "act", "B": "w2", "C": "d"})
    resid = ir.rename_buffers(ir.elementwise_kernel(64 * 256, {"inp": "f32", "d": "f32"}, [("a", "multiply", ["d", 0.04419417]), ("b", "add", ["inp", "a"])], name="k_resid"),
                              {"out": "y"})
    kernels = [
        (norm, [_arg("inp", "f32", (64, 256), seed=0), _arg("g", "f32", (256,), seed=1), _arg("h", "f32", (64, 256), output=True)]),
        (up1, [_arg("h", "f32", (64, 256), intermediate=True), _arg("w1", "f32", (256, 512), seed=2), _arg("u1", "f32", (64, 512), output=True)]),
        (up3, [_arg("h", "f32", (64, 256), intermediate=True), _arg("w3", "f32", (256, 512), seed=3), _arg("u3", "f32", (64, 512), output=True)]),
        (gate, [_arg("u1", "f32", (64 * 512,), intermediate=True), _arg("u3", "f32", (64 * 512,), intermediate=True), _arg("act", "f32", (64 * 512,), output=True)]),
        (down, [_arg("act", "f32", (64, 512), intermediate=True), _arg("w2", "f32", (512, 256), seed=4), _arg("d", "f32", (64, 256), output=True)]),
        (resid, [_arg("inp", "f32", (64 * 256,), seed=0), _arg("d", "f32", (64 * 256,), intermediate=True), _arg("y", "f32", (64 * 256,), output=True)]),
    ]
    t = lambda a: torch.from_numpy(a).double()
    xd = t(x)
    h = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-6) * t(g)
    a = torch.nn.functional.silu((h @ t(w1)) * 0.0625) * ((h @ t(w3)) * 0.0625)
    y = xd + (a @ t(w2)) * 0.04419417
    return _write_problem(folder, kernels, {"h": h.numpy(), "y": y.numpy()}, MM)


def _soft_xent(folder):
    import torch
    x, p = _seeded(0, (32, 100)), _seeded(1, (32, 100))
    ls = ir.rename_buffers(ir.rowwise_kernel("log_softmax", 32, 100, name="k_logsm"), {"X": "logits", "Y": "ls"})
    sm = ir.rename_buffers(ir.rowwise_kernel("softmax", 32, 100, name="k_sm"), {"X": "target", "Y": "sm"})
    mul = ir.rename_buffers(ir.elementwise_kernel(3200, {"ls": "f32", "sm": "f32"}, [("a", "multiply", ["ls", "sm"])], name="k_mul"), {"out": "prod"})
    rows = ir.rename_buffers(ir.rowwise_kernel("sum", 32, 100, name="k_rows"), {"X": "prod", "Y": "per_row"})
    mean = ir.rename_buffers(ir.rowwise_kernel("mean", 1, 32, name="k_mean"), {"X": "per_row", "Y": "avg"})
    neg = ir.rename_buffers(ir.elementwise_kernel(1, {"avg": "f32"}, [("a", "negative", ["avg"])], name="k_neg"), {"out": "loss"})
    kernels = [
        (ls, [_arg("logits", "f32", (32, 100), seed=0), _arg("ls", "f32", (32, 100), output=True)]),
        (sm, [_arg("target", "f32", (32, 100), seed=1), _arg("sm", "f32", (32, 100), output=True)]),
        (mul, [_arg("ls", "f32", (3200,), intermediate=True), _arg("sm", "f32", (3200,), intermediate=True), _arg("prod", "f32", (3200,), output=True)]),
        (rows, [_arg("prod", "f32", (32, 100), intermediate=True), _arg("per_row", "f32", (32,), output=True)]),
        (mean, [_arg("per_row", "f32", (1, 32), intermediate=True), _arg("avg", "f32", (1,), output=True)]),
        (neg, [_arg("avg", "f32", (1,), intermediate=True), _arg("loss", "f32", (1,), output=True)]),
    ]
    t = lambda a: torch.from_numpy(a).double()
    loss = -(torch.log_softmax(t(x), -1) * torch.softmax(t(p), -1)).sum(-1).mean()
    return _write_problem(folder, kernels, {"loss": loss.reshape(1).numpy()}, dict(rtol=1e-3, atol=1e-4))     # fused.py:20


def _addmm(folder):
    """m_addmm (tools/torch_cases/matmul.py:16-17): c + a @ b as a product kernel and an elementwise add."""
    import torch
    c, a, b = _seeded(0, (64, 48)), _seeded(1, (64, 32)), _seeded(2, (32, 48))
    mm = ir.rename_buffers(ir.matmul_f32_kernel(64, 48, 32, name="k_mm"), {"A": "lhs", "B": "rhs", "C": "prod"})
    add = ir.rename_buffers(ir.elementwise_kernel(64 * 48, {"base": "f32", "prod": "f32"}, [("s", "add", ["base", "prod"])], name="k_add"), {"out": "y"})
    kernels = [
        (mm, [_arg("lhs", "f32", (64, 32), seed=1), _arg("rhs", "f32", (32, 48), seed=2), _arg("prod", "f32", (64, 48), output=True)]),
        (add, [_arg("base", "f32", (64 * 48,), seed=0), _arg("prod", "f32", (64 * 48,), intermediate=True), _arg("y", "f32", (64 * 48,), output=True)]),
    ]
    t = lambda v: torch.from_numpy(v).double()
    return _write_problem(folder, kernels, {"y": torch.addmm(t(c), t(a), t(b)).reshape(-1).numpy()}, MM)


PROBLEMS = {"m_addmm": _addmm, "t_module_mlp": _mlp, "t_swiglu_ffn": _swiglu, "f_soft_xent": _soft_xent}


@pytest.mark.parametrize("name", sorted(PROBLEMS))
def test_problem_of_several_kernels(name, tmp_path, cuda):
    folder = PROBLEMS[name](tmp_path / name)
    target = run_local.init()
    ok, detail = run_local.run_problem(folder, target)
    assert ok, detail
    assert "max abs err" in detail


def test_runner_command_line(tmp_path, cuda, capsys):
    """The runner's own command line over a folder of problems: one PASS / FAIL line each, the count, the exit status
    (tools/run_local.py:144-160). A problem whose expected values are wrong fails with the buffer's name and error."""
    _soft_xent(tmp_path / "a_xent")
    bad = _soft_xent(tmp_path / "b_wrong")
    np.savez(bad / "expected.npz", loss=np.array([123.0]))
    assert run_local.main([str(tmp_path), "--only", "a_"]) == 0
    out = capsys.readouterr().out
    assert "PASS  a_xent" in out and "1/1 passed" in out
    assert run_local.main([str(tmp_path)]) == 1
    out = capsys.readouterr().out
    assert "FAIL  b_wrong" in out and "loss: max abs err" in out and "1/2 passed" in out
    # a kernel the facade cannot serve is a failed problem, not a crash
    broken = _soft_xent(tmp_path / "c_broken")
    text = json.loads((broken / "k_neg.ir.json").read_text())
    (broken / "k_neg.ir.json").write_text(json.dumps(text).replace('"negative"', '"no_such_op"'))
    ok, detail = run_local.run_problem(broken, run_local.init())
    assert not ok and detail.startswith("compile.py failed")
