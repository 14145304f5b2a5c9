"""The library's fp32 transcendentals, built for the host (CPU only).

emmy_math.cuh uses IEEE operations only, so the host build (oracle/Makefile) is bit-identical to the device
build; here it is checked against float64 on dense samples of every binade. The exhaustive run over all 2^32
inputs is oracle/ulp_exhaustive.cpp (worst case 1.55 ulp).
"""
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import inputs, reference

ROOT = Path(__file__).resolve().parent.parent
OPS = {"exp_sin_tanh": 0, "exp": 1, "sin": 2, "cos": 3, "tanh": 4, "gelu_tanh": 5}


@pytest.fixture(scope="module")
def host():
    subprocess.run(["make", "-s", "-C", str(ROOT / "oracle")], check=True)
    lib = ctypes.CDLL(str(ROOT / "oracle" / "_build" / "libemmymath_host.so"))
    lib.emmy_host_apply.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long]

    def apply(op, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        lib.emmy_host_apply(OPS[op], x.ctypes.data, y.ctypes.data, x.size)
        return y
    return apply


@pytest.mark.parametrize("op", ["exp", "sin", "cos", "tanh"])
def test_two_ulp_over_all_binades(host, op):
    rng = np.random.default_rng(11)
    x = rng.integers(0, 2**32, 2**22, dtype=np.uint64).astype(np.uint32).view(np.float32)
    x = np.concatenate([x, inputs.c1_input(2**20)])
    got = host(op, x)
    with np.errstate(all="ignore"):
        ref = reference.UNARY_F64[op](x.astype(np.float64))
        nan = np.isnan(ref)
        assert np.array_equal(np.isnan(got), nan)
        ref32 = ref.astype(np.float32)
    inf = np.isinf(ref32) & ~nan
    assert np.array_equal(got[inf], ref32[inf])
    fin = ~nan & ~inf
    assert reference.ulp_error(got[fin], ref[fin]).max() <= 2.0


def test_special_values(host):
    x = np.array([0.0, -0.0, np.inf, -np.inf], np.float32)
    assert np.array_equal(host("exp", x), np.array([1, 1, np.inf, 0], np.float32))
    s = host("sin", x)
    assert s[0] == 0 and not np.signbit(s[0]) and s[1] == 0 and np.signbit(s[1]) and np.isnan(s[2:]).all()
    assert np.array_equal(host("tanh", x), np.array([0, -0.0, 1, -1], np.float32))
    assert np.signbit(host("tanh", x)[1])
    assert np.array_equal(host("cos", x[:2]), np.ones(2, np.float32))


def test_composite_and_gelu_within_reference_class(host):
    x = inputs.c1_input(2**18)
    assert reference.compare(host("exp_sin_tanh", x), reference.c1_f64(x), 1e-5, 1e-5)["ok"]
    assert reference.c1_condition_ulp(host("exp_sin_tanh", x), x).max() <= 5.0
    g = (np.random.default_rng(0).standard_normal(2**18) * 3).astype(np.float32)
    assert reference.compare(host("gelu_tanh", g), reference.UNARY_F64["gelu_tanh"](g.astype(np.float64)), 1e-5, 1e-5)["ok"]
