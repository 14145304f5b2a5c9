"""The C-ABI library: loads without a GPU, exports every symbol include/emmyb200.h declares, and rejects
bad arguments before touching the device (CPU only; no compute calls)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions() -> list[str]:
    text = (ROOT / "include" / "emmyb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(emmyb200_\w+)\s*\(", text)


def test_header_declares_the_documented_entry_points():
    names = declared_functions()
    for n in ("emmyb200_pointwise_f32", "emmyb200_index_gather_i32", "emmyb200_gemm", "emmyb200_attention_fwd",
              "emmyb200_last_error", "emmyb200_device_status", "emmyb200_version"):
        assert n in names


def test_library_exports_every_declared_symbol(lib):
    from emmyptx import runtime
    raw = ctypes.CDLL(str(runtime.LIB_PATH))
    for name in declared_functions():
        assert hasattr(raw, name), name
    assert set(declared_functions()) == set(runtime.EXPORTS)
    assert lib.emmyb200_version() >= 100


def test_argument_checks_need_no_device(lib):
    assert lib.emmyb200_pointwise_f32(0, None, None, -1, None) == -2
    assert b"negative" in lib.emmyb200_last_error()
    assert lib.emmyb200_pointwise_f32(0, None, None, 0, None) == 0            # empty: nothing to do
    assert lib.emmyb200_pointwise_f32(0, None, None, 16, None) == -1          # null buffers
    assert lib.emmyb200_index_gather_i32(None, None, 0, 1, 0, 3, 2, 0, None) == 0
    assert lib.emmyb200_index_gather_i32(None, None, 16, 1, 0, 3, 2, 0, None) == -1
    assert lib.emmyb200_gemm(0, 0, 0, None, None, None, 8, 8, 8, 8, 8, 8, None) == -4
    assert lib.emmyb200_gemm(1, 0, 0, None, None, None, 8, 8, 8, 8, 8, 8, None) == -1
    assert lib.emmyb200_attention_fwd(2, 0, None, None, None, None, 1, 8, 8, 80, 1.0, None) == -4
    assert lib.emmyb200_attention_fwd(2, 0, None, None, None, None, 1, 8, 8, 128, 1.0, None) == -1


def test_newer_entry_points_check_their_arguments_without_a_device(lib):
    """Row / column reductions, cumsum, the float32 product and the multicast flag: all rejected (or accepted as empty)
    before any CUDA call."""
    p = ctypes.c_void_p(4096)                                                  # never dereferenced
    assert lib.emmyb200_rowwise_f32(0, None, None, None, None, 0, 8, 0.0, None, 0, None) == 0
    assert lib.emmyb200_rowwise_f32(0, None, None, None, None, 4, 8, 0.0, None, 0, None) == -1
    assert lib.emmyb200_rowwise_f32(12, p, None, None, p, 4, 8, 0.0, None, 0, None) == -1
    assert lib.emmyb200_rowwise_workspace_bytes(16, 4, 1 << 20) > 0 and lib.emmyb200_rowwise_workspace_bytes(16, 4, 4096) == 0
    assert lib.emmyb200_colwise_f32(19, p, p, 1, 4, 8, 0.0, None, 0, None) == -1  # rms_norm is a row op only
    assert lib.emmyb200_colwise_f32(0, None, None, 0, 4, 8, 0.0, None, 0, None) == 0
    assert lib.emmyb200_cumsum_f32(None, None, 4, 0, None) == 0
    assert lib.emmyb200_cumsum_f32(None, None, 4, 8, None) == -1
    assert lib.emmyb200_gemm_f32_workspace_bytes(0, 1, 128, 128, 128, 1) == 2 * 3 * 128 * 128 * 2
    assert lib.emmyb200_gemm_f32(0, 0, p, p, None, p, 1, 8, 8, 8, 8, 8, 8, 0, 0, 0, None, 0, None) == -1 and b"workspace" in lib.emmyb200_last_error()
    assert lib.emmyb200_gemm(2, 0, 2, p, p, p, 8, 8, 8, 8, 8, 8, None) == -1     # the multicast flag is for the allgather entry
    dst = (ctypes.c_void_p * 2)(4096, 8192)
    assert lib.emmyb200_gemm_allgather(2, 0, 2, p, p, dst, 2, 8, 8, 8, 8, 8, 8, None) == -1      # one multicast address, not two
    assert lib.emmyb200_gemm_allgather(2, 0, 2, p, p, dst, 1, 8, 12, 8, 8, 16, 16, None) == -2    # N must be a multiple of 8
    assert lib.emmyb200_attention_fwd(2, 2, p, p, p, p, 1, 8, 8, 128, 1.0, None) == -1
    assert lib.emmyb200_attention_fwd_allgather(2, 2, p, p, p, dst, 2, 1, 8, 8, 128, 1.0, None) == -1
    assert lib.emmyb200_rowwise_static_capacity() == 1 << 20
    assert lib.emmyb200_launch(b"{}", None, 0, None, 0, None) == -1 and b"handle" in lib.emmyb200_last_error()
    assert lib.emmyb200_launch_workspace_bytes(b"[1, 2") == -1
    handle = b'{"variant": "pointwise_f32", "params": {"op": "exp", "n": 8}, "arg_order": ["x", "y"], "inputs": ["x"], "outputs": ["y"]}'
    assert lib.emmyb200_launch_workspace_bytes(handle) == 0
    assert lib.emmyb200_launch(handle, None, 2, None, 0, None) == -1                  # no parameter array
    null = ctypes.c_void_p(0)
    params = (ctypes.c_void_p * 2)(ctypes.cast(ctypes.byref(null), ctypes.c_void_p), ctypes.cast(ctypes.byref(null), ctypes.c_void_p))
    assert lib.emmyb200_launch(handle, params, 2, None, 0, None) == -1 and b"null" in lib.emmyb200_last_error()
    assert lib.emmyb200_set_wait_limit_ns(1) == -1 and lib.emmyb200_set_wait_limit_ns(0) == 0
    assert lib.emmyb200_selftest_wait_expiry(10, None) == -1 and lib.emmyb200_selftest_wait_expiry(2 * 10**9, None) == -1


def test_python_binding_refuses_cpu_tensors():
    import torch
    from emmyptx import runtime
    with pytest.raises(RuntimeError, match="no CPU path"):
        runtime.pointwise("exp", torch.zeros(4))
    with pytest.raises(RuntimeError, match="no CPU path"):
        runtime.gemm(torch.zeros(8, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))
