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
    assert lib.emmyb200_attention_fwd(2, 0, None, None, None, None, 1, 8, 8, 96, 1.0, None) == -4
    assert lib.emmyb200_attention_fwd(2, 0, None, None, None, None, 1, 8, 8, 128, 1.0, None) == -1


def test_python_binding_refuses_cpu_tensors():
    import torch
    from emmyptx import runtime
    with pytest.raises(RuntimeError, match="no CPU path"):
        runtime.pointwise("exp", torch.zeros(4))
    with pytest.raises(RuntimeError, match="no CPU path"):
        runtime.gemm(torch.zeros(8, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))
