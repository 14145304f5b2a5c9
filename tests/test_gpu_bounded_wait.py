"""The give-up path of the device-side waits, made to happen without a fault (the reference's only device-side error
path is a `trap`, emmyptx/kernel.py:685-691, which kills the context; here a wait that runs out returns a status).

`emmyb200_selftest_wait_expiry` launches one CTA whose first thread waits -- through the same `bounded_wait` that every
TMA / MMA / epilogue / softmax role of the tensor-core kernels uses -- on a barrier nothing arrives on, with a limit
of a few milliseconds. The kernel must return by itself, the status word must name the wait, the host calls must map
it to EMMYB200_ERR_TIMEOUT, and the device must go on working: the next GEMM and attention launches are checked
against the oracle."""
import ctypes

import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu
ERR_TIMEOUT = -6


def test_expired_wait_is_reported_and_the_device_stays_usable(cuda, lib):
    import torch
    from emmyptx import runtime
    torch.cuda.synchronize()
    assert runtime.device_status() == 0
    assert lib.emmyb200_selftest_wait_expiry(5_000_000, None) == ERR_TIMEOUT           # 5 ms
    assert b"expired" in lib.emmyb200_last_error()
    word = ctypes.c_uint32(0)
    assert lib.emmyb200_device_status(ctypes.byref(word)) == ERR_TIMEOUT
    assert word.value == 0x7E570001
    assert b"0x7e570001" in lib.emmyb200_last_error()
    assert lib.emmyb200_device_status(ctypes.byref(word)) == 0 and word.value == 0      # read clears
    with pytest.raises(runtime.KernelError) as e:
        lib.emmyb200_selftest_wait_expiry(2_000_000, None)
        runtime.check_device()
    assert e.value.status == ERR_TIMEOUT
    # the context is intact: normal launches on the same device pass
    a, b = inputs.gemm_inputs(256, 512, 512, "bf16")
    c = runtime.gemm(a.to(cuda), b.to(cuda), epilogue="gelu_tanh").cpu()
    ok, ratio = reference.gemm_tolerance_ok(c, reference.gemm_reference(a, b, "gelu_tanh"))
    assert ok, ratio
    q, k, v = inputs.attention_inputs(2, 256, 256, 128, "bf16")
    o = runtime.attention(q.to(cuda), k.to(cuda), v.to(cuda)).cpu()
    ok, ratio = reference.gemm_tolerance_ok(o, reference.attention_reference(q, k, v))
    assert ok, ratio
    assert runtime.device_status() == 0


def test_wait_limit_is_a_launch_parameter(cuda, lib):
    """A shorter watchdog does not disturb a healthy launch (no wait comes near it); out-of-range values are refused."""
    import torch
    from emmyptx import runtime
    assert lib.emmyb200_set_wait_limit_ns(1) == -1
    assert lib.emmyb200_set_wait_limit_ns(50_000_000) == 0                               # 50 ms
    try:
        a, b = inputs.gemm_inputs(1024, 1024, 1024, "f16")
        c = runtime.gemm(a.to(cuda), b.to(cuda)).cpu()
        ok, ratio = reference.gemm_tolerance_ok(c, reference.gemm_reference(a, b))
        assert ok, ratio
        assert runtime.device_status() == 0
    finally:
        assert lib.emmyb200_set_wait_limit_ns(0) == 0                                    # back to the default
    assert lib.emmyb200_selftest_wait_expiry(10, None) == -1                             # below the accepted range
