"""Loading and launching PTX text through the CUDA driver API, the way the reference's runner does
(tools/run_local.py:22 opens libcuda, :64-72 `cuModuleLoadDataEx` + `cuModuleGetFunction`, :100-102
`cuLaunchKernel` on the NULL stream with one 64-bit pointer per buffer).

The sm_100a kernels never go through here. It exists so that the reference's *own* compiler output (kept as text
fixtures) can run on the same device next to them: kernel-against-kernel parity tests, and the "reference kernel on
this GPU" timings of the benchmark. The text targets sm_89; the driver JITs it forward.
"""
from __future__ import annotations

import ctypes


class PtxModule:
    """One loaded PTX module; unload with close() or use as a context manager."""

    def __init__(self, ptx: str) -> None:
        self.cu = ctypes.CDLL("libcuda.so.1")
        self.module = ctypes.c_void_p()
        self._check(self.cu.cuModuleLoadData(ctypes.byref(self.module), ptx.encode() + b"\0"), "cuModuleLoadData")

    def _check(self, err: int, what: str) -> None:
        if err:
            msg = ctypes.c_char_p()
            self.cu.cuGetErrorString(err, ctypes.byref(msg))
            raise RuntimeError(f"{what}: {msg.value.decode() if msg.value else err}")

    def function(self, entry: str) -> ctypes.c_void_p:
        fn = ctypes.c_void_p()
        self._check(self.cu.cuModuleGetFunction(ctypes.byref(fn), self.module, entry.encode()), "cuModuleGetFunction")
        return fn

    def launch(self, fn, pointers: list[int], grid: int, block: int, smem_bytes: int = 0, stream: int = 0) -> None:
        """Enqueue on `stream` (a CUstream handle; 0 = the NULL stream, which is what the reference's runner uses
        and what torch calls its default stream); does not synchronise."""
        # device pointers as integers; by-value scalar parameters as ctypes values (c_float, c_int32: emmyptx/kernel.py:171-178)
        holders = [p if isinstance(p, ctypes._SimpleCData) else ctypes.c_uint64(p) for p in pointers]
        params = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.byref(h), ctypes.c_void_p) for h in holders])
        self._check(self.cu.cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, smem_bytes, ctypes.c_void_p(stream or None), params, None), "cuLaunchKernel")

    def synchronize(self) -> None:
        self._check(self.cu.cuCtxSynchronize(), "cuCtxSynchronize")

    def close(self) -> None:
        if self.module:
            self.cu.cuModuleUnload(self.module)
            self.module = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()
