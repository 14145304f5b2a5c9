"""emmyptx for B200: the reference's kernel-builder API over a library of hand-written sm_100a kernels.

    from emmyptx.kernel import KernelCompiler, compile_kernel, CompileError     # as in the reference
    from emmyptx import runtime                                                  # ctypes binding of the C ABI
"""
