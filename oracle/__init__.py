"""CPU oracle for the five kernel configurations. TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only `tests/`, `__graft_entry__.smoke()` and
the CPU-baseline legs of `bench.py` may import it, and only as the checker or the timed CPU
reference. The kernels in `emmy-ptx-compiler_b200/` never call into it.

Truth is defined the way the reference's harness defines it (`tools/check_torch.py:194-237`): the
case's torch expression evaluated on CPU in float64 on the same seeded inputs, compared with
`np.isclose` (`tools/check_torch.py:260-278`). Inputs are seeded per argument index with
`np.random.default_rng(seed)` (`tools/run_local.py:86-87`); bf16 is round-to-nearest-even of the
fp32 bits (`tools/run_local.py:31-37`).

Pinning: the reference ships no golden vectors (its `expected.npz` files are generated on the fly
or come from a problem set that is not in its tree). The pins are the outputs of the reference's own
compiler under `tests/golden/`: its PTX for the two streaming configurations, for the single
transcendental ops and for its tensor-core matmul cases (`mma.sync` kernels), executed on the CPU by
`oracle/ptx_interp.py` into `golden.npz` and JIT-loaded next to the sm_100a kernels in the GPU tests.
This oracle is checked against those vectors within the reference's own tolerance classes
(`tests/test_oracle_golden.py`). Attention has no reference-emitted kernel (the reference has no
statement that carries scores from one MMA group into the next): that path is checked against this
oracle only.
"""
