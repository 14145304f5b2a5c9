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
or come from a problem set that is not in its tree). The pins are (a) `tests/golden/`: outputs of
the reference's own compiler -- its PTX for the two streaming configurations, executed by
`oracle/ptx_interp.py` -- and (b) `oracle/emmy_lowering.py`, a numpy restatement of the reference's
instruction sequences for exp / tanh / sin, both checked against this oracle within the
reference's own tolerance classes.
"""
