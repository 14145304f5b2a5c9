"""int32 index-math gather (C2) against the exact-arithmetic oracle: bit-exact."""
import numpy as np
import pytest

from oracle import inputs, reference

pytestmark = pytest.mark.gpu


def _run(x_np, cuda, **kw):
    import torch
    from emmyptx import runtime
    y = runtime.index_gather(torch.from_numpy(x_np).to(cuda), **kw)
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("log_n", [10, 16, 20, 24])
@pytest.mark.parametrize("trunc", [False, True])
def test_c2_expression_power_of_two(log_n, trunc, cuda):
    x = inputs.c2_input(2**log_n)
    got = _run(x, cuda, mul=7919, add=13, div=3, shift=2, trunc=trunc)
    assert np.array_equal(got, reference.c2_reference(x, trunc=trunc))


def test_c2_full_size_bit_exact(cuda):
    """N = 2^26, the benchmark size: the tiled kernel over every cell."""
    x = inputs.c2_input(2**26)
    got = _run(x, cuda, mul=7919, add=13, div=3, shift=2)
    assert np.array_equal(got, reference.c2_reference(x))


@pytest.mark.parametrize("n,mul,add,div,shift", [
    (1, 7919, 13, 3, 2), (2, 1, 0, 1, 0), (7, 3, 1, 2, 1), (1000, 7919, 13, 3, 2),     # direct kernel: tiny n
    (2**20, 6, 5, 3, 2),                                                           # gcd(mul, n) != 1
    (2**20, 1, 0, 7, 3), (2**20, 0, 9, 3, 2),                                      # identity, broadcast
    (10**6 + 3, 7919, 13, 3, 2), (999_983, 65_537, 12_345, 5, 4),                  # tiled, n not a power of two
    (2**22, 2**22 + 7919, 2**22 + 13, 3, 2),                                       # mul, add >= n
    (2**20, 12_345_677, 99, 1_000_003, 31), (2**18, 8191, 1, 2**31 - 1, 0),        # large divisor / shift
])
def test_parameter_edges(n, mul, add, div, shift, cuda):
    x = inputs.c2_input(n, seed=3)
    x[: min(n, 4)] = np.array([-2**31, 2**31 - 1, -1, 0], np.int32)[: min(n, 4)]
    for trunc in (False, True):
        got = _run(x, cuda, mul=mul, add=add, div=div, shift=shift, trunc=trunc)
        assert np.array_equal(got, reference.c2_reference(x, mul, add, div, shift, trunc=trunc)), (n, mul, trunc)


def test_floor_and_trunc_differ_as_documented(cuda):
    """torch floors, the reference's div.s32 truncates (tools/torch_cases/dtypes.py:17-19): on
    C2's inputs the two differ on about a third of the cells."""
    x = inputs.c2_input(2**20)
    a = _run(x, cuda, mul=7919, add=13, div=3, shift=2, trunc=False)
    b = _run(x, cuda, mul=7919, add=13, div=3, shift=2, trunc=True)
    frac = np.mean(a != b)
    assert 0.30 < frac < 0.37


def test_is_a_permutation_checksum(cuda):
    """Size-independent property: with d = 1 and shift = 31 the kernel is a pure permutation of x."""
    x = inputs.c2_input(2**24)
    got = _run(x, cuda, mul=7919, add=13, div=1, shift=31)
    assert int(got.astype(np.int64).sum()) == int(x.astype(np.int64).sum())
    assert np.array_equal(np.sort(got), np.sort(x))


def test_rejects_bad_arguments(cuda, lib):
    import torch
    x = torch.zeros(64, dtype=torch.int32, device=cuda)
    y = torch.zeros(64, dtype=torch.int32, device=cuda)
    f = lib.emmyb200_index_gather_i32
    assert f(x.data_ptr(), y.data_ptr(), 64, 3, 1, 0, 2, 0, None) == -1      # divisor 0
    assert f(x.data_ptr(), y.data_ptr(), 64, 3, 1, 3, 32, 0, None) == -1     # shift
    assert f(x.data_ptr(), x.data_ptr(), 64, 3, 1, 3, 2, 0, None) == -1      # overlap
    assert f(x.data_ptr(), y.data_ptr(), 2**31, 3, 1, 3, 2, 0, None) == -2   # n too large
    assert f(x.data_ptr(), y.data_ptr(), 0, 3, 1, 3, 2, 0, None) == 0        # empty
