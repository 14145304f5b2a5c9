"""emmyb200_rowwise_f32_static: the row kernels with the library's own fixed scratch array instead of a caller
workspace. Called through the C ABI, twice in a row on rows long enough to take the split (multi-block) path; the
results must equal the workspace version bit for bit, agree with the float64 oracle, and the device's free memory
must not move across the calls. Collected last on purpose: it runs after every other kernel has been loaded."""
import numpy as np
import pytest

from oracle import reference

pytestmark = pytest.mark.gpu


def _call(lib, op, x, y, stream=None):
    rows, cols = x.shape
    return lib.emmyb200_rowwise_f32_static(op, x.data_ptr(), None, None, y.data_ptr(), rows, cols, 0.0, stream)


@pytest.mark.parametrize("name", ["sum", "var", "logsumexp", "softmax"])
def test_two_calls_in_a_row_match_the_workspace_version(name, cuda, lib):
    import torch
    from emmyptx import runtime
    op = runtime.ROW_OPS[name]
    x1 = torch.randn(5, 200_000, generator=torch.Generator().manual_seed(1)).to(cuda)
    x2 = torch.randn(3, 1 << 20, generator=torch.Generator().manual_seed(2)).to(cuda)
    assert lib.emmyb200_rowwise_workspace_bytes(op, *x1.shape) > 0          # both shapes need scratch memory
    assert lib.emmyb200_rowwise_workspace_bytes(op, *x2.shape) > 0
    outs = [torch.empty(x.shape if op >= runtime.ROW_MAP_FIRST else x.shape[:1], device=cuda) for x in (x1, x2)]
    for x, y in ((x1, outs[0]), (x2, outs[1])):                             # warm: kernels loaded, scratch address looked up
        assert _call(lib, op, x, y) == 0
    torch.cuda.synchronize()
    for y in outs:
        y.zero_()
    free_before = torch.cuda.mem_get_info()[0]
    assert _call(lib, op, x1, outs[0]) == 0                                   # two calls back to back, no sync between
    assert _call(lib, op, x2, outs[1]) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    for x, y in ((x1, outs[0]), (x2, outs[1])):
        assert torch.equal(y, runtime.rowwise(name, x))
        ref = reference.rowwise_reference(name, x.cpu()).numpy()
        assert reference.compare(y.cpu().numpy(), ref, 1e-4, 1e-4 + 1e-6 * x.shape[1] ** 0.5)["ok"]


def test_short_rows_need_no_scratch(cuda, lib):
    import torch
    from emmyptx import runtime
    x = torch.randn(300, 1000, device=cuda)
    y = torch.empty_like(x)
    assert _call(lib, runtime.ROW_OPS["softmax"], x, y) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, runtime.rowwise("softmax", x))


def test_shapes_beyond_the_capacity_are_rejected(cuda, lib):
    import torch
    from emmyptx import runtime
    cap = lib.emmyb200_rowwise_static_capacity()
    assert cap == 1 << 20
    rows, cols = 60_000, 70_000                                             # would need > 1 MiB of piece states
    assert lib.emmyb200_rowwise_workspace_bytes(0, rows, cols) > cap
    x = torch.zeros(8, device=cuda)                                         # never touched: the call is refused first
    assert lib.emmyb200_rowwise_f32_static(0, x.data_ptr(), None, None, x.data_ptr(), rows, cols, 0.0, None) == -2
    assert b"scratch" in lib.emmyb200_last_error()
    assert lib.emmyb200_rowwise_f32_static(99, x.data_ptr(), None, None, x.data_ptr(), 2, 4, 0.0, None) == -1
