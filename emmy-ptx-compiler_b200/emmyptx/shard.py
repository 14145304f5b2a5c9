"""Splitting the shardable configurations over the GPUs of one box, one process per GPU.

The reference is single-GPU (device 0, one context: tools/run_local.py:51-57), so nothing here replaces
reference code. Large GEMMs split by rows of A and C (B is replicated), attention by its independent
(batch, head) units, streaming arrays by contiguous chunks; every split is a contiguous range, so a rank's
output shard is a contiguous slice of the full output and one `all_gather_into_tensor` assembles it.
The only collective is that all-gather (NCCL over NVLink on GPUs; any backend for the host-side tests).
"""
from __future__ import annotations


def split_range(total: int, world: int, rank: int, align: int = 1) -> tuple[int, int]:
    """[begin, end) of rank's contiguous share of `total` items. Shares are equal multiples of `align` when
    `total` divides evenly (what `all_gather_into_tensor` needs); otherwise the first ranks get one more
    `align`-block and the caller gathers with `all_gather_ragged`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    blocks = -(-total // align)
    base, extra = divmod(blocks, world)
    begin = (rank * base + min(rank, extra)) * align
    end = begin + (base + (1 if rank < extra else 0)) * align
    return min(begin, total), min(end, total)


def even(total: int, world: int, align: int = 1) -> bool:
    return total % (world * align) == 0


def all_gather_rows(full, local, group=None):
    """Assemble equal contiguous shards along dim 0: `full[rank*rows:(rank+1)*rows] = local` on every rank."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if full.shape[0] != local.shape[0] * world:
        raise ValueError(f"{tuple(full.shape)} is not {world} shards of {tuple(local.shape)}")
    dist.all_gather_into_tensor(full, local.contiguous(), group=group)
    return full


def all_gather_ragged(full, local, total: int, align: int = 1, group=None):
    """Same for shares made by `split_range` when they are not all equal: every rank pads its shard to the
    largest share, one all-gather moves the padded shards, and the valid rows are copied into place."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    spans = [split_range(total, world, r, align) for r in range(world)]
    rows = max(e - b for b, e in spans)
    padded = torch.zeros((rows, *local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    staged = torch.empty((world * rows, *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(staged, padded, group=group)
    for r, (b, e) in enumerate(spans):
        full[b:e] = staged[r * rows: r * rows + (e - b)]
    return full


def peer_mapped_empty(shape, dtype, device, group=None, multicast: bool = False):
    """A tensor of the same shape on every rank of the group, each mapped into every other rank's address
    space (torch symmetric memory over NVLink). Returns (local tensor, handle); `handle.buffer_ptrs[r]` is rank
    r's copy as an address valid on this GPU and `handle.barrier()` is a device-side barrier of the group.
    With `multicast`, the copies are also bound to one NVSwitch multicast object where the fabric supports it:
    `multicast_address(handle)` is then the address through which one `multimem.st` reaches every copy (0 if not).
    The choice is made by the first call in a process (torch reads the switch once)."""
    import os
    if not multicast:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(*shape, dtype=dtype, device=device)
    handle = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
    return t, handle


def multicast_address(handle) -> int:
    """The multicast address of a `peer_mapped_empty(..., multicast=True)` buffer, or 0 when the group has none."""
    try:
        return int(getattr(handle, "multicast_ptr", 0) or 0)
    except Exception:  # noqa: BLE001 - an unsupported fabric is not an error here
        return 0
