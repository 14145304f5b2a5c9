"""Two-GPU path: the row-sharded GEMM and the unit-sharded attention whose kernels write every output piece to both
GPUs' copies of the result (TMA stores to peer-mapped memory), against the unsharded oracle. Skipped on a one-GPU box."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_multicast(rank: int, world: int, port: int):
    """The same two kernels storing through the NVSwitch multicast mapping (one multimem.st per 16 bytes reaches both
    copies). Where the fabric has no multicast the mapping's address is 0 and the case is skipped."""
    import torch
    import torch.distributed as dist
    from emmyptx import runtime, shard
    from oracle import inputs, reference
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        m, n, k = 1024, 768, 512
        a, b = inputs.gemm_inputs(m, n, k, "bf16")
        lo, hi = shard.split_range(m, world, rank, 128)
        c_full, peers = shard.peer_mapped_empty((m, n), torch.bfloat16, dev, multicast=True)
        mc = shard.multicast_address(peers)
        flag = torch.tensor([1 if mc else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() == 0:
            print("no multicast mapping on this fabric: skipped")
            return
        c_full.zero_()
        peers.barrier()
        runtime.gemm_allgather(a[lo:hi].to(dev).contiguous(), b.to(dev), [mc + lo * n * 2], n, epilogue="gelu_tanh", multicast=True)
        peers.barrier()
        torch.cuda.synchronize()
        assert runtime.device_status() == 0
        local = runtime.gemm(a[lo:hi].to(dev).contiguous(), b.to(dev), epilogue="gelu_tanh")
        gathered = shard.all_gather_rows(torch.empty(m, n, dtype=torch.bfloat16, device=dev), local)
        assert torch.equal(gathered, c_full), f"rank {rank}: multicast GEMM differs from the gathered shards"
        units, sq, sk, d = 4, 300, 260, 128
        q, k, v = inputs.attention_inputs(units, sq, sk, d, "bf16")
        ulo, uhi = shard.split_range(units, world, rank)
        o_full, opeers = shard.peer_mapped_empty((units, sq, d), torch.bfloat16, dev, multicast=True)
        omc = shard.multicast_address(opeers)
        assert omc != 0
        o_full.zero_()
        opeers.barrier()
        runtime.attention_allgather(q[ulo:uhi].to(dev).contiguous(), k[ulo:uhi].to(dev).contiguous(), v[ulo:uhi].to(dev).contiguous(),
                                    [omc + ulo * sq * d * 2], multicast=True)
        opeers.barrier()
        torch.cuda.synchronize()
        assert runtime.device_status() == 0
        ok, ratio = reference.gemm_tolerance_ok(o_full.cpu(), reference.attention_reference(q, k, v))
        assert ok, f"rank {rank}: multicast attention worst error {ratio:.2f}x the bound"
        plain = runtime.attention(q.to(dev), k.to(dev), v.to(dev))
        assert torch.equal(plain, o_full)
        # the same through the other kernel form (two query tiles per CTA: what long sequences run), plain and causal
        for causal in (False, True):
            o_full.zero_()
            opeers.barrier()
            runtime.attention_allgather(q[ulo:uhi].to(dev).contiguous(), k[ulo:uhi].to(dev).contiguous(), v[ulo:uhi].to(dev).contiguous(),
                                        [omc + ulo * sq * d * 2], multicast=True, causal=causal, form="two_tiles")
            opeers.barrier()
            torch.cuda.synchronize()
            assert runtime.device_status() == 0
            plain = runtime.attention(q.to(dev), k.to(dev), v.to(dev), causal=causal, form="two_tiles")
            assert torch.equal(plain, o_full), f"rank {rank}: two-tile multicast attention (causal={causal}) differs from the local result"
    finally:
        dist.destroy_process_group()


def _worker(rank: int, world: int, port: int):
    import torch
    import torch.distributed as dist
    from emmyptx import runtime, shard
    from oracle import inputs, reference
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        m, n, k = 1024, 768, 512
        a, b = inputs.gemm_inputs(m, n, k, "bf16")
        lo, hi = shard.split_range(m, world, rank, 128)
        c_full, peers = shard.peer_mapped_empty((m, n), torch.bfloat16, dev)
        c_full.zero_()
        peers.barrier()
        off = lo * n * 2
        dst = [c_full.data_ptr() + off] + [p + off for r, p in enumerate(peers.buffer_ptrs) if r != rank]
        runtime.gemm_allgather(a[lo:hi].to(dev).contiguous(), b.to(dev), dst, n, epilogue="gelu_tanh")
        peers.barrier()
        torch.cuda.synchronize()
        assert runtime.device_status() == 0
        ok, ratio = reference.gemm_tolerance_ok(c_full.cpu(), reference.gemm_reference(a, b, "gelu_tanh"))
        assert ok, f"rank {rank}: worst error {ratio:.2f}x the bound"
        # the same through NCCL, as the cross-check of the assembled layout
        local = runtime.gemm(a[lo:hi].to(dev).contiguous(), b.to(dev), epilogue="gelu_tanh")
        gathered = shard.all_gather_rows(torch.empty(m, n, dtype=torch.bfloat16, device=dev), local)
        assert torch.equal(gathered, c_full)
        # attention: units split over the ranks, every output tile stored to both copies of O
        units, sq, sk, d = 4, 300, 260, 128
        q, k, v = inputs.attention_inputs(units, sq, sk, d, "bf16")
        ulo, uhi = shard.split_range(units, world, rank)
        o_full, opeers = shard.peer_mapped_empty((units, sq, d), torch.bfloat16, dev)
        o_full.zero_()
        opeers.barrier()
        ooff = ulo * sq * d * 2
        odst = [o_full.data_ptr() + ooff] + [p + ooff for r, p in enumerate(opeers.buffer_ptrs) if r != rank]
        runtime.attention_allgather(q[ulo:uhi].to(dev).contiguous(), k[ulo:uhi].to(dev).contiguous(), v[ulo:uhi].to(dev).contiguous(), odst)
        opeers.barrier()
        torch.cuda.synchronize()
        assert runtime.device_status() == 0
        ok, ratio = reference.gemm_tolerance_ok(o_full.cpu(), reference.attention_reference(q, k, v))
        assert ok, f"rank {rank}: attention worst error {ratio:.2f}x the bound"
        o_full.zero_()
        opeers.barrier()
        runtime.attention_allgather(q[ulo:uhi].to(dev).contiguous(), k[ulo:uhi].to(dev).contiguous(), v[ulo:uhi].to(dev).contiguous(), odst,
                                    form="two_tiles")
        opeers.barrier()
        torch.cuda.synchronize()
        assert runtime.device_status() == 0
        assert torch.equal(runtime.attention(q.to(dev), k.to(dev), v.to(dev), form="two_tiles"), o_full), f"rank {rank}: two-tile form"
    finally:
        dist.destroy_process_group()


def test_fused_gemm_allgather_two_gpus():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_multicast_stores_two_gpus():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker_multicast, args=(2, _free_port()), nprocs=2, join=True)
