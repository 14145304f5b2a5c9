"""Benchmark driver: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4|c3|c5|c1|c2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

The default workload is configuration 4 of BASELINE.json: bf16 GEMM + tanh-approx GELU epilogue,
M = N = K = 16384, fp32 accumulation, bf16 output, split by M rows over the ranks (the metric is
quoted at 1/2/4/8 GPUs on this case). A step is one pass of the fused GEMM kernel over the rank's
row shard followed, for N > 1, by the all-gather of the output shards. Inputs are seeded synthetic
tensors of the configuration's shape and distribution, resident in HBM before the timed region
(`value`), or staged from pinned host memory through the public Python API every step (`e2e`).

The timed region is `--steps` x `inner_repeats` passes, `inner_repeats` chosen (the same on every rank) so that the
region lasts at least half a second at every GPU count: short regions run at the boost clock, long ones under the
power cap, and a scaling curve must not mix the two. After the timed regions the result the last pass left behind is
checked against the torch CPU evaluation on a seeded sample of rows -- at N > 1 rows that OTHER ranks computed and
the fused gather delivered into this rank's copy -- and reported as `parity`.

`--impl reference` times the reference's CPU path for the same workload -- the torch CPU evaluation of
the same expression (tools/check_torch.py:194-237 defines it as the truth) -- on the host cores: the whole
workload per step when the run then ends within a few minutes, else a bounded sample named in `config.sample`.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "emmy-ptx-compiler_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of each workload's kernel, from the ncu captures summarised
# under profiles/ (c4: a one-pass capture of the two counters at the full M=N=K=16384; c5: captured on 64 of the 256
# units and scaled by 4; c2, c3: captured at full size; c1: 8 MiB working set, L2-resident, no DRAM figure; lerp: the
# kernel compiled for the program, at N=2^26).
DRAM_TRAFFIC = {"c4": 8.83e9 + 0.53713e9, "c5": 4 * (201.55e6 + 46.59e6), "c2": 268.97e6 + 222.76e6,
                "c3": 83.01e6 + 14.28e6, "c1": None, "softmax": 268.46e6 + 216.40e6, "f32mm": None, "lerp": None}

WORKLOADS = {
    "c1": "fp32 exp(x)+sin(x)*tanh(x), N=2^20, x~U[-4,4]",
    "c2": "int32 gather y[i]=(x[(i*7919+13) mod N]//3)^(i>>2), N=2^26",
    "c3": "fp16 GEMM M=N=K=4096, fp32 accumulate, fp16 out",
    "c4": "bf16 GEMM + tanh-GELU epilogue M=N=K=16384, fp32 accumulate, bf16 out, M-row shards",
    "c5": "bf16 attention fwd B16 H16 S4096 d128, non-causal, fp32 softmax, (batch x head) shards",
    "causal": "bf16 causal attention fwd, 64 units of S4096 d128 (the two-tiles-per-CTA kernel form; not one of the five configurations)",
    "transpose": "fp32 transposition of 8192 x 8192 through the indexed elementwise kernel (shared-memory tiles, compiled at first use; not one of the five configurations)",
    "lerp": "fp32 x + 0.3*(y - x) over 2^26 elements, two inputs, through the general elementwise entry point (the program compiled into a kernel of its own at first use; not one of the five configurations)",
    "f32mm": "fp32 matmul M=N=K=4096 with fp32 accuracy (three-way bf16 split on the tensor cores; not one of the five configurations)",
    "softmax": "fp32 softmax over the last axis of [65536, 1024] (the row kernels; not one of the five configurations)",
}


def peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self) -> None:
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- the five workloads -------------------------------------------------------------------------------
def group_has_multicast(address: int, dev) -> bool:
    """True if every rank got a multicast address for the buffer (the ranks must take the same path)."""
    import torch
    import torch.distributed as dist
    flag = torch.tensor([1 if address else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


class Workload:
    """One configuration: device-resident inputs for this rank, the step, its algorithmic work."""

    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"
    scaling = "strong"

    def step(self) -> None: ...
    def work_per_step(self) -> float: ...        # whole job, in the metric's base unit (flop or bytes)
    def kernel_work_per_launch(self) -> float: ...
    def launches_per_step(self) -> int: return 1


def _pipeline_note(self) -> str:
    ring = getattr(self, "ring", None)
    if ring is not None and ring.pipelined:
        return " on a side stream: two copies of the output alternate, so the barrier of step k overlaps the kernel of step k+1 (step k+2 waits for it)"
    return " in line after the kernel"


class GatherRing:
    """The gathered output of a sharded step, in peer-mapped memory on every rank, twice: step k writes copy k % 2.
    The group barrier that tells a consumer "every rank's rows of step k have landed everywhere" is issued on a side
    stream after the producing kernel, so it (and the tail of the kernel's stores through NVLink) overlaps the kernel
    of step k + 1, which writes the other copy and needs no barrier; step k + 2 reuses copy k % 2 and therefore first
    waits for barrier k. That is the form EMMYB200_BENCH_PIPELINE=1 selects; by default there is one copy and the barrier
    runs in line after each kernel.
    No kernel waits on another rank: only the barrier kernels do, and nothing that they wait for queues behind them."""

    def __init__(self, torch, shape, dtype, dev, rank, shard_bytes, mode):
        from emmyptx import shard
        self.torch = torch
        self.pipelined = os.environ.get("EMMYB200_BENCH_PIPELINE", "0") != "0"
        self.mode = mode
        self.copies = []
        for _ in range(2 if self.pipelined else 1):
            full, peers = shard.peer_mapped_empty(shape, dtype, dev, multicast=mode == "multicast")
            self.copies.append([full, peers, None])
        off = rank * shard_bytes
        if self.mode == "multicast" and not all(group_has_multicast(shard.multicast_address(c[1]), dev) for c in self.copies):
            self.mode = "fused"                                           # no multicast object on this fabric
        for c in self.copies:
            full, peers = c[0], c[1]
            c[2] = ([shard.multicast_address(peers) + off] if self.mode == "multicast" else
                    [full.data_ptr() + off] + [p + off for r, p in enumerate(peers.buffer_ptrs) if r != rank])
        self.side = torch.cuda.Stream(device=dev) if self.pipelined else None
        self.landed = [None] * len(self.copies)       # event: the barrier after the last kernel that wrote copy i
        self.count = 0
        self.last = 0

    def begin(self):
        """Destination addresses for the next step's kernel; called on the launching stream before the launch."""
        i = self.count % len(self.copies)
        self.count += 1
        self.last = i
        if self.pipelined and self.landed[i] is not None:
            self.torch.cuda.current_stream().wait_event(self.landed[i])  # the copy's previous contents are no longer needed
        return self.copies[i][2]

    def end(self):
        """After the launch: the group barrier for the copy just written."""
        i = self.last
        if not self.pipelined:
            self.copies[i][1].barrier()
            return
        main = self.torch.cuda.current_stream()
        done = self.torch.cuda.Event()
        done.record(main)
        with self.torch.cuda.stream(self.side):
            self.side.wait_event(done)
            self.copies[i][1].barrier()
            ev = self.torch.cuda.Event()
            ev.record(self.side)
        self.landed[i] = ev

    def finish(self):
        """The launching stream waits for every barrier still in flight (end of a timed region, before reading)."""
        for ev in self.landed:
            if ev is not None:
                self.torch.cuda.current_stream().wait_event(ev)

    @property
    def full(self):
        return self.copies[self.last][0]


class GemmWorkload(Workload):
    metric, unit, bound = "gemm_tflops", "TFLOP/s", "tensor"
    _pipeline_note = _pipeline_note

    def __init__(self, name, m, n, k, dtype, epilogue, rank, world, dev, gather=True):
        import torch
        from emmyptx import runtime
        self.rt, self.torch = runtime, torch
        self.name, self.dtype = name, dtype
        self.m, self.n, self.k, self.epilogue = m, n, k, epilogue
        self.rank, self.world = rank, world
        self.rows = m // world
        td = torch.float16 if dtype == "f16" else torch.bfloat16
        g = torch.Generator(device=dev)
        g.manual_seed(1)
        self.b = (torch.randn(k, n, device=dev, generator=g, dtype=torch.float32) / k**0.5).to(td)
        g.manual_seed(1000 + rank)
        self.a = (torch.randn(self.rows, k, device=dev, generator=g, dtype=torch.float32) / k**0.5).to(td)
        self.gather = gather and world > 1
        self.host = None
        # "multicast" (one multimem.st per piece, replicated by the NVSwitch), "fused" (one TMA store per peer) or "nccl"
        self.mode = os.environ.get("EMMYB200_BENCH_GATHER", "multicast")
        self.ring = None
        if self.gather and self.mode in ("fused", "multicast"):
            # The full C lives in peer-mapped memory on every rank; each rank's kernel writes its rows into all of them.
            try:
                self.ring = GatherRing(torch, (m, n), td, dev, rank, self.rows * n * 2, self.mode)
                self.mode = self.ring.mode
            except Exception as e:  # noqa: BLE001 - no peer mapping on this box: gather with NCCL instead
                print(f"[bench] peer-mapped memory unavailable ({type(e).__name__}: {e}); gathering with NCCL", file=sys.stderr)
                self.mode = "nccl"
        if self.ring is None:
            self._c_full = torch.empty(m, n, device=dev, dtype=td)
        self.c = self.c_full[rank * self.rows:(rank + 1) * self.rows]

    @property
    def c_full(self):
        return self.ring.full if self.ring is not None else self._c_full

    def step(self):
        if self.ring is not None:
            dst = self.ring.begin()
            self.rt.gemm_allgather(self.a, self.b, dst, self.n, epilogue=self.epilogue, multicast=self.mode == "multicast")
            self.ring.end()                     # every rank's rows have landed everywhere once this barrier has run
            return
        self.rt.gemm(self.a, self.b, epilogue=self.epilogue, out=self.c)
        if self.gather:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.c_full, self.c)

    def finish(self):
        if self.ring is not None:
            self.ring.finish()

    def kernel_only(self):
        self.rt.gemm(self.a, self.b, epilogue=self.epilogue, out=self.c)

    @property
    def collective(self):
        if self.mode == "multicast":
            return "fused: the GEMM stores each output piece once through the NVSwitch multicast mapping of C (multimem.st), then a signal barrier" + self._pipeline_note()
        if self.mode == "fused":
            return "fused: the GEMM's TMA stores write each output piece to every peer's C over NVLink, then a signal barrier" + self._pipeline_note()
        return "nccl all_gather of the output shards"

    def work_per_step(self):
        return 2.0 * self.m * self.n * self.k

    def kernel_work_per_launch(self):
        return 2.0 * self.rows * self.n * self.k

    def parity(self, rows_per_owner: int = 0):
        """The C the last pass left behind against the torch CPU evaluation (fp32 product of the rounded operands, the
        epilogue on the fp32 value, tools/check_torch.py:194-237), on a seeded sample of whole rows of every rank's
        slab as this rank holds them after the gather: first / last rows of the slab and of 128-row tiles, the rest
        random. Tolerance |c - ref| <= 1e-2 |ref| + 1e-2 std(ref)."""
        t = self.torch
        per = rows_per_owner or max(32, 256 // self.world)
        g = t.Generator().manual_seed(77 + self.rank)
        b32 = self.b.float().cpu()
        worst, checked, foreign = 0.0, 0, 0
        for owner in range(self.world):
            if not self.gather and owner != self.rank:
                continue
            fixed = [0, 127, 128, self.rows // 2 - 1, self.rows // 2, self.rows - 129, self.rows - 128, self.rows - 1]
            pick = sorted({r for r in fixed if 0 <= r < self.rows} |
                          set(t.randint(0, self.rows, (max(per - len(fixed), 0),), generator=g).tolist()))
            if owner == self.rank:
                a_rows = self.a[pick]
            else:                                   # the owner's A, regenerated from its seed
                gd = t.Generator(device=self.a.device)
                gd.manual_seed(1000 + owner)
                a_rows = (t.randn(self.rows, self.k, device=self.a.device, generator=gd, dtype=t.float32) / self.k**0.5).to(self.a.dtype)[pick]
                foreign += len(pick)
            ref = a_rows.float().cpu() @ b32
            if self.epilogue == "gelu_tanh":
                ref = t.nn.functional.gelu(ref, approximate="tanh")
            got = self.c_full[[owner * self.rows + r for r in pick]].float().cpu()
            bound = 1e-2 * ref.abs() + 1e-2 * ref.std()
            worst = max(worst, float(((got - ref).abs() / bound).max()))
            checked += len(pick)
        return {"checked_rows": checked, "rows_from_other_ranks": foreign, "worst_ratio": worst, "ok": bool(worst <= 1.0),
                "rule": "|c-ref| <= 1e-2|ref| + 1e-2 std(ref), ref = torch CPU fp32 on the same rounded operands"}

    def e2e_setup(self):
        t = self.torch
        self.host = {"a": self.a.cpu().pin_memory(), "b": self.b.cpu().pin_memory(),
                     "c": t.empty_like(self.c, device="cpu").pin_memory()}
        if self.world == 1:
            # the library's host-buffer call: chunked copies overlapped with the kernel (emmyptx.runtime.HostGemm)
            self.host_gemm = self.rt.HostGemm(self.m, self.n, self.k, self.a.dtype, self.a.device, self.epilogue)
        else:
            step = 1024 if self.rows % 1024 == 0 else self.rows
            self.chunks = [(lo, lo + step) for lo in range(0, self.rows, step)]
            self.copy_in = t.cuda.Stream(self.a.device)
            self.ev_in = [t.cuda.Event() for _ in range(len(self.chunks) + 1)]
            kb = self.k // self.world
            self.b_rows = (self.rank * kb, (self.rank + 1) * kb)
            if self.gather and self.mode in ("fused", "multicast"):     # bytes of the whole job: A and B once in, C once out
                return (self.host["a"].numel() + self.b[self.b_rows[0]:self.b_rows[1]].numel()) * 2 * self.world, self.host["c"].numel() * 2 * self.world
        return self.host["a"].numel() * 2 + self.host["b"].numel() * 2, self.host["c"].numel() * 2

    def e2e_step(self):
        h = self.host
        if self.world == 1:
            self.host_gemm(h["a"], h["b"], h["c"])
            return
        if self.gather and self.mode in ("fused", "multicast"):
            # the same overlap across ranks: B once, this rank's rows of A in chunks on a copy stream, one fused
            # GEMM + gather per chunk as it lands; the group barrier, then this rank's rows of C back
            t = self.torch
            main = t.cuda.current_stream()
            self.copy_in.wait_stream(main)
            with t.cuda.stream(self.copy_in):
                # B is replicated on the devices but crosses the host link once: every rank copies its K / world rows
                # and the ranks exchange them over NVLink (NCCL all-gather, in place)
                self.b[self.b_rows[0]:self.b_rows[1]].copy_(h["b"][self.b_rows[0]:self.b_rows[1]], non_blocking=True)
                self.ev_in[0].record()
                for i, (lo, hi) in enumerate(self.chunks):
                    self.a[lo:hi].copy_(h["a"][lo:hi], non_blocking=True)
                    self.ev_in[i + 1].record()
            main.wait_event(self.ev_in[0])
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.b, self.b[self.b_rows[0]:self.b_rows[1]])
            for i, (lo, hi) in enumerate(self.chunks):
                main.wait_event(self.ev_in[i + 1])
                dst = [d + lo * self.n * 2 for d in self.ring.copies[0][2]]       # copy 0, whose rows self.c views
                self.rt.gemm_allgather(self.a[lo:hi], self.b, dst, self.n, epilogue=self.epilogue, multicast=self.mode == "multicast")
            self.ring.copies[0][1].barrier()
            h["c"].copy_(self.c, non_blocking=True)
            return
        self.a.copy_(h["a"], non_blocking=True)
        self.b.copy_(h["b"], non_blocking=True)
        self.step()
        h["c"].copy_(self.c, non_blocking=True)


class PointwiseWorkload(Workload):
    metric, unit, dtype, scaling = "elementwise_gbs", "GB/s", "f32", "weak"

    def __init__(self, n, rank, world, dev):
        import torch
        from emmyptx import runtime
        self.rt, self.torch, self.world = runtime, torch, world
        self.name = "c1"
        self.n = n
        g = torch.Generator(device=dev)
        g.manual_seed(rank)
        self.x = torch.rand(n, device=dev, generator=g) * 8 - 4
        self.y = torch.empty_like(self.x)

    def step(self):
        self.rt.pointwise("exp_sin_tanh", self.x, out=self.y)

    kernel_only = step

    def parity(self):
        """The reference's own tolerance class for transcendental cases (rtol = atol = 1e-5, tools/torch_cases/__init__.py:18)
        against the float64 torch CPU evaluation, on a strided sample of at most 2^20 elements."""
        t = self.torch
        idx = t.arange(0, self.n, max(1, self.n // 2**20), device=self.x.device)
        x = self.x[idx].cpu().double()
        ref = t.exp(x) + t.sin(x) * t.tanh(x)
        err = (self.y[idx].cpu().double() - ref).abs() / (1e-5 + 1e-5 * ref.abs())
        return {"checked_elements": int(idx.numel()), "worst_ratio": float(err.max()), "ok": bool(err.max() <= 1.0),
                "rule": "isclose(rtol=1e-5, atol=1e-5) against torch CPU float64"}

    def work_per_step(self):
        return 8.0 * self.n * self.world

    def kernel_work_per_launch(self):
        return 8.0 * self.n

    def e2e_setup(self):
        self.host = {"x": self.x.cpu().pin_memory(), "y": self.torch.empty_like(self.y, device="cpu").pin_memory()}
        return self.n * 4, self.n * 4

    def e2e_step(self):
        self.x.copy_(self.host["x"], non_blocking=True)
        self.step()
        self.host["y"].copy_(self.y, non_blocking=True)


class GemmF32Workload(Workload):
    """emmyb200_gemm_f32 on square fp32 operands; one step = split kernels + the six-pass GEMM."""
    metric, unit, bound, dtype = "gemm_tflops", "TFLOP/s", "tensor", "f32"

    def __init__(self, s, rank, world, dev):
        import torch
        from emmyptx import runtime
        self.rt, self.torch, self.world, self.s, self.name = runtime, torch, world, s, "f32mm"
        g = torch.Generator(device=dev)
        g.manual_seed(rank)
        self.a = torch.randn(s, s, device=dev, generator=g) / s**0.5
        self.b = torch.randn(s, s, device=dev, generator=g) / s**0.5
        self.c = torch.empty(s, s, device=dev)
        need = runtime.library().emmyb200_gemm_f32_workspace_bytes(0, 1, s, s, s, 1)
        self.ws = torch.empty(need, dtype=torch.uint8, device=dev)

    def step(self):
        self.rt.gemm_f32(self.a, self.b, out=self.c, workspace=self.ws)

    kernel_only = step

    def parity(self):
        t = self.torch
        rows = t.randint(0, self.s, (128,), generator=t.Generator().manual_seed(81))
        ref = self.a[rows].cpu().double() @ self.b.cpu().double()
        err = (self.c[rows].cpu().double() - ref).abs() / (1e-3 + 1e-3 * ref.abs())
        return {"checked_rows": 128, "worst_ratio": float(err.max()), "ok": bool(err.max() <= 1.0),
                "rule": "isclose(rtol=1e-3, atol=1e-3) against torch CPU float64 (tools/torch_cases/__init__.py:20)"}

    def launches_per_step(self):
        return 3

    def work_per_step(self):
        return 2.0 * self.s**3 * self.world

    def kernel_work_per_launch(self):
        return 2.0 * self.s**3

    def e2e_setup(self):
        self.host = {"a": self.a.cpu().pin_memory(), "b": self.b.cpu().pin_memory(), "c": self.c.cpu().pin_memory()}
        return 2 * self.s * self.s * 4, self.s * self.s * 4

    def e2e_step(self):
        self.a.copy_(self.host["a"], non_blocking=True)
        self.b.copy_(self.host["b"], non_blocking=True)
        self.step()
        self.host["c"].copy_(self.c, non_blocking=True)


class RowWorkload(PointwiseWorkload):
    """A row kernel on [rows, 1024] fp32; `n` counts elements. Rows shard across ranks like C1's chunks."""

    def __init__(self, op, n, rank, world, dev):
        import torch
        from emmyptx import runtime
        self.rt, self.torch, self.world = runtime, torch, world
        self.name, self.op, self.n = op, op, n
        g = torch.Generator(device=dev)
        g.manual_seed(rank)
        self.x = torch.randn(n // 1024, 1024, device=dev, generator=g)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.rt.rowwise(self.op, self.x, out=self.y)

    kernel_only = step

    def parity(self):
        t = self.torch
        rows = t.randint(0, self.x.shape[0], (256,), generator=t.Generator().manual_seed(80))
        ref = t.softmax(self.x[rows].cpu().double(), -1)
        err = (self.y[rows].cpu().double() - ref).abs() / (1e-5 + 1e-3 * ref.abs())
        return {"checked_rows": 256, "worst_ratio": float(err.max()), "ok": bool(err.max() <= 1.0),
                "rule": "isclose(rtol=1e-3, atol=1e-5) against torch CPU float64 (tools/torch_cases/fused.py:6)"}


class ProgramWorkload(PointwiseWorkload):
    """torch.lerp(x, y, 0.3) (tools/torch_cases/pointwise.py:47 `p_lerp`) compiled from IR by the facade to a program for
    the general elementwise entry point, which compiles it into a kernel of its own at its first launch (a warm-up step):
    12 bytes per element (two reads, one write)."""

    def __init__(self, n, rank, world, dev):
        import json as _json
        import torch
        from emmyptx import ir, runtime
        from emmyptx.kernel import compile_kernel
        self.rt, self.torch, self.world, self.name, self.n = runtime, torch, world, "lerp", n
        built = ir.elementwise_kernel(n, {"x": "f32", "y": "f32"}, [("d", "subtract", ["y", "x"]), ("w", "multiply", ["d", 0.3]), ("o", "add", ["x", "w"])])
        self.handle = _json.loads(compile_kernel(*built))
        assert self.handle["variant"] == "pointwise_program"
        g = torch.Generator(device=dev)
        g.manual_seed(rank)
        self.x = torch.randn(n, device=dev, generator=g)
        self.x2 = torch.randn(n, device=dev, generator=g)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.rt.pointwise_program(self.handle["params"]["program"], [self.x, self.x2], self.y)

    kernel_only = step

    def work_per_step(self):
        return 12.0 * self.n * self.world

    def kernel_work_per_launch(self):
        return 12.0 * self.n

    def e2e_setup(self):
        self.host = {"x": self.x.cpu().pin_memory(), "x2": self.x2.cpu().pin_memory(), "y": self.torch.empty_like(self.y, device="cpu").pin_memory()}
        return self.n * 8, self.n * 4

    def e2e_step(self):
        self.x.copy_(self.host["x"], non_blocking=True)
        self.x2.copy_(self.host["x2"], non_blocking=True)
        self.step()
        self.host["y"].copy_(self.y, non_blocking=True)

    def parity(self):
        t = self.torch
        idx = t.arange(0, self.n, max(1, self.n // 2**20), device=self.x.device)
        x, y = self.x[idx].cpu().double(), self.x2[idx].cpu().double()
        ref = x + 0.3 * (y - x)
        err = (self.y[idx].cpu().double() - ref).abs() / (1e-6 + 1e-6 * ref.abs())
        return {"checked_elements": int(idx.numel()), "worst_ratio": float(err.max()), "ok": bool(err.max() <= 1.0),
                "rule": "isclose(rtol=1e-6, atol=1e-6) against torch CPU float64 (tools/torch_cases/__init__.py:17)"}


class TransposeWorkload(PointwiseWorkload):
    """x.t().contiguous() (tools/torch_cases/shapes.py:6 `s_transpose`, at 8192 x 8192 instead of 64 x 96) from IR through the
    facade to the indexed elementwise kernel (shared-memory tiles): 8 bytes per element."""

    def __init__(self, side, rank, world, dev):
        import json as _json
        import torch
        from emmyptx import ir, runtime
        from emmyptx.kernel import compile_kernel
        self.rt, self.torch, self.world, self.name, self.side, self.n = runtime, torch, world, "transpose", side, side * side
        ax = [ir.Axis("i0", ir.Dim(side)), ir.Axis("j0", ir.Dim(side))]
        body = [ir.Load(["x"], "X", [ir.Var("j0"), ir.Var("i0")]), ir.Write("out", [ir.Var("i0"), ir.Var("j0")], ["x"])]
        k = ir.KernelOp("k_transpose", [ir.Tile(ax, body)])
        g = ir._graph(k, [ir.tensor("X", [side, side], "f32")], [ir.tensor("out", [side, side], "f32")])
        self.handle = _json.loads(compile_kernel(g, k, ir._launch(k, ["X", "out"], side * side)))
        assert self.handle["variant"] == "pointwise_indexed"
        gen = torch.Generator(device=dev)
        gen.manual_seed(rank)
        self.x = torch.randn(side, side, device=dev, generator=gen)
        self.y = torch.empty_like(self.x)

    def step(self):
        p = self.handle["params"]
        self.rt.pointwise_indexed(p["program"], p["index_map"], [self.x.reshape(-1)], self.y.reshape(-1))

    kernel_only = step

    def work_per_step(self):
        return 8.0 * self.n * self.world

    def kernel_work_per_launch(self):
        return 8.0 * self.n

    def e2e_setup(self):
        self.host = {"x": self.x.cpu().pin_memory(), "y": self.torch.empty_like(self.y, device="cpu").pin_memory()}
        return self.n * 4, self.n * 4

    def e2e_step(self):
        self.x.copy_(self.host["x"], non_blocking=True)
        self.step()
        self.host["y"].copy_(self.y, non_blocking=True)

    def parity(self):
        ok = bool(self.torch.equal(self.y, self.x.t().contiguous()))
        return {"checked_elements": self.n, "worst_ratio": 0.0 if ok else float("inf"), "ok": ok, "rule": "bit-exact against torch's transpose"}


class GatherWorkload(PointwiseWorkload):
    dtype = "i32"

    def __init__(self, n, rank, world, dev):
        import torch
        from emmyptx import runtime
        self.rt, self.torch, self.world = runtime, torch, world
        self.name = "c2"
        self.n = n
        g = torch.Generator(device=dev)
        g.manual_seed(rank)
        self.x = torch.randint(-2**30, 2**30 + 1, (n,), device=dev, generator=g, dtype=torch.int32)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.rt.index_gather(self.x, 7919, 13, 3, 2, out=self.y)

    kernel_only = step

    def parity(self):
        """Bit-exact against torch CPU (int64 index arithmetic, floor division) on a seeded sample of 2^20 positions."""
        t = self.torch
        i = t.randint(0, self.n, (2**20,), generator=t.Generator().manual_seed(79), dtype=t.int64)
        x = self.x.cpu()
        ref = t.bitwise_xor(t.div(x[(i * 7919 + 13) % self.n], 3, rounding_mode="floor"), (i >> 2).to(t.int32))
        same = bool(t.equal(self.y.cpu()[i], ref))
        return {"checked_elements": int(i.numel()), "worst_ratio": 0.0 if same else float("inf"), "ok": same, "rule": "bit-exact"}


class AttentionWorkload(Workload):
    metric, unit, dtype, bound = "attention_tflops", "TFLOP/s", "bf16", "tensor"
    _pipeline_note = _pipeline_note

    def __init__(self, units, seq, d, rank, world, dev, gather=True, causal=False):
        import torch
        from emmyptx import runtime
        self.rt, self.torch = runtime, torch
        self.causal = causal
        self.name = "c5"
        self.units, self.seq, self.d, self.world, self.rank = units, seq, d, world, rank
        self.local = units // world
        g = torch.Generator(device=dev)
        g.manual_seed(2000 + rank)
        mk = lambda: torch.randn(self.local, seq, d, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
        self.q, self.k, self.v = mk(), mk(), mk()
        self.gather = gather and world > 1
        self.mode = os.environ.get("EMMYB200_BENCH_GATHER", "multicast")
        self.ring = None
        if self.gather and self.mode in ("fused", "multicast"):
            try:
                self.ring = GatherRing(torch, (units, seq, d), torch.bfloat16, dev, rank, self.local * seq * d * 2, self.mode)
                self.mode = self.ring.mode
            except Exception as e:  # noqa: BLE001
                print(f"[bench] peer-mapped memory unavailable ({type(e).__name__}: {e}); gathering with NCCL", file=sys.stderr)
                self.mode = "nccl"
        if self.ring is None:
            self._o_full = torch.empty(units, seq, d, device=dev, dtype=torch.bfloat16)
        self.o = self.o_full[rank * self.local:(rank + 1) * self.local]

    @property
    def o_full(self):
        return self.ring.full if self.ring is not None else self._o_full

    def finish(self):
        if self.ring is not None:
            self.ring.finish()

    @property
    def collective(self):
        if self.mode == "multicast":
            return "fused: the attention kernel stores each output tile once through the NVSwitch multicast mapping of O (multimem.st), then a signal barrier" + self._pipeline_note()
        if self.mode == "fused":
            return "fused: the attention kernel's TMA stores write each output tile to every peer's O over NVLink, then a signal barrier" + self._pipeline_note()
        return "nccl all_gather of the output shards"

    def step(self):
        if self.ring is not None:
            dst = self.ring.begin()
            self.rt.attention_allgather(self.q, self.k, self.v, dst, multicast=self.mode == "multicast")
            self.ring.end()
            return
        self.rt.attention(self.q, self.k, self.v, causal=self.causal, out=self.o)
        if self.gather:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.o_full, self.o)

    def kernel_only(self):
        self.rt.attention(self.q, self.k, self.v, causal=self.causal, out=self.o)

    def pairs(self):
        return self.seq * (self.seq + 1) / 2 if self.causal else float(self.seq) * self.seq

    def work_per_step(self):
        return 4.0 * self.units * self.pairs() * self.d

    def kernel_work_per_launch(self):
        return 4.0 * self.local * self.pairs() * self.d

    def parity(self, rows_per_unit: int = 64):
        """O as the last pass left it against the torch CPU fp32 evaluation of softmax(q k^T / sqrt(d)) v, on seeded
        query rows of the first and last unit of every rank's share as this rank holds them after the gather."""
        t = self.torch
        g = t.Generator().manual_seed(78 + self.rank)
        worst, checked, foreign = 0.0, 0, 0
        for owner in range(self.world):
            if not self.gather and owner != self.rank:
                continue
            if owner == self.rank:
                q, k, v = self.q, self.k, self.v
            else:
                gd = t.Generator(device=self.q.device)
                gd.manual_seed(2000 + owner)
                q, k, v = (t.randn(self.local, self.seq, self.d, device=self.q.device, generator=gd, dtype=t.float32).to(t.bfloat16)
                           for _ in range(3))
            for u in sorted({0, self.local - 1}):
                fixed = [0, 127, 128, self.seq - 1]
                pick = sorted(set(fixed) | set(t.randint(0, self.seq, (rows_per_unit - len(fixed),), generator=g).tolist()))
                qs, ks, vs = q[u][pick].float().cpu(), k[u].float().cpu(), v[u].float().cpu()
                sc = qs @ ks.t() * self.d ** -0.5
                if self.causal:
                    sc = sc.masked_fill(t.arange(self.seq)[None, :] > t.tensor(pick)[:, None], float("-inf"))
                ref = t.softmax(sc, -1) @ vs
                got = self.o_full[owner * self.local + u][pick].float().cpu()
                bound = 1e-2 * ref.abs() + 1e-2 * ref.std()
                worst = max(worst, float(((got - ref).abs() / bound).max()))
                checked += len(pick)
                foreign += len(pick) if owner != self.rank else 0
            del q, k, v
        return {"checked_rows": checked, "rows_from_other_ranks": foreign, "worst_ratio": worst, "ok": bool(worst <= 1.0),
                "rule": "|o-ref| <= 1e-2|ref| + 1e-2 std(ref), ref = torch CPU fp32 on the same rounded operands"}

    def e2e_setup(self):
        t = self.torch
        self.host = {n: getattr(self, n).cpu().pin_memory() for n in "qkv"}
        self.host["o"] = t.empty_like(self.o, device="cpu").pin_memory()
        # bytes of the whole job, like `value`: every rank copies its own units
        return 3 * self.q.numel() * 2 * self.world, self.o.numel() * 2 * self.world

    def e2e_step(self):
        for n in "qkv":
            getattr(self, n).copy_(self.host[n], non_blocking=True)
        self.step()
        self.finish()
        mine = self.o_full[self.rank * self.local:(self.rank + 1) * self.local] if self.ring is not None else self.o
        self.host["o"].copy_(mine, non_blocking=True)


def make_workload(name, rank, world, dev, size=None):
    """`size` overrides the configuration's extent (GEMM M=N=K, attention units, streaming elements): used for
    small profiler captures of the same kernels, never for the reported line."""
    if name == "c4":
        s = size or 16384
        return GemmWorkload("c4", s, s, s, "bf16", "gelu_tanh", rank, world, dev)
    if name == "c3":
        s = size or 4096
        return GemmWorkload("c3", s, s, s, "f16", None, rank, world, dev)
    if name == "c5":
        return AttentionWorkload(size or 256, 4096, 128, rank, world, dev)
    if name == "c1":
        return PointwiseWorkload(size or 2**20, rank, world, dev)
    if name == "c2":
        return GatherWorkload(size or 2**26, rank, world, dev)
    if name == "causal":
        return AttentionWorkload(size or 64, 4096, 128, rank, world, dev, gather=False, causal=True)
    if name == "lerp":
        return ProgramWorkload(size or 2**26, rank, world, dev)
    if name == "transpose":
        return TransposeWorkload(size or 8192, rank, world, dev)
    if name == "softmax":
        return RowWorkload("softmax", size or 65536 * 1024, rank, world, dev)
    if name == "f32mm":
        return GemmF32Workload(size or 4096, rank, world, dev)
    raise SystemExit(f"unknown workload {name!r}")


# ---- timing ---------------------------------------------------------------------------------------------
def timed(torch, dist, world, fn, steps, warmup, finish=None):
    """Device time of exactly `steps` calls of fn, max over ranks, in ms (total). `finish` (a workload's way of waiting,
    on the launching stream, for work it put on other streams) runs inside the timed region, after the last call."""
    for _ in range(warmup):
        fn()
    if finish is not None:
        finish()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if finish is not None:
        finish()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def graph_timed(torch, fn, launches, reps=5):
    """Average device time per launch of `fn` captured `launches` times in one CUDA graph (takes the
    host's launch cost out of the measurement of kernels that run for a few microseconds)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            fn()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(launches):
                fn()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * launches)


# ---- the reference's CPU path -------------------------------------------------------------------------------
def cpu_reference_step(name: str, threads: int, full: bool = False):
    """(callable running one pass or a bounded sample of it, work of that call in the metric's base unit, unit scale,
    description of the sample). The expression is the case's torch code on CPU, all host threads. `full` asks for
    the whole workload where the default is a sample (the two GEMM configurations and attention)."""
    import torch
    import numpy as np
    torch.set_num_threads(threads)
    if name in ("c3", "c4"):
        n = k = 16384 if name == "c4" else 4096
        rows = n if (full or name == "c3") else 1024
        td = torch.bfloat16 if name == "c4" else torch.float16
        g = torch.Generator().manual_seed(0)
        a = (torch.randn(rows, k, generator=g) / k**0.5).to(td)
        b = (torch.randn(k, n, generator=g) / k**0.5).to(td)
        if name == "c4":
            fn = lambda: torch.nn.functional.gelu(a @ b, approximate="tanh")
        else:
            fn = lambda: a @ b
        what = "the whole product" if rows == n else f"{rows} of {n} rows of A against the full B"
        return fn, 2.0 * rows * n * k, 1e12, f"{what}, torch CPU {str(td).split('.')[-1]}"
    if name == "c5":
        units, s, d = (256 if full else 4), 4096, 128
        g = torch.Generator().manual_seed(0)
        q, kk, v = (torch.randn(units, s, d, generator=g).to(torch.bfloat16) for _ in range(3))
        fn = lambda: torch.nn.functional.scaled_dot_product_attention(q, kk, v)
        return fn, 4.0 * units * s * s * d, 1e12, f"{units} of 256 (batch, head) units, torch CPU bf16 SDPA"
    if name == "c1":
        n = 2**20
        x = torch.from_numpy(np.random.default_rng(0).uniform(-4, 4, n).astype(np.float32))
        fn = lambda: torch.exp(x) + torch.sin(x) * torch.tanh(x)
        return fn, 8.0 * n, 1e9, "the full 2^20 array, torch CPU fp32"
    if name == "c2":
        n = 2**26
        from oracle import inputs, reference
        x = torch.from_numpy(inputs.c2_input(n))
        fn = lambda: reference.c2_torch(x)
        return fn, 8.0 * n, 1e9, "the full 2^26 array, torch CPU int32/int64"
    if name == "causal":
        g = torch.Generator().manual_seed(0)
        q, kk, v = (torch.randn(2, 4096, 128, generator=g).to(torch.bfloat16) for _ in range(3))
        fn = lambda: torch.nn.functional.scaled_dot_product_attention(q, kk, v, is_causal=True)
        return fn, 4.0 * 2 * 4096 * 4097 / 2 * 128, 1e12, "2 of 64 units, torch CPU bf16 causal SDPA"
    if name == "lerp":
        g = torch.Generator().manual_seed(0)
        x, y = torch.randn(2**24, generator=g), torch.randn(2**24, generator=g)
        fn = lambda: torch.lerp(x, y, 0.3)
        return fn, 12.0 * x.numel(), 1e9, "2^24 of 2^26 elements, torch CPU fp32"
    if name == "transpose":
        x = torch.randn(4096, 4096, generator=torch.Generator().manual_seed(0))
        fn = lambda: x.t().contiguous()
        return fn, 8.0 * x.numel(), 1e9, "4096 x 4096 of 8192 x 8192, torch CPU fp32"
    if name == "f32mm":
        g = torch.Generator().manual_seed(0)
        a, b = torch.randn(4096, 4096, generator=g), torch.randn(4096, 4096, generator=g)
        return (lambda: a @ b), 2.0 * 4096**3, 1e12, "the full 4096^3 product, torch CPU fp32"
    if name == "softmax":
        x = torch.randn(65536, 1024, generator=torch.Generator().manual_seed(0))
        fn = lambda: torch.softmax(x, -1)
        return fn, 8.0 * x.numel(), 1e9, "the full [65536, 1024] array, torch CPU fp32"
    raise SystemExit(name)


def time_cpu(fn, budget_s: float = 12.0, min_reps: int = 2) -> float:
    """Best wall time of fn over as many repetitions as fit the budget (after one warm-up)."""
    fn()
    best, t_end, reps = float("inf"), time.perf_counter() + budget_s, 0
    while reps < min_reps or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
        reps += 1
        if reps >= 50:
            break
    return best


METRIC = {"c1": "elementwise_gbs", "c2": "elementwise_gbs", "softmax": "elementwise_gbs", "lerp": "elementwise_gbs", "transpose": "elementwise_gbs", "c5": "attention_tflops",
          "causal": "attention_tflops"}
DTYPE = {"c1": "f32", "c2": "i32", "c3": "f16", "softmax": "f32", "f32mm": "f32", "lerp": "f32", "transpose": "f32"}
SCALING = {"c1": "weak", "c2": "weak", "softmax": "weak", "f32mm": "weak", "lerp": "weak", "transpose": "weak", "causal": "weak"}


def config_for(workload: str, world: int, size=None) -> dict:
    """The `config` object, the same for both arms of a comparison (what differs between them is reported elsewhere:
    `collective` and `inner_repeats` on the GPU arm, `cpu_baseline.sample` on the CPU arm)."""
    return {"workload": WORKLOADS[workload] + (f" [SIZE OVERRIDE {size}: not the benchmark configuration]" if size else ""),
            "l2": "8 MiB working set, L2-resident by construction of the configuration" if workload == "c1" else "inputs larger than L2",
            "parallelism": f"rows/{world}" if workload in ("c3", "c4") else (f"units/{world}" if workload in ("c5", "causal") else f"chunks/{world}")}


def run_reference(args, rank: int) -> int:
    """The reference arm: the torch CPU evaluation of the workload on this box's host cores (rank 0 only). Each step is
    the whole workload when `steps + warmup` of them end within about four minutes, else a bounded sample, named."""
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    fn, work, scale, sample = cpu_reference_step(args.workload, threads)
    t0 = time.perf_counter()
    fn()
    t_sample = time.perf_counter() - t0
    if args.workload in ("c4", "c5"):
        full_work = 2.0 * 16384**3 if args.workload == "c4" else 4.0 * 256 * 4096 * 4096 * 128
        if t_sample * (full_work / work) * (args.steps + args.warmup + 1) < 240.0:
            fn, work, scale, sample = cpu_reference_step(args.workload, threads, full=True)
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = time.perf_counter() - t0
    value = work * args.steps / dt / scale
    unit = "TFLOP/s" if scale == 1e12 else "GB/s"
    cfg = config_for(args.workload, args.gpus, args.size)
    print(json.dumps({
        "impl": "reference", "metric": METRIC.get(args.workload, "gemm_tflops"), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": SCALING.get(args.workload, "strong"), "vs_baseline": None, "dtype": DTYPE.get(args.workload, "bf16"), "data": "synthetic",
        "config": cfg, "sample": sample,
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))
    return 0


# ---- main ---------------------------------------------------------------------------------------------------
MIN_REGION_S = 0.5


def agree(torch, dist, world, x: float) -> float:
    """The maximum of a host number over the ranks (so that every rank takes the same decision from it)."""
    if world == 1:
        return x
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def inner_repeats(torch, dist, world, fn, steps: int) -> int:
    """Passes per step such that `steps` steps last at least MIN_REGION_S, from a short probe; the same on every rank."""
    probe = timed(torch, dist, world, fn, 2, 1) / 2 * 1e-3
    return max(1, int(-(-MIN_REGION_S // max(probe * steps, 1e-9))))


NVLINK_GBS = 770.0     # measured peer-copy rate of this pool's B200s, per direction per GPU (900 nominal)


def fused_roofline(wl, world: int, ms_per_step: float, pk: dict):
    """The bound of a sharded step whose kernel also gathers its output: the slower of the rank's flops at the measured
    sustained tensor peak and the bytes every GPU must take in from its peers ((N-1)/N of the whole output) at the
    measured peer-copy rate. `frac` is that target over the measured step (kernel, gather and group barrier)."""
    if world <= 1 or not getattr(wl, "gather", False) or wl.bound != "tensor":
        return None
    out_bytes = (wl.m * wl.n if hasattr(wl, "m") else wl.units * wl.seq * wl.d) * 2
    cross = out_bytes * (world - 1) / world
    flops_ms = wl.kernel_work_per_launch() / (pk["bf16_tflops_sustained"] * 1e12) * 1e3
    link_ms = cross / (NVLINK_GBS * 1e9) * 1e3
    target = max(flops_ms, link_ms)
    return {"bound": "tensor" if flops_ms >= link_ms else "nvlink", "flops_ms": flops_ms, "link_ms": link_ms,
            "bytes_in_per_gpu": cross, "link_GBps": NVLINK_GBS, "target_ms": target, "frac": target / ms_per_step,
            "note": "a multicast store also comes back to its sender, so through the multicast mapping every GPU takes in the whole "
                    "output: a bare multicast copy of the shards on 8 GPUs takes in 715 GB/s per GPU"}


def roofline_block(wl, k_ms: float, pk: dict, pk_kind: str, traffic, clocks: dict) -> dict:
    if wl.bound == "tensor":
        achieved = wl.kernel_work_per_launch() / (k_ms * 1e-3) / 1e12
        sustained, burst = pk.get("bf16_tflops_sustained", pk["bf16_tflops"]), pk["bf16_tflops"]
        return {"bound": "tensor", "achieved": achieved, "peak": sustained, "unit": "TFLOP/s", "frac": achieved / sustained,
                "frac_sustained": achieved / sustained, "frac_burst": achieved / burst, "peak_burst": burst,
                "peak_source": f"{pk_kind} cuBLAS bf16: the sustained figure (the kernel is timed back to back for >= {MIN_REGION_S} s, under the power cap); frac_burst is against the burst figure",
                "sm_mhz_during": clocks.get("sm_mhz"), "traffic": traffic, "kernel_ms": k_ms}
    achieved = wl.kernel_work_per_launch() / (k_ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
            "peak_source": f"{pk_kind} copy bandwidth", "sm_mhz_during": clocks.get("sm_mhz"), "traffic": traffic, "kernel_ms": k_ms}


def measure(torch, dist, world, local_rank, wl, steps: int, warmup: int, pk, pk_kind, traffic) -> dict:
    """Times one workload: the step (max over ranks), the kernel alone (this rank), end to end from pinned host memory."""
    from emmyptx import runtime
    # a short run first (five launches after warm-up, boost clocks): the burst figure, reported beside the sustained one
    burst_ms = timed(torch, dist, 1, wl.kernel_only, 5, 3) / 5
    inner = inner_repeats(torch, dist, world, wl.step, steps)

    def passes(fn):
        def run():
            for _ in range(inner):
                fn()
        return run

    with ClockSampler(local_rank) as clocks:
        total_ms = timed(torch, dist, world, passes(wl.step), steps, warmup, finish=getattr(wl, "finish", None))
    # kernel-only time for the roofline: the same number of launches, after the timed region, on the launching stream
    with ClockSampler(local_rank) as k_clocks:
        k_ms = timed(torch, dist, 1, passes(wl.kernel_only), steps, warmup) / (steps * inner)
    graph_ms = None
    if k_ms < 0.02:         # a launch of a few microseconds: through the Python path the host's launch cost is what gets timed
        graph_ms = graph_timed(torch, wl.kernel_only, 50)
        k_ms = min(k_ms, graph_ms)
    status = runtime.device_status()
    ms_per_step = total_ms / (steps * inner)
    scale = 1e12 if wl.unit == "TFLOP/s" else 1e9
    try:
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
        parity = wl.parity()                      # of the result the passes above left behind
    except Exception as e:  # noqa: BLE001 - a failed check is reported, not hidden
        parity = {"ok": False, "error": f"{type(e).__name__}: {e}"[:300]}
    if world > 1:
        flag = torch.tensor([1.0 if parity.get("ok") else 0.0, -float(parity.get("worst_ratio", float("inf")))], device="cuda", dtype=torch.float64)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity["ok_on_every_rank"] = bool(flag[0].item() == 1.0)
        parity["worst_ratio_over_ranks"] = -float(flag[1].item())
        parity["ok"] = parity["ok_on_every_rank"]
    # end to end: pinned host inputs in, result out, through the Python API, every step
    h2d, d2h = wl.e2e_setup()
    e2e_steps = max(10, steps)
    e2e_ms = timed(torch, dist, world, wl.e2e_step, e2e_steps, 3) / e2e_steps
    return {"value": wl.work_per_step() / (ms_per_step * 1e-3) / scale, "ms_per_step": ms_per_step, "inner_repeats": inner,
            "timed_region_s": total_ms * 1e-3, "launches": steps * inner * wl.launches_per_step(),
            "roofline": dict(roofline_block(wl, k_ms, pk, pk_kind, traffic, k_clocks.summary()),
                             kernel_ms_burst=burst_ms, achieved_burst=wl.kernel_work_per_launch() / (burst_ms * 1e-3) / scale,
                             frac_burst_run_vs_burst_peak=(wl.kernel_work_per_launch() / (burst_ms * 1e-3) / scale / pk["bf16_tflops"]) if wl.bound == "tensor" else None,
                             timed_in_cuda_graph=graph_ms is not None),
            "clocks": clocks.summary(),
            "e2e": {"value": wl.work_per_step() / (e2e_ms * 1e-3) / scale, "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "warmup": 3,
                    "h2d_GBps_per_rank": h2d / max(world, 1) / (e2e_ms * 1e-3) / 1e9,
                    "limiter": (f"host link: {(h2d + d2h) / (e2e_ms * 1e-3) / 1e9:.0f} GB/s over all ranks, both directions, next to "
                                f"{ms_per_step:.3f} ms of device work per step") if e2e_ms > 1.3 * ms_per_step else "device work"},
            "fused_roofline": fused_roofline(wl, world, ms_per_step, pk),
            "parity": parity, "device_status": status}


def bind_to_gpu_cpus(torch, local_rank: int):
    """Run this rank on the CPUs next to its GPU (NVML's CPU affinity of the device, found by PCI address), so that the
    pinned host buffers it allocates and fills afterwards are first touched on that GPU's NUMA node: with several ranks
    copying at once, host memory on the wrong node is what the host link waits for. Only this process's affinity is set.
    Returns the CPU list, or None when NVML is not there, the mask is empty or EMMYB200_BENCH_AFFINITY=0."""
    if os.environ.get("EMMYB200_BENCH_AFFINITY", "1") == "0" or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        import pynvml
        pynvml.nvmlInit()
        p = torch.cuda.get_device_properties(local_rank)
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(f"{p.pci_domain_id:08x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0".encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1]
        allowed = set(os.sched_getaffinity(0))
        cpus = [c for c in cpus if c in allowed]
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return cpus
    except Exception:  # noqa: BLE001 - a missing NVML binding or an odd topology must not stop the bench
        return None


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=tuple(WORKLOADS), default="c4")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads and the CPU baseline")
    ap.add_argument("--size", type=int, default=None,
                    help="override the workload's extent (profiler captures on a small case); the line is marked")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cpus = bind_to_gpu_cpus(torch, local_rank) if world > 1 else None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from emmyptx import runtime
    runtime.library()

    wl = make_workload(args.workload, rank, world, dev, args.size)
    pk, pk_kind = peaks()
    traffic = None if (args.size or world > 1) else DRAM_TRAFFIC.get(args.workload)
    if args.no_extras and args.size:            # a profiler capture of a small case: one plain pass per step, nothing else
        ms = timed(torch, dist, world, wl.step, args.steps, args.warmup, finish=getattr(wl, "finish", None)) / args.steps
        if rank == 0:
            print(json.dumps({"metric": wl.metric, "ms_per_step": ms, "config": config_for(args.workload, world, args.size), "profiling_run": True}))
        if world > 1:
            dist.destroy_process_group()
        return 0
    m = measure(torch, dist, world, local_rank, wl, args.steps, args.warmup, pk, pk_kind, traffic)

    line = {
        "metric": wl.metric, "value": m["value"], "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m["ms_per_step"], "inner_repeats": m["inner_repeats"], "timed_region_s": m["timed_region_s"],
        "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": config_for(args.workload, world, args.size),
        "collective": "none" if world == 1 else getattr(wl, "collective", "nccl all_gather of the output shards"),
        "roofline": m["roofline"], "e2e": m["e2e"], "parity": m["parity"], "gpu_launches": m["launches"], "clocks": m["clocks"],
        "device_status": m["device_status"], "fused_roofline": m["fused_roofline"],
        "cpu_affinity": None if cpus is None else f"{len(cpus)} CPUs next to the GPU (rank 0: {cpus[0]}..{cpus[-1]})",
        "step_definition": f"one pass of the workload; the timed region is steps x inner_repeats = {args.steps * m['inner_repeats']} passes, "
                           "ms_per_step and value are per pass",
    }
    if world > 1 and args.workload == "c4" and not args.no_extras:
        # the other sharded configuration at this GPU count: unit-sharded attention with the gather fused into the kernel
        del wl
        torch.cuda.empty_cache()
        try:
            wl5 = make_workload("c5", rank, world, dev)
            m5 = measure(torch, dist, world, local_rank, wl5, max(5, args.steps // 2), 3, pk, pk_kind, None)
            line["other_workloads"] = {"c5": {"workload": WORKLOADS["c5"], "value": m5["value"], "unit": wl5.unit,
                                              "ms_per_step": m5["ms_per_step"], "kernel_ms": m5["roofline"]["kernel_ms"],
                                              "inner_repeats": m5["inner_repeats"], "collective": wl5.collective,
                                              "roofline": m5["roofline"], "fused_roofline": m5["fused_roofline"], "e2e": m5["e2e"], "parity": m5["parity"], "clocks": m5["clocks"],
                                              "config": config_for("c5", world)}}
            del wl5
        except Exception as e:  # noqa: BLE001 - must not hide the main line
            line["other_workloads"] = {"c5": {"error": f"{type(e).__name__}: {e}"[:300]}}

    if rank == 0 and world == 1 and not args.no_extras:
        threads = os.cpu_count() or 1
        fn, work, cscale, sample = cpu_reference_step(args.workload, threads)
        best = time_cpu(fn)
        line["cpu_baseline"] = {"value": work / best / cscale, "unit": wl.unit, "cores": threads, "kind": "reference",
                                "sample": sample}
        del fn
        line["other_workloads"] = other_workloads(torch, dist, dev, local_rank, pk, pk_kind, args.workload)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def other_workloads(torch, dist, dev, local_rank, pk, pk_kind, skip: str) -> dict:
    """The remaining configurations on one GPU, each measured like the main line (timed region of at least half a
    second, kernel-only roofline with the peak named, end to end from pinned host memory, parity of the result, the
    torch CPU baseline on this host's cores); kernels of a few microseconds are also timed inside a CUDA graph."""
    out = {}
    threads = os.cpu_count() or 1
    for name in ("c1", "c2", "c3", "c4", "c5"):
        if name == skip:
            continue
        try:
            wl = make_workload(name, 0, 1, dev)
            m = measure(torch, dist, 1, local_rank, wl, 5, 3, pk, pk_kind, DRAM_TRAFFIC.get(name))
            entry = {"workload": WORKLOADS[name], "value": m["value"], "unit": wl.unit, "ms": m["ms_per_step"], "inner_repeats": m["inner_repeats"],
                     "roofline": m["roofline"], "frac_of_peak": m["roofline"]["frac"], "peak_used": m["roofline"]["peak_source"],
                     "e2e": m["e2e"], "parity": m["parity"], "clocks": m["clocks"]}
            if wl.bound == "tensor":
                entry["frac_of_burst_peak"] = m["roofline"]["frac_burst"]
            if wl.bound == "tensor":
                entry["value_burst"] = m["roofline"]["achieved_burst"]
                entry["frac_of_burst_peak_in_a_burst_run"] = m["roofline"]["frac_burst_run_vs_burst_peak"]
            del wl
            torch.cuda.empty_cache()
            fn, work, cscale, sample = cpu_reference_step(name, threads)
            best = time_cpu(fn, budget_s=3.0)
            entry["cpu_baseline"] = {"value": work / best / cscale, "unit": entry["unit"], "cores": threads, "kind": "reference", "sample": sample}
            del fn
            out[name] = entry
        except Exception as e:  # noqa: BLE001 - a missing kernel must not hide the main line
            out[name] = {"workload": WORKLOADS[name], "error": f"{type(e).__name__}: {e}"[:200]}
    try:
        wl = PointwiseWorkload(2**28, 0, 1, dev)
        m = measure(torch, dist, 1, local_rank, wl, 5, 3, pk, pk_kind, None)
        out["c1_at_2^28"] = {"value": m["value"], "unit": "GB/s", "ms": m["ms_per_step"], "frac_of_peak": m["roofline"]["frac"],
                             "peak_used": m["roofline"]["peak_source"], "parity": m["parity"], "e2e": m["e2e"]}
        del wl
        torch.cuda.empty_cache()
    except Exception as e:  # noqa: BLE001
        out["c1_at_2^28"] = {"error": str(e)[:200]}
    # the reference's own kernels (its compiler's PTX, committed as text fixtures) JIT-loaded on this GPU and timed next to
    # ours on the same buffers: the two streaming configurations, and configuration 3 as the one-warp-per-cell mma.sync
    # kernel the stand-in IR compiles to (the tile sizes the reference's tracer would schedule are unknown: a floor).
    try:
        out["reference_ptx_on_this_gpu"] = reference_ptx_timings(torch, dist, dev)
    except Exception as e:  # noqa: BLE001
        out["reference_ptx_on_this_gpu"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    # the rows built after the five configurations: row kernels (256 MiB of fp32, larger than L2) and causal attention
    try:
        from emmyptx import runtime
        x = torch.randn(65536, 1024, device=dev)
        for op in ("sum", "softmax", "layer_norm"):
            y = runtime.rowwise(op, x)
            ms = timed(torch, dist, 1, lambda: runtime.rowwise(op, x, out=y), 5, 3) / 5
            byts = 4.0 * (x.numel() + y.numel())
            out[f"row_{op}_65536x1024"] = {"value": byts / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms": ms,
                                           "frac_of_peak": byts / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], "peak_used": f"{pk_kind} copy bandwidth"}
        del x, y
        for name in ("causal", "lerp", "transpose"):
            wl = make_workload(name, 0, 1, dev)
            m = measure(torch, dist, 1, local_rank, wl, 5, 3, pk, pk_kind, None)
            out[name] = {"workload": WORKLOADS[name], "value": m["value"], "unit": wl.unit, "ms": m["ms_per_step"], "roofline": m["roofline"],
                         "frac_of_peak": m["roofline"]["frac"], "peak_used": m["roofline"]["peak_source"], "parity": m["parity"], "e2e": m["e2e"]}
            if wl.bound == "tensor":
                out[name]["value_burst"] = m["roofline"]["achieved_burst"]
            del wl
            torch.cuda.empty_cache()
    except Exception as e:  # noqa: BLE001
        out["next_rows"] = {"error": str(e)[:200]}
    # convolutions written as scalar loops (tools/torch_cases/conv.py:6-7) through the indexed contraction: the
    # reference's own c_conv2d shape (launch-bound) and a 64-channel 3 x 3 layer over a 256 x 256 image
    try:
        from emmyptx import runtime
        for label, (c, o, h) in (("conv2d_8x32x32_k3", (8, 16, 32)), ("conv2d_64x256x256_k3", (64, 32, 256))):
            x, w = torch.randn(c, h, h, device=dev), torch.randn(o, c, 3, 3, device=dev)
            y = torch.zeros(o, h - 2, h - 2, device=dev)
            cm = {"extents": [o, h - 2, h - 2], "loops": [c, 3, 3], "a": {"offset": 0, "coef": [c * 9, 0, 0], "loop_coef": [9, 3, 1], "dtype": "f32"},
                  "b": {"offset": 0, "coef": [0, h, 1], "loop_coef": [h * h, h, 1], "dtype": "f32"},
                  "out": {"offset": 0, "coef": [(h - 2) ** 2, h - 2, 1], "dtype": "f32"}}
            run = lambda: runtime.contract_indexed(cm, w.reshape(-1), x.reshape(-1), y.reshape(-1))
            run()
            ref = torch.nn.functional.conv2d(x.double()[None], w.double())[0]
            ok = bool(torch.allclose(y.double(), ref, rtol=1e-3, atol=1e-3))
            reps = 200 if h <= 32 else 20
            ms = timed(torch, dist, 1, run, reps, 3) / reps
            flop = 2.0 * o * (h - 2) ** 2 * c * 9
            out[label] = {"value": flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ms, "kernel": "ct_kernel (CUDA cores, fp32 fused multiply-adds in loop order)",
                          "parity": {"ok": ok, "rule": "allclose(rtol=1e-3, atol=1e-3) against torch conv2d in float64"}}
            del x, w, y, ref
    except Exception as e:  # noqa: BLE001
        out["conv"] = {"error": str(e)[:200]}
    return out


def reference_ptx_timings(torch, dist, dev) -> dict:
    import json as _json
    from emmyptx import runtime
    from emmyptx.ptx_driver import PtxModule
    golden = ROOT / "tests" / "golden"
    manifest = _json.loads((golden / "reference_ptx_manifest.json").read_text())
    res = {}
    cases = [("c1_2^20", "c1_exp_sin_tanh_n1048576", torch.float32, lambda x, y: runtime.pointwise("exp_sin_tanh", x, out=y)),
             ("c1_2^28", "c1_exp_sin_tanh_n268435456", torch.float32, lambda x, y: runtime.pointwise("exp_sin_tanh", x, out=y)),
             ("c2_2^26", "c2_gather_n67108864", torch.int32, lambda x, y: runtime.index_gather(x, 7919, 13, 3, 2, trunc=True, out=y))]
    for label, case, dtype, ours in cases:
        info = manifest[case]
        n = info["tensors"]["x"]["shape"][0]
        x = (torch.rand(n, device=dev) * 8 - 4) if dtype == torch.float32 else torch.randint(-2**30, 2**30, (n,), device=dev, dtype=dtype)
        y_ref, y_ours = torch.zeros_like(x), torch.zeros_like(x)
        with PtxModule((golden / f"{case}.ref.ptx").read_text()) as m:
            fn = m.function(info["entry"])
            grid, block = info["launch"]["grid"][0], info["launch"]["block"][0]
            ptrs = [x.data_ptr(), y_ref.data_ptr()]
            ref = lambda: m.launch(fn, ptrs, grid, block, stream=torch.cuda.current_stream().cuda_stream)
            # kernels of a few microseconds: both sides inside a CUDA graph, so that neither host path is measured
            ms_ref = graph_timed(torch, ref, 50) if n <= 2**22 else timed(torch, dist, 1, ref, 5, 3) / 5
        ms_ours = graph_timed(torch, lambda: ours(x, y_ours), 50) if n <= 2**22 else timed(torch, dist, 1, lambda: ours(x, y_ours), 5, 3) / 5
        same = bool(torch.equal(y_ref, y_ours)) if dtype == torch.int32 else bool(torch.allclose(y_ref, y_ours, rtol=1e-5, atol=1e-5))
        res[label] = {"reference_kernel_ms": ms_ref, "this_library_ms": ms_ours, "speedup": ms_ref / ms_ours,
                      "reference_GBps": 8.0 * n / (ms_ref * 1e-3) / 1e9, "outputs_agree": same}
        del x, y_ref, y_ours
        torch.cuda.empty_cache()
    # configuration 3 through the reference's tensor-core lowering: one warp per m16n8k16 cell, fragments read from global
    # memory (emmyptx/mma.py:128-180). Two launches, the second timed.
    info = manifest["c3_f16_mm_4096"]
    g = info["gemm"]
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    a = (torch.randn(g["m"], g["k"], device=dev, generator=gen) / g["k"] ** 0.5).half()
    b = (torch.randn(g["k"], g["n"], device=dev, generator=gen) / g["k"] ** 0.5).half()
    c_ref, c_ours = torch.zeros(g["m"], g["n"], device=dev, dtype=torch.float16), torch.zeros(g["m"], g["n"], device=dev, dtype=torch.float16)
    with PtxModule((golden / "c3_f16_mm_4096.ref.ptx").read_text()) as m:
        fn = m.function(info["entry"])
        ptrs = [a.data_ptr(), b.data_ptr(), c_ref.data_ptr()]
        ref = lambda: m.launch(fn, ptrs, info["launch"]["grid"][0], info["launch"]["block"][0], stream=torch.cuda.current_stream().cuda_stream)
        ms_ref = timed(torch, dist, 1, ref, 1, 1)
    ms_ours = timed(torch, dist, 1, lambda: runtime.gemm(a, b, out=c_ours), 20, 3) / 20
    diff = (c_ref.float() - c_ours.float()).abs()
    res["c3_4096"] = {"reference_kernel_ms": ms_ref, "this_library_ms": ms_ours, "speedup": ms_ref / ms_ours,
                      "reference_TFLOPs": 2.0 * 4096**3 / (ms_ref * 1e-3) / 1e12,
                      "outputs_agree": bool((diff <= 2.0 ** -9 * c_ref.float().abs() + 1e-3).all()),
                      "outputs_identical_fraction": float((c_ref == c_ours).float().mean()),
                      "note": "the reference kernel is its lowering of the stand-in IR (one warp per 16x8 cell, no staging): "
                              "a floor for the reference, whose tracer's real schedule is not available"}
    return res


if __name__ == "__main__":
    sys.exit(main())
