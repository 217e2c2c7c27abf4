#!/usr/bin/env python
"""Headline benchmark: bus bandwidth of the five collectives the baseline names (all-gather,
reduce-scatter, broadcast, reduce, all-reduce) on N GPUs of one node, plus the 8-byte all-reduce
latency.

A "step" runs the five collectives back to back on fp16 buffers of ``--size`` bytes (default 64 MiB, the
size of the baseline's broadcast/reduce configuration; sizes follow the nccl-tests convention, i.e. the
all-gather output and the reduce-scatter input are ``size`` bytes).  ``value`` is the job-wide aggregate
bus bandwidth: N x (sum over the five collectives of busbw_factor x size) / step time, with the
device-measured step time taken as the maximum over ranks.  On a single GPU the bus factors are zero,
so N = 1 reports the algorithmic bandwidth of the same kernels (local copies) instead and says so.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# broadcast runs last: it is the only one that overwrites the step's input (in place, like the reference)
FIVE = ("allgather", "reducescatter", "reduce", "allreduce", "broadcast")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--size", type=int, default=64 << 20, help="message bytes per collective")
    ap.add_argument("--impl", default="mintccl_b200", choices=["mintccl_b200", "reference", "nccl"])
    ap.add_argument("--sweep", action="store_true", help="also print a size sweep table to stderr")
    return ap.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=_gloo_group())
    return float(t[0])


_gg = None


def _gloo_group():
    global _gg
    import torch.distributed as dist
    if _gg is None:
        _gg = dist.new_group(backend="gloo") if "gloo" not in str(dist.get_backend()) else dist.group.WORLD
    return _gg


def host_barrier(world: int) -> None:
    if world > 1:
        import torch.distributed as dist
        dist.barrier(group=_gloo_group())


class Work:
    """Buffers and the five collective calls for one implementation."""

    def __init__(self, impl: str, world: int, rank: int, size: int):
        self.impl, self.world, self.rank, self.size = impl, world, rank, size
        n = world
        self.numel = size // 2
        self.shard = self.numel // n
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev).manual_seed(rank)
        if impl == "mintccl_b200":
            import mintccl_b200
            from mintccl_b200 import Config
            heap = 8 * size + (4 << 30)
            self.comm = mintccl_b200.Communicator(config=Config.from_env(heap_bytes=heap))
            alloc = lambda *shape: self.comm.symm_empty(shape, torch.float16)  # noqa: E731
        else:
            self.comm = None
            alloc = lambda *shape: torch.empty(shape, dtype=torch.float16, device=dev)  # noqa: E731
        self.src = alloc(self.numel)           # the step's input (filled from the host in the e2e loop)
        self.src.copy_(torch.randn(self.numel, generator=g, device=dev, dtype=torch.float32).to(torch.float16))
        self.ag = alloc(n, self.shard)         # all-gather output
        self.rs_in = self.src[: n * self.shard].view(n, self.shard)
        self.rs_out = alloc(self.shard)
        self.rd_out = alloc(self.numel)
        self.ar_out = alloc(self.numel)
        torch.cuda.synchronize()

    def run(self, name: str) -> None:
        n, r = self.world, self.rank
        if self.impl == "mintccl_b200":
            c = self.comm
            if name == "allgather":
                c.allgather(self.ag, inp=self.src[: self.shard])
            elif name == "reducescatter":
                c.reducescatter(self.rs_in, out=self.rs_out)
            elif name == "broadcast":
                c.broadcast(self.src, root=0)
            elif name == "reduce":
                c.reduce(self.src, root=0, out=self.rd_out)
            elif name == "allreduce":
                c.allreduce(self.src, out=self.ar_out)
        else:  # NCCL through torch.distributed
            import torch.distributed as dist
            if name == "allgather":
                dist.all_gather_into_tensor(self.ag.view(-1), self.src[: self.shard])
            elif name == "reducescatter":
                dist.reduce_scatter_tensor(self.rs_out, self.rs_in.view(-1))
            elif name == "broadcast":
                dist.broadcast(self.src, src=0)
            elif name == "reduce":
                self.rd_out.copy_(self.src)
                dist.reduce(self.rd_out, dst=0)
            elif name == "allreduce":
                self.ar_out.copy_(self.src)
                dist.all_reduce(self.ar_out)

    def step(self) -> None:
        for name in FIVE:
            self.run(name)

    def check(self) -> None:
        if self.comm is not None:
            self.comm.check()


def time_region(fn, steps: int, world: int) -> float:
    """Device time of `steps` calls of fn in ms (this rank); barrier + synchronise on both sides."""
    torch.cuda.synchronize()
    host_barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    host_barrier(world)
    return e0.elapsed_time(e1)


def reference_arm(a) -> None:
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_runner  # noqa: WPS433
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/ref_runner.py not importable: {e}"}))
        return
    ref_runner.main(a)


def main() -> None:
    a = parse()
    if a.impl == "reference":
        reference_arm(a)
        return
    rank, world, local = dist_env()
    if world != a.gpus and world == 1 and a.gpus > 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if a.impl == "nccl" else "gloo", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local) if a.impl == "nccl" else None)
    from mintccl_b200 import _native
    from mintccl_b200.utils.busbw import busbw_factor
    from mintccl_b200.utils.clocks import ClockSampler

    sampler = ClockSampler(local).start() if rank == 0 else None
    w = Work(a.impl, world, rank, a.size)
    size = w.numel * 2
    for _ in range(max(3, a.warmup)):
        w.step()
    w.check()

    # per-collective device times (max over ranks); inputs and outputs (about 4 x message_bytes) exceed the 126 MB L2
    per = {}
    for name in FIVE:
        ms = time_region(lambda: w.run(name), a.steps, world) / a.steps
        per[name] = max_over_ranks(ms, world)

    # the headline: K whole steps
    if a.impl == "mintccl_b200":
        _native.lib().mt_reset_launch_count()
    if sampler:
        sampler.mark_begin()
    ms_total = time_region(w.step, a.steps, world)
    if sampler:
        sampler.mark_end()
    launches = int(_native.lib().mt_launch_count()) if a.impl == "mintccl_b200" else 0
    ms_step = max_over_ranks(ms_total / a.steps, world)
    clocks = sampler.stop() if sampler else None
    w.check()

    def factor(name):
        return busbw_factor(name, world) if world > 1 else 1.0

    bus_bytes = sum(factor(n_) * size for n_ in FIVE)
    value = world * bus_bytes / (ms_step * 1e-3) / 1e9

    # end to end: every step copies the step's input from pinned host memory into the device buffers the
    # collectives read, runs the five collectives through the public API and reads a result back
    host_in = torch.empty(w.numel, dtype=torch.float16).pin_memory()
    host_in.copy_(torch.randn(w.numel, dtype=torch.float32).to(torch.float16))
    host_out = torch.empty(2048, dtype=torch.float16).pin_memory()

    def e2e_step():
        w.src.copy_(host_in, non_blocking=True)
        w.step()
        host_out.copy_(w.ar_out[:2048], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    host_barrier(world)
    t0 = time.perf_counter()
    ms_e2e_dev = time_region(e2e_step, a.steps, world)
    wall = (time.perf_counter() - t0) * 1e3
    ms_e2e = max_over_ranks(max(ms_e2e_dev, 0.0) / a.steps, world)
    e2e_value = world * bus_bytes / (ms_e2e * 1e-3) / 1e9

    # 8-byte all-reduce latency (median of 1000 back-to-back device-timed calls)
    lat_us = lat_graph_us = None
    if world > 1:
        small_in = (w.comm.symm_empty(4, torch.float16) if w.comm else torch.ones(4, dtype=torch.float16, device="cuda"))
        small_out = torch.empty(4, dtype=torch.float16, device="cuda")
        small_in.fill_(1.0)

        def small():
            if w.comm:
                w.comm.allreduce(small_in, out=small_out)
            else:
                import torch.distributed as dist
                dist.all_reduce(small_in)

        for _ in range(20):
            small()
        lat_us = max_over_ranks(time_region(small, 1000, world), world)  # 1000 calls: ms total == us per call
        # the same 1000 calls replayed from a CUDA graph: device-side latency without the host's launch cost
        try:
            gr = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(gr, stream=side):
                    for _ in range(100):
                        small()
            torch.cuda.current_stream().wait_stream(side)
            gr.replay()
            lat_graph_us = max_over_ranks(time_region(gr.replay, 10, world), world)  # 10 x 100 calls
        except Exception as e:  # noqa: BLE001
            lat_graph_us = None
            print(f"# graph latency skipped: {type(e).__name__}: {e}", file=sys.stderr)
    w.check()

    if rank == 0:
        busbw = {n_: round(factor(n_) * size / (per[n_] * 1e-3) / 1e9, 2) for n_ in FIVE}
        out = {
            "metric": "aggregate bus GB/s over allgather+reducescatter+broadcast+reduce+allreduce"
                      if world > 1 else "aggregate algorithmic GB/s of the five collectives on one GPU (no bus)",
            "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": a.steps, "warmup": max(3, a.warmup),
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic (randn, seed = rank)", "impl": a.impl,
            "config": {"model": "five collectives (AG, RS, bcast, reduce, AR)", "message_bytes": size,
                       "global_batch": None, "seq_len": None, "parallelism": f"collective x{world}",
                       "l2": "buffers touched per step are about 4.1 x message_bytes (268 MB at the default), larger than the 126 MB L2"},
            "busbw_GBps": busbw, "ms": {k: round(v, 4) for k, v in per.items()},
            "latency_8B_us": None if lat_us is None else round(lat_us, 2),
            "latency_8B_graph_us": None if lat_graph_us is None else round(lat_graph_us, 2),
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": size,
                    "d2h_bytes_per_step": 4096, "ms_per_step": round(ms_e2e, 4), "wall_ms_per_step": round(wall / a.steps, 4)},
            "gpu_launches": launches, "clocks": clocks,
            "algos": None if w.comm is None else {"nvls": bool(w.comm.nvls), "heap": w.comm.heap_kind},
        }
        print(json.dumps(out), flush=True)
    if w.comm is not None:
        w.comm.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
