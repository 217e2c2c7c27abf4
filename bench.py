#!/usr/bin/env python
"""Headline benchmark: bus bandwidth of the five collectives the baseline names (all-gather,
reduce-scatter, broadcast, reduce, all-reduce) on N GPUs of one node, plus the 8-byte all-reduce
latency.

A "step" runs the five collectives back to back on fp16 buffers of ``--size`` bytes (default 64 MiB, the
size of the baseline's broadcast/reduce configuration; sizes follow the nccl-tests convention, i.e. the
all-gather output and the reduce-scatter input are ``size`` bytes).  ``value`` is the job-wide aggregate
bus bandwidth: N x (sum over the five collectives of busbw_factor x size) / step time, with the
device-measured step time taken as the maximum over ranks.  On a single GPU the bus factors are zero,
so N = 1 reports the algorithmic bandwidth of the same kernels (local copies) instead and says so in
``note``; a collective that has nothing to do there (in-place broadcast) is left out.

Before anything is timed (N >= 2) every collective runs once on seeded inputs, on symmetric-heap tensors and
on ordinary ``torch.empty`` tensors, and is compared with the fp32 oracle that every rank can regenerate from
the seeds; a mismatch ends the run with a non-zero exit code.  NCCL (torch.distributed) is timed in the same
process on buffers of the same sizes.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# broadcast runs last: it is the only one that overwrites the step's input (in place, like the reference)
FIVE = ("allgather", "reducescatter", "reduce", "allreduce", "broadcast")
MINI_SWEEP = (8, 4 << 10, 256 << 10, 1 << 20, 16 << 20, 64 << 20, 256 << 20)
METRIC = ("aggregate bus GB/s over allgather+reducescatter+broadcast+reduce+allreduce "
          "(nccl-tests busbw; on one GPU: algorithmic GB/s of the local copies)")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--size", type=int, default=64 << 20, help="message bytes per collective")
    ap.add_argument("--impl", default="mintccl_b200", choices=["mintccl_b200", "reference", "nccl"])
    ap.add_argument("--min-seconds", type=float, default=0.6,
                    help="the block of --steps steps is repeated until this much device time is covered; the "
                         "median block is reported")
    ap.add_argument("--no-nccl", action="store_true", help="skip the in-process NCCL comparison")
    ap.add_argument("--no-sweep", action="store_true", help="skip the mini sweep over message sizes")
    return ap.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


_gloo = None
_nccl = None


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=_gloo)
    return float(t[0])


def all_true(x: bool, world: int) -> bool:
    return max_over_ranks(0.0 if x else 1.0, world) == 0.0


def host_barrier(world: int) -> None:
    if world > 1:
        import torch.distributed as dist
        dist.barrier(group=_gloo)


def gen(rank: int, numel: int) -> torch.Tensor:
    g = torch.Generator(device="cuda").manual_seed(rank)
    return torch.randn(numel, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)


class Work:
    """`nsets` sets of buffers and the five collective calls for one implementation and one kind of memory:
    kind "heap" (tensors of the library's symmetric heap), "ordinary" (torch.empty) or "nccl"."""

    def __init__(self, kind: str, comm, world: int, rank: int, size: int, nsets: int):
        self.kind, self.comm, self.world, self.rank = kind, comm, world, rank
        n = world
        self.shard = max(1, size // 2 // n)
        self.numel = self.shard * n
        self.size = self.numel * 2
        dev = torch.device("cuda", torch.cuda.current_device())
        if kind == "heap":
            alloc = lambda *shape: comm.symm_empty(shape, torch.float16)  # noqa: E731
        else:
            alloc = lambda *shape: torch.empty(shape, dtype=torch.float16, device=dev)  # noqa: E731
        self.sets = []
        for _ in range(nsets):
            s = {"src": alloc(self.numel), "ag": alloc(n, self.shard), "rs_out": alloc(self.shard),
                 "rd_out": alloc(self.numel), "ar_out": alloc(self.numel)}
            s["rs_in"] = s["src"].view(n, self.shard)
            if kind == "nccl":
                for t in s.values():
                    t.zero_()       # in-place sums of zeros stay finite however often they repeat
            else:
                s["src"].copy_(gen(rank, self.numel))
            self.sets.append(s)
        torch.cuda.synchronize()

    def free(self) -> None:
        if self.kind == "heap":
            for s in self.sets:
                for k in ("src", "ag", "rs_out", "rd_out", "ar_out"):
                    self.comm.symm_free(s[k])
        self.sets = []

    def run(self, name: str, k: int = 0) -> None:
        s = self.sets[k % len(self.sets)]
        if self.kind != "nccl":
            c = self.comm
            if name == "allgather":
                c.allgather(s["ag"], inp=s["src"][: self.shard])
            elif name == "reducescatter":
                c.reducescatter(s["rs_in"], out=s["rs_out"])
            elif name == "broadcast":
                c.broadcast(s["src"], root=0)
            elif name == "reduce":
                c.reduce(s["src"], root=0, out=s["rd_out"])
            elif name == "allreduce":
                c.allreduce(s["src"], out=s["ar_out"])
        else:  # NCCL through torch.distributed, in place where NCCL works in place: no extra copy is timed
            import torch.distributed as dist
            if name == "allgather":
                dist.all_gather_into_tensor(s["ag"].view(-1), s["src"][: self.shard], group=_nccl)
            elif name == "reducescatter":
                dist.reduce_scatter_tensor(s["rs_out"], s["src"], group=_nccl)
            elif name == "broadcast":
                dist.broadcast(s["src"], src=0, group=_nccl)
            elif name == "reduce":
                dist.reduce(s["rd_out"], dst=0, group=_nccl)
            elif name == "allreduce":
                dist.all_reduce(s["ar_out"], group=_nccl)

    def step(self, k: int = 0) -> None:
        for name in FIVE:
            self.run(name, k)

    def verify(self) -> dict:
        """Run every collective once on set 0 and compare with what the seeds say (this rank's view)."""
        from mintccl_b200.utils.check import sum_within_bound
        n, r, sh = self.world, self.rank, self.shard
        s = self.sets[0]
        for k in ("ag", "rs_out", "rd_out", "ar_out"):
            s[k].zero_()
        for name in FIVE[:-1]:
            self.run(name, 0)
        torch.cuda.synchronize()
        self.comm.check()
        srcs = [gen(q, self.numel) for q in range(n)]
        ok = {"allgather": bool(torch.equal(s["ag"], torch.stack([x[:sh] for x in srcs]))),
              # which algorithm runs is the library's choice (policy + shipped table): the NVLS variants can sit a
              # second rounding away, a chain or ring rounds into fp16 at each of its n - 1 combines.  A missing or
              # doubled contribution is orders of magnitude outside either bound.
              "reducescatter": sum_within_bound(s["rs_out"], [x[r * sh:(r + 1) * sh] for x in srcs], hops=max(2, n)),
              "allreduce": sum_within_bound(s["ar_out"], srcs, hops=max(2, n)),
              "reduce": r != 0 or sum_within_bound(s["rd_out"], srcs, hops=max(2, n))}
        self.run("broadcast", 0)
        torch.cuda.synchronize()
        self.comm.check()
        ok["broadcast"] = bool(torch.equal(s["src"], srcs[0]))
        s["src"].copy_(srcs[r])
        del srcs
        torch.cuda.synchronize()
        return {k: all_true(v, n) for k, v in ok.items()}


def time_region(fn, steps: int, world: int) -> float:
    """Device time of `steps` calls of fn in ms (this rank); barrier + synchronise on both sides."""
    torch.cuda.synchronize()
    host_barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    host_barrier(world)
    return e0.elapsed_time(e1)


def timed_blocks(fn, steps: int, world: int, min_seconds: float, max_blocks: int = 400):
    """Repeat the block of `steps` calls until `min_seconds` of device time are covered (at least 3 blocks); every
    block is bracketed by barrier + synchronise and its time is the maximum over ranks.  Returns the per-call ms
    of every block."""
    first = max_over_ranks(time_region(fn, steps, world), world)
    blocks = [first]
    want = min(max_blocks, max(3, int(math.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
    for _ in range(want - 1):
        blocks.append(max_over_ranks(time_region(fn, steps, world), world))
    return [b / steps for b in blocks]


def per_collective(w: Work, steps: int, world: int) -> dict:
    """Median of three blocks of `steps` calls per collective, rotating through the buffer sets so that no call
    finds its operands in the L2 left by the previous one."""
    out = {}
    for name in FIVE:
        ms = []
        for _ in range(3):
            ms.append(max_over_ranks(time_region(lambda i: w.run(name, i), steps, world) / steps, world))
        out[name] = statistics.median(ms)
    return out


def reference_arm(a) -> None:
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_runner  # noqa: WPS433
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/ref_runner.py not importable: {e}"}))
        return
    ref_runner.main(a)


def mini_sweep(comm, world: int, rank: int, with_nccl: bool) -> dict:
    """busbw (GB/s) of every collective at a fixed list of sizes, this library (heap tensors, automatic
    algorithm) and NCCL; median of three event-timed blocks.  Small sizes are latency numbers: the calls of a
    block follow each other on the same buffers."""
    from mintccl_b200.utils.busbw import busbw_factor
    out = {}
    kinds = ["heap"] + (["nccl"] if with_nccl else [])
    for size in MINI_SWEEP:
        iters = 50 if size <= (1 << 20) else (20 if size <= (16 << 20) else (10 if size <= (64 << 20) else 5))
        row = {}
        for kind in kinds:
            w = Work(kind, comm, world, rank, max(size, 2 * world), 2 if size >= (16 << 20) else 1)
            for name in FIVE:
                w.run(name, 0)
            res = {}
            for name in FIVE:
                ms = []
                for _ in range(3):
                    ms.append(max_over_ranks(time_region(lambda i: w.run(name, i), iters, world) / iters, world))
                t = statistics.median(ms)
                res[name] = {"us": round(t * 1e3, 2),
                             "busbw_GBps": round(busbw_factor(name, world) * w.size / (t * 1e-3) / 1e9, 3)}
            row["mintccl_b200" if kind == "heap" else "nccl"] = res
            if kind == "heap":
                comm.check()
            w.free()
            del w
        out[str(size)] = row
    return out


def main() -> None:
    global _gloo, _nccl
    a = parse()
    if a.impl == "reference":
        reference_arm(a)
        return
    rank, world, local = dist_env()
    if world != a.gpus and world == 1 and a.gpus > 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    nccl_note = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        _gloo = dist.group.WORLD
        if a.impl == "nccl" or not a.no_nccl:
            try:
                _nccl = dist.new_group(backend="nccl")
                t = torch.zeros(8, device="cuda")
                dist.all_reduce(t, group=_nccl)
                torch.cuda.synchronize()
            except Exception as e:  # noqa: BLE001
                _nccl, nccl_note = None, f"NCCL group not available: {type(e).__name__}: {e}"
                if a.impl == "nccl":
                    raise
    from mintccl_b200 import _native
    from mintccl_b200.utils.busbw import busbw_factor
    from mintccl_b200.utils.clocks import ClockSampler

    steps, warmup = a.steps, max(3, a.warmup)
    sampler = ClockSampler(local).start() if rank == 0 else None
    comm = None
    if a.impl == "mintccl_b200":
        import mintccl_b200
        from mintccl_b200 import Config
        heap = (4 << 30) + 3 * 5 * a.size + 3 * (256 << 20) * 5
        comm = mintccl_b200.Communicator(config=Config.from_env(heap_bytes=heap))
    nsets = 3
    w = Work("heap" if comm else "nccl", comm, world, rank, a.size, nsets)
    size = w.size

    def factor(name):
        return busbw_factor(name, world) if world > 1 else 1.0

    # a one-rank communicator has nothing to do for an in-place broadcast: leave it out of the byte count
    moving = [n_ for n_ in FIVE if not (world == 1 and n_ == "broadcast")]
    bus_bytes = sum(factor(n_) * size for n_ in moving)

    # ---- self-check on seeded inputs, symmetric-heap and ordinary tensors -----------------------------------
    verified = verified_ordinary = None
    wo = None
    if comm is not None:
        verified = w.verify()
        wo = Work("ordinary", comm, world, rank, a.size, 2)
        verified_ordinary = wo.verify()
        if not (all(verified.values()) and all(verified_ordinary.values())):
            if rank == 0:
                print(json.dumps({"metric": METRIC, "impl": a.impl, "n_gpus": world, "verified": verified,
                                  "verified_ordinary": verified_ordinary,
                                  "error": "a collective's result does not match the fp32 oracle"}), flush=True)
            raise SystemExit(1)

    for i in range(warmup):
        w.step(i)
    if comm:
        comm.check()

    # ---- per-collective device times (max over ranks, median of 3 blocks, rotating buffer sets) ------------
    per = per_collective(w, steps, world)
    per_ord = per_nccl = None
    if wo is not None and world > 1:
        for i in range(warmup):
            wo.step(i)
        per_ord = per_collective(wo, steps, world)
        comm.check()
    wn = None
    if comm is not None and _nccl is not None:
        wn = Work("nccl", None, world, rank, a.size, nsets)
        for i in range(warmup):
            wn.step(i)
        per_nccl = per_collective(wn, steps, world)

    # ---- the headline: blocks of K whole steps, median block ---------------------------------------------
    for i in range(warmup):
        w.step(i)
    if comm:
        _native.lib().mt_reset_launch_count()
    if sampler:
        sampler.mark_begin()
    blocks = timed_blocks(w.step, steps, world, a.min_seconds)
    if sampler:
        sampler.mark_end()
    launches = int(_native.lib().mt_launch_count()) // len(blocks) if comm else 0
    ms_step = statistics.median(blocks)
    clocks = sampler.stop() if sampler else None
    if comm:
        comm.check()
    value = world * bus_bytes / (ms_step * 1e-3) / 1e9
    nccl_step_ms = None
    if wn is not None:
        nccl_step_ms = statistics.median(timed_blocks(wn.step, steps, world, min(a.min_seconds, 0.3)))

    # ---- end to end: every step copies the step's input from pinned host memory into the device buffer the
    # collectives read, runs the five collectives through the public API and reads a result back -------------
    host_in = torch.empty(w.numel, dtype=torch.float16).pin_memory()
    host_in.copy_(torch.randn(w.numel, dtype=torch.float32).to(torch.float16))
    host_out = torch.empty(2048, dtype=torch.float16).pin_memory()

    def e2e_step(i):
        s = w.sets[i % nsets]
        s["src"].copy_(host_in, non_blocking=True)
        w.step(i)
        host_out.copy_(s["ar_out"][:2048], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    host_barrier(world)
    t0 = time.perf_counter()
    e2e_blocks = [max_over_ranks(time_region(e2e_step, steps, world), world) / steps for _ in range(3)]
    wall = (time.perf_counter() - t0) * 1e3 / (3 * steps)
    ms_e2e = statistics.median(e2e_blocks)
    e2e_value = world * bus_bytes / (ms_e2e * 1e-3) / 1e9

    # ---- 8-byte all-reduce latency (1000 back-to-back device-timed calls) ---------------------------------
    lat_us = lat_graph_us = lat_nccl_us = None
    if world > 1:
        small_in = comm.symm_empty(4, torch.float16) if comm else torch.ones(4, dtype=torch.float16, device="cuda")
        small_out = torch.empty(4, dtype=torch.float16, device="cuda")
        small_in.fill_(1.0)

        def small(_i=0):
            if comm:
                comm.allreduce(small_in, out=small_out)
            else:
                import torch.distributed as dist
                dist.all_reduce(small_in, group=_nccl)

        for _ in range(20):
            small()
        lat_us = max_over_ranks(time_region(small, 1000, world), world)  # 1000 calls: ms total == us per call
        if comm and _nccl is not None:
            import torch.distributed as dist
            z = torch.zeros(4, dtype=torch.float16, device="cuda")
            for _ in range(20):
                dist.all_reduce(z, group=_nccl)
            lat_nccl_us = max_over_ranks(time_region(lambda _i: dist.all_reduce(z, group=_nccl), 1000, world), world)
        # the same calls replayed from a CUDA graph: device-side latency without the host's launch cost
        if comm:
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
                lat_graph_us = max_over_ranks(time_region(lambda _i: gr.replay(), 10, world), world)  # 10 x 100 calls
            except Exception as e:  # noqa: BLE001
                lat_graph_us = None
                print(f"# graph latency skipped: {type(e).__name__}: {e}", file=sys.stderr)
        if comm:
            comm.check()

    sweep = None
    if comm is not None and world > 1 and not a.no_sweep:
        sweep = mini_sweep(comm, world, rank, _nccl is not None)

    if rank == 0:
        def table(p):
            return None if p is None else {n_: (round(factor(n_) * size / (p[n_] * 1e-3) / 1e9, 2) if n_ in moving else None)
                                           for n_ in FIVE}

        def ratio(x, y):
            return None if x is None or y is None else {n_: (round(x[n_] / y[n_], 3) if x[n_] and y[n_] else None) for n_ in FIVE}

        busbw, busbw_ord, busbw_nccl = table(per), table(per_ord), table(per_nccl)
        out = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic (randn, seed = rank)", "impl": a.impl,
            "config": {"model": "five collectives (AG, RS, bcast, reduce, AR)", "message_bytes": size,
                       "global_batch": None, "seq_len": None, "parallelism": f"collective x{world}",
                       "memory": "tensors of the library's symmetric heap (headline); ordinary torch.empty tensors in "
                                 "ordinary_busbw_GBps; NCCL on ordinary tensors, not registered with NCCL",
                       "timing": f"{len(blocks)} blocks of {steps} steps, each bracketed by barrier + synchronize, "
                                 "CUDA events, maximum over ranks; the median block is reported",
                       "l2": f"three buffer sets used in rotation: consecutive steps touch {3 * 4.1 * size / 1e6:.0f} MB, "
                             "more than the 126 MB L2"},
            "note": None if world > 1 else "one GPU: no bus; the collectives are local copies (an in-place broadcast has "
                                           "nothing to do and is left out), value = algorithmic bytes / time",
            "busbw_GBps": busbw, "ms": {k: round(v, 4) for k, v in per.items()},
            "ordinary_busbw_GBps": busbw_ord,
            "nccl_busbw_GBps": busbw_nccl, "nccl_ms": None if per_nccl is None else {k: round(v, 4) for k, v in per_nccl.items()},
            "vs_nccl": ratio(busbw, busbw_nccl), "ordinary_vs_nccl": ratio(busbw_ord, busbw_nccl),
            "nccl_ms_per_step": None if nccl_step_ms is None else round(nccl_step_ms, 4),
            "step_vs_nccl": None if nccl_step_ms is None else round(nccl_step_ms / ms_step, 3),
            "nccl_note": nccl_note,
            "verified": verified, "verified_ordinary": verified_ordinary,
            "latency_8B_us": None if lat_us is None else round(lat_us, 2),
            "latency_8B_graph_us": None if lat_graph_us is None else round(lat_graph_us, 2),
            "latency_8B_nccl_us": None if lat_nccl_us is None else round(lat_nccl_us, 2),
            "busbw_by_size": sweep,
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": size,
                    "d2h_bytes_per_step": 4096, "ms_per_step": round(ms_e2e, 4), "wall_ms_per_step": round(wall, 4)},
            "gpu_launches": launches, "clocks": clocks,
            "algos": None if comm is None else {"nvls": bool(comm.nvls), "heap": comm.heap_kind,
                                                "shared_allocations": len(comm._segs)},
        }
        print(json.dumps(out), flush=True)
    if comm is not None:
        comm.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
