"""Bus-bandwidth sweep: collective x size x algorithm, this library against NCCL (torch.distributed).

Run with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        mintccl_b200/benchmarks/sweep.py --size-lo 8 --size-hi 1G --out sweep.json

Sizes follow the nccl-tests convention (all-gather: total output bytes; reduce-scatter: total input
bytes).  Every number is the device time (CUDA events, warm-up first, one event pair around `iters`
back-to-back calls, maximum over ranks), taken `--repeats` times; the median is reported, with the fastest
and slowest repeat beside it.  Buffers are rotated through a pool larger than the L2 so that large-message
numbers are not served from cache.  `--memory ordinary` runs this library on plain `torch.empty` tensors
(shared with the peers through CUDA IPC on first use) instead of tensors of its symmetric heap; NCCL always
runs on plain tensors that are not registered with it.  The reference publishes no numbers
(README.md has none), so NCCL on the same box is the yardstick.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def parse_size(s: str) -> int:
    s = s.strip().upper()
    for suf, m in (("K", 1 << 10), ("M", 1 << 20), ("G", 1 << 30)):
        if s.endswith(suf):
            return int(float(s[:-1]) * m)
    return int(s)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size-lo", default="8")
    ap.add_argument("--size-hi", default="256M")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16", "fp32"])
    ap.add_argument("--collectives", default="allreduce,allgather,reducescatter,broadcast,reduce,alltoall")
    ap.add_argument("--impls", default="mintccl,nccl")
    ap.add_argument("--algos", default="auto", help="comma list for mintccl: auto,ring,direct,nvls,ll,oneshot")
    ap.add_argument("--iters", type=int, default=0, help="0 = by size")
    ap.add_argument("--ctas", default="", help="comma list of CTA / channel counts to try for mintccl (default: automatic)")
    ap.add_argument("--sync", action="store_true",
                    help="follow every call with an 8-byte all-reduce of this library (a cross-rank fence), so that "
                         "pipelined algorithms cannot overlap consecutive calls; the fence's own time is subtracted")
    ap.add_argument("--chain-steps", default="",
                    help="comma list of MINTCCL_CHAIN_STEP_BYTES values (0 = whole slots) to try for this library's "
                         "broadcast and reduce (they only matter for algo=ring over the Simple protocol)")
    ap.add_argument("--repeats", type=int, default=5, help="timed blocks per point; the median is reported")
    ap.add_argument("--size-mult", type=int, default=2, help="factor between consecutive sizes (2: every power of two)")
    ap.add_argument("--memory", default="heap", choices=["heap", "ordinary"],
                    help="where this library's buffers live: its symmetric heap, or ordinary torch tensors")
    ap.add_argument("--out", default="")
    a = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    gloo = dist.new_group(backend="gloo")

    import mintccl_b200
    from mintccl_b200 import Config
    from mintccl_b200.utils.busbw import busbw_factor

    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[a.dtype]
    esz = torch.empty((), dtype=dtype).element_size()
    lo, hi = parse_size(a.size_lo), parse_size(a.size_hi)
    pool_bytes = max(4 * hi, 512 << 20)
    comm = mintccl_b200.Communicator(group=gloo, config=Config.from_env(heap_bytes=2 * pool_bytes + (4 << 30)))
    n = world

    sizes = []
    s = lo
    while s <= hi:
        sizes.append(s)
        s *= max(2, a.size_mult)

    def maxr(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return float(t[0])

    spread = {}

    def timed(fn, iters):
        """Median over `--repeats` blocks of `iters` calls (ms per call, maximum over ranks per block)."""
        for _ in range(max(3, iters // 10)):
            fn()
        blocks = []
        for _ in range(max(1, a.repeats)):
            torch.cuda.synchronize()
            dist.barrier(group=gloo)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            blocks.append(maxr(e0.elapsed_time(e1) / iters))
        blocks.sort()
        spread["min"], spread["max"] = blocks[0], blocks[-1]
        return blocks[len(blocks) // 2]

    # rotating pools: inputs and outputs of successive calls do not sit in L2
    sym_in = comm.symm_empty(pool_bytes // esz, dtype)
    sym_out = comm.symm_empty(pool_bytes // esz, dtype)
    sym_in.normal_()
    if a.memory == "ordinary":
        own_in = torch.empty(pool_bytes // esz, device="cuda", dtype=dtype).normal_()
        own_out = torch.empty(pool_bytes // esz, device="cuda", dtype=dtype)
    else:
        own_in, own_out = sym_in, sym_out
    results = []
    state = {"k": 0}

    def make_views(nbytes):
        """Pre-sliced (input, output) pairs rotating through the pools, so that slicing costs nothing
        inside the timed loop and the launch plans of the communicator are reused."""
        per = max(nbytes, 256)
        cnt = max(1, min(64, pool_bytes // per))
        ne = per // esz
        k = max(1, nbytes // esz)
        return [(own_in[j * ne: j * ne + k], own_out[j * ne: j * ne + k]) for j in range(cnt)]

    fence_in = comm.symm_empty(4, torch.float16)
    fence_in.fill_(1.0)
    fence_out = torch.empty(4, device="cuda", dtype=torch.float16)
    fence = (lambda: comm.allreduce(fence_in, out=fence_out, algo="ll")) if (a.sync and n > 1) else None
    fence_ms = timed(fence, 200) if fence else 0.0

    for coll in a.collectives.split(","):
        for size in sizes:
            numel = max(1, size // esz)
            if coll in ("allgather", "reducescatter", "alltoall"):
                numel = max(n, numel // n * n)
            nbytes = numel * esz
            iters = a.iters or (200 if nbytes <= (1 << 20) else 50 if nbytes <= (64 << 20) else 10)
            for impl in a.impls.split(","):
                algos = a.algos.split(",") if impl == "mintccl" else ["nccl"]
                ctas_list = [int(x) for x in a.ctas.split(",")] if (a.ctas and impl == "mintccl") else [0]
                vlist = make_views(nbytes)
                if a.chain_steps:
                    os.environ.pop("MINTCCL_CHAIN_STEP_BYTES", None)  # no value left over from the previous combination
                steps_list = ([int(x) for x in a.chain_steps.split(",")]
                              if (a.chain_steps and impl == "mintccl" and coll in ("broadcast", "reduce")) else [None])
                for algo, ctas, chain_step in [(x, y, z) for x in algos for y in ctas_list for z in steps_list]:
                    if chain_step is not None:  # read by the native library at every call
                        os.environ["MINTCCL_CHAIN_STEP_BYTES"] = str(chain_step)

                    def call():
                        i, o = vlist[state["k"] % len(vlist)]
                        state["k"] += 1
                        if impl == "mintccl":
                            kw = {} if algo == "auto" else {"algo": algo}
                            if ctas:
                                kw["nch"] = ctas
                            if coll == "allreduce":
                                comm.allreduce(i, out=o, **kw)
                            elif coll == "allgather":
                                comm.allgather(o.view(n, -1), inp=i[: numel // n], **kw)
                            elif coll == "reducescatter":
                                comm.reducescatter(i.view(n, -1), out=o[: numel // n], **kw)
                            elif coll == "broadcast":
                                comm.broadcast(o, root=0, **kw)
                            elif coll == "reduce":
                                comm.reduce(i, root=0, out=o, **kw)
                            elif coll == "alltoall":
                                comm.alltoall(i.view(n, -1), o.view(n, -1), nch=kw.get("nch"),
                                              algo=algo if algo in ("bulk", "pull") else None)
                        else:
                            if coll == "allreduce":
                                dist.all_reduce(o)
                            elif coll == "allgather":
                                dist.all_gather_into_tensor(o, i[: numel // n])
                            elif coll == "reducescatter":
                                dist.reduce_scatter_tensor(o[: numel // n], i)
                            elif coll == "broadcast":
                                dist.broadcast(o, src=0)
                            elif coll == "reduce":
                                dist.reduce(o, dst=0)
                            elif coll == "alltoall":
                                dist.all_to_all_single(o, i)
                    try:
                        if fence:
                            def call_f(call=call):
                                call()
                                fence()
                            ms = max(timed(call_f, iters) - fence_ms, 1e-4)
                        else:
                            ms = timed(call, iters)
                        if impl == "mintccl":
                            comm.check()
                    except (ValueError, RuntimeError) as e:
                        from mintccl_b200.parallel.comm import CollectiveError
                        if isinstance(e, CollectiveError):
                            # a device-side wait gave up: the communicator is unusable from here on, and every
                            # further point would only wait out its time limit
                            print(f"# rank {rank}: {coll} {size} {impl}:{algo} failed on the device: {e}", file=sys.stderr, flush=True)
                            raise SystemExit(3)
                        if rank == 0:
                            print(f"# skip {coll} {size} {impl}:{algo}: {e}", file=sys.stderr)
                        continue
                    bus = busbw_factor(coll, n) * nbytes / (ms * 1e-3) / 1e9
                    row = {"collective": coll, "bytes": nbytes, "impl": impl, "algo": algo, "ctas": ctas, "us": round(ms * 1e3, 2),
                           "us_min": round(spread.get("min", ms) * 1e3, 2), "us_max": round(spread.get("max", ms) * 1e3, 2),
                           "repeats": a.repeats, "memory": a.memory if impl == "mintccl" else "ordinary, not registered",
                           "algbw_GBps": round(nbytes / (ms * 1e-3) / 1e9, 3), "busbw_GBps": round(bus, 3), "n": n,
                           "dtype": a.dtype, "sync": bool(fence)}
                    if chain_step is not None:
                        row["chain_step"] = chain_step
                    results.append(row)
                    if rank == 0:
                        print(json.dumps(row), flush=True)
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump({"nvls": bool(comm.nvls), "heap": comm.heap_kind, "rows": results}, f, indent=0)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
