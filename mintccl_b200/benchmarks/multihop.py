"""Multi-hop send/recv benchmark: one rank sends to a rank that is several ring positions away, through the
FIFOs of the ranks in between (store and forward; the jump hosts' user memory is never touched).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        mintccl_b200/benchmarks/multihop.py --hops 4 --size-lo 4K --size-hi 256M --out multihop.json

The route is ring positions 0, 1, ..., `--hops` of the communicator's ring; ``--ring-seed`` fixes the ring as the
seeded permutation of the ranks (``MINTCCL_RING_SEED``), the default ring is 0, 1, ..., n - 1, i.e. rank 0 to
rank 4 through 1, 2 and 3.  For every payload size and both protocols (LL128, Simple) it reports the latency
of one transfer (device time from CUDA events, maximum over the ranks of the route, median of ``--repeats``
blocks) and the bandwidth, checks the received bytes against the sent ones, and ends with back-to-back runs of
1,000 transfers at 4 KiB and at 16 MiB.  The workload of the reference's 2_sendrecv_indirect.py:44-167 and
3_sendrecv_buffer.py:23-151, whose route is hard-coded to [0, 1].
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
    ap.add_argument("--hops", type=int, default=4)
    ap.add_argument("--size-lo", default="4K")
    ap.add_argument("--size-hi", default="256M")
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--ring-seed", type=int, default=None)
    ap.add_argument("--protos", default="ll128,simple")
    ap.add_argument("--out", default="")
    a = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if a.ring_seed is not None:
        os.environ["MINTCCL_RING_SEED"] = str(a.ring_seed)
    import mintccl_b200
    from mintccl_b200 import Config
    comm = mintccl_b200.Communicator(config=Config.from_env(heap_bytes=4 << 30))
    hops = min(a.hops, world - 1)
    route = [comm.ring[i] for i in range(hops + 1)]
    src_rank, dst_rank = route[0], route[-1]
    on_route = rank in route

    def maxr(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    lo, hi = parse_size(a.size_lo), parse_size(a.size_hi)
    g = torch.Generator(device="cuda").manual_seed(0)
    payload = torch.randn(hi // 2, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
    recv = torch.zeros(hi // 2, device="cuda", dtype=torch.float16) if rank == dst_rank else None
    rows = []

    def transfer(nbytes, proto):
        comm.sendrecv_route(route, payload[: nbytes // 2] if rank == src_rank else None,
                            recv[: nbytes // 2] if rank == dst_rank else None, nbytes=nbytes, proto=proto)

    def timed(nbytes, proto, iters):
        for _ in range(3):
            transfer(nbytes, proto)
        blocks = []
        for _ in range(a.repeats):
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                transfer(nbytes, proto)
            e1.record()
            torch.cuda.synchronize()
            blocks.append(maxr(e0.elapsed_time(e1) / iters if on_route else 0.0))
        blocks.sort()
        return blocks[len(blocks) // 2], blocks[0], blocks[-1]

    size = lo
    while size <= hi:
        for proto in a.protos.split(","):
            if recv is not None:
                recv[: size // 2].zero_()
            iters = 100 if size <= (1 << 20) else (20 if size <= (32 << 20) else 5)
            ms, ms_min, ms_max = timed(size, proto, iters)
            comm.check()
            ok = True
            if rank == dst_rank:
                ok = bool(torch.equal(recv[: size // 2], payload[: size // 2]))
            ok = maxr(0.0 if ok else 1.0) == 0.0
            row = {"route": route, "hops": hops, "bytes": size, "proto": proto, "us": round(ms * 1e3, 2),
                   "us_min": round(ms_min * 1e3, 2), "us_max": round(ms_max * 1e3, 2),
                   "GBps": round(size / (ms * 1e-3) / 1e9, 3), "bit_exact": ok, "iters": iters, "repeats": a.repeats,
                   "pipelined": "calls of a block follow each other back to back: us is the time per transfer in a "
                                "stream of transfers, GBps the sustained rate"}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            if not ok:
                raise SystemExit(f"received bytes differ from the sent ones at {size} bytes ({proto})")
        size *= 4 if size < (1 << 20) else 2
    # one transfer at a time: every call is followed by a device synchronisation on every rank and a host barrier
    for nbytes in (4 << 10, 1 << 20):
        for proto in a.protos.split(","):
            ts = []
            for _ in range(20):
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                transfer(nbytes, proto)
                e1.record()
                torch.cuda.synchronize()
                ts.append(maxr(e0.elapsed_time(e1) if on_route else 0.0))
            ts.sort()
            row = {"route": route, "bytes": nbytes, "proto": proto, "single_transfer_us": round(ts[len(ts) // 2] * 1e3, 2)}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    # 1,000 transfers back to back: no deadlock, flags never repeat, the last payload arrives intact
    for nbytes, proto in ((4 << 10, "ll128"), (16 << 20, "simple"), (16 << 20, "ll128")):
        if recv is not None:
            recv[: nbytes // 2].zero_()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(1000):
            transfer(nbytes, proto)
        e1.record()
        torch.cuda.synchronize()
        comm.check()
        ms = maxr(e0.elapsed_time(e1) if on_route else 0.0)
        ok = rank != dst_rank or bool(torch.equal(recv[: nbytes // 2], payload[: nbytes // 2]))
        ok = maxr(0.0 if ok else 1.0) == 0.0
        row = {"route": route, "bytes": nbytes, "proto": proto, "back_to_back": 1000, "total_ms": round(ms, 2),
               "us_per_transfer": round(ms, 2), "GBps": round(nbytes * 1000 / (ms * 1e-3) / 1e9, 3), "bit_exact": ok}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        if not ok:
            raise SystemExit("payload corrupted in the back-to-back run")
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump({"route": route, "ring": comm.ring, "rows": rows}, f, indent=0)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
