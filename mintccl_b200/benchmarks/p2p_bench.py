"""Point-to-point copy between two GPUs: bandwidth against the number of CTAs, for each way of moving the payload
("sys": 16-byte system-scope loads / stores from every thread; "weak": volatile loads, weak stores; "bulk": the
copy engine, cp.async.bulk staged in shared memory) and both directions of control (the receiver pulls, the
sender pushes).  Shows how many SMs a one-hop kernel needs to fill the link, which is what the CTA counts of the
collectives are derived from.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        mintccl_b200/benchmarks/p2p_bench.py --mib 256 --out p2p.json

Device time from CUDA events around `--iters` back-to-back copies, maximum over the two ranks, median of
`--repeats` blocks.  The workload of the reference's 1_sendrecv_direct.py:31-79 (receiver pull, 16 CTAs).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--ctas", default="2,4,8,16,32,64,128")
    ap.add_argument("--modes", default="sys,weak,bulk")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import mintccl_b200
    from mintccl_b200 import Config
    nbytes = a.mib << 20
    comm = mintccl_b200.Communicator(config=Config.from_env(heap_bytes=(4 << 30) + 2 * nbytes))
    buf = comm.symm_empty(nbytes // 4, torch.float32)
    want = torch.arange(nbytes // 4, device="cuda", dtype=torch.float32)
    src, dst = 0, world - 1

    def maxr(x):
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    rows = []
    for mode in a.modes.split(","):
        for pull in (True, False):
            for nctas in [int(x) for x in a.ctas.split(",")]:
                buf.copy_(want if rank == src else torch.zeros_like(want))
                torch.cuda.synchronize()
                dist.barrier()
                for _ in range(2):
                    comm.sendrecv_direct(src, dst, buf, pull=pull, nctas=nctas, mode=mode)
                blocks = []
                for _ in range(a.repeats):
                    torch.cuda.synchronize()
                    dist.barrier()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(a.iters):
                        comm.sendrecv_direct(src, dst, buf, pull=pull, nctas=nctas, mode=mode)
                    e1.record()
                    torch.cuda.synchronize()
                    blocks.append(maxr(e0.elapsed_time(e1) / a.iters))
                comm.check()
                ok = rank != dst or bool(torch.equal(buf, want))
                ok = maxr(0.0 if ok else 1.0) == 0.0
                blocks.sort()
                ms = blocks[len(blocks) // 2]
                row = {"mode": mode, "pull": pull, "ctas": nctas, "bytes": nbytes, "us": round(ms * 1e3, 1),
                       "GBps": round(nbytes / (ms * 1e-3) / 1e9, 1), "GBps_per_cta": round(nbytes / (ms * 1e-3) / 1e9 / nctas, 2),
                       "bit_exact": ok}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump({"rows": rows}, f, indent=0)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
