"""Runs ONE collective kernel a few times on an emulated world (several ranks on one GPU, one cooperative
launch per call), sized for a profiler capture: messages of a few MiB to 16 MiB per rank, a heap of a few
hundred MiB, a handful of launches.

    python -m mintccl_b200.benchmarks.emu_kernels --kernel direct_allreduce --ranks 4 --mib 16 --calls 4
    ncu --set full --clock-control none -k regex:direct_kernel -s 2 -c 2 -o prof \\
        python -m mintccl_b200.benchmarks.emu_kernels --kernel direct_allreduce --ranks 4 --mib 16 --calls 4

The kernels are the ones the multi-GPU paths launch (same code, `gridDim.y` = ranks); what a capture of the
emulated world shows is their instruction mix, occupancy, memory traffic against the algorithmic bytes and
the stalls inside one GPU.  It does not show NVLink: "peer" memory is local here.  The script also prints the
CUDA-event time per call and the bytes each rank's kernel has to move, for the achieved-bandwidth figure.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

KERNELS = ("ring_simple_allreduce", "ring_ll128_allreduce", "ring_simple_allgather", "ring_simple_reducescatter",
           "direct_allreduce", "direct_allgather", "direct_reducescatter", "bulk_allgather", "direct_broadcast",
           "direct_reduce", "direct2_reduce", "ll_oneshot", "mxfp8_allreduce", "p2p_pull", "multihop_ll128")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=KERNELS)
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--mib", type=float, default=16.0, help="message MiB per rank (ignored by ll_oneshot)")
    ap.add_argument("--calls", type=int, default=4)
    ap.add_argument("--dtype", default="bf16", choices=["fp16", "bf16", "fp32"])
    ap.add_argument("--nch", type=int, default=0)
    a = ap.parse_args()

    from mintccl_b200 import Config, emulated
    n = a.ranks
    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[a.dtype]
    esz = torch.empty((), dtype=dtype).element_size()
    nbytes = int(a.mib * (1 << 20))
    numel = nbytes // esz // n * n
    # control region: 16 channels x n peers x (1 MiB Simple + 512 KiB LL128 FIFOs) stays under 128 MiB for n <= 8
    nchan = min(16, 148 // n)
    cfg = Config.from_env(max_channels=nchan, num_blocks=nchan, buff_size=1 << 20, heap_bytes=(256 << 20) + 8 * nbytes,
                          scratch_bytes=1 << 20, wait_timeout_ms=3000)
    w = emulated(n, 0, cfg)
    nch = a.nch or None
    moved = None   # bytes one rank's part of the kernel reads + writes (algorithmic)
    k = a.kernel

    def sym(ne, dt=dtype):
        ts = w.symm_empty(ne, dt)
        for r, t in enumerate(ts):
            t.copy_(torch.randn(ne, device="cuda", dtype=torch.float32).to(dt) if dt.is_floating_point
                    else torch.randint(0, 255, (ne,), device="cuda", dtype=dt))
        return ts

    if k in ("ring_simple_allreduce", "ring_ll128_allreduce"):
        xs = sym(numel)
        proto = "simple" if "simple" in k else "ll128"
        call = lambda: w.allreduce(xs, algo="ring", proto=proto, nch=nch)  # noqa: E731
        moved = 2 * (n - 1) / n * nbytes * 3          # per step: read slot + read own, write next slot (+ own)
    elif k == "ring_simple_allgather":
        gb = sym(numel)
        gbv = [t.view(n, -1) for t in gb]
        call = lambda: w.allgather(gbv, algo="ring", proto="simple", nch=nch)  # noqa: E731
        moved = (n - 1) / n * nbytes * 3
    elif k == "ring_simple_reducescatter":
        gb = sym(numel)
        gbv = [t.view(n, -1) for t in gb]
        call = lambda: w.reducescatter(gbv, algo="ring", proto="simple", nch=nch)  # noqa: E731
        moved = (n - 1) / n * nbytes * 3
    elif k == "direct_allreduce":
        xs, ys = sym(numel), sym(numel)
        call = lambda: w.allreduce(xs, out=ys, algo="direct", nch=nch)  # noqa: E731
        moved = nbytes + nbytes                       # read 1/n of every rank, write 1/n to every rank
    elif k in ("direct_allgather", "bulk_allgather"):
        gb = sym(numel)
        gbv = [t.view(n, -1) for t in gb]
        algo = "direct" if k.startswith("direct") else "bulk"
        call = lambda: w.allgather(gbv, algo=algo, nch=nch)  # noqa: E731
        moved = nbytes / n * (1 if algo == "bulk" else n - 1) + nbytes / n * (n - 1)
    elif k == "direct_reducescatter":
        gb = sym(numel)
        gbv = [t.view(n, -1) for t in gb]
        outs = [torch.empty(numel // n, device="cuda", dtype=dtype) for _ in range(n)]
        call = lambda: w.reducescatter(gbv, out=outs, algo="direct", nch=nch)  # noqa: E731
        moved = nbytes + nbytes / n
    elif k == "direct_broadcast":
        xs = sym(numel)
        call = lambda: w.broadcast(xs, root=0, algo="direct", nch=nch)  # noqa: E731
        moved = nbytes / n + nbytes
    elif k == "direct_reduce":
        xs, ys = sym(numel), sym(numel)
        call = lambda: w.reduce(xs, root=0, out=ys, algo="direct", nch=nch)  # noqa: E731
        moved = nbytes / (n - 1) * n + nbytes / (n - 1)
    elif k == "direct2_reduce":
        xs, ys = sym(numel), sym(numel)
        call = lambda: w.reduce(xs, root=0, out=ys, algo="direct2", nch=nch)  # noqa: E731
        moved = nbytes / (n - 1) * (n - 1) + nbytes / (n - 1) + 3 * nbytes / (n - 1)   # per non-root; the root adds locally
    elif k == "ll_oneshot":
        xs = [torch.randn(8192, device="cuda", dtype=torch.float32).to(dtype) for _ in range(n)]
        ys = [torch.empty_like(x) for x in xs]
        call = lambda: w.allreduce(xs, out=ys, algo="ll")  # noqa: E731
        moved = 8192 * esz * (n + 1)
    elif k == "mxfp8_allreduce":
        from mintccl_b200.ops import mxfp8 as mx
        ne = nbytes // (32 * n) * (32 * n)
        data, scale = sym(ne, torch.uint8), sym(ne // 32, torch.uint8)
        od, os_ = sym(ne, torch.uint8), sym(ne // 32, torch.uint8)
        for s_ in scale:
            s_.fill_(127)
        call = lambda: mx.allreduce_mxfp8(w, data, scale, od, os_)  # noqa: E731
        moved = ne * 33 / 32 * 2
    elif k == "p2p_pull":
        xs = sym(numel)
        call = lambda: w.sendrecv_direct(0, n - 1, xs, pull=True, nctas=nch)  # noqa: E731
        moved = 2 * nbytes
    else:  # multihop_ll128
        src = [torch.randint(0, 255, (nbytes,), device="cuda", dtype=torch.uint8) for _ in range(n)]
        dst = [torch.zeros(nbytes, device="cuda", dtype=torch.uint8) for _ in range(n)]
        call = lambda: w.sendrecv_route(list(range(n)), src, dst, proto="ll128", nch=nch)  # noqa: E731
        moved = 2 * nbytes * 128 / 120

    call()
    call()
    w.check()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.calls):
        call()
    e1.record()
    torch.cuda.synchronize()
    w.check()
    ms = e0.elapsed_time(e1) / a.calls
    print(json.dumps({"kernel": k, "ranks": n, "message_bytes": nbytes, "dtype": a.dtype, "ms_per_call": round(ms, 4),
                      "algorithmic_bytes_per_rank": int(moved), "all_ranks_GBps": round(n * moved / (ms * 1e-3) / 1e9, 1)}),
          flush=True)
    w.close()


if __name__ == "__main__":
    main()
