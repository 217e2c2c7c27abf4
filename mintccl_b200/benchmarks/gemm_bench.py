"""Times the tcgen05 GEMM against cuBLAS (torch.matmul) on one GPU.

    python mintccl_b200/benchmarks/gemm_bench.py [--shapes 8192x1792x4096,8192x4096x1792] [--iters 20]

Each shape is MxNxK for ``a[M, K] @ w[N, K].T``.  Device time from CUDA events after warm-up; operands and
outputs of consecutive calls rotate through a pool larger than the L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192x1792x4096,8192x4096x1792,8192x8192x8192,4096x4096x4096")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nctas", type=int, default=0)
    ap.add_argument("--mxfp8", action="store_true", help="also time the block-scaled fp8 GEMM on each shape")
    a = ap.parse_args()
    from mintccl_b200.ops.gemm import gemm
    for shape in a.shapes.split(","):
        M, N, K = (int(x) for x in shape.split("x"))
        per = (M * K + N * K + M * N) * 2
        copies = max(2, (300 << 20) // per + 1)
        As = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        Ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        Os = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
        row = {"shape": shape, "flop": 2.0 * M * N * K}
        for name, fn in (("tcgen05", lambda i: gemm(As[i], Ws[i], out=Os[i], nctas=a.nctas)),
                         ("cublas", lambda i: torch.matmul(As[i], Ws[i].t(), out=Os[i]))):
            for i in range(5):
                fn(i % copies)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(a.iters):
                fn(i % copies)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.iters
            row[name + "_us"] = round(ms * 1e3, 1)
            row[name + "_tflops"] = round(row["flop"] / (ms * 1e-3) / 1e12, 1)
        row["ratio"] = round(row["tcgen05_tflops"] / row["cublas_tflops"], 3)
        if a.mxfp8 and K % 128 == 0:
            # block-scaled fp8 operands of the same shape (quantised once, scales pre-tiled, outside the timed loop)
            from mintccl_b200.ops import mxfp8 as mx
            c8 = max(2, (300 << 20) // (M * K + N * K + M * N * 2) + 1)
            qa = [mx.quantize_rows_mxfp8(As[i % copies].float()) for i in range(c8)]
            qw = [mx.quantize_rows_mxfp8(Ws[i % copies].float()) for i in range(c8)]
            ta = [(q[0], mx.tile_scales(q[1])) for q in qa]
            tw = [(q[0], mx.tile_scales(q[1])) for q in qw]
            fn = lambda i: mx.gemm_mxfp8(ta[i][0], ta[i][1], tw[i][0], tw[i][1], out=Os[i % copies], nctas=a.nctas,
                                         scales_tiled=True)
            for i in range(5):
                fn(i % c8)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(a.iters):
                fn(i % c8)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.iters
            row["mxfp8_us"] = round(ms * 1e3, 1)
            row["mxfp8_tflops"] = round(row["flop"] / (ms * 1e-3) / 1e12, 1)
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
