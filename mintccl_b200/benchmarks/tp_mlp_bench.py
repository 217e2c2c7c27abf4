"""Tensor-parallel MLP projections, fused kernels against the unfused NCCL + cuBLAS baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        mintccl_b200/benchmarks/tp_mlp_bench.py --tokens 8192 --hidden 4096 --ffn 14336

up:   all-gather of the [tokens / n, hidden] activation shard -> GEMM with the [ffn / n, hidden] weight
down: GEMM with the [hidden, ffn / n] weight -> reduce-scatter of [tokens, hidden] over tokens
Weights are randn x 0.02, activations randn (bf16).  Device time, max over ranks; results are checked
against the unfused path.
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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ncomm", default="0", help="comma list of comm-CTA counts to try for the all-gather fusion")
    ap.add_argument("--split", default="1", help="comma list: comm CTAs that share one 128-row chunk")
    ap.add_argument("--modes", default="push", help="comma list of all-gather transports: push, pull, push_st")
    ap.add_argument("--mxfp8", action="store_true",
                    help="also time both fused kernels on MXFP8 operands (quantised once, outside the timed loop)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    gloo = dist.new_group(backend="gloo")
    import mintccl_b200
    from mintccl_b200 import Config
    from mintccl_b200.ops.gemm import AllGatherGemm, GemmReduceScatter, gemm
    comm = mintccl_b200.Communicator(group=gloo, config=Config.from_env(heap_bytes=6 << 30))
    n, T, H = world, a.tokens, a.hidden
    F = a.ffn // n // 256 * 256  # the kernels tile N in 256 columns
    g = torch.Generator(device="cuda").manual_seed(rank)
    x_shard = comm.symm_empty((T // n, H), torch.bfloat16)
    x_shard.copy_(torch.randn(T // n, H, generator=g, device="cuda").to(torch.bfloat16))
    w_up = (torch.randn(F, H, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(H, F, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    act = torch.randn(T, F, generator=g, device="cuda").to(torch.bfloat16)

    def maxr(x):
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return float(t[0])

    def timed(fn):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier(group=gloo)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return maxr(e0.elapsed_time(e1) / a.iters * 1e3)

    flop = 2.0 * T * H * F
    out = {"n": n, "tokens": T, "hidden": H, "ffn_local": F, "gflop_per_rank": flop / 1e9}
    # ---- unfused baselines
    xg = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    h_ref = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)

    def up_unfused():
        dist.all_gather_into_tensor(xg, x_shard)
        torch.matmul(xg, w_up.t(), out=h_ref)

    y_full = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    y_ref = torch.empty(T // n, H, device="cuda", dtype=torch.bfloat16)

    def down_unfused():
        torch.matmul(act, w_down.t(), out=y_full)
        dist.reduce_scatter_tensor(y_ref, y_full)

    out["up_unfused_us"] = round(timed(up_unfused), 1)
    out["down_unfused_us"] = round(timed(down_unfused), 1)
    out["up_gemm_only_cublas_us"] = round(timed(lambda: torch.matmul(xg, w_up.t(), out=h_ref)), 1)
    out["up_gemm_only_tcgen05_us"] = round(timed(lambda: gemm(xg, w_up, out=h_ref)), 1)
    up_unfused()
    down_unfused()
    # ---- fused
    h = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
    best = None
    for mode, nc, sp in [(m, int(v), int(q)) for m in a.modes.split(",") for v in a.ncomm.split(",") for q in a.split.split(",")]:
        if nc and sp > nc:
            continue
        plan = AllGatherGemm(comm, T, F, H, ncomm=nc or None, mode=mode, split=sp)
        nc = plan.ncomm
        us = timed(lambda: plan(x_shard, w_up, out=h))
        comm.check()
        out[f"up_fused_us_{mode}_ncomm{nc}_split{sp}"] = round(us, 1)
        if best is None or us < best:
            best = us
        comm.symm_free(plan.gathered)
        comm.symm_free(plan.flags)
    out["up_fused_us"] = round(best, 1)
    err_up = (h.float() - h_ref.float()).abs().max().item()
    rs = GemmReduceScatter(comm, T, H, F)
    y = torch.empty(T // n, H, device="cuda", dtype=torch.bfloat16)
    out["down_fused_us"] = round(timed(lambda: rs(act, w_down, out=y)), 1)
    comm.check()
    err_down = (y.float() - y_ref.float()).abs().max().item()
    out["max_abs_err_up"], out["max_abs_err_down"] = round(err_up, 4), round(err_down, 4)
    out["up_speedup"] = round(out["up_unfused_us"] / out["up_fused_us"], 3)
    out["down_speedup"] = round(out["down_unfused_us"] / out["down_fused_us"], 3)
    if a.mxfp8 and H % 128 == 0 and F % 128 == 0:
        # The same two projections on block-scaled fp8 operands.  Activations and weights are quantised before the
        # timed loop (a model would quantise in the epilogue of the producing kernel); the tiling of the activation
        # scales and their small all-gather are inside it.  Checked against the dequantised fp32 product.
        from mintccl_b200.ops import mxfp8 as mx
        qx = mx.quantize_rows_mxfp8(x_shard.float())
        qwu = mx.quantize_rows_mxfp8(w_up.float())
        qwd = mx.quantize_rows_mxfp8(w_down.float())
        qact = mx.quantize_rows_mxfp8(act.float())
        twu, twd = mx.tile_scales(qwu[1]), mx.tile_scales(qwd[1])
        ag8 = AllGatherGemm(comm, T, F, H, fp8=True)
        h8 = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
        out["up_fused_mxfp8_us"] = round(timed(lambda: ag8.call_mxfp8(qx[0], qx[1], qwu[0], twu, out=h8, w_scale_tiled=True)), 1)
        comm.check()
        y8 = torch.empty(T // n, H, device="cuda", dtype=torch.bfloat16)
        out["down_fused_mxfp8_us"] = round(timed(lambda: rs.call_mxfp8(qact[0], qact[1], qwd[0], twd, out=y8, w_scale_tiled=True)), 1)
        comm.check()
        # against the bf16 results: both carry the fp8 quantisation error of operands of unit scale (~2^-4 relative
        # per element, averaged down over K)
        out["mxfp8_rel_err_up"] = round(((h8.float() - h_ref.float()).norm() / h_ref.float().norm()).item(), 4)
        out["mxfp8_rel_err_down"] = round(((y8.float() - y_ref.float()).norm() / y_ref.float().norm()).item(), 4)
        out["up_mxfp8_speedup_vs_unfused_bf16"] = round(out["up_unfused_us"] / out["up_fused_mxfp8_us"], 3)
        out["down_mxfp8_speedup_vs_unfused_bf16"] = round(out["down_unfused_us"] / out["down_fused_mxfp8_us"], 3)
    # roofline: the slower of the GEMM at the measured cuBLAS peak and the bytes over NVLink at 770 GB/s
    link_bytes = (n - 1) / n * T * H * 2
    peak = 1369.5e12
    ideal_us = max(flop / peak, link_bytes / 770e9) * 1e6
    out["roofline_us"] = round(ideal_us, 1)
    out["up_frac_of_roofline"] = round(ideal_us / out["up_fused_us"], 3)
    out["down_frac_of_roofline"] = round(ideal_us / out["down_fused_us"], 3)
    if rank == 0:
        print(json.dumps(out), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
