"""Worker of the multi-GPU tests: run under ``python -m torch.distributed.run`` with one rank per GPU.

Every rank can regenerate every other rank's input from the seed, so each rank checks its own result
against a locally computed fp32 oracle and no second library is needed as a reference."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def gen(rank, numel, dtype, seed0=0):
    g = torch.Generator(device="cuda").manual_seed(seed0 + rank)
    return torch.randn(numel, generator=g, device="cuda", dtype=torch.float32).to(dtype)


def close(got, srcs, dtype, hops=1, what=""):
    """Element-wise bound from the arithmetic: one rounding of an fp32 sum for the one-hop paths, `hops` roundings
    of partial sums (each at most sum |x_r|) for a ring; see tests/test_gpu_emulated.py::assert_sum_close."""
    ref = sum(s.float() for s in srcs)
    absum = sum(s.float().abs() for s in srcs)
    half = torch.finfo(dtype).eps / 2
    acc_err = len(srcs) * 2.0 ** -22 * absum
    bound = (1.01 * half * ref.abs() if hops <= 1 or dtype == torch.float32 else 1.01 * half * hops * absum) + acc_err
    bound = bound + torch.finfo(dtype).smallest_normal * torch.finfo(dtype).eps
    err = (got.float() - ref).abs()
    assert not bool((err > bound).any()), \
        f"{what}: outside the bound by {float((err - bound).max()):.3e} ({dtype}, hops={hops}, {got.numel()} elements)"


def ordinary_and_cast(c, rank, n):
    """Ordinary `torch.empty` tensors (shared with the peers through CUDA IPC on first use, at a different address
    and offset on every rank), heap tensors at offsets that differ between ranks, and reductions into another
    element type: all of them on the one-hop kernels, checked by the launch counters."""
    from mintccl_b200.utils import stats
    stats.reset()
    for dtype in (torch.float16, torch.float32):
        for numel in (1000, 262144 + 8, 3_000_001):
            srcs = [gen(r, numel, dtype, seed0=200) for r in range(n)]
            x = torch.empty(numel + 64, device="cuda", dtype=dtype)[8 * rank:8 * rank + numel]
            y = torch.empty(numel + 64, device="cuda", dtype=dtype)[8 * (n - rank):8 * (n - rank) + numel]
            x.copy_(srcs[rank])
            c.allreduce(x, out=y, algo="direct")
            c.check()
            close(y, srcs, dtype, 1)
            c.allreduce(x)                      # automatic choice, in place (one-shot LL below 32 KiB)
            c.check()
            close(x, srcs, dtype, 1)
            gb = torch.zeros(n, numel, device="cuda", dtype=dtype)
            gb[rank].copy_(srcs[rank])
            c.allgather(gb)
            c.check()
            assert torch.equal(gb, torch.stack(srcs)), "allgather on an ordinary tensor"
            gb.zero_()
            c.allgather(gb, inp=srcs[rank].clone(), algo="pull")
            c.check()
            assert torch.equal(gb, torch.stack(srcs)), "pull allgather on ordinary tensors"
            full = [gen(r, n * numel, dtype, seed0=210).view(n, numel) for r in range(n)]
            rs_in = full[rank].clone()
            shard = torch.empty(numel, device="cuda", dtype=dtype)
            c.reducescatter(rs_in, out=shard)
            c.check()
            close(shard, [f[rank] for f in full], dtype, 1)
            a2a = torch.empty(n, numel, device="cuda", dtype=dtype)
            c.alltoall(rs_in, a2a)
            c.check()
            for p in range(n):
                assert torch.equal(a2a[p], full[p][rank]), "alltoall on ordinary tensors"
            b = torch.empty(numel + 1, device="cuda", dtype=dtype)[1:]      # odd element offset: not 16-byte aligned
            b.copy_(srcs[rank])
            c.broadcast(b, root=n - 1, algo="direct")
            c.check()
            assert torch.equal(b, srcs[n - 1]), "broadcast on an ordinary tensor"
            rin = srcs[rank].clone()
            rout = torch.zeros(numel, device="cuda", dtype=dtype)
            c.reduce(rin, root=0, out=rout, algo="direct")
            c.check()
            if rank == 0:
                close(rout, srcs, dtype, 1)
            # heap tensors whose offsets differ from rank to rank (the allocator is used unevenly on purpose)
            pad = c.symm_empty(4096 * (rank + 1), torch.uint8)
            hx = c.symm_empty(numel, dtype)
            hy = c.symm_empty(numel, dtype)
            hx.copy_(srcs[rank])
            c.allreduce(hx, out=hy, algo="direct")
            c.check()
            close(hy, srcs, dtype, 1)
            for t in (hy, hx, pad):
                c.symm_free(t)
            torch.cuda.synchronize()
            c.control.barrier()
    seen = stats.snapshot(skip_idle=False)
    assert seen["ring_simple"]["calls"] == 0 and seen["ring_ll128"]["calls"] == 0 and seen["direct"]["calls"] > 0, seen
    # 16-bit -> fp32 and fp32 -> 16-bit
    for narrow in (torch.bfloat16, torch.float16):
        numel = 500_000
        srcs = [gen(r, numel, narrow, seed0=220) for r in range(n)]
        x = srcs[rank].clone()
        o32 = torch.zeros(numel, device="cuda", dtype=torch.float32)
        c.allreduce(x, out=o32, algo="oneshot")
        c.check()
        assert torch.equal(o32, sum(s.float() for s in srcs)), "fixed-order fp32 sum must match the oracle bit for bit"
        c.allreduce(x, out=o32)
        c.check()
        close(o32, srcs, torch.float32, 1)
        s32 = [gen(r, n * numel, torch.float32, seed0=230).view(n, numel) for r in range(n)]
        shard = torch.zeros(numel, device="cuda", dtype=narrow)
        c.reducescatter(s32[rank].clone(), out=shard)
        c.check()
        close(shard, [f[rank] for f in s32], narrow, 1)
        rout = torch.zeros(numel, device="cuda", dtype=torch.float32)
        c.reduce(x, root=n - 1, out=rout)
        c.check()
        if rank == n - 1:
            close(rout, srcs, torch.float32, 1)
    torch.cuda.synchronize()
    c.control.barrier()


def main():
    os.environ.setdefault("MINTCCL_TUNING_FILE", "none")   # the built-in policy; bench.py covers the shipped table
    import mintccl_b200
    from mintccl_b200 import Config
    rank, n = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    cfg = Config.from_env(heap_bytes=4 << 30, wait_timeout_ms=5000)
    c = mintccl_b200.Communicator(config=cfg)
    print(f"[r{rank}] heap={c.heap_kind} nvls={c.nvls} ring={c.ring}", flush=True)
    dtypes = [torch.float32, torch.float16, torch.bfloat16]
    sizes = [1, 120, 4099, 300_001, 2_000_000]
    algos_ar = ["ring:simple", "ring:ll128", "direct", "oneshot", "ll"] + (["nvls"] if c.nvls else [])
    for dtype in dtypes:
        for numel in sizes:
            srcs = [gen(r, numel, dtype) for r in range(n)]
            for a in algos_ar:
                if a == "ll" and numel * srcs[0].element_size() > c.ll_capacity:
                    continue
                if a == "nvls" and (numel * srcs[0].element_size()) % 16:
                    continue
                x = c.symm_empty(numel, dtype)
                x.copy_(srcs[rank])
                y = c.symm_empty(numel, dtype)
                if a.startswith("ring"):
                    c.allreduce(x, algo="ring", proto=a.split(":")[1])
                    got, hops = x, n
                elif a in ("oneshot", "ll"):
                    c.allreduce(x, out=y, algo=a)
                    got, hops = y, 1
                else:
                    c.allreduce(x, algo=a)
                    # the switch adds in fp32 but its result can sit one rounding away from the nearest value
                    got, hops = x, (2 if a == "nvls" else 1)
                c.check()
                close(got, srcs, dtype, hops, f"allreduce {a}")
                c.symm_free(x)
                c.symm_free(y)
            # all-gather / reduce-scatter / all-to-all / broadcast / reduce
            for mode, algo, proto in [("temporal", "ring", "simple"), ("spatial", "ring", "ll128"), ("temporal", "direct", None),
                                      ("temporal", "pull", None)] + ([("temporal", "nvls", None)] if c.nvls and (numel * srcs[0].element_size()) % 16 == 0 else []):
                gb = c.symm_zeros((n, numel), dtype)
                gb[rank].copy_(srcs[rank])
                torch.cuda.synchronize()
                c.control.barrier()
                c.allgather(gb, mode=mode, algo=algo, proto=proto)
                c.check()
                assert torch.equal(gb, torch.stack(srcs)), f"allgather {algo} {mode} {dtype} {numel}"
                c.symm_free(gb)
            full = [gen(r, n * numel, dtype, seed0=100).view(n, numel) for r in range(n)]
            for mode, algo, proto in [("temporal", "ring", "simple"), ("spatial", "ring", "ll128"), ("temporal", "direct", None)] + \
                    ([("temporal", "nvls", None)] if c.nvls and (numel * srcs[0].element_size()) % 16 == 0 else []):
                gb = c.symm_empty((n, numel), dtype)
                gb.copy_(full[rank])
                out = torch.empty(numel, device="cuda", dtype=dtype)
                torch.cuda.synchronize()
                c.control.barrier()
                c.reducescatter(gb, out=out, mode=mode, algo=algo, proto=proto)
                c.check()
                close(out, [f[rank] for f in full], dtype, n if algo == "ring" else (2 if algo == "nvls" else 1),
                      f"reducescatter {algo}")
                c.symm_free(gb)
            gi = c.symm_empty((n, numel), dtype)
            go = c.symm_empty((n, numel), dtype)
            gi.copy_(full[rank])
            torch.cuda.synchronize()
            c.control.barrier()
            c.alltoall(gi, go)
            c.check()
            for p in range(n):
                assert torch.equal(go[p], full[p][rank]), "alltoall"
            c.symm_free(gi)
            c.symm_free(go)
            for algo in ["ring", "direct", "pull", "push"] + (["nvls", "nvls1"] if c.nvls and (numel * srcs[0].element_size()) % 16 == 0 else []):
                b = c.symm_empty(numel, dtype)
                b.copy_(srcs[rank])
                torch.cuda.synchronize()
                c.control.barrier()
                c.broadcast(b, root=n - 1, algo=algo)
                c.check()
                assert torch.equal(b, srcs[n - 1]), f"broadcast {algo}"
                b.copy_(srcs[rank])
                o = torch.zeros(numel, device="cuda", dtype=dtype)
                torch.cuda.synchronize()
                c.control.barrier()
                if algo in ("pull", "push"):
                    c.symm_free(b)
                    continue
                c.reduce(b, root=0, out=o, algo=algo)
                c.check()
                if rank == 0:
                    close(o, srcs, dtype, n if algo == "ring" else (2 if algo.startswith("nvls") else 1), f"reduce {algo}")
                if algo == "direct" and n >= 3 and (numel * srcs[0].element_size()) % 16 == 0:
                    o2 = torch.zeros(numel, device="cuda", dtype=dtype)   # the root sums its own input: two roundings
                    torch.cuda.synchronize()
                    c.control.barrier()
                    c.reduce(b, root=1, out=o2, algo="direct2")
                    c.check()
                    if rank == 1:
                        close(o2, srcs, dtype, 2, "reduce direct2")
                if algo in ("direct", "nvls"):  # symmetric output: summing spread over all ranks
                    so = c.symm_zeros(numel, dtype)
                    torch.cuda.synchronize()
                    c.control.barrier()
                    c.reduce(b, root=n - 1, out=so, algo=algo)
                    c.check()
                    if rank == n - 1:
                        close(so, srcs, dtype, 2 if algo.startswith("nvls") else 1, f"reduce {algo} (symmetric output)")
                    c.control.barrier()
                    c.symm_free(so)
                c.symm_free(b)
    ordinary_and_cast(c, rank, n)
    # fused GEMM + collective kernels against the unfused fp32 reference
    from mintccl_b200.ops.gemm import AllGatherGemm, GemmReduceScatter
    M, Nn, K = 128 * n * 2, 512, 256
    ag = AllGatherGemm(c, M, Nn, K, ncomm=4)
    rs = GemmReduceScatter(c, M, Nn, K)
    for it in range(3):
        shards = [gen(r, (M // n) * K, torch.bfloat16, seed0=50 + it).view(M // n, K) for r in range(n)]
        w = (gen(rank, Nn * K, torch.float32, seed0=60 + it) * 0.05).to(torch.bfloat16).view(Nn, K)
        out = ag(shards[rank].contiguous(), w)
        c.check()
        ref = torch.cat(shards, 0).float() @ w.float().t()
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=3e-2)
        As = [gen(r, M * K, torch.bfloat16, seed0=70 + it).view(M, K) for r in range(n)]
        Ws = [(gen(r, Nn * K, torch.float32, seed0=80 + it) * 0.05).to(torch.bfloat16).view(Nn, K) for r in range(n)]
        y = rs(As[rank].contiguous(), Ws[rank].contiguous())
        c.check()
        ref = sum((a_.float() @ w_.float().t()).to(torch.bfloat16).float() for a_, w_ in zip(As, Ws))
        rows = M // n
        torch.testing.assert_close(y.float(), ref[rank * rows:(rank + 1) * rows], rtol=2e-2, atol=4e-2)
    # the same two fusions on MXFP8 operands against the dequantised fp32 product
    from mintccl_b200.ops import mxfp8 as mx
    ag8 = AllGatherGemm(c, M, Nn, K, ncomm=4, fp8=True)
    deq = lambda q, r_, k_: mx.dequantize_mxfp8(q[0].reshape(-1), q[1].reshape(-1)).view(r_, k_)
    for it in range(2):
        qs = [mx.quantize_rows_mxfp8(gen(r, (M // n) * K, torch.float32, seed0=90 + it).view(M // n, K)) for r in range(n)]
        qw = [mx.quantize_rows_mxfp8(gen(r, Nn * K, torch.float32, seed0=95 + it).view(Nn, K) * 0.05) for r in range(n)]
        out = ag8.call_mxfp8(qs[rank][0], qs[rank][1], qw[rank][0], qw[rank][1])
        c.check()
        ref = torch.cat([deq(q, M // n, K) for q in qs], 0) @ deq(qw[rank], Nn, K).t()
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=5e-2)
        qA = [mx.quantize_rows_mxfp8(gen(r, M * K, torch.float32, seed0=100 + it).view(M, K)) for r in range(n)]
        y = rs.call_mxfp8(qA[rank][0], qA[rank][1], qw[rank][0], qw[rank][1])
        c.check()
        ref = sum((deq(qA[r], M, K) @ deq(qw[r], Nn, K).t()).to(torch.bfloat16).float() for r in range(n))
        rows = M // n
        torch.testing.assert_close(y.float(), ref[rank * rows:(rank + 1) * rows], rtol=2e-2, atol=6e-2)
    c.control.barrier()
    # point to point: deferred API over a multi-hop ring route, direct pull and push, registered tensor
    os.environ["MINTCCL_ROUTE"] = "ring"
    a = gen(0, 1_000_003, torch.float16)
    dst = n - 1
    buf = a.clone() if rank == 0 else torch.zeros_like(a)
    if rank == 0:
        c.send(buf, dst)
    elif rank == dst:
        c.recv(buf, 0)
    c.sync()
    c.check()
    if rank == dst:
        assert torch.equal(buf, a), "multi-hop send/recv"
    s = c.symm_empty(500_000, torch.float32)
    s.copy_(gen(rank, 500_000, torch.float32, seed0=7))
    torch.cuda.synchronize()
    c.control.barrier()
    for pull in (True, False):
        c.sendrecv_direct(0, n - 1, s, pull=pull)
        c.check()
        if rank == n - 1:
            assert torch.equal(s, gen(0, 500_000, torch.float32, seed0=7)), f"direct pull={pull}"
        c.control.barrier()
    t = gen(rank, 250_000, torch.float32, seed0=9)
    ptrs = c.register(t)
    out = torch.zeros_like(t)
    c.p2p_copy(0, n - 1, ptrs[0], out.data_ptr() if rank == n - 1 else 0, t.numel() * 4, pull=True)
    c.check()
    if rank == n - 1:
        assert torch.equal(out, gen(0, 250_000, torch.float32, seed0=9)), "registered pull"
    # 1000 back-to-back multi-hop transfers (all ranks on the route)
    route = c.ring[:]
    small = torch.full((1024,), float(rank), device="cuda")
    got = torch.zeros(1024, device="cuda")
    for _ in range(1000):
        c.sendrecv_route(route, small if rank == route[0] else None, got if rank == route[-1] else None,
                         nbytes=4096, proto="ll128")
    c.check()
    if rank == route[-1]:
        assert float(got[0]) == float(route[0])
    c.control.barrier()
    if os.environ.get("MINTCCL_TEST_PROBE") and rank == 0:
        # link discovery on real devices: the peer-access map, and one measured pair (1 MiB copies)
        from mintccl_b200.topology import get_p2p_speed, get_topology
        topo = get_topology("", measure=False, ndev=n)
        assert sorted(topo) == list(range(n)) and all(sorted(d for d, _ in topo[s]) == [d for d in range(n) if d != s]
                                                      for s in range(n)), topo
        bw = get_p2p_speed(0, 1, 1 << 20)
        assert bw > 1.0, bw
        print(f"[r0] probe 0 -> 1: {bw:.1f} GB/s at 1 MiB; discovered ring {c.ring}", flush=True)
    c.control.barrier()
    c.close()
    print(f"[r{rank}] MULTI OK", flush=True)


if __name__ == "__main__":
    main()
