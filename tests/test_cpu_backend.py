"""The public API on the CPU reference backend (torch.distributed gloo, one process per rank).

Covers the plumbing configuration of the baseline: rank 0 sends a 1,048,576-element fp16 tensor drawn
from randn(seed=0) to rank 1, compared bit-exactly."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, init_file, result_q):
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    import mintccl_b200 as m
    try:
        # config 1: direct send/recv, bit exact
        g = torch.Generator().manual_seed(0)
        payload = torch.randn(1_048_576, generator=g).to(torch.float16)
        buf = payload.clone() if rank == 0 else torch.zeros_like(payload)
        if rank == 0:
            m.send(buf, 1)
        elif rank == 1:
            m.recv(buf, 0)
        m.sync()
        if rank == 1:
            assert torch.equal(buf, payload)
        # collectives with the in-place conventions of the reference
        n = world
        srcs = [torch.randn(1000, generator=torch.Generator().manual_seed(r)).to(torch.float16) for r in range(n)]
        ref = sum(s.float() for s in srcs)
        x = srcs[rank].clone()
        m.allreduce(x)
        torch.testing.assert_close(x.float(), ref.to(torch.float16).float(), rtol=1e-2, atol=1e-2)
        gb = torch.zeros(n, 1000, dtype=torch.float16)
        gb[rank] = srcs[rank]
        m.allgather(gb)
        assert torch.equal(gb, torch.stack(srcs))
        m.allgather(gb, mode="spatial")
        assert torch.equal(gb, torch.stack(srcs))
        full = [torch.randn(n, 64, generator=torch.Generator().manual_seed(10 + r)) for r in range(n)]
        rs = full[rank].clone()
        m.reducescatter(rs)
        torch.testing.assert_close(rs[rank], sum(full)[rank], rtol=1e-5, atol=1e-5)
        b = srcs[rank].clone()
        m.broadcast(b, root=n - 1)
        assert torch.equal(b, srcs[n - 1])
        r_ = srcs[rank].clone()
        m.reduce(r_, root=0)
        if rank == 0:
            torch.testing.assert_close(r_.float(), ref.to(torch.float16).float(), rtol=1e-2, atol=1e-2)
        a_in = torch.arange(n * 4, dtype=torch.float32).view(n, 4) + 100 * rank
        a_out = torch.empty_like(a_in)
        m.alltoall(a_in, a_out)
        for p in range(n):
            assert torch.equal(a_out[p], torch.arange(4, dtype=torch.float32) + 4 * rank + 100 * p)
        # a mismatched send/recv pair is rejected on the host before anything is launched
        comm = m.get_comm(buf)
        assert comm.world_size == world and comm.rank == rank
        # block-scaled fp8 sums: fp32 accumulation over the dequantised inputs, one requantisation
        from mintccl_b200.ops import mxfp8 as mx
        xs = [torch.randn(n * 256, generator=torch.Generator().manual_seed(40 + r)) * (r + 1) for r in range(n)]
        qs = [mx.quantize_mxfp8(t) for t in xs]
        total = sum(mx.dequantize_mxfp8(d_, s_) for d_, s_ in qs)
        want_d, want_s = mx.quantize_mxfp8(total)
        d_, s_ = qs[rank][0].clone(), qs[rank][1].clone()
        mx.allreduce_mxfp8(comm, d_, s_)
        assert torch.equal(d_, want_d) and torch.equal(s_, want_s)
        od, os_ = torch.empty(256, dtype=torch.uint8), torch.empty(8, dtype=torch.uint8)
        mx.reducescatter_mxfp8(comm, qs[rank][0], qs[rank][1], od, os_)
        wd, ws = mx.quantize_mxfp8(total[rank * 256:(rank + 1) * 256])
        assert torch.equal(od, wd) and torch.equal(os_, ws)
        result_q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        result_q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        m.shutdown()
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_cpu_backend_world(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        f = os.path.join(d, "rdzv")
        procs = [ctx.Process(target=_worker, args=(r, world, f, q)) for r in range(world)]
        for p in procs:
            p.start()
        results = [q.get(timeout=180) for _ in range(world)]
        for p in procs:
            p.join(60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results


def test_single_process_cpu_backend():
    import mintccl_b200 as m
    from mintccl_b200.parallel.cpu_backend import CpuCommunicator
    from mintccl_b200.parallel.rendezvous import SingleControl
    c = CpuCommunicator(control=SingleControl())
    x = torch.arange(8, dtype=torch.float32)
    y = x.clone()
    c.allreduce(y)
    assert torch.equal(x, y)
    gb = x.view(1, 8).clone()
    c.allgather(gb)
    assert torch.equal(gb[0], x)
    assert m.find_ring(m.uniform_topology(1)) == [0, 0]
