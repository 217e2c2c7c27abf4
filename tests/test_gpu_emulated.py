"""Every collective on an emulated world (n ranks on one GPU, one cooperative kernel per call) against a
plain PyTorch fp32 reference.  Copies must be bit-exact; sums are compared with the fp32-accumulated
oracle at rtol 1e-2 (the reference compares reductions bit-exactly with NCCL, 5_reduce.py:145, which
cannot hold for more than two ranks)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
_worlds = {}


def world(n):
    from mintccl_b200 import Config, emulated
    if n not in _worlds:
        cfg = Config.from_env(max_channels=16, num_blocks=16, buff_size=1 << 20, heap_bytes=768 << 20,
                              scratch_bytes=1 << 20, wait_timeout_ms=3000)
        _worlds[n] = emulated(n, 0, cfg)
    return _worlds[n]


def rand(n, numel, dtype, seed0=0):
    out = []
    for r in range(n):
        g = torch.Generator(device="cuda").manual_seed(seed0 + r)
        out.append(torch.randn(numel, generator=g, device="cuda", dtype=torch.float32).to(dtype))
    return out


class Oracle:
    """fp32 sum of the ranks' inputs plus the sum of their magnitudes, which scales the error bounds."""

    def __init__(self, ref, absum):
        self.ref, self.absum = ref, absum

    def __getitem__(self, i):
        return Oracle(self.ref[i], self.absum[i])

    def view(self, *shape):
        return Oracle(self.ref.view(*shape), self.absum.view(*shape))


def oracle_sum(ts):
    acc = torch.zeros_like(ts[0], dtype=torch.float32)
    mag = torch.zeros_like(acc)
    for t in ts:
        acc += t.float()
        mag += t.float().abs()
    return Oracle(acc, mag)


def assert_sum_close(got, oracle, dtype, hops=1, nranks=8):
    """Element-wise bound that follows from the arithmetic, not a blanket tolerance.  One-hop paths (direct, NVLS,
    one-shot) add all ranks in fp32 and round once into `dtype`: the error is at most half an ulp of the result
    plus the fp32 accumulation error.  A ring rounds the partial sum into `dtype` at each of its `hops` combines,
    and a partial sum is at most sum |x_r|: at most hops half-ulps of that.  A dropped or doubled contribution, a
    wrong rounding mode or a sum in 16-bit arithmetic falls outside these bounds."""
    half = torch.finfo(dtype).eps / 2
    ref, absum = oracle.ref, oracle.absum
    acc_err = nranks * 2.0 ** -22 * absum                       # fp32 accumulation, any order
    if hops <= 1 or dtype == torch.float32:
        bound = 1.01 * half * ref.abs() + acc_err
    else:
        bound = 1.01 * half * hops * absum + acc_err
    err = (got.float() - ref).abs()
    bad = err > bound + torch.finfo(dtype).smallest_normal * torch.finfo(dtype).eps   # subnormal results
    assert not bool(bad.any()), (f"{int(bad.sum())} of {bad.numel()} elements outside the bound; worst excess "
                                 f"{float((err - bound).max()):.3e} ({dtype}, hops={hops})")


SIZES = [1, 7, 120, 1000, 4099, 65536 + 3, 1_500_000]


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("proto", ["simple", "ll128"])
@pytest.mark.parametrize("numel", SIZES)
def test_ring_allreduce(n, proto, numel):
    w = world(n)
    for dtype in DTYPES:
        xs = rand(n, numel, dtype)
        ref = oracle_sum(xs)
        w.allreduce(xs, algo="ring", proto=proto)
        w.check()
        for x in xs:
            assert_sum_close(x, ref, dtype, hops=n)
        for x in xs[1:]:
            assert torch.equal(x, xs[0])  # every rank holds the same bits


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("proto", ["simple", "ll128"])
@pytest.mark.parametrize("mode", ["temporal", "spatial"])
@pytest.mark.parametrize("numel", [1, 33, 5000, 300_001])
def test_ring_allgather(n, proto, mode, numel):
    w = world(n)
    for dtype in (torch.float32, torch.bfloat16):
        src = rand(n, numel, dtype)
        bufs = [torch.zeros(n, numel, device="cuda", dtype=dtype) for _ in range(n)]
        for r in range(n):
            bufs[r][r].copy_(src[r])
        w.allgather(bufs, mode=mode, algo="ring", proto=proto)
        w.check()
        ref = torch.stack(src)
        for b in bufs:
            assert torch.equal(b, ref)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("proto", ["simple", "ll128"])
@pytest.mark.parametrize("mode", ["temporal", "spatial"])
@pytest.mark.parametrize("numel", [1, 33, 5000, 300_001])
def test_ring_reducescatter(n, proto, mode, numel):
    w = world(n)
    for dtype in DTYPES:
        bufs = [t.view(n, numel) for t in rand(n, n * numel, dtype, seed0=11)]
        ref = oracle_sum(bufs)
        w.reducescatter(bufs, mode=mode, algo="ring", proto=proto)
        w.check()
        for r in range(n):
            assert_sum_close(bufs[r][r], ref[r], dtype, hops=n)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("proto", ["simple", "ll128"])
@pytest.mark.parametrize("numel", [1, 1000, 1_000_003])
def test_ring_broadcast_and_reduce(n, proto, numel):
    w = world(n)
    for root in (0, n - 1):
        xs = rand(n, numel, torch.float16, seed0=3)
        want = xs[root].clone()
        w.broadcast(xs, root=root, algo="ring", proto=proto)
        w.check()
        for x in xs:
            assert torch.equal(x, want)
        for dtype in DTYPES:
            ys = rand(n, numel, dtype, seed0=5)
            ref = oracle_sum(ys)
            w.reduce(ys, root=root, algo="ring", proto=proto)
            w.check()
            assert_sum_close(ys[root], ref, dtype, hops=n)


@pytest.mark.parametrize("proto", ["simple", "ll128"])
@pytest.mark.parametrize("nbytes", [8, 4096, 1 << 20, (4 << 20) + 24])
def test_multihop_sendrecv(proto, nbytes):
    """rank 0 -> rank 4 through the jump hosts 1, 2, 3 (the reference hard-codes route [0, 1])."""
    w = world(8)
    src = [torch.randint(0, 255, (nbytes,), device="cuda", dtype=torch.uint8) for _ in range(8)]
    dst = [torch.zeros(nbytes, device="cuda", dtype=torch.uint8) for _ in range(8)]
    w.sendrecv_route([0, 1, 2, 3, 4], src, dst, proto=proto)
    w.check()
    assert torch.equal(dst[4], src[0])
    for r in (0, 1, 2, 3, 5, 6, 7):
        assert int(dst[r].sum()) == 0  # jump hosts never touch their user memory


def test_deferred_send_recv_sync():
    w = world(4)
    a = torch.randn(100_000, device="cuda")
    b = torch.zeros_like(a)
    c = torch.randn(77, device="cuda", dtype=torch.float16)
    d = torch.zeros_like(c)
    w.send(a, 2, rank=1)
    w.recv(b, 1, rank=2)
    w.send(c, 0, rank=3)
    w.recv(d, 3, rank=0)
    w.sync()
    w.check()
    assert torch.equal(a, b) and torch.equal(c, d)


def test_back_to_back_thousand_multihop():
    """1,000 consecutive multi-hop transfers on the same FIFOs: flags never repeat, nothing is cleared."""
    w = world(8)
    nbytes = 4096
    src = [torch.randint(0, 255, (nbytes,), device="cuda", dtype=torch.uint8) for _ in range(8)]
    dst = [torch.zeros(nbytes, device="cuda", dtype=torch.uint8) for _ in range(8)]
    for i in range(1000):
        w.sendrecv_route([0, 1, 2, 3, 4], src, dst, proto="ll128")
    w.check()
    assert torch.equal(dst[4], src[0])


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("numel", [2, 5, 1000, 16 * 1024])
def test_ll_oneshot_allreduce(n, numel):
    w = world(n)
    for dtype in DTYPES:
        for it in range(3):  # both parities of the staging area, back to back
            xs = rand(n, numel, dtype, seed0=it)
            ref = oracle_sum(xs)
            outs = [torch.empty_like(x) for x in xs]
            w.allreduce(xs, out=outs, algo="ll")
            w.check()
            for o in outs:
                assert_sum_close(o, ref, dtype)
            for o in outs[1:]:
                assert torch.equal(o, outs[0])


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("numel", [4, 1001, 262144 + 8, 3_000_000])
def test_direct_collectives(n, numel):
    w = world(n)
    for dtype in DTYPES:
        # all-reduce, two-shot (in place) and one-shot (out of place)
        xs = w.symm_empty(numel, dtype)
        src = rand(n, numel, dtype, seed0=21)
        for x, s in zip(xs, src):
            x.copy_(s)
        ref = oracle_sum(src)
        w.allreduce(xs, algo="direct")
        w.check()
        for x in xs:
            assert_sum_close(x, ref, dtype)
        for x in xs[1:]:
            assert torch.equal(x, xs[0])
        for x, s in zip(xs, src):
            x.copy_(s)
        outs = [torch.empty_like(s) for s in src]
        w.allreduce(xs, out=outs, algo="oneshot")
        w.check()
        for o in outs:
            assert_sum_close(o, ref, dtype)
        for o in outs[1:]:
            assert torch.equal(o, outs[0])
        w.symm_free(xs)
        # all-gather (push and pull)
        gb = w.symm_empty((n, numel), dtype)
        for algo in ("direct", "pull"):
            for r in range(n):
                gb[r].zero_()
                gb[r][r].copy_(src[r])
            w.allgather(gb, algo=algo)
            w.check()
            want = torch.stack(src)
            for b in gb:
                assert torch.equal(b, want)
        # reduce-scatter
        full = rand(n, n * numel, dtype, seed0=31)
        for r in range(n):
            gb[r].view(-1).copy_(full[r])
        ref2 = oracle_sum(full).view(n, numel)
        outs = [torch.empty(numel, device="cuda", dtype=dtype) for _ in range(n)]
        w.reducescatter(gb, out=outs, algo="direct")
        w.check()
        for r in range(n):
            assert_sum_close(outs[r], ref2[r], dtype)
        # all-to-all
        ob = w.symm_empty((n, numel), dtype)
        for r in range(n):
            gb[r].view(-1).copy_(full[r])
        w.alltoall(gb, ob)
        w.check()
        for r in range(n):
            for p in range(n):
                assert torch.equal(ob[r][p], full[p].view(n, numel)[r])
        # broadcast and reduce
        for r in range(n):
            gb[r].view(-1).copy_(full[r])
        for algo, root in (("direct", n - 1), ("direct", 1 % n), ("push", n - 1), ("pull", n - 1), (None, 0)):
            for r in range(n):
                gb[r].view(-1).copy_(full[r])
            w.broadcast(gb, root=root, algo=algo)
            w.check()
            for r in range(n):
                assert torch.equal(gb[r].view(-1), full[root]), (algo, root)
        for r in range(n):
            gb[r].view(-1).copy_(full[r])
        routs = [torch.zeros(n, numel, device="cuda", dtype=dtype) for _ in range(n)]
        w.reduce(gb, root=1, out=routs, algo="direct")
        w.check()
        assert_sum_close(routs[1].view(-1), oracle_sum(full), dtype)
        # symmetric output: every rank sums one sub-slice and stores it into the root's buffer
        for o in ob:
            o.zero_()
        w.reduce(gb, root=0, out=ob, algo="direct")
        w.check()
        assert_sum_close(ob[0].view(-1), oracle_sum(full), dtype)
        w.symm_free(gb)
        w.symm_free(ob)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("numel", [3, 1000, 262144 + 8, 1_000_003])
def test_one_hop_collectives_on_ordinary_tensors(n, numel):
    """Ordinary `torch.empty` tensors (no symmetric heap, a different address on every rank, odd offsets): the
    automatic choice is the one-hop kernel, which learns where every rank's buffers are at its entry barrier."""
    from mintccl_b200.utils import stats
    w = world(n)
    stats.reset()
    for dtype in (torch.float16, torch.float32):
        pad = 16 // torch.empty((), dtype=dtype).element_size()
        src = rand(n, numel, dtype, seed0=41)
        ref = oracle_sum(src)
        # all-reduce out of place and in place; rank r's buffers start r elements into their allocation
        xs = [torch.empty(numel + n, device="cuda", dtype=dtype)[r:r + numel] for r in range(n)]
        ys = [torch.empty(numel + pad * n, device="cuda", dtype=dtype)[pad * r:pad * r + numel] for r in range(n)]
        for x, s_ in zip(xs, src):
            x.copy_(s_)
        w.allreduce(xs, out=ys, algo="direct" if numel * 4 <= 65536 else None)
        w.check()
        for y in ys:
            assert_sum_close(y, ref, dtype, nranks=n)
        for y in ys[1:]:
            assert torch.equal(y, ys[0])
        w.allreduce(xs, algo="direct")
        w.check()
        for x in xs:
            assert torch.equal(x, ys[0])
        # all-gather, in place convention and with a separate contribution
        bufs = [torch.zeros(n, numel, device="cuda", dtype=dtype) for _ in range(n)]
        for r in range(n):
            bufs[r][r].copy_(src[r])
        w.allgather(bufs)
        w.check()
        want = torch.stack(src)
        for b in bufs:
            assert torch.equal(b, want)
        for b in bufs:
            b.zero_()
        w.allgather(bufs, inp=src, algo="pull")
        w.check()
        for b in bufs:
            assert torch.equal(b, want)
        # reduce-scatter into a separate shard, all-to-all
        full = rand(n, n * numel, dtype, seed0=43)
        ins = [f.clone().view(n, numel) for f in full]
        outs = [torch.empty(numel, device="cuda", dtype=dtype) for _ in range(n)]
        w.reducescatter(ins, out=outs)
        w.check()
        ref2 = oracle_sum(full).view(n, numel)
        for r in range(n):
            assert_sum_close(outs[r], ref2[r], dtype, nranks=n)
        a2a = [torch.empty(n, numel, device="cuda", dtype=dtype) for _ in range(n)]
        w.alltoall(ins, a2a)
        w.check()
        for r in range(n):
            for p in range(n):
                assert torch.equal(a2a[r][p], full[p].view(n, numel)[r])
        # broadcast (views at an odd element offset: no 16-byte alignment on any rank) and reduce
        bs = [torch.empty(numel + 1, device="cuda", dtype=dtype)[1:] for _ in range(n)]
        for b, s_ in zip(bs, src):
            b.copy_(s_)
        w.broadcast(bs, root=n - 1, algo="direct")
        w.check()
        for b in bs:
            assert torch.equal(b, src[n - 1])
        rin = [s_.clone() for s_ in src]
        rout = [torch.zeros(numel, device="cuda", dtype=dtype) for _ in range(n)]
        w.reduce(rin, root=n // 2, out=rout, algo="direct")
        w.check()
        assert_sum_close(rout[n // 2], ref, dtype, nranks=n)
    seen = stats.snapshot(skip_idle=False)
    assert seen["direct"]["calls"] >= 16 and seen["ring_simple"]["calls"] == 0 and seen["ring_ll128"]["calls"] == 0


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("numel", [8, 1001, 300_000])
def test_reductions_into_another_element_type(n, numel):
    """16-bit input with fp32 output and fp32 input with 16-bit output: the one-hop kernels sum in fp32 and round
    once, into the output type.  With fp32 output and a fixed summation order the result is the oracle's, bit for
    bit."""
    w = world(n)
    for narrow in (torch.bfloat16, torch.float16):
        # widening
        src = rand(n, numel, narrow, seed0=51)
        ref = oracle_sum(src)
        o32 = [torch.zeros(numel, device="cuda", dtype=torch.float32) for _ in range(n)]
        w.allreduce(src, out=o32, algo="oneshot")          # every rank adds ranks 0..n-1 in that order, like the oracle
        w.check()
        for o in o32:
            assert torch.equal(o, ref.ref)
        for o in o32:
            o.zero_()
        w.allreduce(src, out=o32, algo="direct")           # two-shot: each rank starts the sum at itself
        w.check()
        for o in o32:
            assert_sum_close(o, ref, torch.float32, nranks=n)
            assert torch.equal(o, o32[0])
        full = rand(n, n * numel, narrow, seed0=53)
        shards = [torch.zeros(numel, device="cuda", dtype=torch.float32) for _ in range(n)]
        w.reducescatter([f.view(n, numel) for f in full], out=shards)
        w.check()
        ref2 = oracle_sum(full).view(n, numel)
        for r in range(n):
            assert_sum_close(shards[r], ref2[r], torch.float32, nranks=n)
        rout = [torch.zeros(numel, device="cuda", dtype=torch.float32) for _ in range(n)]
        w.reduce(src, root=n - 1, out=rout)
        w.check()
        assert_sum_close(rout[n - 1], ref, torch.float32, nranks=n)
        # narrowing
        src32 = rand(n, numel, torch.float32, seed0=55)
        ref32 = oracle_sum(src32)
        on = [torch.zeros(numel, device="cuda", dtype=narrow) for _ in range(n)]
        w.allreduce(src32, out=on, algo="oneshot")
        w.check()
        for o in on:
            assert torch.equal(o, ref32.ref.to(narrow))    # one rounding of the exact fp32 sum
        for o in on:
            o.zero_()
        w.allreduce(src32, out=on)
        w.check()
        for o in on:
            assert_sum_close(o, ref32, narrow, nranks=n)
        full32 = rand(n, n * numel, torch.float32, seed0=57)
        sn = [torch.zeros(numel, device="cuda", dtype=narrow) for _ in range(n)]
        w.reducescatter([f.view(n, numel) for f in full32], out=sn, algo="direct")
        w.check()
        ref4 = oracle_sum(full32).view(n, numel)
        for r in range(n):
            assert_sum_close(sn[r], ref4[r], narrow, nranks=n)
        w.reduce(src32, root=0, out=on, algo="direct1")
        w.check()
        assert_sum_close(on[0], ref32, narrow, nranks=n)
    with pytest.raises(ValueError):
        w.allreduce(rand(n, 64, torch.float16), out=[torch.zeros(64, device="cuda") for _ in range(n)], algo="ring")


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("numel", [8, 1001, 65536 + 24, 2_000_003])
def test_copy_engine_variants(n, numel):
    """All-gather, all-to-all and broadcast through bulk copies staged in shared memory (one thread per CTA drives
    the copy engine): bit-exact, any size, falling back to the threads' own copies when an address is not a
    multiple of 16."""
    w = world(n)
    for dtype, off in ((torch.float16, 0), (torch.float32, 0), (torch.float16, 1)):
        src = rand(n, numel, dtype, seed0=61)
        bufs = [torch.zeros(n * numel + off, device="cuda", dtype=dtype)[off:].view(n, numel) for _ in range(n)]
        for r in range(n):
            bufs[r][r].copy_(src[r])
        w.allgather(bufs, algo="bulk")
        w.check()
        want = torch.stack(src)
        for b in bufs:
            assert torch.equal(b, want)
        for b in bufs:
            b.zero_()
        w.allgather(bufs, inp=src, algo="bulk", nch=3)
        w.check()
        for b in bufs:
            assert torch.equal(b, want)
        for use_inp in (False, True):
            for r in range(n):
                bufs[r].zero_()
                bufs[r][r].copy_(src[r])
            w.allgather(bufs, inp=src if use_inp else None, algo="bulkpull")
            w.check()
            for b in bufs:
                assert torch.equal(b, want)
        full = rand(n, n * numel, dtype, seed0=63)
        ins = [f.view(n, numel) for f in full]
        outs = [torch.zeros(n * numel + off, device="cuda", dtype=dtype)[off:].view(n, numel) for _ in range(n)]
        w.alltoall(ins, outs, algo="bulk")
        w.check()
        for r in range(n):
            for p in range(n):
                assert torch.equal(outs[r][p], ins[p][r])
        for root in sorted({0, 1, n - 1}):
            bs = [torch.zeros(numel + off, device="cuda", dtype=dtype)[off:] for _ in range(n)]
            for b, s_ in zip(bs, src):
                b.copy_(s_)
            w.broadcast(bs, root=root, algo="bulk")
            w.check()
            for b in bs:
                assert torch.equal(b, src[root])


def test_direct_sendrecv_symmetric():
    w = world(4)
    bufs = w.symm_empty(1_000_000, torch.float32)
    for r, b in enumerate(bufs):
        b.fill_(float(r))
    bufs[1].copy_(torch.randn(1_000_000, device="cuda"))
    want = bufs[1].clone()
    for mode in ("sys", "weak", "bulk"):
        for pull in (True, False):
            for view in (slice(None), slice(3, 999_990)):     # the second one is not 16-byte aligned
                bufs[3].zero_()
                w.sendrecv_direct(1, 3, [b[view] for b in bufs], pull=pull, mode=mode, nctas=7)
                w.check()
                assert torch.equal(bufs[3][view], want[view]), (mode, pull)
    w.symm_free(bufs)


def test_bounded_wait_reports_instead_of_hanging():
    """A wait that nothing satisfies returns after the time limit with an error record; the context stays
    usable and the communicator reports the failure on the host."""
    from mintccl_b200 import Config, emulated
    from mintccl_b200.parallel.comm import CollectiveError
    cfg = Config.from_env(max_channels=2, num_blocks=2, buff_size=1 << 20, heap_bytes=64 << 20, scratch_bytes=1 << 20,
                          wait_timeout_ms=300)
    w = emulated(2, 0, cfg)
    w.test_wait_timeout()
    sts = [w.status(r) for r in range(2)]
    # the rank whose time limit ran out first reports the timeout (5) and raises the abort flag everywhere;
    # the other one may notice that flag first and report "aborted by a peer" (6)
    assert all(st.code in (5, 6) and st.where == 10 and st.abort == 1 for st in sts)
    assert any(st.code == 5 for st in sts)
    with pytest.raises(CollectiveError):
        w.check()
    x = torch.ones(8, device="cuda")
    assert float((x + 1).sum()) == 16.0  # the CUDA context still works
    w.close()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_mxfp8_block_scaled_reductions(n):
    """Block-scaled fp8 sum: fp32 accumulation over all ranks, one requantisation."""
    from mintccl_b200.ops import mxfp8 as mx
    w = world(n)
    numel = 32 * n * 50 + 32 * n * 3
    xs = [t * (10.0 ** (r % 3 - 1)) for r, t in enumerate(rand(n, numel, torch.float32, seed0=77))]
    q = [mx.quantize_mxfp8(x) for x in xs]
    # the torch quantiser round-trips within fp8 precision
    torch.testing.assert_close(mx.dequantize_mxfp8(*q[0]), xs[0], rtol=0.07, atol=1e-3)
    data, scale = w.symm_empty(numel, torch.uint8), w.symm_empty(numel // 32, torch.uint8)
    od, os_ = w.symm_empty(numel, torch.uint8), w.symm_empty(numel // 32, torch.uint8)
    for r in range(n):
        data[r].copy_(q[r][0])
        scale[r].copy_(q[r][1])
    ref = sum(mx.dequantize_mxfp8(*q[r]) for r in range(n))          # fp32 sum of the dequantised inputs
    ref_q = mx.dequantize_mxfp8(*mx.quantize_mxfp8(ref))               # ... quantised once
    mx.allreduce_mxfp8(w, data, scale, od, os_)
    w.check()
    for r in range(n):
        got = mx.dequantize_mxfp8(od[r], os_[r])
        torch.testing.assert_close(got, ref_q, rtol=0.07, atol=2e-3)
        assert torch.equal(od[r], od[0]) and torch.equal(os_[r], os_[0])
        assert torch.equal(os_[r], mx.quantize_mxfp8(ref)[1])         # identical block scales
    sd = [torch.empty(numel // n, device="cuda", dtype=torch.uint8) for _ in range(n)]
    ss = [torch.empty(numel // n // 32, device="cuda", dtype=torch.uint8) for _ in range(n)]
    mx.reducescatter_mxfp8(w, data, scale, sd, ss)
    w.check()
    per = numel // n
    for r in range(n):
        torch.testing.assert_close(mx.dequantize_mxfp8(sd[r], ss[r]), ref_q[r * per:(r + 1) * per], rtol=0.07, atol=2e-3)
    for t in (data, scale, od, os_):
        w.symm_free(t)


def test_one_rank_communicator_copies_at_any_alignment():
    """A communicator of one rank: every collective is a local copy (its own kernel when source and destination
    share the offset inside a 16-byte line, else the ring kernel); in place nothing runs."""
    import mintccl_b200
    from mintccl_b200 import Config
    comm = mintccl_b200.Communicator(config=Config.from_env(heap_bytes=256 << 20, max_channels=4))
    assert comm.world_size == 1
    from mintccl_b200.utils import stats
    stats.reset()
    base_in = torch.arange(0, 3_000_064, device="cuda", dtype=torch.int32).view(torch.uint8)
    base_out = torch.zeros(base_in.numel() + 64, device="cuda", dtype=torch.uint8)
    for nbytes, oi, oo in [(16, 0, 0), (1, 3, 3), (15, 1, 1), (4096 * 8 + 5, 7, 7), (1_000_003, 0, 0), (2_500_000, 13, 13),
                           (33, 5, 9), (100_001, 2, 0), (8 << 20, 0, 16)]:
        src = base_in[oi:oi + nbytes]
        dst = base_out[oo:oo + nbytes]
        base_out.zero_()
        comm.allgather(dst.view(1, -1), src)
        comm.check()
        assert torch.equal(dst, src), (nbytes, oi, oo)
        assert int(base_out[oo + nbytes:oo + nbytes + 32].sum()) == 0 and int(base_out[:oo].sum()) == 0, "wrote outside"
    seen = stats.snapshot()   # co-aligned pairs went to the copy kernel, the two others to the ring kernel
    assert seen["local_copy"]["calls"] >= 1 and seen["ring_simple"]["calls"] >= 1 and seen["local_copy"]["work"] >= 8 << 20
    x = torch.randn(1, 100_000, device="cuda", dtype=torch.float16)
    y = x.clone()
    comm.allgather(x)          # in place: nothing to do
    comm.reducescatter(x)
    comm.broadcast(x, 0)
    comm.reduce(x, 0)
    comm.check()
    assert torch.equal(x, y)
    out = torch.zeros(100_000, device="cuda", dtype=torch.float16)
    comm.reducescatter(x, out)
    comm.check()
    assert torch.equal(out, x[0])


def test_algorithm_names_are_checked_per_collective():
    w = world(2)
    bufs = [torch.zeros(2, 64, device="cuda", dtype=torch.float16) for _ in range(2)]
    with pytest.raises(ValueError, match="unknown algo"):
        w.reducescatter(bufs, algo="pull")          # an all-gather / broadcast variant only
    with pytest.raises(ValueError, match="unknown algo"):
        w.allgather(bufs, algo="oneshot")
    with pytest.raises(ValueError, match="unknown algo"):
        w.allreduce([b[0] for b in bufs], algo="nonsense")
    # a process-wide default that a collective does not have means "automatic" there
    old = w.cfg.algo
    try:
        w.cfg.algo = "ll"   # MINTCCL_ALGO=ll: the one-shot all-reduce; reduce-scatter has no such variant
        srcs = rand(2, 2 * 64, torch.float16)
        for b, s_ in zip(bufs, srcs):
            b.copy_(s_.view(2, 64))
        w.reducescatter(bufs)
        w.check()
        ref = oracle_sum(srcs).view(2, 64)
        for r in range(2):
            assert_sum_close(bufs[r][r], ref[r], torch.float16, 2)
    finally:
        w.cfg.algo = old


@pytest.mark.gpu
@pytest.mark.parametrize("n", [3, 4, 8])
@pytest.mark.parametrize("numel", [8, 1000, 65536 + 24, 1_500_000])
def test_reduce_with_a_summing_root(n, numel, algo="direct2"):
    """`algo="direct2"`: the other ranks sum their own inputs slice by slice into the root's output, chunk by chunk
    with a progress counter per chunk, and the root adds its own input as the chunks arrive.  Two roundings into the
    element type; every root; several chunks per CTA at the largest size; two calls in a row (the counters of the
    first call must not satisfy the waits of the second)."""
    w = world(n)
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        per16 = 16 // torch.empty((), dtype=dtype).element_size()
        ne = max(per16, numel // per16 * per16)                 # the byte count is a multiple of 16
        for root in sorted({0, 1, n - 1}):
            src = rand(n, ne, dtype, seed0=300 + root)
            outs = [torch.full((ne,), -7.0, device="cuda", dtype=dtype) for _ in range(n)]
            for rep in range(2):
                w.reduce(src, root=root, out=outs, algo=algo, nch=2 if numel > 1_000_000 else None)
                w.check()
                assert_sum_close(outs[root], oracle_sum(src), dtype, hops=2 if algo == "direct2" else 1, nranks=n)
                src = [s_ * 0.5 for s_ in src]                    # other values for the second call
            for r in range(n):
                if r != root:
                    assert bool((outs[r] == -7.0).all())         # only the root's output is written
