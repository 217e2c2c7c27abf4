"""Which native entry point, algorithm variant and CTA count every collective resolves to, checked without a GPU:
the communicator's own (slow-path) code runs on CPU tensors, with the native launch recorded instead of made and
a slab of host memory standing in for the symmetric heap."""
import pytest
import torch

from mintccl_b200 import Config
from mintccl_b200 import _native as N
from mintccl_b200.parallel.comm import Communicator


class Recorder(Communicator):
    def __init__(self, world=8, nvls=True, rank=0, **cfg):   # no device, no native communicator
        heap_mib = int(cfg.pop("_heap_mib", 64))
        cfg.setdefault("auto_register", False)      # ordinary tensors: FIFO ring unless a test shares them
        self.cfg = Config.from_env(**cfg)
        self.lib = N.lib()
        self._segs, self._seg_bases, self._unsharable, self.shared = {}, [], set(), []
        self.world_size, self.rank, self.nlocal, self.emulated, self.nvls = world, rank, 1, False, nvls
        self.device = 0
        self._plans, self._rec_key, self._pending = {}, None, []
        self.heap = torch.empty(heap_mib << 20, dtype=torch.uint8)
        self.heap_base, self.user_off, self.heap_bytes = [self.heap.data_ptr()], 0, self.heap.numel()
        self.ll_capacity = 200 << 10
        self.ring = list(range(world))
        self.calls = []
        self._next = 0

    def sym(self, numel, dtype=torch.float16):
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        off = (self._next + 255) // 256 * 256
        self._next = off + nbytes
        return self.heap[off:off + nbytes].view(dtype)

    def _lists(self, t):
        if t is None:
            return None
        return [t] if isinstance(t, torch.Tensor) else list(t)

    # stands in for CUDA IPC + the peers' registration services
    def _share_allocation(self, t):
        from mintccl_b200.parallel.comm import _Segment
        import bisect
        base = t.untyped_storage().data_ptr()
        seg = _Segment(base, t.untyped_storage().nbytes(), b"h" * 64,
                       [base if p == self.rank else 0x7000_0000_0000 + (p << 40) for p in range(self.world_size)], None)
        self._segs[base] = seg
        bisect.insort(self._seg_bases, base)
        self.shared.append(base)
        return seg

    def _run(self, fn, args):
        self.calls.append((fn.__name__, args))
        self._rec_key = None

    def last(self):
        name, a = self.calls[-1]
        if name == "mt_direct":
            return dict(fn=name, dtype=a[0], out_dtype=a[1], op=a[2], pub_in=None if a[5] is None else list(a[5]),
                        pub_out=None if a[6] is None else list(a[6]), mc_in=a[7], mc_out=a[8], nbytes=a[9], root=a[10],
                        variant=a[11], nvls=a[12], nctas=a[13])
        if name == "mt_ring":
            return dict(fn=name, proto=a[0], dtype=a[1], op=a[2], nbytes=a[5], root=a[6], spatial=a[7], nch=a[10])
        return dict(fn=name, args=a)


def test_allreduce_dispatch_by_size_and_memory():
    c = Recorder(world=8)
    small = torch.zeros(1000, dtype=torch.float16)
    c.allreduce(small)
    assert c.last()["fn"] == "mt_ll_allreduce"                      # <= MINTCCL_LL_MAX_BYTES: one-shot, any memory
    big_plain = torch.zeros(1 << 20, dtype=torch.float16)
    c.allreduce(big_plain)
    l = c.last()
    assert l["fn"] == "mt_ring" and l["op"] == N.OP_ALLREDUCE and l["proto"] == N.PROTO_SIMPLE   # ordinary tensor: ring
    x = c.sym(1 << 20)
    c.allreduce(x)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_ALLREDUCE and l["nvls"] == 1 and l["nctas"] <= c.cfg.nvls_ctas
    c2 = Recorder(world=2)
    y = c2.sym(1 << 20)
    c2.allreduce(y)
    assert c2.last()["fn"] == "mt_direct" and c2.last()["nvls"] == 0            # two ranks: plain peer loads
    c2.allreduce(y, algo="ring", proto="ll128")
    assert c2.last()["fn"] == "mt_ring" and c2.last()["proto"] == N.PROTO_LL128
    with pytest.raises(ValueError):
        c2.allreduce(torch.zeros(1 << 20, dtype=torch.float16), algo="direct")  # needs symmetric memory
    with pytest.raises(ValueError):
        c2.allreduce(y, algo="oneshot")                                          # one-shot cannot run in place
    with pytest.raises(TypeError):
        c2.allreduce(torch.zeros(64, dtype=torch.int32))                         # reductions: float types only


def test_allgather_reducescatter_dispatch():
    c = Recorder(world=4)
    buf = c.sym(4 * 65536).view(4, 65536)
    c.allgather(buf)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_ALLGATHER and l["nvls"] == 1 and l["nbytes"] == 65536 * 2
    c.allgather(buf, algo="pull")
    assert c.last()["variant"] == 1 and c.last()["nvls"] == 0
    plain = torch.zeros(4, 1000, dtype=torch.float32)
    c.allgather(plain, mode="spatial")
    l = c.last()
    assert l["fn"] == "mt_ring" and l["op"] == N.OP_ALLGATHER and l["spatial"] == 1 and l["nch"] % 4 == 0
    c.reducescatter(buf)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_REDUCESCATTER and l["nvls"] == 1
    c.reducescatter(plain)
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_REDUCESCATTER
    with pytest.raises(ValueError):
        c.allgather(torch.zeros(3, 10))                                          # first dimension = world size
    c.alltoall(buf, c.sym(4 * 65536).view(4, 65536))
    assert c.last()["fn"] == "mt_direct" and c.last()["op"] == N.DOP_ALLTOALL


def test_broadcast_and_reduce_dispatch():
    c = Recorder(world=8)
    x, out = c.sym(1 << 20), c.sym(1 << 20)
    c.broadcast(x, root=3)                                  # automatic, 2 MiB on 8 ranks: one hop through the switch
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_BROADCAST and l["nvls"] == 1 and l["variant"] == 2 and l["root"] == 3
    small = c.sym(1 << 17)
    c.broadcast(small, root=3)                              # 256 KiB: the LL128 chain (no barriers, short fill)
    l = c.last()
    assert l["fn"] == "mt_ring" and l["op"] == N.OP_BROADCAST and l["proto"] == N.PROTO_LL128 and l["root"] == 3
    c.broadcast(x, root=3, algo="ring")
    l = c.last()
    assert l["fn"] == "mt_ring" and l["op"] == N.OP_BROADCAST and l["proto"] == N.PROTO_SIMPLE and l["root"] == 3
    c.broadcast(x, root=3, algo="nvls")
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_BROADCAST and l["nvls"] == 1 and l["variant"] == 2 and l["root"] == 3
    c.broadcast(torch.zeros(100, dtype=torch.float16), root=1)
    assert c.last()["fn"] == "mt_ring" and c.last()["proto"] == N.PROTO_LL128    # small, ordinary memory: LL128 chain
    ordinary = torch.zeros(8 << 20, dtype=torch.float16)    # 16 MiB the peers cannot address (not shared): the chain
    c.broadcast(ordinary, root=1)
    assert c.last()["fn"] == "mt_ring" and c.last()["proto"] == N.PROTO_SIMPLE
    c.reduce(x, root=2, out=out)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_REDUCE and l["nvls"] == 1 and l["variant"] == 2
    c.reduce(small, root=2, out=c.sym(1 << 17))             # 256 KiB: a chain hop adds its own input, the switch is faster
    assert c.last()["fn"] == "mt_direct" and c.last()["nvls"] == 1
    tiny = c.sym(1 << 14)
    c.reduce(tiny, root=2, out=c.sym(1 << 14))              # 32 KiB: the LL128 chain
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_REDUCE and c.last()["proto"] == N.PROTO_LL128
    c.reduce(ordinary, root=2, out=torch.zeros(8 << 20, dtype=torch.float16))
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_REDUCE
    c.reduce(x, root=2, out=out, algo="nvls")
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_REDUCE and l["nvls"] == 1 and l["variant"] == 2
    c.reduce(x, root=2)                                                          # in place: the ring reduces in place
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_REDUCE
    with pytest.raises(ValueError):
        c.reduce(x, root=2, algo="direct")                                       # direct reduce needs a separate output
    c2 = Recorder(world=2, _heap_mib=320)
    y, o2 = c2.sym(1 << 20), c2.sym(1 << 20)
    c2.broadcast(y)
    assert c2.last()["fn"] == "mt_ring"                                          # 2 MiB: still the chain
    big, bigo = c2.sym(32 << 20, torch.float32), c2.sym(32 << 20, torch.float32)  # 128 MiB on two ranks: one hop
    c2.broadcast(big)
    assert c2.last()["fn"] == "mt_direct" and c2.last()["nvls"] == 0 and c2.last()["variant"] == 1   # the receiver pulls
    c2.reduce(big, out=bigo)
    assert c2.last()["fn"] == "mt_direct" and c2.last()["variant"] == 0
    c2.broadcast(y, algo="direct")
    assert c2.last()["fn"] == "mt_direct" and c2.last()["variant"] == 0          # two ranks: the root pushes once


def test_one_rank_world_always_takes_the_copy_path():
    c = Recorder(world=1)
    x, out = c.sym(4096), c.sym(4096)
    c.allreduce(x, out=out)
    assert c.last()["fn"] == "mt_ring" and c.last()["proto"] == N.PROTO_SIMPLE   # the native side turns it into a copy
    n0 = len(c.calls)
    c.broadcast(x)
    assert len(c.calls) == n0                                                    # nothing to do


def test_tuning_table_overrides_the_policy_only_where_it_applies(tmp_path, monkeypatch):
    from mintccl_b200.tuning import TuningTable
    table = TuningTable([
        {"collective": "allreduce", "nranks": 8, "max_bytes": 1 << 20, "algo": "direct", "nch": 48},
        {"collective": "allreduce", "nranks": 8, "max_bytes": 1 << 26, "algo": "nvls", "nch": 16},
        {"collective": "broadcast", "nranks": 8, "max_bytes": 1 << 30, "algo": "ring", "nch": 64},
        {"collective": "allgather", "nranks": 8, "max_bytes": 1 << 30, "symmetric": False, "algo": "ring", "nch": 24},
    ])
    c = Recorder(world=8)
    c._tuning = table
    x = c.sym(1 << 18)                                   # 512 KiB, symmetric
    c.allreduce(x)
    assert (c.last()["fn"], c.last()["nvls"], c.last()["nctas"]) == ("mt_direct", 0, 48)
    y = c.sym(1 << 21)                                   # 4 MiB
    c.allreduce(y)
    assert (c.last()["nvls"], c.last()["nctas"]) == (1, 16)
    c.allreduce(y, nch=8)                                # the caller's own choice stands
    assert c.last()["nctas"] == 8
    c.allreduce(y, algo="ring")
    assert c.last()["fn"] == "mt_ring"
    c.allreduce(torch.zeros(1 << 20, dtype=torch.float16))   # ordinary memory: the symmetric rows do not apply
    assert c.last()["fn"] == "mt_ring"
    odd = c.sym((1 << 21) + 4)[: (1 << 21) + 4]          # byte count not a multiple of 16: the NVLS row is skipped
    c.allreduce(odd)
    assert c.last()["fn"] == "mt_direct" and c.last()["nvls"] == 0
    c.broadcast(y, root=1)
    assert c.last()["fn"] == "mt_ring" and c.last()["nch"] == 64
    plain = torch.zeros(8, 4096, dtype=torch.float32)
    c.allgather(plain)
    assert c.last()["fn"] == "mt_ring" and c.last()["nch"] == 24
    c4 = Recorder(world=4)
    c4._tuning = table                                    # no rows for 4 ranks: built-in policy
    z = c4.sym(1 << 18)
    c4.allreduce(z)
    assert c4.last()["nvls"] == 1
    # file round trip and the environment variable
    path = str(tmp_path / "tuning.json")
    table.dump(path)
    monkeypatch.setenv("MINTCCL_TUNING_FILE", path)
    again = TuningTable.from_env()
    assert again.lookup("allreduce", 8, 1 << 19) == ("direct", 48) and again.lookup("allreduce", 8, 1 << 27) is None
    monkeypatch.setenv("MINTCCL_TUNING_FILE", "none")
    assert TuningTable.from_env() is None                 # switched off: the built-in policy alone
    monkeypatch.delenv("MINTCCL_TUNING_FILE")
    shipped = TuningTable.from_env()                      # unset: the table measured on HGX B200 that ships with the package
    assert shipped is not None and shipped.lookup("allgather", 8, 64 << 20, True)[0] == "bulk"
    assert shipped.lookup("broadcast", 8, 64 << 20, True) is None   # rooted collectives: tuned from fenced rows only
    assert shipped.lookup("allreduce", 3, 1 << 20, True) is None    # no rows for rank counts that were not measured


def test_tuning_table_from_sweep_rows(tmp_path):
    from mintccl_b200.tuning import TuningTable
    rows = []
    for nbytes, best in ((1 << 10, ("ll", 0)), (1 << 14, ("ll", 0)), (1 << 20, ("direct", 64)), (1 << 24, ("nvls", 32)), (1 << 28, ("nvls", 32))):
        for algo, ctas in (("ll", 0), ("direct", 64), ("nvls", 32), ("ring", 64)):
            rows.append({"collective": "allreduce", "bytes": nbytes, "impl": "mintccl", "algo": algo, "ctas": ctas,
                         "us": 10.0 if (algo, ctas) == best else 20.0, "n": 8})
        rows.append({"collective": "allreduce", "bytes": nbytes, "impl": "nccl", "algo": "nccl", "ctas": 0, "us": 1.0, "n": 8})
    t = TuningTable.from_sweep(rows)
    got = t.rows[("allreduce", 8, True)]
    assert [(r["algo"], r["nch"]) for r in got] == [("ll", None), ("direct", 64), ("nvls", 32)]     # neighbours merged, NCCL ignored
    assert t.lookup("allreduce", 8, 1 << 12) == ("ll", None)
    assert t.lookup("allreduce", 8, 1 << 20) == ("direct", 64)
    assert t.lookup("allreduce", 8, 1 << 26) == ("nvls", 32)
    assert t.lookup("allreduce", 8, 1 << 29) is None and t.lookup("allreduce", 4, 1 << 20) is None
    # boundaries sit between the measured sizes (geometric mean)
    assert got[0]["max_bytes"] == int((float(1 << 14) * (1 << 20)) ** 0.5)
    # broadcast / reduce on more than two ranks: back-to-back rows rate the barrier-free chain by its steady state, so
    # only fenced rows count
    chain = [{"collective": "broadcast", "bytes": 1 << 26, "impl": "mintccl", "algo": a_, "ctas": 0, "us": us, "n": 8,
              "sync": sync} for a_, us, sync in (("ring", 10.0, False), ("nvls", 20.0, False), ("auto", 20.0, False))]
    assert ("broadcast", 8, True) not in TuningTable.from_sweep(chain).rows
    fenced = [dict(r, sync=True, us={"ring": 60.0, "nvls": 20.0, "auto": 60.0}[r["algo"]]) for r in chain]
    t2 = TuningTable.from_sweep(chain + fenced)
    assert t2.lookup("broadcast", 8, 1 << 26) == ("nvls", None)
    assert t2.lookup("broadcast", 8, 1 << 20) is None       # a sweep says nothing below its smallest size
    path2 = str(tmp_path / "t2.json")
    t2.dump(path2)
    assert TuningTable.load(path2).lookup("broadcast", 8, 1 << 20) is None and TuningTable.load(path2).lookup("broadcast", 8, 1 << 26)
    two = [dict(r, n=2) for r in chain]
    assert TuningTable.from_sweep(two).lookup("broadcast", 2, 1 << 26) == ("ring", None)   # one link: nothing to fill


def test_emulated_world_takes_one_tensor_per_rank():
    """The single-GPU emulation passes lists (one tensor per emulated rank) through the same selection code."""
    n = 4
    c = Recorder(world=n)
    c.emulated, c.nlocal = True, n
    c.heap_base = [c.heap.data_ptr()] * n           # every emulated rank's heap: same offsets
    xs = [c.sym(1 << 16) for _ in range(n)]
    # one address space: every tensor is addressable by every emulated rank, wherever it lies, so the one-hop
    # kernels run and announce the local pointers themselves (no per-peer views)
    c.allreduce(xs)
    assert c.last()["fn"] == "mt_direct" and c.last()["nctas"] <= 148 // n and c.last()["pub_in"] is None
    c.allreduce(xs, algo="ring")
    assert c.last()["fn"] == "mt_ring" and c.last()["nch"] <= 148 // n
    bufs = [torch.zeros(n, 1024, dtype=torch.float16) for _ in range(n)]
    c.allgather(bufs)
    assert c.last()["fn"] == "mt_direct" and c.last()["op"] == N.DOP_ALLGATHER
    c.allgather(bufs, algo="ring")
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_ALLGATHER
    c.reducescatter(bufs, out=[torch.zeros(1024, dtype=torch.float16) for _ in range(n)], algo="ring")
    assert c.last()["op"] == N.OP_REDUCESCATTER
    c.broadcast([torch.zeros(100) for _ in range(n)], root=2)
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_BROADCAST and c.last()["root"] == 2   # small: LL128 chain
    c.reduce([torch.zeros(100) for _ in range(n)], root=1, out=[torch.zeros(100) for _ in range(n)])
    assert c.last()["op"] == N.OP_REDUCE


def test_ring_and_routes_follow_the_topology(tmp_path, monkeypatch):
    """Default: the uniform NVSwitch topology (direct routes).  MINTCCL_TOPO_FILE: a cached link map, here the
    hybrid cube mesh of an 8-GPU board without a switch, gives a ring over existing links only and multi-hop
    routes between GPUs that share no link; MINTCCL_RING / MINTCCL_RING_SEED / MINTCCL_ROUTE still override."""
    import json
    from mintccl_b200.parallel.rendezvous import SingleControl
    for k in ("MINTCCL_TOPO_FILE", "MINTCCL_TOPO_DISCOVER", "MINTCCL_RING", "MINTCCL_RING_SEED", "MINTCCL_ROUTE"):
        monkeypatch.delenv(k, raising=False)
    c = Recorder(world=8)
    c.control = SingleControl()
    assert sorted(c._choose_ring()) == list(range(8)) and c.route(0, 5) == [0, 5]
    # DGX-1 style hybrid cube mesh: two fully connected quads {0..3}, {4..7} plus the links i <-> i + 4
    links = {i: [] for i in range(8)}
    for q in (0, 4):
        for a in range(q, q + 4):
            for b in range(q, q + 4):
                if a != b:
                    links[a].append((b, 50.0))
    for i in range(4):
        links[i].append((i + 4, 25.0))
        links[i + 4].append((i, 25.0))
    path = tmp_path / "topo.json"
    path.write_text(json.dumps({str(k): v for k, v in links.items()}))
    monkeypatch.setenv("MINTCCL_TOPO_FILE", str(path))
    m = Recorder(world=8)
    m.control = SingleControl()
    ring = m._choose_ring()
    assert sorted(ring) == list(range(8))
    has = lambda a, b: any(d == b for d, _ in links[a])  # noqa: E731
    assert all(has(ring[i], ring[(i + 1) % 8]) for i in range(8)), ring       # every hop of the ring is a real link
    r = m.route(0, 5)
    assert r[0] == 0 and r[-1] == 5 and len(r) == 3 and all(has(a, b) for a, b in zip(r, r[1:]))   # via 1 or 4
    monkeypatch.setenv("MINTCCL_RING", "7,6,5,4,3,2,1,0")
    assert m._choose_ring() == [7, 6, 5, 4, 3, 2, 1, 0]
    monkeypatch.delenv("MINTCCL_RING")
    monkeypatch.setenv("MINTCCL_RING_SEED", "3")
    assert sorted(m._choose_ring()) == list(range(8))
    m.ring = [0, 1, 2, 3, 7, 6, 5, 4]
    monkeypatch.setenv("MINTCCL_ROUTE", "ring")
    assert m.route(2, 6) == [2, 3, 7, 6]


def test_ordinary_tensors_take_the_one_hop_kernels_once_shared():
    """With automatic registration an ordinary tensor is shared with the peers on first use (here: recorded) and the
    call goes to the one-hop kernel with one announced address per peer; heap tensors announce a tagged offset."""
    c = Recorder(world=8, auto_register=True, rank=3)
    x, y = torch.zeros(1 << 20, dtype=torch.float16), torch.zeros(1 << 20, dtype=torch.float16)
    c.allreduce(x, out=y)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_ALLREDUCE and l["nvls"] == 0 and l["variant"] == 0
    assert len(c.shared) == 2 and l["pub_in"][3] == x.data_ptr() and l["pub_out"][3] == y.data_ptr()
    assert l["pub_in"][5] == 0x7000_0000_0000 + (5 << 40) + (x.data_ptr() - x.untyped_storage().data_ptr())
    c.allreduce(x, out=y)
    assert len(c.shared) == 2                                      # the allocation is shared once
    h = c.sym(1 << 20)
    c.allreduce(h, algo="direct")
    l = c.last()
    off = h.data_ptr() - c.heap.data_ptr()
    assert l["pub_in"] == [(1 << 63) | off] * 8 and l["pub_out"] == [(1 << 63) | off] * 8
    buf = torch.zeros(8, 4096, dtype=torch.float32)
    c.allgather(buf)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_ALLGATHER and l["variant"] == 0 and l["pub_in"] == [0] * 8
    c.allgather(buf, algo="pull")                                  # the contribution is row `rank` of the buffer
    l = c.last()
    assert l["variant"] == 1 and l["pub_in"][3] == buf.data_ptr() + 3 * 4096 * 4 and l["pub_out"] == [0] * 8
    c.reducescatter(buf, out=torch.zeros(4096, dtype=torch.float32))
    assert c.last()["fn"] == "mt_direct" and c.last()["pub_out"] == [0] * 8    # the shard stays local: not shared
    large = torch.zeros(8 << 20, dtype=torch.float16)              # automatic, 16 MiB: pull + replicate, plain stores
    c.broadcast(large, root=1)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_BROADCAST and l["nvls"] == 0 and l["variant"] == 2
    hl = c.sym(8 << 20)                                            # the same on the heap: no multicast from 8 MiB on
    c.broadcast(hl, root=1)
    assert c.last()["fn"] == "mt_direct" and c.last()["nvls"] == 0 and c.last()["variant"] == 2
    c.broadcast(torch.zeros(1 << 20, dtype=torch.float16), root=1)  # 2 MiB: register-staged pull + replicate
    assert c.last()["fn"] == "mt_direct" and c.last()["nvls"] == 0 and c.last()["variant"] == 2
    c.reduce(large, root=2, out=torch.zeros(8 << 20, dtype=torch.float16))     # the others sum a slice each
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_REDUCE and l["nvls"] == 0 and l["variant"] == 3
    huge = torch.zeros(32 << 20, dtype=torch.float16)              # 64 MiB: nobody reads the root, which adds its own input
    c.reduce(huge, root=2, out=torch.zeros(32 << 20, dtype=torch.float16))
    assert c.last()["fn"] == "mt_direct" and c.last()["variant"] == 5
    c.reduce(large, root=2)                                        # in place: the chain
    assert c.last()["fn"] == "mt_ring"
    c.reduce(large, root=2, out=torch.zeros(8 << 20, dtype=torch.float16), algo="direct2")   # the root sums its own input
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_REDUCE and l["variant"] == 5 and l["nvls"] == 0
    with pytest.raises(ValueError):
        c.reduce(large, root=2, algo="direct2")                    # needs a separate output
    with pytest.raises(ValueError):
        c.reduce(large[:1001], root=2, out=torch.zeros(1001, dtype=torch.float16), algo="direct2")   # 2002 bytes
    big = torch.zeros(1 << 20, dtype=torch.float16)
    c.broadcast(big, root=2, algo="direct")
    assert c.last()["fn"] == "mt_direct" and c.last()["variant"] == 2 and c.last()["nvls"] == 0
    c.reduce(big, root=2, out=torch.zeros(1 << 20, dtype=torch.float16), algo="direct")
    assert c.last()["fn"] == "mt_direct" and c.last()["variant"] == 3           # the other ranks sum, the root receives
    c.broadcast(big[: 1 << 17], root=2)                            # 256 KiB: the LL128 chain, any memory
    assert c.last()["fn"] == "mt_ring"
    with pytest.raises(ValueError):
        c.allreduce(x, algo="nvls")                                # the multicast alias covers the heap only


def test_unaligned_views_never_reach_vector_only_paths():
    """A heap view whose address is not a multiple of 16 takes the plain pull + replicate broadcast (any alignment
    in the kernel) and never the multicast variant."""
    c = Recorder(world=4)
    x = c.sym(1 << 20)
    c.broadcast(x[4:], root=0, algo="direct")                      # 8 bytes into a 256-byte aligned allocation
    l = c.last()
    assert l["fn"] == "mt_direct" and l["nvls"] == 0 and l["variant"] == 2
    with pytest.raises(ValueError):
        c.broadcast(x[4:], root=0, algo="nvls")


def test_output_size_and_type_are_checked_before_launch():
    c = Recorder(world=4)
    x = c.sym(1 << 16)
    n0 = len(c.calls)
    with pytest.raises(ValueError):
        c.allreduce(x, out=c.sym(1 << 15))                         # short output
    with pytest.raises(ValueError):
        c.reduce(x, root=0, out=c.sym((1 << 16) + 8))
    with pytest.raises(ValueError):
        c.reducescatter(x.view(4, -1), out=c.sym(1 << 13))         # the shard has 1 << 14 elements
    with pytest.raises(ValueError):
        c.allreduce(x, out=c.sym(1 << 16, torch.bfloat16))         # fp16 -> bf16 is not a supported conversion
    with pytest.raises(ValueError):
        c.allgather(c.sym(4 << 10).view(4, -1), inp=c.sym(1 << 10, torch.float32))
    assert len(c.calls) == n0                                      # nothing was launched
    # a different out of the same address but another size is a different plan
    k1 = c._key("allreduce", x, c.heap[:64].view(torch.float16))
    k2 = c._key("allreduce", x, c.heap[:128].view(torch.float16))
    assert k1 != k2


def test_reductions_into_another_element_type():
    c = Recorder(world=8)
    x = c.sym(1 << 20, torch.bfloat16)
    o32 = c.sym(1 << 20, torch.float32)
    c.allreduce(x, out=o32)
    l = c.last()
    assert l["fn"] == "mt_direct" and (l["dtype"], l["out_dtype"]) == (N.DT_BF16, N.DT_F32) and l["nvls"] == 0
    assert l["nbytes"] == (1 << 20) * 2                            # counted in input bytes
    f = c.sym(1 << 18, torch.float32)
    c.reducescatter(f.view(8, -1), out=c.sym(1 << 15, torch.float16))
    l = c.last()
    assert (l["dtype"], l["out_dtype"], l["op"]) == (N.DT_F32, N.DT_F16, N.DOP_REDUCESCATTER)
    c.reduce(x, root=1, out=o32)
    assert c.last()["variant"] == 3 and c.last()["out_dtype"] == N.DT_F32
    with pytest.raises(ValueError):
        c.allreduce(x, out=o32, algo="ring")
    small = c.sym(64, torch.float16)
    c.allreduce(small, out=c.sym(64, torch.float32))               # small and converting: the one-hop kernel, not LL
    assert c.last()["fn"] == "mt_direct"


def test_tuning_table_ignores_noise_and_keeps_memory_kinds_apart():
    """A named algorithm needs a margin over the automatic choice, an explicit CTA count needs 3 % over the algorithm's own
    default, ring channel counts above the FIFO layout are the same thing, and rows measured on ordinary tensors do not
    apply to heap tensors."""
    from mintccl_b200.tuning import TuningTable

    def row(algo, ctas, us, nbytes=1 << 24, memory="heap", coll="allgather"):
        return {"collective": coll, "bytes": nbytes, "impl": "mintccl", "algo": algo, "ctas": ctas, "us": us, "n": 8, "memory": memory}

    rows = [row("auto", 0, 100.0), row("bulk", 0, 97.0), row("bulk", 64, 96.0),            # 3-4 % better: noise, no row
            row("auto", 0, 100.0, 1 << 26), row("bulk", 0, 80.0, 1 << 26), row("bulk", 128, 79.0, 1 << 26),   # bulk, default CTAs
            row("auto", 0, 100.0, 1 << 28), row("ring", 64, 70.0, 1 << 28), row("ring", 128, 69.9, 1 << 28),
            row("auto", 0, 50.0, 1 << 26, "ordinary"), row("direct", 64, 40.0, 1 << 26, "ordinary")]
    t = TuningTable.from_sweep(rows)
    assert t.lookup("allgather", 8, 1 << 24, True) == ("auto", None)
    assert t.lookup("allgather", 8, 1 << 26, True) == ("bulk", None)
    assert t.lookup("allgather", 8, 1 << 28, True) == ("ring", 64)
    assert t.lookup("allgather", 8, 1 << 26, False) == ("direct", 64)
    assert t.lookup("allgather", 8, 1 << 28, False) is None
