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
        self.cfg = Config.from_env(**cfg)
        self.lib = N.lib()
        self.world_size, self.rank, self.nlocal, self.emulated, self.nvls = world, rank, 1, False, nvls
        self.device = 0
        self._plans, self._rec_key, self._pending = {}, None, []
        self.heap = torch.zeros(64 << 20, dtype=torch.uint8)
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

    def _run(self, fn, args):
        self.calls.append((fn.__name__, args))
        self._rec_key = None

    def last(self):
        name, a = self.calls[-1]
        if name == "mt_direct":
            return dict(fn=name, dtype=a[0], op=a[1], nbytes=a[6], root=a[7], variant=a[8], nvls=a[9], nctas=a[10])
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
    c.broadcast(x, root=3)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_BROADCAST and l["nvls"] == 1 and l["variant"] == 2 and l["root"] == 3
    c.broadcast(torch.zeros(100, dtype=torch.float16), root=1)
    assert c.last()["fn"] == "mt_ring" and c.last()["proto"] == N.PROTO_LL128    # small, ordinary memory: LL128 chain
    c.reduce(x, root=2, out=out)
    l = c.last()
    assert l["fn"] == "mt_direct" and l["op"] == N.DOP_REDUCE and l["nvls"] == 1 and l["variant"] == 2
    c.reduce(x, root=2)                                                          # in place: the ring reduces in place
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_REDUCE
    with pytest.raises(ValueError):
        c.reduce(x, root=2, algo="direct")                                       # direct reduce needs a separate output
    c2 = Recorder(world=2)
    y, o2 = c2.sym(1 << 20), c2.sym(1 << 20)
    c2.broadcast(y)
    assert c2.last()["fn"] == "mt_direct" and c2.last()["nvls"] == 0 and c2.last()["variant"] == 0   # root pushes once
    c2.reduce(y, out=o2)
    assert c2.last()["fn"] == "mt_direct" and c2.last()["variant"] == 0


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
    monkeypatch.delenv("MINTCCL_TUNING_FILE")
    assert TuningTable.from_env() is None


def test_tuning_table_from_sweep_rows():
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


def test_emulated_world_takes_one_tensor_per_rank():
    """The single-GPU emulation passes lists (one tensor per emulated rank) through the same selection code."""
    n = 4
    c = Recorder(world=n)
    c.emulated, c.nlocal = True, n
    c.heap_base = [c.heap.data_ptr()] * n           # every emulated rank's heap: same offsets
    xs = [c.sym(1 << 16) for _ in range(n)]
    # the ranks' tensors sit at different offsets of one slab here, so they do not count as symmetric: ring
    c.allreduce(xs)
    assert c.last()["fn"] == "mt_ring" and c.last()["nch"] <= 148 // n
    bufs = [torch.zeros(n, 1024, dtype=torch.float16) for _ in range(n)]
    c.allgather(bufs)
    assert c.last()["fn"] == "mt_ring" and c.last()["op"] == N.OP_ALLGATHER
    c.reducescatter(bufs, out=[torch.zeros(1024, dtype=torch.float16) for _ in range(n)])
    assert c.last()["op"] == N.OP_REDUCESCATTER
    c.broadcast([torch.zeros(100) for _ in range(n)], root=2)
    assert c.last()["op"] == N.OP_BROADCAST and c.last()["root"] == 2
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
