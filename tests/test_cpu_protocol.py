"""CPU-only tests of the protocol layer: LL128 wire format against a NumPy oracle, the index arithmetic
shared by kernels and host, the host-side simulator (deadlock-freedom, 1,000 back-to-back operations,
fault injection) and descriptor passing between processes."""
import ctypes as C
import multiprocessing as mp
import os

import numpy as np
import pytest

from mintccl_b200 import _native as N
from mintccl_b200.ops import ll128_ref as ll

lib = N.lib()
lib.mt_sched_split.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
lib.mt_sched_ll128_lines.restype = C.c_uint64
lib.mt_sched_ll128_lines.argtypes = [C.c_uint64]
lib.mt_sched_ll128_line_of.restype = C.c_uint32
lib.mt_sched_ll128_line_of.argtypes = [C.c_uint32, C.c_uint32]
lib.mt_sim_run.restype = C.c_int
lib.mt_sim_run.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int,
                           C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_uint64, C.c_uint32,
                           C.POINTER(N.MtStatus)]


def sim(n, nch, proto, op, count, root=0, spatial=0, chain=None, ring=None, iters=1, jitter=0, dead=-1, timeout_ms=4000,
        seed=1, slot_bytes=4096, slots=2):
    chain = chain or []
    ch = (C.c_int * 9)(*chain)
    rg = (C.c_int * 8)(*(ring or list(range(n))))
    st = (N.MtStatus * 8)()
    rc = lib.mt_sim_run(n, nch, proto, op, count, root, spatial, ch, len(chain), rg, iters, jitter, dead, timeout_ms, seed,
                        slot_bytes, slots, st)
    return rc, st


@pytest.mark.parametrize("nbytes", [1, 8, 119, 120, 121, 127, 128, 129, 239, 240, 241, 1919, 1920, 1921, 5000])
def test_ll128_pack_unpack_roundtrip(nbytes):
    rng = np.random.default_rng(nbytes)
    payload = rng.integers(0, 256, nbytes, dtype=np.uint8).tobytes()
    wire = ll.pack(payload, flag=77)
    assert len(wire) % ll.WARP_WIRE == 0
    assert ll.valid(wire, nbytes, 77) and not ll.valid(wire, nbytes, 78)
    assert ll.unpack(wire, nbytes) == payload
    assert ll.wire_lines(min(nbytes, ll.WARP_PAYLOAD)) == lib.mt_sched_ll128_lines(min(nbytes, ll.WARP_PAYLOAD))


def test_ll128_geometry_matches_native():
    seen = set()
    for pair in range(8):
        for half in range(2):
            a, b = ll.line_of(pair, half), lib.mt_sched_ll128_line_of(pair, half)
            assert a == b
            seen.add(a)
    assert seen == set(range(16))  # the 16 lines of a warp chunk, each used once
    assert ll.efficiency() == 0.9375
    # bytes [120, 128) of a pair travel in the flag lane of the second line: 121..128 bytes need two lines
    assert [ll.wire_lines(x) for x in (0, 1, 120, 121, 128, 240, 241)] == [0, 1, 1, 2, 2, 2, 3]


def test_split_covers_message_without_gaps():
    for total in (0, 1, 127, 128, 129, 4096, 1_000_003, (1 << 30) + 5):
        for parts in (1, 3, 16, 148):
            prev = 0
            for i in range(parts):
                lo, hi = C.c_uint64(), C.c_uint64()
                lib.mt_sched_split(total, parts, i, 128, C.byref(lo), C.byref(hi))
                assert lo.value == prev and hi.value >= lo.value
                if hi.value < total:
                    assert hi.value % 128 == 0
                prev = hi.value
            assert prev == total


def test_rooted_one_hop_split_covers_every_byte_once():
    """The index arithmetic of the rooted one-hop kernels (broadcast pull + replicate, reduce with the other ranks
    summing): the message is split over the CTAs (128-byte boundaries), each CTA's range over the n - 1 ranks that are
    not the root (128-byte boundaries), each sub-slice into 256 KiB chunks.  Every byte belongs to exactly one
    (CTA, rank, chunk), every chunk starts on a 16-byte boundary for a byte count that is a multiple of 16, and the root
    and each producer count the same number of chunks per sub-slice."""
    def split(total, parts, i, align):
        lo, hi = C.c_uint64(), C.c_uint64()
        lib.mt_sched_split(total, parts, i, align, C.byref(lo), C.byref(hi))
        return lo.value, hi.value
    chunk = 256 << 10
    for n in (3, 4, 8):
        for total in (16, 2000, 65536 + 48, 3_000_000 - 3_000_000 % 16, 64 << 20):
            for ncta in (1, 2, 37, 128):
                covered = 0
                for cta in range(ncta):
                    rlo, rhi = split(total, ncta, cta, 128)
                    prev = 0
                    for idx in range(n - 1):
                        lo, hi = split(rhi - rlo, n - 1, idx, 128)
                        assert lo == prev and hi >= lo
                        prev = hi
                        nchunks = -(-(hi - lo) // chunk)
                        for k in range(nchunks):
                            clo, chi = lo + k * chunk, min(lo + (k + 1) * chunk, hi)
                            assert (rlo + clo) % 16 == 0 and (chi - clo) % 16 == 0 and chi > clo
                            covered += chi - clo
                    assert prev == rhi - rlo
                assert covered == total


def test_ring_schedule_visits_every_shard_once():
    lib.mt_sched_ag_shard.restype = C.c_int
    lib.mt_sched_rs_shard.restype = C.c_int
    for n in (2, 3, 4, 8):
        for q in range(n):
            assert sorted(lib.mt_sched_ag_shard(q, j, n) for j in range(n)) == list(range(n))
            assert sorted(lib.mt_sched_rs_shard(q, j, n) for j in range(n)) == list(range(n))
            assert lib.mt_sched_ag_shard(q, 0, n) == q            # all-gather starts with the own shard
            assert lib.mt_sched_rs_shard(q, n - 1, n) == q        # reduce-scatter ends with the own shard
            # what q sends at step j is what q+1 receives at step j+1
            for j in range(n - 1):
                assert lib.mt_sched_ag_shard(q, j, n) == lib.mt_sched_ag_shard((q + 1) % n, j + 1, n)
                assert lib.mt_sched_rs_shard(q, j, n) == lib.mt_sched_rs_shard((q + 1) % n, j + 1, n)


OPS = {"sendrecv": 0, "broadcast": 1, "reduce": 2, "allgather": 3, "reducescatter": 4, "allreduce": 5}


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("proto", [0, 1])
@pytest.mark.parametrize("op", ["broadcast", "reduce", "allgather", "reducescatter", "allreduce"])
def test_simulated_collectives_all_sizes(n, proto, op):
    for count in (1, 30, 31, 32, 61, 1000, 5003):
        for spatial in ((0, 1) if op in ("allgather", "reducescatter") else (0,)):
            nch = n if spatial else 3
            rc, st = sim(n, nch, proto, OPS[op], count, root=n - 1, spatial=spatial, jitter=20, seed=count)
            assert rc == 0, (op, count, spatial, [(s.code, s.where) for s in st[:n]])


def test_simulated_multihop_thousand_back_to_back():
    """rank 0 -> 4 through 1, 2, 3 on a permuted ring, 1,000 operations in a row on two-slot FIFOs:
    counters keep growing, nothing is cleared, nothing deadlocks (the reference documents a deadlock on
    eight GPUs, README.md:62-63)."""
    for proto in (0, 1):
        rc, st = sim(8, 2, proto, OPS["sendrecv"], 600, chain=[0, 1, 2, 3, 4], iters=1000, jitter=0, slot_bytes=2048)
        assert rc == 0, [(s.code, s.where, s.step) for s in st[:8]]


def test_simulated_allreduce_eight_ranks_many_iterations_with_jitter():
    for proto in (0, 1):
        rc, _ = sim(8, 4, proto, OPS["allreduce"], 7001, iters=60, jitter=30, ring=[3, 1, 4, 0, 5, 7, 2, 6], slot_bytes=2048)
        assert rc == 0


@pytest.mark.parametrize("proto", [0, 1])
def test_injected_dead_rank_is_reported_not_hung(proto):
    """A rank that never joins: every rank that depends on it gives up after its time limit, records who was
    waiting for what, and raises the abort flag on its peers.  Nothing spins forever."""
    rc, st = sim(4, 2, proto, OPS["allreduce"], 4000, dead=2, timeout_ms=300)
    assert rc == 2
    codes = [st[r].code for r in range(4)]
    assert codes[2] == 0                      # the dead rank reported nothing
    assert all(c in (1, 2, 3, 6) for i, c in enumerate(codes) if i != 2) and any(c in (1, 2, 3) for c in codes)
    assert all(st[r].abort == 1 for r in range(4))


def _fd_child(name, q):
    from mintccl_b200 import _native as N2
    L = N2.lib()
    r, w = os.pipe()
    os.write(w, b"hello from child")
    assert L.mt_fd_send(name.encode(), 42, r, 5000) == 0
    q.put("sent")


def test_fd_passing_between_processes():
    name = f"mintccl-test-{os.getpid()}"
    sock = lib.mt_fd_listen(name.encode())
    assert sock >= 0
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_fd_child, args=(name, q))
    p.start()
    tag = C.c_int(-1)
    fd = lib.mt_fd_accept(sock, C.byref(tag), 20000)
    assert fd >= 0 and tag.value == 42
    assert os.read(fd, 64) == b"hello from child"
    os.close(fd)
    assert q.get(timeout=20) == "sent"
    p.join(20)
    lib.mt_fd_close(sock)
    assert lib.mt_fd_accept(sock, C.byref(tag), 10) < 0  # closed socket: clean failure, no hang


# ---- fused GEMM + collective protocols (host model: threads for CTAs, stamps for data) ----------------------
def _fused(op, n, per, nbs, ngemm, nextra, pair, iters, seed=1, dead=-1, slow=-1, double_buffer=1, timeout_ms=4000):
    from mintccl_b200 import _native as N
    return N.lib().mt_sim_fused(op, n, per, nbs, ngemm, nextra, pair, iters, seed, dead, slow, double_buffer, timeout_ms)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("pair", [0, 1])
def test_fused_allgather_gemm_protocol_many_calls(n, pair):
    """Arrival counters that only grow, the comm CTAs' entry barrier and both tile sizes: 150 back-to-back calls,
    every block read by a GEMM CTA must carry the stamp of the current call."""
    assert _fused(0, n, 4, 2, 3, 2, pair, 150, seed=n) == 0
    assert _fused(0, n, 4, 2, 3, 2, pair, 20, seed=n, slow=0) == 0   # one rank's GEMM far behind the others


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("pair", [0, 1])
def test_fused_gemm_reducescatter_protocol_many_calls(n, pair):
    """Partial-tile counters, ticketed reducers with two alternating ticket words, two alternating staging halves:
    every tile of every call reduced exactly once from partial tiles of that call."""
    assert _fused(1, n, 4, 3, 3, 2, pair, 150, seed=n) == 0
    assert _fused(1, n, 4, 3, 3, 0, pair, 50, seed=n) == 0           # no dedicated reducers: GEMM CTAs reduce at the end
    assert _fused(1, n, 4, 3, 3, 2, pair, 20, seed=n, slow=0) == 0   # one rank's reducers far behind


def test_fused_gemm_reducescatter_single_staging_buffer_is_a_race():
    """Why the staging area has two halves: with one, a rank that has finished call e overwrites, in call e + 1,
    partial tiles that a slower peer has not reduced yet.  The model reports the foreign stamp."""
    assert _fused(1, 4, 4, 3, 3, 2, 0, 20, seed=3, slow=0, double_buffer=0) == 1


def test_fused_protocols_dead_rank_times_out():
    """A rank that never starts: the others give up after their time limit instead of spinning forever."""
    assert _fused(0, 4, 4, 2, 3, 2, 0, 3, dead=2, timeout_ms=300) == 2
    assert _fused(1, 4, 4, 3, 3, 2, 1, 3, dead=1, timeout_ms=300) == 2


def _tile(mode, t, M, N, n, rank, raster, rows, cols=256):
    import ctypes
    from mintccl_b200 import _native as N_
    out = (ctypes.c_int * 4)()
    N_.lib().mt_sched_fused_tile(mode, t, M, N, n, rank, raster, rows, cols, out)
    return tuple(out)


@pytest.mark.parametrize("rows", [128, 256])
def test_gemm_tile_orders_cover_every_tile_once(rows):
    """The tile order the GEMM kernels walk (single-CTA 128-row tiles, 256-row tiles of a CTA pair), every mode:
    a permutation of all tiles on every rank; owners and blocks consistent; the documented visiting order."""
    M, N = 2048 * 2, 1024
    mbs, nbs = M // rows, N // 256
    for raster in (0, 1, 3, 4, 16):                                   # plain: grouped raster, ragged last group
        seen = {_tile(0, t, M, N, 1, 0, raster, rows)[:2] for t in range(mbs * nbs)}
        assert seen == {(mb, nb) for mb in range(mbs) for nb in range(nbs)}
    for n in (1, 2, 4, 8):
        per = M // n // rows
        for mode in (1, 2):
            for rank in range(n):
                tiles = [_tile(mode, t, M, N, n, rank, 0, rows) for t in range(mbs * nbs)]
                assert {(mb, nb) for mb, nb, _, _ in tiles} == {(mb, nb) for mb in range(mbs) for nb in range(nbs)}
                assert all(mb == owner * per + jb and 0 <= jb < per for mb, _, owner, jb in tiles)
                owners = [owner for _, _, owner, _ in tiles]
                if mode == 1:
                    # all-gather -> GEMM: own rows first, then rank - 1, rank - 2, ... (arrival order of the pushes)
                    firsts = [owners.index(o) for o in [(rank - d) % n for d in range(n)]]
                    assert owners[0] == rank and firsts == sorted(firsts)
                else:
                    # GEMM -> reduce-scatter: the first n * nbs tiles are block 0 of every owner, starting at rank + 1
                    assert owners[0] == (rank + 1) % n
                    assert {(o, jb) for _, _, o, jb in tiles[:n * nbs]} == {(o, 0) for o in range(n)}


def test_chain_operations_with_sub_slot_steps(monkeypatch):
    """MINTCCL_CHAIN_STEP_BYTES: chain operations over the Simple protocol step through the FIFOs in pieces smaller
    than a slot (a shorter fill of the chain).  Same results, many operations back to back, with and without it;
    the LL128 protocol and the closed-ring collectives ignore the knob."""
    for step in ("4096", "8192", "1000000", "0"):
        monkeypatch.setenv("MINTCCL_CHAIN_STEP_BYTES", step)
        for op, kw in (("broadcast", dict(root=3)), ("reduce", dict(root=5)), ("sendrecv", dict(chain=[0, 1, 2, 3, 4]))):
            rc, st = sim(8, 2, 0, OPS[op], 50_003, iters=40, jitter=5, slot_bytes=32768, slots=2, **kw)
            assert rc == 0, (step, op, [(s.code, s.where, s.step) for s in st[:8]])
        rc, _ = sim(8, 2, 1, OPS["broadcast"], 20_001, root=1, iters=10, slot_bytes=32768)
        assert rc == 0
        rc, _ = sim(4, 2, 0, OPS["allreduce"], 20_001, iters=10, slot_bytes=32768)
        assert rc == 0


def test_fused_protocols_under_thread_sanitizer(tmp_path):
    """The host model of the fused kernels with its payload as PLAIN memory, built with -fsanitize=thread: the
    arrival counters, the entry barrier and the tickets must order every payload write before the reads that
    depend on it (no report), and ThreadSanitizer must see the race of a single staging buffer."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "mintccl_b200", "csrc", "sim", "sim_fused.cpp")
    exe = str(tmp_path / "sim_fused_tsan")
    r = subprocess.run([gxx, "-O1", "-g", "-std=c++17", "-fsanitize=thread", "-DMT_SIM_PLAIN_DATA", "-DMT_SIM_MAIN",
                        "-I", os.path.join(root, "mintccl_b200", "csrc"), src, "-o", exe, "-pthread"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip("ThreadSanitizer is not available: " + r.stderr[-300:])
    env = dict(os.environ, TSAN_OPTIONS="exitcode=66 halt_on_error=1")

    def run(*a):
        p = subprocess.run([exe] + [str(x) for x in a], env=env, capture_output=True, text=True, timeout=300)
        return p.returncode, p.stderr

    # op, ranks, row blocks, column blocks, GEMM CTAs, comm / reducer CTAs, pair, calls, seed, dead, slow, halves, ms
    clean = [(0, 4, 4, 2, 3, 2, 0, 20, 1, -1, -1, 1, 4000), (0, 4, 4, 2, 3, 2, 1, 20, 2, -1, 0, 1, 4000),
             (1, 4, 4, 3, 3, 2, 0, 20, 3, -1, -1, 1, 4000), (1, 4, 4, 3, 3, 2, 1, 20, 4, -1, 0, 1, 4000),
             (1, 8, 2, 2, 2, 0, 0, 10, 5, -1, -1, 1, 4000)]
    for a in clean:
        rc, err = run(*a)
        assert rc == 0, (a, err[-1500:])
    rc, err = run(1, 4, 4, 3, 3, 2, 0, 20, 3, -1, 0, 0, 4000)      # one staging buffer, one slow rank
    assert rc == 66 and "data race" in err


def test_ring_protocols_under_thread_sanitizer(tmp_path):
    """The ring / chain simulator (the GPU kernels' own schedule code over host FIFOs) built with
    -fsanitize=thread: payload bytes are plain memory, so ThreadSanitizer checks that the step counters and
    credits (release / acquire) order every slot write before its read and every slot reuse after its drain."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "mintccl_b200", "csrc", "sim", "sim.cpp")
    exe = str(tmp_path / "sim_tsan")
    inc = ["-I", os.path.join(root, "mintccl_b200", "csrc")]
    if os.path.isdir("/usr/local/cuda/include"):
        inc += ["-I", "/usr/local/cuda/include"]
    r = subprocess.run([gxx, "-O1", "-g", "-std=c++17", "-fsanitize=thread", "-DMT_SIM_MAIN", *inc, src, "-o", exe, "-pthread"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip("ThreadSanitizer build not available: " + r.stderr[-300:])
    env = dict(os.environ, TSAN_OPTIONS="exitcode=66 halt_on_error=1")
    # ranks channels proto op count root spatial iters jitter_us slot_bytes slots [chain ...]
    cases = {
        "allreduce simple": "8 2 0 5 7001 0 0 10 5 2048 2",
        "broadcast simple": "8 2 0 1 20001 3 0 10 5 2048 2",
        "reduce simple": "8 2 0 2 20001 5 0 10 5 2048 2",
        "multi-hop send/recv": "8 2 0 0 600 0 0 50 0 2048 2 0 1 2 3 4",
        "allgather spatial": "4 4 0 3 5000 0 1 10 5 2048 2",
        "reducescatter": "4 2 0 4 5000 0 0 10 5 2048 2",
        "allreduce ll128": "8 2 1 5 7001 0 0 5 5 2048 2",
    }
    for name, args in cases.items():
        p = subprocess.run([exe] + args.split(), env=env, capture_output=True, text=True, timeout=300)
        assert p.returncode == 0, (name, p.stderr[-1500:])
    # chain with sub-slot steps
    p = subprocess.run([exe] + "8 2 0 1 50003 2 0 10 5 32768 2".split(), env=dict(env, MINTCCL_CHAIN_STEP_BYTES="4096"),
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-1500:]


# ---- one-hop ("direct") collectives and the one-shot all-reduce (host model) -------------------------------
def _direct(n, nctas, iters, seed=1, only_op=-1, slow=-1, dead=-1, exit_barrier=1, timeout_ms=4000):
    from mintccl_b200 import _native as N
    return N.lib().mt_sim_direct(n, nctas, iters, seed, only_op, slow, dead, exit_barrier, timeout_ms)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_direct_protocols_random_mix_back_to_back(n):
    """Two-shot all-reduce (in place), all-gather, reduce-scatter, all-to-all, the one-shot all-reduce and the reduce
    with a summing root in a random order on the same buffers, which the 'user' rewrites between calls: every value read carries the
    stamp of the expected call and rank; also with one rank far behind."""
    assert _direct(n, 3, 300, seed=n) == 0
    assert _direct(n, 2, 60, seed=10 + n, slow=0) == 0
    for op in range(6):   # 5: reduce with a summing root (chunk counters tagged with the barrier epoch, a new root per call)
        assert _direct(n, 2, 40, seed=20 + op, only_op=op) == 0


def test_direct_protocols_need_the_exit_barrier_and_report_dead_ranks():
    # without the second barrier a rank returns while a slower peer still reads its buffer
    assert _direct(4, 2, 30, seed=5, slow=0, exit_barrier=0) == 1
    assert _direct(4, 2, 3, seed=6, dead=2, timeout_ms=300) == 2


def test_direct_protocols_under_thread_sanitizer(tmp_path):
    """The same model with a plain-memory payload under -fsanitize=thread: the per-CTA barriers must order the
    users' rewrites, the pulls and the pushes of consecutive calls; without the exit barrier a race is reported."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "mintccl_b200", "csrc", "sim", "sim_direct.cpp")
    exe = str(tmp_path / "sim_direct_tsan")
    r = subprocess.run([gxx, "-O1", "-g", "-std=c++17", "-fsanitize=thread", "-DMT_SIM_PLAIN_DATA", "-DMT_SIM_MAIN", src, "-o", exe,
                        "-pthread"], capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip("ThreadSanitizer is not available: " + r.stderr[-300:])
    env = dict(os.environ, TSAN_OPTIONS="exitcode=66 halt_on_error=1")

    def run(*a):
        p = subprocess.run([exe] + [str(x) for x in a], env=env, capture_output=True, text=True, timeout=300)
        return p.returncode, p.stderr

    # ranks, CTAs, calls, seed, operation (-1 mix), slow rank, dead rank, exit barrier, ms
    for a in [(8, 3, 60, 1, -1, -1, -1, 1, 8000), (4, 2, 60, 2, -1, 0, -1, 1, 8000), (4, 2, 60, 3, 0, 1, -1, 1, 8000),
              (4, 4, 100, 4, 4, 2, -1, 1, 8000), (8, 2, 60, 7, 5, -1, -1, 1, 8000), (4, 3, 80, 8, 5, 1, -1, 1, 8000)]:
        rc, err = run(*a)
        assert rc == 0, (a, err[-1500:])
    rc, err = run(4, 2, 30, 5, 0, 0, -1, 0, 8000)
    assert rc == 66 and "data race" in err
