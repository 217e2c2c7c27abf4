"""CPU-only unit tests: configuration parsing, bandwidth formulas, topology search, timers."""
import itertools
import os

import pytest

import mintccl_b200 as m
from mintccl_b200 import config as cfgmod
from mintccl_b200.topology import _find_ring_py, _find_route_py, _matrix, ring_min_bandwidth, ring_plan
from mintccl_b200.utils.busbw import algbw_gbs, busbw_factor, busbw_gbs


def test_env_bool_parses_zero_as_false(monkeypatch):
    # the reference's bool(os.getenv(...)) is true for "0" (common.py:113)
    for v, want in [("0", False), ("false", False), ("", False), ("1", True), ("TRUE", True), ("on", True)]:
        monkeypatch.setenv("MINTCCL_TEST_MODE", v)
        assert cfgmod.env_bool("MINTCCL_TEST_MODE") is want
    monkeypatch.setenv("MINTCCL_TEST_MODE", "maybe")
    with pytest.raises(ValueError):
        cfgmod.env_bool("MINTCCL_TEST_MODE")


def test_config_defaults_match_reference_knobs(monkeypatch):
    for k in list(os.environ):
        if k.startswith("MINTCCL_"):
            monkeypatch.delenv(k)
    c = m.Config.from_env()
    # MINTCCL_NUM_BLOCKS defaults to "automatic" (0) here; the reference always launches 16 CTAs
    assert (c.num_blocks, c.num_warps, c.buff_size, c.test_count) == (0, 16, 4194304, 67108864)
    assert m.WARP_SIZE == 32 and m.VECTORIZED_BYTES == 16 and m.NULL == 0
    monkeypatch.setenv("MINTCCL_NUM_BLOCKS", "8")
    monkeypatch.setenv("MINTCCL_BUFFSIZE", "1M")
    monkeypatch.setenv("MINTCCL_ALGO", "ring")
    c = m.Config.from_env()
    assert c.num_blocks == 8 and c.buff_size == 1 << 20 and c.algo == "ring" and c.simple_slot_bytes == 256 << 10
    monkeypatch.setenv("MINTCCL_BUFFSIZE", "3000000")
    with pytest.raises(ValueError):
        m.Config.from_env()
    monkeypatch.setenv("MINTCCL_BUFFSIZE", "4M")
    monkeypatch.setenv("MINTCCL_PROTO", "bogus")
    with pytest.raises(ValueError):
        m.Config.from_env()


def test_busbw_formulas():
    assert busbw_factor("allreduce", 8) == pytest.approx(1.75)
    assert busbw_factor("allgather", 8) == pytest.approx(0.875)
    assert busbw_factor("reducescatter", 4) == pytest.approx(0.75)
    assert busbw_factor("alltoall", 2) == pytest.approx(0.5)
    assert busbw_factor("broadcast", 8) == busbw_factor("reduce", 8) == busbw_factor("sendrecv", 8) == 1.0
    assert algbw_gbs(1 << 30, 1e-3) == pytest.approx(1073.741824)
    assert busbw_gbs("allreduce", 1 << 30, 1e-3, 8) == pytest.approx(1073.741824 * 1.75)
    with pytest.raises(KeyError):
        busbw_factor("gather", 2)


def _topo(edges, n):
    t = {i: [] for i in range(n)}
    for a, b, bw in edges:
        t[a].append((b, bw))
        t[b].append((a, bw))
    return {k: sorted(v, reverse=True) for k, v in t.items()}


def _ring_ok(ring, n):
    return len(ring) == n + 1 and ring[0] == ring[-1] and sorted(ring[:-1]) == list(range(n))


def test_ring_and_route_on_synthetic_topologies():
    # a line has no ring; routes go through the middle
    line = _topo([(0, 1, 50.0), (1, 2, 25.0)], 3)
    assert m.find_ring(line) == []
    assert m.find_route(0, 2, line) == [0, 1, 2]
    assert m.find_route(2, 2, line) == [2]
    # ring of four: the only ring is the ring itself
    sq = _topo([(0, 1, 50.0), (1, 2, 50.0), (2, 3, 50.0), (3, 0, 50.0)], 4)
    r = m.find_ring(sq)
    assert _ring_ok(r, 4) and ring_min_bandwidth(r, sq) == 50.0
    assert m.find_route(0, 2, sq) in ([0, 1, 2], [0, 3, 2])
    # a direct link wins when it is as wide as the detour, loses when it is narrower (widest path)
    tri = _topo([(0, 1, 50.0), (1, 2, 50.0), (0, 2, 50.0)], 3)
    assert m.find_route(0, 2, tri) == [0, 2]
    tri2 = _topo([(0, 1, 50.0), (1, 2, 50.0), (0, 2, 10.0)], 3)
    assert m.find_route(0, 2, tri2) == [0, 1, 2]
    assert m.find_route(0, 2, tri2, shortest=True) == [0, 2]
    # DGX-1 style hybrid cube mesh (V100 x8): double links inside quads, the best ring uses only them
    dbl, sgl = 50.0, 25.0
    edges = [(0, 3, dbl), (0, 4, dbl), (1, 2, dbl), (1, 5, dbl), (2, 3, dbl), (6, 7, dbl), (4, 7, dbl), (5, 6, dbl),
             (0, 1, sgl), (0, 2, sgl), (1, 3, sgl), (2, 6, sgl), (3, 7, sgl), (4, 5, sgl), (4, 6, sgl), (5, 7, sgl)]
    cube = _topo(edges, 8)
    r = m.find_ring(cube)
    assert _ring_ok(r, 8) and ring_min_bandwidth(r, cube) == dbl
    # NVSwitch: uniform all-to-all, identity ring, direct routes
    sw = m.uniform_topology(8)
    assert m.find_ring(sw) == [0, 1, 2, 3, 4, 5, 6, 7, 0]
    for a, b in itertools.permutations(range(8), 2):
        assert m.find_route(a, b, sw) == [a, b]
    assert ring_plan(m.find_ring(sw), 0) == (7, 1)
    # disconnected
    two = _topo([(0, 1, 50.0)], 3)
    assert m.find_route(0, 2, two) == [] and m.find_ring(two) == []


def test_native_and_python_searches_agree():
    import random
    rng = random.Random(7)
    for trial in range(30):
        n = rng.randint(3, 7)
        edges = [(a, b, float(rng.choice([10, 25, 50]))) for a in range(n) for b in range(a + 1, n) if rng.random() < 0.7]
        t = _topo(edges, n)
        nodes, mat = _matrix(t)
        ring_native = m.find_ring(t)
        ring_py = _find_ring_py(mat, n)
        assert (ring_native == []) == (ring_py == [])
        if ring_native:
            assert ring_min_bandwidth(ring_native, t) == ring_min_bandwidth(ring_py, t)
        for s, d in [(0, n - 1), (1, 2)]:
            a, b = m.find_route(s, d, t), _find_route_py(mat, n, s, d)
            assert len(a) == len(b)
            if a:
                width = lambda p: min(dict(t[x])[y] for x, y in zip(p[:-1], p[1:]))  # noqa: E731
                assert width(a) == width(b)


def test_topology_cache_roundtrip(tmp_path):
    import json
    t = m.uniform_topology(4, 123.0)
    f = tmp_path / "topo.json"
    f.write_text(json.dumps(t))
    assert m.get_topology(str(f)) == t
    # without a GPU and without a cache the topology is the uniform one
    assert m.get_topology(str(tmp_path / "none.json"), ndev=2) in (m.uniform_topology(2), m.get_topology(str(tmp_path / "none.json"), ndev=2))


def test_timer_host(capsys):
    with m.Timer(rank=3) as t:
        sum(range(1000))
    assert t.elapsed > 0
    assert "# rank: 3 time:" in capsys.readouterr().out
    with m.Timer(quiet=True):
        pass
    assert capsys.readouterr().out == ""


def test_fused_plan_cta_counts_follow_the_gemm_to_transfer_ratio():
    """Comm CTAs of all-gather -> GEMM and reducer CTAs of GEMM -> reduce-scatter: as many as keep pace with the
    GEMM, the rest computes (Llama-3-8B MLP, tokens 8192, hidden 4096, ffn 14336 split over the ranks)."""
    from mintccl_b200.ops.gemm import AllGatherGemm, GemmReduceScatter
    T, H = 8192, 4096
    picks = {}
    for n, F in ((8, 1792), (4, 3584), (2, 7168)):
        tiles = (T // 128) * (F // 256)
        picks[n] = (AllGatherGemm.pick_ncomm(tiles, flops=2.0 * T * F * H, bytes_in=(n - 1) / n * T * H * 2),
                    GemmReduceScatter.pick_nred(T, H, F, n))
    assert picks[8] == (24, 12)           # the counts tuned on 8 GPUs
    assert picks[2][0] <= 6 and picks[2][1] <= 4   # GEMM-bound: nearly all SMs compute
    assert picks[8][0] >= picks[4][0] >= picks[2][0] and picks[8][1] >= picks[4][1] >= picks[2][1]
    # without the sizes: the widest transfer that does not add a GEMM wave
    assert AllGatherGemm.pick_ncomm(448) == 24
    # MXFP8 halves the bytes and nearly doubles the GEMM rate: never more comm CTAs than bf16
    assert AllGatherGemm.pick_ncomm(448, flops=2.0 * T * 1792 * H, bytes_in=7 / 8 * T * H, fp8=True) <= 24


def test_launch_statistics_interface():
    """Per-family counters of the native library: names, zero without launches, reset."""
    from mintccl_b200.utils import stats
    stats.reset()
    allf = stats.snapshot(skip_idle=False)
    assert {"ring_simple", "ring_ll128", "direct", "nvls", "ll_oneshot", "p2p", "local_copy", "gemm", "gemm_mxfp8",
            "ag_gemm", "gemm_rs", "mxfp8_reduce"} == set(allf)
    assert all(v == {"calls": 0, "work": 0} for v in allf.values())
    assert stats.snapshot() == {} and stats.report() == "(nothing launched)"


def test_profile_range_is_a_noop_without_cuda():
    from mintccl_b200.utils.profiler import profile_range
    ran = []
    with profile_range("x"):
        ran.append(1)
    with profile_range("y", enabled=False):
        ran.append(2)
    assert ran == [1, 2]


def test_clock_sampler_against_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The sampler only READS clocks (through ``nvidia-smi --query-gpu``).  A stand-in ``nvidia-smi`` on PATH prints
    the CSV it would print under load with a power cap; the summary must report the median clock of the timed
    region, the largest maximum clock and the active reasons."""
    import os
    import stat
    import time
    from mintccl_b200.utils.clocks import ClockSampler
    fake = tmp_path / "nvidia-smi"
    fake.write_text("""#!/usr/bin/env python3
import datetime, sys, time
assert any(a.startswith("--query-gpu=") for a in sys.argv) and "-lms" in sys.argv, sys.argv
clocks = [1965, 1500, 1320, 1335, 1327, 1965]
for i in range(400):
    now = datetime.datetime.now().strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    cap = "Active" if 1 <= i % 6 <= 4 else "Not Active"
    print(f"{now}, {clocks[i % 6]}, 1965, 950.5, Not Active, Not Active, Not Active, {cap}", flush=True)
    time.sleep(0.01)
""")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    s = ClockSampler(0, period_ms=10).start()
    time.sleep(0.15)
    s.mark_begin()
    time.sleep(0.4)
    s.mark_end()
    out = s.stop()
    assert out["samples"] >= 10 and out["note"] == "samples inside the timed region"
    assert out["sm_max_mhz"] == 1965.0 and 1320.0 <= out["sm_mhz"] <= 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    # a region shorter than the sampling period falls back to the nearest samples
    s2 = ClockSampler(0, period_ms=10).start()
    time.sleep(0.2)
    s2.mark_begin()
    s2.mark_end()
    out2 = s2.stop()
    assert out2["samples"] >= 1 and "nearest" in out2["note"]


def test_bench_reference_arm_reports_unavailable():
    """``bench.py --impl reference`` never runs the reference's GPU code (it faulted on its first call on this
    hardware): rank 0 prints one JSON line with the reason, every rank exits 0."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for rank in (0, 1):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT="29987")
        r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2",
                            "--warmup", "1"], env=env, capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-500:]
        lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
        if rank == 0:
            d = json.loads(lines[-1])
            assert d["impl"] == "reference" and "illegal memory access" in d["unavailable"]
        else:
            assert not lines


def test_ctypes_signatures_match_the_c_header():
    """Every function of csrc/mintccl.h (and of the no-alloc entry point's header) has a ctypes signature with the
    same number of parameters: a mismatch would otherwise only show as garbage arguments on a GPU."""
    import os
    import re
    from mintccl_b200 import _native as N
    lib = N.lib()
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mintccl_b200", "csrc")
    text = open(os.path.join(root, "mintccl.h")).read()
    text = re.sub(r"//[^\n]*", "", text)
    decls = re.findall(r"\b(mt_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S)
    assert len(decls) > 40
    missing, wrong = [], []
    for name, params in decls:
        params = params.strip()
        n = 0 if params in ("", "void") else len([p for p in params.split(",") if p.strip()])
        fn = getattr(lib, name, None)
        assert fn is not None, f"{name} is declared but not exported"
        if fn.argtypes is None:
            missing.append(name)
        elif len(fn.argtypes) != n:
            wrong.append((name, n, len(fn.argtypes)))
    assert not wrong, wrong
    # functions without a ctypes signature would be called with default int conversions: none may be left
    assert not missing, missing


def test_heap_smaller_than_its_control_region_is_refused():
    """The FIFOs and control words are sized by the channel count; a heap that cannot hold them must be refused
    when the communicator is created (the layout arithmetic needs no GPU), never found out by a kernel."""
    import ctypes as C
    from mintccl_b200 import _native as N
    lib = N.lib()
    lay_fn = lib.mt_layout_user_off
    lay_fn.restype = C.c_uint64
    lay_fn.argtypes = [C.c_int, C.POINTER(N.MtConfig)]
    mc = N.MtConfig(nchannels=32, simple_slot_bytes=512 << 10, simple_slots=4, ll128_slot_bytes=128 << 10, ll128_slots=4,
                    ll_bytes=256 << 10, scratch_bytes=1 << 20, heap_bytes=288 << 20, timeout_ms=1000, heap_kind=1)
    need = lay_fn(4, C.byref(mc))
    assert need > mc.heap_bytes                      # 32 channels x 4 peers x 2.5 MiB of FIFOs alone are 320 MiB
    mc.nchannels = 16
    mc.simple_slot_bytes = 256 << 10
    assert lay_fn(4, C.byref(mc)) < (128 << 20)
