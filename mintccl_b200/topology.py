"""Topology discovery and routing: which GPUs are linked, the widest route between two of them and the
best ring through all of them.

Public names and types follow the reference (topology.py:18-150: ``Topology``, ``Route``, ``Plan``,
``find_route``, ``find_ring``, ``get_p2p_speed``, ``get_topology``).  The searches are exact and are run
by the native library when it is built (``csrc/host/topology.cpp``) with a pure-Python implementation
of the same algorithms as fall-back and cross-check.  Behavioural differences from the reference, all on
purpose:

* ``find_route`` really prefers a direct link (the reference tests ``dst in topo[src]`` against a list of
  tuples, topology.py:30, so the shortcut never fires) and breaks bandwidth ties by hop count;
* ``find_ring`` is an exhaustive depth-first search with pruning instead of a best-first enumeration
  whose priority mixes hop count and bandwidth (topology.py:84-86);
* ``get_p2p_speed`` warms the path up before timing (the reference times one cold copy);
* on an NVSwitch node (every pair linked at the same speed) nothing is measured unless asked.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Dict, List, Optional, Tuple

Topology = Dict[int, List[Tuple[int, float]]]  # src -> [(dst, GB/s)], sorted by dst descending like the reference
Route = List[int]
Plan = Tuple[int, int]  # (prev, next) of a rank in a ring


def uniform_topology(n: int, bw: float = 900.0) -> Topology:
    """All-to-all topology of an NVSwitch node: every pair linked at ``bw`` GB/s per direction."""
    return {s: sorted(((d, bw) for d in range(n) if d != s), reverse=True) for s in range(n)}


def _matrix(topo: Topology) -> Tuple[List[int], List[float]]:
    nodes = sorted(topo.keys())
    idx = {v: i for i, v in enumerate(nodes)}
    n = len(nodes)
    m = [0.0] * (n * n)
    for s, items in topo.items():
        for d, bw in items:
            if d in idx:
                m[idx[s] * n + idx[d]] = max(m[idx[s] * n + idx[d]], float(bw))
    return nodes, m


def _native():
    try:
        from . import _native as N
        return N.lib() if N.available() else None
    except Exception:
        return None


def _find_route_py(m: List[float], n: int, src: int, dst: int) -> List[int]:
    if src == dst:
        return [src]
    width = [0.0] * n
    hops = [1 << 30] * n
    prev = [-1] * n
    done = [False] * n
    width[src], hops[src] = float("inf"), 0
    for _ in range(n):
        u = -1
        for v in range(n):
            if done[v] or width[v] <= 0:
                continue
            if u < 0 or width[v] > width[u] or (width[v] == width[u] and hops[v] < hops[u]):
                u = v
        if u < 0:
            break
        done[u] = True
        for v in range(n):
            e = m[u * n + v]
            if e <= 0 or done[v]:
                continue
            w = min(width[u], e)
            if w > width[v] or (w == width[v] and hops[u] + 1 < hops[v]):
                width[v], hops[v], prev[v] = w, hops[u] + 1, u
    if width[dst] <= 0:
        return []
    path = []
    v = dst
    while v != -1:
        path.append(v)
        v = prev[v]
    return path[::-1] if path[-1] == src else []


def _find_ring_py(m: List[float], n: int) -> List[int]:
    if n == 1:
        return [0, 0]
    best: List[int] = []
    best_bw = 0.0
    used = [False] * n
    used[0] = True
    path = [0]

    def dfs(u: int, min_bw: float) -> None:
        nonlocal best, best_bw
        if len(path) == n:
            back = m[u * n + path[0]]
            w = min(min_bw, back)
            if back > 0 and w > best_bw:
                best_bw, best = w, list(path)
            return
        for v in range(n):
            if used[v]:
                continue
            e = m[u * n + v]
            if e <= 0:
                continue
            w = min(min_bw, e)
            if w <= best_bw:
                continue
            used[v] = True
            path.append(v)
            dfs(v, w)
            path.pop()
            used[v] = False

    dfs(0, float("inf"))
    return best + [best[0]] if best else []


def find_route(src: int, dst: int, topo: Optional[Topology] = None, shortest: bool = False) -> Route:
    """Widest route ``src -> dst`` (list of ranks, both ends included) or ``[]`` if unreachable.

    ``shortest=True`` ignores bandwidth and returns a route with the fewest hops."""
    if topo is None:
        topo = get_topology()
    nodes, m = _matrix(topo)
    if src not in nodes or dst not in nodes:
        return []
    n = len(nodes)
    if shortest:
        m = [1.0 if x > 0 else 0.0 for x in m]
    s, d = nodes.index(src), nodes.index(dst)
    L = _native()
    if L is not None:
        arr = (C.c_double * (n * n))(*m)
        out = (C.c_int * (n + 1))()
        k = L.mt_find_route(arr, n, s, d, out)
        return [nodes[out[i]] for i in range(k)]
    return [nodes[i] for i in _find_route_py(m, n, s, d)]


def find_ring(topo: Optional[Topology] = None) -> Route:
    """Best ring through all ranks: maximises the slowest link.  Returned with the first rank repeated at
    the end (length n+1) like the reference (topology.py:92), or ``[]`` if there is no ring."""
    if topo is None:
        topo = get_topology()
    nodes, m = _matrix(topo)
    n = len(nodes)
    if n == 0:
        return []
    L = _native()
    if L is not None:
        arr = (C.c_double * (n * n))(*m)
        out = (C.c_int * (n + 1))()
        k = L.mt_find_ring(arr, n, out)
        return [nodes[out[i]] for i in range(k)]
    return [nodes[i] for i in _find_ring_py(m, n)]


def ring_plan(ring: Route, rank: int) -> Plan:
    """(prev, next) of ``rank`` in ``ring`` (either form: with or without the repeated first rank)."""
    r = ring[:-1] if len(ring) > 1 and ring[0] == ring[-1] else list(ring)
    i = r.index(rank)
    return r[(i - 1) % len(r)], r[(i + 1) % len(r)]


def ring_min_bandwidth(ring: Route, topo: Topology) -> float:
    r = ring if ring[0] == ring[-1] else list(ring) + [ring[0]]
    bw = float("inf")
    for a, b in zip(r[:-1], r[1:]):
        link = dict(topo[a]).get(b, 0.0)
        bw = min(bw, link)
    return bw


def get_p2p_speed(src: int, dst: int, size: int = 32 << 20) -> float:
    """Measured copy bandwidth ``src -> dst`` in GB/s (one warm-up copy, one timed copy of ``size`` bytes); 0.0
    when the two devices have no peer access.  Only this pair is probed (topology.py:96-125 of the reference)."""
    L = _native()
    if L is None:
        raise RuntimeError("get_p2p_speed needs the native library and a GPU")
    gbs = C.c_double(0.0)
    if L.mt_topo_probe_pair(src, dst, size, C.byref(gbs)) < 0:
        raise RuntimeError(f"no such device pair: {src} -> {dst}")
    return float(gbs.value)


def get_topology(topo: str = "topo.json", measure: Optional[bool] = None, ndev: Optional[int] = None) -> Topology:
    """Load the cached topology from ``topo`` or discover it and cache it there.

    Discovery asks the driver which pairs have peer access; bandwidth is measured only when ``measure`` is
    true (default: the ``MINTCCL_TOPO_MEASURE`` environment flag), otherwise every link counts 900 GB/s,
    which is exact on an NVSwitch node.  Without a GPU the topology is the uniform one for
    ``ndev`` (default ``WORLD_SIZE`` or 1) ranks and nothing is cached."""
    if topo and os.path.exists(topo):
        with open(topo, "r") as f:
            raw = json.load(f)
        return {int(s): [(int(d), float(bw)) for d, bw in items] for s, items in raw.items()}
    L = _native()
    have_gpu = False
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except ImportError:
        pass
    if L is None or not have_gpu:
        return uniform_topology(ndev or int(os.environ.get("WORLD_SIZE", "1")))
    import torch
    from .config import env_bool
    n = ndev or torch.cuda.device_count()
    if measure is None:
        measure = env_bool("MINTCCL_TOPO_MEASURE", False)
    m = (C.c_double * (n * n))()
    if L.mt_topo_probe(n, m, 1 if measure else 0, 32 << 20) < 0:
        raise RuntimeError("topology probe failed")
    out: Topology = {s: [] for s in range(n)}
    for s in range(n):
        for d in range(n):
            if s != d and m[s * n + d] > 0:
                out[s].append((d, float(m[s * n + d]) if measure else 900.0))
    out = {s: sorted(items, reverse=True) for s, items in out.items()}
    if topo:
        try:
            with open(topo, "w") as f:
                json.dump(out, f)
        except OSError:
            pass
    return out
