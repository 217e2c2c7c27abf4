"""Counters of what the native library launched, per kernel family: calls and work (message bytes for
collectives and copies, floating-point operations for GEMMs).  The reference has no counters, only prints
guarded by ``MINTCCL_TEST_VERBOSE`` (common.py:118).

    from mintccl_b200.utils import stats
    stats.reset(); ...; print(stats.snapshot())   # {'nvls': {'calls': 20, 'work': 1342177280}, ...}
"""
from __future__ import annotations

import ctypes
from typing import Dict

from .. import _native as N


def snapshot(skip_idle: bool = True) -> Dict[str, Dict[str, int]]:
    """Counters since the library was loaded or since :func:`reset`; families never used are left out."""
    lib = N.lib()
    out: Dict[str, Dict[str, int]] = {}
    for k in range(lib.mt_stats_count()):
        calls, work = ctypes.c_uint64(0), ctypes.c_uint64(0)
        lib.mt_stats_get(k, ctypes.byref(calls), ctypes.byref(work))
        if calls.value or not skip_idle:
            out[lib.mt_stats_name(k).decode()] = {"calls": calls.value, "work": work.value}
    return out


def reset() -> None:
    N.lib().mt_stats_reset()


def report() -> str:
    """One line per family, for logs."""
    rows = [f"{name:<13} calls {v['calls']:>8}  work {v['work']:.3e}" for name, v in snapshot().items()]
    return "\n".join(rows) if rows else "(nothing launched)"
