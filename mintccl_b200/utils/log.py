"""Levelled logging controlled by ``MINTCCL_DEBUG`` (warn | info | trace); the reference only has
``print`` guarded by ``MINTCCL_TEST_VERBOSE`` (common.py:118)."""
from __future__ import annotations

import os
import sys

_LEVELS = {"warn": 0, "info": 1, "trace": 2}
_level = _LEVELS.get(os.environ.get("MINTCCL_DEBUG", "warn").lower(), 0)


def set_level(name: str) -> None:
    global _level
    _level = _LEVELS[name]


def log(level: str, msg: str) -> None:
    if _LEVELS[level] <= _level:
        rank = os.environ.get("RANK", "0")
        print(f"[mintccl {level} r{rank}] {msg}", file=sys.stderr, flush=True)
