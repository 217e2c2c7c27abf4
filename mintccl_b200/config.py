"""Configuration knobs, read from the environment once per communicator.

Keeps every knob of the reference (common.py:76-118: ``MINTCCL_NUM_BLOCKS``, ``MINTCCL_NUM_WARPS``,
``MINTCCL_BUFFSIZE``, ``MINTCCL_TEST_MODE``, ``MINTCCL_TEST_COUNT``, ``MINTCCL_TEST_VERBOSE``) under the
same names and adds the ones its roadmap asks for (README.md:57 "fine-grained control of SM layout"):
algorithm, protocol, channel count, FIFO depth, wait time limit, heap size.  Booleans are parsed properly:
the reference's ``bool(os.getenv(...))`` (common.py:113,118) is true for the string ``"0"``.

``MINTCCL_TUNING_FILE`` names a table of measured choices that overrides the size thresholds of the built-in policy
(:mod:`mintccl_b200.tuning`).

``MINTCCL_TOPO_FILE`` / ``MINTCCL_TOPO_DISCOVER`` / ``MINTCCL_TOPO_MEASURE`` choose the link map behind the ring and
the routes (default: uniform, which is exact on an NVSwitch node); ``MINTCCL_RING``, ``MINTCCL_RING_SEED`` and
``MINTCCL_ROUTE=ring`` override the result.

Read by the native library itself, at every call (tuning switches, not part of :class:`Config`):
``MINTCCL_GEMM_PAIR`` (0: single-CTA GEMM kernels instead of CTA pairs), ``MINTCCL_GEMM_RASTER`` (row blocks per
group of the plain GEMM's tile order), ``MINTCCL_CHAIN_STEP_BYTES`` (bytes per FIFO step of chain operations over
the Simple protocol; default: half a channel's share, 64 - 256 KiB, which serves a single call; 0: whole slots, the best for streams of identical calls), ``MINTCCL_NO_LOCAL_COPY`` (one-rank communicators use the ring kernel).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

WARP_SIZE = 32            # common.py:104
VECTORIZED_BYTES = 16     # common.py:105
NULL = 0                  # common.py:71
_TRUE = {"1", "true", "yes", "on", "y", "t"}
_FALSE = {"0", "false", "no", "off", "n", "f", ""}


def env_bool(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    s = v.strip().lower()
    if s in _TRUE:
        return True
    if s in _FALSE:
        return False
    raise ValueError(f"{name}={v!r} is not a boolean")


def env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v.strip() == "":
        return default
    s = v.strip().lower()
    mult = 1
    for suf, m in (("k", 1 << 10), ("m", 1 << 20), ("g", 1 << 30)):
        if s.endswith(suf):
            s, mult = s[:-1], m
            break
    return int(s, 0) * mult


def env_str(name: str, default: str, choices: tuple[str, ...] | None = None) -> str:
    v = os.environ.get(name, default).strip().lower()
    if choices and v not in choices:
        raise ValueError(f"{name}={v!r}: expected one of {choices}")
    return v


def _is_pow2(x: int) -> bool:
    return x > 0 and (x & (x - 1)) == 0


@dataclass
class Config:
    """All tunables of a communicator.  ``Config.from_env()`` reads the environment."""
    # reference knobs
    num_blocks: int = 0                   # MINTCCL_NUM_BLOCKS: most channels (CTAs) of a ring kernel; 0 = up to
                                          # max_channels, by message size (the reference always uses 16)
    num_warps: int = 16                   # MINTCCL_NUM_WARPS: fixed at 16 in the compiled kernels
    buff_size: int = 4 << 20              # MINTCCL_BUFFSIZE: Simple FIFO bytes per connection
    test_mode: bool = False               # MINTCCL_TEST_MODE
    test_count: int = 67108864            # MINTCCL_TEST_COUNT
    verbose: bool = False                 # MINTCCL_TEST_VERBOSE
    # algorithm / protocol selection
    algo: str = "auto"                    # ring | direct | nvls | ll | auto
    proto: str = "auto"                   # simple | ll128 | auto
    max_channels: int = 64                # channels the FIFOs are sized for
    direct_ctas: int = 0                  # CTAs of direct kernels (0 = by message size, at most 128)
    nvls_ctas: int = 32                   # most CTAs of an NVLS kernel (the switch saturates with few)
    bulk_ctas: int = 128                  # MINTCCL_BULK_CTAS: most CTAs of a copy-engine (cp.async.bulk) variant
    simple_slots: int = 4
    ll128_slot_bytes: int = 128 << 10
    ll128_slots: int = 4
    ll_bytes: int = 256 << 10             # one-shot area per (parity, sender)
    scratch_bytes: int = 64 << 20
    heap_bytes: int = 4 << 30
    wait_timeout_ms: int = 10000
    heap_kind: str = "auto"               # vmm | ipc | auto
    nvls: str = "auto"                    # on | off | auto
    auto_register: bool = True            # MINTCCL_AUTO_REGISTER: share ordinary tensors with the peers (CUDA IPC) on
                                          # first use so that they take the one-hop kernels; off: FIFO ring unless
                                          # the tensor was passed to Communicator.share()
    debug: str = "warn"                   # warn | info | trace
    # thresholds of the automatic choice (bytes)
    ll_max_bytes: int = 32 << 10
    ll128_max_bytes: int = 512 << 10
    nvls_min_bytes: int = 48 << 10
    spins_before_abort: int = 1000000     # common.py:106 (kept for parity; waits are time-bounded)

    @property
    def simple_slot_bytes(self) -> int:
        return self.buff_size // self.simple_slots

    def validate(self) -> "Config":
        if not 0 <= self.num_blocks <= self.max_channels <= 96 or self.max_channels < 1:
            raise ValueError("need 0 <= MINTCCL_NUM_BLOCKS <= MINTCCL_MAX_CHANNELS <= 96")
        if self.num_warps != 16:
            raise ValueError("MINTCCL_NUM_WARPS: the compiled kernels use 16 warps per CTA")
        if not _is_pow2(self.buff_size) or self.buff_size < 64 << 10:
            raise ValueError("MINTCCL_BUFFSIZE must be a power of two >= 64 KiB")
        if self.simple_slot_bytes % 128:
            raise ValueError("MINTCCL_BUFFSIZE / MINTCCL_SIMPLE_SLOTS must be a multiple of 128")
        if self.ll128_slot_bytes % 2048 or self.ll_bytes % 2048:
            raise ValueError("LL128 slot and one-shot sizes must be multiples of 2048")
        if self.algo not in ("ring", "direct", "nvls", "ll", "auto"):
            raise ValueError(f"MINTCCL_ALGO={self.algo!r}")
        if self.proto not in ("simple", "ll128", "auto"):
            raise ValueError(f"MINTCCL_PROTO={self.proto!r}")
        return self

    @classmethod
    def from_env(cls, **overrides) -> "Config":
        c = cls(
            num_blocks=env_int("MINTCCL_NUM_BLOCKS", 0),
            num_warps=env_int("MINTCCL_NUM_WARPS", 16),
            buff_size=env_int("MINTCCL_BUFFSIZE", 4 << 20),
            test_mode=env_bool("MINTCCL_TEST_MODE", False),
            test_count=env_int("MINTCCL_TEST_COUNT", 67108864),
            verbose=env_bool("MINTCCL_TEST_VERBOSE", False),
            algo=env_str("MINTCCL_ALGO", "auto", ("ring", "direct", "nvls", "ll", "auto")),
            proto=env_str("MINTCCL_PROTO", "auto", ("simple", "ll128", "auto")),
            max_channels=env_int("MINTCCL_MAX_CHANNELS", 64),
            direct_ctas=env_int("MINTCCL_DIRECT_CTAS", 0),
            nvls_ctas=env_int("MINTCCL_NVLS_CTAS", 32),
            bulk_ctas=env_int("MINTCCL_BULK_CTAS", 128),
            simple_slots=env_int("MINTCCL_SIMPLE_SLOTS", 4),
            ll128_slot_bytes=env_int("MINTCCL_LL128_SLOT_BYTES", 128 << 10),
            ll128_slots=env_int("MINTCCL_LL128_SLOTS", 4),
            ll_bytes=env_int("MINTCCL_LL_BYTES", 256 << 10),
            scratch_bytes=env_int("MINTCCL_SCRATCH_BYTES", 64 << 20),
            heap_bytes=env_int("MINTCCL_HEAP_BYTES", 4 << 30),
            wait_timeout_ms=env_int("MINTCCL_WAIT_TIMEOUT_MS", 10000),
            heap_kind=env_str("MINTCCL_HEAP", "auto", ("vmm", "ipc", "auto")),
            nvls=env_str("MINTCCL_NVLS", "auto", ("on", "off", "auto")),
            auto_register=env_bool("MINTCCL_AUTO_REGISTER", True),
            debug=env_str("MINTCCL_DEBUG", "warn", ("warn", "info", "trace")),
            ll_max_bytes=env_int("MINTCCL_LL_MAX_BYTES", 32 << 10),
            ll128_max_bytes=env_int("MINTCCL_LL128_MAX_BYTES", 512 << 10),
            nvls_min_bytes=env_int("MINTCCL_NVLS_MIN_BYTES", 48 << 10),
        )
        for k, v in overrides.items():
            if not hasattr(c, k):
                raise TypeError(f"unknown config field {k}")
            setattr(c, k, v)
        return c.validate()
