"""Bandwidth conventions (the nccl-tests ones) used for every reported number.

``algbw`` = message bytes / time.  ``busbw`` = ``algbw`` times a factor that makes the number
comparable with the per-GPU link bandwidth: 2(n-1)/n for all-reduce, (n-1)/n for all-gather,
reduce-scatter and all-to-all (message = the whole gathered / scattered buffer), 1 for broadcast,
reduce and send/recv.
"""
from __future__ import annotations

_FACTORS = {
    "allreduce": lambda n: 2.0 * (n - 1) / n,
    "allgather": lambda n: (n - 1) / n,
    "reducescatter": lambda n: (n - 1) / n,
    "alltoall": lambda n: (n - 1) / n,
    "broadcast": lambda n: 1.0,
    "reduce": lambda n: 1.0,
    "sendrecv": lambda n: 1.0,
}


def busbw_factor(collective: str, nranks: int) -> float:
    if collective not in _FACTORS:
        raise KeyError(f"unknown collective {collective!r}")
    return _FACTORS[collective](max(1, nranks))


def algbw_gbs(nbytes: int, seconds: float) -> float:
    return nbytes / seconds / 1e9 if seconds > 0 else 0.0


def busbw_gbs(collective: str, nbytes: int, seconds: float, nranks: int) -> float:
    return algbw_gbs(nbytes, seconds) * busbw_factor(collective, nranks)
