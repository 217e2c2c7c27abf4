"""Host and device timers.

``Timer`` keeps the interface of the reference's context manager (common.py:41-67: ``device`` and
``rank`` arguments, prints ``# rank: r time: Xs``) and additionally stores the result in ``.elapsed`` and
can stay silent.  ``time_device_ms`` is the measurement recipe used for every number this package
reports: warm-up, CUDA events on the launching stream, a synchronise on both sides.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional


class Timer:
    def __init__(self, device: bool = False, rank: Optional[int] = None, quiet: bool = False) -> None:
        self.rank, self.device, self.quiet = rank, device, quiet
        self.elapsed = 0.0

    def __enter__(self) -> "Timer":
        if self.device:
            import torch
            self._start = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            self._start.record()
        else:
            self._start = time.perf_counter_ns()
        return self

    def __exit__(self, exc_type, exc_value, exc_traceback) -> None:
        if self.device:
            import torch
            self._end.record()
            self._end.synchronize()  # only this event, not the whole device
            self.elapsed = self._start.elapsed_time(self._end) / 1e3
        else:
            self.elapsed = (time.perf_counter_ns() - self._start) / 1e9
        if not self.quiet:
            if self.rank is not None:
                print(f"# rank: {self.rank} time: {self.elapsed}s")
            else:
                print(f"# time {self.elapsed}s")


def time_device_ms(fn: Callable[[], None], iters: int = 20, warmup: int = 5, between: Optional[Callable[[], None]] = None,
                   per_iter: bool = False) -> List[float]:
    """Device time of ``fn`` in milliseconds.

    ``between`` runs before every timed call outside the timed interval (e.g. an L2 flush).  With
    ``per_iter`` every call is timed with its own event pair and the list of times is returned; otherwise
    one pair brackets all calls and the list has a single entry, the mean."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if per_iter or between is not None:
        out = []
        for _ in range(iters):
            if between is not None:
                between()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            out.append(e0.elapsed_time(e1))
        return out
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return [e0.elapsed_time(e1) / iters]
