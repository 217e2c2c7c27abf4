"""Timers, bandwidth formulas, clock sampling and logging helpers."""
from .timer import Timer, time_device_ms  # noqa: F401
from .busbw import algbw_gbs, busbw_gbs, busbw_factor  # noqa: F401
from .log import log, set_level  # noqa: F401
