"""Samples SM clocks and throttle reasons while a benchmark runs (read-only NVML queries through
``nvidia-smi``); nothing here changes a GPU setting."""
from __future__ import annotations

import datetime
import statistics
import time
import subprocess
import threading
from typing import Dict, List

_QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
          "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
          "clocks_event_reasons.sw_power_cap")
_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 50):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.samples: List[List[str]] = []
        self._proc = None
        self._thread = None

    def start(self) -> "ClockSampler":
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            for line in self._proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 8:
                    try:
                        ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    except ValueError:
                        ts = time.time()
                    self.samples.append([ts] + parts[1:])

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def mark_begin(self) -> None:
        """Start of the timed region: only samples taken from here to ``mark_end`` are reported."""
        self._t0 = time.time()

    def mark_end(self) -> None:
        self._t1 = time.time()

    def stop(self) -> Dict:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)
        t0, t1 = getattr(self, "_t0", None), getattr(self, "_t1", None)
        rows = self.samples
        in_window = [p for p in rows if t0 is not None and t1 is not None and t0 <= p[0] <= t1]
        note = "samples inside the timed region"
        if not in_window and rows and t0 is not None:
            # the region was shorter than the sampling period: take the samples nearest to it
            mid = 0.5 * (t0 + (t1 or t0))
            in_window = sorted(rows, key=lambda p: abs(p[0] - mid))[:3]
            note = "timed region shorter than the sampling period: nearest samples"
        elif not in_window:
            in_window = rows
            note = "all samples"
        sm, mx, reasons = [], [], set()
        for p in in_window:
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, val in zip(_REASONS, p[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "note": "nvidia-smi gave no samples"}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "note": note}
