"""Benchmark harness: size sweeps of every collective against NCCL, device-timed, max over ranks."""
