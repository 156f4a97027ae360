"""Timing helpers: sync-bracketed wall clock (the reference's tps clock, ``torchure/utils.py:11-38``)
and CUDA-event device timing (the clock benchmarks report)."""

from __future__ import annotations

import functools
import os
import time

import torch


def _sync() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def record_time(fn):
    """Return ``(result, seconds)``; the device is synchronised before and after the call."""

    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        _sync()
        t0 = time.perf_counter()
        out = fn(*args, **kwargs)
        _sync()
        return out, time.perf_counter() - t0

    return wrapped


def debug_time(fn):
    """Print the call's wall time on rank 0."""

    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        t0 = time.perf_counter()
        out = fn(*args, **kwargs)
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"[time] {fn.__qualname__}: {time.perf_counter() - t0:.3f}s", flush=True)
        return out

    return wrapped


class DeviceTimer:
    """CUDA-event stopwatch on the current stream; ``elapsed_ms`` synchronises on the stop event."""

    def __init__(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._stop = torch.cuda.Event(enable_timing=True)

    def start(self) -> None:
        self._start.record()

    def stop(self) -> None:
        self._stop.record()

    def elapsed_ms(self) -> float:
        self._stop.synchronize()
        return self._start.elapsed_time(self._stop)
