"""Device and host timers.

``cuda_time`` is the benchmark primitive: warm-up, then per-iteration CUDA-event timing on
the current stream with an optional L2 flush between iterations.  ``Timer`` is the host
stopwatch with the integer Seconds/MilliSeconds/MicroSeconds/NanoSeconds readouts of the
reference's newplan::Timer (cost_model/timer.h:12-132, vector_add/time_record.h:6-126).
"""
from __future__ import annotations

import time
from typing import Callable

import torch

_flush_buf: dict[int, torch.Tensor] = {}


def flush_l2(device=None) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _flush_buf:
        _flush_buf[idx] = torch.empty(192 << 20, dtype=torch.uint8, device=f"cuda:{idx}")
    _flush_buf[idx].zero_()


def cuda_time(fn: Callable[[], None], iters: int = 10, warmup: int = 3, flush: bool = True) -> list[float]:
    """Milliseconds per call of ``fn`` (list of ``iters`` samples) measured with CUDA events."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        out.append(a.elapsed_time(b))
    return out


class Timer:
    def __init__(self):
        self._t0 = self._t1 = 0

    def Start(self):
        self._t0 = time.perf_counter_ns()

    def Stop(self):
        self._t1 = time.perf_counter_ns()

    def NanoSeconds(self) -> int: return self._t1 - self._t0
    def MicroSeconds(self) -> int: return (self._t1 - self._t0) // 1_000
    def MilliSeconds(self) -> int: return (self._t1 - self._t0) // 1_000_000
    def Seconds(self) -> int: return (self._t1 - self._t0) // 1_000_000_000
