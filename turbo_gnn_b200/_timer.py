"""CUDA-event timing of a zero-argument callable (used by the inline autotuner).

Same contract as the reference's ``turbo_gnn/_timer.py:19-50``: warm up, then time ``iters``
back-to-back calls between two events on the current stream and report the mean.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass
class TimerResult:
    """Mean time of one call in milliseconds over ``iters`` calls."""

    iters: int
    ms_per_iter: float


def time_callable(fn: Callable[[], Any], warmup: int = 10, iters: int = 50) -> TimerResult:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    begin = torch.cuda.Event(enable_timing=True)
    finish = torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        fn()
    finish.record()
    torch.cuda.synchronize()
    return TimerResult(iters=iters, ms_per_iter=begin.elapsed_time(finish) / max(iters, 1))
