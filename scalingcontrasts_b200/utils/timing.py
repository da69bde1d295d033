"""Timing harness: CUDA events on the launching stream, windows of calls, minimum and median, maximum over ranks.

Parity: ``time_steps`` / ``timing_t`` (scalingcontrasts.cu:111-131), which uses the host clock around drained windows;
here each window is bracketed by events and multi-GPU numbers are the maximum over ranks.
"""
from __future__ import annotations

import statistics
import time
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch


@dataclass
class Timing:
    min_ms: float
    median_ms: float
    samples: List[float]


def time_windows(step: Callable[[], None], windows: int, calls: int, device=None, before_window: Optional[Callable[[], None]] = None,
                 group=None) -> Timing:
    """Per-call milliseconds over ``windows`` windows of ``calls`` calls each, device-timed; with a process group the
    per-window time is the maximum over ranks."""
    cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
    samples: List[float] = []
    for _ in range(windows):
        if before_window is not None:
            before_window()
        if cuda:
            torch.cuda.synchronize(device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(calls):
                step()
            stop.record()
            stop.synchronize()
            elapsed = start.elapsed_time(stop) / calls
        else:
            begin = time.perf_counter()
            for _ in range(calls):
                step()
            elapsed = (time.perf_counter() - begin) * 1e3 / calls
        samples.append(max_over_ranks(elapsed, group, device))
    ordered = sorted(samples)
    return Timing(ordered[0], ordered[len(ordered) // 2], samples)


def max_over_ranks(value: float, group=None, device=None) -> float:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value
    backend = dist.get_backend(group)
    where = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    tensor = torch.tensor([value], dtype=torch.float64, device=where)
    dist.all_reduce(tensor, op=dist.ReduceOp.MAX, group=group)
    return float(tensor.item())


def median(values: List[float]) -> float:
    return statistics.median(values) if values else float("nan")


class L2Flusher:
    """Writes a buffer larger than the L2 cache, so that a timed call does not start on warm lines."""

    def __init__(self, device, nbytes: int = 256 << 20) -> None:
        self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.value = 0

    def __call__(self) -> None:
        self.value = (self.value + 1) % 251
        self.buffer.fill_(self.value)
