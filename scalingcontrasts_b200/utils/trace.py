"""Optional NVTX ranges around the phases of a step (publish, barrier, each scored block, finish, reductions, the
projector and optimizer phases of a training step), for timeline tools. Off by default: with ``SC_NVTX=1`` in the
environment (or ``enable()``) every ``phase(...)`` pushes and pops a range; otherwise it costs one attribute test.

The reference has no tracing of any kind (its only instrument is the wall-clock harness, scalingcontrasts.cu:116-131).
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Iterator

_enabled = os.environ.get("SC_NVTX", "0") == "1"


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


@contextmanager
def phase(name: str) -> Iterator[None]:
    if not _enabled:
        yield
        return
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
