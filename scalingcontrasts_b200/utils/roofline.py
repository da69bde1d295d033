"""Roofline denominators and the fractions the benchmark rows report.

The denominators are a machine's measured copy bandwidth and cuBLAS bf16 throughput, read from a small JSON file with
the keys ``hbm_gbs``, ``bf16_tflops`` (a burst measurement: the right denominator for a kernel timed in isolation) and
``bf16_tflops_sustained`` (a seconds-long loop under the power cap: the right one for a step timed inside a long run).
The file is named explicitly (``load_peaks(path)``), or by the environment variable ``SC_MEASURED_PEAKS``, or it is a
``MEASURED_PEAKS.json`` in the working directory; without one the figures of an earlier measurement on the same kind
of GPU are used and labelled ``fallback``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
FALLBACK_BF16_TFLOPS_SUSTAINED = 1400.0
NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy; 900 nominal


@dataclass(frozen=True)
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    source: str  # "measured" or "fallback"


def load_peaks(path: Optional[str] = None) -> Peaks:
    candidates = [path] if path else [os.environ.get("SC_MEASURED_PEAKS"), os.path.join(os.getcwd(), "MEASURED_PEAKS.json")]
    for candidate in candidates:
        if not candidate:
            continue
        try:
            with open(candidate) as handle:
                data = json.load(handle)
            return Peaks(float(data["hbm_gbs"]), float(data["bf16_tflops"]),
                         float(data.get("bf16_tflops_sustained", data["bf16_tflops"])), "measured")
        except (OSError, KeyError, ValueError):
            if path:
                raise
    return Peaks(FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, FALLBACK_BF16_TFLOPS_SUSTAINED, "fallback")


def loss_step_flops(rows: int, world_rows: int, hidden: int) -> float:
    """Tensor-core flops one rank spends per step: every channel once forward and once backward for each cell."""
    return 2.0 * (2.0 * hidden) * rows * world_rows


def loss_step_roofline_ms(rows: int, world: int, hidden: int, peaks: Peaks, sustained: bool = True) -> float:
    """The slower of the rank's tensor-core time and its peer pulls at link bandwidth. A step row is timed over windows of
    whole steps in a long run, so its tensor-core time is taken at the sustained peak; ``sustained=False`` gives the bound
    at the burst peak, for a kernel timed alone."""
    tflops = peaks.bf16_tflops_sustained if sustained else peaks.bf16_tflops
    compute_ms = loss_step_flops(rows, world * rows, hidden) / (tflops * 1e12) * 1e3
    pull_ms = (world - 1) * rows * hidden * 2 / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3
    return max(compute_ms, pull_ms)
