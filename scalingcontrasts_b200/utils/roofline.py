"""Roofline denominators and the two fractions the benchmark rows report.

The denominators are the machine's measured copy bandwidth and cuBLAS bf16 throughput when a ``MEASURED_PEAKS.json``
sits beside the package (it is written by the measuring harness of the pool, not by this library); otherwise the
fallback figures of an earlier measurement on the same kind of GPU are used and labelled as such.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy; 900 nominal


@dataclass(frozen=True)
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    source: str  # "measured" or "fallback"


def load_peaks() -> Peaks:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            data = json.load(handle)
        return Peaks(float(data["hbm_gbs"]), float(data["bf16_tflops"]),
                     float(data.get("bf16_tflops_sustained", data["bf16_tflops"])), "measured")
    except (OSError, KeyError, ValueError):
        return Peaks(FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, 1400.0, "fallback")


def loss_step_flops(rows: int, world_rows: int, hidden: int) -> float:
    """Tensor-core flops one rank spends per step: every channel once forward and once backward for each cell."""
    return 2.0 * (2.0 * hidden) * rows * world_rows


def loss_step_roofline_ms(rows: int, world: int, hidden: int, peaks: Peaks) -> float:
    """The slower of the rank's tensor-core time at the measured peak and its peer pulls at link bandwidth."""
    compute_ms = loss_step_flops(rows, world * rows, hidden) / (peaks.bf16_tflops * 1e12) * 1e3
    pull_ms = (world - 1) * rows * hidden * 2 / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3
    return max(compute_ms, pull_ms)
