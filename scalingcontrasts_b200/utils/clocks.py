"""Samples SM clocks and throttle reasons with ``nvidia-smi`` while a timed region runs. Read-only: nothing here sets,
locks or resets a clock or any other GPU setting."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading
from typing import Dict, List, Optional

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
          "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
          "clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, device_index: int = 0, period_ms: int = 100) -> None:
        self.device_index, self.period_ms = device_index, period_ms
        self._process: Optional[subprocess.Popen] = None
        self._lines: List[str] = []
        self._thread: Optional[threading.Thread] = None

    def start(self) -> "ClockSampler":
        executable = shutil.which("nvidia-smi")
        if executable is None:
            return self
        try:
            self._process = subprocess.Popen(
                [executable, f"--id={self.device_index}", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._process = None
            return self
        self._thread = threading.Thread(target=self._pump, daemon=True)
        self._thread.start()
        return self

    def _pump(self) -> None:
        assert self._process is not None and self._process.stdout is not None
        for line in self._process.stdout:
            self._lines.append(line.strip())

    def stop(self) -> Dict[str, object]:
        if self._process is not None:
            self._process.terminate()  # the exact child started above
            try:
                self._process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._process.kill()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return summarize(self._lines)


def summarize(lines: List[str]) -> Dict[str, object]:
    clocks, maxima, power, reasons = [], [], [], set()
    names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    for line in lines:
        fields = [f.strip() for f in line.split(",")]
        if len(fields) < 9:
            continue
        try:
            clocks.append(float(fields[1]))
            maxima.append(float(fields[2]))
            power.append(float(fields[3]))
        except ValueError:
            continue
        for name, value in zip(names, fields[5:9]):
            if value.lower().startswith("active"):
                reasons.add(name)
    if not clocks:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    busy = [c for c, w in zip(clocks, power) if w >= 0.5 * max(power)] or clocks
    return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(maxima), "reasons": sorted(reasons),
            "samples": len(clocks), "power_w_max": max(power)}
