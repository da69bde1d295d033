"""Samples SM clocks, power and throttle reasons of one GPU while a timed region runs. Read-only: nothing here sets,
locks or resets a clock or any other GPU setting.

The sampler is a thread that polls NVML every few milliseconds (``pynvml``; a query costs tens of microseconds, so
even a timed region of a few tens of milliseconds gets several samples). Where NVML cannot be loaded it falls back to
a ``nvidia-smi`` child process that prints the same fields, which samples far more slowly.
"""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading
import time
from typing import Dict, List, Optional, Tuple

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
          "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
          "clocks_event_reasons.sw_power_cap")

# Bits of NVML's clocks-event-reasons mask that the benchmark records (values from nvml.h).
_REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

Sample = Tuple[float, float, float, int]  # SM MHz, max SM MHz, watts, reasons mask


class ClockSampler:
    """``start()`` before the timed region, ``stop()`` after it; ``stop`` returns the summary dictionary.

    ``device`` is a CUDA device index of this process (``CUDA_VISIBLE_DEVICES`` respected: the NVML handle is looked up
    by the device's UUID)."""

    def __init__(self, device: int = 0, period_ms: float = 5.0) -> None:
        self.device, self.period_s = device, period_ms / 1000.0
        self._samples: List[Sample] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._process: Optional[subprocess.Popen] = None
        self._lines: List[str] = []
        self._nvml = None
        self._handle = None

    # -- NVML ---------------------------------------------------------------------------------------------
    def _open_nvml(self) -> bool:
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self._nvml = pynvml
            self._read()  # a query that fails here sends us to the fallback
            return True
        except Exception:
            self._nvml, self._handle = None, None
            return False

    def _read(self) -> Sample:
        nvml, handle = self._nvml, self._handle
        clock = float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM))
        maximum = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
        watts = nvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
        getter = getattr(nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or nvml.nvmlDeviceGetCurrentClocksThrottleReasons
        return clock, maximum, watts, int(getter(handle))

    def _poll(self) -> None:
        while not self._stop.is_set():
            try:
                self._samples.append(self._read())
            except Exception:
                pass
            self._stop.wait(self.period_s)

    # -- nvidia-smi fallback ------------------------------------------------------------------------------
    def _pump(self) -> None:
        assert self._process is not None and self._process.stdout is not None
        for line in self._process.stdout:
            self._lines.append(line.strip())

    def start(self) -> "ClockSampler":
        if self._open_nvml():
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
            return self
        executable = shutil.which("nvidia-smi")
        if executable is None:
            return self
        try:
            self._process = subprocess.Popen(
                [executable, f"--id={self.device}", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._process = None
            return self
        self._thread = threading.Thread(target=self._pump, daemon=True)
        self._thread.start()
        return self

    def mark(self) -> int:
        """Number of samples taken so far (to cut the record into regions afterwards)."""
        return len(self._samples)

    def region(self, first: int, last: Optional[int] = None) -> Dict[str, object]:
        """Summary of the samples between two marks (NVML source only; empty otherwise)."""
        return summarize_samples(self._samples[first:last])

    def stop(self) -> Dict[str, object]:
        self._stop.set()
        if self._process is not None:
            self._process.terminate()  # the exact child started above
            try:
                self._process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._process.kill()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._nvml is not None:
            if not self._samples:  # a region shorter than one period still gets its one sample
                try:
                    self._samples.append(self._read())
                except Exception:
                    pass
            return summarize_samples(self._samples)
        return summarize(self._lines)


def summarize_samples(samples: List[Sample]) -> Dict[str, object]:
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    power = [s[2] for s in samples]
    busy = [s for s in samples if s[2] >= 0.5 * max(power)] or samples
    mask = 0
    for sample in busy:
        mask |= sample[3]
    return {"sm_mhz": statistics.median(s[0] for s in busy), "sm_min_mhz": min(s[0] for s in busy),
            "sm_max_mhz": max(s[1] for s in samples), "reasons": sorted(name for name, bit in _REASON_BITS.items() if mask & bit),
            "samples": len(samples), "samples_under_load": len(busy), "power_w_max": max(power), "source": "nvml"}


def summarize(lines: List[str]) -> Dict[str, object]:
    """The same summary from ``nvidia-smi --query-gpu`` lines."""
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
            "samples": len(clocks), "power_w_max": max(power), "source": "nvidia-smi"}


def sample_once(device: int = 0) -> Dict[str, object]:
    """One reading, for callers that only want to know the state right now."""
    sampler = ClockSampler(device).start()
    time.sleep(0.02)
    return sampler.stop()
