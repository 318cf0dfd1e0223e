"""Sampling of SM clocks and throttle reasons through NVML while a timed region runs.

Only reads device state; nothing here sets clocks, power limits or any other device setting."""
from __future__ import annotations

import statistics
import threading
import time
from typing import Dict, List, Optional


class ClockSampler:
    """Background thread that polls NVML every ``period_s`` seconds between ``start()`` and ``stop()``."""

    _REASONS = (
        ("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20),
        ("hw_thermal_slowdown", 0x40), ("hw_power_brake", 0x80),
    )

    def __init__(self, device_index: int = 0, period_s: float = 0.05, nvml=None) -> None:
        self.idx = device_index
        self.period = period_s
        self.samples: List[int] = []
        self.reason_bits = 0
        self.max_mhz = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._nvml = nvml
        self._handle = None

    def _open(self) -> bool:
        try:
            if self._nvml is None:
                import pynvml
                self._nvml = pynvml
            self._nvml.nvmlInit()
            self._handle = self._nvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = int(self._nvml.nvmlDeviceGetMaxClockInfo(self._handle, self._nvml.NVML_CLOCK_SM))
            return True
        except Exception:
            self._handle = None
            return False

    def _loop(self) -> None:
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
                self.reason_bits |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                try:
                    self.reason_bits |= int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                except Exception:
                    pass
            self._stop.wait(self.period)

    def start(self) -> "ClockSampler":
        if self._open():
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def stop(self) -> Dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            self._thread = None
        reasons = [name for name, bit in self._REASONS if self.reason_bits & bit]
        return {"sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz or None, "reasons": reasons, "samples": len(self.samples)}
