"""Read-only sampling of SM clocks and throttle reasons while a benchmark runs.

Only NVML *queries* are used; nothing here changes a setting of the GPU.
"""
from __future__ import annotations

import statistics
import threading
import time


class ClockSampler:
    """Samples ``clocks.sm`` and the clock-event (throttle) reasons of one GPU every
    ``period`` seconds on a background thread between :meth:`start` and :meth:`stop`."""

    _REASONS = {
        0x8: "hw_slowdown",
        0x40: "hw_thermal_slowdown",
        0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int = 0, period: float = 0.1):
        self.idx = device_index
        self.period = period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self.power_w: list[float] = []
        self._stop = threading.Event()
        self._thr = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report empty clocks rather than fail the bench
            self._nvml = None
            return self
        self._stop.clear()
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self._REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self) -> dict:
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
               "samples": len(self.samples)}
        if self.samples:
            out["sm_mhz"] = statistics.median(self.samples)
        if self.power_w:
            out["power_w_max"] = round(max(self.power_w), 1)
        return out
