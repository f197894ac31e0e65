"""Read-only sampling of GPU clocks and throttle reasons while a benchmark runs (NVML)."""

from __future__ import annotations

import statistics
import threading
import time

_REASONS = {
    0x1: "gpu_idle",
    0x2: "applications_clocks_setting",
    0x4: "sw_power_cap",
    0x8: "hw_slowdown",
    0x10: "sync_boost",
    0x20: "sw_thermal_slowdown",
    0x40: "hw_thermal_slowdown",
    0x80: "hw_power_brake_slowdown",
    0x100: "display_clock_setting",
}


class ClockSampler:
    """Background thread polling SM clock, power and clock-event reasons of one device."""

    def __init__(self, device_index: int = 0, period_s: float = 0.2):
        self.idx, self.period = device_index, period_s
        self.samples: list[tuple[int, float, int]] = []
        self._stop = threading.Event()
        self._thread = None
        self.sm_max = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.samples.append((sm, pw, rs))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        busy = [s for s in self.samples if not (s[2] & 0x1)] or self.samples
        mask = 0
        for s in busy:
            mask |= s[2]
        reasons = sorted(name for bit, name in _REASONS.items() if mask & bit and name != "gpu_idle")
        return {
            "sm_mhz": statistics.median(s[0] for s in busy),
            "sm_max_mhz": self.sm_max,
            "power_w_max": max(s[1] for s in busy),
            "reasons": reasons,
            "samples": len(busy),
        }
