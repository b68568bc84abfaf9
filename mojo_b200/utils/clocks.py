"""Read-only sampling of GPU clocks and throttle reasons through NVML while a benchmark runs.
Nothing here changes a device setting."""
from __future__ import annotations

import statistics
import threading

_REASONS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
    0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
}


class ClockSampler:
    """`with ClockSampler(device_index) as cs: ...; cs.summary()` -> {"sm_mhz", "sm_max_mhz", "reasons", ...}."""

    def __init__(self, index: int = 0, period_s: float = 0.1):
        self.index, self.period = index, period_s
        self.samples: list[tuple[int, int, float]] = []
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        self.sm_max = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001  (no NVML: the summary says so)
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:  # noqa: BLE001
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                power = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                self.samples.append((mhz, reasons, power))
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return False

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        mask = 0
        for _, r, _ in self.samples:
            mask |= r
        reasons = sorted(name for bit, name in _REASONS.items() if mask & bit and name != "gpu_idle")
        return {
            "sm_mhz": statistics.median(s[0] for s in self.samples),
            "sm_max_mhz": self.sm_max,
            "reasons": reasons,
            "power_w_max": max(s[2] for s in self.samples),
            "samples": len(self.samples),
        }
