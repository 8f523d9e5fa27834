"""Read-only sampling of SM clocks, power and throttle reasons while a benchmark runs.

Polls NVML from a background thread (about once per millisecond, so that even a timed
region of a few milliseconds gets samples) and reports the median SM clock over a given
time window.  Nothing here changes any GPU setting.
"""

import threading
import time

_REASONS = {
    "hw_slowdown": 0x8,
    "sw_power_cap": 0x4,
    "sw_thermal_slowdown": 0x20,
    "hw_thermal_slowdown": 0x40,
}


class NvmlSampler:
    def __init__(self, gpu_index: int, period_s: float = 0.001):
        self.gpu = gpu_index
        self.period = period_s
        self.samples = []          # (t, sm_mhz, power_w, reasons_mask)
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report that instead of numbers
            self._error = f"nvml unavailable: {e}"
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _physical_index(self):
        import os
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                pw = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                self.samples.append((time.perf_counter(), sm, pw, mask))
            except Exception as e:
                self._error = f"nvml read failed: {e}"
                return
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, t0: float, t1: float):
        """Median SM MHz and the throttle reasons seen between host times t0 and t1
        (perf_counter); falls back to the busiest half of all samples when the window is
        shorter than the sampling period."""
        if self._error and not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [self._error], "samples": 0}
        win = [s for s in self.samples if t0 <= s[0] <= t1]
        scope = "timed region"
        if not win:
            hot = sorted(self.samples, key=lambda s: s[2])[len(self.samples) // 2:]
            win, scope = hot, "busiest half of the run (timed region shorter than the sampling period)"
        if not win:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"], "samples": 0}
        sm = sorted(s[1] for s in win)
        mask = 0
        for s in win:
            mask |= s[3]
        reasons = sorted(name for name, bit in _REASONS.items() if mask & bit)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.sm_max, "reasons": reasons, "samples": len(win),
                "power_w_max": max(s[2] for s in win), "scope": scope, "samples_total": len(self.samples)}
