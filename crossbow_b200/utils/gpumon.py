"""GPU sampler + percentile summary (tools/measurements/gpu-measurements.sh:33-63, parse-measurements.py): samples
utilisation, memory, power and SM clock every ``period`` seconds through NVML (read-only) on a background thread."""
import threading
import time
from typing import Dict, List


class GpuMonitor(threading.Thread):
    FIELDS = ("util", "mem_util", "mem_used_mb", "power_w", "sm_mhz")

    def __init__(self, index: int = 0, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.rows: List[tuple] = []
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        while not self._stop.is_set():
            try:
                u = nv.nvmlDeviceGetUtilizationRates(self.h)
                m = nv.nvmlDeviceGetMemoryInfo(self.h)
                self.rows.append((time.time(), u.gpu, u.memory, m.used / 1e6, nv.nvmlDeviceGetPowerUsage(self.h) / 1e3,
                                  nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        self.join(timeout=2)

    def csv(self) -> str:
        return "\n".join(["timestamp," + ",".join(self.FIELDS)] + [",".join(f"{v:.3f}" for v in r) for r in self.rows])

    def summary(self) -> Dict[str, Dict[str, float]]:
        import numpy as np
        out = {}
        for i, f in enumerate(self.FIELDS, 1):
            v = np.array([r[i] for r in self.rows], dtype=float)
            if v.size:
                out[f] = {"mean": float(v.mean()), "p5": float(np.percentile(v, 5)), "p50": float(np.percentile(v, 50)),
                          "p95": float(np.percentile(v, 95)), "max": float(v.max())}
        return out


class ClockSampler(threading.Thread):
    """Samples the SM clock, its maximum and the throttle reasons through NVML (read-only) while a timed region runs;
    `summary()` is the record the benchmarks print next to their numbers."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.stop_flag = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self.stop_flag.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self.stop_flag.set()
        self.join(timeout=2)
        return self.summary()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}
