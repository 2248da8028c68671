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


# ---- the reference's measurement tools as commands ------------------------------------------------------------------------
# tools/measurements/gpu-measurements.sh:33-63 logs `nvidia-smi --query-gpu=timestamp,gpu_serial,temperature.gpu,
# utilization.gpu,utilization.memory,memory.used,memory.free --format=csv,nounits -lms 200` to a file, and
# parse-measurements.py prints min / mean / max / p5 / p25 / p50 / p75 / p99 / std of GPU and memory utilisation per device,
# optionally between two moments (milliseconds since the epoch).  `sampler_command` returns the same command line (reading
# only), `parse_measurements` reads such a log.
QUERY = ("timestamp", "gpu_serial", "temperature.gpu", "utilization.gpu", "utilization.memory", "memory.used", "memory.free")


def sampler_command(period_ms: int = 200):
    return ["nvidia-smi", "--query-gpu=" + ",".join(QUERY), "--format=csv,nounits", "-lms", str(int(period_ms))]


def _stats(values):
    import numpy as np
    v = np.asarray(values, dtype=float)
    return {"min": float(v.min()), "mean": float(v.mean()), "max": float(v.max()), "p5": float(np.percentile(v, 5)),
            "p25": float(np.percentile(v, 25)), "p50": float(np.percentile(v, 50)), "p75": float(np.percentile(v, 75)),
            "p99": float(np.percentile(v, 99)), "std": float(v.std())}


def parse_measurements(path: str, start_ms: int = 0, end_ms: int = 0, idle_below: float = 1.0):
    """{serial: {"gpu_util": stats, "mem_util": stats, "mem_used_mb": stats, "temperature": stats, "samples": n}} plus the
    key "all" over the devices that were busy (mean GPU utilisation of at least `idle_below` %, as the reference's parser
    leaves idle devices out of its aggregate).  Lines outside [start_ms, end_ms] are skipped when a bound is given."""
    from datetime import datetime
    per: Dict[str, Dict[str, list]] = {}
    with open(path) as f:
        for line in f:
            if line.startswith(("timestamp", "#")) or not line.strip():
                continue
            s = [x.strip() for x in line.split(",")]
            if len(s) < 7:
                continue
            try:
                t = int(datetime.strptime(s[0], "%Y/%m/%d %H:%M:%S.%f").timestamp() * 1000)
                temp, gu, mu, used = float(s[2]), float(s[3]), float(s[4]), float(s[5])
            except ValueError:
                continue
            if (start_ms and t < start_ms) or (end_ms and t > end_ms):
                continue
            d = per.setdefault(s[1], {"gpu_util": [], "mem_util": [], "mem_used_mb": [], "temperature": []})
            d["gpu_util"].append(gu), d["mem_util"].append(mu), d["mem_used_mb"].append(used), d["temperature"].append(temp)
    out = {}
    busy_g, busy_m = [], []
    for serial, d in per.items():
        out[serial] = {k: _stats(v) for k, v in d.items()}
        out[serial]["samples"] = len(d["gpu_util"])
        if out[serial]["gpu_util"]["mean"] >= idle_below:
            busy_g += d["gpu_util"]
            busy_m += d["mem_util"]
    if busy_g:
        out["all"] = {"gpu_util": _stats(busy_g), "mem_util": _stats(busy_m), "samples": len(busy_g)}
    return out


def main(argv=None):
    """python -m crossbow_b200.utils.gpumon sample [file]  |  python -m crossbow_b200.utils.gpumon parse <file> [--start ms] [--end ms]"""
    import argparse
    import json
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("what", choices=["sample", "parse"])
    ap.add_argument("file", nargs="?", default="measurements.csv")
    ap.add_argument("--start", type=int, default=0), ap.add_argument("--end", type=int, default=0)
    ap.add_argument("--period-ms", type=int, default=200)
    a = ap.parse_args(argv)
    if a.what == "parse":
        stats = parse_measurements(a.file, a.start, a.end)
        for key, d in stats.items():
            for metric in ("gpu_util", "mem_util"):
                v = d[metric]
                print(f"{key} {metric} " + " ".join(f"{v[k]:7.3f}" for k in ("min", "mean", "max", "p5", "p25", "p50", "p75", "p99", "std")))
        print(json.dumps({k: d["samples"] for k, d in stats.items()}))
        return 0
    import os
    import shutil
    if os.path.exists(a.file):
        raise SystemExit(f"error: {a.file} already exists")
    if shutil.which("nvidia-smi") is None:
        raise SystemExit("error: nvidia-smi is not on this machine's PATH")
    with open(a.file, "w") as f:
        f.write(f"# {time.ctime()}\n")
        f.flush()
        # this process BECOMES the sampler (so that stopping it stops nvidia-smi): it runs until interrupted and only reads
        os.dup2(f.fileno(), 1)
        os.dup2(f.fileno(), 2)
        cmd = sampler_command(a.period_ms)
        os.execvp(cmd[0], cmd)


if __name__ == "__main__":
    raise SystemExit(main())
