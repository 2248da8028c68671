"""Tracing and latency measurements of the device runtime.

What the reference compiles in with macros is a run-time level here (``--trace-level``):

* ``__NVPROF_MARK_TASK`` / ``__NVPROF_MARK_OPERATOR`` (clib-multigpu/utils.h:13-16, executioncontext.c:562-564,634-636):
  level 1 puts an NVTX range around every task submission, level 2 also one around every operator while a program is
  issued or captured.  NVTX is header-only; without a profiler attached the calls do nothing.
* ``INTRA_TASK_MEASUREMENTS`` (taskhandler.c:40-43, callbackhandler.c:101-104, executioncontext.c:751-772): two timing
  events per task, device time collected when the task's result is read -> ``task_device_ms``.
* ``INTER_TASK_MEASUREMENTS`` (executioncontext.c:566-578): host time between consecutive submissions -> ``inter_arrival_us``.
* ``MAKESPAN_MEASUREMENTS`` (executioncontext.c:582-602, kernels/sleep.cu): every learner's stream is first parked behind a
  sleep kernel so that the whole batch of tasks is queued before the first one starts -> ``makespan_ms``.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

import numpy as np


def _lib():
    from ..ops import lib as L
    return L.init_device()


def enable(level: int = 1):
    _lib().xb_trace_set(int(level))


def level() -> int:
    return int(_lib().xb_trace_level())


def _read(which: int, clear: bool, limit: int = 1 << 20) -> np.ndarray:
    buf = (C.c_float * limit)()
    n = _lib().xb_trace_read(which, buf, limit, int(clear))
    return np.ctypeslib.as_array(buf)[:n].copy()


def task_device_ms(clear: bool = False) -> np.ndarray:
    """Device time of every finished task whose result has been read since the last clear (milliseconds)."""
    return _read(0, clear)


def inter_arrival_us(clear: bool = False) -> np.ndarray:
    """Host time between consecutive task submissions (microseconds)."""
    return _read(1, clear)


def percentiles(v: np.ndarray) -> Dict[str, float]:
    if len(v) == 0:
        return {"n": 0}
    q = np.percentile(v, [5, 25, 50, 75, 95, 99])
    return {"n": int(len(v)), "min": float(v.min()), "p5": float(q[0]), "p25": float(q[1]), "p50": float(q[2]), "p75": float(q[3]),
            "p95": float(q[4]), "p99": float(q[5]), "max": float(v.max()), "mean": float(v.mean())}


def summary(clear: bool = False) -> Dict[str, Dict[str, float]]:
    return {"task_device_ms": percentiles(task_device_ms(clear)), "inter_arrival_us": percentiles(inter_arrival_us(clear))}


def makespan_ms(engine, tasks_per_learner: int = 4, park_ms: float = 20.0) -> float:
    """Queue ``tasks_per_learner`` training tasks on every learner behind a (bounded) sleep kernel, then time from the end
    of the sleep to the end of the last task on the device.  The learners' staging buffers must already hold a batch."""
    from ..ops import lib as L
    lib = engine.lib
    cycles = int(park_ms * 1e-3 * 1.9e9)
    begin = [lib.xb_event_create(1) for _ in engine.learners]
    end = [lib.xb_event_create(1) for _ in engine.learners]
    engine.finish()
    for l, ev in zip(engine.learners, begin):
        L.check(lib.xb_sleep(cycles, l.stream), "sleep")
        L.check(lib.xb_event_record(ev, l.stream), "record")
    task = 0
    for _ in range(tasks_per_learner):
        for l in engine.learners:
            p = engine.params(task, True)
            task += 1
            L.check(lib.xb_learner_submit(l.handle, None, None, C.byref(p), 0), "submit")
    for l, ev in zip(engine.learners, end):
        L.check(lib.xb_event_record(ev, l.stream), "record")
    for ev in end:
        lib.xb_event_sync(ev)
    # all streams leave the sleep within microseconds of each other; the span is first begin -> last end
    span = max(lib.xb_event_elapsed_ms(b, e) for b in begin for e in end)
    for ev in begin + end:
        lib.xb_event_destroy(ev)
    engine.finish()
    return float(span)
