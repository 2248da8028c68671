"""ctypes binding of ``libxbow_rt.so``: the host-only C++ runtime (scheduler, replica pool, queues, result ring,
watchdog, data-set pipeline, record reader).  It has no CUDA dependency, so it loads and is tested on machines without
a GPU; the device is reached through executor function pointers exported by ``libxbow_cuda.so``."""
from __future__ import annotations

import ctypes as C
from typing import Optional

from ..ops import build as _build

_lib: Optional[C.CDLL] = None


def _sig(lib, name, restype, *argtypes):
    f = getattr(lib, name)
    f.restype, f.argtypes = restype, list(argtypes)
    return f


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    lib = C.CDLL(str(_build.build_rt()))
    P, I, D, L, U = C.c_void_p, C.c_int, C.c_double, C.c_longlong, C.c_ulonglong
    _sig(lib, "rt_create", P, I, I, I, I, I, I, I, D)
    _sig(lib, "rt_destroy", None, P)
    _sig(lib, "rt_set_executor", None, P, P, P, P, P, P)
    _sig(lib, "rt_set_target_loss", None, P, C.c_float)
    _sig(lib, "rt_set_scheduling_policy", None, P, I)
    _sig(lib, "rt_set_run_ahead", None, P, I, P)
    _sig(lib, "rt_set_affinity", None, P, I)
    _sig(lib, "rt_train", L, P, L, I)
    _sig(lib, "rt_drain", I, P, D)
    _sig(lib, "rt_stop", None, P)
    _sig(lib, "rt_add_learner", I, P)
    _sig(lib, "rt_remove_learner", I, P)
    _sig(lib, "rt_learners", I, P)
    _sig(lib, "rt_clock", U, P)
    _sig(lib, "rt_tasks_issued", U, P)
    _sig(lib, "rt_tasks_completed", U, P)
    _sig(lib, "rt_failed", I, P)
    _sig(lib, "rt_error", C.c_char_p, P)
    _sig(lib, "rt_totals", None, P, I, C.POINTER(D), C.POINTER(D), C.POINTER(U), C.POINTER(C.c_float), C.POINTER(C.c_float))
    _sig(lib, "rt_history", I, P, C.POINTER(U), C.POINTER(C.c_float), C.POINTER(C.c_float), I)
    _sig(lib, "rt_history_since", I, P, U, C.POINTER(U), C.POINTER(U), C.POINTER(C.c_float), C.POINTER(C.c_float), I)
    _sig(lib, "rt_history_count", U, P)
    _sig(lib, "rt_history_follow", None, P, I)
    _sig(lib, "rt_bench_mpmc", D, I, I, L)
    _sig(lib, "rt_bench_theta", D, I, L)
    _sig(lib, "rt_taskq_create", P, I)
    _sig(lib, "rt_taskq_destroy", None, P)
    _sig(lib, "rt_taskq_push", None, P, L, I, I, L)
    _sig(lib, "rt_taskq_poll", L, P, I, C.POINTER(I), I, I, L)
    _sig(lib, "rt_taskq_size", I, P)
    _sig(lib, "rt_theta_create", P, I)
    _sig(lib, "rt_theta_destroy", None, P)
    _sig(lib, "rt_theta_next", I, P, D)
    _sig(lib, "rt_theta_release", None, P, I)
    _sig(lib, "rt_theta_expand", I, P)
    _sig(lib, "rt_theta_shrink", I, P, D)
    _sig(lib, "rt_theta_size", I, P)
    _sig(lib, "rt_theta_enabled", I, P)
    _sig(lib, "rt_set_data_source", None, P, P, P, P)
    V = C.POINTER(C.c_void_p)
    _sig(lib, "ds_meta_load", P, C.c_char_p)
    _sig(lib, "ds_meta_free", None, P)
    _sig(lib, "ds_meta_get", L, P, I)
    _sig(lib, "ds_meta_shape", L, P, I)
    _sig(lib, "ds_writer_create", P, C.c_char_p, C.c_char_p, C.c_char_p, L, C.POINTER(L), I, L, I)
    _sig(lib, "ds_writer_append", I, P, P, P, L)
    _sig(lib, "ds_writer_close", I, P)
    _sig(lib, "ds_basic_open", P, C.c_char_p, I, P, P)
    _sig(lib, "ds_basic_batch", I, P, L, V, V, D)
    _sig(lib, "ds_basic_resident_bytes", L, P)
    _sig(lib, "ds_basic_resident_partitions", I, P)
    _sig(lib, "ds_basic_close", None, P)
    _sig(lib, "ds_light_open", P, C.c_char_p, I, I)
    _sig(lib, "ds_light_ring", P, P, I, C.POINTER(L))
    _sig(lib, "ds_light_take", I, P, L, V, V, D)
    _sig(lib, "ds_light_release", None, P, I)
    _sig(lib, "ds_light_close", None, P)
    _sig(lib, "ds_source_create", P, P, I, L, L, D)
    _sig(lib, "ds_source_free", None, P)
    _sig(lib, "rt_cpu_bind", I, I)
    _sig(lib, "rt_cpu_unbind", I)
    _sig(lib, "rt_cpu_id", I)
    _sig(lib, "rt_cpu_count", I)
    _lib = lib
    return lib


_fake_lib: Optional[C.CDLL] = None


def load_fake() -> C.CDLL:
    """Test-only library with the fake executor (it is not part of the runtime library)."""
    global _fake_lib
    if _fake_lib is None:
        lib = C.CDLL(str(_build.build_rt_fake()))
        P, I, U = C.c_void_p, C.c_int, C.c_ulonglong
        _sig(lib, "rt_fake_create", P, I, I)
        _sig(lib, "rt_fake_destroy", None, P)
        _sig(lib, "rt_fake_table", None, C.POINTER(P), C.POINTER(P), C.POINTER(P), C.POINTER(P))
        _sig(lib, "rt_fake_inject", None, P, I, I)
        _sig(lib, "rt_fake_set_task_us", None, P, I)
        _sig(lib, "rt_fake_syncs", U, P)
        _sig(lib, "rt_fake_last_mask", I, P, C.c_char_p, I)
        _fake_lib = lib
    return _fake_lib


class RuntimeError_(RuntimeError):
    """The native runtime stopped with an error (stuck task, failed submission, watchdog deadline ...)."""


class ThetaQueue:
    """Round-robin slot pool with FREE / BUSY / disabled states (clib-multigpu/thetaqueue.c)."""

    def __init__(self, n: int):
        self.lib = load()
        self.h = self.lib.rt_theta_create(n)

    def next(self, timeout_s: float = 1.0) -> int:
        return self.lib.rt_theta_next(self.h, timeout_s)

    def release(self, i: int):
        self.lib.rt_theta_release(self.h, i)

    def expand(self) -> int:
        return self.lib.rt_theta_expand(self.h)

    def shrink(self, timeout_s: float = 1.0) -> int:
        return self.lib.rt_theta_shrink(self.h, timeout_s)

    def size(self) -> int:
        return self.lib.rt_theta_size(self.h)

    def enabled(self) -> int:
        return self.lib.rt_theta_enabled(self.h)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.rt_theta_destroy(self.h)
            self.h = None


class TaskQueue:
    """Ordered task queue with the reference's scheduling policies (task/TaskQueue.java, task/TaskWindow.java:185-227):
    ``FIFO``, ``HLS`` (hybrid latency scheduling between two processors, 0 = CPU and 1 = GPU, driven by a throughput
    matrix ``[2][graphs]`` in tasks per second) and ``NULL`` (never hands out a task)."""

    def __init__(self, policy="FIFO"):
        from ..types import SchedulingPolicy
        self.lib = load()
        self.policy = SchedulingPolicy.from_string(policy) if isinstance(policy, str) else policy
        self.h = self.lib.rt_taskq_create(int(self.policy))

    def push(self, task: int, graph: int = 0, replica: int = -1, clock: int = 0):
        self.lib.rt_taskq_push(self.h, task, graph, replica, clock)

    def poll(self, processor: int, matrix=None, replica: int = -1, clock: int = 1 << 62) -> int:
        """Next task for ``processor`` (or -1).  ``matrix``: two rows of per-graph throughputs."""
        if matrix is None:
            return int(self.lib.rt_taskq_poll(self.h, processor, None, 1, replica, clock))
        graphs = len(matrix[0])
        flat = (C.c_int * (2 * graphs))(*[int(v) for row in matrix for v in row])
        return int(self.lib.rt_taskq_poll(self.h, processor, flat, graphs, replica, clock))

    def __len__(self):
        return int(self.lib.rt_taskq_size(self.h))

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.rt_taskq_destroy(self.h)
            self.h = None


class Runtime:
    """Native scheduler. ``sync_model``: 0 BSP, 1 SSP, 2 ASP."""

    def __init__(self, learners: int, wpc: int, slack: int = 0, sync_model: int = 0, result_slots: int = 2048,
                 task_handlers: int = 0, callback_handlers: int = 1, task_timeout_s: float = 30.0):
        self.lib = load()
        self.h = self.lib.rt_create(learners, wpc, slack, sync_model, result_slots, task_handlers, callback_handlers, task_timeout_s)
        if not self.h:
            raise ValueError("invalid runtime configuration")
        self._fake, self._fake_lib, self._fake_wait_task = None, None, 0

    def set_executor(self, submit: int, wait: int, synchronise: int, batch: int, ctx: int):
        self.lib.rt_set_executor(self.h, submit, wait, synchronise, batch, ctx)

    def set_run_ahead(self, depth: int, wait_task: int = 0):
        """Let every replica hold up to ``depth`` tasks in flight (``wait_task``: address of the executor's per-task wait;
        0 with an attached fake executor uses the fake's)."""
        self.lib.rt_set_run_ahead(self.h, depth, wait_task or self._fake_wait_task)

    def set_data_source(self, source_handle: int):
        """Batches come from a native data set (``crossbow_b200.data.native``) instead of the executor's own ring."""
        addr = lambda name: C.cast(getattr(self.lib, name), C.c_void_p).value
        self.lib.rt_set_data_source(self.h, addr("ds_source_take"), addr("ds_source_release"), source_handle)

    def attach_fake(self, learners: int, task_us: int = 100):
        """Drive this runtime with the fake executor of the test library (host-only tests)."""
        fl = self._fake_lib = load_fake()
        self._fake = fl.rt_fake_create(learners, task_us)
        sub, wait, sync, wt = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        fl.rt_fake_table(C.byref(sub), C.byref(wait), C.byref(sync), C.byref(wt))
        self._fake_wait_task = wt.value
        self.lib.rt_set_executor(self.h, sub.value, wait.value, sync.value, 0, self._fake)
        return self._fake

    def set_fake_task_us(self, task_us: int):
        self._fake_lib.rt_fake_set_task_us(self._fake, int(task_us))

    def inject(self, fail_task: int = -1, hang_task: int = -1):
        self._fake_lib.rt_fake_inject(self._fake, fail_task, hang_task)

    def fake_syncs(self) -> int:
        return self._fake_lib.rt_fake_syncs(self._fake)

    def fake_last_mask(self):
        buf = C.create_string_buffer(256)
        n = self._fake_lib.rt_fake_last_mask(self._fake, buf, 256)
        return list(buf.raw[:n])

    def train(self, ntasks: int, phase: int = 0) -> int:
        n = self.lib.rt_train(self.h, ntasks, phase)
        if n < 0:
            raise RuntimeError_(self.error())
        return n

    def drain(self, timeout_s: float = 60.0):
        if self.lib.rt_drain(self.h, timeout_s) != 0:
            raise RuntimeError_(self.error())

    def stop(self):
        self.lib.rt_stop(self.h)

    def set_scheduling_policy(self, policy):
        """Order in which the task handlers take queued tasks (``--scheduling-policy``: FIFO, HLS or NULL); only matters
        when tasks are queued, i.e. with task handlers."""
        from ..types import SchedulingPolicy
        p = SchedulingPolicy.from_string(policy) if isinstance(policy, str) else policy
        self.lib.rt_set_scheduling_policy(self.h, int(p))

    def set_target_loss(self, t: float):
        self.lib.rt_set_target_loss(self.h, t)

    def add_learner(self) -> int:
        return self.lib.rt_add_learner(self.h)

    def remove_learner(self) -> int:
        return self.lib.rt_remove_learner(self.h)

    def learners(self) -> int:
        return self.lib.rt_learners(self.h)

    def clock(self) -> int:
        return self.lib.rt_clock(self.h)

    def tasks_issued(self) -> int:
        return self.lib.rt_tasks_issued(self.h)

    def tasks_completed(self) -> int:
        return self.lib.rt_tasks_completed(self.h)

    def failed(self) -> bool:
        return bool(self.lib.rt_failed(self.h))

    def error(self) -> str:
        return self.lib.rt_error(self.h).decode()

    def totals(self, reset=False):
        ls, as_, n, ll, la = C.c_double(), C.c_double(), C.c_ulonglong(), C.c_float(), C.c_float()
        self.lib.rt_totals(self.h, int(reset), C.byref(ls), C.byref(as_), C.byref(n), C.byref(ll), C.byref(la))
        return dict(loss_sum=ls.value, acc_sum=as_.value, n=n.value, last_loss=ll.value, last_acc=la.value)

    def history(self, n: int = 1024):
        t, l, a = (C.c_ulonglong * n)(), (C.c_float * n)(), (C.c_float * n)()
        m = self.lib.rt_history(self.h, t, l, a, n)
        return [(t[i], l[i], a[i]) for i in range(m)]

    def history_since(self, seq: int, n: int = 4096):
        """Results number ``seq``, ``seq + 1``, ... in collection order (every collected result has a sequence number,
        counted from 0).  Returns ``(first, records)``; ``first > seq`` means the reader fell behind the ring and the
        records in between are gone."""
        t, l, a, first = (C.c_ulonglong * n)(), (C.c_float * n)(), (C.c_float * n)(), C.c_ulonglong()
        m = self.lib.rt_history_since(self.h, seq, C.byref(first), t, l, a, n)
        return first.value, [(t[i], l[i], a[i]) for i in range(m)]

    def follow_history(self, on: bool):
        """While on, the runtime never overwrites a result that `history_since` has not returned yet (it waits for the
        reader), so a monitor that keeps reading loses nothing however long the run is."""
        self.lib.rt_history_follow(self.h, int(on))

    def results_collected(self) -> int:
        return int(self.lib.rt_history_count(self.h))

    def close(self):
        if self.h:
            self.lib.rt_destroy(self.h)
            self.h = None
        if self._fake:
            self._fake_lib.rt_fake_destroy(self._fake)
            self._fake = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def cpu_bind(core: int) -> int:
    return load().rt_cpu_bind(core)


def cpu_unbind() -> int:
    return load().rt_cpu_unbind()


def cpu_id() -> int:
    return load().rt_cpu_id()
