"""``ExecutionContext``: the public entry point that trains and tests a model.

API follows the reference (ExecutionContext.java:92-622): ``init()``, ``train(n, unit)``, ``trainAndTest(n, unit)``,
``test()``, ``trainForDuration``, ``trainUntilCondition``, ``trainUntilConditionOrForDuration``, ``destroy()``.

Units on several GPUs (one process per GPU): task counts, `--wpc`, epochs, step values, display and test intervals are
those of the JOB, as in the reference's single process over all GPUs (ExecutionContext.java:257-283,
solverconfiguration.c:116-161).  Rank r of G runs the job's tasks r, G + r, 2 G + r, ... and so issues 1/G of every
count (rounded up); `train(N, "epochs")` is N passes over the data whatever G is.

Scheduling model (what the reference spreads over the dispatcher, task queue, task/callback handler threads, the
result collector and the model manager): tasks are numbered by a ``WorkClock``; each task goes to the next learner
in round-robin order whose replica clock satisfies the staleness bound, the learner's previous result is collected
first (that is the replica "lock"), the batch is copied from pinned host memory on the learner's stream and the
task graph is launched.  Every ``wpc`` tasks the synchronisation step is enqueued on the synchronisation stream;
ordering between tasks and synchronisation is expressed with CUDA events only, the host never blocks for it.
"""
from __future__ import annotations

import threading
import time
from typing import List, Optional

import numpy as np

from .conf import ModelConf, SystemConf
from .graph import Dataflow
from .model import Model, Shape
from .types import DurationUnit, Phase, SynchronisationModel, TrainingUnit, UpdateModel
from .utils.measure import MeasurementQueue, PerformanceMonitor
from .workclock import WorkClock
from .autotune import AutoTuner


class ExecutionContext:
    def __init__(self, dataflows: List[Optional[Dataflow]], system_conf: Optional[SystemConf] = None,
                 model_conf: Optional[ModelConf] = None, input_shape=None, quiet=False):
        self.dataflows = list(dataflows) + [None] * (2 - len(dataflows))
        self.sys = system_conf or SystemConf.getInstance()
        self.mc = model_conf or ModelConf.getInstance()
        self.input_shape = list(input_shape) if input_shape is not None else None
        self.model = Model()
        self.engine = None
        self.clock: Optional[WorkClock] = None
        self.quiet = quiet
        self.measurements = MeasurementQueue()          # every training result
        self.displayed = MeasurementQueue()             # what `--queue-measurements` keeps: one record per display interval
        self._disp_n, self._disp_loss, self._disp_acc = 0, 0.0, 0.0
        self.monitor: Optional[PerformanceMonitor] = None
        self.autotuner: Optional[AutoTuner] = None
        self._call_rate = 0.0                             # tasks/s of the last call of the native training loop
        self._tune = {"tasks": 0, "time": 0.0, "settle": 0, "rate": 0.0}   # since the last decision; tasks/s of the last chunk
        self.autotune_chunks = []                         # (replicas, tasks, seconds, settling) of every chunk issued while tuning
        self.autotune_trace = []                          # (replicas per GPU after the decision, job examples/s it was based on)
        self.rank, self.world = 0, 1
        self.tasks_done = 0
        self.last_loss = float("nan")
        self.last_accuracy = float("nan")
        self.test_accuracy = float("nan")
        self._next_learner = 0
        self._checkpoint_version = 0
        self._native = self._native_test = None
        self._hist_seq, self.results_lost = 0, 0         # native scheduler: results read so far / overwritten before they were read
        self._pump_lock = threading.Lock()
        self.emit = lambda line: print(line, flush=True)  # where display and monitor lines go

    # ---- set-up ----
    def init(self):
        sys, mc = self.sys, self.mc
        train_df, test_df = self.dataflows[0], self.dataflows[1]
        if train_df is None:
            raise ValueError("error: a training dataflow is required")
        ds = mc.getDataset(Phase.TRAIN)
        if self.input_shape is None:
            if ds is None:
                raise ValueError("error: neither an input shape nor a training data set is given")
            self.input_shape = list(ds.example_shape)
        while len(self.input_shape) < 3:
            self.input_shape.append(1)
        batch = mc.batch_size
        ishape, lshape = Shape([batch] + self.input_shape), Shape([batch])
        nid = train_df.executable().init(ishape, lshape, self.model, 0)
        self.model.finalise()
        if test_df is not None:
            test_df.executable().init(ishape, lshape, self.model, nid)
        solver = mc.getSolverConf()
        if ds is not None:
            solver.set_tasks_per_epoch(mc.numberOfTasksPerEpoch(Phase.TRAIN))
        init = self.model.initial_values(sys.random_seed)
        from .parallel.peer import dist_info
        self.rank, self.world, local = dist_info()
        # `--wpc` counts the job's tasks between two synchronisations; this process issues its share of them
        wpc = self._local(mc.wpc_in_tasks())
        if mc.wpc_in_tasks() % self.world and not self.quiet:
            print(f"warning: --wpc {mc.wpc_in_tasks()} is not a multiple of the {self.world} GPUs; every GPU runs {wpc} tasks per clock", flush=True)
        tg = train_df.executable()                       # (a chain of sub-graphs runs as one program)
        sg = test_df.executable() if test_df is not None else None
        if sys.gpu:
            from .engine import GpuEngine
            if sys.number_of_gpu_streams not in (1, sys.number_of_gpu_models) and not self.quiet:
                # (the reference warns when the two differ, executioncontext.c:1724-1725; here a learner IS a replica bound to
                # its own stream, so the replica count decides)
                print(f"warning: --number-of-gpu-streams {sys.number_of_gpu_streams} is ignored: every one of the "
                      f"{sys.number_of_gpu_models} replicas has its own stream", flush=True)
            if sys.trace_level > 0:                      # before the task programs are captured (operator ranges)
                from .utils import trace
                trace.enable(sys.trace_level)
            self.engine = GpuEngine(tg, sg, self.model, init, batch, self.input_shape, solver, mc.update_model,
                                    replicas=sys.number_of_gpu_models, wpc=wpc, rank=self.rank, world=self.world,
                                    device_index=local, use_graphs=sys.use_cuda_graphs, seed=sys.random_seed,
                                    use_tc=sys.use_tensor_cores, fused_sync=sys.fused_sync,
                                    sync_timeout_s=sys.sync_timeout, splits=mc.splits, reuse_memory=sys.reuse_memory,
                                    gradient_buckets=sys.gradient_buckets, debug_canaries=sys.debug_canaries,
                                    overlap_sync=sys.overlap_sync, operator_branches=sys.operator_branches, nvls_sync=sys.nvls_sync)
            if sys.debug_checksums and not self.quiet:
                print("warning: --debug-checksums prints the CPU engine's operator outputs; the device program fuses operators "
                      "(compare device and CPU group by group with tests/test_gpu_groups.py)", flush=True)
        else:
            from .engine import CpuEngine
            self.engine = CpuEngine(tg, sg, self.model, init, batch, self.input_shape, solver, mc.update_model,
                                    replicas=sys.number_of_cpu_models, wpc=wpc, devices=1, seed=sys.random_seed,
                                    splits=mc.splits, rank=self.rank, world=self.world)
            if sys.debug_checksums:                       # (Operator.java:232-259: one line per operator and task)
                from .oracle import OracleExecutor
                OracleExecutor.checksum_sink = lambda line: self.emit(line)
        self.clock = WorkClock(wpc)
        self.monitor = PerformanceMonitor(batch, ds.batch_bytes() if ds is not None else 0, sys.monitor_interval / 1000.0,
                                          sink=None if self.quiet else (lambda line: self.emit(line)))
        self.monitor.queue_size = self.getExecutorQueueSize
        if sys.autotune_models:
            self.autotuner = AutoTuner(sys.autotune_threshold, sys.autotune_interval)
        if sys.model_directory:
            from .checkpoint import load_checkpoint
            load_checkpoint(self, sys.model_directory)
        self._native = self._native_test = None
        if sys.gpu and sys.native_scheduler and sys.fused_sync and (hasattr(ds, "examples") or hasattr(ds, "source")):
            self._setup_native()
        if self.world > 1:
            # lowering and graph capture take seconds and not the same number on every rank; the first synchronisation's
            # device-side waits are bounded, so the ranks leave init() together
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                if sys.gpu:
                    import torch
                    torch.cuda.synchronize()
                dist.barrier()
        return self

    def _setup_native(self):
        """Hand scheduling to the C++ runtime: dispatcher + handler threads call the CUDA executor directly."""
        from .runtime import Runtime
        sys, mc, e = self.sys, self.mc, self.engine
        test_ds = mc.getDataset(Phase.CHECK) if self.dataflows[1] is not None else None
        if test_ds is not None and not (hasattr(test_ds, "examples") or hasattr(test_ds, "source")):
            test_ds = None
        ctx, sub, wait, sync, batch = e.native_executor(mc.getDataset(Phase.TRAIN), test_ds)
        handlers = 0 if sys.direct_scheduling else max(0, sys.number_of_task_handlers - 1)
        mk = lambda wpc: Runtime(learners=e.k, wpc=wpc, slack=mc.slack, sync_model=int(sys.synchronisation_model),
                                 result_slots=sys.number_of_result_slots, task_handlers=handlers,
                                 callback_handlers=max(1, sys.number_of_callback_handlers), task_timeout_s=sys.task_timeout)
        self._native = mk(self.clock.wpc)
        self._native.set_scheduling_policy(sys.scheduling_policy)
        self._native.set_executor(sub, wait, sync, batch, ctx)
        if sys.run_ahead > 1:
            # the next task of a replica is handed to the device while the previous one is still running
            self._native.set_run_ahead(sys.run_ahead, e.native_wait_task())
        train_ds = mc.getDataset(Phase.TRAIN)
        if hasattr(train_ds, "source"):              # C++ data set: batches go from its ring to the device without Python
            self._native.set_data_source(train_ds.source(stride=self.world, offset=self.rank, timeout_s=sys.task_timeout))
        if test_ds is not None:
            self._native_test = mk(1 << 30)          # test tasks never synchronise
            self._native_test.set_executor(sub, wait, 0, batch, ctx)
            if hasattr(test_ds, "source"):
                self._native_test.set_data_source(test_ds.source(stride=1, offset=0, timeout_s=sys.task_timeout))

    def _pump_results(self) -> int:
        """Native scheduler: read the results collected since the last call, in collection order, and pass them to the
        display, the measurement queue and the monitor.  Called by the monitor thread while `train` runs and once more
        when it has returned, so display lines and `[MON]` lines appear while training is in progress
        (result/TrainingResultHandler.java:231-317, PerformanceMonitor.java:59-104)."""
        rt, n = self._native, 0
        if rt is None:
            return 0
        with self._pump_lock:
            while True:
                first, recs = rt.history_since(self._hist_seq, 8192)
                if first > self._hist_seq:
                    self.results_lost += first - self._hist_seq      # the reader fell a whole ring behind
                for task, loss, acc in recs:
                    self.measurements.add(task, loss, acc)
                    self._display(task, loss, acc)
                self._hist_seq = first + len(recs)
                n += len(recs)
                if recs:
                    self.last_loss, self.last_accuracy = recs[-1][1], recs[-1][2]
                    self.monitor.task_done(len(recs))
                if len(recs) < 8192:
                    return n

    def _job_rate(self, images_per_second: float) -> float:
        """Throughput of the whole job: the sum over the GPUs, identical on every rank, so that the auto-tuner takes ONE
        decision for the job (the reference is one process with one monitor, ModelManager.java:257-274)."""
        if self.world <= 1:
            return images_per_second
        import torch
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return images_per_second
        dev = "cuda" if (self.sys.gpu and dist.get_backend() == "nccl") else "cpu"
        t = torch.tensor([images_per_second], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        return float(t.item())

    def _slowest(self, seconds: float) -> float:
        """The largest of the ranks' values (the value itself in a one-process job)."""
        if self.world <= 1:
            return seconds
        import torch
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return seconds
        dev = "cuda" if (self.sys.gpu and dist.get_backend() == "nccl") else "cpu"
        t = torch.tensor([seconds], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def _autotune(self, samples, rt=None) -> int:
        """One auto-tuner decision, applied to the engine (and the native runtimes); returns the change in replicas."""
        e = self.engine
        delta = self.autotuner.decide(samples)
        if delta > 0 and e.k < 16:
            e.add_learner()
            for r in (rt, self._native_test if rt is not None else None):
                if r is not None:
                    r.add_learner()
            if not self.quiet:
                print(f"[autotune] {samples[-1]:.1f} examples/s: +1 replica -> {e.k}", flush=True)
        elif delta < 0:
            for r in (rt, self._native_test if rt is not None else None):
                if r is not None:
                    r.remove_learner()
            e.remove_learner()
            if not self.quiet:
                print(f"[autotune] {samples[-1]:.1f} examples/s: -1 replica -> {e.k}; tuning stops", flush=True)
        self.autotune_trace.append((e.k, float(samples[-1]) if samples else 0.0))
        return delta

    def _train_native(self, ntasks: int) -> int:
        rt, e = self._native, self.engine
        e.epoch_to_native()
        wpc = self.clock.wpc
        ci = self.sys.checkpoint_interval if self.sys.checkpoint_directory else 0
        done = 0
        tune = self._tune                                   # sampling state of the auto-tuner: outlives the call, as the
                                                            # reference's monitor thread does (PerformanceMonitor.java:59-104)
        stop = threading.Event()
        period = max(0.01, min(0.2, self.sys.monitor_interval / 1000.0 if self.sys.monitor_interval > 0 else 0.2))

        def follow():
            while not stop.wait(period):
                self._pump_results()
        # (a call that will be over before the monitor's first look needs no monitor thread: starting and joining one
        # costs more than such a call's bookkeeping; the rate of the previous call tells)
        rate = self._call_rate
        pump = threading.Thread(target=follow, name="xbow-monitor", daemon=True) if not (rate > 0 and ntasks / rate < 0.5 * period and ntasks <= 16384) else None   # (16384: a followed ring blocks the scheduler when nobody reads it)
        self._pump_results()
        rt.follow_history(True)                             # nothing is overwritten before this context has read it
        t_call = time.perf_counter()
        if pump is not None:
            pump.start()
        try:
            while done < ntasks:
                # a chunk ends where the host has something to do between two clocks: an auto-tuner decision, a checkpoint
                n = ntasks - done
                tuning = self.autotuner is not None and self.autotuner.active
                if tuning:
                    # about one chunk per monitor interval (every chunk ends with a drained pipeline, and a sample made of
                    # many short chunks reads several per cent low, more so the more replicas there are to refill); the
                    # chunk that lets a new replica settle, and the first one of all, are short
                    short = max(wpc, self.sys.autotune_interval * wpc * 4)
                    per_interval = int(tune["rate"] * self.sys.monitor_interval / 1000.0) // wpc * wpc if tune["settle"] == 0 else 0
                    n = min(n, max(short, per_interval))
                if ci > 0:
                    to_next = (ci - rt.clock() % ci) * wpc - (rt.tasks_issued() % wpc)
                    n = min(n, max(1, to_next))
                t0 = time.perf_counter()
                issued = rt.train(n, 0)
                rt.drain(max(60.0, self.sys.task_timeout))
                dt = time.perf_counter() - t0
                done += issued
                if issued < n:
                    break                                   # target loss reached
                if tuning:
                    # Every rank issues the same chunks, so the slowest rank's time is the job's: with it the chunk sizes,
                    # the moment of a decision and the decision itself are the same on every GPU.
                    dt = self._slowest(dt)
                    tune["rate"] = issued / max(dt, 1e-9)
                    if len(self.autotune_chunks) < 4096:
                        self.autotune_chunks.append((e.k, issued, dt, tune["settle"]))
                    # one throughput sample per monitor interval, as the reference's monitor takes them; the tuner compares
                    # the latest sample with the one before.  (The first chunk after a replica has been added is left out:
                    # its graphs are uploaded to the device on their first launch, which is not the throughput the new
                    # replica count will have.)
                    if tune["settle"] > 0:
                        tune["settle"] -= 1
                    else:
                        tune["tasks"], tune["time"] = tune["tasks"] + issued, tune["time"] + dt
                    if tune["tasks"] and tune["time"] >= self.sys.monitor_interval / 1000.0:
                        self.monitor.samples.append(self._job_rate(tune["tasks"] * self.mc.batch_size / tune["time"]))
                        if self._autotune(list(self.monitor.samples), rt) != 0:
                            tune["settle"] = 1
                        tune["tasks"], tune["time"] = 0, 0.0
                if ci > 0 and rt.tasks_issued() % wpc == 0 and rt.clock() % ci == 0:
                    self.checkpoint()
        finally:
            stop.set()
            if pump is not None:
                pump.join()
            rt.follow_history(False)
        if done > 0:
            self._call_rate = done / max(time.perf_counter() - t_call, 1e-9)
        self._pump_results()
        self.tasks_done += done
        self.clock.clock = rt.clock()
        self.clock.task = rt.tasks_issued() - 1
        e.epoch_from_native()
        e.finish()
        return done

    # ---- helpers ----
    def _learner_count(self):
        e = self.engine
        return e.k * (len(e.devs) if hasattr(e, "devs") else 1)

    def _collect(self, learner: int, inflight: dict):
        if learner in inflight:
            task, phase = inflight.pop(learner)
            loss, acc = self.engine.wait(learner)
            if phase == Phase.TRAIN:
                self.last_loss, self.last_accuracy = loss, acc
                self.measurements.add(task, loss, acc)
                self.monitor.task_done()
                self.tasks_done += 1
                self._display(task, loss, acc)
            return loss, acc
        return None

    def _drain(self, inflight: dict):
        for l in list(inflight):
            self._collect(l, inflight)

    def _train_tasks(self, ntasks: int):
        if getattr(self, "_native", None) is not None:
            return self._train_native(ntasks)
        e, mc, ds = self.engine, self.mc, self.mc.getDataset(Phase.TRAIN)
        inflight = {}
        solver = mc.getSolverConf()
        done = 0
        while done < ntasks:
            task = self.clock.next_task()
            nl = self._learner_count()
            learner = self._next_learner % nl
            self._next_learner += 1
            self._collect(learner, inflight)                       # replica is free once its last result is in
            x, y = ds.batch(task * self.world + self.rank)
            e.submit(learner, x, y, task, Phase.TRAIN)
            inflight[learner] = (task, Phase.TRAIN)
            done += 1
            if self.clock.is_barrier():
                copy = solver.consume_copy_signal()
                e.synchronise(copy=copy)
                self.clock.tick()
                if self.autotuner is not None and self.autotuner.active:
                    self._drain(inflight)
                    window = self.monitor.throughput_window()
                    if window:
                        window[-1] = self._job_rate(window[-1])
                    self._autotune(window)
                ci = self.sys.checkpoint_interval
                if ci > 0 and self.sys.checkpoint_directory and self.clock.clock % ci == 0:
                    self._drain(inflight)
                    self.checkpoint()
        self._drain(inflight)
        e.finish()
        return done

    def _display(self, task: int, loss: float, acc: float):
        """One training result (result/TrainingResultHandler.java:231-317): every `--display-interval` tasks a line is
        printed - the last task's values, or with `--display-accumulated-loss` the mean over the interval with the last
        value in parentheses.  With `--queue-measurements` the displayed pair goes to a queue that is dumped at shutdown
        and the line is only printed if `--tee-measurements` is set."""
        di = self.sys.display_interval
        if di > 0 and TrainingUnit.from_string(self.sys.display_interval_unit) == TrainingUnit.EPOCHS and getattr(self, "mc", None) is not None:
            di *= max(1, self.mc.numberOfTasksPerEpoch(Phase.TRAIN))           # `--display-interval-unit epochs`
        if di <= 0:
            return
        di = self._local(di)                                  # the interval counts the job's tasks; `task` is this process's
        self._disp_n += 1
        self._disp_loss += loss
        self._disp_acc += acc
        if (task + 1) % di:
            return
        n = max(1, self._disp_n)
        shown_task = (task + 1) * getattr(self, "world", 1)                  # the job's task count at this point
        if self.sys.display_accumulated_loss:
            shown_loss, shown_acc = self._disp_loss / n, self._disp_acc / n
            text = f"[{shown_task:06d}] loss {shown_loss:9.5f} ({loss:9.5f}) accuracy {shown_acc:7.4f} ({acc:7.4f})"
        else:
            shown_loss, shown_acc = loss, acc
            text = f"[{shown_task:06d}] loss {loss:9.5f} accuracy {acc:7.4f}"
        self._disp_n, self._disp_loss, self._disp_acc = 0, 0.0, 0.0
        if self.sys.queue_measurements:
            self.displayed.add(task, shown_loss, shown_acc)
            if not self.sys.tee_measurements:
                return
        if not self.quiet:
            getattr(self, "emit", print)(f"{text} ({self.monitor.last_rate():9.1f} examples/s)")

    def _local(self, job_tasks: int) -> int:
        """This process's share of a count given in tasks of the whole job (rounded up, at least one)."""
        return max(1, -(-int(job_tasks) // max(1, getattr(self, "world", 1))))

    def _tasks_of(self, n: int, unit) -> int:
        """Tasks THIS process issues for `n` tasks / epochs of the job."""
        unit = TrainingUnit.from_string(unit)
        return self._local(n * self.mc.numberOfTasksPerEpoch(Phase.TRAIN) if unit == TrainingUnit.EPOCHS else n)

    # ---- public API ----
    def train(self, n: int, unit=TrainingUnit.TASKS):
        return self._train_tasks(self._tasks_of(n, unit))

    def test(self) -> float:
        """Run every test batch through the test graph against the central model; returns mean accuracy."""
        e, ds = self.engine, self.mc.getDataset(Phase.CHECK)
        if ds is None or self.dataflows[1] is None:
            raise ValueError("error: no test dataflow / data set")
        if getattr(self, "_native_test", None) is not None:
            rt = self._native_test
            rt.totals(reset=True)
            rt.train(ds.number_of_batches(), 1)
            rt.drain(max(60.0, self.sys.task_timeout))
            t = rt.totals()
            e.finish()
            self.test_accuracy = t["acc_sum"] / max(1, t["n"])
            if not self.quiet:
                print(f"[{self.clock.clock:06d}] Test accuracy is {self.test_accuracy:7.4f}", flush=True)
            return self.test_accuracy
        accs, inflight = [], {}
        nl = self._learner_count()
        for t in range(ds.number_of_batches()):
            learner = t % nl
            r = self._collect(learner, inflight)
            if r is not None:
                accs.append(r[1])
            x, y = ds.batch(t)
            e.submit(learner, x, y, t, Phase.CHECK)
            inflight[learner] = (t, Phase.CHECK)
        for l in list(inflight):
            accs.append(self._collect(l, inflight)[1])
        e.finish()
        self.test_accuracy = float(np.mean(accs)) if accs else float("nan")
        if not self.quiet:
            print(f"[{self.clock.clock:06d}] Test accuracy is {self.test_accuracy:7.4f}", flush=True)
        return self.test_accuracy

    def trainAndTest(self, n: int, unit=TrainingUnit.TASKS):
        """Interleave: every test interval (rounded up to a multiple of wpc, ExecutionContext.java:168-172) run the test set."""
        total = self._tasks_of(n, unit)
        interval = self._tasks_of(self.mc.test_interval, self.mc.test_interval_unit)
        wpc = self.clock.wpc
        interval = max(wpc, (interval + wpc - 1) // wpc * wpc)
        done = 0
        while done < total:
            step = min(interval, total - done)
            self._train_tasks(step)
            done += step
            self.test()
        return done

    def trainForDuration(self, duration: float, unit=DurationUnit.SECONDS):
        deadline = time.time() + DurationUnit(unit).seconds(duration)
        done = 0
        chunk = max(self.clock.wpc, 4 * self._learner_count())
        chunk = (chunk + self.clock.wpc - 1) // self.clock.wpc * self.clock.wpc
        while time.time() < deadline:
            done += self._train_tasks(chunk)
        return done

    def trainUntilCondition(self, target_loss: float, max_tasks: int = 1 << 30):
        done = 0
        chunk = (max(self.clock.wpc, self._learner_count()) + self.clock.wpc - 1) // self.clock.wpc * self.clock.wpc
        while done < max_tasks:
            done += self._train_tasks(chunk)
            if self.last_loss <= target_loss:
                break
        return done

    def trainUntilConditionOrForDuration(self, target_loss: float, duration: float, unit=DurationUnit.SECONDS):
        deadline = time.time() + DurationUnit(unit).seconds(duration)
        done = 0
        chunk = (max(self.clock.wpc, self._learner_count()) + self.clock.wpc - 1) // self.clock.wpc * self.clock.wpc
        while time.time() < deadline:
            done += self._train_tasks(chunk)
            if self.last_loss <= target_loss:
                break
        return done

    def checkpoint(self, directory: Optional[str] = None):
        from .checkpoint import save_checkpoint
        return save_checkpoint(self, directory or self.sys.checkpoint_directory)

    def destroy(self):
        if getattr(self.sys, "debug_checksums", False):
            from .oracle import OracleExecutor
            OracleExecutor.checksum_sink = None
        for rt in (getattr(self, "_native", None), getattr(self, "_native_test", None)):
            if rt is not None:
                rt.close()
        self._native = self._native_test = None
        if self.engine is not None:
            if self.sys.gpu and self.sys.trace_level > 0:
                from .utils import trace
                self.trace_summary = trace.summary(clear=True)
                if not self.quiet:                       # what the reference prints per callback handler at shutdown
                    for name, st in self.trace_summary.items():
                        print(f"[TRACE] {name}: " + " ".join(f"{k}={v:.3f}" if isinstance(v, float) else f"{k}={v}" for k, v in st.items()), flush=True)
                trace.enable(0)
            self.engine.destroy()
            self.engine = None
        if self.sys.queue_measurements and not self.quiet:
            print(self.displayed.dump())

    # ---- accessors of the reference's ExecutionContext (ExecutionContext.java:51-90) ----
    def getDataflows(self):
        return list(self.dataflows)

    def getDataflow(self, phase):
        return self.dataflows[int(Phase.from_string(phase))]

    def getModel(self):
        return self.model

    def getModelManager(self):
        """The engine owns what the reference's ModelManager does: replicas, the central model, synchronisation."""
        return self.engine

    def getWorkClock(self):
        return self.clock

    def getThroughputMatrix(self):
        """[processor][dataflow] tasks per second as the hybrid scheduler reads it (row 0 CPU, row 1 GPU); only the row of
        the processor this context runs on is measured."""
        rate = int(self.monitor.last_rate() / max(1, self.mc.batch_size)) if getattr(self, "monitor", None) is not None else 0
        row = [rate, 0]
        return [[0, 0], row] if self.sys.gpu else [row, [0, 0]]

    def getExecutorQueueSize(self) -> int:
        """Tasks handed to the scheduler that have not completed yet."""
        rt = getattr(self, "_native", None)
        return int(rt.tasks_issued() - rt.tasks_completed()) if rt is not None else 0

    # snake_case aliases
    train_and_test = trainAndTest
    train_for_duration = trainForDuration
    train_until_condition = trainUntilCondition

