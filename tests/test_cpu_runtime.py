"""Native host runtime against a fake executor: scheduling order, clocks, synchronisation models, auto-tuner slots,
result ring, failure detection (failed task, stuck task -> watchdog) - all injected on the host, no GPU involved."""
import threading
import time

import pytest

from crossbow_b200.runtime import Runtime, RuntimeError_, ThetaQueue, cpu_bind, cpu_id, cpu_unbind


def test_theta_queue_round_robin_expand_shrink():
    q = ThetaQueue(3)
    got = [q.next() for _ in range(3)]
    assert got == [0, 1, 2]
    assert q.next(0.05) == -1            # all busy: bounded wait reports failure instead of spinning for ever
    q.release(1)
    # strict round robin: the cursor is at slot 0, which is still busy
    assert q.next(0.05) == -1
    q.release(0)
    assert q.next() == 0 and q.next() == 1
    i = q.expand()
    assert i == 3 and q.size() == 4 and q.enabled() == 4
    q.release(3)
    q.release(2)
    assert q.shrink() == 3 and q.enabled() == 3
    q.release(0)
    q.release(1)
    assert sorted(q.next() for _ in range(3)) == [0, 1, 2]   # the disabled slot is skipped from now on
    assert q.next(0.05) == -1
    # growing again re-enables the disabled slot (the replica that takes it gets the same index as the one removed)
    assert q.expand() == 3 and q.size() == 4 and q.enabled() == 4
    for i in range(4):
        q.release(i)
    assert sorted(q.next() for _ in range(4)) == [0, 1, 2, 3]


@pytest.mark.parametrize("handlers", [0, 2])
def test_tasks_results_and_clock(handlers):
    rt = Runtime(learners=4, wpc=4, task_handlers=handlers, callback_handlers=2, task_timeout_s=5)
    rt.attach_fake(4, task_us=200)
    assert rt.train(40) == 40
    rt.drain(10)
    assert rt.tasks_completed() == 40 and rt.clock() == 10 and rt.fake_syncs() == 10
    hist = rt.history(64)
    assert [h[0] for h in hist] == list(range(40))           # collected strictly in task order
    assert all(abs(h[1] - 1.0 / (1 + h[0])) < 1e-6 for h in hist)
    assert sorted(set(int(h[2]) for h in hist)) == [0, 1, 2, 3]   # every learner took part, round robin
    assert [int(h[2]) for h in hist[:8]] == [0, 1, 2, 3, 0, 1, 2, 3]
    t = rt.totals()
    assert t["n"] == 40 and abs(t["last_loss"] - 1.0 / 40) < 1e-6
    rt.close()


@pytest.mark.parametrize("handlers", [0, 2])
def test_run_ahead_keeps_two_tasks_per_replica_in_flight(handlers):
    # every replica is released at submission until two of its tasks are in flight; results are still attributed per task
    rt = Runtime(learners=4, wpc=4, task_handlers=handlers, callback_handlers=2, task_timeout_s=5)
    rt.attach_fake(4, task_us=10000)
    rt.set_run_ahead(2)
    assert rt.train(8) == 8                                   # two rounds are handed over without waiting for a completion
    assert rt.tasks_completed() < 8                           # (each fake task takes 10 ms, two at a time: 40 ms for eight)
    assert rt.train(32) == 32
    rt.drain(10)
    assert rt.tasks_completed() == 40 and rt.clock() == 10 and rt.fake_syncs() == 10
    hist = rt.history(64)
    assert [h[0] for h in hist] == list(range(40))
    assert all(abs(h[1] - 1.0 / (1.0 + h[0])) < 1e-6 for h in hist)          # the loss of task t, not of a later task
    assert all(int(h[2]) == h[0] % 4 for h in hist)                          # round robin over the four replicas
    # a failed task is still reported with run-ahead on
    rt.inject(fail_task=43)
    with pytest.raises(RuntimeError_):
        rt.train(8)
        rt.drain(5)
    assert rt.failed()
    rt.close()


def _hls_model(queue, p, matrix):
    """The reference's rule (task/TaskWindow.java:185-227) restated: index of the task processor p takes, or None."""
    other, skip = (p + 1) % 2, 0.0
    for i, g in enumerate(queue):
        if matrix[p][g] >= matrix[other][g] or skip >= 1.0 / matrix[p][g]:
            return i
        skip += 1.0 / matrix[other][g]
    return None


def test_task_queue_policies_fifo_hls_null():
    import random
    from crossbow_b200.runtime import TaskQueue
    q = TaskQueue("FIFO")
    for t in range(4):
        q.push(t, graph=t % 2)
    assert [q.poll(0), q.poll(1), q.poll(0)] == [0, 1, 2] and len(q) == 1
    assert TaskQueue("NULL").poll(0) == -1
    # replica / clock filter (the reference's select()): a task bound to replica 1 at clock 3
    q = TaskQueue("FIFO")
    q.push(7, replica=1, clock=3)
    assert q.poll(0, replica=0, clock=5) == -1 and q.poll(0, replica=1, clock=2) == -1 and q.poll(0, replica=1, clock=3) == 7
    # HLS: graph 0 is ten times faster on the GPU (processor 1), graph 1 twice as fast on the CPU
    matrix = [[10, 40], [100, 20]]
    q = TaskQueue("HLS")
    for t, g in enumerate([0, 0, 1, 0]):
        q.push(t, graph=g)
    assert q.poll(1, matrix) == 0          # the GPU takes its own kind first
    assert q.poll(0, matrix) == 2          # the CPU skips the two GPU-friendly tasks (cost 2/100 < 1/10) and takes graph 1
    assert q.poll(0, matrix) == -1         # ... and leaves the rest to the GPU: 2/100 has not reached 1/10
    assert q.poll(1, matrix) == 1 and q.poll(1, matrix) == 3
    # against the restated rule on random queues
    rng = random.Random(5)
    for _ in range(50):
        graphs = [rng.randrange(3) for _ in range(rng.randrange(1, 12))]
        matrix = [[rng.randrange(1, 50) for _ in range(3)] for _ in range(2)]
        q, model = TaskQueue("HLS"), list(graphs)
        ids = list(range(len(graphs)))
        for t, g in zip(ids, graphs):
            q.push(t, graph=g)
        while True:
            p = rng.randrange(2)
            want = _hls_model(model, p, matrix)
            got = q.poll(p, matrix)
            assert got == (-1 if want is None else ids[want])
            if want is None:
                if _hls_model(model, 1 - p, matrix) is None:
                    break
                continue
            del model[want], ids[want]
            if not model:
                break


def test_bsp_masks_all_ssp_masks_idle_only():
    rt = Runtime(learners=3, wpc=3, sync_model=0)
    rt.attach_fake(3, task_us=2000)
    rt.train(3)
    assert rt.fake_last_mask() == [1, 1, 1]
    rt.drain(5)
    rt.close()
    rt = Runtime(learners=3, wpc=3, slack=2, sync_model=1)
    rt.attach_fake(3, task_us=20000)
    rt.train(3)                           # the synchronisation is issued while all three tasks still run
    assert rt.fake_syncs() == 0 and rt.clock() == 1      # nobody was idle: the clock ticks, nothing is synchronised
    rt.drain(5)
    rt.close()


def test_staleness_bound_blocks_stale_replicas():
    # SSP with slack 0: a replica that missed the synchronisation may not take a new task until it has been synchronised
    rt = Runtime(learners=2, wpc=2, slack=0, sync_model=1, task_timeout_s=0.3)
    rt.attach_fake(2, task_us=50000)
    rt.train(2)                           # sync skipped both replicas (busy) -> their clocks stay at 0, global clock is 1
    rt.drain(5)
    assert rt.clock() == 1
    # bound = clock - slack - 1 = 0 -> still allowed; after another clock the stale replicas are refused
    rt.train(2)
    rt.drain(5)
    with pytest.raises(RuntimeError_):
        rt.train(2)
    assert "no replica became free" in rt.error()
    rt.close()


def test_auto_tuner_slots():
    rt = Runtime(learners=1, wpc=1)
    rt.attach_fake(8, task_us=100)
    rt.train(4)
    rt.drain(5)
    assert rt.add_learner() == 1 and rt.learners() == 2
    rt.train(6)
    rt.drain(5)
    assert sorted(set(int(h[2]) for h in rt.history(6))) == [0, 1]
    assert rt.remove_learner() == 1 and rt.learners() == 1
    rt.train(3)
    rt.drain(5)
    assert all(int(h[2]) == 0 for h in rt.history(3))
    rt.close()


def test_failed_task_is_reported_not_fatal():
    rt = Runtime(learners=2, wpc=100, task_timeout_s=2)
    rt.attach_fake(2, task_us=100)
    rt.inject(fail_task=5)
    with pytest.raises(RuntimeError_) as e:
        rt.train(50)
        rt.drain(5)
    import re
    assert re.search(r"task 5 failed on learner \d+ with code 77", str(e.value))      # (which learner took it depends on timing)
    assert rt.failed()
    rt.close()


def test_watchdog_detects_stuck_task():
    rt = Runtime(learners=2, wpc=100, task_timeout_s=0.3)
    rt.attach_fake(2, task_us=100)
    rt.inject(hang_task=3)                # its completion takes 1.5 s, far beyond the 0.3 s deadline
    t0 = time.time()
    with pytest.raises(RuntimeError_):
        rt.train(20)
        rt.drain(5)
    assert time.time() - t0 < 3.0
    assert "watchdog" in rt.error() or "no replica became free" in rt.error()
    rt.close()


def test_target_loss_stops_dispatch():
    rt = Runtime(learners=2, wpc=2)
    rt.attach_fake(2, task_us=1000)
    rt.set_target_loss(0.1)               # fake loss = 1/(1+task) reaches 0.1 at task 9
    n = rt.train(10000)
    rt.drain(5)
    assert 10 <= n < 200
    rt.close()


def test_cpu_affinity():
    assert cpu_bind(0) == 0
    assert cpu_id() == 0
    assert cpu_unbind() == 0


def test_results_are_displayed_while_training_runs_and_none_are_lost():
    """Native scheduler: a monitor thread reads the result ring incrementally while `train` runs, so display lines and
    `[MON]` lines appear during training (result/TrainingResultHandler.java:231-317, PerformanceMonitor.java:59-104) and a
    run far longer than the ring loses nothing."""
    import time
    from crossbow_b200 import ModelConf, SystemConf
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.runtime import Runtime
    from crossbow_b200.utils.measure import MeasurementQueue, PerformanceMonitor
    from crossbow_b200.workclock import WorkClock

    class Engine:                      # what _train_native needs from an engine
        k = 4
        def epoch_to_native(self): pass
        def epoch_from_native(self): pass
        def finish(self): pass

    total = 200_000
    ctx = ExecutionContext([None], SystemConf.reset(), ModelConf.reset(), quiet=False)
    ctx.sys.display_interval, ctx.sys.monitor_interval = 1000, 50
    ctx.mc.setBatchSize(8)
    ctx.engine, ctx.clock = Engine(), WorkClock(4)
    lines = []
    ctx.emit = lambda line: lines.append((time.perf_counter(), line))
    ctx.monitor = PerformanceMonitor(8, 1024, 0.05, sink=ctx.emit)
    ctx.monitor.queue_size = ctx.getExecutorQueueSize
    ctx.measurements = MeasurementQueue(capacity=total)
    rt = Runtime(learners=4, wpc=4, result_slots=256, callback_handlers=2, task_timeout_s=30.0)
    rt.attach_fake(4, task_us=0)
    ctx._native = rt
    try:
        done = ctx._train_native(total)
        t_end = time.perf_counter()
    finally:
        rt.close()
    assert done == total and ctx.results_lost == 0 and ctx.tasks_done == total
    assert len(ctx.measurements) == total
    assert sorted(m[1] for m in ctx.measurements.items) == list(range(total))          # every task's result, once
    shown = [l for _, l in lines if l.startswith("[") and not l.startswith("[MON]")]
    assert len(shown) == total // 1000 and shown[0].startswith("[001000]") and shown[-1].startswith(f"[{total:06d}]")
    mon = [(t, l) for t, l in lines if l.startswith("[MON]")]
    assert mon and "examples/s" in mon[0][1] and " q " in mon[0][1]
    # lines appeared while training was in progress, not after it
    early = [t for t, _ in lines if t < t_end - 0.5 * (t_end - lines[0][0])]
    assert len(early) > 5


def test_scheduling_policy_orders_the_queued_tasks():
    """With task handlers (queued scheduling) the dispatcher's tasks pass through the policy queue: FIFO and HLS hand them
    to the handlers, the NULL policy never does, so nothing runs and the run is reported as stuck."""
    from crossbow_b200.runtime import Runtime, RuntimeError_
    for policy in ("FIFO", "HLS"):
        rt = Runtime(learners=3, wpc=3, task_handlers=2, callback_handlers=2, task_timeout_s=5.0)
        rt.attach_fake(3, task_us=20)
        rt.set_scheduling_policy(policy)
        assert rt.train(300) == 300
        rt.drain(20.0)
        assert rt.tasks_completed() == 300 and rt.clock() == 100 and rt.fake_syncs() == 100
        assert [t for t, _, _ in rt.history(300)] == list(range(300))
        rt.close()
    rt = Runtime(learners=2, wpc=2, task_handlers=1, callback_handlers=1, task_timeout_s=0.5)
    rt.attach_fake(2, task_us=0)
    rt.set_scheduling_policy("NULL")
    with pytest.raises(RuntimeError_):
        rt.train(8)
        rt.drain(2.0)
    assert rt.tasks_completed() == 0
    rt.close()


def test_auto_tuner_samples_chunks_of_one_monitor_interval_across_calls():
    """The auto-tuner's throughput samples under the native scheduler: one drained chunk per monitor interval, the chunk
    right after a replica change is short and left out, the state survives `train()` calls that are shorter than an
    interval, and the hill climb of the reference (ModelManager.java:257-274) ends one below the first replica count that
    did not bring 10 %.  The fake executor's task time follows a throughput curve with its knee at three replicas."""
    from crossbow_b200 import ModelConf, SystemConf
    from crossbow_b200.autotune import AutoTuner
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.runtime import Runtime
    from crossbow_b200.utils.measure import MeasurementQueue, PerformanceMonitor
    from crossbow_b200.workclock import WorkClock

    rate = {1: 500.0, 2: 900.0, 3: 1100.0, 4: 1150.0, 5: 1175.0}           # tasks/s of the whole "GPU" at k replicas
    rt = Runtime(learners=1, wpc=12, result_slots=256, callback_handlers=8, task_timeout_s=30.0)    # a task "runs" in its callback handler
    rt.attach_fake(8, task_us=int(1e6 / rate[1]))

    class Engine:
        k = 1
        def epoch_to_native(self): pass
        def epoch_from_native(self): pass
        def finish(self): pass
        def add_learner(self):
            self.k += 1
            rt.set_fake_task_us(int(1e6 * self.k / rate[self.k]))
        def remove_learner(self):
            self.k -= 1
            rt.set_fake_task_us(int(1e6 * self.k / rate[self.k]))

    ctx = ExecutionContext([None], SystemConf.reset(), ModelConf.reset(), quiet=True)
    ctx.sys.display_interval, ctx.sys.monitor_interval = 0, 100
    ctx.mc.setBatchSize(8)
    ctx.engine, ctx.clock = Engine(), WorkClock(12)
    ctx.monitor = PerformanceMonitor(8, 1024, 0.1)
    ctx.measurements = MeasurementQueue(capacity=1 << 16)
    ctx.autotuner = AutoTuner(0.1, 1)
    ctx._native = rt
    try:
        assert ctx._train_native(12) == 12 and ctx._train_native(12) == 12      # ~25 ms each: no sample yet
        assert ctx.autotune_trace == [] and ctx._tune["tasks"] == 24
        for _ in range(60):
            if not ctx.autotuner.active:
                break
            ctx._train_native(240)
    finally:
        rt.close()
    assert not ctx.autotuner.active
    ks = [k for k, _ in ctx.autotune_trace]
    assert ks == [2, 3, 4, 3] and ctx.engine.k == 3, ctx.autotune_trace
    samples = [r for _, r in ctx.autotune_trace]
    for k, r in zip((1, 2, 3, 4), samples):                                   # examples/s = 8 x tasks/s, a little below the curve
        assert 0.5 * 8 * rate[k] < r < 1.02 * 8 * rate[k], (k, r)
    chunks = ctx.autotune_chunks
    # the first chunk after every change is a short one that is marked as settling; no other chunk is
    changes = [i for i in range(1, len(chunks)) if chunks[i][0] != chunks[i - 1][0]]
    assert len(changes) == 3
    for i, (k, n, dt, settling) in enumerate(chunks):
        assert settling == (1 if i in changes else 0), (i, chunks[i])
        if settling:
            assert n == 48
    # once the rate is known, a chunk is sized to one monitor interval (or to what is left of the call)
    assert max(n for _, n, _, s in chunks if not s) >= 0.6 * 0.1 * rate[1] // 12 * 12
