"""Two gloo ranks on the CPU, one device group each, against one process that holds both groups: the host-side twin of
the multi-GPU protocol (same data split, same synchronisation maths, all-reduce across processes)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys
    import numpy as np, torch
    import torch.distributed as dist
    sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
    from helpers import build_model, make_batches
    from crossbow_b200 import Phase, UpdateModel
    from crossbow_b200.engine import CpuEngine
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    um = UpdateModel.from_string(sys.argv[3])
    spec, m, solver = build_model("lenet-caffe", 4)
    eng = CpuEngine(spec.train, spec.test, m, m.initial_values(7), 4, spec.input_shape, solver, um, replicas=2, wpc=2, seed=7)
    xs, ys = make_batches(spec, 4, 8, seed=3)
    # global task t goes to rank t % world, replica (t // world) % 2
    for t in range(8):
        if t % world == rank:
            l = (t // world) % 2
            eng.submit(l, xs[t], ys[t], t, Phase.TRAIN); eng.wait(l)
        if (t + 1) % 4 == 0:
            eng.synchronise()
    np.save(os.path.join(sys.argv[2], f"z{rank}.npy"), eng.central_model())
    np.save(os.path.join(sys.argv[2], f"r{rank}.npy"), eng.replica_model(1))
    dist.destroy_process_group()
''')


@pytest.mark.parametrize("update_model", ["SMA", "WORKER"])
def test_two_gloo_ranks_equal_one_process_with_two_device_groups(tmp_path, update_model):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + (os.getpid() % 300)), str(script), ROOT, str(tmp_path), update_model]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    z0, z1 = np.load(tmp_path / "z0.npy"), np.load(tmp_path / "z1.npy")
    assert np.array_equal(z0, z1)                      # every rank holds the same central model
    # single process, two virtual devices
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import build_model, make_batches
    from crossbow_b200 import Phase, UpdateModel
    from crossbow_b200.engine import CpuEngine
    from crossbow_b200.oracle import DeviceState, ReplicaState
    import torch
    um = UpdateModel.from_string(update_model)
    spec, m, solver = build_model("lenet-caffe", 4)
    eng = CpuEngine(spec.train, spec.test, m, m.initial_values(7), 4, spec.input_shape, solver, um, replicas=2, wpc=4, seed=7)
    w = torch.from_numpy(m.initial_values(7))
    d2 = DeviceState(w)
    d2.replicas = [ReplicaState(w) for _ in range(2)]
    eng.devs.append(d2)
    xs, ys = make_batches(spec, 4, 8, seed=3)
    for t in range(8):
        dev, l = t % 2, (t // 2) % 2
        eng.submit(dev * 2 + l, xs[t], ys[t], t, Phase.TRAIN)
        if (t + 1) % 4 == 0:
            eng.synchronise()
    assert np.allclose(eng.central_model(), z0, rtol=1e-5, atol=1e-6)
    assert np.allclose(eng.replica_model(1), np.load(tmp_path / "r0.npy"), rtol=1e-5, atol=1e-6)
    assert np.allclose(eng.replica_model(3), np.load(tmp_path / "r1.npy"), rtol=1e-5, atol=1e-6)


TUNER = textwrap.dedent('''
    import json, os, sys
    import torch.distributed as dist
    sys.path.insert(0, sys.argv[1])
    from crossbow_b200 import ModelConf, SystemConf
    from crossbow_b200.autotune import AutoTuner
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.runtime import Runtime
    from crossbow_b200.utils.measure import MeasurementQueue, PerformanceMonitor
    from crossbow_b200.workclock import WorkClock
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    slow = 1.0 if rank == 0 else 1.15                                  # the second "GPU" is 15 % slower at every replica count
    rate = {1: 500.0, 2: 900.0, 3: 1100.0, 4: 1150.0, 5: 1175.0}      # tasks/s of one "GPU" with k replicas
    rt = Runtime(learners=1, wpc=12, result_slots=256, callback_handlers=8, task_timeout_s=30.0)
    rt.attach_fake(8, task_us=int(slow * 1e6 / rate[1]))

    class Engine:
        k = 1
        def epoch_to_native(self): pass
        def epoch_from_native(self): pass
        def finish(self): pass
        def add_learner(self):
            self.k += 1
            rt.set_fake_task_us(int(slow * 1e6 * self.k / rate[self.k]))
        def remove_learner(self):
            self.k -= 1
            rt.set_fake_task_us(int(slow * 1e6 * self.k / rate[self.k]))

    ctx = ExecutionContext([None], SystemConf.reset(), ModelConf.reset(), quiet=True)
    ctx.rank, ctx.world = rank, world
    ctx.sys.gpu, ctx.sys.display_interval, ctx.sys.monitor_interval = False, 0, 100
    ctx.mc.setBatchSize(8)
    ctx.engine, ctx.clock = Engine(), WorkClock(12)
    ctx.monitor = PerformanceMonitor(8, 1024, 0.1)
    ctx.measurements = MeasurementQueue(capacity=1 << 16)
    ctx.autotuner = AutoTuner(0.1, 1)
    ctx._native = rt
    try:
        for _ in range(60):
            if not ctx.autotuner.active:
                break
            ctx._train_native(240)
    finally:
        rt.close()
    json.dump({"active": ctx.autotuner.active, "k": ctx.engine.k, "trace": ctx.autotune_trace,
               "chunks": [(k, n, s) for k, n, _, s in ctx.autotune_chunks], "times": [dt for _, _, dt, _ in ctx.autotune_chunks]},
              open(os.path.join(sys.argv[2], f"tuner{rank}.json"), "w"))
    dist.destroy_process_group()
''')


def test_auto_tuner_takes_one_decision_for_the_job_on_two_gloo_ranks(tmp_path):
    """Two ranks whose (fake) devices differ in speed: every chunk is timed by the slower rank, so both ranks issue the same
    chunks, take their samples at the same moments, see the same job-wide throughput and end with the same replica count
    (the reference is one process with one monitor and one decision, ModelManager.java:257-274)."""
    import json
    script = tmp_path / "tuner.py"
    script.write_text(TUNER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29900 + (os.getpid() % 90)), str(script), ROOT, str(tmp_path)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    a, b = (json.load(open(tmp_path / f"tuner{i}.json")) for i in (0, 1))
    assert not a["active"] and not b["active"]
    assert a["k"] == b["k"] == 3
    assert a["trace"] == b["trace"] and [k for k, _ in a["trace"]] == [2, 3, 4, 3]        # same samples, same decisions
    assert a["chunks"] == b["chunks"]                                                      # same chunks, same settling marks
    assert a["times"] == b["times"]                                                        # both use the slower rank's time
    # the samples are the JOB's throughput: twice one rank's tasks over the slower rank's time
    k1 = a["trace"][0][1]
    assert 0.5 * 2 * 8 * 500.0 / 1.15 < k1 < 1.02 * 2 * 8 * 500.0 / 1.15
