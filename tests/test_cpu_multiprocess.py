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
