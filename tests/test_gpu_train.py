"""Device training against the CPU oracle, task by task: loss, accuracy, replica weights and the central model."""
import numpy as np
import pytest
import torch

from crossbow_b200 import Phase, UpdateModel
from helpers import engines, make_batches

pytestmark = pytest.mark.gpu


def run_both(name, batch, k, tasks, update_model=UpdateModel.SMA, tol=2e-3, use_graphs=True, use_tc=False, **kw):
    spec, m, gpu, cpu = engines(name, batch, k=k, update_model=update_model, use_graphs=use_graphs, use_tc=use_tc, **kw)
    xs, ys = make_batches(spec, batch, tasks, seed=3)
    pinned = [(x.pin_memory(), y.pin_memory()) for x, y in zip(xs, ys)]
    try:
        for t in range(tasks):
            l = t % k
            gpu.submit(l, pinned[t][0], pinned[t][1], t, Phase.TRAIN)
            cpu.submit(l, xs[t], ys[t], t, Phase.TRAIN)
            gl, ga = gpu.wait(l)
            cl, ca = cpu.wait(l)
            assert abs(gl - cl) <= tol * max(1.0, abs(cl)), f"task {t}: loss {gl} vs {cl}"
            assert abs(ga - ca) <= 1.0 / batch + 1e-6, f"task {t}: accuracy {ga} vs {ca}"
            if (t + 1) % k == 0:
                gpu.synchronise()
                cpu.synchronise()
        gpu.finish()
        for i in range(k):
            a, b = gpu.replica_model(i), cpu.replica_model(i)
            err = np.abs(a - b).max() / (np.abs(b).max() + 1e-12)
            assert err < tol, f"replica {i}: rel err {err}"
        a, b = gpu.central_model(), cpu.central_model()
        assert np.abs(a - b).max() / (np.abs(b).max() + 1e-12) < tol
        # test graph against the central model
        gpu.submit(0, pinned[0][0], pinned[0][1], 0, Phase.CHECK)
        cpu.submit(0, xs[0], ys[0], 0, Phase.CHECK)
        assert abs(gpu.wait(0)[1] - cpu.wait(0)[1]) <= 1.0 / batch + 1e-6
        gpu.finish()
    finally:
        gpu.destroy()


@pytest.mark.parametrize("graphs", [False, True])
def test_lenet_sma(graphs):
    # (the reference application's LeNet with its sigma=0.1 initialisation saturates the soft-max on random inputs and
    # amplifies a 1e-7 perturbation to order one within three steps; the classic 20/50/500 LeNet is well conditioned)
    run_both("lenet-caffe", 8, 2, 6, use_graphs=graphs)


def test_lenet_caffe_default():
    run_both("lenet-caffe", 16, 1, 3, update_model=UpdateModel.DEFAULT)


def test_logistic_ssgd():
    run_both("logistic-regression", 32, 2, 4, update_model=UpdateModel.WORKER)


@pytest.mark.parametrize("graphs", [False, True])
def test_ssgd_gradient_buckets_against_oracle(graphs):
    # the accumulate step and the synchronisation run bucket by bucket (marks in the program, one event per bucket)
    spec, m, gpu, cpu = engines("lenet-caffe", 8, k=2, update_model=UpdateModel.WORKER, gradient_buckets=3, use_graphs=graphs)
    try:
        assert len(gpu.bucket_syncs) >= 2 and gpu.lib.xb_program_marks(gpu.learners[0].prog_train) == len(gpu.bucket_syncs)
        assert sum(c.n for c in gpu.bucket_syncs) == m.device_elements
    finally:
        gpu.destroy()
    run_both("lenet-caffe", 8, 2, 6, update_model=UpdateModel.WORKER, gradient_buckets=3, use_graphs=graphs)


def test_ssgd_gradient_buckets_match_one_synchronisation_with_concurrent_learners():
    from crossbow_b200.engine import GpuEngine
    from helpers import build_model
    # (a well-conditioned model: the replicas' atomic accumulation order differs from run to run, and a deep batch-norm
    # network at batch 8 amplifies that rounding noise to 1e-3 within a few steps)
    spec, m, solver = build_model("lenet-caffe", 8)
    init = m.initial_values(5)
    xs, ys = make_batches(spec, 8, 8, seed=11)
    pinned = [(x.pin_memory(), y.pin_memory()) for x, y in zip(xs, ys)]
    out = []
    for nb in (1, 4):
        import copy
        # (fp32 kernels: with tf32 tiles the run-to-run noise of the atomic accumulation order is itself ~1e-3 here)
        eng = GpuEngine(spec.train, None, m, init, 8, spec.input_shape, copy.deepcopy(solver), UpdateModel.WORKER, replicas=2, wpc=2,
                        use_tc=False, gradient_buckets=nb)
        assert (len(eng.bucket_syncs) > 1) == (nb > 1)
        for t in range(0, 8, 2):
            eng.submit(0, *pinned[t], t, Phase.TRAIN)
            eng.submit(1, *pinned[t + 1], t + 1, Phase.TRAIN)
            eng.synchronise()                      # enqueued while both learners are still running
        for l in range(2):
            eng.wait(l)
        eng.finish()
        out.append((eng.central_model(), eng.replica_model(1), eng.central_momentum().cpu().numpy()))
        eng.destroy()
    for a, b in zip(out[0], out[1]):
        assert np.isfinite(a).all() and np.abs(a - b).max() <= 2e-4 * (np.abs(a).max() + 1e-12), np.abs(a - b).max() / np.abs(a).max()


def test_debug_canaries_stay_intact_and_catch_an_overrun():
    from crossbow_b200.engine import GpuEngine
    from helpers import build_model
    spec, m, solver = build_model("resnet8", 8)
    eng = GpuEngine(spec.train, spec.test, m, m.initial_values(5), 8, spec.input_shape, solver, UpdateModel.SMA, replicas=2, wpc=2,
                    use_tc=True, debug_canaries=True)
    try:
        xs, ys = make_batches(spec, 8, 4, seed=2)
        for t in range(4):
            eng.submit(t % 2, xs[t].pin_memory(), ys[t].pin_memory(), t, Phase.TRAIN)
            eng.wait(t % 2)
            if t % 2:
                eng.synchronise()
        eng.submit(0, xs[0].pin_memory(), ys[0].pin_memory(), 0, Phase.CHECK)
        eng.wait(0)
        eng.finish()                                           # every kernel stayed inside its buffers
        arena = eng.learners[1].low_train.arena
        assert len(arena.guards) > 20 and arena.check_canaries() == 0
        arena.guards[7][3] = 0                                 # what an overrun by four words would leave behind (written from the host)
        with pytest.raises(RuntimeError, match="written past their end"):
            eng.finish()
    finally:
        eng.destroy()


def test_resnet8_sma():
    run_both("resnet8", 8, 2, 4)


def test_resnet8_reference_pool():
    run_both("resnet8", 4, 1, 2, reference_pool=True)


def test_resnet8_transform():
    run_both("resnet8", 8, 1, 2, transform=True)


def test_mini_inception():
    run_both("mini-inception", 4, 1, 2)


def test_convnet_polyak():
    run_both("convnet", 8, 2, 4, update_model=UpdateModel.POLYAK_RUPPERT)


def test_lenet_batchnorm_eamsgd():
    run_both("lenet-batchnorm", 8, 2, 4, update_model=UpdateModel.EAMSGD)


def test_reuse_memory_same_results_less_memory():
    """--reuse-memory: buffers with disjoint lifetimes share storage; training results are unchanged."""
    run_both("resnet8", 8, 2, 4, reuse_memory=True)
    run_both("convnet", 8, 1, 3, reuse_memory=True)
    from helpers import engines
    sizes = []
    for reuse in (False, True):
        spec, m, gpu, _ = engines("resnet20", 16, k=1, reuse_memory=reuse)
        sizes.append(gpu.learners[0].low_train.arena.total)
        gpu.destroy()
    assert sizes[1] < 0.8 * sizes[0], sizes


def test_sleep_kernel_waits_roughly_the_requested_cycles():
    from crossbow_b200.ops import lib as L
    lib = L.init_device()
    s = torch.cuda.current_stream()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    L.check(lib.xb_sleep(1000, s.cuda_stream), "sleep")
    torch.cuda.synchronize()
    a.record(s)
    L.check(lib.xb_sleep(2_000_000, s.cuda_stream), "sleep")      # ~1 ms at ~2 GHz
    b.record(s)
    b.synchronize()
    assert 0.5 < a.elapsed_time(b) < 5.0
    assert lib.xb_sleep(-1, s.cuda_stream) != 0


def test_batch_splits():
    """--splits 2: every task runs the graph (optimiser included) over two consecutive sub-batches."""
    run_both("convnet", 8, 2, 4, splits=2)
    run_both("lenet-batchnorm", 16, 1, 3, splits=2)


def test_matrix_factorisation():
    """(row, column, rating) triples: loss, factor gradients and the SMA step agree with the CPU definition."""
    from helpers import build_model
    from crossbow_b200.engine import CpuEngine, GpuEngine
    import copy
    batch, k = 32, 2
    spec, m, solver = build_model("matrix-factorisation", batch)
    init = m.initial_values(5)
    gpu = GpuEngine(spec.train, None, m, init, batch, spec.input_shape, solver, UpdateModel.SMA, replicas=k, wpc=k, seed=5)
    cpu = CpuEngine(spec.train, None, m, init, batch, spec.input_shape, copy.deepcopy(solver), UpdateModel.SMA, replicas=k, wpc=k, seed=5)
    g = torch.Generator().manual_seed(8)
    try:
        for t in range(6):
            x = torch.stack([torch.randint(0, 1000, (batch,), generator=g).float(), torch.randint(0, 500, (batch,), generator=g).float(),
                             torch.rand(batch, generator=g) * 5.0], 1).reshape(batch, 3, 1, 1).contiguous()
            y = torch.randint(0, 6, (batch,), generator=g).to(torch.int32)      # ratings travel as labels
            l = t % k
            gpu.submit(l, x.pin_memory(), y.pin_memory(), t, Phase.TRAIN)
            cpu.submit(l, x, y, t, Phase.TRAIN)
            gl, cl = gpu.wait(l)[0], cpu.wait(l)[0]
            assert abs(gl - cl) <= 1e-4 * max(1.0, abs(cl)), f"task {t}: loss {gl} vs {cl}"
            if (t + 1) % k == 0:
                gpu.synchronise()
                cpu.synchronise()
        gpu.finish()
        a, b = gpu.central_model(), cpu.central_model()
        assert np.abs(a - b).max() / np.abs(b).max() < 1e-4
        for i in range(k):
            a, b = gpu.replica_model(i), cpu.replica_model(i)
            assert np.abs(a - b).max() / np.abs(b).max() < 1e-4
    finally:
        gpu.destroy()


def test_bottleneck_resnet():
    run_both("tiny-bottleneck", 16, 1, 2, tol=5e-3)


def test_full_size_models_run():
    """VGG-16 and ResNet-50 (64x64 inputs) lower, run and produce finite losses on the device."""
    for name, batch, kw in (("vgg16", 8, {}), ("resnet50", 4, dict(size=64, classes=10))):
        spec, m, gpu, _ = engines(name, batch, k=1, **kw)
        try:
            xs, ys = make_batches(spec, batch, 1, seed=3)
            x, y = xs[0].pin_memory(), ys[0].pin_memory()
            losses = []
            for t in range(6):
                gpu.submit(0, x, y, t, Phase.TRAIN)
                losses.append(gpu.wait(0)[0])
                gpu.synchronise()
            gpu.finish()
            assert all(np.isfinite(losses)) and all(l >= 0 for l in losses), losses
        finally:
            gpu.destroy()


@pytest.mark.parametrize("name,use_tc", [("lenet-caffe", False), ("resnet8", True)])
def test_operator_branches_change_nothing_but_the_schedule(name, use_tc):
    """Weight / bias gradients on a parallel branch of the task graph (joined in front of the optimiser) against the same
    program captured as one chain: same losses and weights up to the rounding of the atomic gradient sums."""
    from crossbow_b200.engine import GpuEngine
    from helpers import build_model
    import copy
    spec, m, solver = build_model(name, 8)
    xs, ys = make_batches(spec, 8, 6, seed=5)
    outs = []
    for branches in (False, True):
        eng = GpuEngine(spec.train, spec.test, m, m.initial_values(7), 8, spec.input_shape, copy.deepcopy(solver), UpdateModel.SMA, replicas=2,
                        wpc=2, use_tc=use_tc, operator_branches=branches)
        side = sum(1 for o in eng.learners[0].low_train.ops if o.flags & 0x1000)
        assert (side > 0) == branches
        losses = []
        try:
            for t in range(0, 6, 2):
                eng.submit(0, xs[t].pin_memory(), ys[t].pin_memory(), t, Phase.TRAIN)
                eng.submit(1, xs[t + 1].pin_memory(), ys[t + 1].pin_memory(), t + 1, Phase.TRAIN)
                losses += [eng.wait(0)[0], eng.wait(1)[0]]
                eng.synchronise()
            eng.finish()
            outs.append((losses, eng.central_model(), eng.replica_model(1)))
        finally:
            eng.destroy()
    (la, za, ra), (lb, zb, rb) = outs
    assert np.allclose(la, lb, rtol=2e-3, atol=1e-5)
    assert np.abs(za - zb).max() <= 2e-3 * np.abs(za).max() and np.abs(ra - rb).max() <= 2e-3 * np.abs(ra).max()


def test_tasks_in_flight_keep_their_own_parameters():
    """A learner may hold several tasks in flight; the parameters of a task (learning rate, task number) are read on the
    device when the task runs, which can be after the NEXT task has been submitted.  Each task must still see its own:
    task A runs with learning rate 0 (the weights stay put), task B on the same batch must report exactly A's loss."""
    import ctypes as C
    from crossbow_b200.engine import GpuEngine
    from crossbow_b200.ops import lib as L
    from helpers import build_model
    spec, m, solver = build_model("lenet-caffe", 8)
    eng = GpuEngine(spec.train, None, m, m.initial_values(7), 8, spec.input_shape, solver, UpdateModel.SMA, replicas=1, wpc=1)
    try:
        lib, ln = eng.lib, eng.learners[0]
        xs, ys = make_batches(spec, 8, 1, seed=9)
        x, y = xs[0].pin_memory(), ys[0].pin_memory()
        w0 = ln.rep.w.clone()
        L.check(lib.xb_sleep(30_000_000, ln.stream), "sleep")          # ~15 ms: both submissions happen before task A starts
        pa, pb = eng.params(0, True), eng.params(1, True)
        pa.lr, pb.lr = 0.0, 0.5
        ln.submit(x, y, pa, Phase.TRAIN)
        ln.submit(x, y, pb, Phase.TRAIN)
        la, lb, acc = C.c_float(), C.c_float(), C.c_float()
        L.check(lib.xb_learner_wait_task(ln.handle, pa.task_id, 0, C.byref(la), C.byref(acc)), "wait A")
        L.check(lib.xb_learner_wait_task(ln.handle, pb.task_id, 0, C.byref(lb), C.byref(acc)), "wait B")
        eng.finish()
        assert la.value == lb.value and la.value > 0                     # A did not move the weights
        assert float((ln.rep.w - w0).abs().max()) > 0                    # B did
    finally:
        eng.destroy()
