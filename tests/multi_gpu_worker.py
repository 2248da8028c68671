"""Launched by tests/test_gpu_multi.py with torch.distributed.run, one rank per GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from crossbow_b200.parallel.peer import init_process_group
    from crossbow_b200.parallel.sync import ALGO_SMA, ALGO_SSGD, FusedSynchroniser, ReferenceSynchroniser
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    init_process_group("nccl", timeout_s=120)
    s = torch.cuda.current_stream().cuda_stream
    for n, two_shot, k in ((4096 * 5 + 1024, False, 2), (4096 * 9, True, 3), (1 << 20, True, 1)):
        g = torch.Generator(device="cuda").manual_seed(10 + rank)
        ws = [torch.randn(n, device="cuda", generator=g) * 0.01 for _ in range(k)]
        ps = [torch.randn(n, device="cuda", generator=g) * 0.01 for _ in range(k)]
        z, zl = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        ws2, ps2, z2, zl2 = [w.clone() for w in ws], [p.clone() for p in ps], z.clone(), zl.clone()
        fs = FusedSynchroniser(n, rank, world, two_shot=two_shot, timeout_s=10.0)
        rs = ReferenceSynchroniser(n, rank, world)
        if fs.owner_apply and n != 4096 * 9:
            # owner-apply: the central model lives in the synchroniser's peer-visible buffer, chunk owners store the new
            # model into every rank's copy and keep the momentum of their chunks
            z = fs.central_storage()
            z.zero_()
        for it in range(3):
            fs.synchronise(s, ALGO_SMA, ws, ps, z, zl, alpha=0.1, mu=0.9)
            rs.synchronise(s, ALGO_SMA, ws2, ps2, z2, zl2, alpha=0.1, mu=0.9)
            torch.cuda.synchronize()
            fs.check()
            assert torch.allclose(z, z2, rtol=1e-4, atol=1e-7), (n, two_shot, it, float((z - z2).abs().max()))
            for a, b in zip(ws, ws2):
                assert torch.allclose(a, b, rtol=1e-4, atol=1e-7)
            # all ranks hold bit-identical central models
            zs = [torch.empty_like(z) for _ in range(world)]
            dist.all_gather(zs, z.clone())
            assert all(torch.equal(zs[0], t) for t in zs)
            assert torch.allclose(fs.gather_momentum(zl), zl2, rtol=1e-4, atol=1e-7)
        # S-SGD
        gacc, gacc2 = torch.randn(n, device="cuda", generator=g) * 0.01, None
        gacc2 = gacc.clone()
        fs.synchronise(s, ALGO_SSGD, ws, None, z, zl, gacc, mu=0.9, scale=1.0 / (k * world))
        rs.synchronise(s, ALGO_SSGD, ws2, None, z2, zl2, gacc2, mu=0.9, scale=1.0 / (k * world))
        torch.cuda.synchronize()
        fs.check()
        assert torch.allclose(z, z2, rtol=1e-4, atol=1e-7)
        assert float(gacc.abs().max()) == 0.0 and torch.equal(ws[0], z)
        dist.barrier()
        fs.close()
    # NVLink multicast variant of the two-shot exchange (multimem.ld_reduce / multimem.st), where the box offers multicast.
    # Nothing is asserted while memory is bound to the multicast object: a rank that left at that point would take the
    # others' NVLink traffic down with it.  The verdicts are collected, every rank unbinds, and only then are they checked.
    if os.environ.get("XBOW_TEST_NVLS", "1") == "1":
        import gc
        n, k = 4096 * 9 + 2048, 2
        fs = FusedSynchroniser(n, rank, world, two_shot=True, timeout_s=10.0, nvls=True)
        used, problems = fs.nvls, []
        if used:
            g = torch.Generator(device="cuda").manual_seed(40 + rank)
            ws = [torch.randn(n, device="cuda", generator=g) * 0.01 for _ in range(k)]
            ps = [torch.randn(n, device="cuda", generator=g) * 0.01 for _ in range(k)]
            z, zl = fs.central_storage(), torch.zeros(n, device="cuda")
            z.zero_()
            ws2, ps2, z2, zl2 = [w.clone() for w in ws], [p.clone() for p in ps], z.clone(), zl.clone()
            rs = ReferenceSynchroniser(n, rank, world)
            for it in range(3):
                fs.synchronise(s, ALGO_SMA, ws, ps, z, zl, alpha=0.1, mu=0.9)
                rs.synchronise(s, ALGO_SMA, ws2, ps2, z2, zl2, alpha=0.1, mu=0.9)
                torch.cuda.synchronize()
                if int(fs.status.item()) != 0:
                    problems.append(f"status {int(fs.status.item())} at iteration {it}")
                    fs.status.zero_()
                if not torch.allclose(z, z2, rtol=1e-4, atol=1e-7):
                    problems.append(f"central model differs at iteration {it}: {float((z - z2).abs().max())}")
                if not all(torch.allclose(a_, b_, rtol=1e-4, atol=1e-7) for a_, b_ in zip(ws, ws2)):
                    problems.append(f"replicas differ at iteration {it}")
                zs = [torch.empty_like(z) for _ in range(world)]
                dist.all_gather(zs, z.clone())
                if not all(torch.equal(zs[0], t) for t in zs):
                    problems.append(f"central models differ across ranks at iteration {it}")
                if not torch.allclose(fs.gather_momentum(zl), zl2, rtol=1e-4, atol=1e-7):
                    problems.append(f"momentum differs at iteration {it}")
            del z, zs
        torch.cuda.synchronize()
        dist.barrier()
        fs.close()
        del fs
        gc.collect()
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        dist.barrier()
        assert not problems, problems
        if rank == 0:
            print("NVLS_SYNC_OK" if used else "NVLS_SYNC_UNAVAILABLE")
    # end to end: two ranks train with SMA through the engine and stay in step
    from crossbow_b200 import Phase, UpdateModel
    from crossbow_b200.engine import GpuEngine
    from helpers import build_model, make_batches
    spec, m, solver = build_model("resnet8", 8)
    eng = GpuEngine(spec.train, None, m, m.initial_values(7), 8, spec.input_shape, solver, UpdateModel.SMA, replicas=2, wpc=2,
                    rank=rank, world=world, device_index=local, use_tc=True)
    xs, ys = make_batches(spec, 8, 8, seed=100 + rank)
    for t in range(8):
        eng.submit(t % 2, xs[t].pin_memory(), ys[t].pin_memory(), t, Phase.TRAIN)
        eng.wait(t % 2)
        if t % 2 == 1:
            eng.synchronise()
    eng.finish()
    zs = [torch.empty_like(eng.shared.z) for _ in range(world)]
    dist.all_gather(zs, eng.shared.z)
    assert all(torch.equal(zs[0], t) for t in zs), "central models diverged across ranks"
    assert float(eng.shared.z.abs().sum()) > 0 and torch.isfinite(eng.shared.z).all()
    eng.destroy()
    dist.barrier()
    # model averaging overlapped with the next tasks (the learners follow the kernel's release word) against the serialised
    # order (they wait for the whole synchronisation): same arithmetic, so the weights must be bit-identical
    import copy as _copy
    spec, m, solver = build_model("lenet-caffe", 8)          # well conditioned: rounding noise is not amplified
    xs, ys = make_batches(spec, 8, 12, seed=200 + rank)
    finals = []
    for overlap in (False, True):
        eng = GpuEngine(spec.train, None, m, m.initial_values(7), 8, spec.input_shape, _copy.deepcopy(solver), UpdateModel.SMA, replicas=2,
                        wpc=2, rank=rank, world=world, device_index=local, use_tc=False, overlap_sync=overlap)
        assert eng.overlap_sync == overlap
        for t in range(0, 12, 2):                     # both learners in flight, nothing waits on the host between clocks
            eng.submit(0, xs[t].pin_memory(), ys[t].pin_memory(), t, Phase.TRAIN)
            eng.submit(1, xs[t + 1].pin_memory(), ys[t + 1].pin_memory(), t + 1, Phase.TRAIN)
            eng.synchronise()
        eng.wait(0), eng.wait(1)
        eng.finish()
        tl = eng.synchroniser.timeline()
        assert tl["launches"] == 6 and 0 < tl["release_us"] <= tl["total_us"], tl
        finals.append([eng.shared.z.clone()] + [l.rep.w.clone() for l in eng.learners])
        eng.destroy()
        dist.barrier()
    # (gradient sums are accumulated with atomics, so two runs agree to rounding, not to the bit; a task that started
    # before its replica was corrected would be off by the size of the correction, orders of magnitude more)
    for a, b in zip(*finals):
        assert torch.isfinite(a).all() and float((a - b).abs().max()) <= 3e-4 * float(a.abs().max()) + 1e-9, float((a - b).abs().max())
    # synchronous SGD with gradient buckets (owner-apply exchange per bucket, overlapping the backward pass) against one
    # synchronisation per clock; both learners of a rank run concurrently
    import copy
    outs = []
    spec, m, solver = build_model("lenet-caffe", 8)          # well conditioned: rounding noise is not amplified
    xs, ys = make_batches(spec, 8, 8, seed=100 + rank)
    for nb in (1, 3):
        eng = GpuEngine(spec.train, None, m, m.initial_values(7), 8, spec.input_shape, copy.deepcopy(solver), UpdateModel.WORKER, replicas=2,
                        wpc=2, rank=rank, world=world, device_index=local, use_tc=False, two_shot=True, gradient_buckets=nb)
        assert (len(eng.bucket_syncs) > 1) == (nb > 1)
        for t in range(0, 8, 2):
            eng.submit(0, xs[t].pin_memory(), ys[t].pin_memory(), t, Phase.TRAIN)
            eng.submit(1, xs[t + 1].pin_memory(), ys[t + 1].pin_memory(), t + 1, Phase.TRAIN)
            eng.synchronise()
        eng.wait(0), eng.wait(1)
        eng.finish()
        zs = [torch.empty_like(eng.shared.z) for _ in range(world)]
        dist.all_gather(zs, eng.shared.z.clone())
        assert all(torch.equal(zs[0], t) for t in zs), "central models diverged across ranks (bucketed S-SGD)"
        outs.append((eng.shared.z.clone(), eng.central_momentum().clone(), eng.learners[1].rep.w.clone()))
        eng.destroy()
        dist.barrier()
    for a, b in zip(outs[0], outs[1]):
        assert torch.isfinite(a).all() and float((a - b).abs().max()) <= 3e-4 * float(a.abs().max()) + 1e-9, float((a - b).abs().max())
    # the auto-tuner takes ONE decision for the job: every rank sees the same (summed) throughput sample, so all ranks add
    # and remove replicas together
    from crossbow_b200 import Dataflow, ModelConf, SystemConf
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.data import SyntheticDataset
    from crossbow_b200.models import build
    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setGPU(True).setCPU(False).setNumberOfGpuModels(1).setDisplayInterval(0)
    sysc.autotune_models, sysc.autotune_threshold, sysc.monitor_interval = True, -1.0, 1
    sv = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01).setMomentum(0.9).setAlpha(0.1)
    mc.setBatchSize(16).setWpc(2 * world).setUpdateModel("SMA")
    mc.setDataset(Phase.TRAIN, SyntheticDataset([1, 28, 28], 10, 16, batches=8 * world, seed=1, distribution="uniform"))
    spec = build("lenet-caffe", solver_conf=sv)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), None], quiet=True)
    ctx.init()
    assert ctx.world == world and ctx.clock.wpc == 2          # --wpc counts the job's tasks
    ctx.train(16 * world, "tasks")
    ctx.train(16 * world, "tasks")
    ctx.autotuner.threshold = 1e9
    ctx.train(16 * world, "tasks")
    mine = torch.tensor([ctx.engine.k, int(ctx.autotuner.active), len(ctx.autotune_trace)] + [k for k, _ in ctx.autotune_trace][:6], device="cuda")
    alls = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(alls, mine)
    assert all(torch.equal(alls[0], t) for t in alls), [t.tolist() for t in alls]
    ks = [k for k, _ in ctx.autotune_trace]
    assert not ctx.autotuner.active and max(ks) >= 3 and ctx.engine.k == max(ks) - 1 == ks[-1], (ctx.engine.k, ctx.autotune_trace)
    assert ctx.tasks_done == 48                                # this rank's share of 3 x 16 x world job tasks
    zs = [torch.empty_like(ctx.engine.shared.z) for _ in range(world)]
    dist.all_gather(zs, ctx.engine.shared.z.clone())
    assert all(torch.equal(zs[0], t) for t in zs), "central models diverged across ranks (context, auto-tuned)"
    ctx.destroy()
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
