#!/usr/bin/env python
"""Headline benchmark: small-batch SMA training throughput (images/s) of a CIFAR ResNet-32 / ImageNet ResNet-50.

    python bench.py --gpus N --steps K --warmup W [--model resnet32|resnet50] [--replicas k] [--impl reference|cudnn]

One STEP = one synchronisation clock: every one of the k replicas of every GPU runs one task (forward, backward,
local momentum-SGD update on a batch of 64 / 32 images) and then the fused SMA synchronisation runs across all
replicas and GPUs.  Work per GPU is fixed (weak scaling); the reported value is the whole-job images/s.

Two measurements, each K steps after W warm-up steps, bracketed by a barrier + device synchronise:
  value     device time (CUDA events) of the step loop with the batches already staged on the device;
  e2e.value the same loop through the public API (ExecutionContext.train), which copies every batch from pinned host
            memory to the device and reads every task's loss/accuracy back on the host.
The block of K steps is repeated until at least one second has been measured; the reported figure is the median repeat
and the spread is printed next to it.  The same process then runs the library arm (stock PyTorch: cuDNN / cuBLAS / NCCL,
CUDA graphs, channels-last, TF32; baseline/cudnn_arm.py) for the same steps and prints the ratio, and - for the default
model - a shorter ResNet-50 run, so that one line carries both models of the headline metric and the synchronisation
time per step.  Data is synthetic (seeded N(0,1) images, uniform labels); weights are freshly initialised.
"""
import argparse
import ctypes
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

CONFIGS = {
    "resnet32": dict(build="resnet32", batch=64, shape=[3, 32, 32], classes=10, replicas=4),
    "resnet50": dict(build="resnet50", batch=32, shape=[3, 224, 224], classes=1000, replicas=2),
    "vgg16": dict(build="vgg16", batch=128, shape=[3, 32, 32], classes=10, replicas=1),
    "lenet": dict(build="lenet-caffe", batch=16, shape=[1, 28, 28], classes=10, replicas=2),
}


from crossbow_b200.utils.gpumon import ClockSampler  # noqa: E402  (NVML, read-only)


def reference_arm(args):
    # The reference is a Java/Maven + CUDA 8 / cuDNN 6 project: `pip install <reference tree>` finds neither setup.py
    # nor pyproject.toml, there is no JVM on the image and its native code uses cuDNN APIs removed in cuDNN 8.
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a Java/Maven project (no setup.py/pyproject.toml; pip install fails), no JVM on the "
                      "image, native code needs cuDNN<=7 APIs; cannot be installed or run offline"}))
    return 0


def measure_ours(args, model_name, steps, warmup, k=0, batch=0, min_seconds=1.0):
    """Build the model, run the device-only loop and the end-to-end loop, return the record (every rank) - see main()."""
    import torch
    import torch.distributed as dist
    from crossbow_b200 import Dataflow, ModelConf, Phase, SystemConf, UpdateModel
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.data import SyntheticDataset
    from crossbow_b200.models import build
    from crossbow_b200.ops import lib as L

    cfg = CONFIGS[model_name]
    k = k or cfg["replicas"]
    batch = batch or cfg["batch"]
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))

    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setGPU(True).setCPU(False).setNumberOfGpuModels(k).setDisplayInterval(0)
    sysc.use_cuda_graphs = not args.no_graphs
    sysc.use_tensor_cores = not args.no_tc
    sysc.fused_sync = args.sync == "fused"
    sysc.overlap_sync = not args.no_overlap
    sysc.operator_branches = not args.no_branches
    sysc.nvls_sync = args.nvls
    solver = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.1).setMomentum(0.9) \
        .setWeightDecay(1e-4).setAlpha(0.1)
    # work per clock counts the job's tasks: every replica of every GPU runs one task between two synchronisations
    mc.setBatchSize(batch).setWpc(k * world).setUpdateModel(UpdateModel.SMA if args.update_model == "sma" else UpdateModel.WORKER)
    sysc.gradient_buckets = args.gradient_buckets
    ring = max(2 * k, 8)
    ds = SyntheticDataset(cfg["shape"], cfg["classes"], batch, batches=ring * world, seed=1234)
    mc.setDataset(Phase.TRAIN, ds)
    spec = build(cfg["build"], solver_conf=solver)
    if args.bn_blocks or args.bn_reduce_blocks or args.wgrad_ctas or args.tn_ctas:   # (launch shapes are baked into the task graphs at init)
        _lib = L.init_device()
        L.launch_shapes_pinned = True               # the engine keeps its hands off the launch shapes set here
        if args.bn_blocks:
            _lib.xb_bn_set_stream_blocks(args.bn_blocks)
        if args.bn_reduce_blocks:
            _lib.xb_bn_set_reduce_blocks(args.bn_reduce_blocks)
        if args.wgrad_ctas:
            _lib.xb_conv3x3_wgrad_set_ctas(args.wgrad_ctas)
        if args.tn_ctas:
            _lib.xb_gemm_set_tn_ctas(args.tn_ctas)
    if args.gemm_smem:
        many, few = (int(v) for v in args.gemm_smem.split(","))
        L.init_device().xb_gemm_set_smem_budgets(many, few)
    if args.gemm_max_bn:
        nt, tn = (int(v) for v in args.gemm_max_bn.split(","))
        L.init_device().xb_gemm_set_max_bn(nt, tn)
    if args.tma_conv_min:
        L.init_device().xb_tc_set_tma_conv_min(args.tma_conv_min)
    if args.side_low_priority:
        L.init_device().xb_program_side_priority(1)
    if args.pdl is not None:
        L.init_device().xb_set_pdl(args.pdl)
    if args.fuse_bn_sums:
        import crossbow_b200.lower as _lower
        _lower.FUSE_BN_BACKWARD_SUMS = True
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), None], quiet=True)
    ctx.init()
    eng = ctx.engine
    lib = eng.lib

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def repeat(fn):
        """Run fn (one timed block of `steps` steps, milliseconds, max over ranks) until `min_seconds` have been measured
        (3..50 repeats; every rank derives the same count from the first, rank-maximal, value); median and sorted list."""
        first = fn()
        n = max(3, min(50, int(-(-min_seconds * 1e3 // max(first, 1e-3))))) if min_seconds > 0 else 1
        v = sorted([first] + [fn() for _ in range(n - 1)])
        return v[len(v) // 2], v

    # ---------------- device-only loop: batches staged on the device once, no host copies in the timed region --------
    x0, y0 = ds.batch(rank)
    for l in eng.learners:
        ex, lab = l.staging(Phase.TRAIN)
        ex.copy_(x0.reshape(-1), non_blocking=True)
        lab.copy_(y0, non_blocking=True)
    torch.cuda.synchronize()
    task_counter = [0]

    native = getattr(eng, "_exec", None)
    mask = (ctypes.c_ubyte * k)(*([1] * k))
    eng.epoch_to_native()

    def device_step():
        if native:
            # the same C entry points the native scheduler calls (task parameters and the synchronisation descriptor are
            # filled in C++): the host stays far ahead of the device even with eight ranks sharing the machine's cores
            for i in range(k):
                L.check(lib.xb_exec_submit(native, i, None, None, task_counter[0], 0), "submit")
                task_counter[0] += 1
            L.check(lib.xb_exec_synchronise(native, 0, mask, k, 0), "synchronise")
            return
        for l in eng.learners:
            p = eng.params(task_counter[0], True)
            task_counter[0] += 1
            L.check(lib.xb_learner_submit(l.handle, None, None, ctypes.byref(p), 0), "submit")
        eng.synchronise()

    ev0, ev1 = lib.xb_event_create(1), lib.xb_event_create(1)

    def timed_device():
        barrier()
        lib.xb_event_record(ev0, eng.sync_stream)       # sync stream is idle: everything has been synchronised
        for _ in range(steps):
            device_step()
        for l in eng.learners:                           # join: the end event follows every learner's last task
            lib.xb_stream_wait_learner(eng.sync_stream, l.handle)
        lib.xb_event_record(ev1, eng.sync_stream)
        lib.xb_event_sync(ev1)
        barrier()
        return max_over_ranks(lib.xb_event_elapsed_ms(ev0, ev1))

    for _ in range(warmup):
        device_step()
    barrier()
    if hasattr(eng.synchroniser, "timeline"):
        eng.synchroniser.timeline(reset=True)
    sampler = ClockSampler(local)
    sampler.start()
    dev_ms, dev_all = repeat(timed_device)
    eng.epoch_from_native()
    eng.finish()
    tl = eng.synchroniser.timeline() if hasattr(eng.synchroniser, "timeline") else {"launches": 0, "release_us": 0.0, "total_us": 0.0}
    sync_us, release_us = max_over_ranks(tl["total_us"]), max_over_ranks(tl["release_us"])

    # ---------------- end to end through the public API ----------------------------------------------------------------
    ctx.train(warmup * k * world, "tasks")

    def timed_e2e():
        barrier()
        t0 = time.perf_counter()
        ctx.train(steps * k * world, "tasks")      # copies every batch H2D, reads every loss back; ends synchronised
        torch.cuda.synchronize()
        return max_over_ranks(time.perf_counter() - t0) * 1e3

    e2e_ms, e2e_all = repeat(timed_e2e)
    barrier()
    sampler.stop_flag.set()
    sampler.join(timeout=2)

    # every GPU must hold the same central model, bit for bit
    z_identical = True
    if world > 1:
        digest = eng.shared.z.view(torch.int32).to(torch.int64).sum().reshape(1)
        all_d = [torch.empty_like(digest) for _ in range(world)]
        dist.all_gather(all_d, digest)
        z_identical = all(int(d.item()) == int(all_d[0].item()) for d in all_d)

    images_per_step = batch * k * world
    value = images_per_step * steps / (dev_ms / 1e3)
    e2e = images_per_step * steps / (e2e_ms / 1e3)
    launches_per_task = eng.gpu_launches_per_task()
    arena_mb = sum(l.low_train.arena.total for l in eng.learners) / 1e6
    algo = "SMA" if args.update_model == "sma" else "S-SGD"
    syncs_per_step = max(1, len(eng.bucket_syncs))
    out = {
        "metric": f"{model_name} {algo} training throughput", "value": round(value, 1), "unit": "images/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(dev_ms / steps, 4),
        "repeats": len(dev_all), "ms_per_step_min_max": [round(dev_all[0] / steps, 4), round(dev_all[-1] / steps, 4)],
        "timed_seconds": round(sum(dev_all) / 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "tf32 tensor-core tiles, fp32 storage/accumulate" if eng.use_tc else "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {"model": model_name, "global_batch": images_per_step, "batch_per_replica": batch, "replicas_per_gpu": k,
                   "input": cfg["shape"], "parallelism": f"dp{world} x {k} replicas/GPU, " + ("SMA alpha 0.1" if algo == "SMA" else f"synchronous SGD, {syncs_per_step} gradient bucket(s)")
                                  + ", wpc = k*G",
                   "optimizer": "momentum 0.9, wd 1e-4, lr 0.1", "sync": args.sync,
                   "sync_overlap": bool(getattr(eng, "overlap_sync", False)),
                   "operator_branches": bool(getattr(eng, "operator_branches", False)),
                   "nvls": bool(getattr(eng.synchroniser, "nvls", False)),
                   "l2": f"no explicit flush: per-step working set {arena_mb:.0f} MB of activations/gradients exceeds the 126 MB L2"
                         if arena_mb > 252 else f"working set {arena_mb:.0f} MB",
                   "cuda_graphs": eng.use_graphs},
        "e2e": {"value": round(e2e, 1), "unit": "images/s", "ms_per_step": round(e2e_ms / steps, 4), "repeats": len(e2e_all),
                "ms_per_step_min_max": [round(e2e_all[0] / steps, 4), round(e2e_all[-1] / steps, 4)],
                "h2d_bytes_per_step": k * ds.batch_bytes(), "d2h_bytes_per_step": k * 8,
                "timing": "host wall clock around ExecutionContext.train, synchronised on both sides, max over ranks"},
        "gpu_launches": steps * (k * (launches_per_task + 1) + syncs_per_step),   # + the per-task result copy
        "launches_per_task": launches_per_task,
        # device-side time line of the fused synchronisation kernel (%globaltimer in the kernel, mean per launch, max over
        # ranks): entry -> exit of its last block, and entry -> release of the replicas (what the learners wait for)
        "sync_us_per_step": round(sync_us, 2), "sync_release_us": round(release_us, 2),
        "z_identical": z_identical,
        "clocks": sampler.summary(),
        "final_loss": ctx.last_loss,
    }
    lib.xb_event_destroy(ev0)
    lib.xb_event_destroy(ev1)
    ctx.destroy()
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="resnet32", choices=sorted(CONFIGS))
    ap.add_argument("--replicas", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--no-tc", action="store_true", help="CUDA-core convolution kernels only")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="the learners wait for the whole synchronisation (no early release)")
    ap.add_argument("--no-branches", action="store_true", help="weight gradients stay on the task's main chain (no parallel branch in the task graph)")
    ap.add_argument("--nvls", action="store_true", help="two-shot exchange through NVLink multicast (multimem) instead of peer stores")
    ap.add_argument("--pdl", type=int, default=None, help="tuning: 1 / 0 = launch the kernels of a task's critical path with / without programmatic dependent launch")
    ap.add_argument("--side-low-priority", action="store_true", help="tuning: the weight-gradient branch of the task graph runs at the lowest stream priority")
    ap.add_argument("--fuse-bn-sums", action="store_true", help="tuning: data-gradient kernels produce the batch-norm backward sums in their epilogue")
    ap.add_argument("--gemm-smem", default="", help="tuning: shared-memory budgets of the TMA GEMM pipeline in KB, 'many,few' (default 72,100)")
    ap.add_argument("--gemm-max-bn", default="", help="tuning: widest output tile of the TMA GEMM, 'nt,tn' (forward / data gradient, weight gradient; default 128,256)")
    ap.add_argument("--tma-conv-min", type=int, default=0, help="tuning: fewest channels for which R x S convolutions take the TMA implicit GEMM (default 32)")
    ap.add_argument("--no-library-arm", action="store_true", help="skip the library (cuDNN) arm that gives vs_baseline")
    ap.add_argument("--no-resnet50", action="store_true", help="skip the nested ResNet-50 run of the default benchmark")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the timed block until this much has been measured")
    ap.add_argument("--sync", default="fused", choices=["fused", "reference"])
    ap.add_argument("--update-model", default="sma", choices=["sma", "ssgd"], help="sma (headline) or synchronous SGD")
    ap.add_argument("--gradient-buckets", type=int, default=0, help="synchronous SGD: buckets overlapping the backward pass (0 = automatic)")
    ap.add_argument("--bn-blocks", type=int, default=0, help="tuning: blocks of the batch-norm normalise / apply kernels")
    ap.add_argument("--bn-reduce-blocks", type=int, default=0, help="tuning: blocks of the batch-norm reduction kernels")
    ap.add_argument("--wgrad-ctas", type=int, default=0, help="tuning: CTAs of the 3x3 weight-gradient kernel")
    ap.add_argument("--tn-ctas", type=int, default=0, help="tuning: CTAs of the 1x1 weight-gradient GEMM")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "cudnn":
        # library baseline (stock PyTorch operators: cuDNN / cuBLAS / NCCL), same workload; none of this repository's kernels
        from baseline.cudnn_arm import run
        args.clock_sampler = ClockSampler
        return run(args, CONFIGS[args.model], json.dumps)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from crossbow_b200.parallel.peer import init_process_group

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    # ---------------- same box, same run: the library arm (none of this repository's kernels) --------------------------
    # It runs FIRST, as a child process with a deadline, before this process creates its own CUDA context: stock library
    # kernels replayed from several CUDA graphs on several streams have stalled on this hardware before, and a stall
    # there must not take this program's own measurement down with it.  One GPU only: a child cannot join this job's
    # process group.
    base = None
    if not args.no_library_arm and args.update_model == "sma" and args.sync == "fused" and world == 1:
        import subprocess
        cmd = [sys.executable, os.path.abspath(__file__), "--impl", "cudnn", "--gpus", "1", "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--model", args.model, "--min-seconds", str(args.min_seconds)]
        if args.replicas:
            cmd += ["--replicas", str(args.replicas)]
        if args.batch:
            cmd += ["--batch", str(args.batch)]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=150)
            lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
            base = json.loads(lines[-1]) if lines else {"impl": "cudnn", "unavailable": f"exit code {r.returncode}: {r.stderr[-200:]}"}
        except subprocess.TimeoutExpired:
            base = {"impl": "cudnn", "unavailable": "the library arm did not finish within 150 s"}
        except Exception as e:                                   # the product's number stands without it
            base = {"impl": "cudnn", "unavailable": f"{type(e).__name__}: {e}"[:200]}

    torch.cuda.set_device(local)
    init_process_group("nccl", timeout_s=300)

    out = measure_ours(args, args.model, args.steps, args.warmup, args.replicas, args.batch, args.min_seconds)

    if base is not None:
        if "value" in base:
            out["vs_baseline"] = round(out["value"] / base["value"], 3)
            out["baseline_value"] = base["value"]
            out["baseline_impl"] = ("pytorch: cuDNN convolutions (TF32), PyTorch batch norm, CUDA graphs on k streams, channels-last + reference-style "
                                    "averaging (element-wise kernels); child process on the same GPU, run before this arm")
            out["baseline"] = {"ms_per_step": base["ms_per_step"], "repeats": base["repeats"], "e2e_value": base["e2e"]["value"],
                               "clocks": base.get("clocks"), "vs_baseline_e2e": round(out["e2e"]["value"] / base["e2e"]["value"], 3)}
        else:
            out["baseline"] = base

    # ---------------- the other model of the headline metric ------------------------------------------------------------
    if args.model == "resnet32" and not args.no_resnet50:
        r50_steps = max(5, args.steps // 2)
        r50 = measure_ours(args, "resnet50", r50_steps, 3, 0, 0, min(args.min_seconds, 1.0))
        out["resnet50"] = {key: r50[key] for key in ("metric", "value", "unit", "steps", "ms_per_step", "repeats", "ms_per_step_min_max", "config",
                                                     "e2e", "launches_per_task", "sync_us_per_step", "sync_release_us", "z_identical", "clocks")}
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
