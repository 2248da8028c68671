"""Execution engines: what actually runs a task and a synchronisation step.

``GpuEngine`` owns, for ONE GPU (= one process): the central average model ``z``, ``k`` learners (replica flat
vectors + activation arena + CUDA stream + captured task graph each), the synchronisation stream and the fused
synchroniser.  It is the counterpart of the reference's native execution context + model manager + streams
(clib-multigpu/executioncontext.c, modelmanager.c, stream.c), restructured so that a replica, its stream and its
buffers form one fixed unit ("learner") whose whole task is a single CUDA-graph launch.

``CpuEngine`` runs the same protocol on the CPU oracle (``--gpu false``).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np
import torch

from .conf import ModelConf, SolverConf, SystemConf
from .graph import SubGraph
from .model import Model
from .oracle import (DeviceState, OracleExecutor, ReplicaState, local_update, sma_base_momentum, synchronise)
from .types import MomentumMethod, Phase, Regularisation, UpdateModel


def task_params(solver: SolverConf, task: int, seed: int, training: bool, bn_updates: int = 0):
    from .ops import lib as L
    p = L.XbTaskParams()
    p.lr = solver.learning_rate(task) if training else 0.0
    p.momentum = solver.momentum_at(task)
    p.weight_decay = solver.weight_decay
    p.bn_factor = 1.0 / (1.0 + bn_updates)
    p.clip = solver.clip_gradient_threshold if solver.clip_gradient_threshold is not None else -1.0
    p.alpha = solver.alpha
    p.task_id = task & 0xFFFFFFFF
    p.seed_lo, p.seed_hi = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    p.training = int(training)
    p.l1 = int(solver.regularisation_type == Regularisation.L1)
    p.nesterov = int(solver.momentum_method == MomentumMethod.NESTEROV)
    return p


class Learner:
    """Replica + stream + arena + programs."""

    def __init__(self, engine: "GpuEngine", index: int, init: torch.Tensor):
        from .lower import Lowering, ReplicaBuffers
        from .ops import lib as L
        lib = engine.lib
        self.engine, self.index = engine, index
        self.rep = ReplicaBuffers(engine.model, engine.device, init)
        self.params_dev = torch.zeros(16, dtype=torch.int32, device=engine.device)
        self.low_train = self.low_test = None
        self.handle = None
        self.clock = 0
        self.pending = None          # (task_id, phase) in flight
        self._held = []              # host tensors of submitted tasks whose asynchronous copies may not have run yet
        c, h, w = engine.input_chw
        # the first lowering allocates the staging buffers the native learner copies into
        self.handle_placeholder = None
        self._create(L, lib)

    def _create(self, L, lib):
        from .lower import Lowering
        e = self.engine
        # native learner first (it owns the pinned parameter block and the result slot), staging set afterwards
        self.handle = lib.xb_learner_create(0, 0, 0, 0, 0)
        if not self.handle:
            raise L.CudaError("could not create a learner stream")
        params_host = C.cast(lib.xb_learner_params(self.handle), C.c_void_p).value
        result_dev = lib.xb_learner_result_dev(self.handle)
        self.low_train = Lowering(e.train_graph, e.model, e.batch, e.input_chw, e.device, self.rep.w, self.rep, e.shared,
                                  self.params_dev, params_host, result_dev, update_model=e.update_model, training=True,
                                  use_tc=e.use_tc, clip=e.solver.clip_gradient_threshold >= 0, lr_mult=e.lr_mult, splits=e.splits, reuse_memory=e.reuse_memory,
                                  gradient_buckets=e.gradient_buckets, canaries=e.debug_canaries, operator_branches=e.operator_branches)
        ops = self.low_train.op_array()
        self.prog_train = lib.xb_program_create(ops, len(ops), int(e.use_tc), e.tc_status.data_ptr())
        self.prog_test = None
        if e.test_graph is not None:
            # test tasks read the CENTRAL model (the reference checks with the master copy) and share the staging buffers
            self.low_test = Lowering(e.test_graph, e.model, e.batch, e.input_chw, e.device, e.shared.z, None, e.shared,
                                     self.params_dev, params_host, result_dev, update_model=e.update_model, training=False,
                                     use_tc=e.use_tc, reuse_memory=e.reuse_memory, canaries=e.debug_canaries)
            tops = self.low_test.op_array()
            self.prog_test = lib.xb_program_create(tops, len(tops), int(e.use_tc), e.tc_status.data_ptr())
        lib.xb_learner_set_programs(self.handle, self.prog_train, self.prog_test)
        self.stream = lib.xb_learner_stream(self.handle)
        if e.use_graphs:
            L.check(lib.xb_program_capture(self.prog_train, self.stream), "capture of the training program")
            if self.prog_test:
                L.check(lib.xb_program_capture(self.prog_test, self.stream), "capture of the test program")

    def staging(self, phase):
        low = self.low_train if phase == Phase.TRAIN else self.low_test
        return low.examples, low.labels

    def submit(self, examples: torch.Tensor, labels: torch.Tensor, params, phase=Phase.TRAIN):
        from .ops import lib as L
        lib = self.engine.lib
        ex, lab = self.staging(phase)
        s = self.stream
        L.check(lib.xb_memcpy_h2d_async(ex.data_ptr(), examples.data_ptr(), examples.numel() * 4, s), "H2D examples")
        L.check(lib.xb_memcpy_h2d_async(lab.data_ptr(), labels.data_ptr(), labels.numel() * 4, s), "H2D labels")
        L.check(lib.xb_learner_submit(self.handle, None, None, C.byref(params), int(phase)), "task submit")
        self.pending = (params.task_id, phase)
        # The copies above are asynchronous: the (pinned) source must stay alive - and out of the pinned allocator's
        # free list - until they have run.  A caller that passes a temporary (`x.pin_memory()`) is covered by these
        # references; they are dropped once a wait has shown the tasks to be complete.
        self._held.append((examples, labels))
        if len(self._held) > 256:
            del self._held[0]

    def wait(self):
        from .ops import lib as L
        loss, acc = C.c_float(), C.c_float()
        L.check(self.engine.lib.xb_learner_wait(self.handle, C.byref(loss), C.byref(acc)), "task wait")
        self.pending = None
        self._held.clear()           # the learner's last task has finished, so every copy before it has run
        return loss.value, acc.value

    def destroy(self):
        lib = self.engine.lib
        if self.handle:
            lib.xb_learner_destroy(self.handle)
            self.handle = None
        for p in (self.prog_train, self.prog_test):
            if p:
                lib.xb_program_destroy(p)
        self.prog_train = self.prog_test = None


class GpuEngine:
    def __init__(self, train_graph: SubGraph, test_graph: Optional[SubGraph], model: Model, init_canonical: np.ndarray,
                 batch: int, input_chw, solver: SolverConf, update_model: UpdateModel, replicas: int = 1, wpc: int = 1,
                 rank: int = 0, world: int = 1, device_index: int = 0, use_tc: bool = True, use_graphs: bool = True,
                 seed: int = 0, fused_sync: bool = True, two_shot: Optional[bool] = None, sync_timeout_s: float = 5.0,
                 splits: int = 1, reuse_memory: bool = False, gradient_buckets: int = 0,
                 debug_canaries: bool = False, overlap_sync: bool = True, operator_branches: bool = True, nvls_sync: bool = False):
        """`overlap_sync`: model averaging on several GPUs - the learners' next tasks start as soon as their replicas have
        been corrected (the kernel's release word), under the cross-GPU exchange and the central update; off = they wait
        for the whole synchronisation.
        `gradient_buckets`: synchronous SGD only - number of gradient buckets whose all-reduce + update overlaps the
        backward pass (0 = 4 for models of at least 32 MB, otherwise 1; 1 = one synchronisation after the task)."""
        from .ops import lib as L
        from .parallel.sync import FusedSynchroniser, ReferenceSynchroniser
        if not torch.cuda.is_available():
            raise RuntimeError("GpuEngine needs a CUDA device")
        torch.cuda.set_device(device_index)
        self.lib = L.init_device()   # raises if the extension cannot be built / loaded: no fallback on the device path
        self.device = torch.device("cuda", device_index)
        self.train_graph, self.test_graph, self.model = train_graph, test_graph, model
        self.batch, self.input_chw, self.solver, self.update_model = batch, tuple(input_chw), solver, update_model
        self.splits = max(1, int(splits))
        self.reuse_memory = bool(reuse_memory)
        self.operator_branches = bool(operator_branches)   # weight gradients on a parallel branch of the task graph
        self.debug_canaries = bool(debug_canaries)      # guard words behind every activation buffer, checked in finish()
        nb = int(gradient_buckets) if gradient_buckets else (4 if model.device_elements * 4 >= (32 << 20) else 1)
        self.gradient_buckets = min(8, nb) if (fused_sync and update_model == UpdateModel.WORKER) else 1
        self.bucket_syncs = []
        # `wpc` counts THIS rank's tasks per clock; a clock of the job is wpc * world tasks, which is what synchronous SGD
        # divides the summed gradient by (the reference's single process counts all GPUs' tasks, synch/synchronoussgd.c:60-75)
        self.rank, self.world, self.wpc, self.seed = rank, world, wpc, seed
        self.use_tc, self.use_graphs = use_tc, use_graphs
        self.tc_status = torch.zeros(4, dtype=torch.int32, device=self.device)
        init = torch.from_numpy(model.to_device(init_canonical)).to(self.device)
        from .lower import DeviceShared
        n = model.device_elements
        Sync = FusedSynchroniser if fused_sync else ReferenceSynchroniser
        # (created first: with several GPUs and a large model it provides the peer-visible home of the central model)
        # (`nvls_sync`: exchange through NVLink multicast - multimem.ld_reduce / multimem.st - where the two-shot path applies)
        self.synchroniser = Sync(n, rank, world, two_shot, sync_timeout_s, nvls=nvls_sync) if fused_sync else Sync(n, rank, world)
        z_storage = self.synchroniser.central_storage() if hasattr(self.synchroniser, "central_storage") else None
        self.shared = DeviceShared(model, self.device, init, z_storage)
        self.lr_mult = torch.from_numpy(model.to_device(model.lr_multipliers())).to(self.device) if model.has_lr_multipliers() else None
        self.learners: List[Learner] = []
        self._apply_launch_shapes(replicas)
        for i in range(replicas):
            self.learners.append(Learner(self, i, init))
        ranges = self.learners[0].low_train.buckets if self.learners else []
        if len(ranges) > 1:
            self.bucket_syncs = self.synchroniser.make_buckets(ranges)
        self.sync_stream = self.lib.xb_stream_create(-1)
        self.sync_event = self.lib.xb_event_create(0)
        self.overlap_sync = bool(overlap_sync) and fused_sync and world > 1 and bool(self.lib.xb_stream_wait_value_supported())
        self.poly_count = 0
        self.bn_updates = 0
        self._exec = None
        torch.cuda.synchronize()

    # ---- replicas ----
    @property
    def k(self):
        return len(self.learners)

    def _apply_launch_shapes(self, k: int):
        """CTA counts of the reductions and weight-gradient kernels, which are baked into a learner's task graph when it is
        lowered.  A small model (under 2 M parameters: kernels of a few microseconds) at one or two replicas leaves SMs idle,
        so those kernels spread wide (ResNet-32: +7.5 % at one replica, +4 % at two); from three replicas on, and for larger
        models at any replica count (VGG-16 -4 %, ResNet-50 -4 % with the wide shapes), fewer, longer-lived CTAs win."""
        from .ops import lib as L
        if getattr(L, "launch_shapes_pinned", False):      # a benchmark set them by hand
            return
        small = self.model.elements < (2 << 20)
        wide = k <= 2 and small
        # (with the weight gradients on a parallel branch of the task graph they are off the critical path: for small models
        # at three or more replicas 74 long-lived CTAs measured +0.9 % over 148)
        self.lib.xb_conv3x3_wgrad_set_ctas(296 if wide else (74 if small and self.operator_branches else 148))
        self.lib.xb_gemm_set_tn_ctas(148 if wide else 111)
        self.lib.xb_bn_set_reduce_blocks(592 if wide else 296)

    def add_learner(self) -> Learner:
        """Auto-tuner: clone a new replica from an existing one (modelmanager.c:362-472)."""
        torch.cuda.synchronize()
        self._apply_launch_shapes(len(self.learners) + 1)
        src = self.learners[0].rep.w
        l = Learner(self, len(self.learners), src)
        l.rep.last.copy_(self.learners[0].rep.last)
        l.rep.prev.copy_(self.learners[0].rep.prev)
        self.learners.append(l)
        if self._exec:
            self._exec_add(l)
        torch.cuda.synchronize()
        return l

    def remove_learner(self):
        if len(self.learners) <= 1:
            return
        torch.cuda.synchronize()
        if self._exec:
            self.lib.xb_exec_remove_learner(self._exec)
        self.learners.pop().destroy()

    # ---- tasks ----
    def global_task(self, task: int) -> int:
        """Job-wide number of this rank's task `task`: rank r of G runs the job's tasks r, G + r, 2 G + r, ...  The
        learning-rate schedule, the random streams (dropout, crops) and the data set are indexed with it, as the
        reference's single task counter over all GPUs is (solverconfiguration.c:116-161)."""
        return task * self.world + self.rank

    def params(self, task: int, training: bool):
        return task_params(self.solver, self.global_task(task) if training else task, self.seed, training, self.bn_updates)

    def submit(self, learner: int, examples, labels, task: int, phase=Phase.TRAIN):
        p = self.params(task, phase == Phase.TRAIN)
        if phase == Phase.TRAIN:
            self.bn_updates += 1
        elif self.overlap_sync:
            # a test task reads the central model: it waits for the whole synchronisation, not only for the release
            from .ops import lib as L
            L.check(self.lib.xb_learner_wait_event(self.learners[learner].handle, self.sync_event), "test task waits for sync")
        self.learners[learner].submit(examples, labels, p, phase)

    def wait(self, learner: int):
        return self.learners[learner].wait()

    # ---- synchronisation ----
    def synchronise(self, copy: bool = False, learners: Optional[List[int]] = None):
        """Enqueue one synchronisation over the given (default: all) learners; returns immediately.

        Ordering is on the device: the synchronisation stream waits for every participating learner's last task,
        and those learners' next tasks wait for the synchronisation to finish."""
        from .ops import lib as L
        from .parallel import sync as S
        lib, ss = self.lib, self.sync_stream
        ls = [self.learners[i] for i in (learners if learners is not None else range(len(self.learners)))]
        um, sv = self.update_model, self.solver
        bucketed = bool(self.bucket_syncs) and um == UpdateModel.WORKER
        early = False
        if not bucketed:
            for l in ls:
                L.check(lib.xb_stream_wait_learner(ss, l.handle), "sync waits for learner")
        ws, prevs = [l.rep.w for l in ls], [l.rep.prev for l in ls]
        sh = self.shared
        if um in (UpdateModel.SMA, UpdateModel.SYNCHRONOUSEAMSGD):
            self.synchroniser.synchronise(ss, S.ALGO_SMA, ws, prevs, sh.z, sh.zlast, None, alpha=sv.alpha,
                                          mu=sma_base_momentum(sv), copy=copy, use_prev=True)
            early = self.overlap_sync and self.synchroniser.releases_early(S.ALGO_SMA, copy)
        elif um == UpdateModel.EAMSGD:
            self.synchroniser.synchronise(ss, S.ALGO_SMA, ws, prevs, sh.z, sh.zlast, None, alpha=sv.alpha,
                                          mu=sv.base_model_momentum, copy=copy, use_prev=False)
            early = self.overlap_sync and self.synchroniser.releases_early(S.ALGO_SMA, copy)
        elif bucketed:
            # bucket b starts as soon as every learner has accumulated that bucket's gradients (the learners are then still
            # in the backward pass of the earlier layers)
            self.synchroniser.epoch += 1
            for b, c in enumerate(self.bucket_syncs):
                for l in ls:
                    L.check(lib.xb_stream_wait_learner_bucket(ss, l.handle, b), "sync waits for a gradient bucket")
                sl = slice(c.offset, c.offset + c.n)
                c.epoch = self.synchroniser.epoch - 1
                c.synchronise(ss, S.ALGO_SSGD, [w[sl] for w in ws], None, sh.z[sl], sh.zlast[sl], sh.gacc[sl], mu=sv.momentum,
                              scale=1.0 / (self.wpc * self.world))
            for l in ls:
                L.check(lib.xb_stream_wait_learner(ss, l.handle), "sync waits for learner")
        elif um == UpdateModel.WORKER:
            self.synchroniser.synchronise(ss, S.ALGO_SSGD, ws, None, sh.z, sh.zlast, sh.gacc, mu=sv.momentum, scale=1.0 / (self.wpc * self.world))
        elif um == UpdateModel.POLYAK_RUPPERT:
            self.synchroniser.synchronise(ss, S.ALGO_POLYAK, ws, None, sh.z, sh.zlast, None, alpha=0.0,
                                          scale=1.0 / (len(ls) * self.world), blend=1.0 / (self.poly_count + 1.0))
            self.poly_count += 1
        elif um == UpdateModel.DEFAULT:
            arr = torch.tensor([w.data_ptr() for w in ws], dtype=torch.int64, device=self.device)
            self._keep = arr
            L.check(lib.xb_broadcast_model(sh.z.data_ptr(), arr.data_ptr(), len(ws), self.model.device_elements, ss), "broadcast")
        else:
            raise NotImplementedError(f"error: {um} is not supported (a stub in the reference as well)")
        L.check(lib.xb_event_record(self.sync_event, ss), "record sync event")
        for l in ls:
            if early:        # the replica is final once phase 1 of the kernel is through: the next task runs under the exchange
                self.synchroniser.wait_release(l.stream)
            else:
                L.check(lib.xb_learner_wait_event(l.handle, self.sync_event), "learner waits for sync")

    # ---- native scheduling: hand the learners to the C++ runtime ----
    def native_executor(self, train_ds=None, test_ds=None):
        """Build the native executor (csrc/runtime/program.cu) for this engine and return
        ``(ctx, submit, wait, synchronise, batch)`` as raw addresses for ``Runtime.set_executor``."""
        from .ops import lib as L
        from .parallel import sync as S
        from .types import LearningRateDecayPolicy as P
        lib, sv = self.lib, self.solver
        if not hasattr(self.synchroniser, "descriptor"):
            raise RuntimeError("the native scheduler needs the fused synchroniser")
        st = L.XbSolverState()
        st.policy = {P.FIXED: 0, P.INV: 1, P.STEP: 2, P.MULTISTEP: 3, P.LSR: 4, P.EXP: 5}.get(sv.learning_rate_decay_policy, 0)
        st.base_lr, st.gamma, st.power, st.momentum = sv.base_learning_rate, sv.gamma, sv.power, sv.momentum
        st.weight_decay, st.alpha = sv.weight_decay, sv.alpha
        st.clip = sv.clip_gradient_threshold if sv.clip_gradient_threshold is not None else -1.0
        st.step_size, st.warmup = sv._in_tasks(sv.step_size), sv._in_tasks(sv.warmup_steps)
        steps = sv.steps_in_tasks()[:32]
        st.nsteps = len(steps)
        for i, v in enumerate(steps):
            st.steps[i] = v
        st.l1 = int(sv.regularisation_type == Regularisation.L1)
        st.nesterov = int(sv.momentum_method == MomentumMethod.NESTEROV)
        st.step_cursor, st.copy_signal = sv._step, 0
        if self._exec:
            lib.xb_exec_destroy(self._exec)
        self._exec = lib.xb_exec_create(C.byref(st), self.seed, self.sync_stream, getattr(self.synchroniser, "max_blocks", 0))
        lib.xb_exec_set_rank(self._exec, self.rank, self.world)
        for l in self.learners:
            self._exec_add(l)
        um, sh = self.update_model, self.shared
        ws = [l.rep.w for l in self.learners]
        prevs = [l.rep.prev for l in self.learners]
        sy = self.synchroniser
        if um in (UpdateModel.SMA, UpdateModel.SYNCHRONOUSEAMSGD):
            d = sy.descriptor(S.ALGO_SMA, ws, prevs, sh.z, sh.zlast, None, sv.alpha, sma_base_momentum(sv), 1.0, 0.0, False, True)
        elif um == UpdateModel.EAMSGD:
            d = sy.descriptor(S.ALGO_SMA, ws, prevs, sh.z, sh.zlast, None, sv.alpha, sv.base_model_momentum, 1.0, 0.0, False, False)
        elif um == UpdateModel.WORKER:
            d = sy.descriptor(S.ALGO_SSGD, ws, None, sh.z, sh.zlast, sh.gacc, 0.0, sv.momentum, 1.0 / (self.wpc * self.world), 0.0, False, True)
        elif um == UpdateModel.POLYAK_RUPPERT:
            d = sy.descriptor(S.ALGO_POLYAK, ws, None, sh.z, sh.zlast, None, 0.0, 0.0, 1.0, 1.0, False, True)
        elif um == UpdateModel.DEFAULT:
            d = sy.descriptor(S.ALGO_SMA, ws, prevs, sh.z, sh.zlast, None, 0.0, 0.0, 1.0, 0.0, False, True)
        else:
            raise NotImplementedError(f"error: {um} is not supported (a stub in the reference as well)")
        lib.xb_exec_set_sync(self._exec, C.byref(d), int(um == UpdateModel.DEFAULT))
        lib.xb_exec_set_early_release(self._exec, int(self.overlap_sync))
        if um == UpdateModel.WORKER:
            for c in self.bucket_syncs:
                sl = slice(c.offset, c.offset + c.n)
                db = c.descriptor(S.ALGO_SSGD, [w[sl] for w in ws], None, sh.z[sl], sh.zlast[sl], sh.gacc[sl], 0.0, sv.momentum,
                                  1.0 / (self.wpc * self.world), 0.0, False, True)
                L.check(min(0, lib.xb_exec_add_bucket(self._exec, C.byref(db), c.offset)), "gradient bucket")
        lib.xb_exec_set_epoch(self._exec, sy.epoch)
        for phase, ds in ((0, train_ds), (1, test_ds)):
            if ds is None:
                continue
            if hasattr(ds, "examples"):      # contiguous pinned ring owned by Python: the executor indexes it itself
                lib.xb_exec_set_data(self._exec, phase, ds.examples.data_ptr(), ds.examples[0].numel() * 4, ds.labels.data_ptr(),
                                     ds.labels[0].numel() * 4, ds.examples.shape[0], self.world if phase == 0 else 1,
                                     self.rank if phase == 0 else 0)
            else:                            # native data source: the runtime asks it for addresses, sizes are all we need
                n = int(np.prod(ds.example_shape)) * ds.batch_size
                lib.xb_exec_set_data(self._exec, phase, 0, n * 4, 0, ds.batch_size * 4, 0, 1, 0)
        addr = lambda name: C.cast(getattr(lib, name), C.c_void_p).value
        return self._exec, addr("xb_exec_submit"), addr("xb_exec_wait"), addr("xb_exec_synchronise"), addr("xb_exec_batch")

    def native_wait_task(self) -> int:
        """Address of the executor's per-task wait (run-ahead scheduling)."""
        return C.cast(self.lib.xb_exec_wait_task, C.c_void_p).value

    def epoch_to_native(self):
        """The synchronisation epoch is one counter whichever side enqueues the kernels: the flags in peer memory hold the
        epochs already used, so the native executor must continue after the last one enqueued from Python."""
        if self._exec and hasattr(self.synchroniser, "epoch"):
            self.lib.xb_exec_set_epoch(self._exec, max(int(self.lib.xb_exec_epoch(self._exec)), int(self.synchroniser.epoch)))

    def epoch_from_native(self):
        if self._exec and hasattr(self.synchroniser, "epoch"):
            self.synchroniser.epoch = max(int(self.synchroniser.epoch), int(self.lib.xb_exec_epoch(self._exec)))

    def _exec_add(self, l: Learner):
        ext, lat = l.staging(Phase.TRAIN)
        exs, las = l.staging(Phase.CHECK) if l.low_test is not None else (None, None)
        p = lambda t: t.data_ptr() if t is not None else 0
        self.lib.xb_exec_add_learner(self._exec, l.handle, l.rep.w.data_ptr(), l.rep.prev.data_ptr(), p(ext), p(lat), p(exs), p(las))

    def finish(self):
        torch.cuda.synchronize()
        self.synchroniser.check()
        s = self.tc_status.cpu()
        if int(s[0]) != 0:
            raise RuntimeError(f"a tensor-core kernel reported status {int(s[0])} (bounded wait expired)")
        if self.debug_canaries:
            for l in self.learners:
                for low in (l.low_train, l.low_test):
                    bad = low.arena.check_canaries() if low is not None else 0
                    if bad:
                        raise RuntimeError(f"learner {l.index}: {bad} activation buffer(s) were written past their end (guard words changed)")

    # ---- model access (canonical order, host) ----
    def central_momentum(self) -> torch.Tensor:
        """Momentum vector of the central model (device order).  Collective when the chunk owners keep it in shares."""
        self.finish()
        sy = self.synchroniser
        return sy.gather_momentum(self.shared.zlast) if getattr(sy, "owner_apply", False) else self.shared.zlast

    def central_model(self) -> np.ndarray:
        return self.model.to_canonical(self.shared.z.cpu().numpy())

    def replica_model(self, i: int) -> np.ndarray:
        return self.model.to_canonical(self.learners[i].rep.w.cpu().numpy())

    def load_central(self, canonical: np.ndarray):
        self.shared.z.copy_(torch.from_numpy(self.model.to_device(canonical)))

    def load_replica(self, i: int, canonical: np.ndarray):
        self.learners[i].rep.w.copy_(torch.from_numpy(self.model.to_device(canonical)))

    def gpu_launches_per_task(self) -> int:
        return self.lib.xb_program_launches(self.learners[0].prog_train)

    def destroy(self):
        torch.cuda.synchronize()
        for l in self.learners:
            l.destroy()
        self.learners = []
        if self._exec:
            self.lib.xb_exec_destroy(self._exec)
            self._exec = None
        self.synchroniser.close()
        self.lib.xb_stream_destroy(self.sync_stream)


class CpuEngine:
    """Same protocol on the CPU oracle, with k replicas x G virtual devices in one process."""

    def __init__(self, train_graph, test_graph, model: Model, init_canonical, batch, input_chw, solver: SolverConf,
                 update_model: UpdateModel, replicas=1, wpc=1, devices=1, seed=0, splits=1, rank=0, world=1):
        """`rank` / `world`: when given (one process per device group under torch.distributed), training task t of this
        process is task t * world + rank of the job for the learning-rate schedule and the random streams."""
        self.model, self.solver, self.update_model, self.wpc, self.seed = model, solver, update_model, wpc, seed
        self.rank, self.world = rank, max(1, world)
        self.splits = max(1, int(splits))
        w = torch.from_numpy(np.asarray(init_canonical, dtype=np.float32))
        self.devs = [DeviceState(w) for _ in range(devices)]
        for d in self.devs:
            d.replicas = [ReplicaState(w) for _ in range(replicas)]
        self.train_exec = OracleExecutor(train_graph, model, seed)
        self.test_exec = OracleExecutor(test_graph, model, seed) if test_graph is not None else None
        self.results = {}
        self.lr_mult = torch.from_numpy(model.lr_multipliers()) if model.has_lr_multipliers() else None

    @property
    def k(self):
        return len(self.devs[0].replicas)

    def _slot(self, learner):
        return self.devs[learner // self.k], self.devs[learner // self.k].replicas[learner % self.k]

    def submit(self, learner, examples, labels, task, phase=Phase.TRAIN):
        dev, rep = self._slot(learner)
        x, y = torch.as_tensor(examples, dtype=torch.float32), torch.as_tensor(labels)
        if phase == Phase.TRAIN:
            task = task * self.world + self.rank
            # `--splits`: the graph (optimiser included) runs once per sub-batch; the task reports the mean loss / accuracy
            sub = x.shape[0] // self.splits
            parts = []
            for s in range(self.splits):
                rep.g.zero_()
                parts.append(self.train_exec.run(rep.w, x[s * sub:(s + 1) * sub], y[s * sub:(s + 1) * sub], Phase.TRAIN, task, dev.op_state, rep.g))
                local_update(rep, dev, self.solver, self.update_model, task, self.lr_mult)
            r = {k_: (None if parts[0][k_] is None else float(sum(p_[k_] for p_ in parts)) / self.splits) for k_ in ("loss", "accuracy")}
        else:
            r = self.test_exec.run(dev.z, x, y, Phase.CHECK, task, dev.op_state)
        self.results[learner] = (r["loss"] if r["loss"] is not None else 0.0, r["accuracy"] if r["accuracy"] is not None else 0.0)

    def wait(self, learner):
        return self.results.pop(learner)

    def synchronise(self, copy=False, learners=None):
        """With ``torch.distributed`` initialised (gloo) every process holds one device group and the partial sums are
        all-reduced across processes: the host-side twin of the multi-GPU path."""
        import torch.distributed as dist
        ar, world = None, 1
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            world = dist.get_world_size()

            def ar(t):
                t = t.clone()
                dist.all_reduce(t)
                return t
        synchronise(self.update_model, self.devs, self.solver, self.wpc * world if self.update_model == UpdateModel.WORKER else self.wpc,
                    copy, allreduce=ar, world=world)

    def add_learner(self):
        for d in self.devs:
            d.replicas.append(d.replicas[0].clone())

    def remove_learner(self):
        for d in self.devs:
            if len(d.replicas) > 1:
                d.replicas.pop()

    def finish(self):
        pass

    def central_model(self):
        return self.devs[0].z.numpy().copy()

    def replica_model(self, i):
        return self._slot(i)[1].w.numpy().copy()

    def load_central(self, canonical):
        for d in self.devs:
            d.z = torch.from_numpy(np.asarray(canonical, dtype=np.float32)).clone()

    def load_replica(self, i, canonical):
        self._slot(i)[1].w = torch.from_numpy(np.asarray(canonical, dtype=np.float32)).clone()

    def destroy(self):
        pass
