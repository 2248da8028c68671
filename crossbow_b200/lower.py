"""Lowers a dataflow graph to a device program (array of ``XbOp`` launches) for one learner.

The reference registers every operator with the native side and then, per task, walks the operator list and
calls one function per operator, gradient operators included (SubGraph.java:397-552; executioncontext.c:558-726).
Here the forward nodes of the graph are compiled once into a fused launch list:

* activations are channels-last; convolution / inner-product weights use the device element order of ``model.py``;
* ``Conv -> BatchNorm``: the convolution epilogue produces the per-channel sum / sum of squares, so batch-norm is
  one more pass; ``BatchNorm (-> Sum with a shortcut) -> ReLU`` is a single normalise kernel; ``Conv/InnerProduct
  -> ReLU`` folds the activation into the GEMM epilogue; ``SoftMax -> {SoftMaxLoss, Accuracy}`` and the loss
  gradient are one kernel that also writes loss/accuracy into the learner's host-mapped result slot;
* the backward pass is derived from the same forward nodes in reverse topological order (the graph's explicit
  gradient nodes define WHICH operators are differentiated; the CPU oracle executes them one by one), with
  first-write / accumulate tracking for tensors that feed several consumers (the reference's "merge" operators);
* weight gradients go straight into the replica's flat gradient vector, which the fused optimiser consumes
  and clears.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import numpy as np
import torch

from .graph import SubGraph
from .model import Model
from .ops import lib as L
from .types import (ActivationMode, BatchNormEstimatedMeanAndVarianceType, ElementWiseOpType, NormalisationMode,
                    Phase, PoolMethod, UpdateModel)


# Let the data-gradient kernel that completes dy of a normalisation layer also produce that layer's backward sums (and skip
# the layer's own reduction kernel).  Measured on B200: ResNet-32 -6 %, ResNet-50 -4 % images/s - the extra loads and
# column sums lengthen the epilogue of CTAs that hold tensor memory and a full operand pipeline, which costs more than the
# lean stand-alone reduction it saves.  Off; the kernels keep the capability (tests/test_gpu_conv_kernels.py).
FUSE_BN_BACKWARD_SUMS = False

# Normalisation layers with ReLU and a residual input write a packed sign mask of their output (a sixteenth of its size) in
# the forward pass; both backward passes read the mask instead of the output.
PACKED_RELU_MASK = True


class Arena:
    """Bump allocator over one CUDA allocation (activations, gradients of activations, scratch of one learner)."""

    GUARD_WORDS = 64                     # canary words behind every allocation (debug option)
    GUARD_PATTERN = 0x5AC0FFEE

    def __init__(self, device, nbytes: int = 0, canaries: bool = False):
        self.device = device
        self.chunks: List[torch.Tensor] = []
        self.total = 0
        self.canaries = canaries
        self.guards: List[torch.Tensor] = []

    def alloc(self, numel: int, dtype=torch.float32, zero=False) -> torch.Tensor:
        # separate torch allocations keep this simple; 256-byte alignment is guaranteed by the caching allocator
        numel = max(1, numel)
        if not self.canaries:
            t = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=self.device)
            self.chunks.append(t)
            self.total += t.numel() * t.element_size()
            return t
        # debug: a guard of known words follows the tensor; a kernel that writes past the end of its output changes it
        full = (torch.zeros if zero else torch.empty)(numel + self.GUARD_WORDS, dtype=dtype, device=self.device)
        guard = full[numel:].view(torch.int32)
        guard.fill_(self.GUARD_PATTERN)
        self.chunks.append(full)
        self.guards.append(guard)
        self.total += full.numel() * full.element_size()
        return full[:numel]

    def check_canaries(self) -> int:
        """Number of guards that no longer hold the pattern (0 when intact or when the option is off)."""
        if not self.guards:
            return 0
        bad = torch.stack([(g != self.GUARD_PATTERN).any() for g in self.guards])
        return int(bad.sum().item())


class T:
    """A device tensor in the program: storage + logical channels-last shape."""
    __slots__ = ("buf", "n", "h", "w", "c", "grad", "grad_written", "needs_grad", "name", "bn_info")

    def __init__(self, buf, n, h, w, c, name=""):
        self.buf, self.n, self.h, self.w, self.c = buf, n, h, w, c
        self.grad: Optional[torch.Tensor] = None
        self.grad_written = False
        self.needs_grad = False
        self.name = name
        self.bn_info = None          # node_info of the normalisation group that produced this tensor, if any

    @property
    def rows(self):
        return self.n * self.h * self.w

    @property
    def numel(self):
        return self.rows * self.c

    def nhwc(self):
        return self.buf[: self.numel].view(self.n, self.h, self.w, self.c)


class ReplicaBuffers:
    """Flat device vectors of one replica (device element order, padded)."""

    def __init__(self, model: Model, device, init: Optional[torch.Tensor] = None):
        n = model.device_elements
        self.n = n
        self.w = torch.zeros(n, device=device) if init is None else init.clone()
        self.g = torch.zeros(n, device=device)
        self.last = torch.zeros(n, device=device)
        self.prev = self.w.clone()
        self.wt = torch.zeros(max(1, n), device=device)      # transposed copies of convolution weights for dgrad


class DeviceShared:
    """State shared by all learners of one GPU: central model z, its momentum, S-SGD accumulator, BN running stats."""

    def __init__(self, model: Model, device, init: torch.Tensor, z_storage: Optional[torch.Tensor] = None):
        n = model.device_elements
        if z_storage is not None:            # peer-visible memory provided by the synchroniser
            self.z = z_storage
            self.z.copy_(init)
        else:
            self.z = init.clone()
        self.zlast = torch.zeros(n, device=device)
        self.gacc = torch.zeros(n, device=device)
        self.run_mean: Dict[int, torch.Tensor] = {}
        self.run_var: Dict[int, torch.Tensor] = {}
        self.device = device

    def running(self, op_uid: int, channels: int):
        if op_uid not in self.run_mean:
            self.run_mean[op_uid] = torch.zeros(channels, device=self.device)
            self.run_var[op_uid] = torch.ones(channels, device=self.device)
        return self.run_mean[op_uid], self.run_var[op_uid]


def _op(kind, flags=0, ia=(), fa=(), la=(), p=()) -> L.XbOp:
    o = L.XbOp()
    o.kind, o.flags = kind, flags
    for i, v in enumerate(ia):
        o.ia[i] = int(v)
    for i, v in enumerate(fa):
        o.fa[i] = float(v)
    for i, v in enumerate(la):
        o.la[i] = int(v)
    for i, v in enumerate(p):
        o.p[i] = v if isinstance(v, int) else (0 if v is None else v.data_ptr())
    return o


class Lowering:
    def __init__(self, graph: SubGraph, model: Model, batch: int, input_chw, device, weights: torch.Tensor,
                 replica: Optional[ReplicaBuffers], shared: DeviceShared, params_dev: torch.Tensor, params_host_ptr: int,
                 result_dev_ptr: int,
                 update_model: UpdateModel = UpdateModel.SMA, training=True, use_tc=True, clip=False,
                 lr_mult: Optional[torch.Tensor] = None, seed_stream_base=0, splits: int = 1, reuse_memory: bool = False,
                 gradient_buckets: int = 1, canaries: bool = False, operator_branches: bool = True):
        """`operator_branches`: put every layer's weight / bias gradient on a parallel branch of the task graph (they are
        only read by the optimiser), so that the backward pass's critical path is the chain of data gradients alone.  Off
        with `reuse_memory` (buffer lifetimes are derived from the list order) and with gradient buckets (their segments
        are cut where the optimiser steps stand)."""
        if splits < 1 or batch % splits:
            raise ValueError("error: the batch size must be a multiple of the number of splits")
        # `--splits` (taskhandler.c:65-114): one task runs the whole graph `splits` times over consecutive sub-batches of
        # the staged batch.  The program is lowered for ONE sub-batch and its operator list repeated with shifted inputs.
        self.splits, full_batch = splits, batch
        batch = batch // splits
        self.g, self.model, self.batch, self.device = graph, model, batch, device
        self.weights = weights              # flat vector the forward pass reads (replica weights, or z for tests)
        self.replica, self.shared = replica, shared
        self.params_dev, self.params_host_ptr, self.result_ptr = params_dev, params_host_ptr, result_dev_ptr
        self.update_model, self.training, self.use_tc, self.clip = update_model, training, use_tc, clip
        self.lr_mult = lr_mult
        self.arena = Arena(device, canaries=canaries)
        self._count_pass, self._gout_count, self._gout_total = False, {}, {}
        self.all_tensors: List[T] = []
        self.reuse_memory = reuse_memory
        self.gradient_buckets = gradient_buckets
        self.side = L.F_SIDE if (operator_branches and training and not reuse_memory
                                 and not (gradient_buckets > 1 and update_model == UpdateModel.WORKER)) else 0
        self.buckets: List[tuple] = []      # (offset, elements) of each gradient bucket, in the order the backward pass completes them
        self.bytes_before_reuse = 0
        self.ops: List[L.XbOp] = []
        self.keep = []                      # python objects that must outlive the program (descriptor tables ...)
        c, h, w = input_chw
        self.input_chw = (c, h, w)
        self.examples = self.arena.alloc(full_batch * c * h * w)            # NCHW staging buffer (H2D target), whole batch
        self.labels = self.arena.alloc(full_batch, dtype=torch.int32)
        self.tensors: Dict[int, T] = {}     # id(node) -> output tensor
        bn_channels = sum(n.op.output_shape.dims[1] for n in graph.order if n.op.kernel.kind == "batchnorm")
        self.zero_region = self.arena.alloc(4 * bn_channels + 64, zero=True)   # per-task accumulators, cleared by one memset
        self.zero_used = 0
        self.x_in: Optional[T] = None
        self.node_info: Dict[int, dict] = {}
        self.logits: Optional[T] = None
        self.probs: Optional[T] = None
        self._build()

    # ---- helpers ----
    def wptr(self, var, base: Optional[torch.Tensor] = None) -> int:
        base = self.weights if base is None else base
        return base.data_ptr() + 4 * var.doffset

    def new_tensor(self, n, h, w, c, name="") -> T:
        t = T(self.arena.alloc(n * h * w * c), n, h, w, c, name)
        self.all_tensors.append(t)
        return t

    def grad_of(self, t: T) -> torch.Tensor:
        if t.grad is None:
            t.grad = self.arena.alloc(t.numel)
        return t.grad

    def gout(self, t: T):
        """(pointer, accumulate) for a backward op that contributes to t's gradient."""
        g = self.grad_of(t)
        acc = t.grad_written
        t.grad_written = True
        self._gout_count[id(t)] = self._gout_count.get(id(t), 0) + 1
        return g, int(acc)

    def _last_contribution(self, t: T) -> bool:
        """True (in the emitting pass) when the gout() just issued for t was the final one: t's gradient is complete after it."""
        return (not self._count_pass) and self._gout_total.get(id(t), -1) == self._gout_count.get(id(t), 0)

    def emit(self, op):
        self.ops.append(op)

    # ---- build ----
    def _consumers(self, node):
        return [m for m in node.next if not m.op.kernel.is_gradient and not m.op.kernel.is_optimiser
                and not getattr(m.op.kernel, "is_gradient_merge", False)]

    def _inputs(self, node):
        return [p for p in node.prev if not p.op.kernel.is_gradient]

    def _build(self):
        fwd = [n for n in self.g.order if not n.op.kernel.is_gradient and not n.op.kernel.is_optimiser
               and not getattr(n.op.kernel, "is_gradient_merge", False)]
        self.fwd = fwd
        has_grad = self.training and any(n.op.kernel.is_gradient for n in self.g.order)
        self.has_backward = has_grad
        differentiated = {n.op.peer.uid for n in self.g.order if n.op.kernel.is_gradient and n.op.peer is not None}
        # task parameters first, then zero the per-task accumulators (filled in at the end, once sizes are known)
        self.emit(_op(L.OP_UPLOAD, la=[C.sizeof(L.XbTaskParams)], p=[self.params_dev, self.params_host_ptr]))
        zero_slot = len(self.ops)
        self.emit(_op(L.OP_MEMSET, la=[4], p=[self.params_dev]))                              # placeholder, patched below
        transpose_slot = None
        if has_grad:
            transpose_slot = len(self.ops)
            self.emit(_op(L.OP_MEMSET, la=[0], p=[0]))                                        # placeholder
        self._plan_fusion(fwd)
        c, h, w = self.input_chw
        x_in = None
        if not fwd[0].op.kernel.is_data_transform:
            x_in = self.new_tensor(self.batch, h, w, c, "input")
            self.x_in = x_in
            self.emit(_op(L.OP_TRANSFORM, ia=[self.batch, c, h, w, h, w, 0, 0, 0, 0], fa=[1.0],
                          p=[self.examples, x_in.buf, 0, self.params_dev]))
        for n in fwd:
            self._forward(n, x_in)
        if has_grad:
            # Pass 1 only counts the contributions every activation gradient receives, so that pass 2 knows which operator
            # completes a gradient (that operator's epilogue can then produce the batch-norm backward sums of its owner).
            mark_ops, mark_zero = len(self.ops), self.zero_used
            written = {id(t): t.grad_written for t in self.tensors.values() if t is not None}
            self._count_pass, self._gout_count, self._gout_total = True, {}, {}
            self._backward(fwd, differentiated)
            del self.ops[mark_ops:]
            self.zero_used = mark_zero
            for t in self.tensors.values():
                if t is not None:
                    t.grad_written = written.get(id(t), False)
            if self.x_in is not None:
                self.x_in.grad_written = False
            self._count_pass, self._gout_total, self._gout_count = False, self._gout_count, {}
            self._backward(fwd, differentiated)
            self._finish_transposes(transpose_slot)
            self._optimiser()
        # one memset clears all per-task accumulators (BN sums, BN backward sums)
        self.ops[zero_slot] = _op(L.OP_MEMSET, la=[4 * self.zero_used], p=[self.zero_region])
        if (self.gradient_buckets > 1 and self.update_model == UpdateModel.WORKER and not self.clip and self.splits == 1
                and self.ops and self.ops[-1].kind == L.OP_OPTIMISER):
            self._bucket_gradients(self.gradient_buckets)
        if self.splits > 1:
            self._repeat_for_splits()
        if self.reuse_memory:
            self._reuse_buffers()

    def _reuse_buffers(self):
        """`--reuse-memory` (MemoryPlannerV2.java:117-296): activations and activation gradients whose lifetimes do not overlap
        share storage.  Lifetimes are read off the finished operator list (first and last operator that names a buffer), a
        best-fit scan assigns buffers to slots, and the operators' pointers are patched; a learner's operators run in
        stream order, so the aliasing is safe.  Inspecting intermediate tensors after a run is meaningless with this on."""
        cands = {}
        for t in self.all_tensors:
            for b in (t.buf, t.grad):
                if b is not None:
                    cands[b.data_ptr()] = b
        first, last = {}, {}
        for i, o in enumerate(self.ops):
            for j in range(len(o.p)):
                p = o.p[j]
                if p in cands:
                    first.setdefault(p, i)
                    last[p] = i
        slots = []                                           # [capacity in elements, last operator that uses it, members]
        home = {}
        for p in sorted(first, key=first.get):
            need = cands[p].numel()
            best = None
            for sl in slots:
                if sl[1] < first[p] and sl[0] >= need and (best is None or sl[0] < best[0]):
                    best = sl
            if best is None:
                best = [need, -1, []]
                slots.append(best)
            best[1] = last[p]
            best[2].append(p)
            home[p] = best
        self.bytes_before_reuse = self.arena.total
        storage = {id(sl): torch.empty(sl[0], device=self.device) for sl in slots}
        new_ptr = {p: storage[id(sl)].data_ptr() for p, sl in home.items()}
        for o in self.ops:
            for j in range(len(o.p)):
                if o.p[j] in new_ptr:
                    o.p[j] = new_ptr[o.p[j]]
        for t in self.all_tensors:
            if t.buf is not None and t.buf.data_ptr() in home:
                t.buf = storage[id(home[t.buf.data_ptr()])][: t.buf.numel()]
            if t.grad is not None and t.grad.data_ptr() in home:
                t.grad = storage[id(home[t.grad.data_ptr()])][: t.grad.numel()]
        dropped = set(home)
        self.arena.chunks = [c for c in self.arena.chunks if c.data_ptr() not in dropped] + list(storage.values())
        self.arena.total = sum(c.numel() * c.element_size() for c in self.arena.chunks)

    def _repeat_for_splits(self):
        """Operator list of one sub-batch -> `splits` copies reading consecutive windows of the staged batch.  The loss and
        accuracy slot receives the mean over the sub-batches."""
        c, h, w = self.input_chw
        ex0, lab0 = self.examples.data_ptr(), self.labels.data_ptr()
        ex_step, lab_step = 4 * self.batch * c * h * w, 4 * self.batch
        head, body = self.ops[:1], self.ops[1:]          # (the task parameters are uploaded once)
        out = list(head)
        for s in range(self.splits):
            for o in body:
                q = L.XbOp()
                C.memmove(C.byref(q), C.byref(o), C.sizeof(L.XbOp))
                for i in range(len(q.p)):
                    if q.p[i] == ex0:
                        q.p[i] = ex0 + s * ex_step
                    elif q.p[i] == lab0:
                        q.p[i] = lab0 + s * lab_step
                if q.kind == L.OP_SOFTMAX_XENT:
                    q.ia[4], q.ia[5] = s, self.splits
                out.append(q)
        self.ops = out

    def scratch_zeroed(self, numel) -> torch.Tensor:
        if self.zero_used + numel > self.zero_region.numel():
            raise RuntimeError("per-task accumulator region is too small")
        t = self.zero_region[self.zero_used:self.zero_used + numel]
        self.zero_used += (numel + 3) // 4 * 4
        return t

    def _plan_fusion(self, fwd):
        info = self.node_info
        for n in fwd:
            info[id(n)] = dict(fused_into=None, relu=None, stats_from=None, deferred=False, carrier=None, res=None)
        for n in fwd:
            k = n.op.kernel
            cons = self._consumers(n)
            if k.kind in ("conv", "innerproduct") and len(cons) == 1 and cons[0].op.kernel.kind == "relu" \
                    and cons[0].op.kernel.conf.activation_mode == ActivationMode.RELU and cons[0].op.kernel.conf.negative_slope == 0:
                info[id(n)]["relu"] = cons[0]
                info[id(cons[0])]["fused_into"] = n
            if k.kind == "batchnorm":
                if len(cons) == 1 and cons[0].op.kernel.kind == "relu" and cons[0].op.kernel.conf.negative_slope == 0 \
                        and cons[0].op.kernel.conf.activation_mode == ActivationMode.RELU:
                    info[id(n)]["relu"] = cons[0]
                    info[id(cons[0])]["fused_into"] = n
                elif len(cons) == 1 and cons[0].op.kernel.kind == "elementwise" and len(self._inputs(cons[0])) == 2 \
                        and cons[0].op.kernel.conf.type == ElementWiseOpType.SUM \
                        and all(cons[0].op.kernel.conf.getCoefficient(i) == 1.0 for i in range(2)) \
                        and info[id(cons[0])]["carrier"] is None and not getattr(cons[0].op.kernel, "is_gradient_merge", False):
                    s = cons[0]
                    info[id(n)]["deferred"] = True
                    info[id(s)]["carrier"] = n
                    sc = self._consumers(s)
                    if len(sc) == 1 and sc[0].op.kernel.kind == "relu" and sc[0].op.kernel.conf.negative_slope == 0 \
                            and sc[0].op.kernel.conf.activation_mode == ActivationMode.RELU:
                        info[id(s)]["relu"] = sc[0]
                        info[id(sc[0])]["fused_into"] = s
        # conv epilogue statistics: producer (after optional fused relu) feeds exactly one BN, training mode
        if self.training:
            for n in fwd:
                if n.op.kernel.kind != "batchnorm":
                    continue
                src = self._inputs(n)[0]
                prod = info[id(src)]["fused_into"] or src
                if prod.op.kernel.kind == "conv" and len(self._consumers(src)) == 1:
                    info[id(n)]["stats_from"] = prod

    def out_tensor(self, node) -> T:
        return self.tensors[id(node)]

    def _forward(self, n, x_in):
        k, info = n.op.kernel, self.node_info[id(n)]
        ins_nodes = self._inputs(n)
        ins = [self.out_tensor(p) for p in ins_nodes] if ins_nodes else [x_in]
        kind = k.kind
        P = self.params_dev
        if info["fused_into"] is not None:           # ReLU folded into its producer
            self.tensors[id(n)] = self.out_tensor(info["fused_into"])
            return
        if kind == "datatransform":
            c, h, w = self.input_chw
            oh, ow = n.op.output_shape.dims[2], n.op.output_shape.dims[3]
            out = self.new_tensor(self.batch, oh, ow, c, "transform")
            conf = k.conf
            mean, mode = None, 0
            if conf.subtract_mean and conf.mean_pixel_values:
                mean, mode = torch.tensor(conf.mean_pixel_values, dtype=torch.float32, device=self.device), 1
            elif conf.subtract_mean and conf.mean_image_filename:
                mean, mode = torch.from_numpy(np.fromfile(conf.mean_image_filename, dtype=np.float32)).to(self.device), 2
            self.keep.append(mean)
            self.emit(_op(L.OP_TRANSFORM, ia=[self.batch, c, h, w, oh, ow, int(bool(conf.mirror)), int(self.training), mode, n.op.uid],
                          fa=[conf.scale_factor], p=[self.examples, out.buf, mean, P]))
            self.tensors[id(n)] = out
            return
        x = ins[0]
        if kind in ("conv", "innerproduct"):
            if kind == "conv":
                conf = k.conf
                K = conf.number_of_outputs
                geom = [x.n, x.h, x.w, x.c, K, conf.kernel_height, conf.kernel_width, n.op.output_shape.dims[2],
                        n.op.output_shape.dims[3], conf.stride_height, conf.stride_width, conf.padding_height, conf.padding_width]
                out = self.new_tensor(x.n, geom[7], geom[8], K, n.op.name)
            else:
                K = k.conf.number_of_outputs
                geom = [x.n, 1, 1, x.h * x.w * x.c, K, 1, 1, 1, 1, 1, 1, 0, 0]
                out = self.new_tensor(x.n, 1, 1, K, n.op.name)
            out.needs_grad = True
            wv = k.variables[0]
            bias = self.wptr(k.variables[1]) if len(k.variables) > 1 else 0
            flags = L.F_TC if self.use_tc else 0
            if info["relu"] is not None:
                flags |= L.F_RELU
            stats = None
            # does a BN take its statistics from this convolution?
            for m in self.fwd:
                if self.node_info[id(m)].get("stats_from") is n:
                    stats = self.scratch_zeroed(2 * K)
                    self.node_info[id(m)]["stats_buf"] = stats
                    flags |= L.F_STATS
            info["geom"] = geom
            # layers no direct tensor-core kernel covers are lowered to a patch matrix + GEMM and need scratch for it
            info["im2col"] = self._im2col_scratch(geom) if self.use_tc else None
            self.emit(_op(L.OP_CONV_FPROP, flags, ia=geom, p=[x.buf, self.wptr(wv), bias, out.buf, stats,
                                                              info["im2col"] if L.load().xb_conv_im2col_wanted(self._geom_struct(geom), 0) else None]))
            self.tensors[id(n)] = out
            return
        if kind == "batchnorm":
            if info["stats_from"] is None and self.training:
                info["stats_buf"] = self.scratch_zeroed(2 * x.c)
                self.emit(_op(L.OP_BN_STATS, ia=[x.rows, x.c], p=[x.buf, info["stats_buf"]]))
            if info["deferred"]:
                self.tensors[id(n)] = None   # materialised by the sum node
                return
            self._emit_bn(n, x, None, info["relu"] is not None)
            return
        if kind == "elementwise":
            carrier = info["carrier"]
            if carrier is not None:
                other = [p for p in ins_nodes if p is not carrier][0]
                bn_in = self.out_tensor(self._inputs(carrier)[0])
                res = self.out_tensor(other)
                info["res"] = other
                out = self._emit_bn(carrier, bn_in, res, info["relu"] is not None, at=n)
                return
            out = self.new_tensor(x.n, x.h, x.w, x.c, n.op.name)
            out.needs_grad = any(t.needs_grad for t in ins)
            if k.conf.type != ElementWiseOpType.SUM:
                raise NotImplementedError("error: only SUM element-wise operators run on the GPU (as in the reference)")
            coefs = [k.conf.getCoefficient(i) for i in range(len(ins))]
            for base in range(0, len(ins), 4):
                part = ins[base:base + 4]
                self.emit(_op(L.OP_SUM, ia=[len(part), int(base > 0)], fa=coefs[base:base + 4], la=[x.numel],
                              p=[(part[i].buf if i < len(part) else None) for i in range(4)] + [out.buf]))
            self.tensors[id(n)] = out
            return
        if kind == "relu":
            out = self.new_tensor(x.n, x.h, x.w, x.c, n.op.name)
            out.needs_grad = x.needs_grad
            conf = k.conf
            self.emit(_op(L.OP_ACT_FWD, ia=[int(conf.activation_mode)], fa=[conf.negative_slope, conf.ceiling], la=[x.numel], p=[x.buf, out.buf]))
            self.tensors[id(n)] = out
            return
        if kind == "pool":
            conf = k.conf
            oh, ow = n.op.output_shape.dims[2], n.op.output_shape.dims[3]
            out = self.new_tensor(x.n, oh, ow, x.c, n.op.name)
            out.needs_grad = x.needs_grad
            geom = [x.n, x.h, x.w, x.c, oh, ow, conf.kernel_height, conf.kernel_width, conf.stride_height, conf.stride_width,
                    conf.padding_height, conf.padding_width]
            info["geom"] = geom
            self.emit(_op(L.OP_POOL_FWD, int(conf.method == PoolMethod.AVERAGE), ia=geom, p=[x.buf, out.buf]))
            self.tensors[id(n)] = out
            return
        if kind == "dropout":
            if not self.training:
                self.tensors[id(n)] = x
                return
            out = self.new_tensor(x.n, x.h, x.w, x.c, n.op.name)
            out.needs_grad = x.needs_grad
            self.emit(_op(L.OP_DROPOUT, ia=[n.op.uid, 0], fa=[k.conf.ratio], la=[x.numel], p=[x.buf, out.buf, P]))
            self.tensors[id(n)] = out
            return
        if kind == "concat":
            ct = sum(t.c for t in ins)
            out = self.new_tensor(x.n, x.h, x.w, ct, n.op.name)
            out.needs_grad = any(t.needs_grad for t in ins)
            off = 0
            for t in ins:
                self.emit(_op(L.OP_CONCAT, ia=[t.c, ct, off, 1, 0], la=[t.rows], p=[t.buf, out.buf]))
                off += t.c
            self.tensors[id(n)] = out
            return
        if kind == "lrn":
            out = self.new_tensor(x.n, x.h, x.w, x.c, n.op.name)
            out.needs_grad = x.needs_grad
            info["scale"] = self.arena.alloc(x.numel)
            c = k.conf
            self.emit(_op(L.OP_LRN_FWD, ia=[x.c, c.local_size], fa=[c.alpha, c.beta, c.k], la=[x.rows], p=[x.buf, out.buf, info["scale"]]))
            self.tensors[id(n)] = out
            return
        if kind == "softmax":
            probs = self.new_tensor(x.n, 1, 1, x.numel // x.n, "probs")
            self.logits, self.probs = x, probs
            cons = self._consumers(n)
            loss = next((m for m in cons if m.op.kernel.kind == "softmaxloss"), None)
            want_grad = self.has_backward and loss is not None and x.needs_grad
            dl = None
            if want_grad:
                dl, _ = self.gout(x)
            lconf = loss.op.kernel.conf if loss is not None else None
            mode = 0 if lconf is None or lconf.mode in (NormalisationMode.BATCH, NormalisationMode.FULL) else \
                (1 if lconf.mode == NormalisationMode.VALID else 2)
            ignore = lconf.ignored_label_value if lconf is not None else -1
            self.emit(_op(L.OP_SOFTMAX_XENT, ia=[x.n, x.numel // x.n, ignore, mode], p=[x.buf, self.labels, probs.buf, dl, self.result_ptr]))
            self.tensors[id(n)] = probs
            return
        if kind in ("softmaxloss", "accuracy"):
            self.tensors[id(n)] = None
            return
        if kind == "classify":
            out = self.new_tensor(x.n, 1, 1, 1, "classes")
            self.emit(_op(L.OP_CLASSIFY, ia=[x.n, x.numel // x.n], p=[x.buf, out.buf]))
            self.tensors[id(n)] = out
            return
        if kind == "matfact":
            conf = k.conf
            u, v = k.variables
            train = self.has_backward and self.replica is not None
            du = self.wptr(u, self.replica.g) if train else 0
            dv = self.wptr(v, self.replica.g) if train else 0
            # examples are (row, column[, rating]) rows; the ratings are the task's labels, as in the reference (matfact.cu:26-29)
            src = self.x_in if self.x_in is not None else x
            self.emit(_op(L.OP_MATFACT, ia=[src.numel // src.n, src.n, conf.number_of_latent_variables, conf.number_of_rows, conf.number_of_columns],
                          fa=[conf.lambda_], p=[src.buf, self.labels, self.wptr(u), self.wptr(v), du, dv, self.result_ptr]))
            self.tensors[id(n)] = None
            return
        if kind == "noop":
            self.tensors[id(n)] = x
            return
        raise NotImplementedError(f"error: operator kind {kind} has no device lowering")

    def _emit_bn(self, bn_node, x: T, res: Optional[T], relu: bool, at=None) -> T:
        k, info = bn_node.op.kernel, self.node_info[id(bn_node)]
        conf = k.conf
        out = self.new_tensor(x.n, x.h, x.w, x.c, bn_node.op.name)
        out.needs_grad = True
        rm, rv = self.shared.running(bn_node.op.uid, x.c)
        sm = self.arena.alloc(x.c)
        si = self.arena.alloc(x.c)
        # ReLU with a residual input: the mask cannot be re-derived from x alone, so the forward pass leaves a packed sign
        # mask (one byte per four channels) and the backward passes read that instead of the whole output
        mask = None
        if self.training and self.has_backward and relu and res is not None and x.c % 4 == 0 and PACKED_RELU_MASK:
            mask = self.arena.alloc((x.numel // 4 + 3) // 4 + 4)
        info.update(save_mean=sm, save_invstd=si, x=x, res=res, relu_fused=relu, out=out, mask=mask)
        out.bn_info = info
        cma = int(conf.estimated_mean_and_variance_type == BatchNormEstimatedMeanAndVarianceType.CMA)
        self.emit(_op(L.OP_BN_FWD, ia=[x.rows, x.c, int(relu), int(self.training), cma], fa=[k.epsilon(), 1.0 - float(conf.fraction)],
                      p=[x.buf, res.buf if res is not None else None, out.buf, info.get("stats_buf"), self.wptr(k.variables[0]),
                         self.wptr(k.variables[1]), rm, rv, sm, si, self.params_dev, mask]))
        self.tensors[id(at if at is not None else bn_node)] = out
        if at is not None:
            self.tensors[id(bn_node)] = None
        return out

    def _geom_struct(self, geom):
        g = L.XbConvGeom()
        (g.N, g.H, g.W, g.C, g.K, g.R, g.S, g.P, g.Q, g.sh, g.sw, g.ph, g.pw) = [int(v) for v in geom]
        return C.byref(g)

    def _im2col_scratch(self, geom):
        """Scratch for the patch-matrix path of one layer (shared by its forward and weight-gradient operators)."""
        need = max(L.load().xb_conv_im2col_wanted(self._geom_struct(geom), 0), L.load().xb_conv_im2col_wanted(self._geom_struct(geom), 2))
        return self.arena.alloc((need + 3) // 4) if need > 0 else None

    # ---- backward ----
    def _backward(self, fwd, differentiated):
        rep = self.replica
        self.transposes = []
        for n in reversed(fwd):
            k, info = n.op.kernel, self.node_info[id(n)]
            kind = k.kind
            if info["fused_into"] is not None or kind in ("softmax", "softmaxloss", "accuracy", "classify", "datatransform", "noop", "matfact"):
                continue
            if kind == "batchnorm" and info["deferred"]:
                continue          # handled at its sum node
            active = n.op.uid in differentiated or (kind == "elementwise" and info["carrier"] is not None
                                                    and info["carrier"].op.uid in differentiated)
            if not active:
                continue
            ins_nodes = self._inputs(n)
            out = self.tensors.get(id(n))
            if out is None or out.grad is None or not out.grad_written:
                continue          # nothing flows back through this node
            dy = out.grad
            if kind in ("conv", "innerproduct"):
                x = self.out_tensor(ins_nodes[0]) if ins_nodes else self.x_in
                geom = info["geom"]
                if info["relu"] is not None:   # mask by the fused ReLU, in place
                    self.emit(_op(L.OP_ACT_BWD, ia=[1, 0], fa=[0.0, 0.0], la=[out.numel], p=[dy, out.buf, out.buf, dy]))
                wv = k.variables[0]
                tc = L.F_TC if self.use_tc else 0
                scratch = info.get("im2col") if (tc and L.load().xb_conv_im2col_wanted(self._geom_struct(geom), 2)) else None
                # 0x20: the layer's forward pass went through the same patch matrix and left it in the scratch
                keep = 0x20 if (scratch is not None and L.load().xb_conv_im2col_wanted(self._geom_struct(geom), 0)) else 0
                # (weight and bias gradients feed nothing but the optimiser: a parallel branch of the task graph)
                self.emit(_op(L.OP_CONV_WGRAD, tc | keep | self.side, ia=geom, p=[dy, x.buf, self.wptr(wv, rep.g), scratch]))
                if len(k.variables) > 1:
                    self.emit(_op(L.OP_COLSUM, self.side, ia=[out.rows, out.c], p=[dy, self.wptr(k.variables[1], rep.g)]))
                if x.needs_grad:
                    gx, acc = self.gout(x)
                    K, R, S, Cc = geom[4], geom[5], geom[6], geom[3]
                    self.transposes.append((wv.doffset, K, R * S, Cc))
                    up = None
                    if tc:
                        if "s2up" not in info:
                            need = L.load().xb_conv3x3_s2_dgrad_scratch(self._geom_struct(geom))
                            info["s2up"] = self.arena.alloc(need // 4) if need > 0 else None   # zero-inserted output gradient
                        up = info["s2up"]
                    bnp, bflags = [None] * 5, 0
                    bi = x.bn_info
                    if (FUSE_BN_BACKWARD_SUMS and tc and bi is not None and self._last_contribution(x)
                            and (up is not None or L.load().xb_conv_dgrad_fuses_bn(self._geom_struct(geom)))):
                        # this operator completes the gradient of a normalisation layer's output: its epilogue also produces
                        # that layer's backward sums, and the layer's own reduction kernel is skipped
                        bi["dsums_fused"] = self.scratch_zeroed(2 * x.c)
                        bnp = [bi["x"].buf, x.buf, bi["save_mean"], bi["save_invstd"], bi["dsums_fused"]]
                        bflags = 0x8 | (0x10 if bi["relu_fused"] else 0)
                    self.emit(_op(L.OP_CONV_DGRAD, tc | acc | bflags, ia=geom, p=[dy, rep.wt.data_ptr() + 4 * wv.doffset, gx, up] + bnp))
                continue
            if kind == "batchnorm" or (kind == "elementwise" and info["carrier"] is not None):
                bn = n if kind == "batchnorm" else info["carrier"]
                bi = self.node_info[id(bn)]
                bk = bn.op.kernel
                x, res, relu = bi["x"], bi["res"], bi["relu_fused"]
                fused = bi.pop("dsums_fused", None)        # sums already produced by the operator that completed dy
                dsums = fused if fused is not None else self.scratch_zeroed(2 * x.c)
                gx, accx = self.gout(x)
                gres, accr = (None, 0)
                if res is not None and res.needs_grad:
                    gres, accr = self.gout(res)
                # ReLU fused, no residual: the kernels re-derive the mask from x and never read the layer's output
                remask = self.wptr(bk.variables[1]) if (relu and res is None and fused is None) else None
                packed = bi.get("mask") if fused is None else None
                self.emit(_op(L.OP_BN_BWD, ia=[x.rows, x.c, 3 if packed is not None else int(relu), accx, accr, int(fused is not None)],
                              p=[dy, x.buf, packed if packed is not None else out.buf, bi["save_mean"], bi["save_invstd"], self.wptr(bk.variables[0]), dsums, gx, gres,
                                 self.wptr(bk.variables[0], rep.g), self.wptr(bk.variables[1], rep.g), remask]))
                continue
            x = self.out_tensor(ins_nodes[0])
            if kind == "elementwise":
                for i, p in enumerate(ins_nodes):
                    t = self.out_tensor(p)
                    if not t.needs_grad:
                        continue
                    gx, acc = self.gout(t)
                    self.emit(_op(L.OP_SUM, ia=[1, acc], fa=[k.conf.getCoefficient(i)], la=[t.numel], p=[dy, None, None, None, gx]))
                continue
            if not x.needs_grad:
                continue
            if kind == "relu":
                gx, acc = self.gout(x)
                conf = k.conf
                self.emit(_op(L.OP_ACT_BWD, ia=[int(conf.activation_mode), acc], fa=[conf.negative_slope, conf.ceiling], la=[x.numel],
                              p=[dy, x.buf, out.buf, gx]))
            elif kind == "pool":
                gx, acc = self.gout(x)
                avg = int(k.conf.method == PoolMethod.AVERAGE)
                self.emit(_op(L.OP_POOL_BWD, avg | (acc << 1), ia=info["geom"], p=[dy, x.buf, gx]))
            elif kind == "dropout":
                gx, acc = self.gout(x)
                self.emit(_op(L.OP_DROPOUT, ia=[n.op.uid, acc], fa=[k.conf.ratio], la=[x.numel], p=[dy, gx, self.params_dev]))
            elif kind == "concat":
                off = 0
                for p in ins_nodes:
                    t = self.out_tensor(p)
                    if t.needs_grad:
                        gx, acc = self.gout(t)
                        self.emit(_op(L.OP_CONCAT, ia=[t.c, out.c, off, 0, acc], la=[t.rows], p=[dy, gx]))
                    off += t.c
            elif kind == "lrn":
                gx, acc = self.gout(x)
                c = k.conf
                self.emit(_op(L.OP_LRN_BWD, ia=[x.c, c.local_size, acc], fa=[c.alpha, c.beta], la=[x.rows], p=[dy, x.buf, out.buf, info["scale"], gx]))
            else:
                raise NotImplementedError(f"error: no backward lowering for {kind}")

    def _finish_transposes(self, slot):
        if not self.transposes:
            self.ops[slot] = _op(L.OP_MEMSET, la=[0], p=[self.params_dev])
            return
        descs = (L.XbTransposeDesc * len(self.transposes))()
        blocks = 0
        for i, (off, K, RS, Cc) in enumerate(self.transposes):
            descs[i].src_off, descs[i].dst_off, descs[i].K, descs[i].RS, descs[i].C = off, off, K, RS, Cc
            descs[i].first_block = blocks
            blocks += L.load().xb_transpose_blocks(K, RS, Cc)
        raw = torch.frombuffer(bytearray(bytes(descs)), dtype=torch.uint8).to(self.device)
        self.keep.append(raw)
        # The transposed copy is only read by the data gradients: it is written on the task graph's parallel branch, under
        # the forward pass, and the first data gradient joins that branch.
        self.ops[slot] = _op(L.OP_TRANSPOSE_W, self.side, ia=[len(self.transposes), blocks], p=[self.weights, self.replica.wt, raw])
        if self.side:
            for o in self.ops[slot + 1:]:
                if o.kind == L.OP_CONV_DGRAD:
                    o.flags |= L.F_JOIN
                    break

    def _optimiser(self):
        rep, sh = self.replica, self.shared
        mode = {UpdateModel.WORKER: 2, UpdateModel.DEFAULT: 1}.get(self.update_model, 0)
        target = sh.gacc if mode == 2 else (sh.z if mode == 1 else None)
        norm2 = None
        if self.clip:
            norm2 = self.arena.alloc(1, zero=True)
            self.emit(_op(L.OP_GRAD_SUMSQ, la=[rep.n], p=[rep.g, norm2]))
        self.emit(_op(L.OP_OPTIMISER, ia=[mode], la=[rep.n], p=[rep.w, rep.g, rep.last, rep.prev, target, self.lr_mult, norm2, self.params_dev]))

    def _bucket_gradients(self, nb: int):
        """Synchronous SGD overlapped with the backward pass: the flat vector is cut into up to `nb` contiguous buckets
        of whole variables, from the last layer backwards.  The accumulate step of a bucket (the optimiser operator over
        that range) is issued right after the last operator that writes a gradient of the bucket, followed by a mark at
        which the learner records an event; the synchronisation of that bucket (gradient all-reduce fused with the
        momentum update, what synch/synchronoussgd.c:13-110 does once for the whole vector) waits for that event only,
        and so runs next to the backward pass of the earlier layers."""
        import bisect
        rep = self.replica
        opt = self.ops.pop()
        assert opt.kind == L.OP_OPTIMISER
        g0, n = rep.g.data_ptr(), rep.n
        vs = sorted(self.model.variables, key=lambda v: v.doffset)
        starts = [v.doffset for v in vs]
        # last operator that names an address inside the variable's slice of the gradient vector - or of the weight vector:
        # the synchronisation overwrites the replica's weights of the bucket, so their last reader must have been issued
        w0 = rep.w.data_ptr()
        last = [-1] * len(vs)
        for i, o in enumerate(self.ops):
            for j in range(12):
                a = o.p[j]
                for base in (g0, w0):
                    if a and base <= a < base + 4 * n:
                        last[bisect.bisect_right(starts, (a - base) // 4) - 1] = i
        # cut from the tail: a bucket closes once it holds its share of the vector
        share, cuts, hi, ready = (n + nb - 1) // nb, [], n, -1
        for vi in range(len(vs) - 1, -1, -1):
            ready = max(ready, last[vi])
            if hi - starts[vi] >= share or vi == 0:
                cuts.append((starts[vi] if vi else 0, hi, ready))
                hi = starts[vi]
        merged = []                            # buckets that complete at the same operator are one bucket
        for lo, hi, ready in cuts:
            if merged and merged[-1][2] >= ready:
                merged[-1] = (lo, merged[-1][1], merged[-1][2])
            else:
                merged.append((lo, hi, ready))
        if len(merged) < 2:
            self.ops.append(opt)
            return
        after: Dict[int, list] = {}
        for b, (lo, hi, ready) in enumerate(merged):
            sl = lambda t: (t.data_ptr() + 4 * lo) if t is not None else None
            o = _op(L.OP_OPTIMISER, ia=[2], la=[hi - lo],
                    p=[sl(rep.w), sl(rep.g), sl(rep.last), sl(rep.prev), sl(self.shared.gacc), sl(self.lr_mult), None, self.params_dev])
            after.setdefault(ready, []).extend([o, _op(L.OP_MARK, ia=[b])])
            self.buckets.append((lo, hi - lo))
        ops = list(after.get(-1, []))
        for i, o in enumerate(self.ops):
            ops.append(o)
            ops.extend(after.get(i, []))
        self.ops = ops

    def op_array(self):
        arr = (L.XbOp * len(self.ops))(*self.ops)
        return arr
