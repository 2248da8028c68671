"""CPU oracle: executes a dataflow graph and the optimiser / synchronisation algorithms in fp32 PyTorch.

Three jobs:

1. the definition every CUDA kernel and the fused synchronisation kernels are tested against;
2. the CPU execution mode (``--gpu false``): the reference runs ``kernel.compute`` per operator on the
   CPU (SubGraph.java:244-266) but cannot synchronise replicas there (ModelManager.java:329-350 calls
   into the GPU library unconditionally) - here CPU replicas synchronise with the same algorithms;
3. the timed CPU baseline for the LeNet / SMA / 2-replica configuration.

Algorithms (reference file:line):

* per-task local update  - kernels/optimisers/sma.cu:3-100, default.cu:3-132, synchronoussgd.cu:3-57
* SMA                    - synch/sma.c:13-231   (+ all-reduce synch/common.c:3-57)
* synchronous SGD        - synch/synchronoussgd.c:13-110, synch/common.c:198-220
* DEFAULT                - synch/default.c:5-44
* synchronous EAMSGD     - synch/synchronouseamsgd.c:5-101
* Polyak-Ruppert         - synch/polyakruppert.c:5-138
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .conf import SolverConf
from .graph import SubGraph
from .kernels import FLT_MIN, OpEnv
from .model import Model
from .types import MomentumMethod, NormalisationMode, Phase, Regularisation, UpdateModel


class ReplicaState:
    """Flat fp32 vectors of one model copy: weights, gradient, momentum (``last``) and the pre-update
    snapshot (``diff`` in clib-multigpu/model.h:40-45, written by the local optimiser)."""

    def __init__(self, w: torch.Tensor):
        self.w = w.clone()
        self.g = torch.zeros_like(w)
        self.last = torch.zeros_like(w)
        self.prev = w.clone()
        self.clock = 0
        self.updates = 0

    def clone(self) -> "ReplicaState":
        r = ReplicaState(self.w)
        r.g, r.last, r.prev = self.g.clone(), self.last.clone(), self.prev.clone()
        r.clock, r.updates = self.clock, self.updates
        return r


class DeviceState:
    """Per-GPU state shared by its replicas: central average model z (+ its momentum and gradient
    accumulator) and the batch-norm running statistics."""

    def __init__(self, w: torch.Tensor):
        self.z = w.clone()
        self.z_last = torch.zeros_like(w)
        self.G = torch.zeros_like(w)       # base-model gradient accumulator (S-SGD, SMA partial)
        self.op_state: Dict = {}
        self.replicas: List[ReplicaState] = []
        self.avg_count = 0                 # Polyak-Ruppert running-average counter


# --------------------------------------------------------------------------------------------
# Graph execution
# --------------------------------------------------------------------------------------------

class OracleExecutor:
    # Debug cross-check of the reference (Operator.java:232-259, SubGraph.java:261-262: under debug logging every operator
    # prints the checksum of its output): when `checksum_sink` is set, it is called with one line per operator and task,
    # "Kernel's <name> output checksum is <sum, 5 decimals>" (gradient operators: one sum per input gradient).
    checksum_sink = None

    def __init__(self, graph: SubGraph, model: Model, seed: int = 0):
        self.graph = graph
        self.model = model
        self.seed = seed

    def _checksum(self, op, value):
        sink = OracleExecutor.checksum_sink
        if sink is None:
            return
        vals = [v for v in (value if isinstance(value, list) else [value]) if v is not None]
        if not vals:
            sink(f"Kernel's {op.name} output list is empty")
            return
        sums = ", ".join(f"{float(v.double().sum()):.5f}" for v in vals)
        sink(f"Kernel's {op.name} output checksum{'s are' if len(vals) > 1 else ' is'} {sums}")

    def _params(self, kernel, w: torch.Tensor, requires_grad: bool):
        out = []
        for v in kernel.variables:
            p = w[v.offset:v.offset + v.elements()].reshape(v.shape.dims).detach().clone()
            out.append(p.requires_grad_(requires_grad))
        return out

    def run(self, w: torch.Tensor, examples: torch.Tensor, labels: Optional[torch.Tensor], phase=Phase.TRAIN,
            task_id=0, device_state: Optional[dict] = None, grad_out: Optional[torch.Tensor] = None,
            keep_outputs=False):
        """One task. Returns dict(loss, accuracy, outputs?).  If the graph has gradient nodes and
        ``grad_out`` is given, parameter gradients are ACCUMULATED into it (callers zero it per task)."""
        env = OpEnv(phase=phase, labels=labels, task_id=task_id, seed=self.seed,
                    device_state=device_state if device_state is not None else {})
        outs: Dict[int, object] = {}
        saved: Dict[int, tuple] = {}      # forward op uid -> (inputs_rg, params_rg, output)
        result = dict(loss=None, accuracy=None)
        train = phase == Phase.TRAIN
        for node in self.graph.order:
            op, k = node.op, node.op.kernel
            if k.is_optimiser:
                continue
            if not k.is_gradient:
                ins = [outs[id(p)] for p in node.prev if not p.op.kernel.is_gradient] or [examples]
                if getattr(k, "is_gradient_merge", False):
                    ins = [self._pick(outs[id(p)], p, node) for p in node.prev]
                    outs[id(node)] = sum(ins[1:], ins[0])
                    continue
                need_grad = train and grad_out is not None
                xin = [x.detach().clone().requires_grad_(need_grad and x.is_floating_point()) for x in ins]
                params = self._params(k, w, need_grad)
                with torch.enable_grad() if need_grad else torch.no_grad():
                    y = k.forward(xin, params, env)
                saved[op.uid] = (xin, params, y)
                outs[id(node)] = y.detach()
                self._checksum(op, outs[id(node)])
                if k.is_loss:
                    result["loss"] = float(y.detach().reshape(-1)[0])
                elif k.kind == "accuracy":
                    result["accuracy"] = float(y.detach().reshape(-1)[0])
                continue
            # ---- gradient operator ----
            if grad_out is None:
                continue
            peer = op.peer
            xin, params, y = saved[peer.uid]
            pk = peer.kernel
            if pk.is_loss and pk.kind == "softmaxloss":
                # gradient w.r.t. the logits that produced the probabilities: (p - onehot)/N
                p = xin[0].detach()
                lab = labels.long()
                valid = (lab != pk.conf.ignored_label_value)
                g = p.clone()
                g[torch.arange(p.shape[0]), lab.clamp(min=0)] -= 1.0
                g = g * valid.unsqueeze(1)
                denom = p.shape[0] if pk.conf.mode != NormalisationMode.VALID else max(1, int(valid.sum()))
                outs[id(node)] = [g / denom]
                self._checksum(op, outs[id(node)])
                continue
            ups = [self._pick(outs[id(p)], p, node) for p in node.prev]
            if pk.is_loss:
                gy = torch.ones_like(y)
            else:
                gy = ups[0]
                for u in ups[1:]:
                    gy = gy + u
                gy = gy.reshape(y.shape)
            wrt = [x for x in xin if x.requires_grad] + params
            grads = torch.autograd.grad(y, wrt, gy, allow_unused=True) if wrt else []
            gi, gin = 0, []
            for x in xin:
                if x.requires_grad:
                    gin.append(grads[gi] if grads[gi] is not None else torch.zeros_like(x))
                    gi += 1
                else:
                    gin.append(None)
            for v, gp in zip(pk.variables, grads[gi:]):
                if gp is not None:
                    grad_out[v.offset:v.offset + v.elements()] += gp.reshape(-1)
            outs[id(node)] = gin
            self._checksum(op, gin)
        if keep_outputs:
            result["outputs"] = {n.op.uid: (o if not isinstance(o, list) else o) for n in self.graph.order
                                 for o in [outs.get(id(n))] if o is not None}
        return result

    def _pick(self, value, producer_node, consumer_node):
        """A gradient node yields one gradient per input of its peer; give the consumer the one that
        belongs to the forward edge (consumer.peer -> producer.peer)."""
        if not isinstance(value, list):
            return value
        if len(value) == 1:
            return value[0]
        cpeer = consumer_node.op.peer or getattr(consumer_node.op, 'merge_of', None)
        ppeer = producer_node.op.peer
        if cpeer is not None and ppeer is not None:
            # find which input slot of ppeer is fed by cpeer
            fwd_inputs = self._forward_inputs(ppeer)
            for i, op in enumerate(fwd_inputs):
                if op is cpeer and value[i] is not None:
                    return value[i]
        return next(v for v in value if v is not None)

    def _forward_inputs(self, op):
        for n in self.graph.order:
            if n.op is op and not op.kernel.is_gradient:
                return [p.op for p in n.prev if not p.op.kernel.is_gradient]
        return []


# --------------------------------------------------------------------------------------------
# Per-task local update
# --------------------------------------------------------------------------------------------

def clip_and_regularise(r: ReplicaState, s: SolverConf):
    if s.clip_gradient_threshold is not None and s.clip_gradient_threshold >= 0:
        l2 = float(torch.sqrt((r.g * r.g).sum()))
        if l2 > s.clip_gradient_threshold:
            r.g *= s.clip_gradient_threshold / l2
    if s.weight_decay > 0:
        if s.regularisation_type == Regularisation.L1:
            r.g += s.weight_decay * torch.sign(r.w)
        else:
            r.g += s.weight_decay * r.w


def local_update(r: ReplicaState, dev: DeviceState, s: SolverConf, update_model: UpdateModel, task: int,
                 lr_mult: Optional[torch.Tensor] = None):
    """What the GradientDescentOptimiser node does after the backward pass of ONE task."""
    clip_and_regularise(r, s)
    lr = s.learning_rate(task)
    mu = s.momentum_at(task)
    g = r.g if lr_mult is None else r.g * lr_mult
    if update_model == UpdateModel.WORKER:
        dev.G += -lr * g                       # synchronoussgd.cu:36-54; replica weights untouched
    else:
        r.prev = r.w.clone()                   # snapshot BEFORE the step (sma.cu:71,87)
        if mu > 0:
            step = -lr * g + mu * r.last
            if s.momentum_method == MomentumMethod.NESTEROV:
                r.last = step.clone()
                step = -lr * g + mu * step
            else:
                r.last = step.clone()
        else:
            step = -lr * g
        r.w += step
        if update_model == UpdateModel.DEFAULT:
            dev.z += step                      # default.cu: same step applied to the device base model
    r.updates += 1
    r.g.zero_()


# --------------------------------------------------------------------------------------------
# Synchronisation algorithms (one call = one clock)
# --------------------------------------------------------------------------------------------

def _reduce(total: torch.Tensor, allreduce) -> torch.Tensor:
    """Sum over the devices of THIS process is in ``total``; ``allreduce`` (if given) adds the other processes'."""
    return allreduce(total) if allreduce is not None else total


def synchronise_sma(devs: Sequence[DeviceState], alpha: float, base_momentum: float = 0.9, copy: bool = False,
                    use_prev: bool = True, allreduce=None):
    """Synchronous model averaging over k replicas x G devices.

    Per device d: D_r = alpha*(prev_r - z_d); w_r -= D_r; G_d = sum_r D_r.  Then D = sum_d G_d (all-reduce);
    if momentum: D += mu*last_z; last_z = D; z_d += D on every device.  ``copy`` (raised when the
    learning rate has just dropped) overwrites every replica with z.  ``use_prev=False`` uses the replica's
    current weights instead of the pre-update snapshot.
    """
    for d in devs:
        d.G.zero_()
        for r in d.replicas:
            src = r.prev if use_prev else r.w
            diff = alpha * (src - d.z)
            r.w -= diff
            d.G += diff
    total = _reduce(sum((d.G for d in devs[1:]), devs[0].G.clone()), allreduce)
    for d in devs:
        D = total.clone()
        if base_momentum > 0:
            D += base_momentum * d.z_last
            d.z_last = D.clone()
        d.z += D
        if copy:
            for r in d.replicas:
                r.w = d.z.clone()


def synchronise_ssgd(devs: Sequence[DeviceState], wpc: int, momentum: float, allreduce=None):
    """S-SGD: all-reduce the accumulated -lr*(g+wd*w), scale by 1/wpc, momentum, apply to z, copy z to replicas."""
    total = _reduce(sum((d.G for d in devs[1:]), devs[0].G.clone()), allreduce)
    for d in devs:
        D = total / float(wpc)
        if momentum > 0:
            D = D + momentum * d.z_last
            d.z_last = D.clone()
        d.z += D
        d.G.zero_()
        for r in d.replicas:
            r.w = d.z.clone()


def synchronise_default(devs: Sequence[DeviceState]):
    """DEFAULT (single device): the base model already received every step; copy it to the replicas."""
    for d in devs:
        for r in d.replicas:
            r.w = d.z.clone()


def synchronise_eamsgd(devs: Sequence[DeviceState], alpha: float, base_momentum: float = 0.0, allreduce=None):
    """Elastic averaging, synchronous variant: each replica is pulled towards z by alpha*(w_r - z) and z moves
    by the sum of the pulls (optionally with momentum on z).  Multi-device: pulls are summed across devices."""
    for d in devs:
        d.G.zero_()
        for r in d.replicas:
            diff = alpha * (r.w - d.z)
            r.w -= diff
            d.G += diff
    total = _reduce(sum((d.G for d in devs[1:]), devs[0].G.clone()), allreduce)
    for d in devs:
        D = total.clone()
        if base_momentum > 0:
            D += base_momentum * d.z_last
            d.z_last = D.clone()
        d.z += D


def synchronise_polyak_ruppert(devs: Sequence[DeviceState], alpha: float = 0.0, allreduce=None, world: int = 1):
    """z becomes the running average (factor 1/(count+1)) of the mean of all replicas; optional elastic pull of
    the replicas towards z with strength alpha (polyakruppert.c:5-138)."""
    n = sum(len(d.replicas) for d in devs) * world
    mean = _reduce(sum((r.w for d in devs for r in d.replicas)), allreduce) / float(n)
    for d in devs:
        f = 1.0 / (d.avg_count + 1.0)
        d.z = (1.0 - f) * d.z + f * mean
        d.avg_count += 1
        if alpha > 0:
            for r in d.replicas:
                r.w -= alpha * (r.w - d.z)


def sma_base_momentum(solver: SolverConf) -> float:
    """Momentum applied to the central average model.  The reference overwrites it with 0.9 whenever the
    replicas use momentum (synch/sma.c:150-153) and never reads ``--base-model-momentum``; here that flag
    wins when it is set, otherwise the 0.9 rule applies."""
    if solver.base_model_momentum and solver.base_model_momentum > 0:
        return float(solver.base_model_momentum)
    return 0.9 if solver.momentum > 0 else 0.0


def synchronise(update_model: UpdateModel, devs: Sequence[DeviceState], solver: SolverConf, wpc: int, copy=False,
                allreduce=None, world: int = 1):
    """Dispatch as clib-multigpu/executioncontext.c:2262-2334 does.  ``allreduce`` sums a tensor over processes
    (one process per device group); ``world`` is the number of such processes."""
    if update_model in (UpdateModel.SMA, UpdateModel.SYNCHRONOUSEAMSGD):
        synchronise_sma(devs, solver.alpha, sma_base_momentum(solver), copy, allreduce=allreduce)
    elif update_model == UpdateModel.WORKER:
        synchronise_ssgd(devs, wpc, solver.momentum, allreduce=allreduce)
    elif update_model == UpdateModel.DEFAULT:
        synchronise_default(devs)
    elif update_model == UpdateModel.EAMSGD:
        synchronise_eamsgd(devs, solver.alpha, solver.base_model_momentum, allreduce=allreduce)
    elif update_model == UpdateModel.POLYAK_RUPPERT:
        synchronise_polyak_ruppert(devs, 0.0, allreduce=allreduce, world=world)
    else:
        raise NotImplementedError(f"error: {update_model} is not supported (stub in the reference as well)")
    for d in devs:
        for r in d.replicas:
            r.updates = 0
