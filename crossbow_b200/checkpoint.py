"""Checkpoint store / load in the reference's on-disk layout.

``<dir>/<%06d version>/gpu-<dd>-theModel-data.dat`` (+ ``-last.dat`` momentum), ``gpu-<dd>-replica-<ddd>-data.dat``
(+ ``-last.dat``), ``gpu-<dd>-bn-avg-<ddd>.dat`` / ``gpu-<dd>-bn-var-<ddd>.dat`` per batch-norm operator id: raw
little-endian fp32, no header, variables in operator-id order with weights before bias
(clib-multigpu/executioncontext.c:2340-2367, modelmanager.c:267-343, model.c:396-405, cudnnbatchnormparams.c:102-143).
Files always hold the canonical (reference) element order, whatever the device layout is.
Replica files carry the reference's job-wide replica id: replicas are dealt round-robin over the devices
(modelmanager.c:51-62), so the j-th replica of device d on G devices is replica j * G + d.
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch


def _write(path, arr):
    np.asarray(arr, dtype="<f4").tofile(path)


def _read(path, n):
    a = np.fromfile(path, dtype="<f4")
    if a.size != n:
        raise ValueError(f"error: checkpoint file {path} has {a.size} values, expected {n}")
    return a


def _replica_id(j: int, dev: int, devices: int) -> int:
    return j * max(1, devices) + dev


def _bn_ops(ctx):
    g = ctx.dataflows[0].executable()
    return [n.op for n in g.order if n.op.kernel.kind == "batchnorm"]


def save_checkpoint(ctx, directory: str) -> str:
    if not directory:
        raise ValueError("error: checkpoint directory is not set")
    ctx._checkpoint_version += 1
    d = os.path.join(directory, f"{ctx._checkpoint_version:06d}")
    os.makedirs(d, exist_ok=True)
    e, dev = ctx.engine, ctx.rank
    gpu = hasattr(e, "shared")
    e.finish()                       # the last synchronisation may still be updating the central model on its own stream
    _write(os.path.join(d, f"gpu-{dev:02d}-theModel-data.dat"), e.central_model())
    if gpu:
        m = ctx.model
        _write(os.path.join(d, f"gpu-{dev:02d}-theModel-last.dat"), m.to_canonical(e.central_momentum().cpu().numpy()))
        for i, l in enumerate(e.learners):
            rid = _replica_id(i, dev, ctx.world)
            _write(os.path.join(d, f"gpu-{dev:02d}-replica-{rid:03d}-data.dat"), e.replica_model(i))
            _write(os.path.join(d, f"gpu-{dev:02d}-replica-{rid:03d}-last.dat"), m.to_canonical(l.rep.last.cpu().numpy()))
        for op in _bn_ops(ctx):
            if op.uid in e.shared.run_mean:
                _write(os.path.join(d, f"gpu-{dev:02d}-bn-avg-{op.id:03d}.dat"), e.shared.run_mean[op.uid].cpu().numpy())
                _write(os.path.join(d, f"gpu-{dev:02d}-bn-var-{op.id:03d}.dat"), e.shared.run_var[op.uid].cpu().numpy())
    else:
        for di, dv in enumerate(e.devs):
            _write(os.path.join(d, f"gpu-{di:02d}-theModel-last.dat"), dv.z_last.numpy())
            for i, r in enumerate(dv.replicas):
                rid = _replica_id(i, di, len(e.devs))
                _write(os.path.join(d, f"gpu-{di:02d}-replica-{rid:03d}-data.dat"), r.w.numpy())
                _write(os.path.join(d, f"gpu-{di:02d}-replica-{rid:03d}-last.dat"), r.last.numpy())
            for op in _bn_ops(ctx):
                st = dv.op_state.get(("bn", op.uid))
                if st:
                    _write(os.path.join(d, f"gpu-{di:02d}-bn-avg-{op.id:03d}.dat"), st["mean"].numpy())
                    _write(os.path.join(d, f"gpu-{di:02d}-bn-var-{op.id:03d}.dat"), st["var"].numpy())
    return d


def latest_version(directory: str) -> Optional[str]:
    vs = sorted(x for x in os.listdir(directory) if x.isdigit() and os.path.isdir(os.path.join(directory, x)))
    return os.path.join(directory, vs[-1]) if vs else None


def load_checkpoint(ctx, directory: str):
    """``directory`` is either a version directory or its parent (the newest version is taken)."""
    d = directory
    if not any(f.endswith("theModel-data.dat") for f in os.listdir(d)):
        d = latest_version(directory)
        if d is None:
            raise FileNotFoundError(f"error: no checkpoint under {directory}")
    e, dev, m = ctx.engine, ctx.rank, ctx.model
    n = m.elements
    gpu = hasattr(e, "shared")
    e.load_central(_read(os.path.join(d, f"gpu-{dev:02d}-theModel-data.dat"), n))
    if gpu:
        p = os.path.join(d, f"gpu-{dev:02d}-theModel-last.dat")
        if os.path.exists(p):
            e.shared.zlast.copy_(torch.from_numpy(m.to_device(_read(p, n))))
        for i, l in enumerate(e.learners):
            rid = _replica_id(i, dev, ctx.world)
            p = os.path.join(d, f"gpu-{dev:02d}-replica-{rid:03d}-data.dat")
            if not os.path.exists(p) and not getattr(ctx, "quiet", False):
                # (more replicas than the checkpoint was written with: the extra ones start from the central model)
                print(f"warning: {p} not found; replica {rid} starts from the central model", flush=True)
            src = _read(p, n) if os.path.exists(p) else e.central_model()
            e.load_replica(i, src)
            l.rep.prev.copy_(l.rep.w)
            p = os.path.join(d, f"gpu-{dev:02d}-replica-{rid:03d}-last.dat")
            if os.path.exists(p):
                l.rep.last.copy_(torch.from_numpy(m.to_device(_read(p, n))))
        for op in _bn_ops(ctx):
            pa = os.path.join(d, f"gpu-{dev:02d}-bn-avg-{op.id:03d}.dat")
            if os.path.exists(pa) and op.uid in e.shared.run_mean:
                c = e.shared.run_mean[op.uid].numel()
                e.shared.run_mean[op.uid].copy_(torch.from_numpy(_read(pa, c)))
                e.shared.run_var[op.uid].copy_(torch.from_numpy(_read(os.path.join(d, f"gpu-{dev:02d}-bn-var-{op.id:03d}.dat"), c)))
        torch.cuda.synchronize()
    else:
        for di, dv in enumerate(e.devs):
            dv.z = torch.from_numpy(_read(os.path.join(d, f"gpu-{di:02d}-theModel-data.dat"), n)).clone()
            p = os.path.join(d, f"gpu-{di:02d}-theModel-last.dat")
            if os.path.exists(p):
                dv.z_last = torch.from_numpy(_read(p, n)).clone()
            for i, r in enumerate(dv.replicas):
                rid = _replica_id(i, di, len(e.devs))
                p = os.path.join(d, f"gpu-{di:02d}-replica-{rid:03d}-data.dat")
                r.w = torch.from_numpy(_read(p, n)).clone() if os.path.exists(p) else dv.z.clone()
                r.prev = r.w.clone()
                p = os.path.join(d, f"gpu-{di:02d}-replica-{rid:03d}-last.dat")
                if os.path.exists(p):
                    r.last = torch.from_numpy(_read(p, n)).clone()
            for op in _bn_ops(ctx):
                pa = os.path.join(d, f"gpu-{di:02d}-bn-avg-{op.id:03d}.dat")
                if os.path.exists(pa):
                    mean = torch.from_numpy(np.fromfile(pa, dtype="<f4")).clone()
                    var = torch.from_numpy(np.fromfile(os.path.join(d, f"gpu-{di:02d}-bn-var-{op.id:03d}.dat"), dtype="<f4")).clone()
                    dv.op_state[("bn", op.uid)] = dict(mean=mean, var=var, updates=1)
    return d
