"""Every fused launch group of a lowered model against the fp32 CPU definition of the operators it contains.

Deep networks trained at tiny batch sizes amplify rounding differences by several orders of magnitude from layer to
layer (batch-norm over a handful of rows, saturated soft-max), so comparing end-to-end weights says little about a
kernel.  Here the device runs one whole task (forward + backward, optimiser excluded); then, for every tensor the
device materialises, the CPU recomputes it from the DEVICE's own inputs of that group (forward), and recomputes every
gradient from the device's upstream gradients (backward).  Errors therefore never compound across groups, and the
test works for any model at any size.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from crossbow_b200 import Phase, UpdateModel
from crossbow_b200.kernels import OpEnv
from helpers import build_model, make_batches

pytestmark = pytest.mark.gpu


def nchw(t):
    """Device tensor (channels-last) -> CPU tensor in the operator API's layout."""
    x = t.nhwc().detach().cpu()
    return x.permute(0, 3, 1, 2).contiguous()


def grad_nchw(t):
    return t.grad[: t.numel].view(t.n, t.h, t.w, t.c).detach().cpu().permute(0, 3, 1, 2).contiguous()


def check_model(name, batch, use_tc, tol_f=2e-4, tol_b=1e-3, **kw):
    from crossbow_b200.engine import GpuEngine, task_params
    from crossbow_b200.ops import lib as L
    spec, m, solver = build_model(name, batch, **kw)
    init = m.initial_values(3)
    gpu = GpuEngine(spec.train, None, m, init, batch, spec.input_shape, solver, UpdateModel.SMA, replicas=1, wpc=1,
                    use_graphs=False, use_tc=use_tc, seed=11)
    try:
        lib = gpu.lib
        ln = gpu.learners[0]
        low = ln.low_train
        xs, ys = make_batches(spec, batch, 1, seed=5)
        ex, lab = ln.staging(Phase.TRAIN)
        ex.copy_(xs[0].reshape(-1).cuda())
        lab.copy_(ys[0].cuda())
        p = task_params(solver, 4, 11, True)
        lib.xb_learner_params(ln.handle)[0] = p
        nops = lib.xb_program_num_ops(ln.prog_train)
        last = nops - 1 - int(solver.clip_gradient_threshold >= 0)      # stop before the optimiser
        L.check(lib.xb_program_run_range(ln.prog_train, 0, last, ln.stream), "run")
        torch.cuda.synchronize()
        assert int(gpu.tc_status[0]) == 0

        w = torch.from_numpy(init)
        g_dev = torch.from_numpy(m.to_canonical(ln.rep.g.cpu().numpy()))
        env = OpEnv(Phase.TRAIN, ys[0], 4, 11, {})
        info = low.node_info
        fwd = low.fwd
        groups = []          # (value_node, members)
        # group = maximal set of nodes that end in one materialised tensor
        owner = {}
        for n in fwd:
            t = low.tensors.get(id(n))
            i = info[id(n)]
            if t is None:
                continue
            if i["fused_into"] is not None:
                continue
            value = i["relu"] if i["relu"] is not None else n
            owner[id(value)] = (n, t)
        materialised = {vid: t for vid, (_, t) in owner.items()}
        node_by_id = {id(n): n for n in fwd}

        def inputs_of(n):
            return [p for p in n.prev if not p.op.kernel.is_gradient]

        # ---- forward: recompute each group from the device's inputs ----
        worst_f = 0.0
        params_cache = {}

        def params_for(k, requires_grad=False):
            return [w[v.offset:v.offset + v.elements()].reshape(v.shape.dims).clone().requires_grad_(requires_grad) for v in k.variables]

        def eval_node(n, leaves, stop_at, rg):
            """CPU value of node n; tensors of other groups are leaves taken from the device."""
            if id(n) in stop_at and id(n) in materialised:
                if id(n) not in leaves:
                    leaves[id(n)] = nchw(materialised[id(n)]).requires_grad_(rg)
                return leaves[id(n)]
            ins = inputs_of(n)
            if not ins:
                xin = [leaves.setdefault("input", xs[0].clone())]
            else:
                xin = [eval_node(p, leaves, stop_at, rg) for p in ins]
            k = n.op.kernel
            if id(n) not in params_cache or rg:
                params_cache[id(n)] = params_for(k, rg)
            return k.forward(xin, params_cache[id(n)], env)

        all_values = set(materialised)
        for vid, (head, t) in owner.items():
            v = node_by_id[vid]
            if v.op.kernel.kind in ("softmaxloss", "accuracy"):
                continue
            leaves = {}
            with torch.no_grad():
                ref = eval_node(v, leaves, all_values - {vid}, False)
            dev = nchw(t).reshape(ref.shape)
            err = float((dev - ref).abs().max()) / (float(ref.abs().max()) + 1e-6)
            worst_f = max(worst_f, err)
            assert err < tol_f, f"{name}: forward of group ending in {v.op} off by {err:.3e}"

        # ---- backward: per group, VJP of the device's upstream gradient ----
        expected_dx = {}      # id(value node) -> accumulated expected gradient
        expected_dw = torch.zeros_like(w)
        for vid, (head, t) in owner.items():
            v = node_by_id[vid]
            if v.op.kernel.kind in ("softmaxloss", "accuracy", "datatransform") or t.grad is None or not t.grad_written:
                continue
            if v.op.kernel.kind == "softmax":
                continue
            leaves = {}
            params_cache.clear()
            # a ReLU folded into a GEMM epilogue: the device has already masked this group's upstream gradient in
            # place with ITS OWN output sign, so differentiate the GEMM alone (a CPU-side mask could differ by
            # rounding for pre-activations that are almost zero)
            relu_fused = info[id(head)]["relu"] is not None
            target = head if relu_fused else v
            with torch.enable_grad():
                out = eval_node(target, leaves, all_values - {vid}, True)
            gy = grad_nchw(t).reshape(out.shape)
            if relu_fused and head.op.kernel.kind not in ("conv", "innerproduct"):
                # normalisation (+ residual sum) + ReLU in one kernel: apply the DEVICE's mask to the upstream gradient and
                # differentiate the part in front of the ReLU, for the same reason (an output within rounding of zero
                # would otherwise flip one element of the reference now and then)
                gy = gy * (nchw(t).reshape(out.shape) > 0)
            leaf_items = [(k, x) for k, x in leaves.items() if k != "input" and x.requires_grad]
            group_params = [(nid, ps) for nid, ps in params_cache.items()]
            wrt = [x for _, x in leaf_items] + [p_ for _, ps in group_params for p_ in ps]
            if not wrt:
                continue
            grads = torch.autograd.grad(out, wrt, gy, allow_unused=True)
            gi = 0
            for k, x in leaf_items:
                if grads[gi] is not None:
                    expected_dx[k] = expected_dx.get(k, 0) + grads[gi]
                gi += 1
            for nid, ps in group_params:
                for var, p_ in zip(node_by_id[nid].op.kernel.variables, ps):
                    if grads[gi] is not None:
                        expected_dw[var.offset:var.offset + var.elements()] += grads[gi].reshape(-1)
                    gi += 1
        # the loss group: d logits = (p - onehot)/N on the device's probabilities
        worst_b = 0.0
        for vid, ref in expected_dx.items():
            t = materialised[vid]
            if t.grad is None or not t.needs_grad:
                continue
            dev = grad_nchw(t).reshape(ref.shape)
            head = owner[vid][0]
            if head.op.kernel.kind in ("conv", "innerproduct") and info[id(head)]["relu"] is not None:
                # the GEMM epilogue applied the ReLU, and the backward pass masks this gradient buffer in place
                ref = ref * (nchw(t).reshape(ref.shape) > 0)
            err = float((dev - ref).abs().max()) / (float(ref.abs().max()) + 1e-9)
            worst_b = max(worst_b, err)
            if err >= tol_b:          # say where: which images / channels / how many elements
                bad = ((dev - ref).abs() > tol_b * float(ref.abs().max())).nonzero()
                where = {d: sorted(set(bad[:, d].tolist()))[:12] for d in range(bad.shape[1])}
                i0 = tuple(bad[0].tolist())
                raise AssertionError(f"{name}: gradient w.r.t. output of {node_by_id[vid].op} off by {err:.3e}; {bad.shape[0]} of {dev.numel()} "
                                     f"elements, index sets per dim {where}, first {i0}: dev {float(dev[i0]):.4e} ref {float(ref[i0]):.4e}")
        for var in m.variables:
            s = slice(var.offset, var.offset + var.elements())
            ref, dev = expected_dw[s], g_dev[s]
            if float(ref.abs().max()) == 0.0:
                continue
            err = float((dev - ref).abs().max()) / float(ref.abs().max())
            worst_b = max(worst_b, err)
            assert err < tol_b, f"{name}: parameter gradient of {var.name} (op {var.op_id}) off by {err:.3e}"
        # soft-max / loss head
        probs = low.probs.buf[: low.probs.numel].view(batch, -1).cpu()
        logits = low.logits.buf[: low.logits.numel].view(batch, -1).cpu()
        assert torch.allclose(probs, torch.softmax(logits, 1), atol=1e-5)
        onehot = torch.nn.functional.one_hot(ys[0].long(), probs.shape[1]).float()
        dl = low.logits.grad[: low.logits.numel].view(batch, -1).cpu()
        assert torch.allclose(dl, (probs - onehot) / batch, atol=1e-6)
        return worst_f, worst_b
    finally:
        gpu.destroy()


CASES = [
    ("lenet", 8, {}),
    ("tiny-vgg", 16, {}),
    ("vgg16", 4, {}),
    ("resnet20", 4, dict(transform=True)),
    ("resnet32", 8, {}),
    ("resnet50", 2, dict(size=64, classes=10)),
    ("mini-inception", 4, {}),
    ("alexnet", 2, dict(size=96, classes=10)),
    ("inception-v3", 2, dict(size=139, width=0.25, classes=10)),        # rectangular 1x7 / 7x1 / 1x3 / 3x1 filters, six-way concat
    ("googlenet", 2, dict(size=64, width=0.5, classes=10)),
]


@pytest.mark.parametrize("name,batch,kw", CASES)
def test_groups_cuda_cores(name, batch, kw):
    check_model(name, batch, use_tc=False, **kw)


@pytest.mark.parametrize("name,batch,kw", CASES)
def test_groups_tensor_cores(name, batch, kw):
    # tf32 operands: 10-bit mantissa, errors ~1e-3 relative to the tensor's scale
    check_model(name, batch, use_tc=True, tol_f=5e-3, tol_b=1e-2, **kw)
