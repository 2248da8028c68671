"""Shared helpers: build a model + engines with identical initial weights and data."""
import numpy as np
import torch

from crossbow_b200 import Dataflow, Model, ModelConf, Phase, Shape, SolverConf, SystemConf, UpdateModel
from crossbow_b200.models import build


def make_solver(lr=0.05, momentum=0.9, wd=1e-4, alpha=0.1):
    return SolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(lr).setMomentum(momentum) \
        .setWeightDecay(wd).setAlpha(alpha)


def build_model(name, batch, solver=None, **kw):
    solver = solver or make_solver()
    spec = build(name, solver_conf=solver, **kw)
    m = Model()
    ishape = Shape([batch] + spec.input_shape)
    nid = spec.train.init(ishape, Shape([batch]), m)
    m.finalise()
    if spec.test is not None:
        spec.test.init(ishape, Shape([batch]), m, nid)
    return spec, m, solver


def make_batches(spec, batch, n, seed=0):
    g = np.random.default_rng(seed)
    xs = [torch.from_numpy(g.standard_normal((batch, *spec.input_shape), dtype=np.float32)) for _ in range(n)]
    ys = [torch.from_numpy(g.integers(0, spec.classes, size=batch, dtype=np.int32)) for _ in range(n)]
    return xs, ys


def engines(name, batch, k=1, update_model=UpdateModel.SMA, wpc=None, solver=None, use_graphs=True, use_tc=False, seed=7, splits=1, reuse_memory=False,
            gradient_buckets=0, **kw):
    from crossbow_b200.engine import CpuEngine, GpuEngine
    spec, m, solver = build_model(name, batch, solver, **kw)
    init = m.initial_values(seed)
    wpc = wpc or k
    gpu = GpuEngine(spec.train, spec.test, m, init, batch, spec.input_shape, solver, update_model, replicas=k, wpc=wpc,
                    use_graphs=use_graphs, use_tc=use_tc, seed=seed, splits=splits, reuse_memory=reuse_memory,
                    gradient_buckets=gradient_buckets)
    import copy
    cpu = CpuEngine(spec.train, spec.test, m, init, batch, spec.input_shape, copy.deepcopy(solver), update_model, replicas=k, wpc=wpc, seed=seed,
                    splits=splits)
    return spec, m, gpu, cpu


def tiny_vgg(solver_conf=None):
    """Conv-ReLU-BN-Dropout blocks + FC-ReLU-BN-Dropout head: every fused pattern of VGG-16 on a well-conditioned size."""
    from crossbow_b200.models._builder import Net
    from crossbow_b200.types import PoolMethod
    n = Net()
    for item in ((16, 0.3), (16, None), "M", (32, 0.4), (32, None), "M"):
        if item == "M":
            n.pool("Pool", PoolMethod.MAX, 2, 2)
            continue
        feat, drop = item
        n.conv("Conv", feat, 3, 1, 1, bias=True)
        n.relu("ReLU")
        n.bn("BatchNorm")
        if drop:
            n.dropout("Dropout", drop)
    n.dropout("Dropout", 0.5)
    n.fc("InnerProduct", 64)
    n.relu("ReLU")
    n.bn("BatchNorm")
    n.dropout("Dropout", 0.5)
    n.fc("InnerProduct", 10)
    n.classifier_tail()
    return n.finish("tiny-vgg", [3, 16, 16], 10, solver_conf)


def tiny_bottleneck(solver_conf=None):
    """Two bottleneck units (identity-free: both have projection shortcuts, one strided)."""
    from crossbow_b200.models._builder import Net
    from crossbow_b200.models.resnet import _bottleneck
    from crossbow_b200.types import PoolMethod
    n = Net()
    n.conv("Conv", 16, 3, 1, 1)
    n.bn("BatchNorm")
    x = n.relu("ReLU")
    x = _bottleneck(n, x, "u1", 16, 8, 1)
    x = _bottleneck(n, x, "u2", 32, 8, 1)
    x = _bottleneck(n, x, "u3", 32, 16, 2)
    n.pool("Pool", PoolMethod.AVERAGE, 1, 1, global_pooling=True)
    n.fc("InnerProduct", 10)
    n.classifier_tail()
    return n.finish("tiny-bottleneck", [3, 16, 16], 10, solver_conf)


from crossbow_b200.models import REGISTRY as _REG
_REG.setdefault("tiny-vgg", tiny_vgg)
_REG.setdefault("tiny-bottleneck", tiny_bottleneck)
