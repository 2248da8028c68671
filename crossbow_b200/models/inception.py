"""Inception-v3 (Inceptionv3.java:32-108 unit / pool helpers, :110-500 blocks 7A-7E, :502-640 network) and GoogLeNet v1 of the
convnet-benchmarks suite (convnet/benchmarks/ModelBuilder.java:611-764 unit, :766-960 network).

Every Inception-v3 convolution is Conv (no bias, Gaussian 0.1) -> BatchNorm -> ReLU; GoogLeNet's are Conv -> ReLU.  The towers
of a block read the same tensor and meet in a channel Concat; gradients of the towers are merged by the graph builder."""
from ..types import InitialiserType, PoolMethod
from ._builder import Net
from ..conf import InitialiserConf


def _gauss():
    return InitialiserConf().setType(InitialiserType.GAUSSIAN).setStd(0.1)


def _unit(n, x, name, outputs, k=1, stride=1, pad=0):
    """Conv -> BatchNorm -> ReLU on `x`; kernel / stride / padding as one number or (height, width)."""
    n.conv(f"{name}-Conv", outputs, k, stride, pad, bias=False, inputs=[x] if x is not None else None, winit=_gauss())
    n.bn(f"{name}-BatchNorm")
    return n.relu(f"{name}-ReLU")


def _pool(n, x, name, method, k, stride, pad):
    return n.pool(f"{name}-Pool", method, k, stride, pad, inputs=[x])


def _block_a(n, x, p, t1, t3a, t3b, t3c, t2a, t2b, pool, t4):
    a = _unit(n, x, f"{p}-tower-1(a)-1x1", t1)
    b = _unit(n, _unit(n, x, f"{p}-tower-2(a)-1x1", t2a), f"{p}-tower-2(b)-5x5", t2b, 5, 1, 2)
    c = _unit(n, x, f"{p}-tower-3(a)-1x1", t3a)
    c = _unit(n, c, f"{p}-tower-3(b)-3x3", t3b, 3, 1, 1)
    c = _unit(n, c, f"{p}-tower-3(c)-3x3", t3c, 3, 1, 1)
    d = _unit(n, _pool(n, x, f"{p}-tower-4(a)-3x3", pool, 3, 1, 1), f"{p}-tower-4(b)-1x1", t4)
    return n.concat(f"{p}-Concat", [a, b, c, d])


def _block_b(n, x, p, t1, t2a, t2b, t2c, pool):
    a = _unit(n, x, f"{p}-tower-1(a)-3x3", t1, 3, 2, 0)
    b = _unit(n, x, f"{p}-tower-2(a)-1x1", t2a)
    b = _unit(n, b, f"{p}-tower-2(b)-3x3", t2b, 3, 1, 1)
    b = _unit(n, b, f"{p}-tower-2(c)-3x3", t2c, 3, 2, 0)
    c = _pool(n, x, f"{p}-tower-3(a)-3x3", pool, 3, 2, 0)
    return n.concat(f"{p}-Concat", [a, b, c])


def _block_c(n, x, p, t1, t2a, t2b, t2c, t3a, t3b, t3c, t3d, t3e, pool, t4):
    # "1x7" is one column wide and seven rows high (kernel {width, height} in the reference's unit helper)
    a = _unit(n, x, f"{p}-tower-1(a)-1x1", t1)
    b = _unit(n, x, f"{p}-tower-2(a)-1x1", t2a)
    b = _unit(n, b, f"{p}-tower-2(b)-1x7", t2b, (7, 1), 1, (3, 0))
    b = _unit(n, b, f"{p}-tower-2(c)-7x1", t2c, (1, 7), 1, (0, 3))
    c = _unit(n, x, f"{p}-tower-3(a)-1x1", t3a)
    c = _unit(n, c, f"{p}-tower-3(b)-7x1", t3b, (1, 7), 1, (0, 3))
    c = _unit(n, c, f"{p}-tower-3(c)-1x7", t3c, (7, 1), 1, (3, 0))
    c = _unit(n, c, f"{p}-tower-3(d)-7x1", t3d, (1, 7), 1, (0, 3))
    c = _unit(n, c, f"{p}-tower-3(e)-1x7", t3e, (7, 1), 1, (3, 0))
    d = _unit(n, _pool(n, x, f"{p}-tower-4(a)-3x3", pool, 3, 1, 1), f"{p}-tower-4(b)-1x1", t4)
    return n.concat(f"{p}-Concat", [a, b, c, d])


def _block_d(n, x, p, t1a, t1b, t2a, t2b, t2c, t2d, pool):
    a = _unit(n, _unit(n, x, f"{p}-tower-1(a)-1x1", t1a), f"{p}-tower-1(b)-3x3", t1b, 3, 2, 0)
    b = _unit(n, x, f"{p}-tower-2(a)-1x1", t2a)
    b = _unit(n, b, f"{p}-tower-2(b)-1x7", t2b, (7, 1), 1, (3, 0))
    b = _unit(n, b, f"{p}-tower-2(c)-7x1", t2c, (1, 7), 1, (0, 3))
    b = _unit(n, b, f"{p}-tower-2(d)-3x3", t2d, 3, 2, 0)
    c = _pool(n, x, f"{p}-tower-3(a)-3x3", pool, 3, 2, 0)
    return n.concat(f"{p}-Concat", [a, b, c])


def _block_e(n, x, p, t1, t2a, t2b, t2c, t3a, t3b, t3c, t3d, pool, t4):
    a = _unit(n, x, f"{p}-tower-1(a)-1x1", t1)
    b0 = _unit(n, x, f"{p}-tower-2(a)-1x1", t2a)
    b1 = _unit(n, b0, f"{p}-tower-2(b)-1x3", t2b, (3, 1), 1, (1, 0))
    b2 = _unit(n, b0, f"{p}-tower-2(c)-3x1", t2c, (1, 3), 1, (0, 1))
    c0 = _unit(n, _unit(n, x, f"{p}-tower-3(a)-1x1", t3a), f"{p}-tower-3(b)-3x3", t3b, 3, 1, 1)
    c1 = _unit(n, c0, f"{p}-tower-3(c)-1x3", t3c, (3, 1), 1, (1, 0))
    c2 = _unit(n, c0, f"{p}-tower-3(d)-3x1", t3d, (1, 3), 1, (0, 1))
    d = _unit(n, _pool(n, x, f"{p}-tower-4(a)-3x3", pool, 3, 1, 1), f"{p}-tower-4(b)-1x1", t4)
    return n.concat(f"{p}-Concat", [a, b1, b2, c1, c2, d])


def inception_v3(solver_conf=None, classes=1000, size=299, width=1.0):
    """Inception-v3 for `size` x `size` inputs (299 in the reference).  `width` scales every channel count (tests use a
    narrow network on small images; sizes from 75 keep every stage at least one pixel wide)."""
    w = lambda c: max(4, int(round(c * width / 4)) * 4)
    AVG, MAX = PoolMethod.AVERAGE, PoolMethod.MAX
    n = Net(InitialiserType.GAUSSIAN)
    x = _unit(n, None, "stage-1-unit-1", w(32), 3, 2, 0)
    x = _unit(n, x, "stage-1-unit-2", w(32), 3, 1, 0)
    x = _unit(n, x, "stage-1-unit-3", w(64), 3, 1, 1)
    x = _pool(n, x, "stage-1", MAX, 3, 2, 0)
    x = _unit(n, x, "stage-2-unit-1", w(80), 1, 1, 0)
    x = _unit(n, x, "stage-2-unit-2", w(192), 3, 1, 0)
    x = _pool(n, x, "stage-2", MAX, 3, 2, 0)
    for i, t4 in enumerate((32, 64, 64)):
        x = _block_a(n, x, f"stage-3-7A-{i + 1}", w(64), w(64), w(96), w(96), w(48), w(64), AVG, w(t4))
    x = _block_b(n, x, "stage-3-7B-1", w(384), w(64), w(96), w(96), MAX)
    for i, (m, pool) in enumerate(((128, MAX), (160, AVG), (160, AVG), (192, AVG))):
        x = _block_c(n, x, f"stage-4-7C-{i + 1}", w(192), w(m), w(m), w(192), w(m), w(m), w(m), w(m), w(192), pool, w(192))
    x = _block_d(n, x, "stage-4-7D-1", w(192), w(320), w(192), w(192), w(192), w(192), MAX)
    for i, pool in enumerate((AVG, MAX)):
        x = _block_e(n, x, f"stage-5-7E-{i + 1}", w(320), w(384), w(384), w(384), w(448), w(384), w(384), w(384), pool, w(192))
    n.pool("Wrap-up-Pool", AVG, 1, 1, 0, inputs=[x], global_pooling=True)
    n.fc("InnerProduct", classes, winit=_gauss())
    n.classifier_tail()
    return n.finish("inception-v3", [3, size, size], classes, solver_conf)


def _g_unit(n, x, p, cfg):
    """GoogLeNet unit: 1x1 | 1x1 -> 3x3 | 1x1 -> 5x5 | max-pool 3x3 -> 1x1, every convolution followed by ReLU."""
    def cr(src, name, outputs, k=1, pad=0):
        n.conv(f"{p}-{name}", outputs, k, 1, pad, bias=False, inputs=[src], winit=_gauss())
        return n.relu(f"{p}-{name}-ReLU")
    a = cr(x, "tower-1-1x1", cfg[0][0])
    b = cr(cr(x, "tower-2-1x1", cfg[1][0]), "tower-2-3x3", cfg[1][1], 3, 1)
    c = cr(cr(x, "tower-3-1x1", cfg[2][0]), "tower-3-5x5", cfg[2][1], 5, 2)
    d = cr(n.pool(f"{p}-tower-4-Pool", PoolMethod.MAX, cfg[3][0], 1, 1, inputs=[x]), "tower-4-1x1", cfg[3][1])
    return n.concat(f"{p}-Concat", [a, b, c, d])


def googlenet_v1(solver_conf=None, classes=1000, size=224, width=1.0):
    """GoogLeNet v1 of the convnet-benchmarks suite (no auxiliary classifiers, no LRN, as in the reference's builder)."""
    w = lambda c: max(4, int(round(c * width / 4)) * 4)
    MAX = PoolMethod.MAX
    n = Net(InitialiserType.GAUSSIAN)
    n.conv("Conv-1", w(64), 7, 2, 3, bias=False, winit=_gauss())
    n.relu("ReLU-1")
    n.pool("Pool-1", MAX, 3, 2, 1)
    n.conv("Conv-2", w(64), 1, 1, 0, bias=False, winit=_gauss())
    n.relu("ReLU-2")
    n.conv("Conv-3", w(192), 3, 1, 1, bias=False, winit=_gauss())
    n.relu("ReLU-3")
    x = n.pool("Pool-3", MAX, 3, 2, 1)
    sc = lambda cfg: [[w(v) for v in cfg[0]], [w(v) for v in cfg[1]], [w(v) for v in cfg[2]], [cfg[3][0], w(cfg[3][1])]]
    for name, cfg in (("Stage-3 (a)", [[64], [96, 128], [16, 32], [3, 32]]), ("Stage-3 (b)", [[128], [128, 192], [32, 96], [3, 64]])):
        x = _g_unit(n, x, name, sc(cfg))
    x = n.pool("Pool-4", MAX, 3, 2, 1, inputs=[x])
    for name, cfg in (("Stage-4 (a)", [[192], [96, 208], [16, 48], [3, 64]]), ("Stage-4 (b)", [[160], [112, 224], [24, 64], [3, 64]]),
                      ("Stage-4 (c)", [[128], [128, 256], [24, 64], [3, 64]]), ("Stage-4 (d)", [[112], [144, 288], [32, 64], [3, 64]]),
                      ("Stage-4 (e)", [[256], [160, 320], [32, 128], [3, 128]])):
        x = _g_unit(n, x, name, sc(cfg))
    x = n.pool("Pool-5", MAX, 3, 2, 1, inputs=[x])
    for name, cfg in (("Stage-5 (a)", [[256], [160, 320], [32, 128], [3, 128]]), ("Stage-5 (b)", [[384], [192, 384], [48, 128], [3, 128]])):
        x = _g_unit(n, x, name, sc(cfg))
    n.pool("Pool-6", PoolMethod.AVERAGE, 1, 1, 0, inputs=[x], global_pooling=True)
    n.fc("InnerProduct", classes, winit=_gauss())
    n.classifier_tail()
    return n.finish("googlenet-v1", [3, size, size], classes, solver_conf)
