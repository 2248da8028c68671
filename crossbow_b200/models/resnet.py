"""The ResNet v1 family.

CIFAR variants (ResNet-20/32/44/56/110: 3 stages x n basic blocks, 16/32/64 channels) follow
ResNetv1ForCifar.java:633-795; ImageNet variants (ResNet-18/34/50/101/152, basic or bottleneck blocks
[..], 64-2048 channels, 1x1 projection shortcuts with batch-norm) follow ResNetv1.java:81-432,489-693.
Convolutions have no bias, Xavier initialisation, batch-norm epsilon 1e-5 and moving-average fraction 0.9.
"""
from ..types import PoolMethod
from ._builder import Net

_IMAGENET = {18: ([2, 2, 2, 2], False), 34: ([3, 4, 6, 3], False), 50: ([3, 4, 6, 3], True),
             101: ([3, 4, 23, 3], True), 152: ([3, 8, 36, 3], True)}


def _shortcut(n: Net, x, prefix, cin, cout, stride):
    if cin == cout and stride == 1:
        return x
    c = n.conv(f"{prefix}-Conv (shortcut)", cout, 1, stride, 0, inputs=[x])
    return n.bn(f"{prefix}-BatchNorm (shortcut)", inputs=[c])


def _basic(n: Net, x, prefix, cin, cout, stride):
    a = n.conv(f"{prefix}-Conv (a)", cout, 3, stride, 1, inputs=[x])
    a = n.bn(f"{prefix}-BatchNorm (a)")
    a = n.relu(f"{prefix}-ReLU (a)")
    b = n.conv(f"{prefix}-Conv (b)", cout, 3, 1, 1)
    b = n.bn(f"{prefix}-BatchNorm (b)")
    s = _shortcut(n, x, prefix, cin, cout, stride)
    y = n.sum(f"{prefix}-Sum", [b, s])
    return n.relu(f"{prefix}-ReLU (b)")


def _bottleneck(n: Net, x, prefix, cin, mid, stride):
    cout = 4 * mid
    a = n.conv(f"{prefix}-Conv (a)", mid, 1, stride, 0, inputs=[x])
    n.bn(f"{prefix}-BatchNorm (a)")
    n.relu(f"{prefix}-ReLU (a)")
    n.conv(f"{prefix}-Conv (b)", mid, 3, 1, 1)
    n.bn(f"{prefix}-BatchNorm (b)")
    n.relu(f"{prefix}-ReLU (b)")
    n.conv(f"{prefix}-Conv (c)", cout, 1, 1, 0)
    c = n.bn(f"{prefix}-BatchNorm (c)")
    s = _shortcut(n, x, prefix, cin, cout, stride)
    n.sum(f"{prefix}-Sum", [c, s])
    return n.relu(f"{prefix}-ReLU (c)")


def resnet_cifar(layers=32, solver_conf=None, classes=10, transform=False, reference_pool=False, size=32):
    """ResNet-(6n+2) for 3x32x32 inputs.  ``reference_pool`` keeps the application's 7x7 stride-1 average pool
    (2x2 output) instead of a global one; ``transform`` prepends the crop-32 + mirror DataTransform."""
    if (layers - 2) % 6 != 0:
        raise ValueError("error: CIFAR ResNet depth must be 6n+2")
    blocks = (layers - 2) // 6
    n = Net()
    if transform:
        n.transform(crop=size, mirror=True)
    n.conv("Conv", 16, 3, 1, 1)
    n.bn("BatchNorm")
    x = n.relu("ReLU")
    cin = 16
    for stage, feat in enumerate((16, 32, 64), 1):
        for unit in range(1, blocks + 1):
            stride = 2 if (unit == 1 and stage != 1) else 1
            x = _basic(n, x, f"stage-{stage}-unit-{unit}", cin, feat, stride)
            cin = feat
    if reference_pool:
        n.pool("Pool", PoolMethod.AVERAGE, 7, 1)
    else:
        n.pool("Pool", PoolMethod.AVERAGE, 1, 1, global_pooling=True)
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish(f"resnet-{layers}", [3, size, size], classes, solver_conf)


def resnet_imagenet(layers=50, solver_conf=None, classes=1000, size=224):
    if layers not in _IMAGENET:
        raise ValueError(f"error: unsupported ResNet depth {layers}")
    units, bottleneck = _IMAGENET[layers]
    n = Net()
    # 7x7/2; the reference drops the padding for TensorFlow parity, which needs 230x230 inputs - keep pad 3
    n.conv("Conv", 64, 7, 2, 3)
    n.bn("BatchNorm")
    n.relu("ReLU")
    x = n.pool("Pool", PoolMethod.MAX, 3, 2, 0)   # ceil-mode extent: 112 -> 56, as in the reference (ResNetv1.java:548-556)
    cin = 64
    for stage, (feat, count) in enumerate(zip((64, 128, 256, 512), units), 1):
        for unit in range(1, count + 1):
            stride = 2 if (unit == 1 and stage != 1) else 1
            prefix = f"stage-{stage}-unit-{unit}"
            if bottleneck:
                x = _bottleneck(n, x, prefix, cin, feat, stride)
                cin = 4 * feat
            else:
                x = _basic(n, x, prefix, cin, feat, stride)
                cin = feat
    n.pool("Pool", PoolMethod.AVERAGE, 1, 1, global_pooling=True)
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish(f"resnet-{layers}", [3, size, size], classes, solver_conf)
