"""VGG-16, CIFAR variant (VGG.java:234-375): 13 conv3x3 layers (64,64,128,128,256x3,512x3,512x3), each
Conv - ReLU - BatchNorm - Dropout(0.3/0.4) with no dropout before a max-pool, five 2x2 max-pools, then
Dropout .5 - FC512 - ReLU - BatchNorm - Dropout .5 - FC10."""
from ..types import PoolMethod
from ._builder import Net

_CFG = [(64, 0.3), (64, None), "M", (128, 0.4), (128, None), "M", (256, 0.4), (256, 0.4), (256, None), "M",
        (512, 0.4), (512, 0.4), (512, None), "M", (512, 0.4), (512, 0.4), (512, None), "M"]


def vgg16_cifar(solver_conf=None, classes=10, size=32):
    n = Net()
    for i, item in enumerate(_CFG):
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
    n.fc("InnerProduct", 512)
    n.relu("ReLU")
    n.bn("BatchNorm")
    n.dropout("Dropout", 0.5)
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("vgg-16", [3, size, size], classes, solver_conf)
