"""Model zoo: builders return a ``ModelSpec`` (training + test sub-graphs)."""
from ._builder import ModelSpec, Net
from .lenet import lenet, lenet_caffe
from .resnet import resnet_cifar, resnet_imagenet
from .vgg import vgg16_cifar
from .inception import googlenet_v1, inception_v3
from .simple import (alexnet_v2, convnet_cifar, lenet_batchnorm, logistic_regression, matrix_factorisation, mini_inception, mlp,
                     overfeat, vgg_a)

REGISTRY = {
    "lenet": lenet, "lenet-caffe": lenet_caffe, "vgg16": vgg16_cifar, "logistic-regression": logistic_regression,
    "mlp": mlp, "convnet": convnet_cifar, "lenet-batchnorm": lenet_batchnorm, "alexnet": alexnet_v2,
    "mini-inception": mini_inception, "overfeat": overfeat, "vgg-a": vgg_a, "matrix-factorisation": matrix_factorisation,
    "inception-v3": inception_v3, "googlenet": googlenet_v1,
    **{f"resnet{d}": (lambda d=d, **kw: resnet_cifar(d, **kw)) for d in (8, 20, 32, 44, 56, 110)},
    **{f"resnet{d}": (lambda d=d, **kw: resnet_imagenet(d, **kw)) for d in (18, 34, 50, 101, 152)},
}


REGISTRY["baby-resnet"] = REGISTRY["resnet8"]          # the reference's BabyResNet.java: one basic block per stage


def build(name: str, **kw) -> ModelSpec:
    import re
    m = re.fullmatch(r"resnet(\d+)", name)
    if name not in REGISTRY and m and (int(m.group(1)) - 2) % 6 == 0 and int(m.group(1)) >= 8:
        return resnet_cifar(int(m.group(1)), **kw)        # any CIFAR depth 6n + 2 (ResNetv1ForCifar.java:952-960)
    if name not in REGISTRY:
        raise ValueError(f"error: unknown model {name}; choose from {sorted(REGISTRY)}")
    return REGISTRY[name](**kw)
