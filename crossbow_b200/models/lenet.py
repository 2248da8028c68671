"""LeNet. Two variants:

* ``lenet()``       - the application in the reference (LeNet.java:118-238): conv5x5x32 - ReLU - maxpool2 -
  conv5x5x64 - ReLU - maxpool2 - FC1024 - ReLU - dropout 0.4 - FC10 - softmax - loss/accuracy;
* ``lenet_caffe()`` - the classic 20/50/500 network named by the CPU/SMA baseline configuration:
  conv5x5x20 - maxpool2 - conv5x5x50 - maxpool2 - FC500 - ReLU - FC10 - softmax loss.
"""
from ..conf import InitialiserConf
from ..types import InitialiserType, PoolMethod
from ._builder import Net


def _g(std=0.1):
    return InitialiserConf().setType(InitialiserType.GAUSSIAN).setStd(std).truncate(True)


def _c(v):
    return InitialiserConf().setType(InitialiserType.CONSTANT).setValue(v)


def lenet(solver_conf=None, channels=1, size=28, classes=10):
    n = Net()
    n.conv("Conv", 32, 5, bias=True, winit=_g(), binit=_c(0.0))
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.conv("Conv", 64, 5, bias=True, winit=_g(), binit=_c(0.1))
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.fc("InnerProduct", 1024, winit=_g(), binit=_c(0.1))
    n.relu("ReLU")
    n.dropout("Dropout", 0.4)
    n.fc("InnerProduct", classes, winit=_g(), binit=_c(0.1))
    n.classifier_tail()
    return n.finish("lenet", [channels, size, size], classes, solver_conf)


def lenet_caffe(solver_conf=None, channels=1, size=28, classes=10):
    n = Net()
    n.conv("Conv", 20, 5, bias=True, binit=_c(0.0))
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.conv("Conv", 50, 5, bias=True, binit=_c(0.0))
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.fc("InnerProduct", 500)
    n.relu("ReLU")
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("lenet-caffe", [channels, size, size], classes, solver_conf)
