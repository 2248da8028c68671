"""Small applications of the reference: logistic regression (LogisticRegression.java), the dlbench
multi-layer perceptron, BabyResNet / ConvNet-style CIFAR networks, LeNet with batch-norm, AlexNet v2 and a
small Inception-style network that exercises Concat."""
from ..conf import InitialiserConf
from ..types import InitialiserType, PoolMethod
from ._builder import Net


def logistic_regression(solver_conf=None, features=784, classes=10, input_shape=None):
    n = Net()
    n.fc("InnerProduct", classes, winit=InitialiserConf().setType(InitialiserType.GAUSSIAN).setStd(0.1),
         binit=InitialiserConf().setType(InitialiserType.CONSTANT).setValue(1.0))
    n.classifier_tail()
    return n.finish("logistic-regression", input_shape or [features, 1, 1], classes, solver_conf)


def mlp(solver_conf=None, features=784, hidden=(2048, 4096, 1024), classes=10):
    n = Net()
    for h in hidden:
        n.fc("InnerProduct", h)
        n.relu("ReLU")
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("mlp", [features, 1, 1], classes, solver_conf)


def convnet_cifar(solver_conf=None, classes=10):
    n = Net()
    for feat in (32, 64, 128):
        n.conv("Conv", feat, 3, 1, 1, bias=True)
        n.relu("ReLU")
        n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.fc("InnerProduct", 256)
    n.relu("ReLU")
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("convnet", [3, 32, 32], classes, solver_conf)


def lenet_batchnorm(solver_conf=None, classes=10):
    n = Net()
    n.conv("Conv", 32, 5, bias=False)
    n.bn("BatchNorm")
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.conv("Conv", 64, 5, bias=False)
    n.bn("BatchNorm")
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.fc("InnerProduct", 1024)
    n.relu("ReLU")
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("lenet-batchnorm", [1, 28, 28], classes, solver_conf)


def alexnet_v2(solver_conf=None, classes=1000, size=224):
    n = Net()
    n.conv("Conv", 64, 11, 4, 2, bias=True)
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 3, 2)
    n.conv("Conv", 192, 5, 1, 2, bias=True)
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 3, 2)
    for feat in (384, 384, 256):
        n.conv("Conv", feat, 3, 1, 1, bias=True)
        n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 3, 2)
    n.fc("InnerProduct", 4096)
    n.relu("ReLU")
    n.dropout("Dropout", 0.5)
    n.fc("InnerProduct", 4096)
    n.relu("ReLU")
    n.dropout("Dropout", 0.5)
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("alexnet-v2", [3, size, size], classes, solver_conf)


def mini_inception(solver_conf=None, classes=10, size=32):
    """Two inception modules (1x1 | 3x3 | 5x5 | pool-proj, concatenated on channels)."""
    n = Net()
    n.conv("Conv", 32, 3, 1, 1, bias=True)
    x = n.relu("ReLU")
    for m in range(2):
        b1 = n.relu("ReLU", [n.conv(f"mixed-{m}-1x1", 16, 1, bias=True, inputs=[x])])
        b3 = n.relu("ReLU", [n.conv(f"mixed-{m}-3x3", 24, 3, 1, 1, bias=True, inputs=[x])])
        b5 = n.relu("ReLU", [n.conv(f"mixed-{m}-5x5", 8, 5, 1, 2, bias=True, inputs=[x])])
        bp = n.pool(f"mixed-{m}-pool", PoolMethod.MAX, 3, 1, 1, inputs=[x])
        bp = n.relu("ReLU", [n.conv(f"mixed-{m}-proj", 16, 1, bias=True, inputs=[bp])])
        x = n.concat(f"mixed-{m}-concat", [b1, b3, b5, bp])
        x = n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.pool("Pool", PoolMethod.AVERAGE, 1, 1, global_pooling=True)
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("mini-inception", [3, size, size], classes, solver_conf)


def overfeat(solver_conf=None, classes=1000, size=231):
    """OverFeat (fast) of the convnet-benchmarks suite (convnet/benchmarks/ModelBuilder.java)."""
    n = Net()
    n.conv("Conv", 96, 11, 4, 0, bias=True)
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.conv("Conv", 256, 5, 1, 0, bias=True)
    n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    for feat in (512, 1024, 1024):
        n.conv("Conv", feat, 3, 1, 1, bias=True)
        n.relu("ReLU")
    n.pool("Pool", PoolMethod.MAX, 2, 2)
    n.fc("InnerProduct", 3072)
    n.relu("ReLU")
    n.fc("InnerProduct", 4096)
    n.relu("ReLU")
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("overfeat", [3, size, size], classes, solver_conf)


def vgg_a(solver_conf=None, classes=1000, size=224):
    """VGG model A (11 layers) of the convnet-benchmarks suite."""
    n = Net()
    for item in (64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"):
        if item == "M":
            n.pool("Pool", PoolMethod.MAX, 2, 2)
        else:
            n.conv("Conv", item, 3, 1, 1, bias=True)
            n.relu("ReLU")
    n.fc("InnerProduct", 4096)
    n.relu("ReLU")
    n.fc("InnerProduct", 4096)
    n.relu("ReLU")
    n.fc("InnerProduct", classes)
    n.classifier_tail()
    return n.finish("vgg-a", [3, size, size], classes, solver_conf)


def matrix_factorisation(solver_conf=None, rows=1000, columns=500, latents=16, lambda_=0.05):
    """SGD matrix factorisation over (row, column, rating) triples (MatrixFactorisation.java); the input "image" is a
    [3, 1, 1] example holding the two indices and the rating."""
    from ..conf import MatFactConf, ModelConf
    from ..graph import DataflowNode, Operator, SubGraph, append_gradients
    from ..kernels import MatFact
    from ._builder import ModelSpec
    conf = MatFactConf().setNumberOfRows(rows).setNumberOfColumns(columns).setNumberOfLatentVariables(latents)
    conf.lambda_ = lambda_
    conf.model_variable_initialiser = InitialiserConf().setType(InitialiserType.GAUSSIAN).setStd(0.1)
    head = DataflowNode(Operator("MatFact", MatFact(conf)))
    append_gradients(head, solver_conf or ModelConf.getInstance().getSolverConf())
    return ModelSpec("matrix-factorisation", SubGraph(head), None, [3, 1, 1], 1)
