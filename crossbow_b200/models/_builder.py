"""Small helper used by the model builders: creates nodes, wires them, derives gradients and the test graph."""
from __future__ import annotations

from typing import List, Optional, Sequence

from ..conf import (AccuracyConf, BatchNormConf, ConvConf, DataTransformConf, DropoutConf, ElementWiseOpConf,
                    InitialiserConf, InnerProductConf, LossConf, ModelConf, PoolConf, ReLUConf, SoftMaxConf,
                    ConcatConf, LRNConf)
from ..graph import DataflowNode, Operator, SubGraph, append_gradients, shallow_copy_forward
from ..kernels import (Accuracy, BatchNorm, Conv, DataTransform, Dropout, ElementWiseOp, InnerProduct, Pool, ReLU,
                       SoftMax, SoftMaxLoss, Concat, LRN)
from ..types import InitialiserType, PoolMethod


class ModelSpec:
    """What a builder returns: training and test sub-graphs plus the input description."""

    def __init__(self, name, train: SubGraph, test: Optional[SubGraph], input_shape: Sequence[int], classes: int):
        self.name = name
        self.train = train
        self.test = test
        self.input_shape = list(input_shape)   # [C, H, W] of one example
        self.classes = classes

    def graphs(self):
        return [self.train, self.test]


class Net:
    def __init__(self, init_type=InitialiserType.XAVIER):
        self.head: Optional[DataflowNode] = None
        self.cur: Optional[DataflowNode] = None
        self.init_type = init_type

    def add(self, name, kernel, inputs: Optional[List[DataflowNode]] = None) -> DataflowNode:
        node = DataflowNode(Operator(name, kernel))
        if inputs is None:
            inputs = [self.cur] if self.cur is not None else []
        for i in inputs:
            i.connectTo(node)
        if self.head is None:
            self.head = node
        self.cur = node
        return node

    # ---- layer shorthands ----
    def winit(self):
        return InitialiserConf().setType(self.init_type)

    def conv(self, name, outputs, k, stride=1, pad=0, bias=False, inputs=None, winit=None, binit=None):
        """`k`, `stride`, `pad`: one number, or (height, width)."""
        hw = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)
        (kh, kw), (sh, sw), (ph, pw) = hw(k), hw(stride), hw(pad)
        c = ConvConf().setNumberOfOutputs(outputs).setKernelSize(2, kh, kw).setStrideSize(2, sh, sw) \
            .setPaddingSize(2, ph, pw).setBias(bias)
        c.setWeightInitialiser(winit or self.winit())
        if binit is not None:
            c.setBiasInitialiser(binit)
        return self.add(name, Conv(c), inputs)

    def bn(self, name, eps=1e-5, fraction=0.9, inputs=None):
        return self.add(name, BatchNorm(BatchNormConf().setEpsilon(eps).setMovingAverageFraction(fraction)), inputs)

    def relu(self, name, inputs=None):
        return self.add(name, ReLU(ReLUConf()), inputs)

    def pool(self, name, method, k, stride, pad=0, inputs=None, global_pooling=False):
        c = PoolConf().setMethod(method).setKernelSize(k).setStrideSize(stride).setPaddingSize(pad)
        c.global_pooling = global_pooling
        return self.add(name, Pool(c), inputs)

    def fc(self, name, outputs, inputs=None, winit=None, binit=None, bias=True):
        c = InnerProductConf().setNumberOfOutputs(outputs).setBias(bias)
        c.setWeightInitialiser(winit or self.winit())
        c.setBiasInitialiser(binit or InitialiserConf().setType(InitialiserType.CONSTANT).setValue(0))
        return self.add(name, InnerProduct(c), inputs)

    def dropout(self, name, ratio, inputs=None):
        return self.add(name, Dropout(DropoutConf().setRatio(ratio)), inputs)

    def sum(self, name, inputs):
        return self.add(name, ElementWiseOp(ElementWiseOpConf()), inputs)

    def concat(self, name, inputs):
        return self.add(name, Concat(ConcatConf()), inputs)

    def lrn(self, name, size=5, alpha=1e-4, beta=0.75, k=1.0):
        return self.add(name, LRN(LRNConf().setLocalSize(size).setAlpha(alpha).setBeta(beta).setK(k)))

    def transform(self, crop=0, mirror=False, mean=None, scale=1.0):
        c = DataTransformConf().setCropSize(crop).setMirror(mirror).setScaleFactor(scale)
        if mean is not None:
            c.setMeanPixelValues(mean)
        return self.add("DataTransform", DataTransform(c))

    def classifier_tail(self):
        """softmax -> loss and softmax -> accuracy."""
        sm = self.add("SoftMax", SoftMax(SoftMaxConf()))
        self.add("SoftMaxLoss", SoftMaxLoss(LossConf()), [sm])
        self.add("Accuracy", Accuracy(AccuracyConf()), [sm])
        return sm

    def finish(self, name, input_shape, classes, solver_conf=None, keep_in_test=None) -> ModelSpec:
        append_gradients(self.head, solver_conf or ModelConf.getInstance().getSolverConf())
        keep = keep_in_test or (lambda k: k.kind not in ("dropout", "softmaxloss"))
        test_head = shallow_copy_forward(self.head, keep)
        return ModelSpec(name, SubGraph(self.head), SubGraph(test_head), input_shape, classes)
