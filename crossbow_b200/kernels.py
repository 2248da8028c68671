"""Operator ("kernel") classes: shape inference, model-variable registration and the fp32 CPU definition.

One class per operator of the reference's ``kernel`` package (kernel/*.java, ~7.9 K lines).  ``setup``
does what ``Kernel.setup`` does there (output shape + ``model.register``); ``forward`` is the CPU
definition of the operator in plain PyTorch fp32 (the role of ``compute`` in the reference, which goes
through OpenBLAS) and is THE oracle that every CUDA kernel is tested against.  Gradient operators are
defined as the vector-Jacobian product of their peer's ``forward`` so the two can never drift apart.

Shapes in this API are the reference's NCHW (``[examples, channels, height, width]``); the device
executor runs channels-last internally and converts at the boundary.
"""
from __future__ import annotations

import math
from typing import List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from .conf import (AccuracyConf, BatchNormConf, ClassifyConf, ConcatConf, ConvConf, DataTransformConf,
                   DropoutConf, ElementWiseOpConf, InnerProductConf, LRNConf, LossConf, MatFactConf,
                   NoopConf, PoolConf, ReLUConf, SoftMaxConf, SolverConf)
from .model import Model, Shape, Variable
from .types import (ActivationMode, BatchNormEstimatedMeanAndVarianceType, ElementWiseOpType,
                    NormalisationMode, Phase, PoolMethod)
from .utils.philox import philox_uniform, philox_uint32

FLT_MIN = 1.17549435e-38
BN_MIN_EPSILON = 1e-5  # CUDNN_BN_MIN_EPSILON


class Kernel:
    kind = "noop"
    is_gradient = False
    is_loss = False
    is_accuracy = False
    is_data_transform = False
    is_optimiser = False
    needs_labels = False

    def __init__(self, conf=None):
        self.conf = conf
        self.variables: List[Variable] = []
        self.operator = None

    # -- graph construction ----------------------------------------------------------------
    def setup(self, ins: List[Shape], model: Model, label_shape: Shape) -> Shape:
        return ins[0].copy()

    def _register(self, model: Model, var: Variable, order: int):
        self.variables.append(var)
        model.register(self.operator.id, var, order)

    def make_gradient(self) -> Optional["Kernel"]:
        cls = _GRADIENT_CLASSES.get(type(self).__name__)
        return cls(self.conf) if cls else GradientKernel(self.conf)

    # -- CPU definition ------------------------------------------------------------------
    def forward(self, xs: List[torch.Tensor], params: List[torch.Tensor], env: "OpEnv") -> torch.Tensor:
        return xs[0]


class OpEnv:
    """What an operator may look at besides inputs and parameters while it runs on the CPU oracle."""

    def __init__(self, phase=Phase.TRAIN, labels=None, task_id=0, seed=0, device_state=None, replica_updates=0):
        self.phase = phase
        self.labels = labels
        self.task_id = task_id
        self.seed = seed
        self.device_state = device_state if device_state is not None else {}   # shared by replicas of one device
        self.replica_updates = replica_updates

    @property
    def training(self):
        return self.phase == Phase.TRAIN


class GradientKernel(Kernel):
    """Gradient of the peer operator; evaluated as a VJP of the peer's ``forward``."""
    kind = "gradient"
    is_gradient = True


class GradientDescentOptimiser(Kernel):
    """Marks where the per-task local update runs (kernel/GradientDescentOptimiser.java:93-153)."""
    kind = "optimiser"
    is_optimiser = True

    def __init__(self, conf: Optional[SolverConf] = None):
        super().__init__(conf or SolverConf())


# --------------------------------------------------------------------------------------------

def _conv_geometry(conf: ConvConf):
    """ConvConf keeps 'size' = number of spatial dims and per-dim values (Conv.java:50-229)."""
    kh, kw = conf.kernel_height, conf.kernel_width
    sh, sw = conf.stride_height, conf.stride_width
    ph, pw = conf.padding_height, conf.padding_width
    return kh, kw, sh, sw, ph, pw


class Conv(Kernel):
    kind = "conv"

    def setup(self, ins, model, label_shape):
        c: ConvConf = self.conf
        if c.groups != 1:
            raise ValueError("error: grouped convolution is not supported")  # Conv.java:107-109
        n, ch, h, w = ins[0].dims
        kh, kw, sh, sw, ph, pw = _conv_geometry(c)
        oh = (h + 2 * ph - kh) // sh + 1
        ow = (w + 2 * pw - kw) // sw + 1
        k = c.number_of_outputs
        wv = Variable("weights", Shape([k, ch, kh, kw]), device_perm=(0, 2, 3, 1)).initialise(c.weight_initialiser)
        wv.lr_multiplier = c.weights_lr_multiplier
        self._register(model, wv, 1)
        if c.bias:
            bv = Variable("bias", Shape([k])).initialise(c.bias_initialiser)
            bv.lr_multiplier = c.bias_lr_multiplier
            self._register(model, bv, 2)
        return Shape([n, k, oh, ow])

    def forward(self, xs, params, env):
        kh, kw, sh, sw, ph, pw = _conv_geometry(self.conf)
        b = params[1] if self.conf.bias else None
        return F.conv2d(xs[0], params[0], b, stride=(sh, sw), padding=(ph, pw))


class InnerProduct(Kernel):
    kind = "innerproduct"

    def setup(self, ins, model, label_shape):
        c: InnerProductConf = self.conf
        dims = ins[0].dims
        n = dims[0]
        feat = ins[0].countAllElements(1)
        if len(dims) == 4 and dims[2] * dims[3] > 1:
            wv = Variable("weights", Shape([c.number_of_outputs, feat]),
                          view_shape=[c.number_of_outputs, dims[1], dims[2], dims[3]], device_perm=(0, 2, 3, 1))
        else:
            wv = Variable("weights", Shape([c.number_of_outputs, feat]))
        wv.initialise(c.weight_initialiser)
        wv.lr_multiplier = c.weights_lr_multiplier
        self._register(model, wv, 1)
        if c.bias:
            bv = Variable("bias", Shape([c.number_of_outputs])).initialise(c.bias_initialiser)
            bv.lr_multiplier = c.bias_lr_multiplier
            self._register(model, bv, 2)
        return Shape([n, c.number_of_outputs])

    def forward(self, xs, params, env):
        x = xs[0].reshape(xs[0].shape[0], -1)
        return F.linear(x, params[0], params[1] if self.conf.bias else None)


class MatMul(InnerProduct):
    """Product of the input with one model variable, no bias (the reference's test kernel, matmul.cu:3-35): an inner
    product whose configuration has the bias switched off."""

    def setup(self, ins, model, label_shape):
        self.conf.bias = False
        return super().setup(ins, model, label_shape)


class MatMulGradient(GradientKernel): pass


def pool_output_size(size, k, s, p):
    """Caffe ceil-mode extent with the clip that keeps the last window inside image+padding (Pool.java:159-175)."""
    o = int(math.ceil((size + 2 * p - k) / s)) + 1
    if p != 0 and (o - 1) * s >= size + p:
        o -= 1
    return o


class Pool(Kernel):
    kind = "pool"

    def setup(self, ins, model, label_shape):
        c: PoolConf = self.conf
        n, ch, h, w = ins[0].dims
        if c.global_pooling:
            c.kernel_height, c.kernel_width = h, w
            c.stride_height = c.stride_width = 1
            c.padding_height = c.padding_width = 0
        if c.padding_height >= c.kernel_height or c.padding_width >= c.kernel_width:
            raise ValueError("error: padding must be less than kernel size")
        oh = pool_output_size(h, c.kernel_height, c.stride_height, c.padding_height)
        ow = pool_output_size(w, c.kernel_width, c.stride_width, c.padding_width)
        return Shape([n, ch, oh, ow])

    def forward(self, xs, params, env):
        c: PoolConf = self.conf
        x = xs[0]
        n, ch, h, w = x.shape
        oh, ow = self.operator.output_shape.dims[2:]
        # explicit padding so ceil-mode windows that overhang are handled the cuDNN way:
        # max ignores the overhang, average always divides by kernel area (COUNT_INCLUDE_PADDING)
        need_h = (oh - 1) * c.stride_height + c.kernel_height
        need_w = (ow - 1) * c.stride_width + c.kernel_width
        pb = max(0, need_h - h - c.padding_height)
        pr = max(0, need_w - w - c.padding_width)
        if c.method == PoolMethod.MAX:
            xp = F.pad(x, (c.padding_width, pr, c.padding_height, pb), value=float("-inf"))
            return F.max_pool2d(xp, (c.kernel_height, c.kernel_width), (c.stride_height, c.stride_width))
        if c.method == PoolMethod.AVERAGE:
            xp = F.pad(x, (c.padding_width, pr, c.padding_height, pb), value=0.0)
            return F.avg_pool2d(xp, (c.kernel_height, c.kernel_width), (c.stride_height, c.stride_width))
        raise ValueError("error: stochastic pooling is not supported")


class ReLU(Kernel):
    kind = "relu"

    def forward(self, xs, params, env):
        c: ReLUConf = self.conf
        m = c.activation_mode
        if m == ActivationMode.RELU:
            return F.leaky_relu(xs[0], c.negative_slope) if c.negative_slope != 0 else F.relu(xs[0])
        if m == ActivationMode.SIGMOID:
            return torch.sigmoid(xs[0])
        if m == ActivationMode.TANH:
            return torch.tanh(xs[0])
        if m == ActivationMode.CLIPPEDRELU:
            return torch.clamp(xs[0], 0.0, float(c.ceiling))
        raise ValueError("error: invalid activation mode")


class SoftMax(Kernel):
    kind = "softmax"

    def forward(self, xs, params, env):
        return F.softmax(xs[0].reshape(xs[0].shape[0], -1), dim=1)


class SoftMaxLoss(Kernel):
    """Input: probabilities. loss = -sum(log(max(p[label], FLT_MIN))) / normaliser (SoftMaxLoss.java:109-170)."""
    kind = "softmaxloss"
    is_loss = True
    needs_labels = True

    def setup(self, ins, model, label_shape):
        return Shape([1])

    def forward(self, xs, params, env):
        p = xs[0]
        labels = env.labels.long()
        c: LossConf = self.conf
        valid = labels != c.ignored_label_value
        picked = p.gather(1, labels.clamp(min=0).unsqueeze(1)).squeeze(1).clamp(min=FLT_MIN)
        losses = -torch.log(picked) * valid
        if c.mode == NormalisationMode.BATCH:
            denom = p.shape[0]
        elif c.mode == NormalisationMode.VALID:
            denom = max(1, int(valid.sum()))
        elif c.mode == NormalisationMode.FULL:
            denom = p.shape[0]
        else:
            denom = 1
        return (losses.sum() / denom).reshape(1)


class Accuracy(Kernel):
    kind = "accuracy"
    is_accuracy = True
    needs_labels = True

    def setup(self, ins, model, label_shape):
        return Shape([1])

    def forward(self, xs, params, env):
        p = xs[0].reshape(xs[0].shape[0], -1)
        pred = p.argmax(dim=1)
        return (pred == env.labels.long()).float().mean().reshape(1)


class Classify(Kernel):
    kind = "classify"
    is_accuracy = True  # terminal, no gradient

    def setup(self, ins, model, label_shape):
        return Shape([ins[0].dims[0]])

    def forward(self, xs, params, env):
        return xs[0].reshape(xs[0].shape[0], -1).argmax(dim=1).float()


class BatchNorm(Kernel):
    """Spatial batch normalisation (BatchNorm.java:158-412; cudnnbatchnorm.cu:99-151).

    Training normalises with batch statistics (biased variance) and updates ONE running mean/variance per
    (operator, device) shared by all replicas on that device, with factor ``1 - fraction`` (FIXED) or
    ``1/(1+updates)`` (CMA); the running variance receives the unbiased batch variance (cuDNN).  Test uses
    the running statistics.
    """
    kind = "batchnorm"

    def setup(self, ins, model, label_shape):
        c: BatchNormConf = self.conf
        ch = ins[0].dims[1]
        wv = Variable("weights", Shape([ch])).initialise(c.weight_initialiser)
        wv.lr_multiplier = c.weights_lr_multiplier
        bv = Variable("bias", Shape([ch])).initialise(c.bias_initialiser)
        bv.lr_multiplier = c.bias_lr_multiplier
        self._register(model, wv, 1)
        self._register(model, bv, 2)
        self.channels = ch
        return ins[0].copy()

    def epsilon(self):
        return max(float(self.conf.epsilon), BN_MIN_EPSILON)

    def running(self, env: OpEnv):
        st = env.device_state.setdefault(("bn", self.operator.uid), None)
        if st is None:
            st = dict(mean=torch.zeros(self.channels), var=torch.ones(self.channels), updates=0)
            env.device_state[("bn", self.operator.uid)] = st
        return st

    def forward(self, xs, params, env):
        x = xs[0]
        st = self.running(env)
        eps = self.epsilon()
        shape = [1, -1] + [1] * (x.dim() - 2)
        red = [d for d in range(x.dim()) if d != 1]
        if env.training:
            mean = x.mean(dim=red)
            var = x.var(dim=red, unbiased=False)
            m = x.numel() // x.shape[1]
            with torch.no_grad():
                if self.conf.estimated_mean_and_variance_type == BatchNormEstimatedMeanAndVarianceType.CMA:
                    f = 1.0 / (1.0 + st["updates"])
                else:
                    f = 1.0 - float(self.conf.fraction)
                unb = var * (m / max(1, m - 1))
                st["mean"] = (1 - f) * st["mean"] + f * mean.detach()
                st["var"] = (1 - f) * st["var"] + f * unb.detach()
                st["updates"] += 1
        else:
            mean, var = st["mean"], st["var"]
        xhat = (x - mean.reshape(shape)) * torch.rsqrt(var.reshape(shape) + eps)
        return xhat * params[0].reshape(shape) + params[1].reshape(shape)


class Dropout(Kernel):
    """Inverted dropout: kept units are scaled by 1/(1-ratio) in training, identity at test
    (cudnndropout.cu:4-75).  The mask is a pure function of (seed, task, operator, element) through
    Philox4x32-10 so the CPU oracle and the CUDA kernel draw identical masks."""
    kind = "dropout"

    def mask(self, n, env: OpEnv):
        u = philox_uniform(n, env.seed, stream=self.operator.uid, offset=env.task_id)
        return torch.from_numpy((u >= self.conf.ratio).astype(np.float32))

    def forward(self, xs, params, env):
        if not env.training:
            return xs[0]
        x = xs[0]
        # mask is indexed in channels-last element order (the device layout)
        if x.dim() == 4:
            n, c, h, w = x.shape
            m = self.mask(x.numel(), env).reshape(n, h, w, c).permute(0, 3, 1, 2)
        else:
            m = self.mask(x.numel(), env).reshape(x.shape)
        return x * m * (1.0 / (1.0 - self.conf.ratio))


class ElementWiseOp(Kernel):
    kind = "elementwise"

    def setup(self, ins, model, label_shape):
        for s in ins[1:]:
            if s.dims != ins[0].dims:
                raise ValueError(f"error: element-wise inputs differ in shape: {ins}")
        return ins[0].copy()

    def forward(self, xs, params, env):
        c: ElementWiseOpConf = self.conf
        if c.type == ElementWiseOpType.SUM:
            out = xs[0] * c.getCoefficient(0)
            for i, x in enumerate(xs[1:], 1):
                out = out + x * c.getCoefficient(i)
            return out
        if c.type == ElementWiseOpType.PRODUCT:
            out = xs[0]
            for x in xs[1:]:
                out = out * x
            return out
        out = xs[0]
        for x in xs[1:]:
            out = torch.maximum(out, x)
        return out


class Concat(Kernel):
    kind = "concat"

    def setup(self, ins, model, label_shape):
        ax = self.conf.axis
        dims = list(ins[0].dims)
        dims[ax] = sum(s.dims[ax] for s in ins)
        return Shape(dims)

    def forward(self, xs, params, env):
        return torch.cat(xs, dim=self.conf.axis)


class LRN(Kernel):
    """Across-channel local response normalisation (Caffe definition). The reference has CPU stubs only."""
    kind = "lrn"

    def forward(self, xs, params, env):
        c: LRNConf = self.conf
        return F.local_response_norm(xs[0], c.local_size, alpha=c.alpha, beta=c.beta, k=c.k)


class DataTransform(Kernel):
    """Random crop + mirror + mean subtraction + scale on the input batch (datatransform.cu:3-76).

    Training: per example, crop offsets and mirror flag come from three Philox draws; test: centre crop,
    no mirror.
    """
    kind = "datatransform"
    is_data_transform = True
    no_gradient = True

    def setup(self, ins, model, label_shape):
        c: DataTransformConf = self.conf
        n, ch, h, w = ins[0].dims
        cs = c.crop_size or 0
        if cs > 0:
            if cs > h or cs > w:
                raise ValueError("error: crop size exceeds image size")
            return Shape([n, ch, cs, cs])
        return ins[0].copy()

    def make_gradient(self):
        return None

    def randoms(self, n, env):
        return philox_uint32(3 * n, env.seed, stream=self.operator.uid, offset=env.task_id).reshape(n, 3)

    def mean_tensor(self, shape):
        c = self.conf
        if c.mean_pixel_values:
            return torch.tensor(c.mean_pixel_values, dtype=torch.float32).reshape(1, -1, 1, 1)
        if c.mean_image_filename:
            m = np.fromfile(c.mean_image_filename, dtype=np.float32)
            return torch.from_numpy(m).reshape(1, *shape[1:])
        return None

    def forward(self, xs, params, env):
        c: DataTransformConf = self.conf
        x = xs[0]
        n, ch, h, w = x.shape
        cs = c.crop_size or 0
        oh, ow = (cs, cs) if cs > 0 else (h, w)
        mean = self.mean_tensor(x.shape) if c.subtract_mean else None
        if mean is not None and mean.shape[-1] == w:   # per-pixel mean image is subtracted before cropping
            x = x - mean
            mean = None
        out = torch.empty(n, ch, oh, ow)
        r = self.randoms(n, env) if env.training else None
        for i in range(n):
            if env.training:
                ho = int(r[i, 0] % (h - oh + 1))
                wo = int(r[i, 1] % (w - ow + 1))
                flip = bool(c.mirror and (r[i, 2] & 1))
            else:
                ho, wo, flip = (h - oh) // 2, (w - ow) // 2, False
            img = x[i, :, ho:ho + oh, wo:wo + ow]
            out[i] = torch.flip(img, dims=[2]) if flip else img
        if mean is not None:
            out = out - mean
        return out * float(c.scale_factor)


class Noop(Kernel):
    """Has one model variable of the input's shape and copies input to output (noop.cu:3-47)."""
    kind = "noop"

    def setup(self, ins, model, label_shape):
        v = Variable("weights", Shape(ins[0].dims[1:] if len(ins[0].dims) > 1 else ins[0].dims))
        self._register(model, v, 1)
        return ins[0].copy()


class NoopStateless(Kernel):
    kind = "noop"


class Dummy(Kernel):
    """Shape-preserving placeholder used by the memory-planner tests (TestMemoryPlanner.java:26-60)."""
    kind = "noop"


class MatFact(Kernel):
    """SGD matrix factorisation over (row, column, rating) triples (matfact.cu:6-61).

    Model: user factors [rows, latents], item factors [columns, latents].  forward returns the mean squared
    error of the batch; the gradient is the usual regularised MF gradient.
    """
    kind = "matfact"
    is_loss = True

    def setup(self, ins, model, label_shape):
        c: MatFactConf = self.conf
        init = c.model_variable_initialiser
        u = Variable("weights", Shape([c.number_of_rows, c.number_of_latent_variables]))
        v = Variable("bias", Shape([c.number_of_columns, c.number_of_latent_variables]))
        if init is not None:
            u.initialise(init)
            v.initialise(init)
        self._register(model, u, 1)
        self._register(model, v, 2)
        return Shape([1])

    def forward(self, xs, params, env):
        x = xs[0].reshape(xs[0].shape[0], -1)
        rows, cols = x[:, 0].long(), x[:, 1].long()
        rating = env.labels.float() if env.labels is not None else x[:, 2]
        pred = (params[0][rows] * params[1][cols]).sum(dim=1)
        err = rating - pred
        reg = self.conf.lambda_ * (params[0][rows].pow(2).sum() + params[1][cols].pow(2).sum())
        return ((err * err).sum() + reg).reshape(1) / x.shape[0]


# ---- named gradient classes (API parity with kernel/*Gradient.java) ------------------------

class ConvGradient(GradientKernel): pass
class InnerProductGradient(GradientKernel): pass
class PoolGradient(GradientKernel): pass
class ReLUGradient(GradientKernel): pass
class SoftMaxGradient(GradientKernel): pass
class BatchNormGradient(GradientKernel): pass
class DropoutGradient(GradientKernel): pass
class ElementWiseOpGradient(GradientKernel): pass
class ConcatGradient(GradientKernel): pass
class LRNGradient(GradientKernel): pass
class NoopGradient(GradientKernel): pass
class MatFactGradient(GradientKernel): pass


class SoftMaxLossGradient(GradientKernel):
    """(p - onehot)/N: the gradient w.r.t. the LOGITS, so graphs skip SoftMaxGradient
    (SoftMaxLossGradient.java:117-180).  The oracle evaluates softmax+loss jointly to honour that."""
    fused_with_softmax = True


_GRADIENT_CLASSES = {
    "Conv": ConvGradient, "InnerProduct": InnerProductGradient, "Pool": PoolGradient, "ReLU": ReLUGradient,
    "SoftMax": SoftMaxGradient, "SoftMaxLoss": SoftMaxLossGradient, "BatchNorm": BatchNormGradient,
    "Dropout": DropoutGradient, "ElementWiseOp": ElementWiseOpGradient, "Concat": ConcatGradient,
    "LRN": LRNGradient, "Noop": NoopGradient, "MatFact": MatFactGradient,
}
