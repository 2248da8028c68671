"""Model variables, initialisers and the flat parameter layout.

A model is an ordered list of variables (ascending operator id; inside an operator: weights, then
bias) stored back to back in ONE contiguous fp32 vector, exactly like the reference's
``crossbow_model_t.data`` (clib-multigpu/model.c:30-47,127-157; Model.java:121-143,346-354).  The flat
vector is what the fused optimiser and synchronisation kernels operate on and what a checkpoint file
contains.

Two element orders exist for the same (offset, length) slot of a variable:

* canonical - the reference's order (convolution ``[K,C,R,S]``, inner product ``[out, C*H*W]``), used by
  the CPU oracle and by checkpoint files;
* device - channels-last (convolution ``[K,R,S,C]``, inner product columns in ``H,W,C`` order), which makes
  the implicit-GEMM reduction axis contiguous for the sm_100a kernels.

``Model.to_device`` / ``Model.to_canonical`` convert a whole flat vector between them.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import numpy as np

from .conf import InitialiserConf
from .types import InitialiserType, VarianceNormalisation


DEVICE_ALIGN = 64   # floats; keeps every variable 256-byte aligned for 16-byte vector loads and bulk copies


class Shape:
    """N-d extent with the reference's accessor names (model/Shape.java)."""

    def __init__(self, dims: Sequence[int]):
        self.dims = [int(d) for d in dims]

    def dimensions(self):
        return len(self.dims)

    def get(self, i):
        return self.dims[i]

    def set(self, i, v):
        self.dims[i] = int(v)
        return self

    def numberOfExamples(self):
        return self.dims[0]

    def numberOfChannels(self):
        return self.dims[1] if len(self.dims) > 1 else 1

    def height(self):
        return self.dims[2] if len(self.dims) > 2 else 1

    def width(self):
        return self.dims[3] if len(self.dims) > 3 else 1

    def countAllElements(self, start=0, end=None):
        n = 1
        for d in self.dims[start:end]:
            n *= d
        return n

    count = countAllElements

    def copy(self):
        return Shape(self.dims)

    def tuple(self):
        return tuple(self.dims)

    # remaining names of model/Shape.java
    def push(self, value):
        self.dims.append(int(value))

    def countElements(self, start, end=None):
        return self.countAllElements(start, end)

    def offset(self, n, c):
        """Element offset of (example n, channel c) in a contiguous N x C x H x W tensor."""
        return ((n * self.numberOfChannels() + c) * self.height()) * self.width()

    def array(self):
        return self.dims

    def getNCHW(self, out=None):
        v = [self.numberOfExamples(), self.numberOfChannels(), self.height(), self.width()]
        if out is not None:
            out[:4] = v
        return v

    def equals(self, other):
        return self == other

    def toString(self):
        return repr(self)

    def __eq__(self, o):
        return isinstance(o, Shape) and self.dims == o.dims

    def __repr__(self):
        return "[" + ", ".join(str(d) for d in self.dims) + "]"


class RandomGenerator:
    """Seeded Mersenne-Twister source for initialisers (random/generator.cpp:22-110 uses mt19937 too)."""

    def __init__(self, seed: int):
        self.rng = np.random.Generator(np.random.MT19937(int(seed) & 0xFFFFFFFF))

    def uniform_fill(self, n, low, high):
        return self.rng.uniform(low, high, size=n).astype(np.float32)

    def gaussian_fill(self, n, mean, std, truncate):
        """Truncation re-draws values outside mean +- 2 std, at most 100 times per element (generator.cpp)."""
        out = self.rng.normal(mean, std, size=n)
        if truncate:
            for _ in range(100):
                bad = np.abs(out - mean) > 2.0 * std
                nb = int(bad.sum())
                if nb == 0:
                    break
                out[bad] = self.rng.normal(mean, std, size=nb)
        return out.astype(np.float32)


class Variable:
    """One learnable tensor: name, canonical shape, initialiser, learning-rate multiplier, flat-vector slot."""

    def __init__(self, name: str, shape: Shape, learnable=True, device_perm: Optional[Sequence[int]] = None,
                 view_shape: Optional[Sequence[int]] = None):
        self.name = name
        self.shape = shape
        self.learnable = learnable
        self.initialiser: InitialiserConf = InitialiserConf()
        self.lr_multiplier = 1.0
        self.offset = -1            # element offset in the packed (canonical / checkpoint) flat vector
        self.doffset = -1           # element offset in the device flat vector (every variable 256-byte aligned)
        self.op_id = -1
        self.order = 0              # 1 = weights, 2 = bias (Model.java linked-list order)
        # canonical -> device element order: reshape to view_shape, permute by device_perm, flatten
        self.view_shape = list(view_shape) if view_shape is not None else list(shape.dims)
        self.device_perm = list(device_perm) if device_perm is not None else None

    def elements(self):
        return self.shape.countAllElements()

    def setLearningRateMultiplier(self, m):
        self.lr_multiplier = float(m)
        return self

    # accessors of model/Variable.java
    def getLearningRateMultiplier(self):
        return self.lr_multiplier

    def getName(self):
        return self.name

    def getShape(self):
        return self.shape

    def getOrder(self):
        return self.order

    def setOrder(self, order):
        self.order = int(order)
        return self

    def capacity(self):
        """Bytes of the variable."""
        return 4 * self.elements()

    def initialise(self, conf: InitialiserConf):
        self.initialiser = conf
        return self

    def generate(self, rng: RandomGenerator) -> np.ndarray:
        """Canonical-order initial values (model/Initialiser.java:44-176)."""
        c, n = self.initialiser, self.elements()
        t = c.type
        if t == InitialiserType.CONSTANT:
            return np.full(n, c.value, dtype=np.float32)
        if t == InitialiserType.UNIFORM:
            # not implemented in the reference (Initialiser.java:73); plain U[min,max) here
            return rng.uniform_fill(n, c.min, c.max)
        if t == InitialiserType.XAVIER:
            fan_in = n / self.shape.numberOfExamples()
            fan_out = n / self.shape.numberOfChannels()
            k = {VarianceNormalisation.FAN_IN: fan_in, VarianceNormalisation.FAN_OUT: fan_out,
                 VarianceNormalisation.AVG: 0.5 * (fan_in + fan_out)}[c.norm]
            scale = math.sqrt(3.0 / k)
            return rng.uniform_fill(n, -scale, scale)
        if t == InitialiserType.GAUSSIAN:
            if c.std <= 0:
                raise ValueError("error: standard deviation must be greater than 0")
            return rng.gaussian_fill(n, c.mean, c.std, c.truncated)
        if t == InitialiserType.MSRA:
            std = math.sqrt(2.0 / (n / self.shape.numberOfChannels()))
            return rng.gaussian_fill(n, c.mean, std, c.truncated)
        raise ValueError("error: invalid initialiser type")

    # ---- element-order conversion ----
    def to_device(self, canonical: np.ndarray) -> np.ndarray:
        if self.device_perm is None:
            return canonical
        return np.ascontiguousarray(canonical.reshape(self.view_shape).transpose(self.device_perm)).reshape(-1)

    def to_canonical(self, device: np.ndarray) -> np.ndarray:
        if self.device_perm is None:
            return device
        dshape = [self.view_shape[i] for i in self.device_perm]
        inv = np.argsort(self.device_perm)
        return np.ascontiguousarray(device.reshape(dshape).transpose(inv)).reshape(-1)

    def __repr__(self):
        return f"Variable({self.name}, {self.shape}, offset={self.offset})"


class Model:
    """Registry of variables + the flat layout.  ``register`` is called by operators during graph init."""

    def __init__(self):
        self.variables: List[Variable] = []
        self._final = False
        self.elements = 0
        self.device_elements = 0

    # accessors of model/Model.java
    def getVariables(self):
        return list(self.variables)

    def getVariable(self, op_id: int, order: int = 1):
        """Variable `order` (1 = weights, 2 = bias) of an operator, or None."""
        for v in self.variables:
            if v.op_id == op_id and v.order == order:
                return v
        return None

    def getSize(self):
        return len(self.variables)

    def capacity(self):
        return self.bytes()

    def toString(self):
        return self.dump()

    def register(self, op_id: int, var: Variable, order: int):
        if self._final:
            raise RuntimeError("error: model is already finalised")
        var.op_id, var.order = op_id, order
        self.variables.append(var)

    def finalise(self):
        """Sort by (operator id, weights-before-bias) and assign offsets (Model.java:346-354)."""
        self.variables.sort(key=lambda v: (v.op_id, v.order))
        off = 0
        for v in self.variables:
            v.offset = off
            off += v.elements()
        self.elements = off
        doff = 0
        for v in self.variables:
            v.doffset = doff
            doff += (v.elements() + DEVICE_ALIGN - 1) // DEVICE_ALIGN * DEVICE_ALIGN
        self.device_elements = doff
        self._final = True
        return self

    def bytes(self):
        return 4 * self.elements

    def variables_of(self, op_id: int) -> List[Variable]:
        return [v for v in self.variables if v.op_id == op_id]

    def initial_values(self, seed: int) -> np.ndarray:
        """Flat canonical-order vector of freshly initialised parameters."""
        rng = RandomGenerator(seed)
        out = np.empty(self.elements, dtype=np.float32)
        for v in self.variables:
            out[v.offset:v.offset + v.elements()] = v.generate(rng)
        return out

    def lr_multipliers(self) -> np.ndarray:
        out = np.ones(self.elements, dtype=np.float32)
        for v in self.variables:
            out[v.offset:v.offset + v.elements()] = v.lr_multiplier
        return out

    def has_lr_multipliers(self) -> bool:
        return any(v.lr_multiplier != 1.0 for v in self.variables)

    def to_device(self, flat) -> np.ndarray:
        """Packed canonical vector -> padded channels-last device vector (padding is zero and stays zero)."""
        flat = np.asarray(flat, dtype=np.float32)
        out = np.zeros(self.device_elements, dtype=np.float32)
        for v in self.variables:
            out[v.doffset:v.doffset + v.elements()] = v.to_device(flat[v.offset:v.offset + v.elements()])
        return out

    def to_canonical(self, dflat) -> np.ndarray:
        dflat = np.asarray(dflat, dtype=np.float32)
        out = np.empty(self.elements, dtype=np.float32)
        for v in self.variables:
            out[v.offset:v.offset + v.elements()] = v.to_canonical(dflat[v.doffset:v.doffset + v.elements()])
        return out

    def dump(self) -> str:
        lines = [f"=== [Model: {len(self.variables)} variables, {self.elements} elements, {self.bytes()} bytes] ==="]
        for v in self.variables:
            lines.append(f"op {v.op_id:4d} {v.name:<24s} {str(v.shape):<22s} offset {v.offset:10d} lr x{v.lr_multiplier}")
        return "\n".join(lines)
