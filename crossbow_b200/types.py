"""Enumerations shared by the whole framework.

Same vocabulary as the reference's ``types`` package
(src/main/java/uk/ac/imperial/lsds/crossbow/types/*.java) so that a user can carry
flag values (``--update-model SMA``, ``--synchronisation-model BSP`` ...) over unchanged.
"""
from __future__ import annotations

import enum


class _NamedEnum(enum.IntEnum):
    @classmethod
    def from_string(cls, s):
        if isinstance(s, cls):
            return s
        key = str(s).strip().upper().replace("-", "_")
        if key in cls.__members__:              # (includes aliases)
            return cls.__members__[key]
        raise ValueError(f"error: invalid {cls.__name__}: {s}")

    fromString = from_string

    def __str__(self):
        return self.name


class UpdateModel(_NamedEnum):
    """types/UpdateModel.java: which per-task optimiser + per-clock synchronisation pair runs."""
    DEFAULT = 0
    WORKER = 1  # synchronous SGD
    EAMSGD = 2
    SYNCHRONOUSEAMSGD = 3
    DOWNPOUR = 4
    HOGWILD = 5
    POLYAK_RUPPERT = 6
    SMA = 7


class SynchronisationModel(_NamedEnum):
    BSP = 0
    SSP = 1
    ASP = 2


class SchedulingPolicy(_NamedEnum):
    HLS = 0
    FIFO = 1
    NULL = 2


class ReplicationModel(_NamedEnum):
    SRSW = 0
    MRSW = 1


class Phase(_NamedEnum):
    TRAIN = 0
    CHECK = 1


class TrainingUnit(_NamedEnum):
    EPOCHS = 0
    TASKS = 1

    @classmethod
    def from_string(cls, s):
        if isinstance(s, cls):
            return s
        k = str(s).strip().lower()
        if k in ("epoch", "epochs"):
            return cls.EPOCHS
        if k in ("task", "tasks"):
            return cls.TASKS
        raise ValueError(f"error: invalid training unit: {s}")

    fromString = from_string


class DurationUnit(_NamedEnum):
    SECONDS = 0
    MINUTES = 1
    HOURS = 2

    def seconds(self, n):
        return n * (1, 60, 3600)[int(self)]


class LearningRateDecayPolicy(_NamedEnum):
    FIXED = 0
    INV = 1
    STEP = 2
    MULTISTEP = 3
    LSR = 4   # linear warm-up followed by multistep
    EXP = 5
    CLR = 6


class MomentumMethod(_NamedEnum):
    POLYAK = 0
    NESTEROV = 1


class Regularisation(_NamedEnum):
    L1 = 0
    L2 = 1


class InitialiserType(_NamedEnum):
    CONSTANT = 0
    UNIFORM = 1
    XAVIER = 2
    GAUSSIAN = 3
    MSRA = 4


class VarianceNormalisation(_NamedEnum):
    FAN_IN = 0
    FAN_OUT = 1
    AVG = 2


class PoolMethod(_NamedEnum):
    MAX = 0
    AVERAGE = 1
    STOCHASTIC = 2


class ActivationMode(_NamedEnum):
    SIGMOID = 0
    RELU = 1
    TANH = 2
    CLIPPEDRELU = 3


class BatchNormEstimatedMeanAndVarianceType(_NamedEnum):
    FIXED = 0
    CMA = 1


class ElementWiseOpType(_NamedEnum):
    PRODUCT = 0
    SUM = 1
    MAX = 2


class NormalisationMode(_NamedEnum):
    FULL = 0
    VALID = 1
    BATCH = 2
    NONE = 3


class NormalisationRegion(_NamedEnum):
    ACROSS_CHANNELS = 0
    WITHIN_CHANNEL = 1
    WITHIN_CHANNELS = 1      # the reference's spelling (types/NormalisationRegion.java); same member


class CudnnKernelType(_NamedEnum):
    """types/CudnnKernelType.java: which library descriptor family a kernel used in the reference.  Kept for programs that
    name it; the kernels here are hand-written and need no such tag."""
    UNDEFINED = 0
    CONV = 1
    POOL = 2
    RELU = 3
    SOFTMAX = 4
    BATCHNORM = 5
    DROPOUT = 6


class DatasetType(_NamedEnum):
    BASIC = 0
    LIGHT = 1
    RECORD = 2
    SYNTHETIC = 3  # generated in pinned memory; has no counterpart file format


class DatasetFileType(_NamedEnum):
    EXAMPLES = 0
    LABELS = 1


class DataType(_NamedEnum):
    INT = 0
    FLOAT = 1

    def sizeOf(self):
        return 4


class ExecutionMode(_NamedEnum):
    CPU = 0
    GPU = 1
    HYBRID = 2


class HandlerType(_NamedEnum):
    TASK = 0
    CALLBACK = 1
    DATASET = 2


class ModelAccess(_NamedEnum):
    NA = 0
    RO = 1
    RW = 2


class DependencyType(_NamedEnum):
    END_BEFORE_START = 0
    START_BEFORE_START = 1
    END_BEFORE_END = 2
    START_BEFORE_END = 3
