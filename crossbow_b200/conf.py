"""Configuration objects: system, model, solver, initialiser and per-operator ``Conf`` classes.

Covers the reference's ``SystemConf`` (SystemConf.java:134-235, 597-786), ``ModelConf``
(ModelConf.java:53-83, 253-441), ``SolverConf`` (kernel/conf/SolverConf.java:15-107, 411-440) and the
operator configuration classes in ``kernel/conf/*.java``.  Every class has snake_case attributes plus
the fluent camelCase setters/getters of the reference (``conf.setNumberOfOutputs(10)``), generated from
the field table so the two spellings can never disagree.
"""
from __future__ import annotations

import math
import re
from typing import Any, Dict, List, Optional

from .types import (ActivationMode, BatchNormEstimatedMeanAndVarianceType, ElementWiseOpType,
                    InitialiserType, LearningRateDecayPolicy, MomentumMethod, NormalisationMode,
                    NormalisationRegion, PoolMethod, Regularisation, ReplicationModel,
                    SchedulingPolicy, SynchronisationModel, TrainingUnit, UpdateModel,
                    VarianceNormalisation, DurationUnit, Phase)


def _camel_to_snake(name: str) -> str:
    s = re.sub(r"(.)([A-Z][a-z]+)", r"\1_\2", name)
    return re.sub(r"([a-z0-9])([A-Z])", r"\1_\2", s).lower()


class Fluent:
    """Base class: attributes listed in ``FIELDS`` get ``setX``/``getX``/``isX``/``hasX`` accessors."""
    FIELDS: Dict[str, Any] = {}
    ALIASES: Dict[str, str] = {}

    def __init__(self, **kw):
        for klass in reversed(type(self).__mro__):
            for k, v in getattr(klass, "FIELDS", {}).items():
                setattr(self, k, list(v) if isinstance(v, list) else v)
        for k, v in kw.items():
            if not hasattr(self, k):
                raise TypeError(f"{type(self).__name__}: unknown field {k}")
            setattr(self, k, v)

    def _field(self, camel: str) -> Optional[str]:
        f = _camel_to_snake(camel)
        f = self.ALIASES.get(f, f)
        return f if f in self.__dict__ else None

    def __getattr__(self, name):
        # only called when normal lookup fails
        for prefix in ("set", "get", "is", "has", "use"):
            if name.startswith(prefix) and len(name) > len(prefix) and name[len(prefix)].isupper():
                f = self.__dict__ and self._field(name[len(prefix):])
                if f:
                    if prefix == "set":
                        def setter(*a, _f=f):
                            setattr(self, _f, a[0] if len(a) == 1 else list(a))
                            return self
                        return setter
                    return lambda _f=f: getattr(self, _f)
        raise AttributeError(f"{type(self).__name__} has no attribute {name}")

    def dump(self) -> str:
        return "\n".join(f"{k:<32s} {getattr(self, k)}" for k in sorted(self.__dict__) if not k.startswith("_"))

    def __repr__(self):
        return f"{type(self).__name__}({', '.join(f'{k}={v!r}' for k, v in self.__dict__.items() if not k.startswith('_'))})"


# --------------------------------------------------------------------------------------------
# Initialisers
# --------------------------------------------------------------------------------------------

class InitialiserConf(Fluent):
    """model/InitialiserConf.java:21-31 — how a model variable is filled at start-up."""
    FIELDS = dict(type=InitialiserType.CONSTANT, value=0.0, std=1.0, mean=0.0, truncated=False,
                  norm=VarianceNormalisation.FAN_IN, min=0.0, max=1.0)

    def truncate(self, flag=True):
        self.truncated = bool(flag)
        return self

    def setType(self, t):
        self.type = InitialiserType.from_string(t)
        return self


# --------------------------------------------------------------------------------------------
# Operator confs
# --------------------------------------------------------------------------------------------

class ConvConf(Fluent):
    """kernel/conf/ConvConf.java:30-53."""
    FIELDS = dict(number_of_outputs=1, bias=True, axis=1, groups=1,
                  kernel_size=2, kernel_height=1, kernel_width=1,
                  stride_size=2, stride_height=1, stride_width=1,
                  padding_size=2, padding_height=0, padding_width=0,
                  weight_initialiser=None, bias_initialiser=None,
                  weights_lr_multiplier=1.0, bias_lr_multiplier=1.0)

    def __init__(self, **kw):
        super().__init__(**kw)
        self.weight_initialiser = self.weight_initialiser or InitialiserConf()
        self.bias_initialiser = self.bias_initialiser or InitialiserConf()

    def setKernelSize(self, dims, h=None, w=None):
        """Reference style: ``setKernelSize(2).setKernelHeight(5).setKernelWidth(5)``; shortcut ``setKernelSize(2, 5, 5)``."""
        self.kernel_size = dims
        if h is not None:
            self.kernel_height, self.kernel_width = h, (w if w is not None else h)
        return self

    def setStrideSize(self, dims, h=None, w=None):
        self.stride_size = dims
        if h is not None:
            self.stride_height, self.stride_width = h, (w if w is not None else h)
        return self

    def setPaddingSize(self, dims, h=None, w=None):
        self.padding_size = dims
        if h is not None:
            self.padding_height, self.padding_width = h, (w if w is not None else h)
        return self

    def setBias(self, flag):
        self.bias = bool(flag)
        return self

    def hasBias(self):
        return self.bias

    # indexed access as in ConvConf.java:117-221 (index 0 = height, 1 = width)
    def setKernel(self, ndx, val):
        setattr(self, ("kernel_height", "kernel_width")[ndx], int(val))
        return self

    def getKernel(self, ndx):
        return (self.kernel_height, self.kernel_width)[ndx]

    def setStride(self, ndx, val):
        setattr(self, ("stride_height", "stride_width")[ndx], int(val))
        return self

    def getStride(self, ndx):
        return (self.stride_height, self.stride_width)[ndx]

    def setPadding(self, ndx, val):
        setattr(self, ("padding_height", "padding_width")[ndx], int(val))
        return self

    def getPadding(self, ndx):
        return (self.padding_height, self.padding_width)[ndx]

    def numberOfOutputs(self):
        return self.number_of_outputs

    def setNumberOfGroup(self, groups):
        self.groups = int(groups)
        return self

    def numberOfGroups(self):
        return self.groups

    # learning-rate multipliers under the reference's names
    def setWeightsLearningRateMultiplier(self, v):
        self.weights_lr_multiplier = float(v)
        return self

    def setBiasLearningRateMultiplier(self, v):
        self.bias_lr_multiplier = float(v)
        return self

    def getWeightsLearningRateMultiplier(self):
        return self.weights_lr_multiplier

    def getBiasLearningRateMultiplier(self):
        return self.bias_lr_multiplier


class PoolConf(Fluent):
    """kernel/conf/PoolConf.java:20-33. Scalar setters apply to both spatial dims."""
    FIELDS = dict(method=PoolMethod.MAX, kernel_height=1, kernel_width=1, stride_height=1, stride_width=1,
                  padding_height=0, padding_width=0, global_pooling=False)

    def setKernelSize(self, k):
        self.kernel_height = self.kernel_width = k
        return self

    def setStrideSize(self, s):
        self.stride_height = self.stride_width = s
        return self

    def setPaddingSize(self, p):
        self.padding_height = self.padding_width = p
        return self

    def setMethod(self, m):
        self.method = PoolMethod.from_string(m)
        return self

    def getKernelSize(self):
        return self.kernel_height

    def getStrideSize(self):
        return self.stride_height

    def getPaddingSize(self):
        return self.padding_height

    def setGlobal(self, flag):
        self.global_pooling = bool(flag)
        return self

    def isGlobal(self):
        return self.global_pooling


class BatchNormConf(Fluent):
    """kernel/conf/BatchNormConf.java:24-39."""
    FIELDS = dict(epsilon=1e-5, fraction=0.9, global_statistics=True,
                  estimated_mean_and_variance_type=BatchNormEstimatedMeanAndVarianceType.FIXED,
                  weight_initialiser=None, bias_initialiser=None, axis=1,
                  weights_lr_multiplier=1.0, bias_lr_multiplier=1.0)
    ALIASES = {"moving_average_fraction": "fraction", "use_global_statistics": "global_statistics"}

    def __init__(self, **kw):
        super().__init__(**kw)
        self.weight_initialiser = self.weight_initialiser or InitialiserConf(value=1.0)
        self.bias_initialiser = self.bias_initialiser or InitialiserConf(value=0.0)

    def setBias(self, flag):
        """Accepted for the reference's API; the shift term is always a model variable here (as in its kernels)."""
        return self

    def hasBias(self):
        return True

    # learning-rate multipliers under the reference's names
    def setWeightsLearningRateMultiplier(self, v):
        self.weights_lr_multiplier = float(v)
        return self

    def setBiasLearningRateMultiplier(self, v):
        self.bias_lr_multiplier = float(v)
        return self

    def getWeightsLearningRateMultiplier(self):
        return self.weights_lr_multiplier

    def getBiasLearningRateMultiplier(self):
        return self.bias_lr_multiplier


class InnerProductConf(Fluent):
    """kernel/conf/InnerProductConf.java:17-23."""
    FIELDS = dict(number_of_outputs=1, bias=True, axis=1,
                  weight_initialiser=None, bias_initialiser=None,
                  weights_lr_multiplier=1.0, bias_lr_multiplier=1.0)

    def __init__(self, **kw):
        super().__init__(**kw)
        self.weight_initialiser = self.weight_initialiser or InitialiserConf()
        self.bias_initialiser = self.bias_initialiser or InitialiserConf()

    def setBias(self, flag):
        self.bias = bool(flag)
        return self

    def hasBias(self):
        return self.bias

    def numberOfOutputs(self):
        return self.number_of_outputs

    # learning-rate multipliers under the reference's names
    def setWeightsLearningRateMultiplier(self, v):
        self.weights_lr_multiplier = float(v)
        return self

    def setBiasLearningRateMultiplier(self, v):
        self.bias_lr_multiplier = float(v)
        return self

    def getWeightsLearningRateMultiplier(self):
        return self.weights_lr_multiplier

    def getBiasLearningRateMultiplier(self):
        return self.bias_lr_multiplier


class DropoutConf(Fluent):
    """kernel/conf/DropoutConf.java:8 — ratio = probability of dropping a unit."""
    FIELDS = dict(ratio=0.5)


class ReLUConf(Fluent):
    """kernel/conf/ReLUConf.java:17-20."""
    FIELDS = dict(negative_slope=0.0, activation_mode=ActivationMode.RELU, ceiling=0.0)

    def setReLUCeiling(self, ceiling):
        self.ceiling = float(ceiling)
        return self

    def getReLUCeiling(self):
        return self.ceiling


class SoftMaxConf(Fluent):
    FIELDS = dict(axis=1)


class LossConf(Fluent):
    """kernel/conf/LossConf.java:11-13."""
    FIELDS = dict(ignored_label_value=-1, mode=NormalisationMode.BATCH)


class AccuracyConf(Fluent):
    """kernel/conf/AccuracyConf.java:9-12."""
    FIELDS = dict(axis=1, top_k=1, ignored_label_value=-1)


class ClassifyConf(Fluent):
    FIELDS = dict(axis=1)


class ElementWiseOpConf(Fluent):
    """kernel/conf/ElementWiseOpConf.java — SUM with per-input coefficients is the only wired mode."""
    FIELDS = dict(type=ElementWiseOpType.SUM, coefficients=None)

    def getCoefficient(self, i):
        return 1.0 if not self.coefficients else float(self.coefficients[i])

    def numberOfCoefficients(self):
        return 0 if self.coefficients is None else len(self.coefficients)

    def resizeCoefficients(self, length):
        """Grow the coefficient list to `length` entries, new ones 1 (ElementWiseOpConf.java:39-60)."""
        cur = list(self.coefficients or [])
        self.coefficients = cur[:length] + [1.0] * max(0, length - len(cur))


class ConcatConf(Fluent):
    """kernel/conf/ConcatConf.java:13-14."""
    FIELDS = dict(axis=1, offset=0)


class DataTransformConf(Fluent):
    """kernel/conf/DataTransformConf.java:21-32."""
    FIELDS = dict(crop_size=0, scale_factor=1.0, mirror=False, mean_image_filename=None, mean_pixel_values=None,
                  subtract_mean=False)
    ALIASES = {"mean_pixels": "mean_pixel_values", "mean_image": "mean_image_filename"}

    def setMeanPixelValues(self, *v):
        self.mean_pixel_values = [float(x) for x in (v[0] if len(v) == 1 and hasattr(v[0], "__len__") else v)]
        self.subtract_mean = True
        return self

    def setMeanImageFilename(self, f):
        self.mean_image_filename = f
        self.subtract_mean = True
        return self

    def hasMeanPixel(self):
        return self.mean_pixel_values is not None

    def subtractMean(self):
        return self.mean_image_filename is not None or self.mean_pixel_values is not None


class LRNConf(Fluent):
    """kernel/conf/LRNConf.java:34-39."""
    FIELDS = dict(local_size=5, alpha=1.0, beta=0.75, k=1.0, region=NormalisationRegion.ACROSS_CHANNELS)

    def setSize(self, size):
        self.local_size = int(size)
        return self

    def getSize(self):
        return self.local_size

    def setKappa(self, kappa):
        self.k = float(kappa)
        return self

    def getKappa(self):
        return self.k

    def setNormalisationRegion(self, region):
        self.region = NormalisationRegion.from_string(region)
        return self

    def getNormalisationRegion(self):
        return self.region


class MatFactConf(Fluent):
    """kernel/conf/MatFactConf.java:19-29."""
    FIELDS = dict(number_of_latent_variables=10, number_of_rows=0, number_of_columns=0, learning_rate_eta0=0.001,
                  lambda_=0.05, model_variable_initialiser=None)
    ALIASES = {"lambda": "lambda_"}

    def numberOfLatentVariables(self):
        return self.number_of_latent_variables

    def numberOfRows(self):
        return self.number_of_rows

    def numberOfColumns(self):
        return self.number_of_columns


class NoopConf(Fluent):
    FIELDS = dict(axis=1)


# --------------------------------------------------------------------------------------------
# Solver
# --------------------------------------------------------------------------------------------

class SolverConf(Fluent):
    """Learning-rate schedule, momentum, regularisation and averaging constants.

    Defaults follow kernel/conf/SolverConf.java:63-107; the schedule arithmetic follows the native
    evaluation in clib-multigpu/solverconfiguration.c:116-162, including the ``copy`` signal that is
    raised whenever a multistep boundary is crossed (used by SMA to overwrite replicas with the
    central average model, synch/sma.c:185-228).
    """
    FIELDS = dict(learning_rate_decay_policy=LearningRateDecayPolicy.INV, base_learning_rate=0.0,
                  gamma=0.0, power=0.0, momentum=0.0, momentum_method=MomentumMethod.POLYAK,
                  weight_decay=0.0, regularisation_type=Regularisation.L2, clip_gradient_threshold=-1.0,
                  step_size=0, step_values=None, step_unit=TrainingUnit.TASKS, warmup_steps=0,
                  alpha=0.5, tau=1, base_model_momentum=0.0,
                  min_learning_rate=0.0, max_learning_rate=0.0, learning_rate_increment=0.0,
                  super_convergence=False, min_momentum=0.0, max_momentum=0.0, momentum_increment=0.0)
    ALIASES = {"learning_rate": "base_learning_rate", "learning_rate_step_unit": "step_unit",
               "regularization_type": "regularisation_type", "stepsize": "step_size"}

    def __init__(self, **kw):
        super().__init__(**kw)
        self._step = 0          # multistep cursor (solverconfiguration.c `step`)
        self._copy = False      # raised when the rate drops; consumed by the synchroniser
        self._tasks_per_epoch = 1

    def setLearningRateDecayPolicy(self, p):
        self.learning_rate_decay_policy = LearningRateDecayPolicy.from_string(p)
        return self

    def setStepValues(self, *v):
        vals = v[0] if len(v) == 1 and hasattr(v[0], "__len__") else v
        self.step_values = [int(x) for x in vals]
        return self

    def setMomentumMethod(self, m):
        self.momentum_method = MomentumMethod.from_string(m)
        return self

    def set_tasks_per_epoch(self, n):
        """Step values/sizes given in epochs are converted with this factor (SolverConf.java converts once)."""
        self._tasks_per_epoch = max(1, int(n))
        return self

    def _in_tasks(self, v):
        return v * self._tasks_per_epoch if self.step_unit == TrainingUnit.EPOCHS else v

    def steps_in_tasks(self) -> List[int]:
        return [self._in_tasks(v) for v in (self.step_values or [])]

    def reset(self):
        self._step, self._copy = 0, False

    def consume_copy_signal(self) -> bool:
        c, self._copy = self._copy, False
        return c

    def setCurrentStep(self, step: int):
        """Position in the multi-step schedule (SolverConf.java:209-212), e.g. after a resume."""
        self._step = int(step)
        return self

    def getCurrentStep(self):
        return self._step

    def getStepValuesToString(self):
        v = self.steps_in_tasks() if hasattr(self, "steps_in_tasks") else []
        return None if not v else ",".join(str(int(x)) for x in v)

    def GPURegister(self):
        """The reference pushes the solver's constants to its native library here; the device reads them from the task
        parameter block, so there is nothing to register."""
        return None

    def toString(self):
        return self.dump() if hasattr(self, "dump") else repr(self)

    def setModelConf(self, parent):
        self.parent = parent
        return self

    def learning_rate(self, task: int) -> float:
        """Learning rate used by task number ``task`` (0-based). Stateful for MULTISTEP/LSR like the reference."""
        p = self.learning_rate_decay_policy
        lr = float(self.base_learning_rate)
        if p == LearningRateDecayPolicy.FIXED:
            return lr
        if p == LearningRateDecayPolicy.INV:
            return lr * math.pow(1.0 + self.gamma * (task + 1), -self.power)
        if p == LearningRateDecayPolicy.STEP:
            size = self._in_tasks(self.step_size)
            if size <= 0:
                raise ValueError("error: STEP policy needs a positive step size")
            return lr * math.pow(self.gamma, math.floor((task + 1) / size))
        if p in (LearningRateDecayPolicy.MULTISTEP, LearningRateDecayPolicy.LSR):
            if self.step_values is None:
                raise ValueError("error: step values are not set")
            if p == LearningRateDecayPolicy.LSR:
                warm = self._in_tasks(self.warmup_steps)
                if warm <= 0:
                    raise ValueError("error: invalid number of warm-up steps")
                if task < warm:
                    return lr * task / warm
            steps = self.steps_in_tasks()
            if self._step < len(steps) and (task + 1) >= steps[self._step]:
                self._step += 1
                self._copy = True
            return lr * math.pow(self.gamma, self._step)
        if p == LearningRateDecayPolicy.EXP:
            return lr * math.pow(self.gamma, task + 1)
        if p == LearningRateDecayPolicy.CLR:
            # Triangular cyclical rate; the reference registers the parameters and then throws
            # (SolverConf.java:390-405) - here the schedule is actually evaluated.
            size = max(1, self._in_tasks(self.step_size))
            cycle = math.floor(1 + task / (2 * size))
            x = abs(task / size - 2 * cycle + 1)
            return self.min_learning_rate + (self.max_learning_rate - self.min_learning_rate) * max(0.0, 1 - x)
        raise ValueError("error: invalid learning rate decay policy type")

    def momentum_at(self, task: int) -> float:
        if self.learning_rate_decay_policy == LearningRateDecayPolicy.CLR and self.super_convergence:
            size = max(1, self._in_tasks(self.step_size))
            cycle = math.floor(1 + task / (2 * size))
            x = abs(task / size - 2 * cycle + 1)
            return self.max_momentum - (self.max_momentum - self.min_momentum) * max(0.0, 1 - x)
        return float(self.momentum)

    OPTIONS = {
        "--learning-rate-decay-policy": ("learning_rate_decay_policy", LearningRateDecayPolicy.from_string),
        "--learning-rate": ("base_learning_rate", float), "--gamma": ("gamma", float), "--power": ("power", float),
        "--momentum": ("momentum", float), "--momentum-method": ("momentum_method", MomentumMethod.from_string),
        "--weight-decay": ("weight_decay", float),
        "--regularisation-type": ("regularisation_type", Regularisation.from_string),
        "--clip-gradient-threshold": ("clip_gradient_threshold", float), "--step-size": ("step_size", int),
        "--step-values": ("step_values", lambda s: [int(x) for x in str(s).split(",") if x != ""]),
        "--warmup-steps": ("warmup_steps", int),
        "--learning-rate-step-unit": ("step_unit", TrainingUnit.from_string),
        "--alpha": ("alpha", float), "--tau": ("tau", int), "--base-model-momentum": ("base_model_momentum", float),
        "--min-learning-rate": ("min_learning_rate", float), "--max-learning-rate": ("max_learning_rate", float),
        "--learning-rate-increment": ("learning_rate_increment", float),
        "--super-convergence": ("super_convergence", lambda s: str(s).lower() == "true"),
        "--min-momentum": ("min_momentum", float), "--max-momentum": ("max_momentum", float),
        "--momentum-increment": ("momentum_increment", float),
    }


def _parse_bool(s):
    if isinstance(s, bool):
        return s
    k = str(s).strip().lower()
    if k in ("true", "1", "yes"):
        return True
    if k in ("false", "0", "no"):
        return False
    raise ValueError(f"error: invalid boolean value: {s}")


def _parse_devices(s):
    if isinstance(s, (list, tuple)):
        return [int(x) for x in s]
    return [int(x) for x in str(s).split(",") if x != ""]


class _OptionHolder(Fluent):
    OPTIONS: Dict[str, tuple] = {}

    def parse(self, arg: str, value) -> bool:
        """Apply one ``--flag value`` pair; returns False if the flag is not ours (SystemConf.java:597-786)."""
        spec = self.OPTIONS.get(arg)
        if spec is None:
            return False
        field, conv = spec
        setattr(self, field, conv(value))
        return True


class SystemConf(_OptionHolder):
    """System-wide flags; one instance per process (``SystemConf.getInstance()``).

    The 37 options and their defaults are those of SystemConf.java:134-235.  ``gpu_devices`` lists the
    devices of ONE process in the reference; here each process drives one GPU and the list names the
    world (ranks are spawned with ``torch.distributed.run``), so ``numberOfGPUs()`` is the world size.
    """
    FIELDS = dict(cpu=True, gpu=False, gpu_devices=[0], checkpoint_directory=None, model_directory=None,
                  number_of_workers=1, number_of_cpu_models=1, number_of_gpu_models=1,
                  number_of_result_slots=2048, scheduling_policy=SchedulingPolicy.FIFO,
                  synchronisation_model=SynchronisationModel.BSP, replication_model=ReplicationModel.SRSW,
                  readers_per_model=1, data_buffer_size=1 << 20, number_of_buffers=256, use_direct_buffers=True,
                  number_of_gpu_streams=1, number_of_callback_handlers=1, number_of_task_handlers=1,
                  number_of_file_handlers=1, display_interval=1, display_interval_unit=TrainingUnit.TASKS,
                  display_accumulated_loss=False, checkpoint_interval=0, checkpoint_interval_unit=TrainingUnit.TASKS,
                  queue_measurements=False, file_partition_size=1 << 30, task_queue_size=32,
                  random_seed=123456789, reuse_memory=False, mapped_partitions_window=4, monitor_interval=1000,
                  tee_measurements=True, autotune_models=False, autotune_threshold=0.1, autotune_interval=1,
                  direct_scheduling=False, core_mapper_offset=1, use_cuda_graphs=True, use_tensor_cores=True,
                  fused_sync=True, overlap_sync=True, operator_branches=True, nvls_sync=False, sync_timeout=5.0, native_scheduler=True, task_timeout=60.0, gradient_buckets=0, run_ahead=2, trace_level=0, debug_canaries=False, debug_checksums=False)
    ALIASES = {"gpu_models": "number_of_gpu_models", "gpu_streams": "number_of_gpu_streams"}

    OPTIONS = {
        "--cpu": ("cpu", _parse_bool), "--gpu": ("gpu", _parse_bool), "--gpu-devices": ("gpu_devices", _parse_devices),
        "--checkpoint-directory": ("checkpoint_directory", str), "--model-directory": ("model_directory", str),
        "--number-of-workers": ("number_of_workers", int), "--number-of-cpu-models": ("number_of_cpu_models", int),
        "--number-of-gpu-models": ("number_of_gpu_models", int),
        "--number-of-result-slots": ("number_of_result_slots", int),
        "--scheduling-policy": ("scheduling_policy", SchedulingPolicy.from_string),
        "--synchronisation-model": ("synchronisation_model", SynchronisationModel.from_string),
        "--replication-model": ("replication_model", ReplicationModel.from_string),
        "--readers-per-model": ("readers_per_model", int), "--data-buffer-size": ("data_buffer_size", int),
        "--number-of-buffers": ("number_of_buffers", int), "--use-direct-buffers": ("use_direct_buffers", _parse_bool),
        "--number-of-gpu-streams": ("number_of_gpu_streams", int),
        "--number-of-callback-handlers": ("number_of_callback_handlers", int),
        "--number-of-task-handlers": ("number_of_task_handlers", int),
        "--number-of-file-handlers": ("number_of_file_handlers", int),
        "--display-interval": ("display_interval", int),
        "--display-interval-unit": ("display_interval_unit", TrainingUnit.from_string),
        "--display-accumulated-loss": ("display_accumulated_loss", _parse_bool),
        "--checkpoint-interval": ("checkpoint_interval", int),
        "--checkpoint-interval-unit": ("checkpoint_interval_unit", TrainingUnit.from_string),
        "--queue-measurements": ("queue_measurements", _parse_bool),
        "--file-partition-size": ("file_partition_size", int), "--task-queue-size": ("task_queue_size", int),
        "--random-seed": ("random_seed", int), "--reuse-memory": ("reuse_memory", _parse_bool),
        "--mapped-partitions-window": ("mapped_partitions_window", int), "--monitor-interval": ("monitor_interval", int),
        "--tee-measurements": ("tee_measurements", _parse_bool), "--autotune-models": ("autotune_models", _parse_bool),
        "--autotune-threshold": ("autotune_threshold", float), "--autotune-interval": ("autotune_interval", int),
        "--direct-scheduling": ("direct_scheduling", _parse_bool),
        "--use-cuda-graphs": ("use_cuda_graphs", _parse_bool),
        "--use-tensor-cores": ("use_tensor_cores", _parse_bool), "--fused-sync": ("fused_sync", _parse_bool), "--overlap-sync": ("overlap_sync", _parse_bool), "--operator-branches": ("operator_branches", _parse_bool), "--nvls-sync": ("nvls_sync", _parse_bool),
        "--sync-timeout": ("sync_timeout", float), "--native-scheduler": ("native_scheduler", _parse_bool),
        "--task-timeout": ("task_timeout", float), "--gradient-buckets": ("gradient_buckets", int), "--run-ahead": ("run_ahead", int), "--trace-level": ("trace_level", int), "--debug-canaries": ("debug_canaries", _parse_bool), "--debug-checksums": ("debug_checksums", _parse_bool),
    }

    _instance: Optional["SystemConf"] = None

    @classmethod
    def getInstance(cls) -> "SystemConf":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    get_instance = getInstance

    @classmethod
    def reset(cls) -> "SystemConf":
        cls._instance = cls()
        return cls._instance

    def setGPU(self, flag):
        self.gpu = bool(flag)
        return self

    def setCPU(self, flag):
        self.cpu = bool(flag)
        return self

    def setGPUDevices(self, *ids):
        self.gpu_devices = _parse_devices(ids[0] if len(ids) == 1 and not isinstance(ids[0], int) else ids)
        return self

    def numberOfGPUs(self):
        return len(self.gpu_devices)

    # ---- the reference's setter names that differ from the generated set<Field> ones (SystemConf.java:237-780) ----
    def _set(self, field, value):
        setattr(self, field, value)
        return self

    def setNumberOfWorkerThreads(self, n): return self._set("number_of_workers", int(n))
    def setNumberOfCPUModelReplicas(self, n): return self._set("number_of_cpu_models", int(n))
    def setNumberOfGPUModelReplicas(self, n): return self._set("number_of_gpu_models", int(n))
    def setNumberOfReadersPerModel(self, n): return self._set("readers_per_model", int(n))
    def setNumberOfGPUCallbackHandlers(self, n): return self._set("number_of_callback_handlers", int(n))
    def setNumberOfGPUTaskHandlers(self, n): return self._set("number_of_task_handlers", int(n))
    def setPerformanceMonitorInterval(self, ms): return self._set("monitor_interval", int(ms))
    def setTaskQueueSizeLimit(self, n): return self._set("task_queue_size", int(n))
    def setVariableBufferSize(self, nbytes): return self._set("data_buffer_size", int(nbytes))
    def setMaxNumberOfMappedPartitions(self, n): return self._set("mapped_partitions_window", int(n))
    def allowMemoryReuse(self, flag): return self._set("reuse_memory", bool(flag))
    def autotuneModels(self, flag): return self._set("autotune_models", bool(flag))
    def displayAccumulatedLossValue(self, flag): return self._set("display_accumulated_loss", bool(flag))
    def queueMeasurements(self, flag): return self._set("queue_measurements", bool(flag))
    def useDirectBuffers(self, flag): return self._set("use_direct_buffers", bool(flag))

    # ---- and its getter names (SystemConf.java) ----
    def numberOfWorkerThreads(self): return self.number_of_workers
    def numberOfCPUModelReplicas(self): return self.number_of_cpu_models
    def numberOfGPUModelReplicas(self): return self.number_of_gpu_models
    def numberOfGPUStreams(self): return self.number_of_gpu_streams
    def numberOfGPUCallbackHandlers(self): return self.number_of_callback_handlers
    def numberOfGPUTaskHandlers(self): return self.number_of_task_handlers
    def numberOfReadersPerModel(self): return self.readers_per_model
    def numberOfResultSlots(self): return self.number_of_result_slots
    def numberOfBuffers(self): return self.number_of_buffers
    def numberOfFileHandlers(self): return self.number_of_file_handlers
    def maxNumberOfMappedPartitions(self): return self.mapped_partitions_window
    def getPerformanceMonitorInterval(self): return self.monitor_interval
    def getTaskQueueSizeLimit(self): return self.task_queue_size
    def getVariableBufferSize(self): return self.data_buffer_size
    def teeMeasurements(self): return self.tee_measurements
    def tryReuseMemory(self): return self.reuse_memory
    def getExecutionMode(self): return self.executionMode()
    def getOptions(self): return dict(self.OPTIONS)

    def getPageSize(self):
        import mmap
        return mmap.PAGESIZE

    def getHomeDirectory(self):
        """`CROSSBOW_HOME` in the reference (mandatory there); here the directory of the package unless set."""
        import os
        return getattr(self, "_home", None) or os.environ.get("CROSSBOW_HOME") or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def setHomeDirectory(self, d):
        self._home = d
        return self

    def getCoreMapper(self):
        from .utils.coremap import CoreMapper
        return CoreMapper()

    def isHybrid(self):
        return self.cpu and self.gpu

    def executionMode(self):
        from .types import ExecutionMode
        return ExecutionMode.HYBRID if self.isHybrid() else (ExecutionMode.GPU if self.gpu else ExecutionMode.CPU)


class ModelConf(_OptionHolder):
    """Per-model flags (ModelConf.java:53-83): work per clock, slack, batch size, splits, test interval,
    update model, data sets and the solver configuration."""
    FIELDS = dict(wpc=1, wpc_unit=TrainingUnit.TASKS, slack=0, batch_size=32, splits=1, test_interval=1,
                  test_interval_unit=TrainingUnit.EPOCHS, update_model=UpdateModel.DEFAULT)

    OPTIONS = {
        "--wpc": ("wpc", int), "--wpc-unit": ("wpc_unit", TrainingUnit.from_string), "--slack": ("slack", int),
        "--batch-size": ("batch_size", int), "--splits": ("splits", int), "--test-interval": ("test_interval", int),
        "--test-interval-unit": ("test_interval_unit", TrainingUnit.from_string),
        "--update-model": ("update_model", UpdateModel.from_string),
    }

    _instance: Optional["ModelConf"] = None

    def __init__(self, **kw):
        super().__init__(**kw)
        self.solver_conf = SolverConf()
        self.datasets = [None, None]   # [train, test]

    @classmethod
    def getInstance(cls) -> "ModelConf":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    get_instance = getInstance

    @classmethod
    def reset(cls) -> "ModelConf":
        cls._instance = cls()
        return cls._instance

    def getSolverConf(self) -> SolverConf:
        return self.solver_conf

    def setSolverConf(self, s: SolverConf):
        self.solver_conf = s
        return self

    def setUpdateModel(self, m):
        self.update_model = UpdateModel.from_string(m)
        return self

    def setDataset(self, phase, dataset):
        self.datasets[int(phase)] = dataset
        return self

    def getDataset(self, phase):
        return self.datasets[int(phase)]

    # reference names (ModelConf.java:150-214)
    def setTrainingDataset(self, dataset):
        return self.setDataset(Phase.TRAIN, dataset)

    def setValidationDataset(self, dataset):
        return self.setDataset(Phase.CHECK, dataset)

    def setNumberOfSplits(self, n):
        self.splits = int(n)
        return self

    def numberOfSplits(self):
        return self.splits

    def getTrainingDataset(self):
        return self.getDataset(Phase.TRAIN)

    def getValidationDataset(self):
        return self.getDataset(Phase.CHECK)

    def getOptions(self):
        return dict(self.OPTIONS)

    def getInputShape(self, phase=Phase.TRAIN):
        ds = self.getDataset(phase)
        return None if ds is None else [self.batch_size] + list(ds.example_shape)

    def getTaskSize(self, phase=Phase.TRAIN):
        """Bytes of one task's examples."""
        ds = self.getDataset(phase)
        return 0 if ds is None else int(ds.batch_bytes())

    def numberOfTestTasks(self):
        return self.numberOfTasksPerEpoch(Phase.CHECK) if self.getDataset(Phase.CHECK) is not None else 0

    def getDatasetType(self, phase=Phase.TRAIN):
        ds = self.getDataset(phase)
        return None if ds is None else type(ds).__name__

    def isLightWeight(self, phase=Phase.TRAIN):
        return self.getDatasetType(phase) == "LightDataset"

    def init(self):
        """The reference opens its data sets here; data sets open themselves when constructed."""
        return self

    def setBatchSize(self, n):
        self.batch_size = int(n)
        return self

    def parse(self, arg, value):
        if super().parse(arg, value):
            return True
        spec = SolverConf.OPTIONS.get(arg)
        if spec is None:
            return False
        setattr(self.solver_conf, spec[0], spec[1](value))
        return True

    def numberOfTasksPerEpoch(self, phase=0) -> int:
        """ModelConf.java:222-230: examples must be a multiple of the batch size."""
        ds = self.datasets[int(phase)]
        if ds is None:
            raise ValueError("error: dataset is not set")
        n = ds.number_of_examples()
        if n % self.batch_size != 0:
            raise ValueError(f"error: number of examples ({n}) is not a multiple of the batch size ({self.batch_size})")
        return n // self.batch_size

    def wpc_in_tasks(self) -> int:
        if self.wpc_unit == TrainingUnit.EPOCHS:
            return self.wpc * self.numberOfTasksPerEpoch(0)
        return self.wpc
