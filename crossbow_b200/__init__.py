"""crossbow_b200: a Blackwell-native small-batch multi-replica training framework.

Public surface: graph builder (``DataflowNode``, ``Operator``, ``SubGraph``, ``Dataflow``), operator
classes and their ``Conf`` objects, ``SystemConf`` / ``ModelConf`` / ``SolverConf``, ``ExecutionContext``
and the model zoo under ``crossbow_b200.models``.
"""
import os as _os

# Every replica issues its work on two streams of its own (the task and its weight-gradient branch), next to the
# synchronisation and copy streams.  The driver maps streams onto 8 hardware queues unless told otherwise, and streams that
# share a queue wait for each other: with five replicas per GPU ResNet-32 ran at 88 K images/s instead of 125 K.  The
# setting is read when the process creates its CUDA context, so it has to be in place before the first CUDA call; a value
# the user has set is left alone.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

from .types import *  # noqa: F401,F403
from .conf import *  # noqa: F401,F403
from .model import Model, Shape, Variable
from .graph import DataflowNode, Operator, SubGraph, Dataflow, append_gradients, shallow_copy_forward
from .kernels import *  # noqa: F401,F403

__version__ = "0.1.0"
