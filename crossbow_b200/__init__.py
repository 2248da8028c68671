"""crossbow_b200: a Blackwell-native small-batch multi-replica training framework.

Public surface: graph builder (``DataflowNode``, ``Operator``, ``SubGraph``, ``Dataflow``), operator
classes and their ``Conf`` objects, ``SystemConf`` / ``ModelConf`` / ``SolverConf``, ``ExecutionContext``
and the model zoo under ``crossbow_b200.models``.
"""
from .types import *  # noqa: F401,F403
from .conf import *  # noqa: F401,F403
from .model import Model, Shape, Variable
from .graph import DataflowNode, Operator, SubGraph, Dataflow, append_gradients, shallow_copy_forward
from .kernels import *  # noqa: F401,F403

__version__ = "0.1.0"
