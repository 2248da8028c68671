"""Dataflow-graph builder API: ``DataflowNode`` / ``Operator`` / ``SubGraph`` / ``Dataflow``.

Usage mirrors the reference (README.md:100-137)::

    conv = DataflowNode(Operator("Conv", Conv(conv_conf)))
    relu = DataflowNode(Operator("ReLU", ReLU(ReLUConf())))
    conv.connectTo(relu).connectTo(...)
    grad = DataflowNode(Operator("ReLUGradient", ReLUGradient(conf)).setPeer(relu.getOperator()))
    df = Dataflow(SubGraph(conv)).setPhase(Phase.TRAIN)

Reference behaviour reproduced here: edges + depth-first topological order (DataflowNode.java:97-106,
158-178; SubGraph.java:77-98), shape propagation and model-variable registration at ``init``
(SubGraph.java:293-359), gradient peers (Operator.java:117-121), ``shallowCopy`` nodes that share the
operator for the test graph (DataflowNode.java:230-232), DOT export (SubGraph.java:633-656).

New: ``append_gradients(head)`` derives the whole gradient chain (one gradient node per forward node in
reverse topological order, a SUM merge node wherever a forward output has several consumers, and the
optimiser node) so model builders do not have to spell it out by hand as the reference's apps do.
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional

from .model import Model, Shape
from .types import Phase


class Operator:
    _ids = itertools.count()

    def __init__(self, name: str, kernel):
        self.id = -1                     # assigned at SubGraph.init in topological order
        self.uid = next(Operator._ids)   # creation order; stable identity across shallow copies
        self.name = name
        self.kernel = kernel
        self.peer: Optional["Operator"] = None
        self.input_shapes: List[Shape] = []
        self.output_shape: Optional[Shape] = None
        self.initialised = False
        kernel.operator = self

    def setPeer(self, peer: "Operator"):
        self.peer = peer
        return self

    def getPeer(self):
        return self.peer

    def getKernel(self):
        return self.kernel

    def getName(self):
        return self.name

    def getId(self):
        return self.id

    def isGradient(self):
        return self.kernel.is_gradient

    def isLossKernel(self):
        return self.kernel.is_loss

    def isAccuracyKernel(self):
        return self.kernel.is_accuracy

    def isDataTransformationKernel(self):
        return self.kernel.is_data_transform

    def getOutputShape(self):
        return self.output_shape

    def __repr__(self):
        return f"{self.name}#{self.id}"


class DataflowNode:
    def __init__(self, op: Operator):
        self.op = op
        self.next: List["DataflowNode"] = []
        self.prev: List["DataflowNode"] = []
        self.label = 0  # stream-branch label; the reference's labelling pass is disabled, factor stays 1

    def getOperator(self):
        return self.op

    def connectTo(self, node: "DataflowNode") -> "DataflowNode":
        """Add edge self -> node and return ``node`` so calls can be chained."""
        self.next.append(node)
        node.prev.append(self)
        return node

    connect_to = connectTo

    def shallowCopy(self) -> "DataflowNode":
        """New node around the SAME operator (shares variables); used to build the test graph."""
        return DataflowNode(self.op)

    shallow_copy = shallowCopy

    def isMostUpstream(self):
        return not self.prev

    def isMostDownstream(self):
        return not self.next

    # accessors under the reference's names (DataflowNode.java)
    def getNextList(self):
        return list(self.next)

    def getPreviousList(self):
        return list(self.prev)

    def getNextOperators(self):
        return [n.op for n in self.next]

    def getPreviousOperators(self):
        return [n.op for n in self.prev]

    def getLabel(self):
        return self.label

    def setLabel(self, label):
        self.label = int(label)
        return self

    def getOrder(self):
        """Position in the topological order of the sub-graph that owns the node (-1 before it is part of one)."""
        return getattr(self, "order_index", -1)

    def __repr__(self):
        return f"Node({self.op})"


class SubGraph:
    def __init__(self, head: DataflowNode):
        self.head = head
        self.id = 0
        self.next_graph: Optional["SubGraph"] = None
        self.order: List[DataflowNode] = self._topological_sort(head)
        self.model: Optional[Model] = None
        self.phase = Phase.TRAIN

    @staticmethod
    def _topological_sort(head: DataflowNode) -> List[DataflowNode]:
        seen, out = set(), []

        def visit(n: DataflowNode):
            if id(n) in seen:
                return
            seen.add(id(n))
            for m in n.next:
                visit(m)
            out.append(n)

        # iterative DFS would be safer for very deep graphs; raise the limit instead (ResNet-152 ~ 1.2k nodes)
        import sys
        lim = sys.getrecursionlimit()
        sys.setrecursionlimit(max(lim, 20000))
        try:
            visit(head)
        finally:
            sys.setrecursionlimit(lim)
        out.reverse()
        return out

    def connectTo(self, g: "SubGraph"):
        """Chain sub-graphs: the output batch of this graph feeds ``g`` on the same replica (SubGraph.java:230-234)."""
        self.next_graph = g
        g.prev_graph = self
        return g

    def nodes(self):
        return list(self.order)

    def forward_nodes(self):
        return [n for n in self.order if not n.op.kernel.is_gradient and not n.op.kernel.is_optimiser]

    def numberOfOperators(self):
        return len(self.order)

    cardinality = numberOfOperators

    # accessors under the reference's names (SubGraph.java)
    def getId(self):
        return self.id

    def getName(self):
        return f"SubGraph #{self.id}"

    def getDataflowNode(self):
        return self.head

    def getNext(self):
        return self.next_graph

    def getPrevious(self):
        return getattr(self, "prev_graph", None)

    def setPrevious(self, g):
        self.prev_graph = g
        return self

    def isMostUpstream(self):
        return self.getPrevious() is None

    def getBranchFactor(self):
        return 1                      # the reference's labelling pass is disabled: one stream branch per learner

    def getInputShape(self):
        return getattr(self, "input_shape", None)

    def getOutputShape(self):
        last = [n for n in self.forward_nodes() if n.op.getOutputShape() is not None]
        return last[-1].op.getOutputShape() if last else None

    def dump(self) -> str:
        return f"=== [{self.getName()}: {self.numberOfOperators()} operators] ===\n" + " -> ".join(str(n.op) for n in self.order)

    def export(self) -> str:
        return self.exportDot()

    def init(self, input_shape: Shape, label_shape: Shape, model: Model, first_id=0):
        """Assign operator ids, propagate shapes and register model variables (once per operator)."""
        self.model = model
        self.input_shape = input_shape
        for i, n in enumerate(self.order):
            n.order_index = i
        next_id = first_id
        for n in self.order:
            op = n.op
            if op.id < 0:
                op.id = next_id
                next_id += 1
        for n in self.order:
            op = n.op
            if op.kernel.is_gradient or op.kernel.is_optimiser:
                if op.kernel.is_gradient and op.peer is None:
                    raise ValueError(f"error: gradient operator {op.name} has no peer")
                ins = [p.op.output_shape for p in n.prev]
                op.input_shapes = ins
                if op.kernel.is_gradient:
                    peer_in = op.peer.input_shapes
                    op.output_shape = peer_in[0].copy() if peer_in else None
                continue
            ins = [p.op.output_shape.copy() for p in n.prev if not p.op.kernel.is_gradient] or [input_shape.copy()]
            if op.initialised:
                # shallow copy of an operator already set up by the training graph
                if [s.dims[1:] for s in op.input_shapes] != [s.dims[1:] for s in ins]:
                    raise ValueError(f"error: operator {op} is shared by graphs with different input shapes")
                continue
            op.input_shapes = ins
            op.output_shape = op.kernel.setup(ins, model, label_shape)
            op.initialised = True
        return next_id

    def getLossNode(self):
        for n in self.order:
            if n.op.kernel.is_loss:
                return n
        return None

    def getAccuracyNode(self):
        for n in self.order:
            if n.op.kernel.is_accuracy:
                return n
        return None

    def getOptimiserNode(self):
        for n in self.order:
            if n.op.kernel.is_optimiser:
                return n
        return None

    def is_training_graph(self):
        return any(n.op.kernel.is_gradient for n in self.order)

    def exportDot(self) -> str:
        lines = ["digraph dataflow {"]
        ids = {id(n): i for i, n in enumerate(self.order)}
        for n in self.order:
            lines.append(f'  n{ids[id(n)]} [label="{n.op.name} ({n.op.id})"];')
        for n in self.order:
            for m in n.next:
                lines.append(f"  n{ids[id(n)]} -> n{ids[id(m)]};")
        lines.append("}")
        return "\n".join(lines)

    export_dot = exportDot

    def dumpMemoryRequirements(self) -> str:
        """Per-operator output/model/local memory table (SubGraph.java:658-698)."""
        rows = ["operator                      output(B)    model(B)"]
        for n in self.order:
            k = n.op.kernel
            out_b = 4 * n.op.output_shape.countAllElements() if n.op.output_shape is not None else 0
            mod_b = 4 * sum(v.elements() for v in k.variables)
            rows.append(f"{n.op.name + '#' + str(n.op.id):<28s} {out_b:>10d} {mod_b:>11d}")
        return "\n".join(rows)


class Dataflow:
    def __init__(self, graph: SubGraph):
        self.graph = graph
        self.phase = Phase.TRAIN
        self.id = 0

    def setPhase(self, phase):
        self.phase = Phase(phase)
        g = self.graph
        while g is not None:
            g.phase = self.phase
            g = g.next_graph
        return self

    def getPhase(self):
        return self.phase

    def getSubGraph(self):
        return self.graph

    def subgraphs(self):
        g, out = self.graph, []
        while g is not None:
            out.append(g)
            g = g.next_graph
        return out

    def executable(self) -> SubGraph:
        """The graph a task of this dataflow runs.  A single sub-graph is returned as it is.  A chain built with
        ``SubGraph.connectTo`` is executed back to back on one replica, the output batch of a sub-graph being the input
        of the next (dispatcher/TransientTaskDispatcher.java:41-52 hands the batch on with the replica id); here the chain
        is joined once - the last forward operator of every sub-graph gets an edge to the head of the next - and lowered
        as ONE program, so the hand-over costs nothing and fusion works across the seam."""
        chain = self.subgraphs()
        if len(chain) == 1:
            return self.graph
        if getattr(self, "_joined", None) is None:
            for a, b in zip(chain, chain[1:]):
                tails = [n for n in a.order if not (n.op.kernel.is_gradient or n.op.kernel.is_optimiser or n.op.kernel.is_loss
                                                    or n.op.kernel.is_accuracy or getattr(n.op.kernel, "is_gradient_merge", False))
                         and not any(not (m.op.kernel.is_gradient or m.op.kernel.is_optimiser) for m in n.next)]
                if not tails:
                    raise ValueError(f"error: {a.getName()} has no output to feed {b.getName()}")
                if b.head not in tails[-1].next:
                    tails[-1].connectTo(b.head)
            joined = SubGraph(self.graph.head)
            joined.id, joined.phase = self.graph.id, self.phase
            self._joined = joined
        return self._joined

    def isTest(self):
        return self.phase == Phase.CHECK

    # accessors under the reference's names (Dataflow.java)
    def getId(self):
        return self.id

    def numberOfSubGraphs(self):
        return len(self.subgraphs())

    def numberOfOperators(self):
        return self.graph.numberOfOperators()

    def totalNumberOfOperators(self):
        return sum(g.numberOfOperators() for g in self.subgraphs())

    cardinality = totalNumberOfOperators

    def exportDot(self) -> str:
        return self.export()

    def dumpMemoryRequirements(self) -> str:
        return "\n".join(g.dumpMemoryRequirements() for g in self.subgraphs())

    def init(self, input_shape, label_shape, model, first_id=0):
        """Initialise the executable graph (the whole chain of sub-graphs); returns the next free operator id."""
        return self.executable().init(input_shape, label_shape, model, first_id)

    def export(self) -> str:
        return "\n".join(g.exportDot() for g in self.subgraphs())

    def dump(self) -> str:
        g = self.graph
        return f"=== [Dataflow ({self.phase.name}): {g.numberOfOperators()} operators] ===\n" + \
            " -> ".join(str(n.op) for n in g.order)


# --------------------------------------------------------------------------------------------
# Gradient-chain derivation
# --------------------------------------------------------------------------------------------

def append_gradients(head: DataflowNode, solver_conf=None, with_optimiser=True) -> DataflowNode:
    """Attach gradient nodes (+ merge nodes + optimiser) for every forward node reachable from ``head``.

    Returns the optimiser node (or the last gradient node).  Accuracy / classify nodes get no gradient.
    """
    from . import kernels as K

    fwd = [n for n in SubGraph._topological_sort(head)]
    loss = next((n for n in fwd if n.op.kernel.is_loss), None)
    if loss is None:
        raise ValueError("error: graph has no loss operator")
    grad_of: Dict[int, DataflowNode] = {}
    last = None
    for n in reversed(fwd):
        k = n.op.kernel
        if k.is_accuracy or k.is_gradient or k.is_optimiser or getattr(k, "no_gradient", False):
            continue
        if k.kind == "softmax" and any(c is loss for c in n.next):
            # the loss gradient is already w.r.t. the logits (SoftMaxLossGradient.java:117-180)
            grad_of[id(n)] = grad_of[id(loss)]
            continue
        gk = k.make_gradient()
        if gk is None:
            continue
        g = DataflowNode(Operator(n.op.name + "Gradient", gk).setPeer(n.op))
        consumers = [grad_of[id(c)] for c in n.next if id(c) in grad_of]
        if n is loss:
            n.connectTo(g)
        elif not consumers:
            continue      # dead branch (does not reach the loss)
        elif len(consumers) == 1:
            consumers[0].connectTo(g)
        else:
            from .conf import ElementWiseOpConf
            merge = DataflowNode(Operator("GradientMerge", K.ElementWiseOp(ElementWiseOpConf())))
            merge.op.kernel.no_gradient = True
            merge.op.kernel.is_gradient_merge = True
            merge.op.merge_of = n.op
            for c in consumers:
                c.connectTo(merge)
            merge.connectTo(g)
        grad_of[id(n)] = g
        last = g
    if with_optimiser:
        from .conf import ModelConf
        opt = DataflowNode(Operator("Optimiser", K.GradientDescentOptimiser(solver_conf or ModelConf.getInstance().getSolverConf())))
        last.connectTo(opt)
        return opt
    return last


def shallow_copy_forward(head: DataflowNode, keep=lambda k: True) -> DataflowNode:
    """Copy the forward part of a training graph (dropping loss-gradient chain, optimiser and any node
    for which ``keep(kernel)`` is false, e.g. dropout) into a test graph sharing the operators."""
    fwd = [n for n in SubGraph._topological_sort(head)
           if not n.op.kernel.is_gradient and not n.op.kernel.is_optimiser
           and not getattr(n.op.kernel, "is_gradient_merge", False)]
    copies: Dict[int, DataflowNode] = {}

    def resolve(n):
        # skip dropped nodes by forwarding to their (single) input
        while not keep(n.op.kernel):
            n = n.prev[0]
        return copies[id(n)]

    for n in fwd:
        if not keep(n.op.kernel):
            continue
        c = n.shallowCopy()
        copies[id(n)] = c
        for p in n.prev:
            if p.op.kernel.is_gradient:
                continue
            resolve(p).connectTo(c)
    return copies[id(fwd[0])]
