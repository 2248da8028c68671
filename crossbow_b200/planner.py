"""Static output-buffer reuse plan (MemoryPlannerV2.java:117-296): every operator's output is reference-counted by its
consumers (and by the gradient operator that needs it as its peer's output); when the count drops to zero the buffer
goes to a free pool, and a later operator whose output is not larger re-uses it.  The result is, per operator, either a
fresh buffer or ``(provider operator, position)``.  The device lowering uses the plan's buffer ids to alias arena
tensors when ``--reuse-memory true``."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

from .graph import SubGraph


class MemoryPlan:
    def __init__(self):
        self.buffer_of: Dict[int, int] = {}          # id(node) -> buffer id
        self.capacity: List[int] = []                # bytes per buffer id
        self.provider: Dict[int, Optional[int]] = {}  # id(node) -> id(node) that first owned the buffer (None = fresh)

    def total_bytes(self) -> int:
        return sum(self.capacity)

    def naive_bytes(self, graph: SubGraph) -> int:
        return sum(4 * n.op.output_shape.countAllElements() for n in graph.order if n.op.output_shape is not None)


def plan(graph: SubGraph, inplace_relu: bool = False) -> MemoryPlan:
    order = graph.order
    pos = {id(n): i for i, n in enumerate(order)}
    # last position at which each node's output is read
    last_use = {id(n): pos[id(n)] for n in order}
    for n in order:
        for p in n.prev:
            last_use[id(p)] = max(last_use[id(p)], pos[id(n)])
        # a gradient operator reads its peer's output (and the peer's inputs)
        if n.op.kernel.is_gradient and n.op.peer is not None:
            for m in order:
                if m.op is n.op.peer and not m.op.kernel.is_gradient:
                    last_use[id(m)] = max(last_use[id(m)], pos[id(n)])
                    for p in m.prev:
                        last_use[id(p)] = max(last_use[id(p)], pos[id(n)])
    mp = MemoryPlan()
    free: List[Tuple[int, int, int]] = []            # (capacity, buffer id, owner node id)
    expiring: Dict[int, List[int]] = {}
    for n in order:
        expiring.setdefault(last_use[id(n)], []).append(id(n))
    owner_of_buffer: Dict[int, int] = {}
    for i, n in enumerate(order):
        need = 4 * n.op.output_shape.countAllElements() if n.op.output_shape is not None else 0
        chosen = None
        # best fit among dead buffers that are large enough
        cands = [f for f in free if f[0] >= need]
        if cands and need > 0:
            chosen = min(cands, key=lambda f: f[0])
            free.remove(chosen)
            mp.buffer_of[id(n)] = chosen[1]
            mp.provider[id(n)] = owner_of_buffer[chosen[1]]
        else:
            bid = len(mp.capacity)
            mp.capacity.append(need)
            mp.buffer_of[id(n)] = bid
            mp.provider[id(n)] = None
            owner_of_buffer[bid] = id(n)
        for dead in expiring.get(i, []):
            if dead in mp.buffer_of:
                b = mp.buffer_of[dead]
                free.append((mp.capacity[b], b, owner_of_buffer[b]))
    return mp
