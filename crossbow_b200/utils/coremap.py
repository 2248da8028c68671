"""Thread-to-core plan (CoreMapper.java:19-52): core 0 the dispatcher, core 1 the device worker, then task handlers,
file handlers and callback handlers.  The reference hard-codes one particular two-socket host; here the plan is computed
from the number of cores that are actually online."""
import os
from typing import Dict, List


def plan(task_handlers: int, file_handlers: int, callback_handlers: int, offset: int = 1) -> Dict[str, List[int]]:
    n = os.cpu_count() or 1
    nxt = [offset + 1]

    def take(k):
        out = [(nxt[0] + i) % n for i in range(k)]
        nxt[0] += k
        return out

    return {"dispatcher": [0], "worker": [offset % n], "task": take(task_handlers), "file": take(file_handlers), "callback": take(callback_handlers)}


class CoreMapper:
    """The plan for the current system configuration (what `SystemConf.getCoreMapper()` hands out in the reference)."""

    def __init__(self, conf=None):
        if conf is None:
            from ..conf import SystemConf
            conf = SystemConf.getInstance()
        self.cores = plan(max(0, conf.number_of_task_handlers), max(0, conf.number_of_file_handlers),
                          max(1, conf.number_of_callback_handlers), conf.core_mapper_offset)

    def get(self, role: str, index: int = 0) -> int:
        """Core of the index-th thread of a role: dispatcher, worker, task, file, callback."""
        ids = self.cores[role]
        return ids[index % len(ids)] if ids else 0

    def dump(self) -> str:
        return "\n".join(f"{k:<10s} {v}" for k, v in self.cores.items())
