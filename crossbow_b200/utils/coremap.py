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
