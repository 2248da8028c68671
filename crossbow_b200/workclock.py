"""Task numbering and synchronisation epochs (WorkClock.java:24-84): a task counter and a clock that advances every
``wpc`` tasks; ``is_barrier`` tells whether the task just issued closes a clock."""


class WorkClock:
    def __init__(self, wpc: int, max_tasks: int = 1 << 62):
        if wpc < 1:
            raise ValueError("error: work per clock must be positive")
        self.wpc = wpc
        self.max = max_tasks
        self.task = -1          # id of the last task handed out
        self.inner = 0          # tasks issued since the last barrier
        self.clock = 0

    def next_task(self) -> int:
        self.task = (self.task + 1) % self.max
        self.inner += 1
        return self.task

    incrementAndGetNext = next_task

    def is_barrier(self) -> bool:
        return self.inner >= self.wpc

    isBarrier = is_barrier

    def tick(self):
        self.inner = 0
        self.clock += 1
        return self.clock

    def lower_bound(self, slack: int) -> int:
        """Oldest replica clock a new task may run on (ExecutionContext.java:274-276)."""
        return self.clock - slack - 1
