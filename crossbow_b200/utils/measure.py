"""Measurement queue and performance monitor (result/MeasurementQueue.java:162-237, PerformanceMonitor.java:59-172)."""
import time
from collections import deque


class MeasurementQueue:
    """(timestamp ns, task, loss, accuracy) records, dumped as ``timestamp loss accuracy`` lines."""

    def __init__(self, capacity: int = 1 << 20):
        self.items = deque(maxlen=capacity)

    def add(self, task, loss, accuracy):
        self.items.append((time.time_ns(), task, loss, accuracy))

    def dump(self) -> str:
        return "\n".join(f"{ts} {loss:.6f} {acc:.6f}" for ts, _, loss, acc in self.items)

    def losses(self):
        return [x[2] for x in self.items]

    def __len__(self):
        return len(self.items)


class PerformanceMonitor:
    """Counts finished tasks and turns them into examples/s and MB/s per interval; keeps a bounded window of samples
    that feeds the auto-tuner."""

    def __init__(self, batch_size: int, batch_bytes: int, interval_s: float = 1.0, window: int = 64, sink=None):
        """`sink`: called with every `[MON]` line as it is produced (the execution context prints it); the most recent
        lines are also kept in `lines`."""
        self.batch_size, self.batch_bytes, self.interval = batch_size, batch_bytes, interval_s
        self.samples = deque(maxlen=window)
        self.t0 = time.perf_counter()
        self.count = 0
        self.total = 0
        self.lines = deque(maxlen=256)
        self.sink = sink
        self.queue_size = None           # callable returning the number of tasks in flight, if known

    def task_done(self, n: int = 1):
        """`n` more tasks have finished.  Once per interval this produces the reference's monitor line
        (PerformanceMonitor.java:75-98: examples/s and MB/s of sub-graph S000, executor queue length)."""
        self.count += n
        self.total += n
        now = time.perf_counter()
        dt = now - self.t0
        if dt >= self.interval > 0:
            rate = self.count * self.batch_size / dt
            self.samples.append(rate)
            q = int(self.queue_size()) if self.queue_size is not None else 0
            line = f"[MON] S000 {rate:10.3f} examples/s {self.count * self.batch_bytes / dt / 1048576.0:10.3f} MB/s q {q:6d}"
            self.lines.append(line)
            if self.sink is not None:
                self.sink(line)
            self.t0, self.count = now, 0

    def flush(self):
        now = time.perf_counter()
        dt = now - self.t0
        if self.count and dt > 0:
            self.samples.append(self.count * self.batch_size / dt)
            self.t0, self.count = now, 0

    def last_rate(self) -> float:
        return self.samples[-1] if self.samples else 0.0

    def throughput_window(self):
        self.flush()
        return list(self.samples)
