"""Throughput-driven replica auto-tuner (ModelManager.java:238-274).

At every ``interval``-th synchronisation the latest throughput sample is compared with the previous one: a relative
gain above ``threshold`` adds one replica per GPU; the first sample that fails to improve removes one replica and
switches tuning off for good."""
from typing import Optional, Sequence


class AutoTuner:
    def __init__(self, threshold: float = 0.1, interval: int = 1):
        self.threshold, self.interval = threshold, max(1, interval)
        self.active = True
        self.calls = 0
        self.previous: Optional[float] = None
        self.history = []

    def has_improved(self, current: float) -> bool:
        if self.previous is None or self.previous <= 0:
            return True
        return (current - self.previous) / self.previous > self.threshold

    def decide(self, samples: Sequence[float]) -> int:
        """+1 add a replica, -1 remove one (and stop), 0 do nothing."""
        if not self.active:
            return 0
        self.calls += 1
        if self.calls % self.interval or not samples:
            return 0
        current = float(samples[-1])
        self.history.append(current)
        if self.has_improved(current):
            self.previous = current
            return 1
        self.active = False
        return -1
