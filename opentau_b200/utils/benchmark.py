"""``TimeBenchmark``: a re-entrant, thread-safe stopwatch context manager
(reference ``src/opentau/utils/benchmark.py:20-98``)."""

from __future__ import annotations

import threading
import time
from contextlib import ContextDecorator


class TimeBenchmark(ContextDecorator):
    def __init__(self, print: bool = False):  # noqa: A002 - reference signature
        self.local = threading.local()
        self.print_time = print

    def __enter__(self):
        self.local.start_time = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.local.end_time = time.perf_counter()
        self.local.elapsed_time = self.local.end_time - self.local.start_time
        if self.print_time:
            print(f"Elapsed time: {self.local.elapsed_time:.4f} seconds")
        return False

    @property
    def result(self) -> float:
        return getattr(self.local, "elapsed_time", None)

    @property
    def result_ms(self) -> float:
        return self.result * 1e3
