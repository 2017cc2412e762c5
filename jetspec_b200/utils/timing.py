"""Device and host phase timers.

``CudaTimer`` brackets a region with CUDA events on the current stream and skips
recording while a graph is being captured (events recorded during capture would
become graph nodes).  ``PhaseTimer`` accumulates named phases per decode round,
the equivalent of the reference's ``profile_phases`` accounting
(``jetspec/core/llm.py:423-432``).
"""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is present, no-op otherwise."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class CudaTimer:
    """Accumulates device time of ``with timer:`` regions, read with ``total_ms()``."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._pairs: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []
        self._open = None
        self.calls = 0

    def __enter__(self):
        if self.enabled and not torch.cuda.is_current_stream_capturing():
            s = torch.cuda.Event(enable_timing=True)
            s.record()
            self._open = s
        return self

    def __exit__(self, *exc):
        if self._open is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pairs.append((self._open, e))
            self._open = None
            self.calls += 1
        return False

    def total_ms(self) -> float:
        if not self._pairs:
            return 0.0
        torch.cuda.synchronize()
        return float(sum(s.elapsed_time(e) for s, e in self._pairs))

    def reset(self) -> None:
        self._pairs.clear()
        self.calls = 0


class PhaseTimer:
    """Wall-clock per-phase accumulator with optional device synchronisation."""

    def __init__(self, enabled: bool = False, sync: bool = True):
        self.enabled = enabled
        self.sync = sync and torch.cuda.is_available()
        self.totals: dict[str, float] = defaultdict(float)
        self.counts: dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.sync:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.sync:
                torch.cuda.synchronize()
            self.totals[name] += time.perf_counter() - t0
            self.counts[name] += 1

    def summary_ms_per_round(self, rounds: int) -> dict[str, float]:
        r = max(1, rounds)
        return {k: 1e3 * v / r for k, v in self.totals.items()}
