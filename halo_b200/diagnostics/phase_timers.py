"""Opt-in spans timed with CUDA events recorded on the current stream - never a host clock read that
would drain the queue. Nested spans report exclusive time; what no span covers goes to
``unaccounted`` (the role of halo/diagnostics/phase_timers.py:65-152)."""

from __future__ import annotations

import time
from contextlib import contextmanager

import torch

GRPO_PHASES = ("rollout", "sync", "build", "no_grad", "micro_step", "loss_forward", "post_backward_finish", "reduce",
               "optimizer")


class PhaseTimers:
    def __init__(self, enabled: bool = True, device=None):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._open: list = []
        self._records: list = []   # (name, start, end, depth)
        self.totals: dict[str, float] = {}

    def _mark(self):
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    @contextmanager
    def span(self, name: str):
        if not self.enabled:
            yield
            return
        start = self._mark()
        self._open.append(name)
        try:
            yield
        finally:
            self._open.pop()
            self._records.append((name, start, self._mark(), len(self._open)))

    def _elapsed(self, a, b) -> float:
        return a.elapsed_time(b) / 1e3 if self.cuda else b - a

    def collect(self, window_start=None, window_end=None) -> dict[str, float]:
        """Synchronising: call once per logging step. Returns seconds per phase (exclusive)."""
        if self.cuda:
            torch.cuda.synchronize()
        incl = [(n, self._elapsed(s, e), d) for n, s, e, d in self._records]
        out: dict[str, float] = {}
        # records close in post-order: a span's children precede it and have depth + 1
        stack: list[tuple[float, int]] = []
        for name, dur, depth in incl:
            child = 0.0
            while stack and stack[-1][1] > depth:
                child += stack.pop()[0]
            out[name] = out.get(name, 0.0) + max(0.0, dur - child)
            stack.append((dur, depth))
        if window_start is not None and window_end is not None:
            total = self._elapsed(window_start, window_end)
            out["unaccounted"] = max(0.0, total - sum(d for _, d, dep in incl if dep == 0))
        self._records.clear()
        for k, v in out.items():
            self.totals[k] = self.totals.get(k, 0.0) + v
        return out
