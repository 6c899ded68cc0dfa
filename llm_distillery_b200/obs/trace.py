"""Phase timers and NVTX ranges.

The reference has no timers at all (its only signal is tqdm's it/s) and runs with ``CUDA_LAUNCH_BLOCKING=1``
(classes/teacher/model.py:21, classes/student/model.py:20). Here a ``PhaseTimer`` brackets the phases of a step
(forward+loss, backward, optimizer/communication, collection) with CUDA events on the launching stream - nothing is
synchronised while the step runs; the events are resolved when ``summary()`` is called (once per logging interval) -
and, when enabled, opens an NVTX range per phase so that a timeline tool shows the same names.

Enable with ``B200_TRACE=1`` (timers) and ``B200_NVTX=1`` (ranges), or construct with ``enabled=True``.
On CPU the timer falls back to ``time.perf_counter``.
"""
from __future__ import annotations

import os
import time
from collections import defaultdict
from contextlib import contextmanager

import torch


class PhaseTimer:
    def __init__(self, enabled: bool | None = None, nvtx: bool | None = None, device=None):
        self.enabled = (os.environ.get("B200_TRACE", "0") == "1") if enabled is None else enabled
        self.nvtx = (os.environ.get("B200_NVTX", "0") == "1") if nvtx is None else nvtx
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._pending: list = []                       # (name, start event, end event)
        self._cpu: dict[str, float] = defaultdict(float)
        self._count: dict[str, int] = defaultdict(int)

    @contextmanager
    def phase(self, name: str):
        if not (self.enabled or self.nvtx):
            yield
            return
        if self.nvtx and self.cuda:
            torch.cuda.nvtx.range_push(name)
        if self.enabled and self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.enabled:
                if self.cuda:
                    e1.record()
                    self._pending.append((name, e0, e1))
                else:
                    self._cpu[name] += (time.perf_counter() - t0) * 1e3
                self._count[name] += 1
            if self.nvtx and self.cuda:
                torch.cuda.nvtx.range_pop()

    def summary(self, reset: bool = True) -> dict[str, float]:
        """{phase: total milliseconds since the last reset} (device time on CUDA). Synchronises the device once."""
        out: dict[str, float] = defaultdict(float)
        if self._pending:
            torch.cuda.synchronize()
            for name, e0, e1 in self._pending:
                out[name] += e0.elapsed_time(e1)
        for k, v in self._cpu.items():
            out[k] += v
        res = dict(out)
        if reset:
            self._pending.clear()
            self._cpu.clear()
            self._count.clear()
        return res
