"""Named interval timers for the training loop, measured on the device without stalling it.

``Timers`` mirrors the reference's timer registry (paddleformers/trainer/plugins/timer.py:100: ``timers("name").start()
/ .stop()``, a one-line log of all timers every logging interval). On a CUDA device each interval is a pair of events
recorded on the current stream; elapsed times are read only when the log line is built, after the events have
completed anyway, so that enabling timers adds no synchronisation to the step path. On CPU it falls back to
``time.perf_counter``.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch


class _Timer:
    def __init__(self, name: str, use_cuda: bool):
        self.name = name
        self.use_cuda = use_cuda
        self._pairs: List[tuple] = []
        self._open = None
        self._cpu_total = 0.0
        self.count = 0

    def start(self):
        assert self._open is None, f"timer {self.name} already started"
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open = ev
        else:
            self._open = time.perf_counter()
        return self

    def stop(self):
        assert self._open is not None, f"timer {self.name} was not started"
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pairs.append((self._open, ev))
        else:
            self._cpu_total += time.perf_counter() - self._open
        self._open = None
        self.count += 1

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()

    def elapsed(self, reset: bool = True) -> float:
        """Seconds accumulated since the last reset (waits for the last recorded event when on CUDA)."""
        total = self._cpu_total
        if self.use_cuda and self._pairs:
            self._pairs[-1][1].synchronize()
            total += sum(a.elapsed_time(b) for a, b in self._pairs) / 1e3
        if reset:
            self._pairs, self._cpu_total, self.count = [], 0.0, 0
        return total


class Timers:
    def __init__(self, use_cuda: Optional[bool] = None):
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.timers: Dict[str, _Timer] = {}

    def __call__(self, name: str) -> _Timer:
        if name not in self.timers:
            self.timers[name] = _Timer(name, self.use_cuda)
        return self.timers[name]

    def info(self, normalizer: float = 1.0, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per ``normalizer`` (e.g. steps of the interval) for every timer that ran."""
        out = {}
        for name, t in self.timers.items():
            if t.count or t._pairs or t._cpu_total:
                out[name] = t.elapsed(reset) * 1e3 / max(normalizer, 1e-12)
        return out

    def log(self, normalizer: float = 1.0, reset: bool = True) -> str:
        return " | ".join(f"{k}: {v:.2f} ms" for k, v in self.info(normalizer, reset).items())


_GLOBAL: Optional[Timers] = None


def get_timers() -> Optional[Timers]:
    return _GLOBAL


def set_timers(t: Optional[Timers] = None) -> Timers:
    global _GLOBAL
    _GLOBAL = t if t is not None else Timers()
    return _GLOBAL


def disable_timers():
    global _GLOBAL
    _GLOBAL = None
