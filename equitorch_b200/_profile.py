"""Optional per-kernel timing with CUDA events on the launching stream.

Disabled by default (zero overhead beyond one ``if``).  When enabled, every kernel call that
goes through :func:`timed` is bracketed by two events recorded on the current stream; elapsed
times are read after the caller synchronises.  Used by ``bench.py`` to attribute the step time to
kernels inside the timed region itself.
"""
from __future__ import annotations

from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, List, Tuple

import torch

_enabled = False
_pending: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []


def enable(flag: bool = True) -> None:
    global _enabled
    _enabled = flag
    if not flag:
        _pending.clear()


@contextmanager
def timed(name: str):
    if not _enabled:
        yield
        return
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    try:
        yield
    finally:
        stop.record()
        _pending.append((name, start, stop))


def collect() -> Dict[str, Tuple[int, float]]:
    """After a synchronize: ``{name: (launches, total milliseconds)}``; clears the record."""
    out: Dict[str, List[float]] = defaultdict(lambda: [0, 0.0])
    for name, a, b in _pending:
        out[name][0] += 1
        out[name][1] += a.elapsed_time(b)
    _pending.clear()
    return {k: (int(v[0]), float(v[1])) for k, v in out.items()}
