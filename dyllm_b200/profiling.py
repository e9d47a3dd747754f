"""Optional CUDA-event timing of named regions of the hot path (off by default; bench.py turns it on
to measure the per-launch duration of the dominant kernels inside its timed region)."""

from __future__ import annotations

import contextlib
from collections import defaultdict

import torch

_enabled = False
_records: dict[str, list] = defaultdict(list)


def enable(flag: bool = True) -> None:
    global _enabled
    _enabled = flag


def reset() -> None:
    _records.clear()
    _counts.clear()


@contextlib.contextmanager
def region(name: str, work: float = 0.0):
    """Times the enclosed launches with CUDA events on the current stream; ``work`` is the algorithmic
    flop or byte count of the region."""
    if not _enabled:
        yield
        return
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    try:
        yield
    finally:
        end.record()
        _records[name].append((start, end, work))


_counts: dict[str, list] = defaultdict(list)


def count(name: str, value: float) -> None:
    """Records a host-side number (for example the salient rows of a layer) when profiling is on."""
    if _enabled:
        _counts[name].append(value)


def counts() -> dict:
    return {k: list(v) for k, v in _counts.items()}


def summary() -> dict:
    """name -> {launches, total_ms, avg_ms, work} after a device synchronisation."""
    torch.cuda.synchronize()
    out = {}
    for name, recs in _records.items():
        total = sum(s.elapsed_time(e) for s, e, _ in recs)
        out[name] = {"launches": len(recs), "total_ms": total, "avg_ms": total / max(len(recs), 1),
                     "work": sum(w for _, _, w in recs)}
    return out
