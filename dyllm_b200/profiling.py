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


def enabled() -> bool:
    return _enabled


def reset() -> None:
    _records.clear()
    _counts.clear()


@contextlib.contextmanager
def region(name: str, work: float = 0.0, nbytes: float = 0.0):
    """Times the enclosed launches with CUDA events on the current stream; ``work`` is the algorithmic
    flop count of the region and ``nbytes`` its algorithmic HBM bytes."""
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
        _records[name].append((start, end, work, nbytes))


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
        total = sum(r[0].elapsed_time(r[1]) for r in recs)
        out[name] = {"launches": len(recs), "total_ms": total, "avg_ms": total / max(len(recs), 1),
                     "work": sum(r[2] for r in recs), "bytes": sum(r[3] for r in recs)}
    return out
