"""Python wrappers over the fused entry points of the C ABI that have no one-to-one counterpart in
the reference's extension modules (they replace short sequences of torch ops in the reference's
layer code; each docstring names the lines replaced).
"""

from __future__ import annotations

import torch

from ._lib import call, load, ptr, require_cuda, stream_ptr


def context_stats(c_old: torch.Tensor, c_new: torch.Tensor, out: torch.Tensor | None = None,
                  accumulate: bool = False) -> torch.Tensor:
    """[dot(new, old), |new|^2, |old|^2] per row in fp32.

    Stand-alone form of the attention epilogue statistics
    (ref: dyllm/csrc/attention/attention_ops_kernels_sm80.cu:407-481).
    """
    require_cuda(c_old, "c_old", torch.bfloat16)
    require_cuda(c_new, "c_new", torch.bfloat16)
    if c_old.shape != c_new.shape:
        raise RuntimeError("c_old and c_new must have the same shape")
    rows = c_old.size(0)
    width = c_old.numel() // max(rows, 1)
    if out is None:
        out = torch.empty((rows, 3), dtype=torch.float32, device=c_old.device)
        accumulate = False
    else:
        require_cuda(out, "out", torch.float32, 2)
    call("dyllm_context_stats", ptr(c_old), ptr(c_new), ptr(out), rows, width, int(accumulate),
         stream_ptr(c_old.device))
    return out


def cosine_mask(stats: torch.Tensor, threshold: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """ref: dyllm/csrc/attention/attention_aux_kernels.cu:10-20."""
    require_cuda(stats, "stats", torch.float32, 2)
    rows = stats.size(0)
    if out is None:
        out = torch.empty((rows,), dtype=torch.bool, device=stats.device)
    call("dyllm_cosine_mask", ptr(stats), ptr(out), rows, float(threshold), stream_ptr(stats.device))
    return out


class SalientSelection:
    """Worst-case-sized output buffers of :func:`salient_select`; ``count`` stays on the device."""

    __slots__ = ("idx", "idx32", "idx_k", "cu_salientlens", "count", "mask")

    def __init__(self, idx, idx32, idx_k, cu_salientlens, count, mask):
        self.idx, self.idx32, self.idx_k = idx, idx32, idx_k
        self.cu_salientlens, self.count, self.mask = cu_salientlens, count, mask


_workspaces: dict = {}


def _select_workspace(rows: int, device: torch.device) -> torch.Tensor:
    need = load().dyllm_salient_select_workspace_bytes(rows)
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 4096), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


def salient_select(stats: torch.Tensor, threshold: float, cu_seqlens_q: torch.Tensor,
                   cu_promptlens: torch.Tensor | None = None, want_mask: bool = False,
                   want_idx32: bool = True) -> SalientSelection:
    """Mask + ordered compaction (+ K-space offsets) in one launch, no host synchronisation.

    Replaces ``nonzero`` / ``searchsorted`` / ``fused_offset_launch`` of
    dyllm/model_executor/layers/attention.py:147-166.  Every list has ``rows`` entries of which the first
    ``count`` are valid.
    """
    require_cuda(stats, "stats", torch.float32, 2)
    require_cuda(cu_seqlens_q, "cu_seqlens_q", torch.int32, 1)
    rows, dev = stats.size(0), stats.device
    batch = cu_seqlens_q.numel() - 1
    idx = torch.empty((rows,), dtype=torch.int64, device=dev)
    idx32 = torch.empty((rows,), dtype=torch.int32, device=dev) if want_idx32 else None
    idx_k = None
    if cu_promptlens is not None:
        require_cuda(cu_promptlens, "cu_promptlens", torch.int32, 1)
        idx_k = torch.empty((rows,), dtype=torch.int64, device=dev)
    cu_sal = torch.empty((batch + 1,), dtype=torch.int32, device=dev)
    count = torch.empty((1,), dtype=torch.int32, device=dev)
    mask = torch.empty((rows,), dtype=torch.bool, device=dev) if want_mask else None
    ws = _select_workspace(rows, dev)
    call("dyllm_salient_select", ptr(stats), rows, float(threshold), ptr(cu_seqlens_q), batch, ptr(cu_promptlens),
         ptr(idx), ptr(idx32), ptr(idx_k), ptr(cu_sal), ptr(count), ptr(mask), ptr(ws), ws.numel(), stream_ptr(dev))
    return SalientSelection(idx, idx32, idx_k, cu_sal, count, mask)
