"""Drop-in for the reference's ``dyllm.cache`` extension module (ref: dyllm/csrc/cache/cache.cpp:3-25).

Same five function names, argument order, shapes and error type (``RuntimeError``); the copies run as
16-byte-vectorised sm_100a kernels behind the C ABI.
"""

from __future__ import annotations

import torch

from . import _lib
from ._lib import call, ptr, stream_ptr


def _check_common(cache, seq_starts, cu_seqlens, seq_ids):
    for t, name in ((cache, "cache"), (seq_starts, "seq_starts"), (cu_seqlens, "cu_seqlens"), (seq_ids, "seq_ids")):
        if not (t.is_cuda and t.is_contiguous()):
            raise RuntimeError(f"{name} must be CUDA contiguous")
    if cu_seqlens.dtype != torch.int32:
        raise RuntimeError("cu_seqlens must be int32")
    if cache.dim() != 2:
        raise RuntimeError("cache must be [T, D]")
    if seq_starts.dtype != torch.int64 or seq_ids.dtype != torch.int64:
        raise RuntimeError("seq_starts and seq_ids must be int64")
    if (cache.size(1) * cache.element_size()) % 16 != 0:
        raise RuntimeError("D must be multiple of 8 for vec16 path")


def get_seqs_cuda(cache, seq_starts, cu_seqlens, seq_ids, total_seqlen: int) -> torch.Tensor:
    """ref: dyllm/csrc/cache/cache_kernels.cu:66-108."""
    _check_common(cache, seq_starts, cu_seqlens, seq_ids)
    out = torch.empty((int(total_seqlen), cache.size(1)), dtype=cache.dtype, device=cache.device)
    batch = seq_ids.size(0)
    if total_seqlen == 0 or batch == 0:
        return out
    call("dyllm_cache_get_seqs", ptr(cache), ptr(out), ptr(seq_starts), ptr(cu_seqlens), ptr(seq_ids), batch,
         int(total_seqlen), cache.size(1), cache.element_size(), stream_ptr(cache.device))
    return out


def get_block_cuda(cache, seq_starts, cu_seqlens, cu_seqlens_q, seq_ids, total_seqlen: int) -> torch.Tensor:
    """ref: dyllm/csrc/cache/cache_kernels.cu:249-294."""
    _check_common(cache, seq_starts, cu_seqlens, seq_ids)
    if cu_seqlens_q.dtype != torch.int32 or not cu_seqlens_q.is_cuda:
        raise RuntimeError("cu_seqlens_q must be a CUDA int32 tensor")
    out = torch.empty((int(total_seqlen), cache.size(1)), dtype=cache.dtype, device=cache.device)
    batch = seq_ids.size(0)
    if total_seqlen == 0 or batch == 0:
        return out
    call("dyllm_cache_get_block", ptr(cache), ptr(out), ptr(seq_starts), ptr(cu_seqlens), ptr(cu_seqlens_q),
         ptr(seq_ids), batch, int(total_seqlen), cache.size(1), cache.element_size(), stream_ptr(cache.device))
    return out


def reset_full_cuda(cache, inp, seq_starts, cu_seqlens, seq_ids, total_seqlen: int) -> None:
    """ref: dyllm/csrc/cache/cache_kernels.cu:158-198."""
    _check_common(cache, seq_starts, cu_seqlens, seq_ids)
    if not (inp.is_cuda and inp.is_contiguous()):
        raise RuntimeError("in must be CUDA contiguous")
    if inp.size(1) != cache.size(1):
        raise RuntimeError("in and cache must have same D")
    batch = seq_ids.size(0)
    if total_seqlen == 0 or batch == 0:
        return
    call("dyllm_cache_reset_full", ptr(cache), ptr(inp), ptr(seq_starts), ptr(cu_seqlens), ptr(seq_ids), batch,
         int(total_seqlen), cache.size(1), cache.element_size(), stream_ptr(cache.device))


def reset_block_cuda(cache, inp, seq_starts, cu_seqlens, cu_seqlens_q, seq_ids, total_seqlen: int) -> None:
    """ref: dyllm/csrc/cache/cache_kernels.cu:345-386."""
    _check_common(cache, seq_starts, cu_seqlens, seq_ids)
    if not (inp.is_cuda and inp.is_contiguous()):
        raise RuntimeError("in must be CUDA contiguous")
    if inp.size(1) != cache.size(1):
        raise RuntimeError("in and cache must have same D")
    batch = seq_ids.size(0)
    if total_seqlen == 0 or batch == 0:
        return
    call("dyllm_cache_reset_block", ptr(cache), ptr(inp), ptr(seq_starts), ptr(cu_seqlens), ptr(cu_seqlens_q),
         ptr(seq_ids), batch, int(total_seqlen), cache.size(1), cache.element_size(), stream_ptr(cache.device))


def scatter_update_cuda(cache, new_vals, row_idx, cu_seqlens, seq_starts, seq_ids, num_rows_dev=None) -> None:
    """ref: dyllm/csrc/cache/cache_kernels.cu:428-459.

    ``num_rows_dev`` (extension): device int32 scalar that bounds the number of rows consumed, so a
    caller holding a worst-case-sized index buffer needs no host synchronisation.
    """
    for t, name in ((cache, "cache"), (new_vals, "new_vals"), (row_idx, "row_idx"), (cu_seqlens, "cu_seqlens"),
                    (seq_starts, "seq_starts"), (seq_ids, "seq_ids")):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be CUDA")
    if row_idx.dtype != torch.int64:
        raise RuntimeError("row_idx must be int64")
    if cu_seqlens.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("cu_seqlens must be int32 or int64")
    m = new_vals.size(0)
    if m == 0:
        return
    if not new_vals.is_contiguous():
        new_vals = new_vals.contiguous()
    if num_rows_dev is None and row_idx.numel() < m:
        raise RuntimeError("row_idx has fewer entries than new_vals has rows")
    call("dyllm_cache_scatter_update", ptr(cache), ptr(new_vals), ptr(row_idx.contiguous()),
         ptr(cu_seqlens.contiguous()), 1 if cu_seqlens.dtype == torch.int64 else 0, ptr(seq_starts), ptr(seq_ids),
         seq_ids.size(0), m, ptr(num_rows_dev), new_vals.size(1), cache.element_size(), stream_ptr(cache.device))


__all__ = ["get_seqs_cuda", "get_block_cuda", "reset_full_cuda", "reset_block_cuda", "scatter_update_cuda"]
