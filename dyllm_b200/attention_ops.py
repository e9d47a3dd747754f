"""Drop-in for the reference's ``dyllm.attention_ops`` extension module
(ref: dyllm/csrc/attention/attention.cpp:197-208): same function names, argument order and error type.
"""

from __future__ import annotations

import torch

from ._lib import call, load, ptr, stream_ptr

_EMPTY = None
_workspaces: dict = {}


def _workspace(nbytes: int, device) -> torch.Tensor:
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


def _check_tensor(t, name, device, dtype, dim):
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be defined")
    if not (t.is_cuda and t.device == device):
        raise RuntimeError(f"{name} must be on {device}")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} has an invalid dtype")
    if t.dim() != dim or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous {dim}D tensor")


def attention_sparse_varlen(Q, K, V, C, o_sal, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int,
                            total_seqlen: int, cu_salientlens, idx_salient_row, cosine_stats, cosine_out,
                            threshold: float = 0.0, is_q_pruned: bool = False, idx_salient_row_k=None,
                            force_mask_v_rows: int = -1, v_layout: int = 1, num_salient_dev=None,
                            c_cache=None) -> torch.Tensor:
    """ref: dyllm/csrc/attention/attention.cpp:64-179.

    Same arguments, checks and return value (a fresh ``O`` shaped like ``Q``).  ``force_mask_v_rows``
    is accepted and ignored (it switches between two load strategies of the reference kernel that
    compute the same result).  ``V`` must be zero outside the listed salient key rows, as the
    reference's caller builds it.  ``v_layout`` (extension): bit 0 = feed the delta-V tile as an
    MN-major operand, bit 1 = ``V`` is compact ``[num_salient, Hkv, D]`` (row i = key
    ``idx_salient_row_k[i]``) instead of the zero-padded ``[T_k, Hkv, D]`` tensor.  ``num_salient_dev``
    (extension): device int32 scalar with the live length of the index lists, whose tensors are then
    only capacity-sized.  bit 2 of ``v_layout`` (extension): ``cosine_stats`` is overwritten, not added to.
    With ``c_cache`` and ``is_q_pruned``, ``idx_salient_row_k`` may be None: a listed query row's key row is
    the row at the same distance from the end of its sequence.  ``c_cache`` (extension): ``(seq_starts, seq_ids, update_in_place)``; ``C`` is then the
    context cache arena ``[cache_rows, H, D]`` read (and optionally updated) in place instead of a packed copy.
    """
    if not (isinstance(Q, torch.Tensor) and Q.is_cuda):
        raise RuntimeError("Q must be CUDA")
    dev, bf16, i32 = Q.device, torch.bfloat16, torch.int32
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (C, "C"), (o_sal, "o_sal")):
        _check_tensor(t, n, dev, bf16, 3)
    compact = bool(v_layout & 2)
    for t, n in ((cu_seqlens_q, "cu_seqlens_q"), (cu_seqlens_k, "cu_seqlens_k"), (cu_salientlens, "cu_salientlens"),
                 (idx_salient_row, "idx_salient_row")):
        _check_tensor(t, n, dev, i32, 1)
    _check_tensor(cosine_stats, "cosine_stats", dev, torch.float32, 2)
    _check_tensor(cosine_out, "cosine_out", dev, torch.bool, 1)
    if compact:
        if V.shape != (idx_salient_row.numel(), K.size(1), K.size(2)):
            raise RuntimeError("compact V must be [idx_salient_row.numel(), K.size(1), K.size(2)]")
    elif K.shape != V.shape:
        raise RuntimeError("K and V must have the same shape")
    if not (Q.size(0) > 0 and K.size(0) > 0):
        raise RuntimeError("Q and K/V token dimensions must be non-empty")
    if Q.size(2) != K.size(2):
        raise RuntimeError("Q, K, and V must have the same head dimension")
    if c_cache is None and C.shape != Q.shape:
        raise RuntimeError("C must have the same shape as Q")
    if c_cache is not None and C.shape[1:] != Q.shape[1:]:
        raise RuntimeError("the context cache must be [cache_rows, Q.size(1), Q.size(2)]")
    if not (o_sal.size(0) == idx_salient_row.numel() and o_sal.size(1) == Q.size(1) and o_sal.size(2) == Q.size(2)):
        raise RuntimeError("o_sal must be [idx_salient_row.numel(), Q.size(1), Q.size(2)]")
    if not (Q.size(1) > 0 and K.size(1) > 0 and Q.size(1) % K.size(1) == 0):
        raise RuntimeError(f"local TP query heads must be a positive multiple of local KV heads; got {Q.size(1)} "
                           f"and {K.size(1)}")
    if Q.size(2) != 128:
        raise RuntimeError(f"supported head dimension is 128; got {Q.size(2)}")
    if not (cu_seqlens_q.numel() >= 2 and cu_seqlens_q.numel() == cu_seqlens_k.numel() == cu_salientlens.numel()):
        raise RuntimeError("cu_seqlens_q, cu_seqlens_k, and cu_salientlens must have the same B+1 length")
    if total_seqlen != Q.size(0):
        raise RuntimeError("total_seqlen must equal Q.size(0)")
    if not (cosine_stats.size(0) == Q.size(0) and cosine_stats.size(1) == 3):
        raise RuntimeError("cosine_stats must be [Q.size(0), 3]")
    if cosine_out.numel() != Q.size(0):
        raise RuntimeError("cosine_out must contain Q.size(0) elements")
    if not (0 < max_seqlen_q <= Q.size(0) and 0 < max_seqlen_k <= K.size(0)):
        raise RuntimeError("maximum sequence lengths must be positive and fit their packed token dimensions")
    if idx_salient_row.numel() > Q.size(0):
        raise RuntimeError("salient Q index count cannot exceed Q.size(0)")
    if force_mask_v_rows not in (-1, 0, 1):
        raise RuntimeError("force_mask_v_rows must be -1, 0, or 1")
    idx_k = idx_salient_row
    if is_q_pruned and idx_salient_row_k is None and c_cache is not None:
        idx_k = None        # extension: key rows derived from the query rows (queries = last rows of a sequence)
    elif is_q_pruned:
        _check_tensor(idx_salient_row_k, "idx_salient_row_k", dev, i32, 1)
        if idx_salient_row_k.numel() != idx_salient_row.numel():
            raise RuntimeError("parallel Q/K pruning requires matching salient Q and K index counts")
        if idx_salient_row_k.numel() > K.size(0):
            raise RuntimeError("salient K index count cannot exceed K.size(0)")
        idx_k = idx_salient_row_k

    out = torch.empty_like(Q)
    H = Q.size(1)
    need = load().dyllm_attention_sparse_workspace_bytes(Q.size(0), H)
    ws = _workspace(need, dev)
    call("dyllm_attention_sparse_varlen", ptr(Q), ptr(K), ptr(V), ptr(C), ptr(o_sal), ptr(out), ptr(cu_seqlens_q),
         ptr(cu_seqlens_k), cu_seqlens_q.numel() - 1, int(max_seqlen_q), int(max_seqlen_k), Q.size(0), K.size(0), H,
         K.size(1), Q.size(2), ptr(cu_salientlens), ptr(idx_salient_row), ptr(idx_k), idx_salient_row.numel(),
         ptr(num_salient_dev), ptr(cosine_stats), ptr(cosine_out), float(threshold), ptr(ws), ws.numel(), int(v_layout),
         ptr(c_cache[0]) if c_cache else None, ptr(c_cache[1]) if c_cache else None,
         int(bool(c_cache[2])) if c_cache else 0, stream_ptr(dev))
    return out


def attention_kernel_info(dim: int, mask_v_rows: bool = False) -> list[int]:
    """ref: dyllm/csrc/attention/attention.cpp:184-208."""
    import ctypes

    buf = (ctypes.c_int64 * 10)()
    call("dyllm_attention_kernel_info", int(dim), ctypes.cast(buf, ctypes.c_void_p))
    return list(buf)


def _check_i32_vector(t: torch.Tensor, name: str, device) -> None:
    if not (t.is_cuda and t.device == device):
        raise RuntimeError(f"{name} must be on {device}")
    if t.dtype != torch.int32:
        raise RuntimeError(f"{name} must be int32")
    if t.dim() != 1 or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous 1D tensor")


def fused_offset_launch(idxs, num_idxs, cu_promptlens, cu_salientlens, out_tensor, max_threads: int) -> None:
    """ref: dyllm/csrc/attention/attention_aux_kernels.cu:173-200."""
    device = idxs.device
    _check_i32_vector(idxs, "idxs", device)
    _check_i32_vector(num_idxs, "num_idxs", device)
    _check_i32_vector(cu_promptlens, "cu_promptlens", device)
    _check_i32_vector(cu_salientlens, "cu_salientlens", device)
    if num_idxs.numel() != 1:
        raise RuntimeError("num_idxs must contain exactly one element")
    if cu_promptlens.numel() != cu_salientlens.numel():
        raise RuntimeError("cu_promptlens and cu_salientlens must have the same length")
    if not (out_tensor.is_cuda and out_tensor.device == device and out_tensor.dtype == torch.int64
            and out_tensor.dim() == 1 and out_tensor.is_contiguous()):
        raise RuntimeError(f"out_tensor must be a contiguous int64 CUDA vector on {device}")
    if not (0 <= max_threads <= out_tensor.numel()):
        raise RuntimeError("max_threads must fit out_tensor")
    if max_threads == 0:
        return
    call("dyllm_fused_offset", ptr(idxs), ptr(num_idxs), ptr(cu_promptlens), ptr(cu_salientlens),
         cu_promptlens.numel() - 1, ptr(out_tensor), int(max_threads), stream_ptr(device))




def attention_salient_rows(q, k, v, cu_seqlens_k, cu_salientlens, idx_salient_row, max_rows_per_seq: int,
                           num_salient: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Exact non-causal attention of the salient query rows against the whole K / V of their sequence.

    Replaces ``flash_attn_varlen_func(q[idx_salient_row], k, v_cache, cu_seqlens_q=cu_salientlens, ...)`` of
    dyllm/model_executor/layers/attention.py:76-87 without materialising ``q[idx]``.  ``idx_salient_row`` is
    int32 in Q space; rows past ``cu_salientlens[-1]`` of ``out`` are left untouched.
    """
    dev = q.device
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_tensor(t, n, dev, torch.bfloat16, 3)
    for t, n in ((cu_seqlens_k, "cu_seqlens_k"), (cu_salientlens, "cu_salientlens"), (idx_salient_row, "idx_salient_row")):
        _check_tensor(t, n, dev, torch.int32, 1)
    if k.shape != v.shape:
        raise RuntimeError("K and V must have the same shape")
    if q.size(2) != 128 or k.size(2) != 128:
        raise RuntimeError(f"supported head dimension is 128; got {q.size(2)}")
    n = idx_salient_row.numel() if num_salient is None else num_salient
    if out is None:
        out = torch.empty((n, q.size(1), q.size(2)), dtype=q.dtype, device=dev)
    if n == 0 or max_rows_per_seq == 0:
        return out
    call("dyllm_attention_salient_rows", ptr(q), ptr(k), ptr(v), ptr(out), ptr(cu_seqlens_k), cu_seqlens_k.numel() - 1,
         int(max_rows_per_seq), q.size(0), k.size(0), q.size(1), k.size(1), q.size(2), ptr(cu_salientlens),
         ptr(idx_salient_row), stream_ptr(dev))
    return out


__all__ = ["attention_sparse_varlen", "attention_salient_rows", "fused_offset_launch", "attention_kernel_info"]
