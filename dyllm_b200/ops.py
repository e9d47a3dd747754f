"""Python wrappers over the fused entry points of the C ABI that have no one-to-one counterpart in
the reference's extension modules (they replace short sequences of torch ops in the reference's
layer code; each docstring names the lines replaced).
"""

from __future__ import annotations

import torch

from . import _lib as _lib_mod
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


def cache_dest_rows(row_idx: torch.Tensor, cu_seqlens: torch.Tensor, seq_starts: torch.Tensor,
                    seq_ids: torch.Tensor, num_rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Cache row that ``scatter_update`` would write for each packed row (int32, -1 past the live rows).

    ref: dyllm/csrc/cache/cache_kernels.cu:398-421.
    """
    require_cuda(row_idx, "row_idx", torch.int64, 1)
    require_cuda(cu_seqlens, "cu_seqlens", torch.int32, 1)
    n = row_idx.numel()
    dest = torch.empty((n,), dtype=torch.int32, device=row_idx.device)
    call("dyllm_cache_dest_rows", ptr(row_idx), ptr(cu_seqlens), ptr(seq_starts), ptr(seq_ids), seq_ids.numel(), n,
         ptr(num_rows_dev), ptr(dest), stream_ptr(row_idx.device))
    return dest


_gemm_workspaces: dict = {}


def _gemm_workspace(nbytes: int, device) -> torch.Tensor:
    """One shared scratch tensor per device for the row staging, the FFN intermediate and split-K sums
    (kernels on one stream use it one after the other)."""
    ws = _gemm_workspaces.get(device)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _gemm_workspaces[device] = ws
    return ws


def gathered_linear(x: torch.Tensor, weight: torch.Tensor, idx: torch.Tensor | None = None,
                    num_rows: int | None = None, num_rows_dev: torch.Tensor | None = None, rows_hint: int = 0,
                    out: torch.Tensor | None = None, out2: torch.Tensor | None = None, split_col: int = 0,
                    out_row_map: torch.Tensor | None = None, row_scale: torch.Tensor | None = None, a_mode: int = -1,
                    tile_n: int = 0) -> torch.Tensor:
    """``out[map[m]] = scale[m] * (x[idx[m]] @ weight.T)`` on the tcgen05 tensor cores.

    ref: dyllm/model_executor/models/llada.py:108 (``kv_proj(hidden_states[idx_salient_row])``).
    """
    require_cuda(x, "x", torch.bfloat16, 2)
    require_cuda(weight, "weight", torch.bfloat16, 2)
    if idx is not None:
        require_cuda(idx, "idx", torch.int32, 1)
    if num_rows is None:
        num_rows = idx.numel() if idx is not None else x.size(0)
    n_out = weight.size(0)
    if out is None:
        out = torch.empty((num_rows, n_out if out2 is None else split_col), dtype=torch.bfloat16, device=x.device)
    if num_rows == 0:
        return out
    need = load().dyllm_gathered_linear_workspace_bytes(num_rows, x.size(1), n_out)
    ws = _gemm_workspace(need, x.device)
    call("dyllm_gathered_linear", ptr(x), x.size(0), x.size(1), x.stride(0), ptr(idx), num_rows, ptr(num_rows_dev),
         int(rows_hint), ptr(weight), n_out, ptr(out), out.stride(0), ptr(out2), out2.stride(0) if out2 is not None else 0,
         int(split_col), ptr(out_row_map), ptr(row_scale), ptr(ws), ws.numel(), a_mode, tile_n, stream_ptr(x.device))
    return out


def swiglu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, idx: torch.Tensor | None = None,
               num_rows: int | None = None, num_rows_dev: torch.Tensor | None = None, rows_hint: int = 0,
               out: torch.Tensor | None = None, out_row_map: torch.Tensor | None = None, a_mode: int = -1,
               tile_n: int = 0) -> torch.Tensor:
    """``out[map[m]] = down(silu(x[idx[m]] Wg^T) * (x[idx[m]] Wu^T))`` for the gathered rows.

    ref: dyllm/model_executor/models/llada.py:38-43,184-185.
    """
    require_cuda(x, "x", torch.bfloat16, 2)
    require_cuda(w_gate_up, "w_gate_up", torch.bfloat16, 2)
    require_cuda(w_down, "w_down", torch.bfloat16, 2)
    hidden, inter = x.size(1), w_down.size(1)
    if w_gate_up.shape != (2 * inter, hidden) or w_down.size(0) != hidden:
        raise RuntimeError("w_gate_up must be [2 * inter, hidden] and w_down [hidden, inter]")
    if idx is not None:
        require_cuda(idx, "idx", torch.int32, 1)
    if num_rows is None:
        num_rows = idx.numel() if idx is not None else x.size(0)
    if out is None:
        out = torch.empty((num_rows, hidden), dtype=torch.bfloat16, device=x.device)
    if num_rows == 0:
        return out
    ws = _gemm_workspace(load().dyllm_swiglu_ffn_workspace_bytes(num_rows, hidden, inter), x.device)
    call("dyllm_swiglu_ffn", ptr(x), x.size(0), hidden, x.stride(0), ptr(idx), num_rows, ptr(num_rows_dev),
         int(rows_hint), ptr(w_gate_up), ptr(w_down), inter, ptr(out), out.stride(0), ptr(out_row_map), ptr(ws),
         ws.numel(), a_mode, tile_n, stream_ptr(x.device))
    if idx is None:
        _lib_mod.launch_count -= 1      # no row staging launch when the rows arrive packed
    return out


def delta_v_update(v_new: torch.Tensor, cache: torch.Tensor, rows: torch.Tensor, dv: torch.Tensor | None = None,
                   num_rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """``dv[i] = v_new[i] - cache[rows[i]]; cache[rows[i]] = v_new[i]`` in one pass (bf16).

    ref: dyllm/model_executor/layers/attention.py:67-74,89-96.
    """
    require_cuda(v_new, "v_new", torch.bfloat16, 2)
    require_cuda(cache, "cache", torch.bfloat16, 2)
    require_cuda(rows, "rows", torch.int32, 1)
    if dv is None:
        dv = torch.empty_like(v_new)
    if v_new.size(0) == 0:
        return dv
    call("dyllm_delta_v_update", ptr(v_new), ptr(cache), ptr(rows), v_new.size(0), ptr(num_rows_dev), v_new.size(1),
         ptr(dv), stream_ptr(v_new.device))
    return dv


def kv_cache_update(k_new: torch.Tensor, v_new: torch.Tensor, rows_k: torch.Tensor, positions: torch.Tensor,
                    pos_idx: torch.Tensor | None, cos_sin: torch.Tensor, cu_seqlens_k: torch.Tensor,
                    k_seq_starts: torch.Tensor, v_seq_starts: torch.Tensor, seq_ids: torch.Tensor,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, num_rows_dev: torch.Tensor | None = None,
                    dv: torch.Tensor | None = None) -> torch.Tensor:
    """Rotary embedding of the new K rows + K-cache scatter + delta-V + V-cache update in one launch;
    returns dV ``[rows, kv_heads, 128]``.

    ref: dyllm/model_executor/models/llada.py:108-118; dyllm/model_executor/layers/attention.py:67-74,89-96.
    """
    require_cuda(k_new, "k_new", torch.bfloat16, 3)
    require_cuda(v_new, "v_new", torch.bfloat16, 3)
    require_cuda(rows_k, "rows_k", torch.int64, 1)
    require_cuda(positions, "positions", torch.int64, 1)
    require_cuda(cos_sin, "cos_sin", torch.float32)
    require_cuda(cu_seqlens_k, "cu_seqlens_k", torch.int32, 1)
    require_cuda(k_cache, "k_cache", torch.bfloat16, 2)
    require_cuda(v_cache, "v_cache", torch.bfloat16, 2)
    if dv is None:
        dv = torch.empty_like(v_new)
    n = k_new.size(0)
    if n == 0:
        return dv
    call("dyllm_kv_cache_update", ptr(k_new), ptr(v_new), ptr(rows_k), ptr(positions), ptr(pos_idx), ptr(cos_sin),
         cos_sin.size(0), ptr(cu_seqlens_k), ptr(k_seq_starts), ptr(v_seq_starts), ptr(seq_ids), seq_ids.numel(), n,
         ptr(num_rows_dev), k_new.size(1), k_new.size(2), ptr(k_cache), ptr(v_cache), ptr(dv), stream_ptr(k_new.device))
    return dv


def add_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """RMSNorm with the residual add fused in; returns ``y`` or ``(y, new_residual)`` as packed 2-D tensors.

    ``x`` is ``[rows, width]`` contiguous, or ``[segments, seg_rows, width]`` whose rows are contiguous and
    whose segments lie a whole number of rows apart (a view of a block of every sequence inside a cache).

    ref: dyllm/model_executor/layers/layernorm.py:17-53.
    """
    if not isinstance(x, torch.Tensor) or not x.is_cuda or x.dtype != torch.bfloat16:
        raise RuntimeError("x must be a CUDA bfloat16 tensor")
    require_cuda(weight, "weight", torch.bfloat16, 1)
    width = x.size(-1)
    if x.dim() == 2:
        require_cuda(x, "x", torch.bfloat16, 2)
        rows, seg_rows, seg_pitch = x.size(0), max(x.size(0), 1), max(x.size(0), 1)
    elif x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == width and x.stride(0) % width == 0 \
            and x.stride(0) >= x.size(1) * width:
        rows, seg_rows, seg_pitch = x.size(0) * x.size(1), x.size(1), x.stride(0) // width
    else:
        raise RuntimeError("x must be [rows, width] contiguous or [segments, rows, width] with contiguous rows")
    y = torch.empty((rows, width), dtype=x.dtype, device=x.device)
    res_out = None
    if residual is not None:
        require_cuda(residual, "residual", torch.bfloat16, 2)
        if residual.shape != y.shape:
            raise RuntimeError("residual must be [rows, width]")
        res_out = torch.empty_like(y)
    call("dyllm_add_rms_norm_segmented", ptr(x), seg_rows, seg_pitch, ptr(residual), ptr(weight), float(eps), ptr(y),
         ptr(res_out), rows, width, stream_ptr(x.device))
    return y if residual is None else (y, res_out)


def add_rms_norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None,
                      sel_idx: torch.Tensor, sel_count_dev: torch.Tensor | None = None, all_rows: bool = False):
    """RMSNorm (with the residual add) whose listed rows also come out packed in list order.  Returns
    ``(y_sel [len(sel_idx), width], new_residual [rows, width] or None, y_all [rows, width] or None)``: ``y_sel[m]`` is
    the normalised row ``sel_idx[m]`` (the packed input of a gathered GEMM), ``new_residual`` exists when a residual
    came in, ``y_all`` only with ``all_rows``.  ``x`` as for :func:`add_rms_norm`.

    ref: dyllm/model_executor/models/llada.py:176-185.
    """
    if not isinstance(x, torch.Tensor) or not x.is_cuda or x.dtype != torch.bfloat16:
        raise RuntimeError("x must be a CUDA bfloat16 tensor")
    require_cuda(weight, "weight", torch.bfloat16, 1)
    require_cuda(sel_idx, "sel_idx", torch.int32, 1)
    width = x.size(-1)
    if x.dim() == 2:
        require_cuda(x, "x", torch.bfloat16, 2)
        rows, seg_rows, seg_pitch = x.size(0), max(x.size(0), 1), max(x.size(0), 1)
    elif x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == width and x.stride(0) % width == 0 \
            and x.stride(0) >= x.size(1) * width:
        rows, seg_rows, seg_pitch = x.size(0) * x.size(1), x.size(1), x.stride(0) // width
    else:
        raise RuntimeError("x must be [rows, width] contiguous or [segments, rows, width] with contiguous rows")
    res_out = None
    if residual is not None:
        require_cuda(residual, "residual", torch.bfloat16, 2)
        if residual.shape != (rows, width):
            raise RuntimeError("residual must be [rows, width]")
        res_out = torch.empty_like(residual)
    elif not all_rows:
        raise RuntimeError("without a residual the normalised rows are the only output: pass all_rows=True")
    y_all = torch.empty((rows, width), dtype=x.dtype, device=x.device) if all_rows else None
    y_sel = torch.empty((sel_idx.numel(), width), dtype=x.dtype, device=x.device)
    call("dyllm_add_rms_norm_rows", ptr(x), seg_rows, seg_pitch, ptr(residual), ptr(weight), float(eps), ptr(y_all),
         ptr(res_out), rows, width, ptr(sel_idx), sel_idx.numel(), ptr(sel_count_dev), ptr(y_sel), stream_ptr(x.device))
    return y_sel, res_out, y_all


def head_rms_norm_(x: torch.Tensor, weight: torch.Tensor, eps: float, num_rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """In-place RMSNorm over the last dimension (128) of ``x [rows, heads, 128]``: the per-head q / k norm.

    ref: dyllm/model_executor/models/lladamoe.py:195-207.
    """
    require_cuda(x, "x", torch.bfloat16, 3)
    require_cuda(weight, "weight", torch.bfloat16, 1)
    call("dyllm_head_rms_norm", ptr(x), ptr(weight), float(eps), x.size(0), ptr(num_rows_dev), x.size(1), x.size(2),
         stream_ptr(x.device))
    return x


def rope_neox_(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, pos_idx: torch.Tensor | None = None,
               num_rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """In-place NeoX rotary embedding of ``x [rows, heads, 128]``.

    ref: dyllm/model_executor/layers/rotary_embedding.py:8-54.
    """
    require_cuda(x, "x", torch.bfloat16, 3)
    require_cuda(positions, "positions", torch.int64, 1)
    require_cuda(cos_sin, "cos_sin", torch.float32)
    if pos_idx is not None:
        require_cuda(pos_idx, "pos_idx", torch.int64, 1)
    call("dyllm_rope_neox", ptr(x), ptr(positions), ptr(pos_idx), ptr(cos_sin), x.size(0), ptr(num_rows_dev), x.size(1),
         x.size(2), cos_sin.size(0), stream_ptr(x.device))
    return x


def row_confidence(logits: torch.Tensor):
    """(max softmax probability fp32 [rows], its token int64 [rows]) of bf16 logits [rows, vocab].

    ref: dyllm/model_executor/layers/sampler.py:286-288.
    """
    require_cuda(logits, "logits", torch.bfloat16, 2)
    rows = logits.size(0)
    conf = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    token = torch.empty((rows,), dtype=torch.int64, device=logits.device)
    call("dyllm_row_confidence", ptr(logits), rows, logits.size(1), logits.stride(0), ptr(conf), ptr(token),
         stream_ptr(logits.device))
    return conf, token


def confidence_unmask_(conf: torch.Tensor, best_token: torch.Tensor, tokens: torch.Tensor, step_counter: torch.Tensor | None,
                       steps_per_block: int, prompt_len: int, block_len: int, num_transfer: int, mask_id: int,
                       picked_pos: torch.Tensor | None = None):
    """Unmasks, in place in ``tokens [batch, length]``, the ``num_transfer`` most confident still-masked positions
    of every sequence's current block and returns their positions ``[batch, num_transfer]`` (ascending; -1 padding).

    ref: dyllm/model_executor/layers/sampler.py:244-315.
    """
    require_cuda(conf, "conf", torch.float32, 2)
    require_cuda(best_token, "best_token", torch.int64, 2)
    if not (tokens.is_cuda and tokens.dtype == torch.int64 and tokens.dim() == 2 and tokens.stride(1) == 1):
        raise RuntimeError("tokens must be a CUDA int64 matrix with unit column stride")
    batch, length = tokens.shape
    num_blocks = (length - prompt_len) // block_len
    if picked_pos is None:
        picked_pos = torch.empty((batch, num_transfer), dtype=torch.int64, device=tokens.device)
    call("dyllm_confidence_unmask", ptr(conf), ptr(best_token), ptr(tokens), batch, tokens.stride(0), ptr(step_counter),
         int(steps_per_block), int(num_blocks), int(prompt_len), int(block_len), int(num_transfer), int(mask_id),
         ptr(picked_pos), None, stream_ptr(tokens.device))
    return picked_pos


def moe_route(x: torch.Tensor, router_weight: torch.Tensor, top_k: int, renormalize: bool = False,
              idx: torch.Tensor | None = None, num_rows: int | None = None, num_rows_dev: torch.Tensor | None = None):
    """fp32 softmax router with top-k selection; returns (weights fp32 [rows, k], expert ids int32 [rows, k]).

    ref: dyllm/model_executor/layers/fused_moe.py:375-407.
    """
    require_cuda(x, "x", torch.bfloat16, 2)
    require_cuda(router_weight, "router_weight", torch.bfloat16, 2)
    if num_rows is None:
        num_rows = idx.numel() if idx is not None else x.size(0)
    w = torch.empty((num_rows, top_k), dtype=torch.float32, device=x.device)
    ids = torch.empty((num_rows, top_k), dtype=torch.int32, device=x.device)
    call("dyllm_moe_route", ptr(x), x.size(0), x.size(1), x.stride(0), ptr(idx), num_rows, ptr(num_rows_dev),
         ptr(router_weight), router_weight.size(0), int(top_k), int(bool(renormalize)), ptr(w), ptr(ids),
         stream_ptr(x.device))
    return w, ids


def moe_ffn(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
            expert_start: int = 0, idx: torch.Tensor | None = None, num_rows: int | None = None,
            num_rows_dev: torch.Tensor | None = None, rows_hint: int = 0, out: torch.Tensor | None = None,
            out_row_map: torch.Tensor | None = None) -> torch.Tensor:
    """Expert-grouped SwiGLU FFN with the routing weights folded in and the top-k slots summed.

    ref: dyllm/model_executor/layers/fused_moe.py:269-335; dyllm/model_executor/models/lladamoe.py:107-142.
    """
    require_cuda(x, "x", torch.bfloat16, 2)
    require_cuda(w1, "w1", torch.bfloat16, 3)
    require_cuda(w2, "w2", torch.bfloat16, 3)
    require_cuda(topk_weights, "topk_weights", torch.float32, 2)
    require_cuda(topk_ids, "topk_ids", torch.int32, 2)
    e_local, hidden, inter = w2.size(0), w2.size(1), w2.size(2)
    if w1.shape != (e_local, 2 * inter, hidden):
        raise RuntimeError("w1 must be [E, 2 * inter, hidden] and w2 [E, hidden, inter]")
    top_k = topk_ids.size(1)
    if num_rows is None:
        num_rows = idx.numel() if idx is not None else x.size(0)
    if out is None:
        out = torch.empty((num_rows, hidden), dtype=torch.bfloat16, device=x.device)
    if num_rows == 0:
        return out
    ws = _gemm_workspace(load().dyllm_moe_ffn_workspace_bytes(num_rows, top_k, e_local, hidden, inter), x.device)
    call("dyllm_moe_ffn", ptr(x), x.size(0), hidden, x.stride(0), ptr(idx), num_rows, ptr(num_rows_dev), int(rows_hint),
         ptr(topk_weights), ptr(topk_ids), top_k, ptr(w1), ptr(w2), e_local, int(expert_start), inter, ptr(out),
         out.stride(0), ptr(out_row_map), ptr(ws), ws.numel(), stream_ptr(x.device))
    return out
