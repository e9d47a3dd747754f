"""CPU restatement of the reference's saliency hot path (scale-snu/DyLLM).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it is the checker
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``.  It is plain fp32 PyTorch on the CPU with numpy for the integer bookkeeping.

Each function cites the reference file:line it restates (paths relative to the reference project).

Pinning status
--------------
* ``cosine_mask`` / ``tensor_parallel_cosine_mask``: pinned by the reference's own known-answer test
  (tests/test_parallelism.py:34-44), reproduced in tests/test_oracle.py, and against the reference's
  Python imported in the development container (tests/golden/make_golden.py).
* ``compact``, ``swiglu_ffn``, ``moe_gate``, ``naive_experts``, ``rms_norm``, ``rope`` and the layer-level
  orchestration: pinned against the reference's Python run on CPU (tests/golden/make_golden.py writes
  the fixtures under tests/golden/).
* ``attention_sparse_varlen``, the cache functions, ``fused_offset``: the reference implements these only
  as CUDA kernels and ships no test or golden vector for them -> PARITY UNPINNED by the reference's
  tests; this module restates the kernels' arithmetic from their source.
* ``exact_attention_varlen`` stands for flash-attn 2.8.3 (third party, not vendored in the reference;
  pinned version from setup_env.sh:26-30): plain softmax attention, its published algorithm.
"""

from __future__ import annotations

import math

import numpy as np
import torch

BF16 = torch.bfloat16


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", torch.float32)


def _bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(BF16).to(torch.float32)


# --------------------------------------------------------------------------------------------------
# statistics, mask, compaction
# --------------------------------------------------------------------------------------------------
def context_stats(c_old: torch.Tensor, c_new: torch.Tensor) -> torch.Tensor:
    """[dot(new, old), |new|^2, |old|^2] per row over all trailing dims.

    ref: dyllm/csrc/attention/attention_ops_kernels_sm80.cu:436-443 and
    dyllm/csrc/attention/attention_aux_kernels.cu:34-41 (column order of ``cosine_stats``).
    """
    o = _f32(c_old).flatten(1)
    n = _f32(c_new).flatten(1)
    return torch.stack([(n * o).sum(-1), (n * n).sum(-1), (o * o).sum(-1)], dim=-1)


def cosine_mask(stats: torch.Tensor, threshold: float) -> torch.Tensor:
    """ref: dyllm/distributed/parallel_state.py:52-66; dyllm/csrc/attention/attention_aux_kernels.cu:10-20."""
    s = _f32(stats)
    dot = s[..., 0]
    a = s[..., 1].clamp_min(1e-8)
    b = s[..., 2].clamp_min(1e-8)
    cosine = dot * torch.rsqrt(a) * torch.rsqrt(b)
    return cosine < threshold


def cosine_values(stats: torch.Tensor) -> torch.Tensor:
    s = _f32(stats).double()
    return s[..., 0] / (s[..., 1].clamp_min(1e-8).sqrt() * s[..., 2].clamp_min(1e-8).sqrt())


def compact(mask: torch.Tensor, cu_seqlens_q: torch.Tensor):
    """Ascending selected rows and per-sequence prefix counts.

    ref: dyllm/model_executor/layers/attention.py:147-150 (``nonzero`` then ``searchsorted`` left).
    """
    m = np.asarray(mask.detach().cpu().numpy()).astype(bool)
    idx = np.flatnonzero(m).astype(np.int64)
    cu = np.asarray(cu_seqlens_q.detach().cpu().numpy()).astype(np.int64)
    cu_sal = np.searchsorted(idx, cu, side="left").astype(np.int32)
    return torch.from_numpy(idx), torch.from_numpy(cu_sal)


def fused_offset(idxs: torch.Tensor, cu_promptlens: torch.Tensor, cu_salientlens: torch.Tensor) -> torch.Tensor:
    """out[t] = idxs[t] + cu_promptlens[g + 1], g = group of t in cu_salientlens.

    ref: dyllm/csrc/attention/attention_aux_kernels.cu:112-128.
    """
    idx = np.asarray(idxs.detach().cpu().numpy()).astype(np.int64)
    cp = np.asarray(cu_promptlens.detach().cpu().numpy()).astype(np.int64)
    cs = np.asarray(cu_salientlens.detach().cpu().numpy()).astype(np.int64)
    t = np.arange(idx.shape[0])
    # first g with cs[g + 1] > t
    g = np.searchsorted(cs[1:], t, side="right")
    return torch.from_numpy(idx + cp[g + 1])


def salient_select(stats, threshold, cu_seqlens_q, cu_promptlens=None):
    """mask -> compact (-> K-space offsets).  ref: dyllm/model_executor/layers/attention.py:145-173."""
    mask = cosine_mask(stats, threshold)
    idx, cu_sal = compact(mask, cu_seqlens_q)
    out = {"mask": mask, "idx": idx, "cu_salientlens": cu_sal, "count": int(idx.numel())}
    if cu_promptlens is not None:
        out["idx_k"] = fused_offset(idx, cu_promptlens, cu_sal)
    return out


# --------------------------------------------------------------------------------------------------
# per-sequence activation cache
# --------------------------------------------------------------------------------------------------
def _np(t):
    return np.asarray(t.detach().cpu().numpy())


def cache_get_seqs(cache, seq_starts, cu_seqlens, seq_ids, total_rows, fill=0.0):
    """ref: dyllm/csrc/cache/cache_kernels.cu:18-64 (rows not covered by cu_seqlens stay unwritten)."""
    out = torch.full((int(total_rows), cache.size(1)), fill, dtype=cache.dtype)
    cu, ss, ids = _np(cu_seqlens), _np(seq_starts), _np(seq_ids)
    for b in range(len(ids)):
        n = int(cu[b + 1] - cu[b])
        if n <= 0:
            continue
        s0 = int(ss[ids[b]])
        out[int(cu[b]) : int(cu[b]) + n] = cache[s0 : s0 + n]
    return out


def cache_get_block(cache, seq_starts, cu_seqlens_k, cu_seqlens_q, seq_ids, total_rows, fill=0.0):
    """ref: dyllm/csrc/cache/cache_kernels.cu:200-247 (last len_q rows of each sequence)."""
    out = torch.full((int(total_rows), cache.size(1)), fill, dtype=cache.dtype)
    ck, cq, ss, ids = _np(cu_seqlens_k), _np(cu_seqlens_q), _np(seq_starts), _np(seq_ids)
    for b in range(len(ids)):
        n = int(cq[b + 1] - cq[b])
        if n <= 0:
            continue
        s0 = int(ss[ids[b]]) + int(ck[b + 1] - ck[b]) - n
        out[int(cq[b]) : int(cq[b]) + n] = cache[s0 : s0 + n]
    return out


def cache_reset_full(cache, inp, seq_starts, cu_seqlens, seq_ids):
    """In place.  ref: dyllm/csrc/cache/cache_kernels.cu:110-156."""
    cu, ss, ids = _np(cu_seqlens), _np(seq_starts), _np(seq_ids)
    for b in range(len(ids)):
        n = int(cu[b + 1] - cu[b])
        if n <= 0:
            continue
        s0 = int(ss[ids[b]])
        cache[s0 : s0 + n] = inp[int(cu[b]) : int(cu[b]) + n]
    return cache


def cache_reset_block(cache, inp, seq_starts, cu_seqlens_k, cu_seqlens_q, seq_ids):
    """In place.  ref: dyllm/csrc/cache/cache_kernels.cu:296-343."""
    ck, cq, ss, ids = _np(cu_seqlens_k), _np(cu_seqlens_q), _np(seq_starts), _np(seq_ids)
    for b in range(len(ids)):
        n = int(cq[b + 1] - cq[b])
        if n <= 0:
            continue
        s0 = int(ss[ids[b]]) + int(ck[b + 1] - ck[b]) - n
        cache[s0 : s0 + n] = inp[int(cq[b]) : int(cq[b]) + n]
    return cache


def cache_scatter_update(cache, new_vals, row_idx, cu_seqlens, seq_starts, seq_ids):
    """In place.  ref: dyllm/csrc/cache/cache_kernels.cu:388-426."""
    cu, ss, ids, rows = _np(cu_seqlens).astype(np.int64), _np(seq_starts), _np(seq_ids), _np(row_idx)
    for m in range(new_vals.size(0)):
        r = int(rows[m])
        b = int(np.searchsorted(cu[1:], r, side="right"))
        b = min(b, len(ids) - 1)
        dest = int(ss[ids[b]]) + r - int(cu[b])
        cache[dest] = new_vals[m]
    return cache


def delta_v_update(v_new, v_cache, rows):
    """dV of the step's salient rows and the value-cache update: ``dv = v_new - cache[rows]`` in the
    tensors' own dtype (bf16 in the reference: one rounding of the difference), then ``cache[rows] = v_new``
    in place.  Returns dv.  ref: dyllm/model_executor/layers/attention.py:67-74 (v_delta and the update of
    the gathered copy), :89-96 (the same rows written back to the cache by scatter_update)."""
    r = torch.as_tensor(_np(rows).astype(np.int64))
    dv = v_new - v_cache[r]
    v_cache[r] = v_new
    return dv


def kv_cache_update(k_new, v_new, rows_k, positions_of_rows, k_cache, v_cache, k_rows, v_rows, head_dim, base, max_position):
    """What the reference does between the K/V projection of the salient rows and the attention kernels:
    rotary embedding of the new keys (dyllm/model_executor/models/llada.py:110-130: the keys are placed in a
    zero tensor, rotated with every row's position and read back, i.e. row i is rotated with its own
    position), ``k_cache.scatter_update`` (llada.py:136-143) and the delta-V / value-cache update above.
    ``k_rows`` / ``v_rows`` are the cache rows of the salient tokens in the two caches.  In place; returns dv."""
    kr = rope(positions_of_rows, k_new, head_dim, base, max_position)
    k_cache[torch.as_tensor(_np(k_rows).astype(np.int64))] = kr.flatten(1).to(k_cache.dtype)
    return delta_v_update(v_new.flatten(1), v_cache, v_rows)


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
def exact_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, scale=None):
    """Non-causal varlen softmax attention, fp32.  Stands for ``flash_attn_varlen_func`` at the
    reference's call sites dyllm/model_executor/layers/attention.py:41-52,76-87.

    q [Tq, H, D], k/v [Tk, Hkv, D] -> [Tq, H, D] (fp32).
    """
    q, k, v = _f32(q), _f32(k), _f32(v)
    H, Hkv, D = q.size(1), k.size(1), q.size(2)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rep = H // Hkv
    out = torch.zeros_like(q)
    cq, ck = _np(cu_seqlens_q), _np(cu_seqlens_k)
    for b in range(len(cq) - 1):
        q0, q1, k0, k1 = int(cq[b]), int(cq[b + 1]), int(ck[b]), int(ck[b + 1])
        if q1 <= q0 or k1 <= k0:
            continue
        qb = q[q0:q1].transpose(0, 1)  # [H, Lq, D]
        kb = k[k0:k1].transpose(0, 1).repeat_interleave(rep, dim=0)
        vb = v[k0:k1].transpose(0, 1).repeat_interleave(rep, dim=0)
        p = torch.softmax(qb @ kb.transpose(1, 2) * scale, dim=-1)
        out[q0:q1] = (p @ vb).transpose(0, 1)
    return out


def attention_sparse_varlen(
    Q, K, V, C, o_sal, cu_seqlens_q, cu_seqlens_k, cu_salientlens, idx_salient_row, threshold,
    is_q_pruned=False, idx_salient_row_k=None, round_p_bf16=True, stats_in=None,
):
    """Approximate attention update ``O = bf16(C_old + softmax(Q K^T / sqrt(D)) dV)`` with the salient
    rows replaced by ``o_sal`` and the per-row cosine statistics.

    Returns (O bf16 [Tq,H,D], stats f32 [Tq,3], mask bool [Tq]).

    ref: dyllm/csrc/attention/attention_ops_kernels_sm80.cu:166-168 (scale 1/sqrt(D), exp2 domain),
    :278-359 (softmax over ALL keys of the sequence, P rounded to bf16 for the second product),
    :361-382 (P.dV on the 16-row chunks whose mask is non-zero; equal to the dense product because the
    caller's dV is zero on every other row), :396-451 (new = old + acc / rowsum, stats from the fp32
    value before rounding), :466-481 (stats added across heads);
    dyllm/csrc/attention/attention_aux_kernels.cu:22-72 (salient rows overwritten from bf16 o_sal,
    their stats recomputed from bf16 values), :10-20 (mask).
    """
    Qf, Kf, Vf, Cf = _f32(Q), _f32(K), _f32(V), _f32(C)
    Tq, H, D = Qf.shape
    Hkv = Kf.size(1)
    rep = H // Hkv
    scale = 1.0 / math.sqrt(D)
    cq, ck = _np(cu_seqlens_q), _np(cu_seqlens_k)
    new = Cf.clone()
    for b in range(len(cq) - 1):
        q0, q1, k0, k1 = int(cq[b]), int(cq[b + 1]), int(ck[b]), int(ck[b + 1])
        if q1 <= q0 or k1 <= k0:
            continue
        qb = Qf[q0:q1].transpose(0, 1)
        kb = Kf[k0:k1].transpose(0, 1).repeat_interleave(rep, dim=0)
        vb = Vf[k0:k1].transpose(0, 1).repeat_interleave(rep, dim=0)
        s = qb @ kb.transpose(1, 2) * scale
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        rowsum = p.sum(-1, keepdim=True)
        pv = (_bf16_round(p) if round_p_bf16 else p) @ vb
        new[q0:q1] = Cf[q0:q1] + (pv / rowsum).transpose(0, 1)
    O = new.to(BF16)
    stats = context_stats(Cf, new)
    if stats_in is not None:
        stats = stats + _f32(stats_in)
    idx = _np(idx_salient_row).astype(np.int64)
    if idx.size:
        osal = o_sal.detach().cpu().to(BF16)
        O[idx] = osal
        stats[idx] = context_stats(Cf[idx], osal.to(torch.float32))
    mask = cosine_mask(stats, threshold)
    return O, stats, mask


# --------------------------------------------------------------------------------------------------
# FFN, MoE, norms, rotary embedding
# --------------------------------------------------------------------------------------------------
def swiglu_ffn(x, w_gate_up, w_down, round_bf16=True):
    """down( silu(x Wg^T) * (x Wu^T) ), gate rows first in the merged weight.

    ref: dyllm/model_executor/models/llada.py:38-43; dyllm/model_executor/layers/linear.py:76-93,195-220;
    dyllm/model_executor/layers/activations.py:9-14.  With round_bf16 the intermediate tensors are
    rounded to bf16 where the reference's bf16 modules materialise them.
    """
    x, w1, w2 = _f32(x), _f32(w_gate_up), _f32(w_down)
    r = _bf16_round if round_bf16 else (lambda t: t)
    gu = r(x @ w1.t())
    g, u = gu.chunk(2, dim=-1)
    h = r(torch.nn.functional.silu(g) * u)
    return r(h @ w2.t())


def confidence_unmask(conf, best_token, tokens, block_start, block_len, num_transfer, mask_id):
    """Unmasking rule of the confidence sampler for one block (ref: dyllm/model_executor/layers/sampler.py:244-315:
    candidates = still-masked positions of the block, scores sorted descending per sequence, the first
    num_transfer kept; engine/sequence.py:69-75 writes the kept tokens).  Ties go to the lowest position.
    Returns (tokens_after, picked positions per sequence ascending)."""
    conf, best_token, tokens = _np(conf), _np(best_token), _np(tokens).copy()
    picked = []
    for b in range(tokens.shape[0]):
        cand = [i for i in range(block_len) if tokens[b, block_start + i] == mask_id]
        cand.sort(key=lambda i: (-float(conf[b, i]), i))
        keep = sorted(cand[:num_transfer])
        for i in keep:
            tokens[b, block_start + i] = best_token[b, i]
        picked.append([block_start + i for i in keep])
    return tokens, picked


def moe_gate(x, router_weight, top_k, renormalize=False):
    """fp32 softmax router, top-k.  ref: dyllm/model_executor/layers/fused_moe.py:375-407."""
    logits = _f32(x) @ _f32(router_weight).t()
    probs = torch.softmax(logits, dim=-1)
    w, i = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, i.to(torch.int32)


def naive_experts(x, w1, w2, topk_weights, topk_ids, round_bf16=True):
    """Per-expert loop, silu gate.  ref: dyllm/model_executor/layers/fused_moe.py:341-369."""
    x, w1, w2, tw = _f32(x), _f32(w1), _f32(w2), _f32(topk_weights)
    r = _bf16_round if round_bf16 else (lambda t: t)
    out = torch.zeros_like(x)
    for e in range(w1.size(0)):
        tok, slot = (topk_ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = r(x[tok] @ w1[e].t())
        g, u = gu.chunk(2, dim=-1)
        h = r(torch.nn.functional.silu(g) * u)
        y = (h @ w2[e].t()) * tw[tok, slot].unsqueeze(-1)
        out.index_add_(0, tok, r(y))
    return r(out)


def rms_norm(x, weight, eps, residual=None):
    """ref: dyllm/model_executor/layers/layernorm.py:17-41."""
    xf = _f32(x)
    if residual is not None:
        xf = xf + _f32(residual)
        res_out = xf.to(x.dtype)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    y = (xf * torch.rsqrt(var + eps)).to(x.dtype) * weight.to(x.dtype).cpu()
    return (y, res_out) if residual is not None else y


def rope(positions, x, head_dim, base, max_position):
    """NeoX-style rotary embedding.  ref: dyllm/model_executor/layers/rotary_embedding.py:8-54."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    pos = positions.detach().cpu().clamp(0, max_position - 1).to(torch.float)
    freqs = torch.einsum("i,j->ij", pos, inv_freq)
    cos, sin = freqs.cos().unsqueeze(1), freqs.sin().unsqueeze(1)
    x1, x2 = torch.chunk(_f32(x), 2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


# --------------------------------------------------------------------------------------------------
# seeded generators shared by tests, smoke() and bench.py
# --------------------------------------------------------------------------------------------------
def make_context_pair(rows, width, threshold=0.99, salient_fraction=0.10, seed=0, band=1e-4, response_rows=None):
    """Previous / current attention context with a controlled salient set.

    C_old ~ N(0,1); C_new = C_old + eps_r * n_r (both rounded to bf16).  About ``salient_fraction`` of the
    candidate rows get a cosine below ``threshold``; every row's cosine (evaluated in float64 on the
    bf16 values) is at least ``band`` away from the threshold.
    """
    g = torch.Generator().manual_seed(seed)
    c_old = torch.randn(rows, width, generator=g)
    noise = torch.randn(rows, width, generator=g)
    cand = torch.arange(rows) if response_rows is None else response_rows
    pick = torch.rand(rows, generator=g) < salient_fraction
    is_sal = torch.zeros(rows, dtype=torch.bool)
    is_sal[cand] = pick[cand]
    # cos ~ 1/sqrt(1+eps^2): eps 0.25 -> 0.970, eps 0.05 -> 0.9988
    eps = torch.where(is_sal, 0.20 + 0.15 * torch.rand(rows, generator=g), 0.01 + 0.05 * torch.rand(rows, generator=g))
    c_old_b = c_old.to(BF16)
    for _ in range(8):
        c_new_b = (c_old + eps.unsqueeze(1) * noise).to(BF16)
        cosv = cosine_values(context_stats(c_old_b, c_new_b))
        bad = (cosv - threshold).abs() < band
        if not bool(bad.any()):
            break
        eps = torch.where(bad, eps * 1.15, eps)
    return c_old_b, c_new_b


def make_batch_layout(batch, prompt, response, response_only, device="cpu"):
    """cu_seqlens_q / cu_seqlens_k / cu_promptlens for equal-length sequences."""
    L = prompt + response
    lq = response if response_only else L
    ar = torch.arange(batch + 1, dtype=torch.int32)
    return (ar * lq).to(device), (ar * L).to(device), (ar * prompt).to(device)
