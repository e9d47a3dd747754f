"""Self-check of the tensor-parallel path on the machine it runs on: one LLaDA-8B-shaped decoder layer
(hidden 4096, 32 heads of 128, FFN intermediate 12288) takes a dense step and a sparse step, once sharded
over all ranks (every collective of the path included) and once, on rank 0 only, unsharded from the same
seeded weights.  Reported: whether the two salient sets agree on every row whose cosine is clear of the
threshold, and the distance between the two layer outputs.

The sharded and the unsharded layer compute the same function with different rounding: each rank rounds its
partial o_proj / down-projection sums to bf16 before they are added (as the reference does,
dyllm/model_executor/layers/linear.py:216-220).
"""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from . import layers, model as model_mod, ops
from .context import get_context, get_metadata, set_context, set_metadata

BAND = 2e-3      # decisions are compared where the unsharded cosine is at least this far from the threshold


@contextlib.contextmanager
def _single_rank():
    """Makes the layer classes see a world of one rank (construction and forward of the unsharded layer)."""
    saved = layers._tp_comm
    layers._tp_comm = None
    try:
        with layers.replicated():
            yield
    finally:
        layers._tp_comm = saved


def _build_layer(dev, shape, tau, seed):
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            layer = model_mod.LLaDADecoderLayer(shape, tau)
    finally:
        torch.set_default_dtype(torch.float32)
    model_mod.init_weights_(layer, seed=seed, std=0.02)
    return layer.eval()


def _two_steps(layer, dev, xs, B, P, R, sal_pos, seq_ids):
    """Dense step on xs[0], then a full-sequence sparse step on xs[1] whose initial salient rows are
    ``sal_pos``.  Returns (output of the sparse step, new salient rows, the statistics the selection saw)."""
    L = P + R
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    cu = [b * L for b in range(B + 1)]
    positions = torch.arange(L, device=dev).repeat(B)
    seen = {}
    real_select = ops.salient_select

    def recording_select(stats, *a, **k):
        seen["stats"] = stats.clone()
        return real_select(stats, *a, **k)

    with torch.inference_mode():
        set_metadata(seq_ids, seq_ids, [])
        get_metadata().running_seqs_tensor = torch.tensor(seq_ids, dtype=torch.long, device=dev)
        set_context(True, cu_seqlens_q=i32(cu), cu_seqlens_q_cpu=cu, cu_seqlens_k=i32(cu), max_seqlen_q=L, max_seqlen_k=L,
                    context_lens=i32([L] * B), context_lens_cpu=[L] * B, total_seqlen=B * L, total_seqlen_k=B * L)
        layer(positions, xs[0].clone(), None)
        idx = [p + cu[b] for b in range(B) for p in sal_pos[b]]
        cu_sal = [0]
        for b in range(B):
            cu_sal.append(cu_sal[-1] + len(sal_pos[b]))
        set_context(False, cu_seqlens_q=i32(cu), cu_seqlens_q_cpu=cu, cu_seqlens_k=i32(cu),
                    cu_promptlens=i32([b * P for b in range(B + 1)]), cu_salientlens=i32(cu_sal), max_seqlen_q=L,
                    max_seqlen_k=L, idx_salient_row=torch.tensor(idx, dtype=torch.long, device=dev),
                    idx_salient_row_k=None, idx_salient_row32=i32(idx), max_salient_per_seq=max(len(s) for s in sal_pos),
                    context_lens=i32([L] * B), context_lens_cpu=[L] * B, total_seqlen_k=B * L, total_seqlen=B * L)
        ops.salient_select = layers.ops.salient_select = recording_select
        try:
            out, residual = layer(positions, xs[1].clone(), None)
        finally:
            ops.salient_select = layers.ops.salient_select = real_select
        rows, _ = get_context().salient_rows()
    return out.float(), rows.clone(), seen["stats"]


def run(dev: torch.device, tau: float = 0.99, seed: int = 7) -> dict:
    """Collective over the default process group (call it on every rank).  Returns the report on rank 0 and
    ``None`` elsewhere."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    shape = model_mod.LLaDAShape(num_hidden_layers=1, max_sequence_length=1024)
    B, P, R = 2, 256, 256
    L = P + R
    g = torch.Generator(device=dev).manual_seed(seed)
    x0 = torch.randn(B * L, shape.hidden_size, generator=g, device=dev).bfloat16()
    sal_pos = [[P + 3, P + 40, P + 41, P + 200], [P + 0, P + 17, P + 128, P + 129, P + 250]]
    bump = torch.full((B * L, 1), 0.003, device=dev)
    for b in range(B):
        for p in sal_pos[b]:
            bump[b * L + p] = 0.6
        extra = torch.randperm(R, generator=g, device=dev)[:20] + P + b * L
        bump[extra] = 0.6
    x1 = (x0.float() + bump * torch.randn(B * L, shape.hidden_size, generator=g, device=dev)).bfloat16()

    sharded = _build_layer(dev, shape, tau, seed)
    out_tp, rows_tp, _ = _two_steps(sharded, dev, (x0, x1), B, P, R, sal_pos, [0, 1])
    torch.cuda.synchronize(dev)
    report = None
    if rank == 0:
        with _single_rank():
            single = _build_layer(dev, shape, tau, seed)
            out_1, rows_1, stats_1 = _two_steps(single, dev, (x0, x1), B, P, R, sal_pos, [0, 1])
        cos = stats_1[:, 0].double() / (stats_1[:, 1].double().clamp_min(1e-8).sqrt() * stats_1[:, 2].double().clamp_min(1e-8).sqrt())
        clear = (cos - tau).abs() >= BAND
        m_tp = torch.zeros(B * L, dtype=torch.bool, device=dev)
        m_tp[rows_tp] = True
        m_1 = torch.zeros(B * L, dtype=torch.bool, device=dev)
        m_1[rows_1] = True
        same_rows = clear & (m_tp == m_1)
        diff = (out_tp - out_1)[same_rows]
        ref = out_1[same_rows]
        report = {
            "world": world, "rows": B * L, "salient_unsharded": int(m_1.sum()), "salient_sharded": int(m_tp.sum()),
            "rows_clear_of_band": int(clear.sum()), "decisions_equal_outside_band": bool(torch.equal(m_tp[clear], m_1[clear])),
            "out_rel_l2": float(diff.norm() / ref.norm()), "out_max_abs": float(diff.abs().max()),
            "out_peak": float(ref.abs().max()),
        }
        report["ok"] = bool(report["decisions_equal_outside_band"] and report["out_rel_l2"] <= 2e-2)
        del single
    del sharded
    if world > 1:
        dist.barrier()
    return report
