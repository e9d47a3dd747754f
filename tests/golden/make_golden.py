"""Generates tests/golden/llada_layer_small.pt and tests/golden/llada_layer_c1.pt by running the REFERENCE's own Python
(`LLaDADecoderLayer`, `Attention`, `CacheManager`, `MLPcache`, `tensor_parallel_cosine_mask`, ...) on the CPU with
bf16 modules and caches (as the reference runs them on a GPU; in fp32 its in-place RMSNorm would alias
the residual), with the three native modules it imports replaced by the oracle's fp32 restatements.

Run in the development container only (it needs the reference checkout):

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/reference [small|c1|dream|moe]

"small" is a toy LLaDA shape; "dream" a toy Dream layer (grouped-query attention, biased q/k/v; the
reference's DreamDecoderLayer); "moe" a toy LLaDA-MoE layer (per-head q/k RMSNorm, 8 experts top-2; the
reference's LLaDAMoEDecoderLayer with its own naive_experts loop standing for its Triton grouped GEMM); "c1" is the single-layer LLaDA-8B configuration (hidden 4096, 32 heads of 128, FFN
intermediate 12288, one sequence of 256 prompt + 256 response positions).  The inputs are bimodal: the
listed rows and a few more response rows change a lot between steps, all others little, and the generator
asserts that every cosine the reference computes lies at least 1e-4 from the threshold.  A fixture holds seeds, shapes and outputs (for "c1": the
outputs of a fixed subset of rows in bf16 plus per-row sums and norms of all rows, to stay small); weights
and inputs are regenerated from the seeds by `golden_inputs()` below, which the tests import.
"""
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CONFIGS = {
    "small": dict(shape=dict(hidden=256, heads=2, kv_heads=2, head_dim=128, inter=512, eps=1e-5, theta=500000.0, max_pos=512),
                  batch=2, prompt=24, resp=40, seq_ids=[5, 3], seed=1234, wscale=0.05,
                  salient={1: [[1, 7, 20], [3, 33]], 2: [[2, 9], [5, 30, 31]]}, extra=5, margin=0.0, subset=None),
    "c1": dict(shape=dict(hidden=4096, heads=32, kv_heads=32, head_dim=128, inter=12288, eps=1e-5, theta=500000.0, max_pos=4096),
               batch=1, prompt=256, resp=256, seq_ids=[0], seed=4321, wscale=0.02,
               salient={1: [[3, 40, 41, 97, 130, 200, 255]], 2: [[0, 17, 64, 128, 129, 250]]}, extra=20, margin=1e-4,
               subset=64),
}
CONFIGS["dream"] = dict(shape=dict(hidden=512, heads=4, kv_heads=2, head_dim=128, inter=1024, eps=1e-6, theta=1000000.0, max_pos=512),
                        family="dream", batch=2, prompt=24, resp=40, seq_ids=[1, 4], seed=2234, wscale=0.05,
                        salient={1: [[1, 7, 20], [3, 33]], 2: [[2, 9], [5, 30, 31]]}, extra=5, margin=0.0, subset=None)
CONFIGS["moe"] = dict(shape=dict(hidden=256, heads=2, kv_heads=2, head_dim=128, inter=128, eps=1e-5, theta=50000.0, max_pos=512,
                                 experts=8, top_k=2),
                      family="lladamoe", batch=2, prompt=24, resp=40, seq_ids=[2, 0], seed=3234, wscale=0.05,
                      salient={1: [[1, 7, 20], [3, 33]], 2: [[2, 9], [5, 30, 31]]}, extra=5, margin=0.0, subset=None)
TAU = 0.99
_cfg = CONFIGS["small"]
SHAPE, BATCH, PROMPT, RESP = _cfg["shape"], _cfg["batch"], _cfg["prompt"], _cfg["resp"]


def use_config(name):
    """Selects the configuration the module-level names (SHAPE, BATCH, PROMPT, RESP) and the functions below
    refer to."""
    global _cfg, SHAPE, BATCH, PROMPT, RESP
    _cfg = CONFIGS[name]
    SHAPE, BATCH, PROMPT, RESP = _cfg["shape"], _cfg["batch"], _cfg["prompt"], _cfg["resp"]
    return _cfg


def golden_inputs(seed=None):
    """Weights N(0, 0.02) (a larger scale for the value/FFN paths keeps cosines spread around the
    threshold) and three hidden-state inputs, all from one CPU generator."""
    g = torch.Generator().manual_seed(_cfg["seed"] if seed is None else seed)
    ws = _cfg["wscale"]
    h, H, Hkv, D, I = SHAPE["hidden"], SHAPE["heads"], SHAPE["kv_heads"], SHAPE["head_dim"], SHAPE["inter"]
    w = {
        "q_proj": torch.randn(H * D, h, generator=g) * ws,
        "kv_proj": torch.randn(2 * Hkv * D, h, generator=g) * ws,
        "o_proj": torch.randn(h, H * D, generator=g) * ws,
        "gate_up_proj": torch.randn(2 * I, h, generator=g) * ws,
        "down_proj": torch.randn(h, I, generator=g) * ws,
    }
    fam = _cfg.get("family", "llada")
    if fam == "dream":          # biased q / k / v projections
        w["q_bias"] = torch.randn(H * D, generator=g) * 0.1
        w["kv_bias"] = torch.randn(2 * Hkv * D, generator=g) * 0.1
    if fam == "lladamoe":       # per-head q / k norm weights, router, experts (gate rows first)
        E = SHAPE["experts"]
        w["q_norm"] = 1.0 + 0.1 * torch.randn(D, generator=g)
        w["k_norm"] = 1.0 + 0.1 * torch.randn(D, generator=g)
        w["router"] = torch.randn(E, h, generator=g) * 0.3
        w["experts_gate_up"] = torch.randn(E, 2 * I, h, generator=g) * ws
        w["experts_down"] = torch.randn(E, h, I, generator=g) * ws
        del w["gate_up_proj"], w["down_proj"]
    w = {k: v.bfloat16().float() for k, v in w.items()}
    L = PROMPT + RESP
    x0 = torch.randn(BATCH * L, h, generator=g).bfloat16().float()
    # later steps: small perturbations of the same hidden states, large ones on the rows the step lists
    # as salient (their tokens changed) and medium ones on a few more response rows
    xs = [x0]
    for step in (1, 2):
        bump = torch.zeros(BATCH * L, 1)
        for b in range(BATCH):
            bump[b * L + PROMPT + torch.randperm(RESP, generator=g)[:_cfg["extra"]]] = 0.05 if _cfg["margin"] == 0.0 else 0.6
            for p in step_layout(step)[2][b]:
                bump[b * L + p] = 0.6
        xs.append((xs[-1] + (0.003 + bump) * torch.randn(BATCH * L, h, generator=g)).bfloat16().float())
    return w, xs


def step_layout(step):
    """(is_full, response_only, initial salient positions per sequence) of the three recorded steps."""
    if step == 0:
        return True, False, None
    sal = [[PROMPT + o for o in seq] for seq in _cfg["salient"][step]]
    return False, step == 2, sal


def load_layer_weights(layer, w):
    """Copies golden_inputs() weights into a decoder layer with the reference's module tree (either
    implementation; which tensors exist depends on the model family)."""
    with torch.no_grad():
        layer.self_attn.q_proj.weight.copy_(w["q_proj"])
        layer.self_attn.kv_proj.weight.copy_(w["kv_proj"])
        layer.self_attn.o_proj.weight.copy_(w["o_proj"])
        if "q_bias" in w:
            layer.self_attn.q_proj.bias.copy_(w["q_bias"])
            layer.self_attn.kv_proj.bias.copy_(w["kv_bias"])
        if "q_norm" in w:
            layer.self_attn.q_norm.weight.copy_(w["q_norm"])
            layer.self_attn.k_norm.weight.copy_(w["k_norm"])
        if "router" in w:
            layer.mlp.gate.weight.copy_(w["router"])
            layer.mlp.gate_up_proj.copy_(w["experts_gate_up"])
            layer.mlp.down_proj.copy_(w["experts_down"])
        else:
            layer.mlp.gate_up_proj.weight.copy_(w["gate_up_proj"])
            layer.mlp.down_proj.weight.copy_(w["down_proj"])
        layer.input_layernorm.weight.fill_(1.0)
        layer.post_attention_layernorm.weight.fill_(1.0)


def subset_rows(rows, salient_idx):
    """The rows whose outputs a compact fixture keeps: every salient row and an even spread of the others."""
    n = _cfg["subset"]
    keep = set(int(i) for i in (salient_idx.tolist() if salient_idx is not None else []))
    keep.update(range(0, rows, max(1, rows // n)))
    return torch.tensor(sorted(keep), dtype=torch.long)


def pack_rows(out, residual, is_full, salient_idx):
    """Full fp32 outputs for the toy shape; for the large one the outputs of subset_rows() in bf16 and per-row
    sums / norms of every row."""
    if _cfg["subset"] is None:
        return {"out": out.float().clone(), "residual": residual.float().clone()}
    rows = subset_rows(out.size(0), salient_idx)
    o, r = out.float(), residual.float()
    return {"rows": rows, "out_rows": out[rows].to(torch.bfloat16).clone(), "residual_rows": residual[rows].to(torch.bfloat16).clone(),
            "out_sum": o.sum(1), "out_norm": o.norm(dim=1), "residual_sum": r.sum(1), "residual_norm": r.norm(dim=1)}


def main(ref_root, config="small"):
    use_config(config)
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    import torch.distributed as dist
    from oracle import dyllm_oracle as orc

    # --- stand-ins for the reference's three native modules ------------------------------------
    pkg = types.ModuleType("dyllm")
    pkg.__path__ = [os.path.join(ref_root, "dyllm")]
    sys.modules["dyllm"] = pkg
    cache_mod = types.ModuleType("dyllm.cache")
    cache_mod.get_seqs_cuda = lambda cache, ss, cu, ids, total: orc.cache_get_seqs(cache, ss, cu, ids, total)
    cache_mod.get_block_cuda = lambda cache, ss, cu, cuq, ids, total: orc.cache_get_block(cache, ss, cu, cuq, ids, total)
    cache_mod.reset_full_cuda = lambda cache, inp, ss, cu, ids, total: orc.cache_reset_full(cache, inp, ss, cu, ids)
    cache_mod.reset_block_cuda = lambda cache, inp, ss, cu, cuq, ids, total: orc.cache_reset_block(cache, inp, ss, cu, cuq, ids)
    cache_mod.scatter_update_cuda = lambda cache, new, rows, cu, ss, ids: orc.cache_scatter_update(cache, new, rows, cu, ss, ids)
    sys.modules["dyllm.cache"] = cache_mod

    def attention_sparse_varlen(Q, K, V, C, o_sal, cu_q, cu_k, max_q, max_k, total, cu_sal, idx, stats, mask_out,
                                threshold=0.0, is_q_pruned=False, idx_k=None, force=-1):
        O, st, mask = orc.attention_sparse_varlen(Q, K, V, C, o_sal, cu_q, cu_k, cu_sal, idx, threshold,
                                                  round_p_bf16=False, stats_in=stats)
        stats.copy_(st)
        mask_out.copy_(mask)
        return O.to(Q.dtype)

    def fused_offset_launch(idxs, num_idxs, cu_p, cu_sal, out, max_threads):
        n = int(num_idxs.item())
        out[:n] = orc.fused_offset(idxs[:n], cu_p, cu_sal)

    ops_mod = types.ModuleType("dyllm.attention_ops")
    ops_mod.attention_sparse_varlen = attention_sparse_varlen
    ops_mod.fused_offset_launch = fused_offset_launch
    sys.modules["dyllm.attention_ops"] = ops_mod
    fa = types.ModuleType("flash_attn")
    fa.flash_attn_varlen_func = lambda q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal: \
        orc.exact_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, softmax_scale).to(q.dtype)
    sys.modules["flash_attn"] = fa
    torch.cuda.nvtx.range_pop = lambda: None

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1)
    import dyllm.engine.cache_manager as cm

    cm.CacheManager.__init__.__defaults__ = (16384, torch.bfloat16, torch.device("cpu"))
    import dyllm.distributed as ddist
    import dyllm.model_executor.layers.attention as ref_attn

    seen_stats = []
    real_mask = ddist.tensor_parallel_cosine_mask

    def recording_mask(stats, threshold):
        seen_stats.append(stats.clone())
        return real_mask(stats, threshold)

    ref_attn.tensor_parallel_cosine_mask = recording_mask
    from dyllm.utils.context import get_context, set_context
    from dyllm.utils.metadata import get_metadata, set_metadata

    fam = _cfg.get("family", "llada")
    common = dict(hidden_size=SHAPE["hidden"], num_attention_heads=SHAPE["heads"], rms_norm_eps=SHAPE["eps"],
                  head_dim=SHAPE["head_dim"], rope_theta=SHAPE["theta"])
    if fam == "dream":
        from dyllm.model_executor.models.dream import DreamDecoderLayer

        cfg = types.SimpleNamespace(num_key_value_heads=SHAPE["kv_heads"], max_position_embeddings=SHAPE["max_pos"],
                                    intermediate_size=SHAPE["inter"], **common)
        layer = DreamDecoderLayer(cfg, TAU).bfloat16()
    elif fam == "lladamoe":
        ddist.initialize_parallel_state(1)
        import dyllm.model_executor.layers.fused_moe as fm
        import dyllm.model_executor.models.lladamoe as lm

        # the reference's own per-expert loop (fused_moe.py:341-369) stands for its Triton grouped GEMM
        lm.fused_experts = lambda x, w1, w2, tw, ti, activation="silu": fm.naive_experts(x, w1, w2, tw, ti, activation)
        cfg = types.SimpleNamespace(num_key_value_heads=SHAPE["kv_heads"], max_position_embeddings=SHAPE["max_pos"],
                                    num_experts=SHAPE["experts"], num_experts_per_tok=SHAPE["top_k"],
                                    expert_intermediate_size=SHAPE["inter"], norm_topk_prob=False, qk_layernorm=True,
                                    attention_bias=False, **common)
        layer = lm.LLaDAMoEDecoderLayer(cfg, TAU).bfloat16()
    else:
        from dyllm.model_executor.models.llada import LLaDADecoderLayer

        cfg = types.SimpleNamespace(n_kv_heads=SHAPE["kv_heads"], max_sequence_length=SHAPE["max_pos"],
                                    mlp_hidden_size=SHAPE["inter"], **common)
        layer = LLaDADecoderLayer(cfg, TAU).bfloat16()
    w, xs = golden_inputs()
    load_layer_weights(layer, w)

    L = PROMPT + RESP
    seq_ids = _cfg["seq_ids"]
    record = {"config": config, "shape": SHAPE, "batch": BATCH, "prompt": PROMPT, "resp": RESP, "tau": TAU, "seq_ids": seq_ids, "steps": []}
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    for step in range(3):
        is_full, ro, sal = step_layout(step)
        set_metadata(seq_ids, seq_ids, [])
        get_metadata().running_seqs_tensor = torch.tensor(seq_ids, dtype=torch.long)
        cu_k = [b * L for b in range(BATCH + 1)]
        if is_full:
            positions = torch.arange(L).repeat(BATCH)
            set_context(True, cu_seqlens_q=i32(cu_k), cu_seqlens_q_cpu=cu_k, cu_seqlens_k=i32(cu_k), max_seqlen_q=L,
                        max_seqlen_k=L, context_lens=i32([L] * BATCH), context_lens_cpu=[L] * BATCH, total_seqlen=BATCH * L)
            x = xs[step]
        else:
            lq = RESP if ro else L
            cu_q = [b * lq for b in range(BATCH + 1)]
            idx_q, idx_k, cu_sal = [], [], [0]
            for b in range(BATCH):
                for p in sal[b]:
                    idx_q.append((p - PROMPT if ro else p) + cu_q[b])
                    idx_k.append(p + cu_k[b])
                cu_sal.append(len(idx_q))
            positions = (torch.arange(PROMPT, L) if ro else torch.arange(L)).repeat(BATCH)
            set_context(False, cu_seqlens_q=i32(cu_q), cu_seqlens_q_cpu=cu_q, cu_seqlens_k=i32(cu_k),
                        cu_promptlens=i32([b * PROMPT for b in range(BATCH + 1)]), cu_salientlens=i32(cu_sal),
                        max_seqlen_q=lq, max_seqlen_k=L, idx_salient_row=torch.tensor(idx_q, dtype=torch.long),
                        idx_salient_row_k=torch.tensor(idx_k, dtype=torch.long) if ro else None,
                        context_lens=i32([L] * BATCH), context_lens_cpu=[L] * BATCH, total_seqlen_k=BATCH * L,
                        total_seqlen=BATCH * lq)
            x = xs[step].view(BATCH, L, -1)[:, PROMPT:].reshape(BATCH * RESP, -1) if ro else xs[step]
        with torch.no_grad():
            out, residual = layer(positions, x.clone().bfloat16(), None)
        ctx = get_context()
        rec = pack_rows(out, residual, is_full, None if is_full else ctx.idx_salient_row)
        if not is_full:
            rec["cosine"] = orc.cosine_values(seen_stats[-1]).float()
            gap = float((rec["cosine"] - TAU).abs().min())
            print("   min |cos - tau| =", gap)
            print("   rows within 2e-3 of tau:", int(((rec["cosine"] - TAU).abs() < 2e-3).sum()), "of", rec["cosine"].numel())
            assert gap >= _cfg["margin"], "a cosine lies inside the margin: change the seed"
            rec["idx_salient_row"] = ctx.idx_salient_row.clone()
            rec["cu_salientlens"] = ctx.cu_salientlens.clone()
            if ro:
                rec["idx_salient_row_k"] = ctx.idx_salient_row_k.clone()
        record["steps"].append(rec)
        print("step", step, "out", tuple(out.shape), "salient", None if is_full else ctx.idx_salient_row.tolist())
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), f"llada_layer_{config}.pt")
    torch.save(record, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference [small|c1|dream|moe]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else "small")
