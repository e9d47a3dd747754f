"""Generates tests/golden/llada_tokens_small.pt: the token ids the REFERENCE's own step loop unmasks over a
fixed number of denoising steps of a small LLaDA-shaped model, run on the CPU with bf16 modules.

What runs is the reference's Python: ``ModelRunner.prepare_full`` / ``prepare_sparse`` / ``prepare_sample``
(dyllm/engine/model_runner.py:140-372), ``LLaDAForDLM`` (dyllm/model_executor/models/llada.py), ``LLaDASampler``
(dyllm/model_executor/layers/sampler.py:244-315), ``Sequence.update_token`` / ``update_block_idx`` and the
scheduler's step counting (dyllm/engine/scheduler.py:29-75: ``processed_steps`` is incremented before a step,
the first ``num_full_steps`` steps are dense).  Stand-ins, all on the CPU: the three native modules and
flash-attn are the oracle's restatements (pinned against the reference's kernels by tests/test_ref_golden.py);
the sampler's three Triton helpers (``triton_repeat_interleave``, ``launch_ragged_to_dense``,
``launch_filter_and_count``, sampler.py:16-175) are restated in torch below; ``.cuda()`` / pinned memory are
no-ops.

Besides the chosen (position, token) pairs the fixture records, per step: every candidate row's confidence
(fp32 softmax maximum of the reference's logits), its best token and that token's lead over the runner-up; how
clear the choice among the rows was (margin between the last chosen and the first rejected confidence); and
the cosines every layer's selection saw.  A test can then compare the confidences numerically, require equal
tokens and rows wherever the reference's choice does not hinge on rounding, and notice when a salient decision
inside the rounding band forks the two runs.

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_token_golden.py /path/to/reference
"""
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CFG = dict(hidden=256, heads=2, kv_heads=2, head_dim=128, inter=512, layers=2, vocab=512, eps=1e-5, theta=500000.0,
           max_pos=256, batch=2, prompt=24, gen=32, block=16, steps=32, full_steps=4, tau=0.99, seed=77,
           head_std=0.6, std=0.05)
MASK_ID = CFG["vocab"] - 1


def token_model_weights():
    """name -> tensor for the small model (bf16-representable), from one CPU generator; shared with the test."""
    g = torch.Generator().manual_seed(CFG["seed"])
    h, H, Hkv, D, I, V = CFG["hidden"], CFG["heads"], CFG["kv_heads"], CFG["head_dim"], CFG["inter"], CFG["vocab"]
    r = lambda *shape, std=CFG["std"]: (torch.randn(*shape, generator=g) * std).bfloat16().float()
    w = {"embed": r(V, h, std=1.0), "lm_head": r(V, h, std=CFG["head_std"])}
    for i in range(CFG["layers"]):
        w[f"{i}.q_proj"] = r(H * D, h)
        w[f"{i}.kv_proj"] = r(2 * Hkv * D, h)
        w[f"{i}.o_proj"] = r(h, H * D)
        w[f"{i}.gate_up_proj"] = r(2 * I, h)
        w[f"{i}.down_proj"] = r(h, I)
    return w


def token_prompts():
    g = torch.Generator().manual_seed(CFG["seed"] + 1)
    return torch.randint(0, MASK_ID, (CFG["batch"], CFG["prompt"]), generator=g).tolist()


def load_weights_into(model, w):
    """Copies token_model_weights() into a model with the reference's module tree (either implementation)."""
    with torch.no_grad():
        model.model.embed_tokens.weight.copy_(w["embed"])
        model.lm_head.weight.copy_(w["lm_head"])
        for i, layer in enumerate(model.model.layers):
            layer.self_attn.q_proj.weight.copy_(w[f"{i}.q_proj"])
            layer.self_attn.kv_proj.weight.copy_(w[f"{i}.kv_proj"])
            layer.self_attn.o_proj.weight.copy_(w[f"{i}.o_proj"])
            layer.mlp.gate_up_proj.weight.copy_(w[f"{i}.gate_up_proj"])
            layer.mlp.down_proj.weight.copy_(w[f"{i}.down_proj"])
            layer.input_layernorm.weight.fill_(1.0)
            layer.post_attention_layernorm.weight.fill_(1.0)
        model.model.norm.weight.fill_(1.0)


def _install_standins(ref_root):
    from oracle import dyllm_oracle as orc

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
        O, st, mask = orc.attention_sparse_varlen(Q, K, V, C, o_sal, cu_q, cu_k, cu_sal, idx, threshold, stats_in=stats)
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

    # no GPU here: device moves and pinning are no-ops
    real_tensor, real_to = torch.tensor, torch.Tensor.to
    torch.tensor = lambda *a, pin_memory=False, **k: real_tensor(*a, **k)
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.Tensor.pin_memory = lambda self, *a, **k: self

    def to(self, *a, **k):
        if k.get("device") == "cuda":
            k = {key: v for key, v in k.items() if key not in ("device", "non_blocking")}
            return real_to(self, *a, **k) if (a or k) else self
        return real_to(self, *a, **k)

    torch.Tensor.to = to


def _sampler_standins(sampler_mod):
    """Torch restatements of the sampler's Triton helpers (dyllm/model_executor/layers/sampler.py:16-175)."""

    def repeat_interleave(cu_filtered, total_tokens, out_tensor):
        counts = (cu_filtered[1:] - cu_filtered[:-1]).long()
        out_tensor.copy_(torch.repeat_interleave(torch.arange(counts.numel()), counts))
        return out_tensor

    def ragged_to_dense(scores, tokens, pos, cu_seqlens, B, max_len=32):
        ds = torch.full((B, max_len), float("-inf"), dtype=scores.dtype)
        dt = torch.zeros((B, max_len), dtype=tokens.dtype)
        dp = torch.zeros((B, max_len), dtype=pos.dtype)
        for b in range(B):
            s, e = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
            n = min(e - s, max_len)
            ds[b, :n], dt[b, :n], dp[b, :n] = scores[s:s + n], tokens[s:s + n], pos[s:s + n]
        return ds, dt, dp

    def filter_and_count(dense_scores, dense_tokens, dense_pos, num_transfer, conf_thr, B, max_len):
        offs = torch.arange(max_len).unsqueeze(0)
        keep = ((offs < num_transfer.view(-1, 1)) | (dense_scores >= conf_thr.view(-1, 1))) & (dense_scores > float("-inf"))
        out_tokens = torch.where(keep, dense_tokens, torch.full_like(dense_tokens, -1))
        out_pos = torch.where(keep, dense_pos, torch.zeros_like(dense_pos))
        return out_pos, out_tokens, keep.sum(1).to(torch.int32)

    sampler_mod.triton_repeat_interleave = repeat_interleave
    sampler_mod.launch_ragged_to_dense = ragged_to_dense
    sampler_mod.launch_filter_and_count = filter_and_count


def main(ref_root):
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    import torch.distributed as dist

    _install_standins(ref_root)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29534", rank=0, world_size=1)
    import dyllm.engine.cache_manager as cm

    cm.CacheManager.__init__.__defaults__ = (16384, torch.bfloat16, torch.device("cpu"))
    import dyllm.model_executor.layers.sampler as sampler_mod
    from dyllm.engine.model_runner import ModelRunner
    from dyllm.engine.sequence import Sequence
    from dyllm.model_executor.models.llada import LLaDAForDLM
    from dyllm.sampling_params import SamplingParams
    from dyllm.utils.context import get_context, reset_context
    from dyllm.utils.metadata import get_metadata, set_metadata

    _sampler_standins(sampler_mod)
    # record the cosines every layer's selection sees (dyllm/distributed/parallel_state.py:52-66)
    import dyllm.distributed as ddist
    import dyllm.model_executor.layers.attention as ref_attn
    from oracle import dyllm_oracle as orc

    seen_cos = []
    real_mask = ddist.tensor_parallel_cosine_mask

    def recording_mask(stats, threshold):
        seen_cos.append(orc.cosine_values(stats).float())
        return real_mask(stats, threshold)

    ref_attn.tensor_parallel_cosine_mask = recording_mask
    c = CFG
    cfg = types.SimpleNamespace(hidden_size=c["hidden"], num_attention_heads=c["heads"], n_kv_heads=c["kv_heads"],
                                max_sequence_length=c["max_pos"], rms_norm_eps=c["eps"], head_dim=c["head_dim"],
                                rope_theta=c["theta"], mlp_hidden_size=c["inter"], num_hidden_layers=c["layers"],
                                vocab_size=c["vocab"])
    model = LLaDAForDLM(cfg, c["tau"]).bfloat16()
    load_weights_into(model, token_model_weights())
    runner = object.__new__(ModelRunner)           # only its prepare_* methods are used; they read config.mask_id
    runner.config = types.SimpleNamespace(mask_id=MASK_ID)
    sampler = sampler_mod.LLaDASampler("confidence")
    sp = SamplingParams(temperature=0.0, max_new_tokens=c["gen"], steps=c["steps"], num_full_steps=c["full_steps"],
                        block_size=c["block"], ignore_eos=True, mask_id=MASK_ID)
    seqs = [Sequence(list(p) + [MASK_ID] * c["gen"], sp) for p in token_prompts()]
    set_metadata([s.seq_id for s in seqs], [s.seq_id for s in seqs], [])

    record = {"cfg": CFG, "mask_id": MASK_ID, "seq_ids": [s.seq_id for s in seqs], "steps": []}
    for step in range(c["steps"]):
        for s in seqs:
            s.processed_steps += 1                 # scheduler.py:43,69
        is_full = seqs[0].processed_steps <= c["full_steps"]
        get_metadata().finished_seqs = []
        seen_cos.clear()
        with torch.no_grad():
            input_ids, positions = ModelRunner.prepare_full(runner, seqs) if is_full else ModelRunner.prepare_sparse(runner, seqs)
            ctx = get_context()
            pruned = (not is_full) and ctx.idx_salient_row_k is not None
            logits = model.compute_logits(model(input_ids, positions))
            sampler_params, input_indices, num_transfer = ModelRunner.prepare_sample(runner, seqs)
            pos, toks, counts = sampler(input_logits=logits, ctx=get_context(), input_indices=input_indices,
                                        confidence_thresholds=sampler_params[4], temperatures=sampler_params[0],
                                        num_transfer=num_transfer, top_k=sampler_params[1], top_p=sampler_params[2],
                                        block_size=sampler_params[3])
            # how clear the choice was, from fp32 probabilities of the candidate rows
            rel, offs, cu_f = input_indices
            rows = torch.cat([ctx.cu_seqlens_q[b].long() + rel[int(cu_f[b]):int(cu_f[b + 1])] for b in range(len(seqs))])
            probs = torch.softmax(logits.index_select(0, rows).float(), dim=-1)
            top2 = probs.topk(2, dim=-1).values
        reset_context()
        picks, clear, cand_rec = [], [], []
        for b, s in enumerate(seqs):
            n = int(counts[b])
            p_list, t_list = pos[b, :n].tolist(), toks[b, :n].tolist()
            cand = top2[int(cu_f[b]):int(cu_f[b + 1])]
            conf = cand[:, 0]
            order = torch.argsort(conf, descending=True)
            sel_margin = float(conf[order[n - 1]] / conf[order[n]] - 1.0) if order.numel() > n else float("inf")
            chosen_rows = order[:n]
            tok_margin = float((cand[chosen_rows, 0] / cand[chosen_rows, 1] - 1.0).min()) if n else float("inf")
            picks.append(sorted(zip(p_list, t_list)))
            clear.append((sel_margin, tok_margin))
            lo, hi = int(cu_f[b]), int(cu_f[b + 1])
            cand_pos = (rel[lo:hi] + offs[b]).tolist()
            cand_rec.append([(p, float(cf), int(tk), float(mg)) for p, cf, tk, mg in
                             zip(cand_pos, conf.tolist(), probs[lo:hi].argmax(-1).tolist(),
                                 (cand[:, 0] / cand[:, 1] - 1.0).tolist())])
            s.update_token(p_list, t_list)
            s.update_block_idx()
        gap = min((float((cs - c["tau"]).abs().min()) for cs in seen_cos), default=float("inf"))
        record["steps"].append({"kind": "full" if is_full else ("pruned" if pruned else "sparse"), "picks": picks,
                                "margins": clear, "candidates": cand_rec, "layer_cosines": [cs.clone() for cs in seen_cos], "cosine_gap": gap})
        print(step + 1, record["steps"][-1]["kind"], picks, [tuple(round(x, 3) for x in m) for m in clear], "cos gap %.5f" % gap)
    record["final_tokens"] = [s.token_ids[s.num_prompt_tokens:] for s in seqs]
    print("smallest |cos - tau| of the run:", min(st["cosine_gap"] for st in record["steps"]))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "llada_tokens_small.pt")
    torch.save(record, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_token_golden.py /path/to/reference")
    main(sys.argv[1])
