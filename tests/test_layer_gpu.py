"""Layer-level parity: this package's LLaDADecoderLayer (bf16, sm_100a kernels) against outputs of the
reference's own LLaDADecoderLayer run on the CPU with bf16 modules (fixtures tests/golden/llada_layer_small.pt
and llada_layer_c1.pt, made by tests/golden/make_golden.py): a dense step, a full-sequence sparse step and
a response-only sparse step on the same layer state.  "c1" is the single-layer LLaDA-8B configuration
(hidden 4096, 32 heads, FFN intermediate 12288, 256 prompt + 256 response positions).

The generator keeps every reference cosine at least 1e-4 from the threshold.  Upstream of the statistics the
two pipelines round differently (bf16 GEMMs with different accumulation orders), which moves a cosine by up
to ~1e-3, so the decisions are required to agree on every row whose reference cosine is at least BAND from
the threshold; the kernel-level tests, which feed identical inputs, use the 1e-4 band itself."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))


BAND = 2e-3


def _run_layer(dev, config):
    import make_golden as mg

    mg.use_config(config)
    from dyllm_b200.context import get_context, get_metadata, set_context, set_metadata
    from dyllm_b200.model import LLaDADecoderLayer, LLaDAShape

    S = mg.SHAPE
    from dyllm_b200 import model as M

    family = mg.CONFIGS[config].get("family", "llada")
    if family == "dream":
        cfg = M.DreamShape(hidden_size=S["hidden"], num_attention_heads=S["heads"], num_key_value_heads=S["kv_heads"],
                           head_dim=S["head_dim"], intermediate_size=S["inter"], rms_norm_eps=S["eps"],
                           rope_theta=S["theta"], max_position_embeddings=S["max_pos"], num_hidden_layers=1)
        layer = M.DreamDecoderLayer(cfg, mg.TAU)
    elif family == "lladamoe":
        cfg = M.LLaDAMoEShape(hidden_size=S["hidden"], num_attention_heads=S["heads"], num_key_value_heads=S["kv_heads"],
                              head_dim=S["head_dim"], num_experts=S["experts"], num_experts_per_tok=S["top_k"],
                              expert_intermediate_size=S["inter"], rms_norm_eps=S["eps"], rope_theta=S["theta"],
                              max_position_embeddings=S["max_pos"], num_hidden_layers=1)
        layer = M.LLaDAMoEDecoderLayer(cfg, mg.TAU)
    else:
        cfg = LLaDAShape(hidden_size=S["hidden"], num_attention_heads=S["heads"], n_kv_heads=S["kv_heads"],
                         head_dim=S["head_dim"], mlp_hidden_size=S["inter"], rms_norm_eps=S["eps"], rope_theta=S["theta"],
                         max_sequence_length=S["max_pos"], num_hidden_layers=1)
        layer = LLaDADecoderLayer(cfg, mg.TAU)
    layer = layer.to(dev).bfloat16()
    w, xs = mg.golden_inputs()
    mg.load_layer_weights(layer, {k: v.to(dev) for k, v in w.items()})
    B, P, R = mg.BATCH, mg.PROMPT, mg.RESP
    L = P + R
    seq_ids = mg.CONFIGS[config]["seq_ids"]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    results = []
    for step in range(3):
        is_full, ro, sal = mg.step_layout(step)
        set_metadata(seq_ids, seq_ids, [])
        get_metadata().running_seqs_tensor = torch.tensor(seq_ids, dtype=torch.long, device=dev)
        cu_k = [b * L for b in range(B + 1)]
        if is_full:
            positions = torch.arange(L, device=dev).repeat(B)
            set_context(True, cu_seqlens_q=i32(cu_k), cu_seqlens_q_cpu=cu_k, cu_seqlens_k=i32(cu_k), max_seqlen_q=L,
                        max_seqlen_k=L, context_lens=i32([L] * B), context_lens_cpu=[L] * B, total_seqlen=B * L,
                        total_seqlen_k=B * L)
            x = xs[step]
        else:
            lq = R if ro else L
            cu_q = [b * lq for b in range(B + 1)]
            idx_q, idx_k, cu_sal = [], [], [0]
            for b in range(B):
                for p in sal[b]:
                    idx_q.append((p - P if ro else p) + cu_q[b])
                    idx_k.append(p + cu_k[b])
                cu_sal.append(len(idx_q))
            positions = (torch.arange(P, L, device=dev) if ro else torch.arange(L, device=dev)).repeat(B)
            set_context(False, cu_seqlens_q=i32(cu_q), cu_seqlens_q_cpu=cu_q, cu_seqlens_k=i32(cu_k),
                        cu_promptlens=i32([b * P for b in range(B + 1)]), cu_salientlens=i32(cu_sal), max_seqlen_q=lq,
                        max_seqlen_k=L, idx_salient_row=torch.tensor(idx_q, dtype=torch.long, device=dev),
                        idx_salient_row_k=torch.tensor(idx_k, dtype=torch.long, device=dev) if ro else None,
                        idx_salient_row32=i32(idx_q), max_salient_per_seq=max(len(s) for s in sal),
                        context_lens=i32([L] * B), context_lens_cpu=[L] * B, total_seqlen_k=B * L, total_seqlen=B * lq)
            x = xs[step].view(B, L, -1)[:, P:].reshape(B * R, -1) if ro else xs[step]
        with torch.inference_mode():
            out, residual = layer(positions, x.to(dev).bfloat16(), None)
        ctx = get_context()
        idx, idx_k = (None, None) if is_full else ctx.salient_rows()
        results.append(dict(out=out.float().cpu(), residual=residual.float().cpu(),
                            idx=None if is_full else idx.cpu(),
                            cu_sal=None if is_full else ctx.cu_salientlens.cpu(),
                            idx_k=idx_k.cpu() if (not is_full and ro) else None))
    return results


@pytest.mark.parametrize("config", ["small", "c1", "dream", "moe"])
def test_decoder_layer_matches_reference_fixture(cuda_device, config):
    from dyllm_b200 import _lib

    fx = torch.load(os.path.join(os.path.dirname(__file__), "golden", f"llada_layer_{config}.pt"))
    got = _run_layer(cuda_device, config)
    assert _lib.load().dyllm_device_status() == 0
    tau = fx["tau"]
    for step, (g, want) in enumerate(zip(got, fx["steps"])):
        rows = g["out"].size(0)
        clear = torch.ones(rows, dtype=torch.bool)
        if step > 0:
            clear = (want["cosine"] - tau).abs() >= BAND
            assert clear.float().mean() >= (0.95 if config == "c1" else 0.8)
            ref_mask = torch.zeros(rows, dtype=torch.bool)
            ref_mask[want["idx_salient_row"]] = True
            got_mask = torch.zeros(rows, dtype=torch.bool)
            got_mask[g["idx"]] = True
            assert torch.equal(got_mask[clear], ref_mask[clear]), f"step {step}: salient sets differ"
            assert bool((g["idx"][1:] > g["idx"][:-1]).all())
            assert g["cu_sal"][-1].item() == g["idx"].numel()
            if g["idx_k"] is not None:
                # K-space list: row r of sequence b maps to r + prompt * (b + 1)
                b_of = torch.div(g["idx"], fx["resp"], rounding_mode="floor")
                assert torch.equal(g["idx_k"], g["idx"] + fx["prompt"] * (b_of + 1))
            # rows whose decision differs inside the band went through (or skipped) the FFN: not comparable
            clear = clear & (got_mask == ref_mask)
        if "out" in want:
            pairs = [("out", g["out"][clear], want["out"][clear]), ("residual", g["residual"], want["residual"])]
        else:
            # compact fixture: a subset of rows in full, per-row sums and norms of every row
            sub = want["rows"]
            keep = clear[sub]
            pairs = [("out", g["out"][sub][keep], want["out_rows"].float()[keep]),
                     ("residual", g["residual"][sub], want["residual_rows"].float())]
            for name in ("out", "residual"):
                sel = clear if name == "out" else torch.ones(rows, dtype=torch.bool)
                norm_got, norm_want = g[name].norm(dim=1)[sel], want[name + "_norm"][sel]
                assert torch.allclose(norm_got, norm_want, rtol=1e-2, atol=1e-3), f"step {step}: {name} row norms"
                sum_err = (g[name].sum(1)[sel] - want[name + "_sum"][sel]).abs()
                assert bool((sum_err <= 2e-2 * want[name + "_norm"][sel] * g[name].size(1) ** 0.5 + 1e-2).all()), \
                    f"step {step}: {name} row sums"
        for name, a, b in pairs:
            diff = a - b
            scale = max(1.0, b.abs().max().item())
            rel = (diff.norm() / b.norm()).item()
            print(f"{config} step {step} {name}: max-abs {diff.abs().max().item():.4g} (peak {scale:.3g}) rel-L2 {rel:.4g}")
            assert diff.abs().max().item() / scale <= 2e-2, f"step {step} {name}: max-abs {diff.abs().max().item()}"
            assert rel <= 1e-2, f"step {step} {name}: rel-L2 {rel}"
