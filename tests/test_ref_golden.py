"""The CPU oracle against outputs of the REFERENCE's own CUDA kernels and of flash-attn, recorded on a
B200 by tests/golden/make_ref_golden.py (fixture tests/golden/ref_kernels.pt; inputs are regenerated from
the case seeds).  This is what pins the oracle's restatement of attention_sparse_varlen, of the cache
kernels and of fused_offset to something the reference produced."""
import os
import sys

import pytest
import torch

from oracle import dyllm_oracle as orc

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_ref_golden as mrg  # noqa: E402

FIXTURE = os.path.join(os.path.dirname(__file__), "golden", "ref_kernels.pt")
BAND = 1e-4          # decisions are compared where the cosine is at least this far from the threshold


@pytest.fixture(scope="module")
def golden():
    return torch.load(FIXTURE)


def check_outputs(got, want, what):
    """The tolerances of the path: bf16 outputs max-abs 2e-2 (relative to the output peak when it exceeds 1) and
    rel-L2 1e-2."""
    got, want = got.float(), want.float()
    diff = got - want
    scale = max(1.0, want.abs().max().item())
    assert diff.abs().max().item() / scale <= 2e-2, f"{what}: max-abs {diff.abs().max().item()} (peak {scale})"
    assert (diff.norm() / want.norm().clamp_min(1e-12)).item() <= 1e-2, f"{what}: rel-L2 {(diff.norm() / want.norm()).item()}"


def check_decisions(mask, stats_ref, mask_ref, tau, what):
    cos = orc.cosine_values(stats_ref)
    clear = (cos - tau).abs() >= BAND
    assert clear.float().mean().item() > 0.95, f"{what}: too many rows inside the band"
    assert torch.equal(mask[clear], mask_ref[clear]), f"{what}: decisions differ outside the band"


@pytest.mark.parametrize("name", list(mrg.ATTENTION_CASES))
def test_oracle_attention_matches_reference_kernel(golden, name):
    if name not in golden["attention"]:
        pytest.skip("case not in the recorded fixture")
    c, rec = mrg.attention_case(name), golden["attention"][name]
    O, stats, mask = orc.attention_sparse_varlen(c["q"], c["k"], c["dv"], c["c_old"], rec["o_sal_used"], c["cu_q"], c["cu_k"],
                                                 c["cu_sal"], c["idx_q"], c["tau"], c["pruned"], c["idx_k"])
    check_outputs(O, rec["O"], name)
    assert torch.allclose(stats, rec["stats"], rtol=2e-3, atol=2e-2), (stats - rec["stats"]).abs().max()
    check_decisions(mask, rec["stats"], rec["mask"], c["tau"], name)
    # the replaced rows are copied, not recomputed
    if c["idx_q"].numel():
        assert torch.equal(rec["O"][c["idx_q"].long()], rec["o_sal_used"])


@pytest.mark.parametrize("name", list(mrg.ATTENTION_CASES))
def test_oracle_exact_attention_matches_flash_attn(golden, name):
    rec = golden["attention"].get(name)
    if rec is None or "flash_o_sal" not in rec:
        pytest.skip("flash-attn output not recorded for this case")
    c = mrg.attention_case(name)
    v_now = c["v_cache"].clone()
    ik = c["idx_k"].long()
    v_now[ik] = (c["v_cache"][ik].float() + c["dv"][ik].float()).to(torch.bfloat16)
    o = orc.exact_attention_varlen(c["q"][c["idx_q"].long()], c["k"], v_now, c["cu_sal"], c["cu_k"])
    check_outputs(o, rec["flash_o_sal"], name)


def test_oracle_cache_functions_match_reference_kernels(golden):
    c, rec = mrg.cache_case(), golden["cache"]
    fill = rec["get_seqs"]     # rows no sequence covers are left as allocated; compare the covered rows only
    got = orc.cache_get_seqs(c["cache"], c["seq_starts"], c["cu"], c["seq_ids"], c["total"])
    assert torch.equal(got, fill)
    got = orc.cache_get_block(c["cache"], c["seq_starts"], c["cu"], c["cu_q"], c["seq_ids"], c["total_q"])
    assert torch.equal(got, rec["get_block"])
    assert torch.equal(orc.cache_reset_full(c["cache"].clone(), c["new_full"], c["seq_starts"], c["cu"], c["seq_ids"]),
                       rec["reset_full"])
    assert torch.equal(orc.cache_reset_block(c["cache"].clone(), c["new_block"], c["seq_starts"], c["cu"], c["cu_q"],
                                             c["seq_ids"]), rec["reset_block"])
    assert torch.equal(orc.cache_scatter_update(c["cache"].clone(), c["new_rows"], c["rows"], c["cu"], c["seq_starts"],
                                                c["seq_ids"]), rec["scatter_update"])


def test_oracle_fused_offset_matches_reference_kernel(golden):
    c, rec = mrg.cache_case(), golden["cache"]
    n = c["idxs"].numel()
    got = orc.fused_offset(c["idxs"], c["cu_prompt"], c["cu_sal"])
    assert torch.equal(got, rec["fused_offset"][:n])
    assert bool((rec["fused_offset"][n:] == -1).all())       # entries past the device-side count stay untouched


def test_unmasking_rule_reproduces_the_reference_samplers_picks():
    """oracle.confidence_unmask against the picks that the reference's LLaDASampler made on its own candidate
    confidences (tests/golden/llada_tokens_small.pt, written by make_token_golden.py from the reference's step loop):
    every step of the generation, both sequences."""
    import os

    path = os.path.join(os.path.dirname(__file__), "golden", "llada_tokens_small.pt")
    fx = torch.load(path, weights_only=False)
    cfg, mask_id = fx["cfg"], fx["mask_id"]
    block, prompt, gen = cfg["block"], cfg["prompt"], cfg["gen"]
    steps_per_block = cfg["steps"] * block // gen
    num_transfer = block // steps_per_block
    checked = 0
    for step, rec in enumerate(fx["steps"]):
        start = prompt + min(step // steps_per_block, gen // block - 1) * block
        for cands, picks, (gap, _lead) in zip(rec["candidates"], rec["picks"], rec["margins"]):
            # the recorded confidences are an fp32 restatement of the scores the reference's sampler sorted (its
            # own come from bf16 logits): where the two best candidates lie closer than that difference the
            # reference's order is not recoverable from the record
            if gap < 5e-3:
                continue
            conf = torch.full((1, block), -1.0)
            best = torch.zeros((1, block), dtype=torch.int64)
            tokens = torch.zeros((1, prompt + gen), dtype=torch.int64)      # 0 = some unmasked token
            for pos, c, tok, _lead in cands:
                assert start <= pos < start + block
                conf[0, pos - start], best[0, pos - start], tokens[0, pos] = c, tok, mask_id
            after, picked = orc.confidence_unmask(conf, best, tokens, start, block, num_transfer, mask_id)
            assert picked[0] == sorted(p for p, _ in picks), (step, picked, picks)
            for p, tok in picks:
                assert int(after[0, p]) == tok
            checked += 1
    assert checked >= cfg["steps"]
