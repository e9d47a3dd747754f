"""CPU checks of the oracle itself: the reference's known-answer test, self-consistency of the
compaction / offset / cache restatements, and the seeded generators' guarantees."""
import math

import numpy as np
import torch

from oracle import dyllm_oracle as orc


def test_reference_known_answer_additive_shard_stats():
    # the reference's only numerical known-answer test on this path: tests/test_parallelism.py:34-44
    old = torch.tensor([[1.0, 2.0, -3.0, 4.0], [1.0, 0.0, 1.0, 0.0]])
    new = torch.tensor([[1.5, 1.0, -2.0, 5.0], [-1.0, 0.0, -1.0, 0.0]])
    stats = torch.zeros(2, 3)
    for o, n in zip(old.chunk(2, dim=-1), new.chunk(2, dim=-1)):
        stats += orc.context_stats(o, n)
    expected = torch.nn.functional.cosine_similarity(old, new, dim=-1) < 0.5
    assert torch.equal(orc.cosine_mask(stats, 0.5), expected)
    assert expected.tolist() == [False, True]


def test_compact_matches_nonzero_and_searchsorted():
    g = torch.Generator().manual_seed(1)
    mask = torch.rand(1000, generator=g) < 0.2
    cu = torch.tensor([0, 100, 100, 512, 1000], dtype=torch.int32)
    idx, cu_sal = orc.compact(mask, cu)
    ref_idx = torch.nonzero(mask, as_tuple=False).squeeze(-1)
    assert torch.equal(idx, ref_idx)
    assert torch.equal(cu_sal, torch.searchsorted(ref_idx, cu.long()).to(torch.int32))
    assert cu_sal[-1].item() == idx.numel()


def test_fused_offset_maps_response_rows_to_key_rows():
    batch, prompt, resp = 3, 5, 4
    cu_q, cu_k, cu_p = orc.make_batch_layout(batch, prompt, resp, response_only=True)
    idx = torch.tensor([0, 3, 4, 9, 11], dtype=torch.int64)
    _, cu_sal = orc.compact(torch.zeros(12, dtype=torch.bool).index_fill_(0, idx, True), cu_q)
    out = orc.fused_offset(idx, cu_p, cu_sal)
    # Q row r of sequence b, offset o in the response -> K row b*(prompt+resp) + prompt + o
    exp = [(r // resp) * (prompt + resp) + prompt + r % resp for r in idx.tolist()]
    assert out.tolist() == exp


def test_cache_roundtrip():
    g = torch.Generator().manual_seed(2)
    cache = torch.randn(40, 8, generator=g)
    seq_starts = torch.full((16,), -1, dtype=torch.int64)
    seq_starts[3], seq_starts[7], seq_starts[1] = 0, 10, 25
    seq_ids = torch.tensor([7, 3, 1])
    cu = torch.tensor([0, 15, 25, 40], dtype=torch.int32)  # lens 15, 10, 15
    got = orc.cache_get_seqs(cache, seq_starts, cu, seq_ids, 40)
    assert torch.equal(got[:15], cache[10:25]) and torch.equal(got[15:25], cache[0:10])
    c2 = torch.zeros_like(cache)
    orc.cache_reset_full(c2, got, seq_starts, cu, seq_ids)
    assert torch.equal(c2, cache)
    cu_q = torch.tensor([0, 4, 8, 12], dtype=torch.int32)
    blk = orc.cache_get_block(cache, seq_starts, cu, cu_q, seq_ids, 12)
    assert torch.equal(blk[:4], cache[21:25]) and torch.equal(blk[4:8], cache[6:10])
    c3 = cache.clone()
    orc.cache_reset_block(c3, blk * 2, seq_starts, cu, cu_q, seq_ids)
    assert torch.equal(c3[21:25], cache[21:25] * 2) and torch.equal(c3[:6], cache[:6])
    c4 = cache.clone()
    rows = torch.tensor([0, 16, 39])
    orc.cache_scatter_update(c4, torch.ones(3, 8), rows, cu, seq_starts, seq_ids)
    assert (c4[10] == 1).all() and (c4[1] == 1).all() and (c4[39] == 1).all()
    assert torch.equal(c4[11:25], cache[11:25])


def test_generator_keeps_cosines_away_from_threshold():
    c_old, c_new = orc.make_context_pair(512, 4096, 0.99, 0.10, seed=0)
    cosv = orc.cosine_values(orc.context_stats(c_old, c_new))
    assert float((cosv - 0.99).abs().min()) >= 1e-4
    frac = float((cosv < 0.99).float().mean())
    assert 0.04 < frac < 0.2


def test_sparse_attention_reduces_to_exact_when_delta_is_full_update():
    # If dV = V_new - V_old on every row and C_old = softmax(QK^T) V_old, then
    # C_old + softmax(QK^T) dV = softmax(QK^T) V_new.
    g = torch.Generator().manual_seed(3)
    B, L, H, Hkv, D = 2, 24, 4, 2, 16
    cu = torch.arange(B + 1, dtype=torch.int32) * L
    q = torch.randn(B * L, H, D, generator=g).bfloat16()
    k = torch.randn(B * L, Hkv, D, generator=g).bfloat16()
    v_old = torch.randn(B * L, Hkv, D, generator=g).bfloat16()
    v_new = torch.randn(B * L, Hkv, D, generator=g).bfloat16()
    c_old = orc.exact_attention_varlen(q, k, v_old, cu, cu)
    dv = (v_new.float() - v_old.float())
    empty = torch.empty(0, dtype=torch.int64)
    O, stats, mask = orc.attention_sparse_varlen(
        q, k, dv, c_old, torch.empty(0, H, D), cu, cu, torch.zeros(B + 1, dtype=torch.int32), empty, 0.99,
        round_p_bf16=False)
    want = orc.exact_attention_varlen(q, k, v_new, cu, cu)
    assert torch.allclose(O.float(), want, atol=3e-2, rtol=3e-2)
    assert stats.shape == (B * L, 3) and mask.shape == (B * L,)


def test_swiglu_and_moe_consistency():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, 32, generator=g)
    w1 = torch.randn(2, 2 * 16, 32, generator=g) * 0.1
    w2 = torch.randn(2, 32, 16, generator=g) * 0.1
    # one expert with weight 1 == the dense FFN
    ids = torch.zeros(5, 1, dtype=torch.int32)
    out = orc.naive_experts(x, w1, w2, torch.ones(5, 1), ids, round_bf16=False)
    assert torch.allclose(out, orc.swiglu_ffn(x, w1[0], w2[0], round_bf16=False), atol=1e-5)
    w, i = orc.moe_gate(x, torch.randn(4, 32, generator=g), 2)
    assert w.shape == (5, 2) and i.dtype == torch.int32 and bool((w[:, 0] >= w[:, 1]).all())


def test_oracle_selection_reproduces_reference_layer_outputs():
    """Golden fixture (reference Python run on CPU, tests/golden/make_golden.py): the oracle's mask ->
    compaction -> K-space offsets reproduce the index lists the reference layer published."""
    import os

    fx = torch.load(os.path.join(os.path.dirname(__file__), "golden", "llada_layer_small.pt"))
    B, P, R = fx["batch"], fx["prompt"], fx["resp"]
    for step, response_only in ((1, False), (2, True)):
        rec = fx["steps"][step]
        cu_q, cu_k, cu_p = orc.make_batch_layout(B, P, R, response_only)
        mask = rec["cosine"] < fx["tau"]
        idx, cu_sal = orc.compact(mask, cu_q)
        assert torch.equal(idx, rec["idx_salient_row"])
        assert torch.equal(cu_sal, rec["cu_salientlens"])
        if response_only:
            assert torch.equal(orc.fused_offset(idx, cu_p, cu_sal), rec["idx_salient_row_k"])
