"""Parity of the MoE router and expert FFN with the oracle's restatement of the reference's
``moe_gate`` / ``naive_experts`` (the reference's stated oracle for its fused kernels)."""
import pytest
import torch

from oracle import dyllm_oracle as orc

pytestmark = pytest.mark.gpu


def _moe_case(rows, hidden, inter, experts, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    wr = torch.randn(experts, hidden, generator=g).bfloat16()     # router logits ~ N(0, hidden): well separated
    wr = (wr * (1.0 / hidden ** 0.5)).bfloat16()
    w1 = (torch.randn(experts, 2 * inter, hidden, generator=g) * 0.03).bfloat16()
    w2 = (torch.randn(experts, hidden, inter, generator=g) * 0.03).bfloat16()
    return x, wr, w1, w2


@pytest.mark.parametrize("rows,experts,top_k,renorm", [(1, 8, 2, False), (130, 64, 8, False), (410, 64, 8, True)])
def test_moe_route_matches_oracle(cuda_device, rows, experts, top_k, renorm):
    from dyllm_b200 import ops

    x, wr, _, _ = _moe_case(rows, 256, 64, experts, seed=rows)
    w, ids = ops.moe_route(x.to(cuda_device), wr.to(cuda_device), top_k, renorm)
    want_w, want_ids = orc.moe_gate(x, wr, top_k, renorm)
    # rows whose k-th and (k+1)-th probabilities nearly tie may legitimately order differently
    probs = torch.softmax(x.float() @ wr.float().t(), dim=-1)
    srt = probs.sort(dim=-1, descending=True).values
    gaps = (srt[:, : top_k] - srt[:, 1 : top_k + 1]).min(dim=-1).values
    clear = gaps > 1e-5
    assert clear.float().mean() > 0.9
    assert torch.equal(ids.cpu()[clear], want_ids[clear])
    torch.testing.assert_close(w.cpu()[clear], want_w[clear].bfloat16().float(), rtol=1e-2, atol=1e-4)


@pytest.mark.parametrize("rows,hidden,inter,experts,top_k", [(7, 256, 128, 8, 2), (130, 512, 256, 16, 4),
                                                              (410, 2048, 1024, 64, 8)])
def test_moe_ffn_matches_naive_experts(cuda_device, rows, hidden, inter, experts, top_k):
    from dyllm_b200 import _lib
    from dyllm_b200.fused_moe import fused_experts, moe_gate

    x, wr, w1, w2 = _moe_case(rows, hidden, inter, experts, seed=rows + 1)
    d = lambda t: t.to(cuda_device)
    w, ids = moe_gate(d(x), d(wr), top_k, renormalize=False)
    got = fused_experts(d(x), d(w1), d(w2), w, ids, activation="silu")
    assert _lib.load().dyllm_device_status() == 0
    want = orc.naive_experts(x, w1, w2, w.float().cpu(), ids.cpu())
    diff = got.float().cpu() - want
    assert diff.abs().max().item() / max(1.0, want.abs().max().item()) <= 2e-2
    assert (diff.norm() / want.norm()).item() <= 1e-2


def test_moe_ffn_expert_parallel_shares_sum_to_the_whole(cuda_device):
    """Two contiguous expert ranges computed separately add up to the all-experts result (the EP all-reduce)."""
    from dyllm_b200 import ops

    rows, hidden, inter, experts, top_k = 200, 512, 256, 16, 4
    x, wr, w1, w2 = _moe_case(rows, hidden, inter, experts, seed=5)
    d = lambda t: t.to(cuda_device)
    w, ids = ops.moe_route(d(x), d(wr), top_k)
    whole = ops.moe_ffn(d(x), d(w1), d(w2), w, ids)
    half = experts // 2
    a = ops.moe_ffn(d(x), d(w1[:half].contiguous()), d(w2[:half].contiguous()), w, ids, expert_start=0)
    b = ops.moe_ffn(d(x), d(w1[half:].contiguous()), d(w2[half:].contiguous()), w, ids, expert_start=half)
    diff = (a.float() + b.float()) - whole.float()
    assert (diff.norm() / whole.float().norm()).item() <= 1e-2


def test_moe_gathered_rows_device_count_and_scatter(cuda_device):
    from dyllm_b200 import ops

    hidden, inter, experts, top_k = 512, 256, 16, 4
    x, wr, w1, w2 = _moe_case(600, hidden, inter, experts, seed=9)
    g = torch.Generator().manual_seed(2)
    idx = torch.sort(torch.randperm(600, generator=g)[:256]).values.to(torch.int32)
    live = 77
    n_dev = torch.tensor([live], dtype=torch.int32, device=cuda_device)
    dest = torch.randperm(300, generator=g)[:256].to(torch.int32)
    d = lambda t: t.to(cuda_device)
    w, ids = ops.moe_route(d(x), d(wr), top_k, idx=d(idx), num_rows=256, num_rows_dev=n_dev)
    out = torch.full((300, hidden), 3.0, dtype=torch.bfloat16, device=cuda_device)
    ops.moe_ffn(d(x), d(w1), d(w2), w, ids, idx=d(idx), num_rows=256, num_rows_dev=n_dev, rows_hint=64, out=out,
                out_row_map=d(dest))
    xs = x[idx[:live].long()]
    ww, ii = orc.moe_gate(xs, wr, top_k)
    want = orc.naive_experts(xs, w1, w2, ww.bfloat16().float(), ii)
    got = out.cpu()[dest[:live].long()].float()
    assert ((got - want).norm() / want.norm()).item() <= 1e-2
    untouched = torch.ones(300, dtype=torch.bool)
    untouched[dest[:live].long()] = False
    assert bool((out.cpu()[untouched] == 3.0).all())
