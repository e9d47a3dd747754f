"""Parity of the statistics / mask / compaction kernels with the CPU oracle (bit-exact index sets)."""
import pytest
import torch

from oracle import dyllm_oracle as orc

pytestmark = pytest.mark.gpu


def _stats_case(rows, width, seed, frac=0.1):
    c_old, c_new = orc.make_context_pair(rows, width, 0.99, frac, seed=seed)
    return c_old, c_new, orc.context_stats(c_old, c_new)


@pytest.mark.parametrize("rows,width", [(1, 8), (33, 128), (512, 4096), (777, 3584), (64, 512)])
def test_context_stats_matches_oracle(cuda_device, rows, width):
    from dyllm_b200 import ops

    c_old, c_new, want = _stats_case(rows, width, seed=rows)
    got = ops.context_stats(c_old.to(cuda_device), c_new.to(cuda_device))
    torch.testing.assert_close(got.cpu(), want, rtol=2e-5, atol=1e-4)
    # run-to-run identical (fixed reduction order)
    again = ops.context_stats(c_old.to(cuda_device), c_new.to(cuda_device))
    assert torch.equal(got, again)
    # accumulate over two column shards == whole row (tensor-parallel additivity)
    if width % 16 == 0:
        h = width // 2
        acc = ops.context_stats(c_old[:, :h].contiguous().to(cuda_device), c_new[:, :h].contiguous().to(cuda_device))
        ops.context_stats(c_old[:, h:].contiguous().to(cuda_device), c_new[:, h:].contiguous().to(cuda_device),
                          out=acc, accumulate=True)
        torch.testing.assert_close(acc.cpu(), want, rtol=2e-5, atol=1e-4)


def test_cosine_mask_matches_reference_known_answer(cuda_device):
    from dyllm_b200 import ops

    old = torch.tensor([[1.0, 2.0, -3.0, 4.0], [1.0, 0.0, 1.0, 0.0]])
    new = torch.tensor([[1.5, 1.0, -2.0, 5.0], [-1.0, 0.0, -1.0, 0.0]])
    stats = orc.context_stats(old, new)
    got = ops.cosine_mask(stats.to(cuda_device), 0.5)
    assert got.cpu().tolist() == [False, True]
    # degenerate rows: zero norms hit the 1e-8 clamp, cosine 0 < threshold
    z = torch.zeros(3, 3)
    assert ops.cosine_mask(z.to(cuda_device), 0.99).cpu().tolist() == [True] * 3


LAYOUTS = [
    # (batch, prompt, response, response_only)
    (1, 256, 256, False),
    (1, 256, 256, True),
    (16, 256, 256, False),
    (16, 256, 256, True),
    (3, 7, 5, True),
    (5, 100, 411, False),  # tiles cut sequences at odd places
]


@pytest.mark.parametrize("batch,prompt,response,response_only", LAYOUTS)
@pytest.mark.parametrize("frac", [0.0, 0.1, 1.0])
def test_salient_select_is_bit_exact(cuda_device, batch, prompt, response, response_only, frac):
    from dyllm_b200 import ops

    cu_q, cu_k, cu_p = orc.make_batch_layout(batch, prompt, response, response_only)
    rows = int(cu_q[-1])
    if frac in (0.0, 1.0):
        stats = torch.zeros(rows, 3)
        stats[:, 1:] = 1.0
        stats[:, 0] = 1.0 if frac == 0.0 else 0.5
    else:
        _, _, stats = _stats_case(rows, 256, seed=batch * 7 + prompt)
    want = orc.salient_select(stats, 0.99, cu_q, cu_p if response_only else None)
    sel = ops.salient_select(stats.to(cuda_device), 0.99, cu_q.to(cuda_device),
                             cu_p.to(cuda_device) if response_only else None, want_mask=True)
    n = int(sel.count.item())
    assert n == want["count"]
    assert torch.equal(sel.idx[:n].cpu(), want["idx"])
    assert torch.equal(sel.idx32[:n].cpu().long(), want["idx"])
    assert torch.equal(sel.cu_salientlens.cpu(), want["cu_salientlens"])
    assert torch.equal(sel.mask.cpu(), want["mask"])
    if response_only:
        assert torch.equal(sel.idx_k[:n].cpu(), want["idx_k"])


def test_salient_select_ragged_and_empty_sequences(cuda_device):
    from dyllm_b200 import ops

    cu_q = torch.tensor([0, 0, 5, 5, 2053, 2053, 4100, 4100], dtype=torch.int32)
    cu_p = torch.tensor([0, 3, 10, 10, 20, 25, 40, 41], dtype=torch.int32)
    rows = 4100
    _, _, stats = _stats_case(rows, 64, seed=11, frac=0.3)
    want = orc.salient_select(stats, 0.99, cu_q, cu_p)
    sel = ops.salient_select(stats.to(cuda_device), 0.99, cu_q.to(cuda_device), cu_p.to(cuda_device))
    n = int(sel.count.item())
    assert n == want["count"]
    assert torch.equal(sel.idx[:n].cpu(), want["idx"])
    assert torch.equal(sel.cu_salientlens.cpu(), want["cu_salientlens"])
    assert torch.equal(sel.idx_k[:n].cpu(), want["idx_k"])
    # zero rows
    e = ops.salient_select(torch.zeros(0, 3, device=cuda_device), 0.99,
                           torch.zeros(3, dtype=torch.int32, device=cuda_device))
    assert int(e.count.item()) == 0 and e.cu_salientlens.cpu().tolist() == [0, 0, 0]


def test_salient_select_large_many_tiles(cuda_device):
    """Full-size property check: sorted, unique, count == popcount of the mask, idempotent."""
    from dyllm_b200 import ops

    rows = 1 << 20
    g = torch.Generator().manual_seed(5)
    stats = torch.ones(rows, 3)
    stats[:, 0] = torch.where(torch.rand(rows, generator=g) < 0.07, 0.5, 0.999)
    cu_q = torch.arange(0, rows + 1, 4096, dtype=torch.int32)
    d = stats.to(cuda_device)
    sel = ops.salient_select(d, 0.99, cu_q.to(cuda_device), want_mask=True)
    n = int(sel.count.item())
    idx = sel.idx[:n]
    assert n == int(sel.mask.sum().item())
    assert bool((idx[1:] > idx[:-1]).all())
    assert torch.equal(idx, torch.nonzero(sel.mask).squeeze(-1))
    assert torch.equal(sel.cu_salientlens.long(), torch.searchsorted(idx, cu_q.to(cuda_device).long()))
    sel2 = ops.salient_select(d, 0.99, cu_q.to(cuda_device))
    assert torch.equal(sel2.idx[:n], idx)
    from dyllm_b200 import _lib
    assert _lib.load().dyllm_device_status() == 0


def test_fused_offset_launch_matches_oracle(cuda_device):
    from dyllm_b200.attention_ops import fused_offset_launch

    cu_q, cu_k, cu_p = orc.make_batch_layout(16, 256, 256, True)
    _, _, stats = _stats_case(int(cu_q[-1]), 64, seed=3)
    want = orc.salient_select(stats, 0.99, cu_q, cu_p)
    n = want["count"]
    out = torch.full((int(cu_q[-1]),), -7, dtype=torch.int64, device=cuda_device)
    fused_offset_launch(want["idx"].to(torch.int32).to(cuda_device),
                        torch.tensor([n], dtype=torch.int32, device=cuda_device), cu_p.to(cuda_device),
                        want["cu_salientlens"].to(cuda_device), out, out.numel())
    assert torch.equal(out[:n].cpu(), want["idx_k"])
    assert bool((out[n:] == -7).all())
    with pytest.raises(RuntimeError):
        fused_offset_launch(want["idx"].to(cuda_device), torch.tensor([n], dtype=torch.int32, device=cuda_device),
                            cu_p.to(cuda_device), want["cu_salientlens"].to(cuda_device), out, out.numel())
