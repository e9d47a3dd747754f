"""Parity of the fused add-RMSNorm and rotary-embedding kernels with the oracle's restatement of the
reference modules (bf16 outputs, one bf16 ulp of slack)."""
import pytest
import torch

from dyllm_b200 import ops
from oracle import dyllm_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,width", [(1, 8), (33, 256), (512, 4096), (100, 3584), (7, 8192)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_add_rms_norm(cuda_device, rows, width, with_residual):
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g).bfloat16()
    w = (1.0 + 0.1 * torch.randn(width, generator=g)).bfloat16()
    res = torch.randn(rows, width, generator=g).bfloat16() if with_residual else None
    got = ops.add_rms_norm(x.to(cuda_device), w.to(cuda_device), 1e-5, res.to(cuda_device) if with_residual else None)
    want = orc.rms_norm(x, w, 1e-5, residual=res)
    if with_residual:
        torch.testing.assert_close(got[1].cpu().float(), want[1].float(), rtol=0, atol=0)
        got, want = got[0], want[0]
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=1.6e-2, atol=1e-3)
    rel = (got.cpu().float() - want.float()).norm() / want.float().norm()
    assert rel < 3e-3


@pytest.mark.parametrize("rows,heads", [(1, 1), (77, 4), (4096, 32)])
def test_rope_neox(cuda_device, rows, heads):
    from dyllm_b200 import ops
    from dyllm_b200.layers import RotaryEmbedding

    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, heads, 128, generator=g).bfloat16()
    pos = torch.randint(0, 600, (rows,), generator=g)  # some beyond the table: clamped
    rope = RotaryEmbedding(128, 128, 512, 500000.0)
    got = ops.rope_neox_(x.to(cuda_device).clone(), pos.to(cuda_device), rope.cos_sin_cache.view(-1, 128).to(cuda_device))
    want = orc.rope(pos, x, 128, 500000.0, 512)
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=8e-3, atol=1e-3)
    # indexed positions (salient K rows use positions[idx])
    idx = torch.randint(0, rows, (max(rows // 2, 1),), generator=g)
    xi = x[: idx.numel()].contiguous()
    got = ops.rope_neox_(xi.to(cuda_device).clone(), pos.to(cuda_device), rope.cos_sin_cache.view(-1, 128).to(cuda_device),
                         pos_idx=idx.to(cuda_device))
    want = orc.rope(pos[idx], xi, 128, 500000.0, 512)
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=8e-3, atol=1e-3)


@pytest.mark.parametrize("rows,vocab", [(7, 126464), (33, 1000), (4, 1021 + 3), (1, 8)])
def test_row_confidence_matches_softmax_max(cuda_device, rows, vocab):
    """max softmax probability and its token (ref: sampler.py:286-288), bf16 logits, fp32 arithmetic."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows * 7 + vocab)
    logits = (torch.randn(rows, vocab, generator=g) * 4.0).bfloat16()
    logits[0, vocab // 2] = 30.0          # one sharply peaked row
    if rows > 1:
        logits[1, 5] = logits[1].max()    # a tie: the first index wins
    conf, tok = ops.row_confidence(logits.to(cuda_device))
    want = torch.softmax(logits.double(), dim=-1)
    want_conf, _ = want.max(dim=-1)
    assert torch.allclose(conf.cpu().double(), want_conf, rtol=1e-4, atol=1e-7)
    lf = logits.float()
    first_max = (lf == lf.max(dim=-1, keepdim=True).values).float().argmax(dim=-1)
    assert torch.equal(tok.cpu(), first_max)


def test_add_rms_norm_reads_equal_blocks_in_place(cuda_device):
    """x given as a strided [segments, rows, width] view (the last rows of every sequence inside a cache)
    gives the same bits as the packed copy."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(11)
    B, L, R, W = 5, 48, 20, 512
    cache = torch.randn(B * L + 7, W, generator=g).bfloat16().to(cuda_device)
    w = (1.0 + 0.1 * torch.randn(W, generator=g)).bfloat16().to(cuda_device)
    res = torch.randn(B * R, W, generator=g).bfloat16().to(cuda_device)
    view = cache[3 : 3 + B * L].view(B, L, W)[:, L - R :, :]
    packed = view.reshape(B * R, W).contiguous()
    y1, r1 = ops.add_rms_norm(packed, w, 1e-5, res)
    y2, r2 = ops.add_rms_norm(view, w, 1e-5, res)
    assert torch.equal(y1, y2) and torch.equal(r1, r2)
    assert torch.equal(ops.add_rms_norm(packed, w, 1e-5), ops.add_rms_norm(view, w, 1e-5))


@pytest.mark.parametrize("rows,width,n_sel,live", [(300, 4096, 300, 37), (64, 3584, 10, 10), (2000, 2048, 1500, 1500), (16, 256, 16, 0)])
def test_add_rms_norm_rows_equals_full_norm_on_listed_rows(cuda_device, rows, width, n_sel, live):
    """Residual sums of every row and normalised values of the listed rows only: the same bits as the full
    norm, packed in list order; rows past the live count are left alone."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows + width)
    dev = cuda_device
    x = torch.randn(rows, width, generator=g).bfloat16().to(dev)
    res = torch.randn(rows, width, generator=g).bfloat16().to(dev)
    w = (1.0 + 0.1 * torch.randn(width, generator=g)).bfloat16().to(dev)
    idx = torch.sort(torch.randperm(rows, generator=g)[:n_sel]).values.to(torch.int32).to(dev)
    count = torch.tensor([live], dtype=torch.int32, device=dev)
    y_full, res_full = ops.add_rms_norm(x, w, 1e-5, res)
    y_sel, res_out, none = ops.add_rms_norm_rows(x, w, 1e-5, res, idx, count)
    assert none is None and torch.equal(res_out, res_full)
    assert torch.equal(y_sel[:live], y_full[idx[:live].long()])
    # without a device-side count the whole list is live
    y_list, _, _ = ops.add_rms_norm_rows(x, w, 1e-5, res, idx, None)
    assert torch.equal(y_list, y_full[idx.long()])
    # every row normalised as well (the input norm of a sparse step), with and without a residual
    y_sel, res_out, y_all = ops.add_rms_norm_rows(x, w, 1e-5, res, idx, count, all_rows=True)
    assert torch.equal(y_all, y_full) and torch.equal(res_out, res_full) and torch.equal(y_sel[:live], y_full[idx[:live].long()])
    y_plain = ops.add_rms_norm(x, w, 1e-5)
    y_sel, res_out, y_all = ops.add_rms_norm_rows(x, w, 1e-5, None, idx, count, all_rows=True)
    assert res_out is None and torch.equal(y_all, y_plain) and torch.equal(y_sel[:live], y_plain[idx[:live].long()])
    # segmented input: a block of every sequence read out of a cache
    if rows % 4 == 0:
        seg = rows // 4
        cache = torch.randn(4, seg + 7, width, generator=g).bfloat16().to(dev)
        view = cache[:, 7:, :]
        y_full, res_full = ops.add_rms_norm(view, w, 1e-5, res)
        y_sel, res_out, y_all = ops.add_rms_norm_rows(view, w, 1e-5, res, idx, count, all_rows=True)
        assert torch.equal(res_out, res_full) and torch.equal(y_sel[:live], y_full[idx[:live].long()])
        assert torch.equal(y_all, y_full)


@pytest.mark.parametrize("rows,heads,live", [(300, 16, 300), (64, 2, 17), (5000, 4, 5000)])
def test_head_rms_norm_matches_the_oracle(cuda_device, rows, heads, live):
    """The per-head q / k normalisation of LLaDA-MoE (lladamoe.py:195-207): RMSNorm over each 128-vector."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows + heads)
    x = torch.randn(rows, heads, 128, generator=g).bfloat16()
    w = (1.0 + 0.2 * torch.randn(128, generator=g)).bfloat16()
    count = torch.tensor([live], dtype=torch.int32, device=cuda_device)
    got = ops.head_rms_norm_(x.to(cuda_device).clone(), w.to(cuda_device), 1e-5, count).cpu()
    want = orc.rms_norm(x.view(-1, 128), w, 1e-5).view(rows, heads, 128)
    torch.testing.assert_close(got[:live].float(), want[:live].float(), rtol=1.6e-2, atol=1e-3)
    assert torch.equal(got[live:], x[live:])
    # the row-wise norm kernel on the flattened view gives the same values up to the order of its fp32 sum
    ref = ops.add_rms_norm(x.view(-1, 128).to(cuda_device), w.to(cuda_device), 1e-5).cpu().view(rows, heads, 128)
    torch.testing.assert_close(got[:live].float(), ref[:live].float(), rtol=1.6e-2, atol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("batch,prompt,block_len,blocks,num_transfer,step", [
    (16, 256, 32, 8, 1, 0), (16, 256, 32, 8, 1, 100), (3, 40, 8, 4, 2, 9), (5, 7, 64, 2, 4, 40), (2, 0, 1024, 1, 64, 0),
    (4, 16, 32, 2, 8, 3),
])
def test_confidence_unmask_matches_the_sampler_rule(cuda_device, batch, prompt, block_len, blocks, num_transfer, step):
    g = torch.Generator().manual_seed(batch * 131 + block_len)
    mask_id, steps_per_block = 126336, 32
    length = prompt + blocks * block_len
    block = min(step // steps_per_block, blocks - 1)
    start = prompt + block * block_len
    tokens = torch.randint(0, 1000, (batch, length), generator=g)
    masked = torch.rand(batch, length, generator=g) < 0.6
    tokens = torch.where(masked, torch.full_like(tokens, mask_id), tokens)
    tokens[0, start:start + block_len] = mask_id                    # everything masked
    if batch > 1:
        tokens[1, start:start + block_len] = 7                       # nothing masked: no pick
    if batch > 2:
        tokens[2, start:start + block_len] = 7
        tokens[2, start + block_len - 1] = mask_id                   # fewer candidates than picks (when picks > 1)
    conf = torch.rand(batch, block_len, generator=g)
    conf[:, ::3] = conf[:, :1]                                       # ties: the lowest position wins
    best = torch.randint(0, 1000, (batch, block_len), generator=g)
    want_tokens, want_picked = orc.confidence_unmask(conf, best, tokens, start, block_len, num_transfer, mask_id)

    dev_tokens = torch.zeros(batch, length + 3, dtype=torch.int64, device=cuda_device)[:, :length]   # pitch != length
    dev_tokens.copy_(tokens)
    assert dev_tokens.stride(0) == length + 3
    counter = torch.tensor([step], dtype=torch.int64, device=cuda_device)
    picked = ops.confidence_unmask_(conf.to(cuda_device), best.to(cuda_device), dev_tokens, counter, steps_per_block, prompt,
                                    block_len, num_transfer, mask_id)
    assert torch.equal(dev_tokens.cpu(), torch.from_numpy(want_tokens))
    for b in range(batch):
        got = [p for p in picked[b].tolist() if p >= 0]
        assert got == want_picked[b], (b, got, want_picked[b])
        assert picked[b].tolist()[len(got):] == [-1] * (num_transfer - len(got))
