"""Parity of the fused add-RMSNorm and rotary-embedding kernels with the oracle's restatement of the
reference modules (bf16 outputs, one bf16 ulp of slack)."""
import pytest
import torch

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
