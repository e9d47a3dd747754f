"""This package's sm_100a kernels, through the C ABI, against outputs of the REFERENCE's own CUDA kernels
and of flash-attn recorded on a B200 (tests/golden/ref_kernels.pt, made by tests/golden/make_ref_golden.py)."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_ref_golden as mrg  # noqa: E402
from test_ref_golden import FIXTURE, check_decisions, check_outputs  # noqa: E402


@pytest.fixture(scope="module")
def golden():
    return torch.load(FIXTURE)


@pytest.mark.parametrize("compact_dv", [False, True])
@pytest.mark.parametrize("name", list(mrg.ATTENTION_CASES))
def test_attention_kernels_match_reference_kernel(cuda_device, golden, name, compact_dv):
    from dyllm_b200 import _lib
    from dyllm_b200.attention_ops import attention_salient_rows, attention_sparse_varlen

    if name not in golden["attention"]:
        pytest.skip("case not in the recorded fixture")
    dev = cuda_device
    rec = golden["attention"][name]
    c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in mrg.attention_case(name).items()}
    S = c["idx_q"].numel()
    ik = c["idx_k"].long()
    # exact attention of the salient rows against flash-attn's output
    v_now = c["v_cache"].clone()
    v_now[ik] = (c["v_cache"][ik].float() + c["dv"][ik].float()).to(torch.bfloat16)
    max_rows = int((c["cu_sal"][1:] - c["cu_sal"][:-1]).max())
    o_sal = attention_salient_rows(c["q"], c["k"], v_now, c["cu_k"], c["cu_sal"], c["idx_q"], max_rows_per_seq=max(max_rows, 1))
    if "flash_o_sal" in rec and S:
        check_outputs(o_sal.cpu(), rec["flash_o_sal"], name + " (salient rows)")
    # approximate attention with the reference run's own o_sal, so that only this kernel is compared
    stats = torch.zeros((c["q"].size(0), 3), dtype=torch.float32, device=dev)
    mask = torch.empty((c["q"].size(0),), dtype=torch.bool, device=dev)
    dv = c["dv"][ik].contiguous() if compact_dv else c["dv"]
    O = attention_sparse_varlen(c["q"], c["k"], dv, c["c_old"], rec["o_sal_used"].to(dev), c["cu_q"], c["cu_k"], c["max_q"],
                                c["max_k"], c["q"].size(0), c["cu_sal"], c["idx_q"], stats, mask, c["tau"], c["pruned"],
                                c["idx_k"] if c["pruned"] else None, v_layout=3 if compact_dv else 1)
    torch.cuda.synchronize()
    assert _lib.load().dyllm_device_status() == 0
    check_outputs(O.cpu(), rec["O"], name)
    assert torch.allclose(stats.cpu(), rec["stats"], rtol=2e-3, atol=2e-2), (stats.cpu() - rec["stats"]).abs().max()
    check_decisions(mask.cpu(), rec["stats"], rec["mask"], c["tau"], name)


def test_cache_kernels_match_reference_kernels(cuda_device, golden):
    from dyllm_b200 import cache as ck

    dev = cuda_device
    rec = golden["cache"]
    c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in mrg.cache_case().items()}
    got = ck.get_seqs_cuda(c["cache"], c["seq_starts"], c["cu"], c["seq_ids"], c["total"])
    assert torch.equal(got.cpu(), rec["get_seqs"])
    got = ck.get_block_cuda(c["cache"], c["seq_starts"], c["cu"], c["cu_q"], c["seq_ids"], c["total_q"])
    assert torch.equal(got.cpu(), rec["get_block"])
    c1 = c["cache"].clone()
    ck.reset_full_cuda(c1, c["new_full"], c["seq_starts"], c["cu"], c["seq_ids"], c["total"])
    assert torch.equal(c1.cpu(), rec["reset_full"])
    c2 = c["cache"].clone()
    ck.reset_block_cuda(c2, c["new_block"], c["seq_starts"], c["cu"], c["cu_q"], c["seq_ids"], c["total_q"])
    assert torch.equal(c2.cpu(), rec["reset_block"])
    c3 = c["cache"].clone()
    ck.scatter_update_cuda(c3, c["new_rows"], c["rows"], c["cu"], c["seq_starts"], c["seq_ids"])
    assert torch.equal(c3.cpu(), rec["scatter_update"])


def test_fused_offset_and_fused_selection_match_reference_kernel(cuda_device, golden):
    from dyllm_b200.attention_ops import fused_offset_launch

    dev = cuda_device
    rec = golden["cache"]
    c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in mrg.cache_case().items()}
    out = torch.full((16,), -1, dtype=torch.int64, device=dev)
    n = torch.tensor([c["idxs"].numel()], dtype=torch.int32, device=dev)
    fused_offset_launch(c["idxs"], n, c["cu_prompt"], c["cu_sal"], out, 16)
    assert torch.equal(out.cpu(), rec["fused_offset"])
