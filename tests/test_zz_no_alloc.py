"""The selection entry point that allocates nothing (scratch memory inside the library) must give the
same lists as the entry point that takes a caller-provided workspace.

Some hosts cannot allocate while they serve: they gave all device memory to their own pool at start-up,
or an allocation in the step loop would stall the device.  This file is collected last so that a run
stopping at the first failure has already run every other test; the test passes both alone in a fresh
process and after the others (the library's scratch array then holds stale content from earlier calls).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _select_static(stats, tau, cu_q, cu_p):
    from dyllm_b200._lib import call, ptr, stream_ptr

    rows, dev = stats.size(0), stats.device
    batch = cu_q.numel() - 1
    out = dict(idx=torch.full((rows,), -1, dtype=torch.int64, device=dev),
               idx32=torch.full((rows,), -1, dtype=torch.int32, device=dev),
               idx_k=torch.full((rows,), -1, dtype=torch.int64, device=dev),
               cu_sal=torch.full((batch + 1,), -1, dtype=torch.int32, device=dev),
               count=torch.full((1,), -1, dtype=torch.int32, device=dev),
               mask=torch.zeros((rows,), dtype=torch.bool, device=dev))
    call("dyllm_salient_select_static", ptr(stats), rows, float(tau), ptr(cu_q), batch, ptr(cu_p), ptr(out["idx"]),
         ptr(out["idx32"]), ptr(out["idx_k"]), ptr(out["cu_sal"]), ptr(out["count"]), ptr(out["mask"]), stream_ptr(dev))
    return out


def _case(rows_per_seq, batch, seed, dev):
    g = torch.Generator().manual_seed(seed)
    rows = rows_per_seq * batch
    stats = torch.ones(rows, 3)
    stats[:, 0] = torch.where(torch.rand(rows, generator=g) < 0.15, 0.6, 0.9995)
    cu_q = (torch.arange(batch + 1) * rows_per_seq).to(torch.int32)
    cu_p = (torch.arange(batch + 1) * 256).to(torch.int32)
    return stats.to(dev), cu_q.to(dev), cu_p.to(dev)


def test_no_alloc_selection_matches_workspace_selection_twice(cuda_device):
    from dyllm_b200 import _lib, ops
    from oracle import dyllm_oracle as orc

    # calls in a row with different sizes: a later one must not see an earlier one's descriptors.  The
    # first case lies above 64 Ki rows, where the selection switches to its wide-tile instance.
    for rows_per_seq, batch, seed in ((9000, 16, 3), (4096, 16, 1), (777, 5, 2)):
        stats, cu_q, cu_p = _case(rows_per_seq, batch, seed, cuda_device)
        want = ops.salient_select(stats, 0.99, cu_q, cu_p, want_mask=True)
        got = _select_static(stats, 0.99, cu_q, cu_p)
        n = int(want.count.item())
        # ... and against the CPU restatement of the reference directly
        ref = orc.salient_select(stats.cpu(), 0.99, cu_q.cpu(), cu_p.cpu())
        assert ref["count"] == int(got["count"].item())
        assert torch.equal(got["idx"][:n].cpu(), ref["idx"])
        assert torch.equal(got["idx_k"][:n].cpu(), ref["idx_k"])
        assert torch.equal(got["cu_sal"].cpu(), ref["cu_salientlens"])
        assert torch.equal(got["mask"].cpu(), ref["mask"])
        assert n > 0 and int(got["count"].item()) == n
        assert torch.equal(got["idx"][:n], want.idx[:n])
        assert torch.equal(got["idx32"][:n], want.idx32[:n])
        assert torch.equal(got["idx_k"][:n], want.idx_k[:n])
        assert torch.equal(got["cu_sal"], want.cu_salientlens)
        assert torch.equal(got["mask"], want.mask)
        assert bool((got["idx"][n:] == -1).all())
    assert _lib.load().dyllm_device_status() == 0


def test_no_alloc_selection_rejects_oversized_input(cuda_device):
    from dyllm_b200 import _lib

    lib = _lib.load()
    limit = lib.dyllm_salient_select_static_max_rows()
    assert limit >= 1 << 20
    dummy = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    rc = lib.dyllm_salient_select_static(dummy.data_ptr(), limit + 1, 0.99, dummy.data_ptr(), 1, None, dummy.data_ptr(),
                                         None, None, dummy.data_ptr(), dummy.data_ptr(), None, None)
    assert rc == -2
    assert str(limit).encode() in lib.dyllm_last_error()
