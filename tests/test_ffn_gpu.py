"""Parity of the tcgen05 gathered GEMMs / SwiGLU FFN with the fp32 oracle.

Tolerances follow the path's contract: bf16 outputs within max-abs 2e-2 and relative L2 1e-2.
Both ways of feeding activation rows are covered: a_mode 0 (rows staged into a compact buffer, plain TMA
boxes) and a_mode 1 (TMA gather4 straight from the activation tensor).
"""
import pytest
import torch

from oracle import dyllm_oracle as orc

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = 2e-2, 1e-2


def _check(got, want, what):
    got, want = got.float().cpu(), want.float().cpu()
    # max-abs is stated for outputs of unit scale; larger outputs are compared relative to their peak
    # (a bf16 ulp at |x| = 8 is already 0.03)
    err = (got - want).abs().max().item() / max(1.0, want.abs().max().item())
    rel = ((got - want).norm() / want.norm().clamp_min(1e-12)).item()
    assert err <= MAX_ABS and rel <= REL_L2, f"{what}: scaled max-abs {err:.4g}, rel-L2 {rel:.4g}"


def _status_ok():
    from dyllm_b200 import _lib

    assert _lib.load().dyllm_device_status() == 0


@pytest.mark.parametrize("a_mode", [0, 1], ids=["staged", "gather4"])
@pytest.mark.parametrize("rows,k,n,tile_n", [(128, 64, 64, 64), (26, 256, 128, 128), (410, 4096, 1024, 0),
                                              (300, 3584, 512, 64)])
def test_gathered_linear(cuda_device, a_mode, rows, k, n, tile_n):
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows + k)
    total = max(rows * 3, 512)
    x = torch.randn(total, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    idx = torch.sort(torch.randperm(total, generator=g)[:rows]).values.to(torch.int32)
    want = x.float()[idx.long()] @ w.float().t()
    got = ops.gathered_linear(x.to(cuda_device), w.to(cuda_device), idx.to(cuda_device), a_mode=a_mode, tile_n=tile_n)
    _status_ok()
    _check(got, want.bfloat16(), f"gathered_linear mode {a_mode}")


@pytest.mark.parametrize("a_mode", [0, 1], ids=["staged", "gather4"])
def test_gathered_linear_scatter_scale_and_device_count(cuda_device, a_mode):
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(5)
    x = torch.randn(700, 512, generator=g).bfloat16()
    w = (torch.randn(256, 512, generator=g) * 0.05).bfloat16()
    idx = torch.sort(torch.randperm(700, generator=g)[:300]).values.to(torch.int32)
    live = 211
    dest = torch.randperm(400, generator=g)[:300].to(torch.int32)
    dest[7] = -1  # dropped row
    scale = torch.rand(300, generator=g)
    out = torch.full((400, 256), 3.0).bfloat16().to(cuda_device)
    ops.gathered_linear(x.to(cuda_device), w.to(cuda_device), idx.to(cuda_device),
                        num_rows_dev=torch.tensor([live], dtype=torch.int32, device=cuda_device), out=out,
                        out_row_map=dest.to(cuda_device), row_scale=scale.to(cuda_device), a_mode=a_mode)
    _status_ok()
    want = torch.full((400, 256), 3.0)
    y = (x.float()[idx.long()] @ w.float().t()) * scale[:, None]
    for m in range(live):
        if dest[m] >= 0:
            want[dest[m]] = y[m]
    _check(out, want.bfloat16(), "scatter/scale")
    untouched = torch.ones(400, dtype=torch.bool)
    untouched[dest[:live][dest[:live] >= 0].long()] = False
    assert bool((out.cpu()[untouched] == 3.0).all())


@pytest.mark.parametrize("a_mode", [0, 1], ids=["staged", "gather4"])
@pytest.mark.parametrize("rows,hidden,inter,tile_n", [(26, 4096, 12288, 0), (410, 4096, 12288, 0), (130, 512, 1024, 64),
                                                       (130, 512, 1024, 128), (1, 256, 128, 64),
                                                       # Dream-7B FFN shards under tensor parallelism 2 and 4, LLaDA-8B under 8
                                                       (410, 3584, 9472, 0), (410, 3584, 4736, 0), (48, 4096, 1536, 0)])
def test_swiglu_ffn_matches_oracle(cuda_device, a_mode, rows, hidden, inter, tile_n):
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows)
    total = max(2 * rows, 512)
    x = torch.randn(total, hidden, generator=g).bfloat16()
    w1 = (torch.randn(2 * inter, hidden, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(hidden, inter, generator=g) * 0.02).bfloat16()
    idx = torch.sort(torch.randperm(total, generator=g)[:rows]).values.to(torch.int32)
    want = orc.swiglu_ffn(x[idx.long()], w1, w2)
    got = ops.swiglu_ffn(x.to(cuda_device), w1.to(cuda_device), w2.to(cuda_device), idx.to(cuda_device),
                         a_mode=a_mode, tile_n=tile_n)
    _status_ok()
    _check(got, want, f"swiglu_ffn mode {a_mode}")


def test_swiglu_ffn_scatters_into_cache_rows(cuda_device):
    """Fused path: rows of the FFN output land in the per-sequence cache rows that scatter_update would write."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(8)
    batch, L, hidden, inter = 4, 128, 512, 1024
    cu = (torch.arange(batch + 1) * L).to(torch.int32)
    seq_ids = torch.tensor([9, 2, 5, 11])
    seq_starts = torch.full((16,), -1, dtype=torch.int64)
    for j, s in enumerate([2, 0, 3, 1]):
        seq_starts[seq_ids[j]] = s * L
    x = torch.randn(batch * L, hidden, generator=g).bfloat16()
    w1 = (torch.randn(2 * inter, hidden, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(hidden, inter, generator=g) * 0.02).bfloat16()
    rows = torch.sort(torch.randperm(batch * L, generator=g)[:77]).values
    cache = torch.randn(batch * L, hidden, generator=g).bfloat16()
    d = lambda t: t.to(cuda_device)
    dest = ops.cache_dest_rows(d(rows), d(cu), d(seq_starts), d(seq_ids))
    dcache = d(cache)
    ops.swiglu_ffn(d(x), d(w1), d(w2), d(rows.to(torch.int32)), out=dcache, out_row_map=dest)
    _status_ok()
    want = orc.cache_scatter_update(cache.clone(), orc.swiglu_ffn(x[rows], w1, w2).bfloat16(), rows, cu, seq_starts,
                                    seq_ids)
    _check(dcache, want, "ffn scatter")
    touched = torch.zeros(batch * L, dtype=torch.bool)
    touched[dest.cpu().long()] = True
    assert torch.equal(dcache.cpu()[~touched], cache[~touched])


@pytest.mark.parametrize("a_mode", [0, 1], ids=["staged", "gather4"])
@pytest.mark.parametrize("bound,live,hint,k,n", [
    (1024, 211, 200, 512, 256),    # device-side count below the bound
    (1024, 700, 100, 512, 256),    # hint too small: each CTA walks over several row tiles; split-K declined on the device
    (512, 26, 26, 4096, 256),      # few rows, few column tiles: split-K
    (1024, 200, 128, 4096, 256),   # two live row tiles under a one-tile hint: fewer splits, chosen on the device
    (1024, 400, 128, 4096, 1024),  # four live row tiles: the splits of the grid are all declined
    (1024, 513, 128, 4096, 256),   # just above the split-K row limit
    (2048, 0, 64, 256, 128),       # nothing live
])
def test_gathered_linear_device_count_hint_and_split_k(cuda_device, a_mode, bound, live, hint, k, n):
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(bound + live)
    x = torch.randn(2048, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.03).bfloat16()
    idx = torch.sort(torch.randperm(2048, generator=g)[:bound]).values.to(torch.int32)
    out = torch.full((bound, n), 5.0, dtype=torch.bfloat16, device=cuda_device)
    ops.gathered_linear(x.to(cuda_device), w.to(cuda_device), idx.to(cuda_device), num_rows=bound,
                        num_rows_dev=torch.tensor([live], dtype=torch.int32, device=cuda_device), rows_hint=hint,
                        out=out, a_mode=a_mode)
    _status_ok()
    if live:
        want = (x.float()[idx[:live].long()] @ w.float().t()).bfloat16()
        _check(out[:live], want, "device count")
    assert bool((out[live:] == 5.0).all())


def test_gathered_linear_column_split_into_two_outputs(cuda_device):
    """Fused K/V projection: the first half of the columns lands in one tensor, the second in another."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(3)
    x = torch.randn(600, 512, generator=g).bfloat16()
    w = (torch.randn(512, 512, generator=g) * 0.03).bfloat16()
    idx = torch.sort(torch.randperm(600, generator=g)[:150]).values.to(torch.int32)
    k_out = torch.zeros(150, 256, dtype=torch.bfloat16, device=cuda_device)
    v_out = torch.zeros(150, 256, dtype=torch.bfloat16, device=cuda_device)
    ops.gathered_linear(x.to(cuda_device), w.to(cuda_device), idx.to(cuda_device), out=k_out, out2=v_out, split_col=256)
    _status_ok()
    want = (x.float()[idx.long()] @ w.float().t()).bfloat16()
    _check(k_out, want[:, :256], "K half")
    _check(v_out, want[:, 256:], "V half")


@pytest.mark.parametrize("bound,live,hint", [(2048, 300, 280), (2048, 900, 128), (256, 40, 0)])
def test_swiglu_ffn_device_count(cuda_device, bound, live, hint):
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(live)
    hidden, inter = 512, 1024
    x = torch.randn(2048, hidden, generator=g).bfloat16()
    w1 = (torch.randn(2 * inter, hidden, generator=g) * 0.03).bfloat16()
    w2 = (torch.randn(hidden, inter, generator=g) * 0.03).bfloat16()
    idx = torch.sort(torch.randperm(2048, generator=g)[:bound]).values.to(torch.int32)
    out = torch.full((bound, hidden), 5.0, dtype=torch.bfloat16, device=cuda_device)
    ops.swiglu_ffn(x.to(cuda_device), w1.to(cuda_device), w2.to(cuda_device), idx.to(cuda_device), num_rows=bound,
                   num_rows_dev=torch.tensor([live], dtype=torch.int32, device=cuda_device), rows_hint=hint, out=out)
    _status_ok()
    _check(out[:live], orc.swiglu_ffn(x[idx[:live].long()], w1, w2), "swiglu device count")
    assert bool((out[live:] == 5.0).all())


@pytest.mark.parametrize("rows,k,n,tile_n,with_idx", [(2500, 256, 4096, 0, True), (2500, 256, 4096, 256, True),
                                                       (4096, 512, 4096, 0, False), (2433, 192, 8192, 0, True)])
def test_gathered_linear_many_rows_on_256_wide_tiles(cuda_device, rows, k, n, tile_n, with_idx):
    """Plain products with thousands of rows run on 256 x 256 tiles (two 128-row accumulators per 256-column
    weight tile); ragged last row tile, index list or every row."""
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(rows + n)
    total = rows * 2 if with_idx else rows
    x = torch.randn(total, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    if with_idx:
        idx = torch.sort(torch.randperm(total, generator=g)[:rows]).values.to(torch.int32)
        want = x.float()[idx.long()] @ w.float().t()
        got = ops.gathered_linear(x.to(cuda_device), w.to(cuda_device), idx.to(cuda_device), tile_n=tile_n)
    else:
        want = x.float() @ w.float().t()
        got = ops.gathered_linear(x.to(cuda_device), w.to(cuda_device), None, num_rows=rows, rows_hint=rows, tile_n=tile_n)
    _status_ok()
    _check(got, want.bfloat16(), "gathered_linear on 256-wide tiles")
