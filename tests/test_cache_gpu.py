"""Parity of the activation-cache copy kernels with the CPU oracle (bit-exact byte movement)."""
import pytest
import torch

from oracle import dyllm_oracle as orc

pytestmark = pytest.mark.gpu


def _setup(lens, width, dtype, seed=0, max_seqs=64):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    cache = torch.randn(total + 5, width, generator=g).to(dtype)
    # sequences live in the cache in a shuffled order with arbitrary ids
    order = torch.randperm(len(lens), generator=g).tolist()
    ids = torch.randperm(max_seqs, generator=g)[: len(lens)]
    seq_starts = torch.full((max_seqs,), -1, dtype=torch.int64)
    pos = 0
    for j in order:
        seq_starts[ids[j]] = pos
        pos += lens[j]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return cache, seq_starts, ids.to(torch.int64), cu


CASES = [([512], 4096, torch.bfloat16), ([5, 0, 17, 33], 128, torch.bfloat16), ([512] * 16, 512, torch.bfloat16),
         ([7, 9], 8, torch.bfloat16), ([3, 4], 12, torch.float32)]


@pytest.mark.parametrize("lens,width,dtype", CASES)
def test_get_and_reset_full(cuda_device, lens, width, dtype):
    from dyllm_b200 import cache as C

    cache, ss, ids, cu = _setup(lens, width, dtype)
    total = int(cu[-1])
    d = lambda t: t.to(cuda_device)
    got = C.get_seqs_cuda(d(cache), d(ss), d(cu), d(ids), total)
    want = orc.cache_get_seqs(cache, ss, cu, ids, total)
    assert torch.equal(got.cpu(), want)
    new = torch.randn(total, width).to(dtype)
    dc = d(cache)
    C.reset_full_cuda(dc, d(new), d(ss), d(cu), d(ids), total)
    assert torch.equal(dc.cpu(), orc.cache_reset_full(cache.clone(), new, ss, cu, ids))


@pytest.mark.parametrize("lens,width,dtype", CASES[:4])
def test_get_and_reset_block(cuda_device, lens, width, dtype):
    from dyllm_b200 import cache as C

    cache, ss, ids, cu_k = _setup(lens, width, dtype, seed=1)
    qlens = [l // 2 for l in lens]
    cu_q = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    total = int(cu_q[-1])
    d = lambda t: t.to(cuda_device)
    got = C.get_block_cuda(d(cache), d(ss), d(cu_k), d(cu_q), d(ids), total)
    assert torch.equal(got.cpu(), orc.cache_get_block(cache, ss, cu_k, cu_q, ids, total))
    new = torch.randn(total, width).to(dtype)
    dc = d(cache)
    C.reset_block_cuda(dc, d(new), d(ss), d(cu_k), d(cu_q), d(ids), total)
    assert torch.equal(dc.cpu(), orc.cache_reset_block(cache.clone(), new, ss, cu_k, cu_q, ids))


@pytest.mark.parametrize("cu_dtype", [torch.int32, torch.int64])
def test_scatter_update(cuda_device, cu_dtype):
    from dyllm_b200 import cache as C

    lens = [512] * 4 + [100]
    cache, ss, ids, cu = _setup(lens, 1024, torch.bfloat16, seed=2)
    total = int(cu[-1])
    g = torch.Generator().manual_seed(9)
    rows = torch.sort(torch.randperm(total, generator=g)[:211]).values
    new = torch.randn(211, 1024, generator=g).bfloat16()
    d = lambda t: t.to(cuda_device)
    dc = d(cache)
    C.scatter_update_cuda(dc, d(new), d(rows), d(cu.to(cu_dtype)), d(ss), d(ids))
    assert torch.equal(dc.cpu(), orc.cache_scatter_update(cache.clone(), new, rows, cu, ss, ids))
    # device-side row count: only the first 100 rows are consumed; zero rows is a no-op
    dc2 = d(cache)
    C.scatter_update_cuda(dc2, d(new), d(rows), d(cu), d(ss), d(ids),
                          num_rows_dev=torch.tensor([100], dtype=torch.int32, device=cuda_device))
    assert torch.equal(dc2.cpu(), orc.cache_scatter_update(cache.clone(), new[:100], rows[:100], cu, ss, ids))
    C.scatter_update_cuda(dc2, d(new[:0]), d(rows[:0]), d(cu), d(ss), d(ids))


def test_errors_are_runtime_errors(cuda_device):
    from dyllm_b200 import cache as C

    cache, ss, ids, cu = _setup([4], 8, torch.bfloat16)
    d = lambda t: t.to(cuda_device)
    with pytest.raises(RuntimeError):
        C.get_seqs_cuda(d(cache), d(ss), d(cu).long(), d(ids), 4)  # cu must be int32
    with pytest.raises(RuntimeError):
        C.get_seqs_cuda(d(cache)[:, :3].contiguous(), d(ss), d(cu), d(ids), 4)  # row not a multiple of 16 bytes
    with pytest.raises(RuntimeError):
        C.reset_full_cuda(d(cache), d(cache)[:, :4].contiguous(), d(ss), d(cu), d(ids), 4)


@pytest.mark.parametrize("live", [37, 0])
def test_kv_cache_update_equals_the_separate_steps(cuda_device, live):
    """rope of the new keys + K-cache scatter + delta-V + V-cache update in one launch gives the same bits
    as rope_neox_ / scatter_update_cuda / cache_dest_rows / delta_v_update one after the other."""
    from dyllm_b200 import cache as C
    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(5)
    B, L, Hkv, D, cap = 3, 96, 2, 128, 64
    dev = cuda_device
    cu = (torch.arange(B + 1) * L).to(torch.int32).to(dev)
    seq_ids = torch.tensor([2, 0, 1], device=dev)
    k_starts = torch.tensor([L, 2 * L + 8, 0], device=dev)          # per sequence id; the two caches differ
    v_starts = torch.tensor([2 * L, 0, L + 5], device=dev)
    k_cache = torch.randn(3 * L + 16, Hkv * D, generator=g).bfloat16().to(dev)
    v_cache = torch.randn(3 * L + 16, Hkv * D, generator=g).bfloat16().to(dev)
    rows_k = torch.sort(torch.randperm(B * L, generator=g)[:cap]).values.to(dev)
    positions = torch.randint(0, 300, (B * L,), generator=g).to(dev)
    pos_idx = torch.randint(0, B * L, (cap,), generator=g).to(dev)
    k_new = torch.randn(cap, Hkv, D, generator=g).bfloat16().to(dev)
    v_new = torch.randn(cap, Hkv, D, generator=g).bfloat16().to(dev)
    t = torch.arange(512, dtype=torch.float)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float) / D))
    f = torch.einsum("i,j->ij", t, inv)
    cos_sin = torch.cat((f.cos(), f.sin()), dim=-1).to(dev)
    n_dev = torch.tensor([live], dtype=torch.int32, device=dev)

    k1, v1 = k_cache.clone(), v_cache.clone()
    kr = ops.rope_neox_(k_new.clone(), positions, cos_sin, pos_idx=pos_idx, num_rows_dev=n_dev)
    C.scatter_update_cuda(k1, kr.view(cap, -1), rows_k, cu, k_starts, seq_ids, n_dev)
    dest = ops.cache_dest_rows(rows_k, cu, v_starts, seq_ids, n_dev)
    dv1 = torch.zeros(cap, Hkv * D, dtype=torch.bfloat16, device=dev)
    ops.delta_v_update(v_new.view(cap, -1), v1, dest, dv1, n_dev)

    k2, v2 = k_cache.clone(), v_cache.clone()
    dv2 = torch.zeros(cap, Hkv, D, dtype=torch.bfloat16, device=dev)
    ops.kv_cache_update(k_new, v_new, rows_k, positions, pos_idx, cos_sin, cu, k_starts, v_starts, seq_ids, k2, v2,
                        n_dev, dv=dv2)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.equal(dv1.view(cap, Hkv, D)[:live], dv2[:live])
    assert bool((dv2[live:] == 0).all())


@pytest.mark.parametrize("live", [41, 64])
def test_delta_v_and_kv_cache_update_match_the_oracle(cuda_device, live):
    """dyllm_delta_v_update and dyllm_kv_cache_update against the CPU restatement of the reference's Python
    (layers/attention.py:67-74,89-96; models/llada.py:108-143): delta-V and both caches bit-exact, the
    rotated keys within the rotary embedding's rounding."""
    from oracle import dyllm_oracle as orc

    from dyllm_b200 import ops

    g = torch.Generator().manual_seed(11 + live)
    B, L, Hkv, D, cap = 3, 80, 2, 128, 64
    dev = cuda_device
    cu = (torch.arange(B + 1) * L).to(torch.int32)
    seq_ids = torch.tensor([1, 2, 0])
    k_starts = torch.tensor([2 * L + 4, 0, L])           # per sequence id
    v_starts = torch.tensor([0, L + 7, 2 * L + 7])
    k_cache = torch.randn(3 * L + 16, Hkv * D, generator=g).bfloat16()
    v_cache = torch.randn(3 * L + 16, Hkv * D, generator=g).bfloat16()
    rows_k = torch.sort(torch.randperm(B * L, generator=g)[:cap]).values
    positions = (torch.arange(B * L) % L)
    k_new = torch.randn(cap, Hkv, D, generator=g).bfloat16()
    v_new = torch.randn(cap, Hkv, D, generator=g).bfloat16()
    theta, max_pos = 500000.0, 256
    t = torch.arange(max_pos, dtype=torch.float)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float) / D))
    f = torch.einsum("i,j->ij", t, inv)
    cos_sin = torch.cat((f.cos(), f.sin()), dim=-1)
    n_dev = torch.tensor([live], dtype=torch.int32, device=dev)

    # oracle on the live rows
    b_of = torch.div(rows_k[:live], L, rounding_mode="floor")
    k_rows = k_starts[seq_ids[b_of]] + rows_k[:live] - b_of * L
    v_rows = v_starts[seq_ids[b_of]] + rows_k[:live] - b_of * L
    k_want, v_want = k_cache.clone(), v_cache.clone()
    dv_want = orc.kv_cache_update(k_new[:live], v_new[:live], rows_k[:live], positions[rows_k[:live]], k_want, v_want,
                                  k_rows, v_rows, D, theta, max_pos)

    d = lambda x: x.to(dev)
    k_got, v_got = d(k_cache.clone()), d(v_cache.clone())
    dv_got = torch.zeros(cap, Hkv, D, dtype=torch.bfloat16, device=dev)
    ops.kv_cache_update(d(k_new), d(v_new), d(rows_k), d(positions), d(rows_k), d(cos_sin), d(cu), d(k_starts),
                        d(v_starts), d(seq_ids), k_got, v_got, n_dev, dv=dv_got)
    assert torch.equal(dv_got[:live].cpu().flatten(1), dv_want)
    assert bool((dv_got[live:] == 0).all())
    assert torch.equal(v_got.cpu(), v_want)
    torch.testing.assert_close(k_got.cpu().float(), k_want.float(), rtol=8e-3, atol=1e-3)
    untouched = torch.ones(k_cache.size(0), dtype=torch.bool)
    untouched[k_rows] = False
    assert torch.equal(k_got.cpu()[untouched], k_cache[untouched])

    # the stand-alone delta-V entry point
    v_got2 = d(v_cache.clone())
    dv2 = ops.delta_v_update(d(v_new).view(cap, -1), v_got2, d(v_rows.to(torch.int32)) if live == cap else
                             d(torch.cat([v_rows, torch.zeros(cap - live, dtype=torch.long)]).to(torch.int32)), None, n_dev)
    assert torch.equal(dv2[:live].cpu(), dv_want) and torch.equal(v_got2.cpu(), v_want)
