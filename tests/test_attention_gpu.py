"""Parity of the tcgen05 approximate-attention kernel with the fp32 oracle.

bf16 outputs: max-abs <= 2e-2 (unit-scale outputs) and relative L2 <= 1e-2; salient decisions
bit-exact (the generators keep every cosine at least 1e-4 away from the threshold).
"""
import pytest
import torch

from oracle import dyllm_oracle as orc

pytestmark = pytest.mark.gpu

TAU = 0.99


def make_case(batch, prompt, response, H, Hkv, response_only, sal_per_seq, seed, ragged=False):
    """One sparse-step attention problem in the reference's calling convention."""
    D = 128
    g = torch.Generator().manual_seed(seed)
    if ragged:
        lens_k = [prompt + response - 17 * b for b in range(batch)]
    else:
        lens_k = [prompt + response] * batch
    lens_q = [response if response_only else lk for lk in lens_k]
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    Tq, Tk = int(cu_q[-1]), int(cu_k[-1])
    q = torch.randn(Tq, H, D, generator=g).bfloat16()
    k = torch.randn(Tk, Hkv, D, generator=g).bfloat16()
    c_old = torch.randn(Tq, H, D, generator=g).bfloat16()
    # salient rows: response positions of each sequence
    idx_q, idx_k, cu_sal = [], [], [0]
    for b in range(batch):
        n = sal_per_seq if isinstance(sal_per_seq, int) else sal_per_seq[b]
        resp0 = lens_k[b] - response
        pos = torch.sort(torch.randperm(response, generator=g)[:n]).values + resp0  # position inside the sequence
        idx_k += (pos + int(cu_k[b])).tolist()
        idx_q += ((pos - resp0 if response_only else pos) + int(cu_q[b])).tolist()
        cu_sal.append(cu_sal[-1] + n)
    idx_q = torch.tensor(idx_q, dtype=torch.int32)
    idx_k = torch.tensor(idx_k, dtype=torch.int32)
    cu_sal = torch.tensor(cu_sal, dtype=torch.int32)
    dv = torch.zeros(Tk, Hkv, D)
    dv[idx_k.long()] = torch.randn(idx_k.numel(), Hkv, D, generator=g) * 2.0
    dv = dv.bfloat16()
    o_sal = torch.randn(idx_q.numel(), H, D, generator=g).bfloat16()
    return dict(q=q, k=k, dv=dv, c_old=c_old, o_sal=o_sal, cu_q=cu_q, cu_k=cu_k, cu_sal=cu_sal, idx_q=idx_q,
                idx_k=idx_k, response_only=response_only, max_q=max(lens_q), max_k=max(lens_k))


def run_gpu(case, dev, v_mn_major):
    from dyllm_b200.attention_ops import attention_sparse_varlen

    d = lambda t: t.to(dev)
    Tq = case["q"].size(0)
    stats = torch.zeros(Tq, 3, device=dev)
    mask = torch.empty(Tq, dtype=torch.bool, device=dev)
    out = attention_sparse_varlen(d(case["q"]), d(case["k"]), d(case["dv"]), d(case["c_old"]), d(case["o_sal"]),
                                  d(case["cu_q"]), d(case["cu_k"]), case["max_q"], case["max_k"], Tq, d(case["cu_sal"]),
                                  d(case["idx_q"]), stats, mask, TAU, case["response_only"],
                                  d(case["idx_k"]) if case["response_only"] else None, v_layout=v_mn_major)
    from dyllm_b200 import _lib
    assert _lib.load().dyllm_device_status() == 0
    return out.cpu(), stats.cpu(), mask.cpu()


def check(case, got):
    out, stats, mask = got
    want_o, want_stats, want_mask = orc.attention_sparse_varlen(
        case["q"], case["k"], case["dv"], case["c_old"], case["o_sal"], case["cu_q"], case["cu_k"], case["cu_sal"],
        case["idx_q"], TAU)
    diff = (out.float() - want_o.float())
    scale = max(1.0, want_o.float().abs().max().item())
    assert diff.abs().max().item() / scale <= 2e-2
    assert (diff.norm() / want_o.float().norm()).item() <= 1e-2
    torch.testing.assert_close(stats, want_stats, rtol=2e-3, atol=2e-2)
    # decisions: bit-exact wherever the oracle's cosine is at least 1e-4 away from the threshold
    cosv = orc.cosine_values(want_stats)
    clear = (cosv - TAU).abs() >= 1e-4
    assert torch.equal(mask[clear], want_mask[clear])
    assert clear.float().mean() > 0.99


CASES = [
    # batch, prompt, response, H, Hkv, response_only, salient per sequence
    (1, 256, 256, 4, 4, False, 26),
    (1, 256, 256, 4, 4, True, 26),
    (2, 100, 156, 4, 2, False, 7),
    (3, 64, 64, 2, 1, True, 64),
    (2, 256, 256, 2, 2, False, 0),
    (2, 128, 256, 2, 2, True, 200),   # more than one salient tile
    (2, 300, 212, 4, 4, False, [1, 130]),
    (2, 256, 256, 4, 4, True, [16, 17]),   # either side of the early-gather limit
    (3, 200, 56, 4, 2, False, [15, 33, 48]),
    (1, 1700, 220, 2, 2, False, 5),     # 15 key tiles: the longest sequence of the few-rows kernel
    (1, 1800, 248, 2, 1, False, 9),     # 16 key tiles: few rows, but left to the general kernel
    (2, 100, 30, 2, 2, True, [16, 1]),  # ragged single key tile
    (2, 128, 128, 14, 2, False, [9, 30]),   # Dream heads under tensor parallelism 2 (7 query heads per KV head)
    (2, 128, 128, 7, 1, True, [20, 3]),     # ... and 4
]


@pytest.mark.parametrize("v_mn_major", [0, 1], ids=["vT", "vMN"])
@pytest.mark.parametrize("case_id", range(len(CASES)))
def test_attention_sparse_varlen_matches_oracle(cuda_device, case_id, v_mn_major):
    batch, prompt, response, H, Hkv, ro, sal = CASES[case_id]
    case = make_case(batch, prompt, response, H, Hkv, ro, sal, seed=case_id)
    check(case, run_gpu(case, cuda_device, v_mn_major))


@pytest.mark.parametrize("v_mn_major", [0, 1], ids=["vT", "vMN"])
def test_attention_ragged_lengths(cuda_device, v_mn_major):
    case = make_case(4, 200, 180, 4, 2, False, [3, 0, 50, 140], seed=42, ragged=True)
    check(case, run_gpu(case, cuda_device, v_mn_major))
    case = make_case(4, 200, 180, 4, 2, True, [3, 0, 50, 140], seed=43, ragged=True)
    check(case, run_gpu(case, cuda_device, v_mn_major))


def test_attention_config_shape_and_determinism(cuda_device):
    """LLaDA-8B layer shape (32 heads), batch 2; two runs give identical bits."""
    case = make_case(2, 256, 256, 32, 32, False, 26, seed=7)
    a = run_gpu(case, cuda_device, 1)
    b = run_gpu(case, cuda_device, 1)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    check(case, a)


def test_attention_delta_identity(cuda_device):
    """Size-independent property: with dV = 0 the output equals C_old exactly and every cosine is 1."""
    case = make_case(4, 256, 256, 8, 8, False, 0, seed=9)
    out, stats, mask = run_gpu(case, cuda_device, 1)
    assert torch.equal(out, case["c_old"])
    assert not bool(mask.any())


def test_attention_argument_errors(cuda_device):
    from dyllm_b200.attention_ops import attention_kernel_info, attention_sparse_varlen

    case = make_case(1, 64, 64, 2, 2, False, 4, seed=1)
    d = lambda t: t.to(cuda_device)
    Tq = case["q"].size(0)
    stats = torch.zeros(Tq, 3, device=cuda_device)
    mask = torch.empty(Tq, dtype=torch.bool, device=cuda_device)
    args = [d(case["q"]), d(case["k"]), d(case["dv"]), d(case["c_old"]), d(case["o_sal"]), d(case["cu_q"]),
            d(case["cu_k"]), case["max_q"], case["max_k"], Tq, d(case["cu_sal"]), d(case["idx_q"]), stats, mask, TAU]
    with pytest.raises(RuntimeError):
        attention_sparse_varlen(*args[:9], Tq + 1, *args[10:])  # total_seqlen mismatch
    bad = list(args)
    bad[11] = d(case["idx_q"]).long()
    with pytest.raises(RuntimeError):
        attention_sparse_varlen(*bad)  # idx must be int32
    bad = list(args)
    bad[0] = d(case["q"])[:, :, :64].contiguous()
    with pytest.raises(RuntimeError):
        attention_sparse_varlen(*bad)
    info = attention_kernel_info(128)
    assert len(info) == 10 and info[9] == 1 and info[0] > 0 and info[5] >= 1


@pytest.mark.parametrize("case_id", range(len(CASES)))
def test_attention_salient_rows_matches_exact_attention(cuda_device, case_id):
    """Replacement of the flash-attn call on q[idx_salient_row]."""
    from dyllm_b200 import _lib
    from dyllm_b200.attention_ops import attention_salient_rows

    batch, prompt, response, H, Hkv, ro, sal = CASES[case_id]
    case = make_case(batch, prompt, response, H, Hkv, ro, sal, seed=100 + case_id)
    g = torch.Generator().manual_seed(case_id)
    v = torch.randn(case["k"].shape, generator=g).bfloat16()
    d = lambda t: t.to(cuda_device)
    n = case["idx_q"].numel()
    out = torch.full((n + 3, H, 128), 7.0, dtype=torch.bfloat16, device=cuda_device)
    attention_salient_rows(d(case["q"]), d(case["k"]), d(v), d(case["cu_k"]), d(case["cu_sal"]), d(case["idx_q"]),
                           max_rows_per_seq=case["max_q"], num_salient=n, out=out)
    assert _lib.load().dyllm_device_status() == 0
    want = orc.exact_attention_varlen(case["q"][case["idx_q"].long()], case["k"], v, case["cu_sal"], case["cu_k"])
    got = out[:n].float().cpu()
    if n:
        diff = got - want
        assert diff.abs().max().item() <= 2e-2
        assert (diff.norm() / want.norm()).item() <= 1e-2
    assert bool((out[n:] == 7.0).all())


@pytest.mark.parametrize("case_id", [0, 1, 3, 5])
def test_attention_compact_delta_v_equals_padded(cuda_device, case_id):
    """The compact delta-V layout (no zero-padded tensor) gives bit-identical results."""
    from dyllm_b200.attention_ops import attention_sparse_varlen

    batch, prompt, response, H, Hkv, ro, sal = CASES[case_id]
    case = make_case(batch, prompt, response, H, Hkv, ro, sal, seed=50 + case_id)
    ref = run_gpu(case, cuda_device, 1)
    d = lambda t: t.to(cuda_device)
    Tq = case["q"].size(0)
    stats = torch.zeros(Tq, 3, device=cuda_device)
    mask = torch.empty(Tq, dtype=torch.bool, device=cuda_device)
    dv_compact = case["dv"][case["idx_k"].long()].contiguous()
    out = attention_sparse_varlen(d(case["q"]), d(case["k"]), d(dv_compact), d(case["c_old"]), d(case["o_sal"]),
                                  d(case["cu_q"]), d(case["cu_k"]), case["max_q"], case["max_k"], Tq, d(case["cu_sal"]),
                                  d(case["idx_q"]), stats, mask, TAU, ro, d(case["idx_k"]) if ro else None, v_layout=3)
    assert torch.equal(out.cpu(), ref[0]) and torch.equal(stats.cpu(), ref[1]) and torch.equal(mask.cpu(), ref[2])


def test_attention_no_salient_rows_with_empty_compact_delta_v(cuda_device):
    """A layer may publish an empty salient set; the next layer then passes empty lists and tensors."""
    from dyllm_b200.attention_ops import attention_sparse_varlen

    case = make_case(2, 128, 128, 2, 2, False, 0, seed=77)
    d = lambda t: t.to(cuda_device)
    Tq = case["q"].size(0)
    stats = torch.zeros(Tq, 3, device=cuda_device)
    mask = torch.ones(Tq, dtype=torch.bool, device=cuda_device)
    empty_dv = torch.empty(0, 2, 128, dtype=torch.bfloat16, device=cuda_device)
    out = attention_sparse_varlen(d(case["q"]), d(case["k"]), empty_dv, d(case["c_old"]), d(case["o_sal"]),
                                  d(case["cu_q"]), d(case["cu_k"]), case["max_q"], case["max_k"], Tq, d(case["cu_sal"]),
                                  d(case["idx_q"]), stats, mask, TAU, v_layout=3)
    assert torch.equal(out.cpu(), case["c_old"]) and not bool(mask.any())


@pytest.mark.parametrize("case_id", [1, 2, 3, 5])
def test_attention_cache_resident_context_equals_packed_path(cuda_device, case_id):
    """Reading the old context from the cache arena and writing the new one back in place gives the same
    bits as gather copy -> kernel -> write-back copy."""
    from dyllm_b200.attention_ops import attention_sparse_varlen

    batch, prompt, response, H, Hkv, ro, sal = CASES[case_id]
    case = make_case(batch, prompt, response, H, Hkv, ro, sal, seed=200 + case_id)
    ref_out, ref_stats, ref_mask = run_gpu(case, cuda_device, 1)
    # cache arena: sequences stored whole (len_k rows each) in reverse batch order, with a gap in front
    cu_q, cu_k = case["cu_q"], case["cu_k"]
    lens_k = (cu_k[1:] - cu_k[:-1]).tolist()
    lens_q = (cu_q[1:] - cu_q[:-1]).tolist()
    g = torch.Generator().manual_seed(1)
    total = sum(lens_k) + 9
    arena = torch.randn(total, H, 128, generator=g).bfloat16()
    seq_ids = torch.tensor([7 + 2 * b for b in range(batch)])
    seq_starts = torch.full((64,), -1, dtype=torch.int64)
    pos = 9
    for b in reversed(range(batch)):
        seq_starts[seq_ids[b]] = pos
        pos += lens_k[b]
    for b in range(batch):   # the old context of the query rows = the last len_q rows of each sequence
        s0 = int(seq_starts[seq_ids[b]]) + lens_k[b] - lens_q[b]
        arena[s0:s0 + lens_q[b]] = case["c_old"][int(cu_q[b]):int(cu_q[b + 1])]
    before = arena.clone()
    d = lambda t: t.to(cuda_device)
    Tq = case["q"].size(0)
    stats = torch.zeros(Tq, 3, device=cuda_device)
    mask = torch.empty(Tq, dtype=torch.bool, device=cuda_device)
    d_arena = d(arena)
    out = attention_sparse_varlen(d(case["q"]), d(case["k"]), d(case["dv"]), d_arena, d(case["o_sal"]), d(cu_q), d(cu_k),
                                  case["max_q"], case["max_k"], Tq, d(case["cu_sal"]), d(case["idx_q"]), stats, mask, TAU,
                                  ro, d(case["idx_k"]) if ro else None, v_layout=1,
                                  c_cache=(d(seq_starts), d(seq_ids), True))
    assert torch.equal(out.cpu(), ref_out) and torch.equal(stats.cpu(), ref_stats) and torch.equal(mask.cpu(), ref_mask)
    after = d_arena.cpu()
    touched = torch.zeros(total, dtype=torch.bool)
    for b in range(batch):
        s0 = int(seq_starts[seq_ids[b]]) + lens_k[b] - lens_q[b]
        assert torch.equal(after[s0:s0 + lens_q[b]], ref_out[int(cu_q[b]):int(cu_q[b + 1])])
        touched[s0:s0 + lens_q[b]] = True
    assert torch.equal(after[~touched], before[~touched])
    # key rows derived from the query rows (no K-space list) and statistics overwritten instead of added to:
    # same bits, with a statistics buffer that holds garbage on entry
    d_arena2 = d(arena)
    stats2 = torch.full((Tq, 3), 123.0, device=cuda_device)
    mask2 = torch.empty(Tq, dtype=torch.bool, device=cuda_device)
    out2 = attention_sparse_varlen(d(case["q"]), d(case["k"]), d(case["dv"]), d_arena2, d(case["o_sal"]), d(cu_q), d(cu_k),
                                   case["max_q"], case["max_k"], Tq, d(case["cu_sal"]), d(case["idx_q"]), stats2, mask2, TAU,
                                   ro, None, v_layout=1 | 4, c_cache=(d(seq_starts), d(seq_ids), True))
    assert torch.equal(out2.cpu(), ref_out) and torch.equal(stats2.cpu(), ref_stats) and torch.equal(mask2.cpu(), ref_mask)


@pytest.mark.parametrize("lens,H,Hkv", [([512] * 4, 4, 4), ([200, 75, 333], 4, 2), ([768] * 2, 14, 2), ([128], 2, 1)])
def test_dense_step_attention_on_the_exact_kernel(cuda_device, lens, H, Hkv):
    """Dense steps list every query row of the batch for the exact-attention kernel (flash-attn varlen call of
    dyllm/model_executor/layers/attention.py:39-52); both backends agree with the fp32 oracle."""
    from types import SimpleNamespace

    from dyllm_b200 import _lib, layers

    g = torch.Generator().manual_seed(sum(lens) + H)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    q, k, v = (torch.randn(T, h, 128, generator=g).bfloat16() for h in (H, Hkv, Hkv))
    want = orc.exact_attention_varlen(q, k, v, cu, cu)
    ctx = SimpleNamespace(cu_seqlens_q=cu.to(cuda_device), cu_seqlens_k=cu.to(cuda_device), max_seqlen_q=max(lens),
                          context_lens_cpu=lens)
    d = lambda t: t.to(cuda_device)
    try:
        for backend in ("tcgen05", "sdpa"):
            layers.set_dense_attention_backend(backend)
            got = layers._dense_attention(d(q), d(k), d(v), ctx, 128 ** -0.5).float().cpu()
            assert _lib.load().dyllm_device_status() == 0
            diff = got - want
            assert diff.abs().max().item() <= 2e-2, backend
            assert (diff.norm() / want.norm()).item() <= 1e-2, backend
    finally:
        layers.set_dense_attention_backend("sdpa")
