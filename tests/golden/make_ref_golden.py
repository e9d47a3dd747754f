"""Golden vectors produced by the REFERENCE's own CUDA kernels (and by flash-attn, the third-party
attention the reference calls), recorded on a B200.

Needs ``oracle/_ref/*.so`` (the reference's extension sources compiled for sm_100 by
``oracle/build_ref.py``) and a CUDA device:

    python tests/golden/make_ref_golden.py            # writes tests/golden/ref_kernels.pt
    python tests/golden/make_ref_golden.py --out DIR  # writes DIR/ref_kernels.pt (+ timing json)

What is recorded, per seeded case (inputs are regenerated from the seed by :func:`attention_case` /
:func:`cache_case`, which the tests import, so the fixture holds outputs only):

* ``attention_sparse_varlen`` of the reference (``dyllm/csrc/attention/attention.cpp:64-179``): O, the
  statistics after the call, the mask;
* ``flash_attn_varlen_func`` on the salient query rows as the reference calls it
  (``dyllm/model_executor/layers/attention.py:76-87``), when flash-attn runs on the device;
* the five ``dyllm.cache`` functions (``dyllm/csrc/cache/cache.cpp:3-25``) and ``fused_offset_launch``
  (``dyllm/csrc/attention/attention_aux_kernels.cu:173-200``).

With ``--time`` it also measures the reference attention kernel at the LLaDA-8B batch-16 shape
(the kernel this package's sm_100a attention is compared with) and writes ``ref_kernel_times.json``.
"""
import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

TAU = 0.99

# name -> (sequence lengths, response lengths, heads, kv heads, response-only queries, salient rows per sequence,
#          seed, query scale, delta-V scale).  The "strong" cases have peaked softmax rows and large value
# updates, so that the P.dV term moves the context by O(1) and the cosines spread around the threshold.
ATTENTION_CASES = {
    "c1_heads4_full": ([512], [256], 4, 4, False, [26], 11, 1.0, 0.7),
    "c1_heads4_pruned": ([512], [256], 4, 4, True, [26], 12, 1.0, 0.7),
    "ragged_gqa_pruned": ([200, 136, 77], [64, 40, 33], 4, 2, True, [5, 0, 3], 13, 1.0, 0.7),
    "ragged_gqa_full_dense_salient": ([192, 130], [96, 66], 4, 1, False, [40, 25], 14, 1.0, 0.7),
    "batch4_mha_full": ([128, 128, 128, 128], [64, 64, 64, 64], 2, 2, False, [1, 16, 0, 7], 15, 1.0, 0.7),
    "c1_heads4_full_strong": ([512], [256], 4, 4, False, [26], 16, 2.5, 6.0),
    "ragged_gqa_pruned_strong": ([200, 136, 77], [64, 40, 33], 4, 2, True, [9, 4, 3], 17, 2.5, 6.0),
    "ragged_gqa_full_strong": ([192, 130], [96, 66], 4, 1, False, [40, 25], 18, 2.0, 3.0),
}


def attention_case(name: str):
    """Seeded inputs of one attention case (CPU tensors; bf16 where the kernels take bf16)."""
    lens, resp, H, Hkv, pruned, n_sal, seed, q_scale, dv_scale = ATTENTION_CASES[name]
    g = torch.Generator().manual_seed(seed)
    D, B = 128, len(lens)
    lq = resp if pruned else lens
    cu_k = [0]
    cu_q = [0]
    cu_p = [0]
    for b in range(B):
        cu_k.append(cu_k[-1] + lens[b])
        cu_q.append(cu_q[-1] + lq[b])
        cu_p.append(cu_p[-1] + lens[b] - resp[b])
    Tk, Tq = cu_k[-1], cu_q[-1]
    idx_q, idx_k, cu_sal = [], [], [0]
    for b in range(B):
        pos = torch.sort(torch.randperm(resp[b], generator=g)[: n_sal[b]]).values + (lens[b] - resp[b])
        for p in pos.tolist():
            idx_k.append(p + cu_k[b])
            idx_q.append((p - (lens[b] - resp[b]) if pruned else p) + cu_q[b])
        cu_sal.append(len(idx_q))
    S = len(idx_q)
    bf = lambda t: t.to(torch.bfloat16)
    q = bf(q_scale * torch.randn(Tq, H, D, generator=g))
    k = bf(torch.randn(Tk, Hkv, D, generator=g))
    v_cache = bf(torch.randn(Tk, Hkv, D, generator=g))
    c_old = bf(torch.randn(Tq, H, D, generator=g))
    dv = torch.zeros(Tk, Hkv, D)
    if S:
        dv[torch.tensor(idx_k)] = dv_scale * torch.randn(S, Hkv, D, generator=g)
    dv = bf(dv)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return dict(q=q, k=k, v_cache=v_cache, dv=dv, c_old=c_old, cu_q=i32(cu_q), cu_k=i32(cu_k), cu_p=i32(cu_p),
                cu_sal=i32(cu_sal), idx_q=i32(idx_q), idx_k=i32(idx_k), pruned=pruned, max_q=max(lq), max_k=max(lens),
                H=H, Hkv=Hkv, tau=TAU)


CACHE_SHAPE = dict(width=64, max_seqs=8, seq_ids=[5, 2, 7], lens=[37, 64, 18], block=[16, 32, 5], seed=21)


def cache_case():
    """Seeded inputs of the cache / offset cases."""
    c = CACHE_SHAPE
    g = torch.Generator().manual_seed(c["seed"])
    width, lens, blk = c["width"], c["lens"], c["block"]
    total_rows = sum(lens) + 40
    cache = torch.randn(total_rows, width, generator=g).to(torch.bfloat16)
    seq_starts = torch.zeros(c["max_seqs"], dtype=torch.int64)
    # sequences stored out of batch order with gaps between them
    seq_starts[5], seq_starts[2], seq_starts[7] = 70, 3, 110
    cu = torch.tensor([0, lens[0], lens[0] + lens[1], sum(lens)], dtype=torch.int32)
    cu_q = torch.tensor([0, blk[0], blk[0] + blk[1], sum(blk)], dtype=torch.int32)
    seq_ids = torch.tensor(c["seq_ids"], dtype=torch.int64)
    new_full = torch.randn(sum(lens), width, generator=g).to(torch.bfloat16)
    new_block = torch.randn(sum(blk), width, generator=g).to(torch.bfloat16)
    rows = torch.sort(torch.randperm(sum(lens), generator=g)[:23]).values.to(torch.int64)
    new_rows = torch.randn(23, width, generator=g).to(torch.bfloat16)
    # fused_offset: response-space indices of three groups, prompt lengths 21 / 32 / 13
    idxs = torch.tensor([0, 3, 9, 16, 17, 40, 47], dtype=torch.int32)
    cu_sal = torch.tensor([0, 3, 5, 7], dtype=torch.int32)
    cu_prompt = torch.tensor([0, 21, 53, 66], dtype=torch.int32)
    return dict(cache=cache, seq_starts=seq_starts, cu=cu, cu_q=cu_q, seq_ids=seq_ids, new_full=new_full,
                new_block=new_block, rows=rows, new_rows=new_rows, idxs=idxs, cu_sal=cu_sal, cu_prompt=cu_prompt,
                total=sum(lens), total_q=sum(blk))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    from oracle.build_ref import load_ref

    dev = torch.device("cuda:0")
    ops = load_ref("dyllm_ref_attention_ops")
    cache_mod = load_ref("dyllm_ref_cache")
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception as e:  # flash-attn is third party; without it the salient rows come from fp32 softmax attention
        flash_attn_varlen_func = None
        print("flash_attn unavailable:", e)
    record = {"attention": {}, "tau": TAU, "device": torch.cuda.get_device_name(0), "torch": str(torch.__version__),
              "kernel_info_d128": list(ops.attention_kernel_info(128, False))}

    for name in ATTENTION_CASES:
        c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in attention_case(name).items()}
        S = c["idx_q"].numel()
        rec = {}
        # exact attention of the salient rows as the reference calls flash-attn (attention.py:76-87)
        v_now = c["v_cache"].clone()          # the value cache after the update: old + dV on the salient rows
        if S:
            ik = c["idx_k"].long()
            v_now[ik] = (c["v_cache"][ik].float() + c["dv"][ik].float()).to(torch.bfloat16)
        o_sal = None
        if flash_attn_varlen_func is not None and S:
            try:
                max_sal = int((c["cu_sal"][1:] - c["cu_sal"][:-1]).max())
                o_sal = flash_attn_varlen_func(c["q"][c["idx_q"].long()], c["k"], v_now, cu_seqlens_q=c["cu_sal"],
                                               cu_seqlens_k=c["cu_k"], max_seqlen_q=max_sal, max_seqlen_k=c["max_k"],
                                               dropout_p=0.0, softmax_scale=1.0 / math.sqrt(128), causal=False)
                torch.cuda.synchronize()
                rec["flash_o_sal"] = o_sal.cpu()
            except Exception as e:
                print(name, "flash_attn failed:", repr(e)[:200])
                o_sal = None
        if o_sal is None:
            from oracle import dyllm_oracle as orc

            o_sal = orc.exact_attention_varlen(c["q"][c["idx_q"].long()].cpu(), c["k"].cpu(), v_now.cpu(), c["cu_sal"].cpu(),
                                               c["cu_k"].cpu()).to(torch.bfloat16).to(dev)
            if S == 0:
                o_sal = torch.empty((0, c["H"], 128), dtype=torch.bfloat16, device=dev)
        rec["o_sal_used"] = o_sal.cpu()
        stats = torch.zeros((c["q"].size(0), 3), dtype=torch.float32, device=dev)
        mask = torch.empty((c["q"].size(0),), dtype=torch.bool, device=dev)
        O = ops.attention_sparse_varlen(c["q"], c["k"], c["dv"], c["c_old"], o_sal.contiguous(), c["cu_q"], c["cu_k"],
                                        c["max_q"], c["max_k"], c["q"].size(0), c["cu_sal"], c["idx_q"], stats, mask,
                                        c["tau"], c["pruned"], c["idx_k"] if c["pruned"] else torch.Tensor(), -1)
        torch.cuda.synchronize()
        rec.update(O=O.cpu(), stats=stats.cpu(), mask=mask.cpu())
        # the other load strategy of the kernel (force_mask_v_rows) must give the same result
        stats2 = torch.zeros_like(stats)
        mask2 = torch.empty_like(mask)
        O2 = ops.attention_sparse_varlen(c["q"], c["k"], c["dv"], c["c_old"], o_sal.contiguous(), c["cu_q"], c["cu_k"],
                                         c["max_q"], c["max_k"], c["q"].size(0), c["cu_sal"], c["idx_q"], stats2, mask2,
                                         c["tau"], c["pruned"], c["idx_k"] if c["pruned"] else torch.Tensor(), 0)
        torch.cuda.synchronize()
        rec["O_equal_across_load_modes"] = bool(torch.equal(O, O2))
        record["attention"][name] = rec
        print(name, "rows", c["q"].size(0), "salient", S, "mask true", int(mask.sum()), "modes equal",
              rec["O_equal_across_load_modes"])

    cc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in cache_case().items()}
    crec = {}
    crec["get_seqs"] = cache_mod.get_seqs_cuda(cc["cache"], cc["seq_starts"], cc["cu"], cc["seq_ids"], cc["total"]).cpu()
    crec["get_block"] = cache_mod.get_block_cuda(cc["cache"], cc["seq_starts"], cc["cu"], cc["cu_q"], cc["seq_ids"],
                                                 cc["total_q"]).cpu()
    c1 = cc["cache"].clone()
    cache_mod.reset_full_cuda(c1, cc["new_full"], cc["seq_starts"], cc["cu"], cc["seq_ids"], cc["total"])
    crec["reset_full"] = c1.cpu()
    c2 = cc["cache"].clone()
    cache_mod.reset_block_cuda(c2, cc["new_block"], cc["seq_starts"], cc["cu"], cc["cu_q"], cc["seq_ids"], cc["total_q"])
    crec["reset_block"] = c2.cpu()
    c3 = cc["cache"].clone()
    cache_mod.scatter_update_cuda(c3, cc["new_rows"], cc["rows"], cc["cu"], cc["seq_starts"], cc["seq_ids"])
    crec["scatter_update"] = c3.cpu()
    out = torch.full((16,), -1, dtype=torch.int64, device=dev)
    n = torch.tensor([cc["idxs"].numel()], dtype=torch.int32, device=dev)
    ops.fused_offset_launch(cc["idxs"], n, cc["cu_prompt"], cc["cu_sal"], out, 16)
    torch.cuda.synchronize()
    crec["fused_offset"] = out.cpu()
    record["cache"] = crec
    print("cache cases recorded; fused_offset ->", out.tolist())

    os.makedirs(args.out, exist_ok=True)
    path = os.path.join(args.out, "ref_kernels.pt")
    torch.save(record, path)
    print("wrote", path, os.path.getsize(path), "bytes")

    if args.time:
        times = {}
        for label, pruned in (("full_sequence_queries", False), ("response_only_queries", True)):
            B, L, R, H = 16, 512, 256, 32
            lq = R if pruned else L
            g = torch.Generator(device=dev).manual_seed(3)
            q = torch.randn(B * lq, H, 128, generator=g, device=dev).bfloat16()
            k = torch.randn(B * L, H, 128, generator=g, device=dev).bfloat16()
            c_old = torch.randn(B * lq, H, 128, generator=g, device=dev).bfloat16()
            n_sal = 3
            idx_k = torch.cat([torch.arange(n_sal) * 37 + b * L + (L - R) for b in range(B)]).to(torch.int32).to(dev)
            idx_q = torch.cat([torch.arange(n_sal) * 37 + b * lq + (0 if pruned else L - R) for b in range(B)]).to(torch.int32).to(dev)
            dv = torch.zeros(B * L, H, 128, device=dev, dtype=torch.bfloat16)
            dv[idx_k.long()] = 0.5
            o_sal = torch.randn(B * n_sal, H, 128, generator=g, device=dev).bfloat16()
            ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
            cu_q, cu_k, cu_sal = ar * lq, ar * L, ar * n_sal
            mask = torch.empty((B * lq,), dtype=torch.bool, device=dev)
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

            def run():
                stats = torch.zeros((B * lq, 3), dtype=torch.float32, device=dev)
                return ops.attention_sparse_varlen(q, k, dv, c_old, o_sal, cu_q, cu_k, lq, L, B * lq, cu_sal, idx_q, stats,
                                                   mask, TAU, pruned, idx_k if pruned else torch.Tensor(), -1)

            for _ in range(3):
                run()
            ms = []
            for _ in range(10):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run()
                e1.record()
                torch.cuda.synchronize()
                ms.append(e0.elapsed_time(e1))
            ms.sort()
            times[label] = {"median_ms": ms[len(ms) // 2], "min_ms": ms[0], "shape": f"B{B} L{L} R{R} H{H} D128, {n_sal} salient rows per sequence",
                            "what": "reference attention_sparse_varlen call (mask kernel + mma.sync main kernel + overwrite + "
                                    "cosine mask + stats zero-fill), L2 flushed before each call"}
            print(label, times[label])
        with open(os.path.join(args.out, "ref_kernel_times.json"), "w") as fh:
            json.dump(times, fh, indent=1)


if __name__ == "__main__":
    main()
