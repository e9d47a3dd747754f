"""Per-kernel timing of the saliency path at the LLaDA-8B layer shape (batch 16, 512 tokens per sequence).

    python -m dyllm_b200.microbench [--kernel NAME ...] [--rows S] [--iters N] [--no-flush]

Each kernel is warmed up, then timed launch by launch with CUDA events on the current stream; L2 is
flushed between launches by writing a 256 MiB buffer.  The report gives the median launch time and the
achieved fraction of the roofline that bounds the kernel (HBM GB/s from algorithmic bytes, or bf16
TFLOP/s), against MEASURED_PEAKS.json at the repository root when present.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import ops
from .attention_ops import attention_salient_rows, attention_sparse_varlen

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B, P, R, H, D, HID, INTER = 16, 256, 256, 32, 128, 4096, 12288
L = P + R


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_launches(fn, iters, flush):
    dev = torch.device("cuda")
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def time_back_to_back(fns, iters):
    """Average duration of one launch when the launches follow one another without host gaps, each on its own
    set of buffers (the sets together are several times the L2 size, so no launch finds its inputs cached): what
    a kernel costs inside a captured step, without the ~5 us of launch latency and event overhead that an
    isolated launch between two events carries.  The sequence is captured into a CUDA graph and the replay timed."""
    for fn in fns:
        fn()
    torch.cuda.synchronize()
    reps = 4
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            for fn in fns:
                fn()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(max(3, iters // 4)):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / (reps * len(fns)))
    return statistics.median(times)


def timed(make, args, sets=4):
    """``make(i)`` builds launch closure number i on fresh buffers.  Isolated launches with L2 flushes by
    default; ``--back-to-back`` rotates over ``sets`` buffer sets instead."""
    if args.back_to_back:
        return time_back_to_back([make(i) for i in range(sets)], args.iters)
    return time_launches(make(0), args.iters, args.flush)


def salient_lists(rows_total, dev, response_only=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    per = max(1, rows_total // B)
    lq = R if response_only else L
    idx_q, idx_k = [], []
    for b in range(B):
        pos = torch.sort(torch.randperm(R, generator=g)[:per]).values + P
        idx_k.append(pos + b * L)
        idx_q.append((pos - P if response_only else pos) + b * lq)
    cu_sal = (torch.arange(B + 1) * per).to(torch.int32)
    return torch.cat(idx_q).to(dev), torch.cat(idx_k).to(dev), cu_sal.to(dev), per


def bench_stats(args):
    dev = torch.device("cuda")
    rows = B * L

    def make(i):
        a = torch.randn(rows, H * D, device=dev).bfloat16()
        b = torch.randn(rows, H * D, device=dev).bfloat16()
        out = torch.empty(rows, 3, device=dev)
        return lambda: ops.context_stats(a, b, out=out)

    ms = timed(make, args)
    return ms, rows * (2 * H * D * 2 + 12), "B"


def bench_select(args):
    dev = torch.device("cuda")
    rows = args.select_rows
    cu = torch.arange(0, rows + 1, L, dtype=torch.int32, device=dev)
    picked = []

    def make(i):
        stats = torch.ones(rows, 3, device=dev)
        stats[:, 0] = torch.where(torch.rand(rows, device=dev) < 0.1, 0.5, 0.999)
        picked.append(int((stats[:, 0] < 0.9).sum()))
        return lambda: ops.salient_select(stats, 0.99, cu, want_mask=True)

    ms = timed(make, args, sets=3)
    return ms, 12 * rows + 12 * picked[0] + rows + 4 * cu.numel(), "B"   # statistics in; lists, mask, prefix counts out


def bench_scatter(args):
    from . import cache as C

    dev = torch.device("cuda")
    rows = B * L
    cache = torch.randn(rows, HID, device=dev).bfloat16()
    idx_q, _, _, _ = salient_lists(args.rows, dev)
    new = torch.randn(idx_q.numel(), HID, device=dev).bfloat16()
    cu = torch.arange(0, rows + 1, L, dtype=torch.int32, device=dev)
    ss = torch.arange(B, device=dev) * L
    ids = torch.arange(B, device=dev)
    ms = time_launches(lambda: C.scatter_update_cuda(cache, new, idx_q, cu, ss, ids), args.iters, args.flush)
    return ms, idx_q.numel() * (2 * HID * 2 + 8), "B"


def bench_get_seqs(args):
    from . import cache as C

    dev = torch.device("cuda")
    rows = B * L
    cu = torch.arange(0, rows + 1, L, dtype=torch.int32, device=dev)
    ss = torch.arange(B, device=dev) * L
    ids = torch.arange(B, device=dev)

    def make(i):
        cache = torch.randn(rows, HID, device=dev).bfloat16()
        return lambda: C.get_seqs_cuda(cache, ss, cu, ids, rows)

    ms = timed(make, args)
    return ms, rows * 2 * HID * 2, "B"


def bench_ffn(args):
    """SwiGLU FFN on ``--rows`` gathered rows; ``--inter`` sets the intermediate size (12288 / 8 = 1536 is the
    weight shard of one of eight tensor-parallel ranks).  More than 4096 rows: a random sorted row list over a
    larger activation (the at-scale workload's batch 64 x 512 response rows)."""
    dev = torch.device("cuda")
    inter = args.inter or INTER
    if args.rows <= B * R:
        x = torch.randn(B * L, HID, device=dev).bfloat16()
        idx_q, _, _, _ = salient_lists(args.rows, dev)
        idx32 = idx_q.to(torch.int32)
    else:
        x = torch.randn(64 * 1024, HID, device=dev).bfloat16()
        g = torch.Generator().manual_seed(0)
        idx32 = torch.sort(torch.randperm(x.size(0), generator=g)[: args.rows]).values.to(torch.int32).to(dev)
    w1 = (torch.randn(2 * inter, HID, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(HID, inter, device=dev) * 0.02).bfloat16()
    out = torch.empty(idx32.numel(), HID, device=dev, dtype=torch.bfloat16)
    ms = time_launches(lambda: ops.swiglu_ffn(x, w1, w2, idx32, out=out, a_mode=args.a_mode, tile_n=args.tile_n),
                       args.iters, args.flush)
    s = idx32.numel()
    flops = 6.0 * s * HID * inter
    wbytes = 3.0 * HID * inter * 2 + s * HID * 2 * 2 + 2.0 * s * inter * 2
    # the bound is whichever roofline gives the longer time
    hbm, tf, _ = peaks()
    if flops / (tf * 1e12) >= wbytes / (hbm * 1e9):
        return ms, flops, "F"
    return ms, wbytes, "B"


def bench_ffn_graph(args):
    """The FFN as the bench runs it: captured into a CUDA graph (no host launch gaps), eight layers' worth of
    distinct weights in one graph so that every launch streams its 302 MB of weights from HBM; rows arrive packed
    (the post-attention norm writes them in list order) and the live count sits on the device."""
    dev = torch.device("cuda")
    n_layers = 8
    s = args.rows
    cap = B * L
    x = torch.randn(cap, HID, device=dev).bfloat16()
    ws = [((torch.randn(2 * INTER, HID, device=dev) * 0.02).bfloat16(), (torch.randn(HID, INTER, device=dev) * 0.02).bfloat16())
          for _ in range(n_layers)]
    cache = torch.zeros(cap, HID, device=dev, dtype=torch.bfloat16)
    dest = torch.arange(cap, device=dev, dtype=torch.int32)
    count = torch.tensor([s], dtype=torch.int32, device=dev)

    def run_all():
        for w1, w2 in ws:
            ops.swiglu_ffn(x, w1, w2, None, num_rows=cap, num_rows_dev=count, rows_hint=min(128, cap), out=cache,
                           out_row_map=dest)

    run_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all()
    ms = time_launches(graph.replay, args.iters, False) / n_layers
    flops = 6.0 * s * HID * INTER
    wbytes = 3.0 * HID * INTER * 2 + s * HID * 2 * 2
    hbm, tf, _ = peaks()
    if flops / (tf * 1e12) >= wbytes / (hbm * 1e9):
        return ms, flops, "F"
    return ms, wbytes, "B"


def bench_norm(args):
    dev = torch.device("cuda")
    rows = B * L
    w = torch.ones(HID, device=dev).bfloat16()

    def make(i):
        x = torch.randn(rows, HID, device=dev).bfloat16()
        r = torch.randn(rows, HID, device=dev).bfloat16()
        return lambda: ops.add_rms_norm(x, w, 1e-5, r)

    ms = timed(make, args)
    return ms, 4.0 * rows * HID * 2, "B"


def bench_norm_rows(args):
    dev = torch.device("cuda")
    rows = B * L
    w = torch.ones(HID, device=dev).bfloat16()
    idx_q, _, _, _ = salient_lists(args.rows, dev)
    idx = torch.zeros(rows, dtype=torch.int32, device=dev)
    idx[: idx_q.numel()] = idx_q.to(torch.int32)
    count = torch.tensor([idx_q.numel()], dtype=torch.int32, device=dev)

    def make(i):
        x = torch.randn(rows, HID, device=dev).bfloat16()
        r = torch.randn(rows, HID, device=dev).bfloat16()
        return lambda: ops.add_rms_norm_rows(x, w, 1e-5, r, idx, count)

    ms = timed(make, args)
    return ms, 3.0 * rows * HID * 2 + 3.0 * idx_q.numel() * HID * 2, "B"


def bench_rope(args):
    dev = torch.device("cuda")
    rows = B * L
    pos = torch.arange(L, device=dev).repeat(B)
    t = torch.arange(4096, dtype=torch.float)
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, dtype=torch.float) / D))
    f = torch.einsum("i,j->ij", t, inv)
    cos_sin = torch.cat((f.cos(), f.sin()), dim=-1).to(dev)

    def make(i):
        x = torch.randn(rows, H, D, device=dev).bfloat16()
        return lambda: ops.rope_neox_(x, pos, cos_sin)

    ms = timed(make, args)
    return ms, 2.0 * rows * H * D * 2, "B"


def bench_kv_proj(args):
    dev = torch.device("cuda")
    x = torch.randn(B * L, HID, device=dev).bfloat16()
    w = (torch.randn(2 * H * D, HID, device=dev) * 0.02).bfloat16()
    idx_q, _, _, _ = salient_lists(args.rows, dev)
    idx32 = idx_q.to(torch.int32)
    out = torch.empty(idx32.numel(), 2 * H * D, device=dev, dtype=torch.bfloat16)
    ms = time_launches(lambda: ops.gathered_linear(x, w, idx32, out=out, a_mode=args.a_mode, tile_n=args.tile_n),
                       args.iters, args.flush)
    s = idx32.numel()
    return ms, 2.0 * HID * 2 * H * D + s * HID * 2 + s * 2 * H * D * 2, "B"


def _attention_inputs(args, response_only):
    dev = torch.device("cuda")
    lq = R if response_only else L
    q = torch.randn(B * lq, H, D, device=dev).bfloat16()
    k = torch.randn(B * L, H, D, device=dev).bfloat16()
    c = torch.randn(B * lq, H, D, device=dev).bfloat16()
    idx_q, idx_k, cu_sal, per = salient_lists(args.rows, dev, response_only)
    dv = torch.randn(idx_q.numel(), H, D, device=dev).bfloat16()
    o_sal = torch.randn(idx_q.numel(), H, D, device=dev).bfloat16()
    cu_q = torch.arange(0, B * lq + 1, lq, dtype=torch.int32, device=dev)
    cu_k = torch.arange(0, B * L + 1, L, dtype=torch.int32, device=dev)
    return q, k, c, dv, o_sal, cu_q, cu_k, cu_sal, idx_q.to(torch.int32), idx_k.to(torch.int32), per, lq


def bench_attention(args):
    q, k, c, dv, o_sal, cu_q, cu_k, cu_sal, iq, ik, per, lq = _attention_inputs(args, args.response_only)
    tq = q.size(0)
    stats = torch.zeros(tq, 3, device=q.device)
    mask = torch.empty(tq, dtype=torch.bool, device=q.device)

    def fn():
        stats.zero_()
        attention_sparse_varlen(q, k, dv, c, o_sal, cu_q, cu_k, lq, L, tq, cu_sal, iq, stats, mask, 0.99,
                                args.response_only, ik if args.response_only else None, v_layout=3)

    ms = time_launches(fn, args.iters, args.flush)
    return ms, 2.0 * tq * L * H * D + 4.0 * tq * per * H * D, "F"


def bench_salient_attention(args):
    q, k, c, dv, o_sal, cu_q, cu_k, cu_sal, iq, ik, per, lq = _attention_inputs(args, False)
    v = torch.randn_like(k)
    ms = time_launches(lambda: attention_salient_rows(q, k, v, cu_k, cu_sal, iq, max_rows_per_seq=per, out=o_sal),
                       args.iters, args.flush)
    return ms, 2.0 * k.numel() * 2 + 2.0 * iq.numel() * H * D * 2, "B"


def _bench_projection(args, backend):
    """q / o projection of every row of the batch (8192 x 4096 x 4096): cuBLAS or this package's tcgen05 GEMM."""
    from . import layers

    dev = torch.device("cuda")
    x = torch.randn(B * L, HID, device=dev).bfloat16()
    w = (torch.randn(HID, HID, device=dev) * 0.02).bfloat16()
    layers.set_projection_backend(backend)
    try:
        ms = time_launches(lambda: layers._project(x, w, None), args.iters, args.flush)
    finally:
        layers.set_projection_backend("cublas")
    return ms, 2.0 * B * L * HID * HID, "F"


def bench_proj_cublas(args):
    return _bench_projection(args, "cublas")


def bench_proj_own(args):
    return _bench_projection(args, "tcgen05")


def _bench_dense_attention(args, backend):
    """Attention of a dense step (every row a query) on the exact-attention kernel or torch's SDPA."""
    from types import SimpleNamespace

    from . import layers

    dev = torch.device("cuda")
    q, k, v = (torch.randn(B * L, H, D, device=dev).bfloat16() for _ in range(3))
    cu = torch.arange(0, B * L + 1, L, dtype=torch.int32, device=dev)
    ctx = SimpleNamespace(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=L, context_lens_cpu=[L] * B)
    layers.set_dense_attention_backend(backend)
    try:
        ms = time_launches(lambda: layers._dense_attention(q, k, v, ctx, D ** -0.5), args.iters, args.flush)
    finally:
        layers.set_dense_attention_backend("sdpa")
    return ms, 4.0 * B * L * L * H * D, "F"


def bench_dense_attention_own(args):
    return _bench_dense_attention(args, "tcgen05")


def bench_dense_attention_sdpa(args):
    return _bench_dense_attention(args, "sdpa")


def bench_steps(args):
    """One refresh period of sparse denoising steps (3 response-only + 1 full-sequence) of the 32-layer
    LLaDA-8B shape at batch 16, launched eagerly after one dense step: the launch sequence of the
    steady state of a generation, short enough to list launch by launch under a profiler."""
    from . import runner
    from .model import LLaDAForDLM, LLaDAShape, init_weights_

    dev = torch.device("cuda")
    shape = LLaDAShape(num_hidden_layers=args.layers)
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = LLaDAForDLM(shape, 0.99)
    finally:
        torch.set_default_dtype(torch.float32)
    init_weights_(model, seed=0)
    model.eval()
    sr = runner.StepRunner(model, shape.mask_token_id, 32, 256, num_full_steps=1, refresh_period=4, use_graphs=False)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, shape.vocab_size - 1024, (B, P), generator=g).tolist()
    seqs = sr.new_batch(prompts, R)
    sr.step(seqs)                         # dense step: fills the caches
    for seq in seqs:                      # continue in the steady state of the refresh schedule
        seq.processed_steps = 5
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(4):
        sr.step(seqs)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / 4, 4.0 * B * (R // 256) , "S"


KERNELS = {"stats": bench_stats, "select": bench_select, "scatter": bench_scatter, "get_seqs": bench_get_seqs,
           "ffn": bench_ffn, "ffn_graph": bench_ffn_graph, "kv_proj": bench_kv_proj, "norm": bench_norm,
           "norm_rows": bench_norm_rows, "rope": bench_rope, "attention": bench_attention,
           "salient_attention": bench_salient_attention, "proj_cublas": bench_proj_cublas, "proj_own": bench_proj_own,
           "dense_attention_own": bench_dense_attention_own, "dense_attention_sdpa": bench_dense_attention_sdpa,
           "steps": bench_steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", nargs="*", default=[k for k in KERNELS if k != "steps"])
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the `steps` case")
    ap.add_argument("--rows", type=int, default=416, help="salient rows in the batch (multiple of 16)")
    ap.add_argument("--select-rows", type=int, default=8 << 20)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", dest="flush", action="store_false")
    ap.add_argument("--back-to-back", action="store_true",
                    help="HBM helper kernels: launches back to back over rotating buffer sets (several times the L2 "
                         "size in all) instead of isolated launches with L2 flushes")
    ap.add_argument("--a-mode", type=int, default=-1)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--inter", type=int, default=0, help="ffn: intermediate size (default 12288)")
    ap.add_argument("--response-only", action="store_true")
    args = ap.parse_args()
    hbm, tf, src = peaks()
    for name in args.kernel:
        ms, work, kind = KERNELS[name](args)
        if kind == "S":
            print(json.dumps({"kernel": name, "ms_per_denoising_step": round(ms, 3), "layers": args.layers}), flush=True)
            continue
        if kind == "B":
            ach, peak, unit = work / ms / 1e6, hbm, "GB/s"
        else:
            ach, peak, unit = work / ms / 1e9, tf, "TFLOP/s"
        print(json.dumps({"kernel": name, "salient_rows": args.rows, "median_ms": round(ms, 4), "achieved": round(ach, 1),
                          "unit": unit, "peak": peak, "frac": round(ach / peak, 3), "peak_source": src,
                          "timing": "back to back in a CUDA graph, rotating buffers" if args.back_to_back else "isolated launches, L2 flushed"}),
              flush=True)


if __name__ == "__main__":
    main()
