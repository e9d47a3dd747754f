#!/usr/bin/env python
"""Throughput of the saliency path: generated tokens/s of complete generations (dense warm-up steps, then
sparse steps with the reference's period-4 full-sequence refresh), random-init bf16 weights and
uniform-random prompt ids (synthetic stand-ins for a checkpoint and a dataset).

    python bench.py --gpus N --steps K --warmup W            this library (one process per GPU, TP over NVLink)
    python bench.py --impl reference ...                      CPU restatement of the reference path on the host cores
    python bench.py --config {1,3,4,5} [--tau T | --dense] [--ep]   the other named workloads

--config 1 (default): LLaDA-8B shape, batch 16, prompt 256, gen 256, block 32, 256 denoising steps, tau 0.99.
--config 3: Dream-7B shape (28 query / 4 KV heads, biased q/k/v), batch 32; tensor parallel 2 or 4.
--config 4: LLaDA-MoE-7B-A1B shape (64 experts, top-8), batch 32; --ep = whole experts per rank.
--config 5: LLaDA-8B shape, batch 64, prompt 512, gen 512, block 64; sweep --tau 0.95 / 0.99 / 0.995 and --dense.

One "step" is one complete generation of the batch, so tokens/s = steps * batch * gen_len / time.
Prints one JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REFRESH = 4
CONFIGS = {
    1: dict(family="llada", batch=16, prompt=256, gen=256, block=32, steps=256, full=8, tau=0.99,
            label="configs[1]: LLaDA-8B shape, 32 layers"),
    3: dict(family="dream", batch=32, prompt=256, gen=256, block=32, steps=256, full=8, tau=0.99,
            label="configs[2]: Dream-7B shape, 28 layers, 28 query / 4 KV heads, qkv bias"),
    4: dict(family="lladamoe", batch=32, prompt=256, gen=256, block=32, steps=256, full=8, tau=0.99,
            label="configs[3]: LLaDA-MoE-7B-A1B shape, 16 layers, 64 experts top-8"),
    5: dict(family="llada", batch=64, prompt=512, gen=512, block=64, steps=512, full=8, tau=0.99,
            label="configs[4]: LLaDA-8B shape, 32 layers, at scale"),
}
MODEL_NAMES = {"llada": "LLaDA-8B", "dream": "Dream-7B", "lladamoe": "LLaDA-MoE-7B-A1B"}


def metric_name(cfg, tau):
    mode = "dense" if tau is None else f"tau={tau:g}"
    return f"generated tokens/s ({MODEL_NAMES[cfg['family']]} bf16, b={cfg['batch']}, gen={cfg['gen']}, {mode})"


def ncu_traffic_bytes():
    """DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of this library's kernels at the
    default workload's shapes, read from the table of profiles/ncu_dram_traffic.md (one ncu capture each)."""
    out = {}
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.md")
    if os.path.exists(path):
        for line in open(path):
            m = re.match(r"\|\s*`?(\w+)`?\s*\|\s*([0-9.]+)\s*MB\s*\|", line)
            if m:
                out[m.group(1)] = float(m.group(2)) * 1e6
    return out


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------
# clocks sampled during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            sm.sort()
            out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


# ----------------------------------------------------------------------------------------------
# CPU restatement of the path (checker code, timed as the reported CPU baseline)
# ----------------------------------------------------------------------------------------------
def layer_shape(cfg):
    """(hidden, heads, kv heads, FFN intermediate, layers, experts, top-k) of a workload's model."""
    if cfg["family"] == "dream":
        return 3584, 28, 4, 18944, 28, 0, 0
    if cfg["family"] == "lladamoe":
        return 2048, 16, 16, 1024, 16, 64, 8
    return 4096, 32, 32, 12288, 32, 0, 0


def cpu_layer_step_seconds(cfg, kind: str, n_seqs: int, sal_per_seq: int, repeats: int, threads: int):
    """Times the oracle's restatement of ONE layer-step of the path for `n_seqs` sequences on the host cores and
    returns (seconds per layer-step, seconds per stage).  `kind`: "dense" (all rows through attention and FFN),
    "sparse" (full-sequence queries) or "pruned" (response-only queries); the sparse kinds process
    `sal_per_seq` salient response rows per sequence.  Stages: norms + q/o projections + rotary embedding
    ("rowwise"), K/V projection + cache update ("kv"), exact attention of the salient rows ("salient_attention"),
    approximate attention + statistics ("delta_attention"), mask + compaction ("select"), FFN ("ffn")."""
    from oracle import dyllm_oracle as orc

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    hid, H, Hkv, I, _, E, topk = layer_shape(cfg)
    D, P, R = 128, cfg["prompt"], cfg["gen"]
    L = P + R
    lq = R if kind == "pruned" else L
    Tk, Tq = n_seqs * L, n_seqs * lq
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.02
    w = dict(q=rnd(H * D, hid), kv=rnd(2 * Hkv * D, hid), o=rnd(hid, H * D))
    if E:
        w.update(router=rnd(E, hid), w1=rnd(E, 2 * I, hid), w2=rnd(E, hid, I))
    else:
        w.update(gu=rnd(2 * I, hid), down=rnd(hid, I))
    x = torch.randn(Tq, hid, generator=g)
    res = torch.randn(Tq, hid, generator=g)
    k_cache = torch.randn(Tk, Hkv, D, generator=g)
    v_cache = torch.randn(Tk, Hkv, D, generator=g)
    c_cache = torch.randn(Tq, H, D, generator=g)
    ffn_cache = torch.randn(Tq, hid, generator=g)
    ar = torch.arange(n_seqs + 1, dtype=torch.int32)
    cu_q, cu_k, cu_sal = ar * lq, ar * L, ar * sal_per_seq
    sal_off = [torch.sort(torch.randperm(R, generator=g)[:sal_per_seq]).values for _ in range(n_seqs)]
    idx_k = torch.cat([o + b * L + P for b, o in enumerate(sal_off)])
    idx_q = torch.cat([o + b * lq + (0 if kind == "pruned" else P) for b, o in enumerate(sal_off)])
    pos_q = (torch.arange(P, L) if kind == "pruned" else torch.arange(L)).repeat(n_seqs)
    pos_k = torch.arange(L).repeat(n_seqs)
    ones = torch.ones(hid)
    stages: dict = {}

    def timed(name, fn):
        t0 = time.perf_counter()
        out = fn()
        stages[name] = stages.get(name, 0.0) + time.perf_counter() - t0
        return out

    def ffn(rows_x):
        if E:
            tw, ti = orc.moe_gate(rows_x, w["router"], topk)
            return orc.naive_experts(rows_x, w["w1"], w["w2"], tw, ti, round_bf16=False)
        return orc.swiglu_ffn(rows_x, w["gu"], w["down"], round_bf16=False)

    def one_step():
        h, r = timed("rowwise", lambda: orc.rms_norm(x, ones, 1e-5, residual=res))
        q = timed("rowwise", lambda: orc.rope(pos_q, (h @ w["q"].t()).view(Tq, H, D), D, 500000.0, 4096))
        if kind == "dense":
            def kv_all():
                kv = h @ w["kv"].t()
                k_cache.copy_(orc.rope(pos_k, kv[:, : Hkv * D].reshape(-1, Hkv, D), D, 500000.0, 4096))
                v_cache.copy_(kv[:, Hkv * D:].reshape(-1, Hkv, D))
            timed("kv", kv_all)
            new_c = timed("salient_attention", lambda: orc.exact_attention_varlen(q, k_cache, v_cache, cu_q, cu_k))
            c_cache.copy_(new_c)
            a = timed("rowwise", lambda: new_c.flatten(1) @ w["o"].t())
            h2, _ = timed("rowwise", lambda: orc.rms_norm(a, ones, 1e-5, residual=r))
            ffn_cache.copy_(timed("ffn", lambda: ffn(h2)))
            return Tq

        def kv_salient():
            kv = h[idx_q] @ w["kv"].t()
            k_cache[idx_k] = orc.rope(pos_k[idx_k], kv[:, : Hkv * D].reshape(-1, Hkv, D), D, 500000.0, 4096)
            dv = torch.zeros_like(v_cache)
            dv[idx_k] = orc.delta_v_update(kv[:, Hkv * D:].reshape(-1, Hkv, D), v_cache, idx_k)
            return dv
        dv = timed("kv", kv_salient)
        o_sal = timed("salient_attention", lambda: orc.exact_attention_varlen(q[idx_q], k_cache, v_cache, cu_sal, cu_k))
        new_c, stats, _ = timed("delta_attention", lambda: orc.attention_sparse_varlen(
            q, k_cache, dv, c_cache, o_sal, cu_q, cu_k, cu_sal, idx_q, cfg["tau"], round_p_bf16=False))
        sel = timed("select", lambda: orc.salient_select(stats, cfg["tau"], cu_q))
        c_cache.copy_(new_c.float())
        a = timed("rowwise", lambda: new_c.float().flatten(1) @ w["o"].t())
        h2, _ = timed("rowwise", lambda: orc.rms_norm(a, ones, 1e-5, residual=r))
        rows = sel["idx"] if sel["count"] else idx_q
        ffn_cache[rows] = timed("ffn", lambda: ffn(h2[rows]))
        return int(rows.numel())

    one_step()  # warm-up
    stages.clear()
    t0 = time.perf_counter()
    for _ in range(repeats):
        one_step()
    total = (time.perf_counter() - t0) / repeats
    return total, {k: v / repeats for k, v in stages.items()}


def step_mix(cfg, dense_only=False):
    """(dense, full-sequence sparse, response-only sparse) denoising steps of one generation, as the
    reference schedules them (dyllm/engine/scheduler.py:29-75, dyllm/engine/model_runner.py:211-222)."""
    if dense_only:
        return cfg["steps"], 0, 0
    dense = min(cfg["full"], cfg["steps"])
    sparse = sum(1 for p in range(dense + 1, cfg["steps"] + 1) if not (p > REFRESH and p % REFRESH != 0))
    return dense, sparse, cfg["steps"] - dense - sparse


def cpu_baseline(cfg, tau, threads: int, repeats: int, n_seqs: int = 1, sal_per_seq: int = 3):
    """CPU tokens/s of the whole job, extrapolated from layer-steps of each kind timed on `n_seqs` sequences."""
    layers = layer_shape(cfg)[4]
    mix = dict(zip(("dense", "sparse", "pruned"), step_mix(cfg, tau is None)))
    per_kind, stages = {}, {}
    for kind, n in mix.items():
        if n:
            per_kind[kind], st = cpu_layer_step_seconds(cfg, kind, n_seqs, sal_per_seq, repeats if kind != "dense" else 1, threads)
            stages[kind] = {k: round(v, 4) for k, v in st.items()}
    total = sum(per_kind[k] * mix[k] for k in per_kind) * layers * (cfg["batch"] / n_seqs)
    value = cfg["batch"] * cfg["gen"] / total
    sample = (f"one layer-step of each kind of the restated path (fp32 torch on {threads} host threads) for {n_seqs} of "
              f"{cfg['batch']} sequences with {sal_per_seq} salient rows per sequence (the GPU arm's measured mean): "
              + ", ".join(f"{k} {per_kind[k]:.2f} s x{mix[k]} steps" for k in per_kind)
              + f"; extrapolated x{layers} layers x{cfg['batch'] // n_seqs} sequences; embedding, lm_head and sampler not included")
    return value, sample, stages, sum(per_kind.values())


def run_reference_arm(args, cfg, tau):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    values, sample, stages, secs = [], "", {}, 0.0
    for _ in range(args.warmup):
        cpu_layer_step_seconds(cfg, "pruned", 1, 3, 1, threads)
    for _ in range(args.steps):
        v, sample, stages, secs = cpu_baseline(cfg, tau, threads, repeats=2)
        values.append(v)
    value = sum(values) / len(values)
    line = {
        "impl": "reference", "metric": metric_name(cfg, tau), "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(cfg, tau, args.gpus, args),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
                         "stage_seconds_per_layer_step": stages},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def config_dict(cfg, tau, n_gpus: int, args):
    dense, sparse, pruned = step_mix(cfg, tau is None)
    par = f"tp{n_gpus}" + (f"+ep{n_gpus}" if getattr(args, "ep", False) and n_gpus > 1 else "")
    return {"workload": f"{cfg['label']}, batch {cfg['batch']}, prompt {cfg['prompt']} uniform-random ids, gen {cfg['gen']}, "
                        f"block {cfg['block']}, {cfg['steps']} denoising steps ({dense} dense + {sparse} full-sequence sparse + "
                        f"{pruned} response-only sparse, refresh period 4 as in the reference code), "
                        + ("dense comparator (no sparse steps)" if tau is None else f"tau {tau:g}"),
            "global_batch": cfg["batch"], "prompt_len": cfg["prompt"], "gen_len": cfg["gen"], "parallelism": par,
            "l2": "inputs_larger_than_l2 (the weights streamed per denoising step exceed the 126 MB L2 many times)",
            "step_driver": "device-resident loop; each denoising step replays one captured CUDA graph (with several "
                           "ranks the graph holds the NCCL o_proj all-reduces and the peer-memory exchanges of the "
                           "statistics and FFN rows); the vocabulary projection runs on the rows the sampler reads"}


# ----------------------------------------------------------------------------------------------
# this library
# ----------------------------------------------------------------------------------------------
def build_model(cfg, tau, dev, layers_override, ep: bool):
    from dyllm_b200 import model as M

    thr = 0.99 if tau is None else tau
    fam = cfg["family"]
    if fam == "dream":
        shape = M.DreamShape()
        ctor = lambda: M.DreamForDLM(shape, thr)
    elif fam == "lladamoe":
        shape = M.LLaDAMoEShape()
        world = int(os.environ.get("WORLD_SIZE", "1"))
        ctor = lambda: M.LLaDAMoEForDLM(shape, thr, world if ep else 1)
    else:
        shape = M.LLaDAShape()
        ctor = lambda: M.LLaDAForDLM(shape, thr)
    if layers_override:
        shape.num_hidden_layers = layers_override
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = ctor()
    finally:
        torch.set_default_dtype(torch.float32)
    M.init_weights_(model, seed=0)
    return model.eval(), shape


def ffn_replay_ms(model, rows: int, cap: int, dev):
    """Average duration of one FFN call of the workload (packed salient rows in, scatter into a cache out, live
    count `rows` on the device, launch shapes of a captured step) measured the way the timed region runs it: all
    layers' calls captured into one CUDA graph (every call streams its own layer's weights from HBM) and the
    replay timed with CUDA events."""
    from dyllm_b200 import ops, runner

    mlps = [layer.mlp for layer in model.model.layers if hasattr(layer.mlp, "gate_up_proj") and hasattr(layer.mlp.gate_up_proj, "weight")]
    if not mlps:
        return None
    hidden = mlps[0].down_proj.weight.size(0)
    x = torch.randn(cap, hidden, device=dev).bfloat16()
    cache = torch.zeros(cap, hidden, device=dev, dtype=torch.bfloat16)
    dest = torch.arange(cap, device=dev, dtype=torch.int32)
    count = torch.tensor([rows], dtype=torch.int32, device=dev)

    def run_all():
        for m in mlps:
            ops.swiglu_ffn(x, m.gate_up_proj.weight, m.down_proj.weight, None, num_rows=cap, num_rows_dev=count,
                           rows_hint=min(runner.GRAPH_ROWS_HINT, cap), out=cache, out_row_map=dest)

    run_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all()
    graph.replay()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    ev0.record()
    for _ in range(reps):
        graph.replay()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / (reps * len(mlps))
    del graph
    return ms


def _exit_after(seconds: float):
    """Teardown guard: the JSON line is out; if releasing the process group still blocks, leave anyway."""
    t = threading.Timer(seconds, lambda: os._exit(0))
    t.daemon = True
    t.start()


def run_ours(args, cfg, tau):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from dyllm_b200 import _lib, layers, profiling, runner

    _lib.load()
    B, P, GEN = cfg["batch"], cfg["prompt"], cfg["gen"]
    comm, exchange = None, "none"
    layout = args.layout if args.layout != "auto" else ("sequence" if world > 1 and B % world == 0 else "tensor")
    if world > 1:
        exchange = "nccl"
        if layout == "sequence" and args.tp_exchange != "peer":
            raise SystemExit("--layout sequence needs --tp-exchange peer")
        if args.tp_exchange == "peer":
            from dyllm_b200.tp_comm import TpComm

            hidden = layer_shape(cfg)[0]
            if layout == "sequence":
                slot_rows = max((B // world) * (P + GEN), 1024)
                exchange = ("peer-memory stores over NVLink: salient rows gathered to every rank, partial FFN outputs "
                            "returned to the rows' owners; no other collective in a step")
            else:
                slot_rows = min(B * (P + GEN), 32768)
                exchange = "peer-memory stores over NVLink (statistics, FFN rows) + NCCL (o_proj)"
            comm = TpComm.from_process_group(dev, slot_bytes=slot_rows * hidden * 2)
            layers.set_tp_comm(comm)
        layers.set_layout(layout)
    layers.set_projection_backend(args.projection)
    layers.set_dense_attention_backend(args.dense_attention)

    tp_parity = None
    if world > 1 and not args.no_tp_parity:
        from dyllm_b200 import tp_selfcheck

        tp_parity = tp_selfcheck.run(dev, 0.99)

    model, shape = build_model(cfg, tau, dev, args.layers, args.ep)
    dsteps = args.denoise_steps or cfg["steps"]
    full_steps = dsteps if tau is None else (args.full_steps if args.full_steps is not None else cfg["full"])
    sr = runner.StepRunner(model, shape.mask_token_id, cfg["block"], dsteps, full_steps, REFRESH,
                           graph_rows_hint=args.rows_hint or runner.GRAPH_ROWS_HINT)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, shape.vocab_size - 1024, (B, P), generator=g).tolist()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        sr.generate(prompts, GEN)

    # ---- device-timed region: K generations (each denoising step replays a captured CUDA graph) ---
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        sr.generate(prompts, GEN)
    ev1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    launches = _lib.launch_count - launches0

    # ---- end-to-end through the public step driver, host buffers in, host tokens out ------------
    runner.io_bytes["h2d"] = runner.io_bytes["d2h"] = 0
    barrier()
    t0 = time.perf_counter()
    e2e_gens = max(1, min(args.steps, 2))
    out_tokens = None
    for _ in range(0 if args.no_e2e else e2e_gens):
        out_tokens = sr.generate(prompts, GEN)
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_s = float(e2e_s.item())
    io_per_gen = {k: v // e2e_gens for k, v in runner.io_bytes.items()}   # read before the profiling pass adds to it
    assert out_tokens is None or (len(out_tokens) == B and len(out_tokens[0]) == GEN)

    # ---- per-kernel durations: one more generation of the same workload with CUDA events around this
    # library's main kernels (events cannot be timed inside a graph, so this pass launches eagerly) ----
    profiling.enable(True)
    profiling.reset()
    barrier()
    ev0.record()
    sr.generate(prompts, GEN)
    ev1.record()
    barrier()
    instr_ms = ev0.elapsed_time(ev1)
    prof = profiling.summary()
    counts = profiling.counts()
    profiling.enable(False)

    def teardown():
        sr.release_graphs()          # graphs that captured NCCL kernels keep the communicator alive
        if comm is not None:
            layers.set_tp_comm(None)
            comm.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    if rank != 0:
        _exit_after(120.0)
        teardown()
        return

    value = args.steps * B * GEN / (total_ms / 1e3)
    peaks = measured_peaks()
    traffic = ncu_traffic_bytes() if args.config == 1 and world == 1 else {}
    # dominant kernel of this library; its bound is the roofline that gives the longer time
    mine = {k: v for k, v in prof.items() if v["launches"]}
    # (the exchange regions of several ranks are NVLink latency, not a roofline of this GPU: listed, never dominant)
    compute = {k: v for k, v in mine.items() if not k.endswith(("_exchange", "_all_reduce"))}
    dominant = max(compute, key=lambda k: compute[k]["total_ms"]) if compute else None
    roofline = None
    if dominant:
        d = mine[dominant]
        secs = d["total_ms"] / 1e3
        t_hbm = d["bytes"] / (peaks["hbm_gbs"] * 1e9)
        t_tensor = d["work"] / (peaks["tflops"] * 1e12)
        common = {"traffic": traffic.get(dominant), "avg_launch_ms": d["avg_ms"], "launches": d["launches"],
                  "algorithmic_bytes_per_launch": d["bytes"] / d["launches"],
                  "algorithmic_flops_per_launch": d["work"] / d["launches"],
                  "timed_in": "one generation of the same workload launched eagerly with CUDA events around the "
                              "kernel, right after the timed region (which replays CUDA graphs)"}
        if t_hbm >= t_tensor:
            gbs = d["bytes"] / secs / 1e9
            roofline = {"kernel": dominant, "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"], **common}
        else:
            tflops = d["work"] / secs / 1e12
            roofline = {"kernel": dominant, "bound": "tensor", "achieved": tflops, "peak": peaks["tflops"],
                        "unit": "TFLOP/s", "frac": tflops / peaks["tflops"],
                        "peak_source": f"{peaks['source']} (sustained bf16)", **common}
    if roofline and dominant == "swiglu_ffn" and world == 1 and cfg["family"] != "lladamoe":
        # the eager figure above contains the host gaps between the region's launches; the same call replayed
        # inside a CUDA graph (as in the timed region) gives the kernel-level figure
        sal_mean = max(1, round(sum(counts.get("salient_rows", [46])) / max(1, len(counts.get("salient_rows", [46])))))
        ms_replay = ffn_replay_ms(model, sal_mean, B * (P + GEN), dev)
        if ms_replay:
            d = mine[dominant]
            per_bytes, per_flops = d["bytes"] / d["launches"], d["work"] / d["launches"]
            roofline["eager_avg_launch_ms"], roofline["eager_frac"] = roofline["avg_launch_ms"], roofline["frac"]
            roofline["avg_launch_ms"] = ms_replay
            if roofline["bound"] == "hbm":
                roofline["achieved"] = per_bytes / (ms_replay / 1e3) / 1e9
            else:
                roofline["achieved"] = per_flops / (ms_replay / 1e3) / 1e12
            roofline["frac"] = roofline["achieved"] / roofline["peak"]
            roofline["timed_in"] = (f"the FFN call of the workload's 32 layers ({sal_mean} salient rows, the measured mean; "
                                    "packed rows in, scatter into a cache out) captured into one CUDA graph and replayed 5 "
                                    "times between CUDA events, right after the timed region; eager_* = the same region "
                                    "timed with events inside an eagerly launched generation (contains host launch gaps)")
    kernels = {}
    for k, v in mine.items():
        secs = v["total_ms"] / 1e3
        kernels[k] = {"avg_ms": round(v["avg_ms"], 4), "launches": v["launches"],
                      "share_of_step": round(v["total_ms"] / instr_ms, 4),
                      "tflops": round(v["work"] / secs / 1e12, 1) if v["work"] else None,
                      "gbs": round(v["bytes"] / secs / 1e9, 1) if v["bytes"] else None}
    sal = counts.get("salient_rows", [])
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        mean_sal = max(1, round((sum(sal) / len(sal)) / B)) if sal else 3
        v, sample, stages, _ = cpu_baseline(cfg, tau, threads, repeats=3, sal_per_seq=mean_sal)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
               "stage_seconds_per_layer_step": stages}
    cfg_d = config_dict(cfg, tau, world, args)
    cfg_d["tp_exchange"] = exchange
    cfg_d["all_row_projections"] = args.projection
    cfg_d["dense_step_attention"] = args.dense_attention
    if world > 1:
        cfg_d["layout"] = layout
        if layout == "sequence":
            cfg_d["parallelism"] = (f"{world} ranks: sequences of the batch sharded for attention and the all-row work "
                                    f"(replicated attention weights), FFN weights tensor-parallel tp{world}"
                                    + (f" / experts ep{world}" if args.ep else ""))
    line = {
        "metric": metric_name(cfg, tau), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg_d,
        "clocks": clocks, "gpu_launches": launches,
        "e2e": None if args.no_e2e else {"value": e2e_gens * B * GEN / e2e_s, "unit": "tokens/s",
                                         "h2d_bytes_per_step": io_per_gen["h2d"], "d2h_bytes_per_step": io_per_gen["d2h"]},
        "roofline": roofline, "cpu_baseline": cpu, "kernels": kernels,
        "salient_rows_per_layer": {"mean": (sum(sal) / len(sal)) if sal else None, "max": max(sal) if sal else None},
    }
    if tp_parity is not None:
        line["tp_parity"] = tp_parity
    if args.layers or args.denoise_steps or args.full_steps is not None:
        line["invalid_reduced_config"] = True
    print(json.dumps(line), flush=True)
    _exit_after(120.0)
    teardown()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=sorted(CONFIGS))
    ap.add_argument("--tau", type=float, default=None, help="salient threshold (default: the workload's, 0.99)")
    ap.add_argument("--dense", action="store_true", help="the tau=None comparator: every denoising step dense")
    ap.add_argument("--ep", action="store_true", help="config 4: whole experts per rank (expert parallelism)")
    ap.add_argument("--tp-exchange", default="peer", choices=["peer", "nccl"],
                    help="carrier of the small per-layer all-reduces under tensor parallelism")
    ap.add_argument("--layout", default="auto", choices=["auto", "tensor", "sequence"],
                    help="several GPUs: 'tensor' = the reference's layout (heads and FFN columns sharded, rows replicated, "
                         "three all-reduces per layer); 'sequence' = every rank owns whole sequences, only the FFN weights "
                         "are sharded and only salient rows travel (auto: sequence when the batch divides evenly)")
    ap.add_argument("--rows-hint", type=int, default=0,
                    help="salient rows per layer the captured steps are shaped for (default 128; any value is correct)")
    ap.add_argument("--no-tp-parity", action="store_true", help="skip the sharded-vs-unsharded layer self-check")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers marks the line invalid")
    ap.add_argument("--denoise-steps", type=int, default=0, help="debug only")
    ap.add_argument("--full-steps", type=int, default=None, help="debug only: dense steps per generation")
    ap.add_argument("--projection", default="cublas", choices=["cublas", "tcgen05"],
                    help="GEMM of the all-row q / o projections: cuBLAS (default) or this package's tcgen05 GEMM")
    ap.add_argument("--dense-attention", default="sdpa", choices=["tcgen05", "sdpa"],
                    help="attention of the dense steps: torch SDPA (default) or this package's exact-attention kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="sweeps: skip the end-to-end leg (e2e is then null)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    tau = None if args.dense else (args.tau if args.tau is not None else cfg["tau"])
    if tau is not None:
        cfg["tau"] = tau
    if args.impl == "reference":
        run_reference_arm(args, cfg, tau)
    else:
        run_ours(args, cfg, tau)


if __name__ == "__main__":
    main()
