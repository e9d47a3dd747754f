#!/usr/bin/env python
"""Throughput of the saliency path on the LLaDA-8B configuration: generated tokens/s at batch 16,
prompt 256, generation length 256, block 32, 256 denoising steps, threshold 0.99, random-init bf16
weights and uniform-random prompt ids (synthetic stand-ins for a checkpoint and a dataset).

    python bench.py --gpus N --steps K --warmup W            this library (one process per GPU, TP over NCCL)
    python bench.py --impl reference ...                      CPU restatement of the reference path on the host cores

One "step" is one complete generation of the batch (256 denoising steps: 8 dense, 248 sparse with the
reference's period-4 full-sequence refresh), so tokens/s = steps * batch * gen_len / time.
Prints one JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, PROMPT, GEN, BLOCK, DSTEPS, TAU, FULL_STEPS, REFRESH = 16, 256, 256, 32, 256, 0.99, 8, 4
METRIC = "generated tokens/s (LLaDA-8B bf16, b=16, gen=256, tau=0.99)"

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch of this library's kernels at this
# workload's shapes, from the ncu captures summarised under profiles/: the gathered FFN at 48 salient
# rows (four launches), the exact attention of the salient rows, and the approximate attention, whose
# capture is a launch with full-sequence queries (252.2 MB) scaled by the algorithmic bytes to the mix of
# one full-sequence and three response-only launches that the bench averages over.
NCU_TRAFFIC_BYTES = {"delta_attention": 181.6e6, "swiglu_ffn": 320.0e6, "salient_attention": 138.4e6}


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
# CPU restatement of one layer-step of the path (checker code, timed as the reported CPU baseline)
# ----------------------------------------------------------------------------------------------
def cpu_layer_step_seconds(n_seqs: int, repeats: int, threads: int):
    """Times the oracle's restatement of one sparse layer-step (RMSNorm, q/kv/o projections, rotary
    embedding, delta-V, salient-row attention, approximate attention, statistics, mask, compaction, gathered
    SwiGLU FFN, cache scatter) at the LLaDA-8B layer shape for `n_seqs` sequences of 512 tokens with ~10 %
    salient response rows.  Returns seconds per layer-step for those sequences."""
    from oracle import dyllm_oracle as orc

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    hid, H, D, I, L = 4096, 32, 128, 12288, PROMPT + GEN
    T = n_seqs * L
    w = {k: torch.randn(s, generator=g) * 0.02 for k, s in
         dict(q=(H * D, hid), kv=(2 * H * D, hid), o=(hid, H * D), gu=(2 * I, hid), down=(hid, I)).items()}
    x = torch.randn(T, hid, generator=g)
    res = torch.randn(T, hid, generator=g)
    k_cache = torch.randn(T, H, D, generator=g)
    v_cache = torch.randn(T, H, D, generator=g)
    c_cache = torch.randn(T, H, D, generator=g)
    ffn_cache = torch.randn(T, hid, generator=g)
    cu = torch.arange(n_seqs + 1, dtype=torch.int32) * L
    idx = torch.cat([torch.sort(torch.randperm(GEN, generator=g)[:26]).values + b * L + PROMPT for b in range(n_seqs)])
    cu_sal = torch.arange(n_seqs + 1, dtype=torch.int32) * 26
    pos = torch.arange(L).repeat(n_seqs)
    ones = torch.ones(hid)

    def one_step():
        h, r = orc.rms_norm(x, ones, 1e-5, residual=res)
        q = orc.rope(pos, (h @ w["q"].t()).view(T, H, D), D, 500000.0, 4096)
        kv = h[idx] @ w["kv"].t()
        k_new = orc.rope(pos[idx], kv[:, : H * D].reshape(-1, H, D), D, 500000.0, 4096)
        v_new = kv[:, H * D:].reshape(-1, H, D)
        k_cache[idx] = k_new
        dv = torch.zeros_like(v_cache)
        dv[idx] = v_new - v_cache[idx]
        v_cache[idx] = v_new
        o_sal = orc.exact_attention_varlen(q[idx], k_cache, v_cache, cu_sal, cu)
        new_c, stats, _ = orc.attention_sparse_varlen(q, k_cache, dv, c_cache, o_sal, cu, cu, cu_sal, idx, TAU,
                                                      round_p_bf16=False)
        sel = orc.salient_select(stats, TAU, cu)
        c_cache.copy_(new_c.float())
        a = new_c.float().flatten(1) @ w["o"].t()
        h2, _ = orc.rms_norm(a, ones, 1e-5, residual=r)
        rows = sel["idx"] if sel["count"] else idx
        ffn_cache[rows] = orc.swiglu_ffn(h2[rows], w["gu"], w["down"], round_bf16=False)
        return int(rows.numel())

    one_step()  # warm-up
    t0 = time.perf_counter()
    for _ in range(repeats):
        one_step()
    return (time.perf_counter() - t0) / repeats


def cpu_tokens_per_s(sec_per_layer_step: float, n_seqs: int, layers: int = 32) -> float:
    # whole job = DSTEPS denoising steps x layers x (BATCH / n_seqs) samples
    total = sec_per_layer_step * (BATCH / n_seqs) * layers * DSTEPS
    return BATCH * GEN / total


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    n_seqs = 2
    times = []
    for _ in range(args.warmup):
        cpu_layer_step_seconds(n_seqs, 1, threads)
    for _ in range(args.steps):
        times.append(cpu_layer_step_seconds(n_seqs, 8, threads))
    sec = sum(times) / len(times)
    value = cpu_tokens_per_s(sec, n_seqs)
    sample = (f"one sparse layer-step of the restated path (fp32 torch on CPU) for {n_seqs} of {BATCH} sequences per step, "
              f"extrapolated x{BATCH // n_seqs} sequences x32 layers x{DSTEPS} denoising steps; embedding, lm_head and "
              f"sampler not included")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def config_dict(n_gpus: int):
    return {"workload": "configs[1]: LLaDA-8B shape, 32 layers, batch 16, prompt 256 uniform-random ids, gen 256, "
                        "block 32, 256 denoising steps (8 dense + 248 sparse, full-sequence refresh every 4th sparse "
                        "step as in the reference code), tau 0.99",
            "global_batch": BATCH, "prompt_len": PROMPT, "gen_len": GEN, "parallelism": f"tp{n_gpus}",
            "l2": "inputs_larger_than_l2 (16 GB of weights streamed per denoising step)",
            "step_driver": "device-resident loop; each denoising step replays a captured CUDA graph (with several "
                           "ranks: a chain of graphs with the NCCL all-reduces issued between them); the "
                           "vocabulary projection runs on the rows the sampler reads (current block)"}


# ----------------------------------------------------------------------------------------------
# this library
# ----------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from dyllm_b200 import _lib, profiling, runner
    from dyllm_b200.model import LLaDAForDLM, LLaDAShape, init_weights_

    _lib.load()
    shape = LLaDAShape(num_hidden_layers=args.layers)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = LLaDAForDLM(shape, TAU)
    torch.set_default_dtype(torch.float32)
    init_weights_(model, seed=0)
    model.eval()
    sr = runner.StepRunner(model, shape.mask_token_id, BLOCK, args.denoise_steps, args.full_steps, REFRESH)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, shape.vocab_size - 1024, (BATCH, PROMPT), generator=g).tolist()

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
    for _ in range(e2e_gens):
        out_tokens = sr.generate(prompts, GEN)
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_s = float(e2e_s.item())
    assert len(out_tokens) == BATCH and len(out_tokens[0]) == GEN

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

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    value = args.steps * BATCH * GEN / (total_ms / 1e3)
    peaks = measured_peaks()
    # dominant kernel of this library; its bound is the roofline that gives the longer time
    mine = {k: v for k, v in prof.items() if v["launches"]}
    dominant = max(mine, key=lambda k: mine[k]["total_ms"]) if mine else None
    roofline = None
    if dominant:
        d = mine[dominant]
        secs = d["total_ms"] / 1e3
        t_hbm = d["bytes"] / (peaks["hbm_gbs"] * 1e9)
        t_tensor = d["work"] / (peaks["tflops"] * 1e12)
        common = {"traffic": NCU_TRAFFIC_BYTES.get(dominant), "avg_launch_ms": d["avg_ms"], "launches": d["launches"],
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
    kernels = {k: {"avg_ms": round(v["avg_ms"], 4), "launches": v["launches"],
                   "share_of_step": round(v["total_ms"] / instr_ms, 4)} for k, v in mine.items()}
    sal = counts.get("salient_rows", [])
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        n_seqs = 2
        sec = cpu_layer_step_seconds(n_seqs, 30, threads)
        cpu = {"value": cpu_tokens_per_s(sec, n_seqs, args.layers), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"30 sparse layer-steps of the restated path for {n_seqs} of {BATCH} sequences "
                         f"({sec:.2f} s each), extrapolated to {args.layers} layers x {DSTEPS} steps x {BATCH} sequences; "
                         f"embedding, lm_head and sampler not included"}
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(world),
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": e2e_gens * BATCH * GEN / e2e_s, "unit": "tokens/s",
                "h2d_bytes_per_step": runner.io_bytes["h2d"] // e2e_gens, "d2h_bytes_per_step": runner.io_bytes["d2h"] // e2e_gens},
        "roofline": roofline, "cpu_baseline": cpu, "kernels": kernels,
        "salient_rows_per_layer": {"mean": (sum(sal) / len(sal)) if sal else None, "max": max(sal) if sal else None},
    }
    if args.layers != 32 or args.denoise_steps != DSTEPS or args.full_steps != FULL_STEPS:
        line["invalid_reduced_config"] = True
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="debug only: fewer layers marks the line invalid")
    ap.add_argument("--denoise-steps", type=int, default=DSTEPS, help="debug only")
    ap.add_argument("--full-steps", type=int, default=FULL_STEPS, help="debug only: dense steps per generation")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
