"""Tensor parallelism on real GPUs (needs at least two; skipped otherwise): one process per GPU, NCCL for
the process group, CUDA IPC for the peer-memory exchange.

* the exchange kernels over IPC-mapped regions give every rank the bit-identical rank-ordered sum;
* a sharded decoder layer agrees with the unsharded one (dyllm_b200.tp_selfcheck);
* a small model generates the same token ids with whole-step CUDA graphs (NCCL all-reduces and exchanges
  captured inside) as with eager launches, and the process group shuts down after the graphs are released.
"""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from dyllm_b200 import _lib, layers, runner, tp_selfcheck
    from dyllm_b200.model import LLaDAForDLM, LLaDAShape, init_weights_
    from dyllm_b200.tp_comm import TpComm

    out = {}
    comm = TpComm.from_process_group(dev, slot_bytes=1024 * 4096 * 2)
    # --- exchange: rows (two rounds, count on the device, scatter map) and fp32 ------------------
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    cap, width, live = 2500, 4096, 1717        # more rows than a slot holds: three rounds
    count = torch.tensor([live], dtype=torch.int32, device=dev)
    ok_rows = True
    for _ in range(3):
        src = torch.randn(cap, width, generator=g, device=dev).bfloat16()
        gathered = [torch.empty_like(src) for _ in range(world)]
        dist.all_gather(gathered, src)
        want = torch.zeros(cap, width, device=dev)
        for t in gathered:
            want += t.float()
        dest = torch.full((cap, width), 5.0, dtype=torch.bfloat16, device=dev)
        comm.all_reduce_rows(src, count, out=dest)
        ref = torch.full((cap, width), 5.0, dtype=torch.bfloat16, device=dev)
        ref[:live] = want.bfloat16()[:live]
        ok_rows &= bool(torch.equal(dest, ref))
    stats = torch.randn(1000, 3, generator=g, device=dev)
    gathered = [torch.empty_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    want = torch.zeros_like(stats)
    for t in gathered:
        want += t
    comm.all_reduce_f32_(stats)
    out["exchange"] = ok_rows and bool(torch.equal(stats, want))

    # --- sharded layer against the unsharded one --------------------------------------------------
    layers.set_tp_comm(comm)
    report = tp_selfcheck.run(dev, 0.99)
    out["selfcheck"] = report

    # --- whole-step graphs with collectives inside == eager; clean shutdown ----------------------
    shape = LLaDAShape(hidden_size=512, num_attention_heads=4, n_kv_heads=4, head_dim=128, mlp_hidden_size=1024,
                       num_hidden_layers=2, vocab_size=1024, mask_token_id=1000, max_sequence_length=256)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = LLaDAForDLM(shape, 0.99)
    torch.set_default_dtype(torch.float32)
    init_weights_(model, seed=3, std=0.05)
    model.eval()
    prompts = torch.randint(0, 900, (3, 40), generator=torch.Generator().manual_seed(0)).tolist()
    eager = runner.StepRunner(model, shape.mask_token_id, block_length=8, steps=32, num_full_steps=4, use_graphs=False)
    graphs = runner.StepRunner(model, shape.mask_token_id, block_length=8, steps=32, num_full_steps=4, use_graphs=True)
    want_tokens = eager.generate(prompts, 32)
    first = graphs.generate(prompts, 32)
    second = graphs.generate(prompts, 32)
    out["graphs_equal_eager"] = first == want_tokens and second == want_tokens
    out["graphs_captured"] = len(graphs._graphs)
    out["status"] = _lib.load().dyllm_device_status()
    graphs.release_graphs()

    # --- sequence-sharded layout: every rank owns whole sequences, the FFN weights stay sharded --------
    layers.set_layout("sequence")
    try:
        out["selfcheck_sequence"] = tp_selfcheck.run(dev, 0.99)
        torch.set_default_dtype(torch.bfloat16)
        with torch.device(dev):
            model_s = LLaDAForDLM(shape, 0.99)
        torch.set_default_dtype(torch.float32)
        init_weights_(model_s, seed=3, std=0.05)
        model_s.eval()
        prompts4 = torch.randint(0, 900, (4, 40), generator=torch.Generator().manual_seed(1)).tolist()
        eager_s = runner.StepRunner(model_s, shape.mask_token_id, block_length=8, steps=32, num_full_steps=4, use_graphs=False)
        graphs_s = runner.StepRunner(model_s, shape.mask_token_id, block_length=8, steps=32, num_full_steps=4, use_graphs=True)
        want_s = eager_s.generate(prompts4, 32)
        got_s = [graphs_s.generate(prompts4, 32) for _ in range(2)]
        out["sequence_graphs_equal_eager"] = all(g == want_s for g in got_s) and len(want_s) == 4
        # attention weights are complete on every rank, FFN weights are shards
        a, m = model_s.model.layers[0].self_attn, model_s.model.layers[0].mlp
        out["sequence_shapes"] = (tuple(a.q_proj.weight.shape), tuple(m.down_proj.weight.shape))
        out["status_sequence"] = _lib.load().dyllm_device_status()
        graphs_s.release_graphs()
    finally:
        layers.set_layout("tensor")
    layers.set_tp_comm(None)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    out["shutdown"] = True
    results[rank] = out


@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_path_on_gpus(cuda_device, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    for p in procs:
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    for r in range(world):
        res = results[r]
        assert res["exchange"], res
        assert res["graphs_equal_eager"] and res["graphs_captured"] == 3, res
        assert res["status"] == 0 and res["shutdown"], res
        assert res["sequence_graphs_equal_eager"] and res["status_sequence"] == 0, res
        assert res["sequence_shapes"] == ((512, 512), (512, 1024 // world)), res
    for key in ("selfcheck", "selfcheck_sequence"):
        report = results[0][key]
        print(f"{key}: sharded vs unsharded layer:", report)
        assert report["ok"], report
