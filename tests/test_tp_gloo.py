"""Host-side tensor-parallel logic on two CPU ranks (gloo): the additive 12-byte-per-token statistics give
the same decisions as the full vectors on every rank, and the shard-aware weight loaders split a
checkpoint tensor the way the reference's linear layers do (ref: dyllm/model_executor/layers/linear.py)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_queue):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dyllm_b200 import layers
    from oracle import dyllm_oracle as orc

    g = torch.Generator().manual_seed(0)
    c_old, c_new = orc.make_context_pair(300, 512, 0.99, 0.15, seed=4)
    shard = 512 // world
    stats = orc.context_stats(c_old[:, rank * shard:(rank + 1) * shard], c_new[:, rank * shard:(rank + 1) * shard])
    layers.all_reduce_sum(stats)                               # the 12-byte-per-token exchange, in place
    mask = orc.cosine_mask(stats, 0.99)                        # CPU ranks: the decision comes from the checker
    full = orc.cosine_mask(orc.context_stats(c_old, c_new), 0.99)
    ok_mask = bool(torch.equal(mask, full))

    # weight loaders: column / merged-column / KV / row parallel shards
    w = torch.randn(64, 32, generator=g)
    col = layers.ColumnParallelLinear(32, 64)
    col.weight_loader(col.weight, w)
    ok_col = torch.equal(col.weight.data, w[rank * 32:(rank + 1) * 32])
    merged = layers.MergedColumnParallelLinear(32, [32, 32])
    merged.weight_loader(merged.weight, w[:32], 0)
    merged.weight_loader(merged.weight, w[32:], 1)
    ok_merged = torch.equal(merged.weight.data[:16], w[rank * 16:(rank + 1) * 16]) and \
        torch.equal(merged.weight.data[16:], w[32 + rank * 16: 32 + (rank + 1) * 16])
    kv = layers.KVParallelLinear(32, 8, 4)          # 4 KV heads of 8 -> 2 per rank
    kv.weight_loader(kv.weight, w[:32], "k")
    kv.weight_loader(kv.weight, w[32:], "v")
    ok_kv = torch.equal(kv.weight.data[:16], w[rank * 16:(rank + 1) * 16]) and \
        torch.equal(kv.weight.data[16:], w[32 + rank * 16: 32 + (rank + 1) * 16])
    row = layers.RowParallelLinear(32, 64)
    row.weight_loader(row.weight, w)
    ok_row = torch.equal(row.weight.data, w[:, rank * 16:(rank + 1) * 16])
    # row-parallel product + all-reduce == full product
    x = torch.randn(5, 32, generator=g)
    with torch.no_grad():
        y = row(x[:, rank * 16:(rank + 1) * 16])
    ok_sum = torch.allclose(y, x @ w.t(), atol=1e-5)
    # seeded random init: every rank's shards are slices of the tensors the single-rank model draws
    from dyllm_b200 import cache_manager, model
    cache_manager.CacheManager.__init__.__defaults__ = (64, torch.float32, torch.device("cpu"))
    cfg = model.LLaDAShape(hidden_size=256, num_attention_heads=4, n_kv_heads=2, mlp_hidden_size=512,
                           num_hidden_layers=1, vocab_size=512, max_sequence_length=64)
    with layers.replicated():
        single = model.LLaDAForDLM(cfg, 0.99)
    model.init_weights_(single, seed=3)
    sharded = model.LLaDAForDLM(cfg, 0.99)
    model.init_weights_(sharded, seed=3)
    a1, a2 = single.model.layers[0].self_attn, sharded.model.layers[0].self_attn
    m1, m2 = single.model.layers[0].mlp, sharded.model.layers[0].mlp
    sl = lambda t, n, d=0: t.narrow(d, rank * n, n)
    ok_init = (torch.equal(a2.q_proj.weight, sl(a1.q_proj.weight, 256))
               and torch.equal(a2.kv_proj.weight[:128], sl(a1.kv_proj.weight[:256], 128))
               and torch.equal(a2.kv_proj.weight[128:], sl(a1.kv_proj.weight[256:], 128))
               and torch.equal(a2.o_proj.weight, sl(a1.o_proj.weight, 256, 1))
               and torch.equal(m2.gate_up_proj.weight[:256], sl(m1.gate_up_proj.weight[:512], 256))
               and torch.equal(m2.gate_up_proj.weight[256:], sl(m1.gate_up_proj.weight[512:], 256))
               and torch.equal(m2.down_proj.weight, sl(m1.down_proj.weight, 256, 1))
               and torch.equal(sharded.lm_head.weight, single.lm_head.weight)
               and torch.equal(sharded.model.embed_tokens.weight, single.model.embed_tokens.weight))
    out_queue.put((rank, ok_mask, bool(ok_col), bool(ok_merged), bool(ok_kv), bool(ok_row), bool(ok_sum), bool(ok_init)))
    dist.destroy_process_group()


def test_two_rank_statistics_and_weight_shards():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for res in results:
        assert all(res[1:]), res
