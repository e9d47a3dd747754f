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
    mask = layers.tensor_parallel_cosine_mask(stats, 0.99)     # all-reduces in place
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
    out_queue.put((rank, ok_mask, bool(ok_col), bool(ok_merged), bool(ok_kv), bool(ok_row), bool(ok_sum)))
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
