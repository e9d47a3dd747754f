"""The peer-memory SUM exchange (dyllm_tp_*) on one GPU: the ranks of a tensor-parallel group are emulated
inside one process (their regions are plain pointers to each other), and their kernels run one after the
other on one stream, every push before the first reduce, so no kernel ever waits for a later launch.
The multi-process path over CUDA IPC is covered by tests/test_tp_multi_gpu.py on boxes with several GPUs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _exchange_rows(comms, srcs, count_dev, outs, maps, cap, width):
    step = max(1, comms[0].max_rows(width))
    for off in range(0, cap, step):
        n = min(step, cap - off)
        for c, s in zip(comms, srcs):
            c.push_rows(s, count_dev, off, n)
        for c, o, m in zip(comms, outs, maps):
            c.reduce_rows(width, count_dev, off, n, o, m)


@pytest.mark.parametrize("world,cap,width,live,slot_rows", [(2, 300, 256, 123, 512), (3, 64, 4096, 64, 64),
                                                           (8, 1000, 512, 777, 256), (2, 128, 256, 0, 128)])
def test_rows_exchange_sums_in_rank_order_and_scatters(cuda_device, world, cap, width, live, slot_rows):
    from dyllm_b200 import _lib
    from dyllm_b200.tp_comm import TpComm

    dev = cuda_device
    comms = TpComm.emulated_world(world, slot_rows * width * 2)
    try:
        g = torch.Generator(device=dev).manual_seed(world * 1000 + cap)
        count = torch.tensor([live], dtype=torch.int32, device=dev)
        for round_ in range(3):          # three exchanges: both buffer parities and a reuse
            srcs = [torch.randn(cap, width, generator=g, device=dev).bfloat16() for _ in range(world)]
            perm = torch.randperm(2 * cap, generator=g, device=dev)[:cap].to(torch.int32)
            perm[5 % cap] = -1           # a dropped row
            outs = [torch.full((2 * cap, width), 7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
            _exchange_rows(comms, srcs, count, outs, [perm] * world, cap, width)
            acc = torch.zeros(cap, width, device=dev)
            for s in srcs:               # rank order, fp32
                acc += s.float()
            want = torch.full((2 * cap, width), 7.0, dtype=torch.bfloat16, device=dev)
            keep = (torch.arange(cap, device=dev) < live) & (perm >= 0)
            want[perm[keep].long()] = acc.bfloat16()[keep]
            for o in outs:
                assert torch.equal(o, want), f"round {round_}"
        assert _lib.load().dyllm_device_status() == 0
    finally:
        for c in comms:
            c.close()


def test_f32_exchange(cuda_device):
    from dyllm_b200 import _lib
    from dyllm_b200._lib import call, ptr, stream_ptr
    from dyllm_b200.tp_comm import TpComm

    dev, world, n = cuda_device, 4, 4096 * 3 + 5
    comms = TpComm.emulated_world(world, 1 << 16)
    try:
        g = torch.Generator(device=dev).manual_seed(5)
        for _ in range(2):
            parts = [torch.randn(n, generator=g, device=dev) for _ in range(world)]
            want = torch.zeros(n, device=dev)
            for p in parts:
                want += p
            for c, p in zip(comms, parts):
                call("dyllm_tp_push_f32", c._comm, ptr(p), n, stream_ptr(dev))
            for c, p in zip(comms, parts):
                call("dyllm_tp_reduce_f32", c._comm, ptr(p), n, stream_ptr(dev))
            for p in parts:
                assert torch.equal(p, want)
        assert _lib.load().dyllm_device_status() == 0
    finally:
        for c in comms:
            c.close()


def test_missing_peer_gives_up_with_a_status_code(cuda_device):
    """A rank whose peer never pushes: the reduce kernel's bounded wait runs out (a flag that nothing sets),
    the kernel returns without touching its output, the status word names the missing rank and the device
    stays usable."""
    from dyllm_b200 import _lib
    from dyllm_b200.tp_comm import TpComm

    dev = cuda_device
    comms = TpComm.emulated_world(2, 1 << 16)
    try:
        comms[0].set_wait_ms(20)
        src = torch.ones(16, 64, dtype=torch.bfloat16, device=dev)
        out = torch.full((16, 64), 3.0, dtype=torch.bfloat16, device=dev)
        comms[0].push_rows(src, None, 0, 16)
        comms[0].reduce_rows(64, None, 0, 16, out, None)      # rank 1 never pushed
        torch.cuda.synchronize()
        assert _lib.load().dyllm_device_status() == 0x7E00 + 1
        assert bool((out == 3.0).all())
        assert float((src + 1).sum()) == 2 * 16 * 64            # the context still works
        assert _lib.load().dyllm_device_status() == 0
    finally:
        for c in comms:
            c.close()


def test_slot_overflow_is_rejected(cuda_device):
    from dyllm_b200 import _lib
    from dyllm_b200.tp_comm import TpComm

    comms = TpComm.emulated_world(1, 4096)
    try:
        src = torch.zeros(64, 64, dtype=torch.bfloat16, device=cuda_device)
        with pytest.raises(RuntimeError, match="exceed the slot"):
            comms[0].push_rows(src, None, 0, 64)
        # one rank: the exchange is a copy through the region
        out = torch.ones(32, 64, dtype=torch.bfloat16, device=cuda_device)
        comms[0].all_reduce_rows(src[:32].contiguous() + 2, None, out=out)
        assert bool((out == 2).all())
        assert _lib.load().dyllm_device_status() == 0
    finally:
        comms[0].close()


@pytest.mark.parametrize("world,width,counts", [(2, 256, [5, 0]), (4, 512, [17, 64, 1, 33]), (8, 4096, [3, 0, 9, 2, 0, 1, 7, 4])])
def test_gather_and_owner_scatter_of_the_sequence_sharded_layout(cuda_device, world, width, counts):
    """Every rank contributes a different number of indexed rows; all ranks then see all rows in rank order;
    per-row partial results travel back to the owner, which adds them in rank order and scatters them."""
    from dyllm_b200 import _lib
    from dyllm_b200._lib import call, ptr, stream_ptr
    from dyllm_b200.tp_comm import TpComm

    dev, slot_rows, x_rows = cuda_device, 64, 200
    comms = TpComm.emulated_world(world, slot_rows * width * 2)
    try:
        g = torch.Generator(device=dev).manual_seed(world + width)
        for round_ in range(3):
            xs = [torch.randn(x_rows, width, generator=g, device=dev).bfloat16() for _ in range(world)]
            idxs = [torch.randperm(x_rows, generator=g, device=dev)[:slot_rows].to(torch.int32) for _ in range(world)]
            cnts = [torch.tensor([counts[(r + round_) % world]], dtype=torch.int32, device=dev) for r in range(world)]
            n = [int(c) for c in cnts]
            for c, x, i, k in zip(comms, xs, idxs, cnts):
                call("dyllm_tp_gather_push", c._comm, ptr(x), x_rows, width, x.stride(0), ptr(i), slot_rows, ptr(k), stream_ptr(dev))
            outs = []
            for c in comms:
                idx_all = torch.full((world * slot_rows,), -1, dtype=torch.int32, device=dev)
                prefix = torch.empty(world + 1, dtype=torch.int32, device=dev)
                total = torch.empty(1, dtype=torch.int32, device=dev)
                call("dyllm_tp_gather_finish", c._comm, width, ptr(idx_all), ptr(prefix), ptr(total), stream_ptr(dev))
                outs.append((c.data_matrix(width, dev), idx_all, prefix, total))
            want_rows = torch.cat([x[i[:k].long()] for x, i, k in zip(xs, idxs, n)])
            want_prefix = [0]
            for k in n:
                want_prefix.append(want_prefix[-1] + k)
            for mat, idx_all, prefix, total in outs:
                assert int(total) == sum(n) and prefix.tolist() == want_prefix
                assert torch.equal(mat[idx_all[: sum(n)].long()], want_rows)
            # partial outputs: rank r computes (r + 1) * row; the owner's sum is row * world * (world + 1) / 2
            ys = [(want_rows.float() * (r + 1)).bfloat16() for r in range(world)]
            for c, y, (_, _, prefix, _) in zip(comms, ys, outs):
                call("dyllm_tp_scatter_push", c._comm, ptr(y), width, world * slot_rows, ptr(prefix), stream_ptr(dev))
            for r, (c, k) in enumerate(zip(comms, cnts)):
                dest = torch.full((slot_rows + 8, width), 9.0, dtype=torch.bfloat16, device=dev)
                rows = torch.arange(slot_rows, dtype=torch.int32, device=dev) + 3       # scatter with an offset
                c.reduce_rows(width, k, 0, slot_rows, dest, rows)
                acc = torch.zeros(n[r], width, device=dev)
                for y in ys:
                    acc += y[want_prefix[r]: want_prefix[r + 1]].float()
                want = torch.full((slot_rows + 8, width), 9.0, dtype=torch.bfloat16, device=dev)
                want[3: 3 + n[r]] = acc.bfloat16()
                assert torch.equal(dest, want), f"round {round_} rank {r}"
        assert _lib.load().dyllm_device_status() == 0
    finally:
        for c in comms:
            c.close()
