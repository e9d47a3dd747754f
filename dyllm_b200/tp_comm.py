"""Tensor-parallel exchange of the small per-layer tensors over peer memory (the C ABI's ``dyllm_tp_*``).

One :class:`TpComm` per rank.  The regions are allocated by the library at set-up and mapped into every rank
with CUDA IPC handles that travel over ``torch.distributed``; after that an exchange is two kernel launches
on the current stream (they capture into CUDA graphs) and never touches the host.

ref: dyllm/distributed/parallel_state.py:52-66 (12-byte-per-token statistics),
dyllm/model_executor/layers/linear.py:216-220 and dyllm/model_executor/models/lladamoe.py:103-104,141
(``[S, hidden]`` outputs of the row-parallel down projection / the experts).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ._lib import call, load, ptr, require_cuda, stream_ptr

DEFAULT_SLOT_BYTES = 64 << 20     # 8192 rows of 4096 bf16 per exchange and rank


class TpComm:
    def __init__(self, rank: int, world: int, slot_bytes: int = DEFAULT_SLOT_BYTES):
        self.rank, self.world, self.slot_bytes = rank, world, int(slot_bytes)
        handle = ctypes.c_void_p()
        call("dyllm_tp_comm_create", rank, world, self.slot_bytes, ctypes.byref(handle))
        self._comm = handle

    # ------------------------------------------------------------------ set-up
    @classmethod
    def from_process_group(cls, device: torch.device, slot_bytes: int = DEFAULT_SLOT_BYTES) -> "TpComm":
        """Collective over the default process group: every rank creates its region, the 64-byte IPC
        handles are all-gathered, every rank maps the others' regions, and a barrier makes sure that all
        regions are zeroed and mapped before the first exchange."""
        rank, world = dist.get_rank(), dist.get_world_size()
        comm = cls(rank, world, slot_bytes)
        buf = (ctypes.c_ubyte * 64)()
        call("dyllm_tp_comm_ipc_handle", comm._comm, ctypes.cast(buf, ctypes.c_void_p))
        mine = torch.tensor(list(buf), dtype=torch.uint8, device=device)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        handles = bytes(torch.cat(gathered).cpu().tolist())
        call("dyllm_tp_comm_open_ipc", comm._comm, ctypes.c_char_p(handles))
        torch.cuda.synchronize(device)
        dist.barrier()
        return comm

    @classmethod
    def emulated_world(cls, world: int, slot_bytes: int) -> list["TpComm"]:
        """``world`` communicators inside one process on the current device (tests: the ranks' kernels are
        then launched one after the other on one stream, every push before the first reduce)."""
        comms = [cls(r, world, slot_bytes) for r in range(world)]
        lib = load()
        regions = (ctypes.c_void_p * world)(*[lib.dyllm_tp_comm_region(c._comm) for c in comms])
        for c in comms:
            call("dyllm_tp_comm_open_local", c._comm, regions)
        return comms

    def set_wait_ms(self, ms: int) -> None:
        call("dyllm_tp_comm_set_wait_ms", self._comm, int(ms))

    def close(self) -> None:
        if self._comm is not None:
            call("dyllm_tp_comm_destroy", self._comm)
            self._comm = None

    # ------------------------------------------------------------------ exchanges
    def max_rows(self, width: int) -> int:
        return self.slot_bytes // (2 * width)

    def push_rows(self, src: torch.Tensor, count_dev: torch.Tensor | None, row_offset: int, max_rows: int) -> None:
        call("dyllm_tp_push_rows", self._comm, src.data_ptr() + row_offset * src.stride(0) * 2, src.size(1), max_rows,
             ptr(count_dev), row_offset, stream_ptr(src.device))

    def reduce_rows(self, width: int, count_dev, row_offset: int, max_rows: int, out: torch.Tensor,
                    out_row_map: torch.Tensor | None) -> None:
        call("dyllm_tp_reduce_rows", self._comm, width, max_rows, ptr(count_dev), row_offset, ptr(out), out.stride(0),
             ptr(out_row_map), stream_ptr(out.device))

    def all_reduce_rows(self, src: torch.Tensor, count_dev: torch.Tensor | None = None, out: torch.Tensor | None = None,
                        out_row_map: torch.Tensor | None = None) -> torch.Tensor:
        """SUM over the ranks of the first ``*count_dev`` rows of ``src [capacity, width]`` (bf16, contiguous),
        written to ``out[map[m]]`` (default: back into ``src``).  A capacity above the slot size is exchanged
        in several rounds; rounds past the live count move no data."""
        require_cuda(src, "src", torch.bfloat16, 2)
        if out is None:
            out = src
        cap, width = src.size(0), src.size(1)
        step = max(1, self.max_rows(width))
        for off in range(0, cap, step):
            n = min(step, cap - off)
            self.push_rows(src, count_dev, off, n)
            self.reduce_rows(width, count_dev, off, n, out, out_row_map)
        return out

    def all_reduce_f32_(self, t: torch.Tensor) -> torch.Tensor:
        """In-place SUM all-reduce of an fp32 tensor (the ``[rows, 3]`` statistics)."""
        require_cuda(t, "t", torch.float32)
        call("dyllm_tp_allreduce_f32", self._comm, ptr(t), t.numel(), stream_ptr(t.device))
        return t

    # ------------------------------------------------------------------ sequence-sharded layout
    def data_matrix(self, width: int, device: torch.device) -> torch.Tensor:
        """The data area of the local region as a bf16 ``[2 * world * slot_rows, width]`` matrix (both buffer
        parities; the row numbers a gather returns point into it).  The tensor aliases library memory."""
        slot_rows = self.slot_bytes // (2 * width)
        if slot_rows * 2 * width != self.slot_bytes:
            raise RuntimeError(f"slot of {self.slot_bytes} bytes is not a whole number of rows of {width} bf16")
        key = (width, device)
        cached = getattr(self, "_matrices", None)
        if cached is None:
            cached = self._matrices = {}
        if key not in cached:
            rows = 2 * self.world * slot_rows
            base = load().dyllm_tp_comm_data(self._comm)
            cached[key] = _device_view(base, rows, width, device)
        return cached[key]

    def gather_rows(self, x: torch.Tensor, idx: torch.Tensor | None, count_dev: torch.Tensor | None, max_rows: int):
        """All ranks' rows ``x[idx[:count]]`` -> (matrix, idx_all int32 [world * slot_rows], prefix int32
        [world + 1], total int32 [1]); see ``dyllm_tp_gather_rows``."""
        require_cuda(x, "x", torch.bfloat16, 2)
        width, dev = x.size(1), x.device
        mat = self.data_matrix(width, dev)
        cap = self.world * (self.slot_bytes // (2 * width))
        idx_all = torch.empty((cap,), dtype=torch.int32, device=dev)
        prefix = torch.empty((self.world + 1,), dtype=torch.int32, device=dev)
        total = torch.empty((1,), dtype=torch.int32, device=dev)
        call("dyllm_tp_gather_rows", self._comm, ptr(x), x.size(0), width, x.stride(0), ptr(idx), int(max_rows),
             ptr(count_dev), ptr(idx_all), ptr(prefix), ptr(total), stream_ptr(dev))
        return mat, idx_all, prefix, total

    def scatter_reduce_rows(self, y: torch.Tensor, prefix: torch.Tensor, max_total: int, count_dev, max_rows: int,
                            out: torch.Tensor, out_row_map: torch.Tensor | None) -> None:
        """Partial output rows ``y`` (one per gathered row) go back to their owners, which add the ranks'
        partials in rank order and write the sums to ``out[map[m]]``."""
        require_cuda(y, "y", torch.bfloat16, 2)
        call("dyllm_tp_scatter_push", self._comm, ptr(y), y.size(1), int(max_total), ptr(prefix), stream_ptr(y.device))
        self.reduce_rows(y.size(1), count_dev, 0, int(max_rows), out, out_row_map)


def _device_view(address: int, rows: int, width: int, device: torch.device) -> torch.Tensor:
    """A bf16 ``[rows, width]`` tensor over device memory owned by the library (no copy, no ownership)."""

    class _Holder:
        __cuda_array_interface__ = {"shape": (rows * width,), "typestr": "<i2", "data": (address, False), "version": 3}

    return torch.as_tensor(_Holder(), device=device).view(torch.bfloat16).view(rows, width)
