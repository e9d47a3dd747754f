"""Per-sequence activation cache with the reference's ``CacheManager`` interface
(ref: dyllm/engine/cache_manager.py:11-181): one ``[rows, hidden_dim]`` tensor, ``seq_id -> start/len``
maps on the host and on the device, and the copy kernels of :mod:`dyllm_b200.cache`.

Differences in mechanism, not in behaviour: storage grows geometrically inside a preallocated arena
instead of by ``torch.cat`` per new sequence, and ``get_seqs`` / ``get_seqs_block`` can hand out a view
of the cache (``allow_view=True``) when the running sequences lie back to back in batch order, which
removes the full-tensor copy the reference makes on every call.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .cache import get_block_cuda, get_seqs_cuda, reset_block_cuda, reset_full_cuda, scatter_update_cuda
from .context import get_context


class CacheManager:
    def __init__(self, hidden_dim: int, max_num_seqs: int = 16384, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device = torch.device("cuda")):
        self._seq_to_start: dict[int, int] = {}
        self._seq_to_len: dict[int, int] = {}
        self.hidden_dim = hidden_dim
        self.dtype = dtype
        self.max_num_seqs = max_num_seqs
        self.device = device
        self._arena = torch.empty((0, hidden_dim), dtype=dtype, device=device)
        self._rows = 0
        self.seq_start_gpu = torch.full((max_num_seqs,), -1, dtype=torch.long, device=device)
        self.seq_len_gpu = torch.zeros((max_num_seqs,), dtype=torch.long, device=device)

    # the reference exposes the storage as ``cache``
    @property
    def cache(self) -> torch.Tensor:
        return self._arena[: self._rows]

    @property
    def num_total_seqs(self) -> int:
        return len(self._seq_to_start)

    def select_seq_range(self, seq_id: int):
        start = self._seq_to_start[seq_id]
        return start, start + self._seq_to_len[seq_id]

    def _reserve(self, extra_rows: int) -> None:
        need = self._rows + extra_rows
        if need > self._arena.size(0):
            cap = max(need, 2 * self._arena.size(0), 1024)
            arena = torch.empty((cap, self.hidden_dim), dtype=self.dtype, device=self.device)
            if self._rows:
                arena[: self._rows].copy_(self._arena[: self._rows])
            self._arena = arena

    # ------------------------------------------------------------------ reads
    def contiguous_start(self, seq_ids_list: Optional[List[int]]) -> int:
        """First cache row if the given sequences lie back to back in this order, else -1."""
        if not seq_ids_list:
            return -1
        start = self._seq_to_start.get(seq_ids_list[0], -1)
        pos = start
        for s in seq_ids_list:
            if self._seq_to_start.get(s, -2) != pos:
                return -1
            pos += self._seq_to_len[s]
        return start

    def get_seqs(self, seq_ids: torch.Tensor, allow_view: bool = False,
                 seq_ids_list: Optional[List[int]] = None) -> torch.Tensor:
        ctx = get_context()
        total = max(ctx.total_seqlen, ctx.total_seqlen_k)
        if allow_view:
            start = self.contiguous_start(seq_ids_list)
            if start >= 0 and ctx.cu_seqlens_k is not None and start + ctx.total_seqlen_k <= self._rows:
                return self._arena[start : start + ctx.total_seqlen_k]
        return get_seqs_cuda(self.cache, self.seq_start_gpu, ctx.cu_seqlens_k, seq_ids, total)

    def get_seqs_block(self, seq_ids: torch.Tensor, allow_view: bool = False,
                       seq_ids_list: Optional[List[int]] = None) -> torch.Tensor:
        """The last ``len_q`` rows of every running sequence, packed.  With ``allow_view``, when the
        sequences lie back to back in batch order and have equal lengths, a strided
        ``[batch, len_q, hidden]`` view of the cache is returned instead of a copy."""
        ctx = get_context()
        if allow_view and ctx.context_lens_cpu and ctx.cu_seqlens_q_cpu:
            lens = ctx.context_lens_cpu
            cu_q = ctx.cu_seqlens_q_cpu
            n = len(lens)
            len_k, len_q = lens[0], cu_q[1] - cu_q[0]
            uniform = all(l == len_k for l in lens) and all(cu_q[i + 1] - cu_q[i] == len_q for i in range(n))
            start = self.contiguous_start(seq_ids_list) if uniform else -1
            if start >= 0 and start + n * len_k <= self._rows and 0 < len_q <= len_k:
                return self._arena[start : start + n * len_k].view(n, len_k, self.hidden_dim)[:, len_k - len_q :, :]
        return get_block_cuda(self.cache, self.seq_start_gpu, ctx.cu_seqlens_k, ctx.cu_seqlens_q, seq_ids,
                              ctx.total_seqlen)

    def get_start_indices(self, seq_ids: List[int]) -> torch.Tensor:
        return torch.tensor([self._seq_to_start[s] for s in seq_ids], dtype=torch.long)

    # ------------------------------------------------------------------ allocation
    def add_seq(self, c: torch.Tensor, seq_id: int) -> None:
        n = c.size(0)
        self._reserve(n)
        start = self._rows
        self._arena[start : start + n].copy_(c)
        self._rows += n
        self._seq_to_start[seq_id] = start
        self._seq_to_len[seq_id] = n
        self.seq_start_gpu[seq_id] = start
        self.seq_len_gpu[seq_id] = n

    def reset_seq(self, c: torch.Tensor, seq_id: int) -> None:
        if seq_id in self._seq_to_start:
            start, end = self.select_seq_range(seq_id)
            if end - start == c.size(0):
                self._arena[start:end] = c
                return
            self.remove_seq(seq_id)
        self.add_seq(c, seq_id)

    def remove_seq(self, seq_id: int) -> None:
        if seq_id not in self._seq_to_start:
            return
        start, end = self.select_seq_range(seq_id)
        length = end - start
        if end < self._rows:
            self._arena[start : self._rows - length] = self._arena[end : self._rows].clone()
        self._rows -= length
        moved = []
        for other, other_start in self._seq_to_start.items():
            if other != seq_id and other_start > start:
                self._seq_to_start[other] = other_start - length
                moved.append(other)
        if moved:
            ids = torch.tensor(moved, device=self.device, dtype=torch.long)
            self.seq_start_gpu[ids] -= length
        del self._seq_to_start[seq_id]
        del self._seq_to_len[seq_id]
        self.seq_start_gpu[seq_id] = -1
        self.seq_len_gpu[seq_id] = 0

    def clear(self) -> None:
        """Forgets every sequence (the arena is kept for reuse)."""
        self._seq_to_start.clear()
        self._seq_to_len.clear()
        self._rows = 0
        self.seq_start_gpu.fill_(-1)
        self.seq_len_gpu.zero_()

    def _allocate_new_seqs(self, new_ids: List[int], new_lengths: List[int]) -> None:
        total = sum(new_lengths)
        if total == 0:
            return
        self._reserve(total)
        starts, pos = [], self._rows
        for n in new_lengths:
            starts.append(pos)
            pos += n
        self._rows = pos
        ids = torch.tensor(new_ids, device=self.device, dtype=torch.long)
        self.seq_start_gpu[ids] = torch.tensor(starts, device=self.device, dtype=torch.long)
        self.seq_len_gpu[ids] = torch.tensor(new_lengths, device=self.device, dtype=torch.long)
        for sid, st, n in zip(new_ids, starts, new_lengths):
            self._seq_to_start[sid] = st
            self._seq_to_len[sid] = n

    # ------------------------------------------------------------------ writes
    def reset_full(self, c: torch.Tensor, seq_ids: torch.Tensor, seq_ids_list: Optional[List[int]] = None) -> None:
        ctx = get_context()
        if not c.is_contiguous():
            c = c.contiguous()
        if seq_ids_list is None:
            seq_ids_list = seq_ids.cpu().tolist()
        new_ids, new_lens = [], []
        for i, sid in enumerate(seq_ids_list):
            known = self._seq_to_len.get(sid)
            if known is not None and known != ctx.context_lens_cpu[i]:
                # the id is being reused for a sequence of another length: its old range cannot hold it
                self.remove_seq(sid)
                known = None
            if known is None:
                new_ids.append(sid)
                new_lens.append(ctx.context_lens_cpu[i])
        if new_ids:
            self._allocate_new_seqs(new_ids, new_lens)
        reset_full_cuda(self.cache, c, self.seq_start_gpu, ctx.cu_seqlens_q, seq_ids, ctx.total_seqlen)

    def reset_block(self, c: torch.Tensor, seq_ids: torch.Tensor) -> None:
        ctx = get_context()
        if not c.is_contiguous():
            c = c.contiguous()
        reset_block_cuda(self.cache, c, self.seq_start_gpu, ctx.cu_seqlens_k, ctx.cu_seqlens_q, seq_ids,
                         ctx.total_seqlen)

    def scatter_update(self, seq_ids: torch.Tensor, row_idx: torch.Tensor, new: torch.Tensor,
                       num_rows_dev: Optional[torch.Tensor] = None) -> None:
        ctx = get_context()
        scatter_update_cuda(self.cache, new, row_idx, ctx.cu_seqlens_k, self.seq_start_gpu, seq_ids, num_rows_dev)

    def finish(self, finished_seq_ids: List[int]) -> bool:
        if len(finished_seq_ids) == 0:
            return False
        for sid in sorted(finished_seq_ids, key=lambda x: self._seq_to_start.get(x, -1), reverse=True):
            self.remove_seq(sid)
        return True
