"""Per-step global state shared by the layer classes: the same ``Context`` / ``MetaData`` carriers and
accessor functions as the reference (ref: dyllm/utils/context.py:6-109, dyllm/utils/metadata.py:6-28).

Fields the DiffusionGemma engine adds in the reference are left out.  Two fields are added for the
device-resident selection: ``idx_salient_row32`` (the int32 copy the kernels consume) and
``max_salient_per_seq`` (host upper bound used to size grids).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class Context:
    is_full: bool = False
    cu_seqlens_q: Optional[torch.Tensor] = None
    cu_seqlens_q_cpu: Optional[List] = None
    cu_seqlens_k: Optional[torch.Tensor] = None
    cu_promptlens: Optional[torch.Tensor] = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    context_lens: Optional[torch.Tensor] = None
    context_lens_cpu: Optional[List] = None
    cu_updatedlens: Optional[torch.Tensor] = None
    cu_salientlens: Optional[torch.Tensor] = None
    idx_salient_row: Optional[torch.Tensor] = None
    idx_salient_row_k: Optional[torch.Tensor] = None
    idx_updated_row: Optional[torch.Tensor] = None
    total_seqlen_k: int = 0
    total_seqlen: int = 0
    positions_k: Optional[torch.Tensor] = None
    idx_salient_row32: Optional[torch.Tensor] = None
    max_salient_per_seq: int = 0
    # Device-resident selection: when num_salient_dev is set, the idx_salient_row* tensors are
    # capacity-sized buffers whose first *num_salient_dev entries are live; salient_hint is the host's
    # estimate of that count (used only to shape launches).
    num_salient_dev: Optional[torch.Tensor] = None
    salient_hint: int = 0
    # When positive, every layer uses this row-count estimate instead of reading its previous count back
    # (a step captured into a CUDA graph cannot depend on host-side state).
    fixed_hint: int = 0

    def salient_rows(self):
        """(idx_salient_row, idx_salient_row_k or None) trimmed to the live length (synchronises)."""
        if self.num_salient_dev is None:
            return self.idx_salient_row, self.idx_salient_row_k
        n = int(self.num_salient_dev.item())
        k = self.idx_salient_row_k[:n] if self.idx_salient_row_k is not None else None
        return self.idx_salient_row[:n], k


_CONTEXT = Context()


def get_context() -> Context:
    return _CONTEXT


def set_context(is_full, **kwargs) -> None:
    global _CONTEXT
    _CONTEXT = Context(is_full=is_full, **kwargs)


def reset_context() -> None:
    global _CONTEXT
    _CONTEXT = Context()


@dataclass
class MetaData:
    all_seqs: List[int] = field(default_factory=list)
    running_seqs: List[int] = field(default_factory=list)
    finished_seqs: List[int] = field(default_factory=list)
    running_seqs_tensor: Optional[torch.Tensor] = None


_METADATA = MetaData()


def get_metadata() -> MetaData:
    return _METADATA


def set_metadata(all_seqs, running_seqs, finished_seqs) -> None:
    global _METADATA
    _METADATA = MetaData(all_seqs=all_seqs, running_seqs=running_seqs, finished_seqs=finished_seqs)


def reset_metadata() -> None:
    global _METADATA
    _METADATA = MetaData()
