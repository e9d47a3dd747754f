"""Drop-in for the reference's ``dyllm.attention_ops`` extension module
(ref: dyllm/csrc/attention/attention.cpp:197-208): same function names, argument order and error type.
"""

from __future__ import annotations

import torch

from ._lib import call, ptr, stream_ptr


def _check_i32_vector(t: torch.Tensor, name: str, device) -> None:
    if not (t.is_cuda and t.device == device):
        raise RuntimeError(f"{name} must be on {device}")
    if t.dtype != torch.int32:
        raise RuntimeError(f"{name} must be int32")
    if t.dim() != 1 or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous 1D tensor")


def fused_offset_launch(idxs, num_idxs, cu_promptlens, cu_salientlens, out_tensor, max_threads: int) -> None:
    """ref: dyllm/csrc/attention/attention_aux_kernels.cu:173-200."""
    device = idxs.device
    _check_i32_vector(idxs, "idxs", device)
    _check_i32_vector(num_idxs, "num_idxs", device)
    _check_i32_vector(cu_promptlens, "cu_promptlens", device)
    _check_i32_vector(cu_salientlens, "cu_salientlens", device)
    if num_idxs.numel() != 1:
        raise RuntimeError("num_idxs must contain exactly one element")
    if cu_promptlens.numel() != cu_salientlens.numel():
        raise RuntimeError("cu_promptlens and cu_salientlens must have the same length")
    if not (out_tensor.is_cuda and out_tensor.device == device and out_tensor.dtype == torch.int64
            and out_tensor.dim() == 1 and out_tensor.is_contiguous()):
        raise RuntimeError(f"out_tensor must be a contiguous int64 CUDA vector on {device}")
    if not (0 <= max_threads <= out_tensor.numel()):
        raise RuntimeError("max_threads must fit out_tensor")
    if max_threads == 0:
        return
    call("dyllm_fused_offset", ptr(idxs), ptr(num_idxs), ptr(cu_promptlens), ptr(cu_salientlens),
         cu_promptlens.numel() - 1, ptr(out_tensor), int(max_threads), stream_ptr(device))


__all__ = ["fused_offset_launch"]
