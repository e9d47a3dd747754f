"""ctypes binding of ``libdyllm_b200.so`` (the C ABI declared in ``include/dyllm_b200.h``).

There is no fallback: if the shared library is missing or a call returns a non-zero status a
``RuntimeError`` is raised, as the reference's pybind11 extensions do through ``TORCH_CHECK``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libdyllm_b200.so")

P, I, F, Z = c_void_p, c_int, c_float, c_size_t

# name -> (restype, argtypes); mirrors include/dyllm_b200.h one to one.
SIGNATURES: dict[str, tuple] = {
    "dyllm_version": (I, []),
    "dyllm_last_error": (c_char_p, []),
    "dyllm_device_status": (I, []),
    "dyllm_context_stats": (I, [P, P, P, I, I, I, P]),
    "dyllm_cosine_mask": (I, [P, P, I, F, P]),
    "dyllm_salient_select_workspace_bytes": (Z, [I]),
    "dyllm_salient_select": (I, [P, I, F, P, I, P, P, P, P, P, P, P, P, Z, P]),
    "dyllm_salient_select_static": (I, [P, I, F, P, I, P, P, P, P, P, P, P, P]),
    "dyllm_salient_select_static_max_rows": (I, []),
    "dyllm_fused_offset": (I, [P, P, P, P, I, P, I, P]),
    "dyllm_cache_get_seqs": (I, [P, P, P, P, P, I, I, I, I, P]),
    "dyllm_cache_get_block": (I, [P, P, P, P, P, P, I, I, I, I, P]),
    "dyllm_cache_reset_full": (I, [P, P, P, P, P, I, I, I, I, P]),
    "dyllm_cache_reset_block": (I, [P, P, P, P, P, P, I, I, I, I, P]),
    "dyllm_cache_scatter_update": (I, [P, P, P, P, I, P, P, I, I, P, I, I, P]),
    "dyllm_gathered_linear_workspace_bytes": (Z, [I, I, I]),
    "dyllm_gathered_linear": (I, [P, I, I, c_int64, P, I, P, I, P, I, P, c_int64, P, c_int64, I, P, P, P, Z, I, I, P]),
    "dyllm_swiglu_ffn_workspace_bytes": (Z, [I, I, I]),
    "dyllm_swiglu_ffn": (I, [P, I, I, c_int64, P, I, P, I, P, P, I, P, c_int64, P, P, Z, I, I, P]),
    "dyllm_cache_dest_rows": (I, [P, P, P, P, I, I, P, P, P]),
    "dyllm_moe_route": (I, [P, I, I, c_int64, P, I, P, P, I, I, I, P, P, P]),
    "dyllm_moe_ffn_workspace_bytes": (Z, [I, I, I, I, I]),
    "dyllm_moe_ffn": (I, [P, I, I, c_int64, P, I, P, I, P, P, I, P, P, I, I, I, P, c_int64, P, P, Z, P]),
    "dyllm_attention_sparse_workspace_bytes": (Z, [I, I]),
    "dyllm_attention_sparse_varlen": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, P, P, I, P, P, P, F, P, Z, I, P, P, I, P]),
    "dyllm_attention_salient_rows": (I, [P, P, P, P, P, I, I, I, I, I, I, I, P, P, P]),
    "dyllm_attention_kernel_info": (I, [I, P]),
    "dyllm_delta_v_update": (I, [P, P, P, I, P, I, P, P]),
    "dyllm_add_rms_norm": (I, [P, P, P, F, P, P, I, I, P]),
    "dyllm_add_rms_norm_segmented": (I, [P, I, c_int64, P, P, F, P, P, I, I, P]),
    "dyllm_add_rms_norm_rows": (I, [P, I, c_int64, P, P, F, P, P, I, I, P, I, P, P, P]),
    "dyllm_head_rms_norm": (I, [P, P, F, I, P, I, I, P]),
    "dyllm_rope_neox": (I, [P, P, P, P, I, P, I, I, I, P]),
    "dyllm_row_confidence": (I, [P, I, I, c_int64, P, P, P]),
    "dyllm_confidence_unmask": (I, [P, P, P, I, c_int64, P, I, I, I, I, I, c_int64, P, P, P]),
    "dyllm_kv_cache_update": (I, [P, P, P, P, P, P, I, P, P, P, P, I, I, P, I, I, P, P, P, P]),
    "dyllm_tp_comm_create": (I, [I, I, Z, P]),
    "dyllm_tp_comm_region_bytes": (Z, [P]),
    "dyllm_tp_comm_region": (P, [P]),
    "dyllm_tp_comm_ipc_handle": (I, [P, P]),
    "dyllm_tp_comm_open_ipc": (I, [P, P]),
    "dyllm_tp_comm_open_local": (I, [P, P]),
    "dyllm_tp_comm_set_wait_ms": (I, [P, I]),
    "dyllm_tp_comm_destroy": (I, [P]),
    "dyllm_tp_push_rows": (I, [P, P, I, I, P, I, P]),
    "dyllm_tp_reduce_rows": (I, [P, I, I, P, I, P, c_int64, P, P]),
    "dyllm_tp_allreduce_rows": (I, [P, P, I, I, P, I, P, c_int64, P, P]),
    "dyllm_tp_gather_rows": (I, [P, P, I, I, c_int64, P, I, P, P, P, P, P]),
    "dyllm_tp_gather_push": (I, [P, P, I, I, c_int64, P, I, P, P]),
    "dyllm_tp_gather_finish": (I, [P, I, P, P, P, P]),
    "dyllm_tp_comm_data": (P, [P]),
    "dyllm_tp_scatter_push": (I, [P, P, I, I, P, P]),
    "dyllm_tp_push_f32": (I, [P, P, I, P]),
    "dyllm_tp_reduce_f32": (I, [P, P, I, P]),
    "dyllm_tp_allreduce_f32": (I, [P, P, I, P]),
}

# kernels of this library launched by one call of each entry point (for launch accounting)
KERNELS_PER_CALL = {
    "dyllm_context_stats": 1, "dyllm_cosine_mask": 1, "dyllm_salient_select": 1, "dyllm_salient_select_static": 1,
    "dyllm_fused_offset": 1,
    "dyllm_cache_get_seqs": 1, "dyllm_cache_get_block": 1, "dyllm_cache_reset_full": 1, "dyllm_cache_reset_block": 1,
    "dyllm_cache_scatter_update": 1, "dyllm_gathered_linear": 2, "dyllm_swiglu_ffn": 3, "dyllm_cache_dest_rows": 1, "dyllm_moe_route": 1, "dyllm_moe_ffn": 5,
    "dyllm_attention_sparse_varlen": 2, "dyllm_attention_salient_rows": 2, "dyllm_delta_v_update": 1,
    "dyllm_add_rms_norm": 1, "dyllm_add_rms_norm_segmented": 1, "dyllm_add_rms_norm_rows": 1, "dyllm_head_rms_norm": 1, "dyllm_rope_neox": 1, "dyllm_row_confidence": 1, "dyllm_confidence_unmask": 1, "dyllm_kv_cache_update": 1,
    "dyllm_tp_push_rows": 1, "dyllm_tp_reduce_rows": 1, "dyllm_tp_allreduce_rows": 2, "dyllm_tp_push_f32": 1,
    "dyllm_tp_reduce_f32": 1, "dyllm_tp_allreduce_f32": 2, "dyllm_tp_gather_rows": 2, "dyllm_tp_gather_push": 1,
    "dyllm_tp_gather_finish": 1, "dyllm_tp_scatter_push": 1,
}
launch_count = 0

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dyllm_b200.build` "
                "(dyllm_b200 has no CPU or PyTorch fallback)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def ptr(t: torch.Tensor | None) -> int | None:
    """Device address of a tensor (None -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr(device: torch.device | None = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def call(name: str, *args) -> None:
    """Calls a status-returning entry point and raises RuntimeError on failure."""
    global launch_count
    lib = load()
    rc = getattr(lib, name)(*args)
    launch_count += KERNELS_PER_CALL.get(name, 0)
    if rc != 0:
        msg = lib.dyllm_last_error().decode(errors="replace")
        raise RuntimeError(f"{name} failed with status {rc}: {msg}")


def require_cuda(t: torch.Tensor, name: str, dtype: torch.dtype | None = None, dim: int | None = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise RuntimeError(f"{name} must be {dim}-D, got {t.dim()}-D")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
