"""Drop-in for the routing and expert functions of the reference's
``dyllm/model_executor/layers/fused_moe.py`` (Triton there; hand-written sm_100a kernels here)."""

from __future__ import annotations

import torch

from . import ops


def moe_gate(hidden_states: torch.Tensor, router_weight: torch.Tensor, top_k: int, router_scale=None,
             per_expert_scale=None, renormalize: bool = True, rms_norm_eps=None):
    """ref: fused_moe.py:375-407.  The Gemma-only options (router_scale, per_expert_scale, rms_norm_eps) belong
    to a model family outside this package and are rejected."""
    if router_scale is not None or per_expert_scale is not None or rms_norm_eps is not None:
        raise RuntimeError("moe_gate: router_scale / per_expert_scale / rms_norm_eps are not supported")
    w, ids = ops.moe_route(hidden_states, router_weight, top_k, renormalize)
    return w.to(hidden_states.dtype), ids


def fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                  topk_ids: torch.Tensor, activation: str = "gelu", block_m: int = 64) -> torch.Tensor:
    """ref: fused_moe.py:269-335.  ``activation`` must be "silu" (the LLaDA-MoE experts)."""
    if activation != "silu":
        raise RuntimeError('fused_experts: only activation="silu" is built')
    if hidden_states.size(0) == 0:
        return hidden_states.new_empty((0, hidden_states.size(1)))
    return ops.moe_ffn(hidden_states, w1, w2, topk_weights.float().contiguous(), topk_ids.to(torch.int32).contiguous())


__all__ = ["moe_gate", "fused_experts"]
