"""LLaDA decoder layer / model with the reference's module structure
(ref: dyllm/model_executor/models/llada.py:46-202) on top of :mod:`dyllm_b200.layers`.

The sparse branch of ``LLaDAAttention.forward`` differs from the reference in mechanism only: the K/V
projection of the salient rows is a gathered tcgen05 GEMM (no ``hidden_states[idx]`` copy), the rotary
embedding is applied to the salient K rows alone (the reference rotates a zero-padded full-length
buffer and then reads back the same rows), and the full K / V / context tensors are views of the
per-sequence caches when the batch lies contiguously in them.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from . import ops
from .cache_manager import CacheManager
from .context import get_context, get_metadata
from .layers import (Attention, ColumnParallelLinear, KVParallelLinear, LLaDAMLP, RMSNorm, RotaryEmbedding,
                     RowParallelLinear, _world_size)


@dataclass
class LLaDAShape:
    """The fields of the reference's ``LLaDAConfig`` that the decoder reads (ref: dyllm/configs/llada.py)."""

    hidden_size: int = 4096
    num_attention_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    mlp_hidden_size: int = 12288
    num_hidden_layers: int = 32
    vocab_size: int = 126464
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_sequence_length: int = 4096
    mask_token_id: int = 126336


class LLaDAAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, max_position: int, head_dim: int,
                 rms_norm_eps: float = 1e-06, qkv_bias: bool = False, rope_theta: float = 10000.0,
                 rope_scaling: tuple | None = None, threshold: float = 0.99, rotary_emb: RotaryEmbedding | None = None):
        super().__init__()
        tp = _world_size()
        self.total_num_heads = num_heads
        self.num_heads = num_heads // tp
        self.total_num_kv_heads = num_kv_heads
        self.num_kv_heads = num_kv_heads // tp
        self.head_dim = head_dim or hidden_size // num_heads
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.scaling = self.head_dim ** -0.5
        self.q_proj = ColumnParallelLinear(hidden_size, self.total_num_heads * self.head_dim, bias=qkv_bias)
        self.kv_proj = KVParallelLinear(hidden_size, self.head_dim, self.total_num_kv_heads, bias=qkv_bias)
        self.o_proj = RowParallelLinear(self.total_num_heads * self.head_dim, hidden_size, bias=False)
        self.k_cache = CacheManager(self.num_kv_heads * self.head_dim)
        assert rope_scaling is None
        self.rotary_emb = rotary_emb or RotaryEmbedding(self.head_dim, self.head_dim, max_position, rope_theta)
        self.attn = Attention(self.num_heads, self.head_dim, self.scaling, self.num_kv_heads, threshold)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        ctx, md = get_context(), get_metadata()
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        q = self.q_proj(hidden_states).view(-1, H, D)
        if ctx.is_full:
            kv = self.kv_proj(hidden_states)
            k, v = kv.split([self.kv_size, self.kv_size], dim=-1)
            k, v = k.reshape(-1, Hkv, D), v.reshape(-1, Hkv, D)
            q, k = self.rotary_emb(positions, q, k)
            self.k_cache.reset_full(k.flatten(-2, -1), md.running_seqs_tensor, seq_ids_list=md.running_seqs)
            o = self.attn(q, k, v)
        else:
            cap = ctx.idx_salient_row.numel()   # capacity; the live count may sit on the device
            n_dev, hint = ctx.num_salient_dev, ctx.salient_hint
            q = self.rotary_emb.rotate(positions, q)
            dv = None
            if cap:
                k_new, v_new = self.kv_proj.forward_gathered(hidden_states, ctx.idx_salient_row32, cap, n_dev, hint,
                                                             split_col=self.kv_size)
                rows_k = ctx.idx_salient_row_k if ctx.idx_salient_row_k is not None else ctx.idx_salient_row
                v_new = v_new.view(cap, Hkv, D)
                # rotary embedding of the new keys, K-cache scatter, delta-V and V-cache update in one launch
                dv = ops.kv_cache_update(k_new.view(cap, Hkv, D), v_new, rows_k, positions, ctx.idx_salient_row,
                                         self.rotary_emb.cos_sin_cache.view(-1, D), ctx.cu_seqlens_k,
                                         self.k_cache.seq_start_gpu, self.attn.v_cache.seq_start_gpu,
                                         md.running_seqs_tensor, self.k_cache.cache, self.attn.v_cache.cache, n_dev)
            else:
                v_new = torch.empty((0, Hkv, D), dtype=q.dtype, device=q.device)
            k_full = self.k_cache.get_seqs(md.running_seqs_tensor, allow_view=True, seq_ids_list=md.running_seqs)
            o = self.attn(q, k_full.view(-1, Hkv, D), v_new, dv=dv)
        out = self.o_proj(o.flatten(-2, -1))
        self.k_cache.finish(md.finished_seqs)
        return out


class LLaDADecoderLayer(nn.Module):
    def __init__(self, config: LLaDAShape, threshold: float, rotary_emb: RotaryEmbedding | None = None) -> None:
        super().__init__()
        self.self_attn = LLaDAAttention(
            hidden_size=config.hidden_size, num_heads=config.num_attention_heads, num_kv_heads=config.n_kv_heads,
            max_position=config.max_sequence_length, rms_norm_eps=config.rms_norm_eps,
            head_dim=getattr(config, "head_dim", None), rope_theta=getattr(config, "rope_theta", 1000000),
            threshold=threshold, rotary_emb=rotary_emb)
        self.mlp = LLaDAMLP(hidden_size=config.hidden_size, intermediate_size=config.mlp_hidden_size)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, positions, hidden_states, residual=None):
        if residual is None:
            hidden_states, residual = self.input_layernorm(hidden_states), hidden_states
        else:
            hidden_states, residual = self.input_layernorm(hidden_states, residual)
        hidden_states = self.self_attn(positions, hidden_states)
        ctx = get_context()
        hidden_states, residual = self.post_attention_layernorm(hidden_states, residual)
        if ctx.is_full:
            hidden_states = self.mlp(hidden_states)
        else:
            hidden_states = self.mlp.forward_salient(hidden_states)
        return hidden_states, residual


class LLaDAModel(nn.Module):
    def __init__(self, config: LLaDAShape, threshold: float):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        rope = RotaryEmbedding(config.head_dim, config.head_dim, config.max_sequence_length, config.rope_theta)
        self.layers = nn.ModuleList([LLaDADecoderLayer(config, threshold, rope) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        # every layer's output goes straight into an RMSNorm of this package (the next layer's or the final
        # one), which reads a block of every sequence out of the FFN-output cache in place
        for layer in self.layers:
            layer.mlp.cache_update.block_view = True

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        hidden_states = self.embed_tokens(input_ids)
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(positions, hidden_states, residual)
        hidden_states, _ = self.norm(hidden_states, residual)
        return hidden_states


class LLaDAForDLM(nn.Module):
    def __init__(self, config: LLaDAShape, threshold: float):
        super().__init__()
        self.config = config
        self.model = LLaDAModel(config, threshold)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    def forward(self, input_ids, positions):
        return self.model(input_ids, positions)

    def compute_logits(self, hidden_states):
        return self.lm_head(hidden_states)


def init_weights_(module: nn.Module, seed: int = 0, std: float = 0.02) -> None:
    """Seeded random-init stand-in for a checkpoint: N(0, std) for every matrix and bias of the UNSHARDED
    model, drawn in parameter order, ones for the norm weights.  Under tensor / expert parallelism every rank
    draws the same unsharded tensors and keeps its shard through the layers' loaders, so the sharded model
    computes the same function as the single-GPU one (and one rank draws exactly the single-GPU values)."""
    gens: dict = {}
    owner = {id(p): m for m in module.modules() for p in m.parameters(recurse=False)}
    for name, p in module.named_parameters():
        if p.dim() < 2 and not name.endswith("bias"):
            p.data.fill_(1.0)
            continue
        g = gens.get(p.device)
        if g is None:
            g = gens[p.device] = torch.Generator(device=p.device).manual_seed(seed)
        m = owner[id(p)]
        full_shape = m.full_shape(p) if hasattr(m, "full_shape") else tuple(p.shape)
        if full_shape == tuple(p.shape):
            p.data.normal_(0.0, std, generator=g)
        else:
            full = torch.empty(full_shape, dtype=p.dtype, device=p.device).normal_(0.0, std, generator=g)
            m.load_full(p, full)
            del full
