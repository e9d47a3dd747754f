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

import os

import torch
from torch import nn

from . import ops
from .cache_manager import CacheManager
from .context import get_context, get_metadata
from .layers import (Attention, ColumnParallelLinear, KVParallelLinear, LLaDAMLP, LLaDAMoESparseBlock, RMSNorm,
                     RotaryEmbedding, RowParallelLinear, _world_size, attention_scope)


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
                 rope_scaling: tuple | None = None, threshold: float = 0.99, rotary_emb: RotaryEmbedding | None = None,
                 qk_layernorm: bool = False):
        super().__init__()
        with attention_scope():      # unsharded when every rank owns whole sequences
            self._build(hidden_size, num_heads, num_kv_heads, max_position, head_dim, rms_norm_eps, qkv_bias,
                        rope_theta, rope_scaling, threshold, rotary_emb, qk_layernorm)

    def _build(self, hidden_size, num_heads, num_kv_heads, max_position, head_dim, rms_norm_eps, qkv_bias, rope_theta,
               rope_scaling, threshold, rotary_emb, qk_layernorm):
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
        # per-head RMSNorm of the projected queries and keys (LLaDA-MoE; ref: lladamoe.py:175-176,195-207)
        self.q_norm = RMSNorm(self.head_dim, eps=rms_norm_eps) if qk_layernorm else None
        self.k_norm = RMSNorm(self.head_dim, eps=rms_norm_eps) if qk_layernorm else None
        self.k_cache = CacheManager(self.num_kv_heads * self.head_dim)
        assert rope_scaling is None
        self.rotary_emb = rotary_emb or RotaryEmbedding(self.head_dim, self.head_dim, max_position, rope_theta)
        self.attn = Attention(self.num_heads, self.head_dim, self.scaling, self.num_kv_heads, threshold)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor, salient_rows=None) -> torch.Tensor:
        """``salient_rows`` (sparse steps, optional): the normalised hidden rows of the step's salient tokens,
        packed in list order (``RMSNorm.forward_with_rows``); the K/V projection then reads them directly."""
        ctx, md = get_context(), get_metadata()
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        if not ctx.is_full and salient_rows is not None and _kv_overlap() and ctx.idx_salient_row.numel():
            return self._forward_sparse_overlapped(positions, hidden_states, salient_rows)
        q = self.q_proj(hidden_states).view(-1, H, D)
        if self.q_norm is not None:
            q = self.q_norm.forward_heads_(q)
        if ctx.is_full:
            kv = self.kv_proj(hidden_states)
            k, v = kv.split([self.kv_size, self.kv_size], dim=-1)
            k, v = k.reshape(-1, Hkv, D), v.reshape(-1, Hkv, D)
            if self.k_norm is not None:
                k = self.k_norm.forward_heads_(k.contiguous())
            q, k = self.rotary_emb(positions, q, k)
            self.k_cache.reset_full(k.flatten(-2, -1), md.running_seqs_tensor, seq_ids_list=md.running_seqs)
            o = self.attn(q, k, v)
        else:
            cap = ctx.idx_salient_row.numel()   # capacity; the live count may sit on the device
            n_dev, hint = ctx.num_salient_dev, ctx.salient_hint
            q = self.rotary_emb.rotate(positions, q)
            dv = None
            if cap:
                if salient_rows is not None:
                    k_new, v_new = self.kv_proj.forward_gathered(salient_rows, None, cap, n_dev, hint, split_col=self.kv_size)
                else:
                    k_new, v_new = self.kv_proj.forward_gathered(hidden_states, ctx.idx_salient_row32, cap, n_dev, hint,
                                                                 split_col=self.kv_size)
                rows_k = ctx.idx_salient_row_k if ctx.idx_salient_row_k is not None else ctx.idx_salient_row
                if self.k_norm is not None:
                    k_new = self.k_norm.forward_heads_(k_new.view(cap, Hkv, D), n_dev).view(cap, -1)
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


_side_streams: dict = {}


def _kv_overlap() -> bool:
    """The K/V branch of a sparse step (projection of the salient rows, K/V cache update) runs on a second stream
    beside the query projection, whose cuBLAS kernel leaves SMs idle in its last wave (DYLLM_KV_OVERLAP=0: one
    stream).  Not with this package's own GEMM for the all-row projections: the two would share its workspace."""
    from . import layers

    return os.environ.get("DYLLM_KV_OVERLAP", "1") != "0" and layers._projection_backend == "cublas"


def _forward_sparse_overlapped(self, positions, hidden_states, salient_rows):
    ctx, md = get_context(), get_metadata()
    H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
    cap = ctx.idx_salient_row.numel()
    n_dev, hint = ctx.num_salient_dev, ctx.salient_hint
    dev = hidden_states.device
    main = torch.cuda.current_stream(dev)
    side = _side_streams.get(dev)
    if side is None:
        side = _side_streams[dev] = torch.cuda.Stream(dev)
    # outputs of the side branch are allocated here, on the stream that uses them afterwards
    k_new = torch.empty((cap, self.kv_size), dtype=hidden_states.dtype, device=dev)
    v_new = torch.empty((cap, self.kv_size), dtype=hidden_states.dtype, device=dev)
    dv = torch.empty((cap, Hkv, D), dtype=hidden_states.dtype, device=dev)
    rows_k = ctx.idx_salient_row_k if ctx.idx_salient_row_k is not None else ctx.idx_salient_row
    side.wait_stream(main)
    with torch.cuda.stream(side):
        self.kv_proj.forward_gathered(salient_rows, None, cap, n_dev, hint, split_col=self.kv_size, out=(k_new, v_new))
        k3 = k_new.view(cap, Hkv, D)
        if self.k_norm is not None:
            k3 = self.k_norm.forward_heads_(k3, n_dev)
        ops.kv_cache_update(k3, v_new.view(cap, Hkv, D), rows_k, positions, ctx.idx_salient_row,
                            self.rotary_emb.cos_sin_cache.view(-1, D), ctx.cu_seqlens_k, self.k_cache.seq_start_gpu,
                            self.attn.v_cache.seq_start_gpu, md.running_seqs_tensor, self.k_cache.cache,
                            self.attn.v_cache.cache, n_dev, dv=dv)
    q = self.q_proj(hidden_states).view(-1, H, D)
    if self.q_norm is not None:
        q = self.q_norm.forward_heads_(q)
    q = self.rotary_emb.rotate(positions, q)
    main.wait_stream(side)
    k_full = self.k_cache.get_seqs(md.running_seqs_tensor, allow_view=True, seq_ids_list=md.running_seqs)
    o = self.attn(q, k_full.view(-1, Hkv, D), v_new.view(cap, Hkv, D), dv=dv)
    out = self.o_proj(o.flatten(-2, -1))
    self.k_cache.finish(md.finished_seqs)
    return out


LLaDAAttention._forward_sparse_overlapped = _forward_sparse_overlapped


def _input_norm(layer, hidden_states, residual):
    """First norm of a decoder layer (ref: llada.py:176-179).  In a sparse step the salient rows (the list the
    previous layer published) also come out packed for the K/V projection.  Returns (normalised, residual,
    packed salient rows or None)."""
    ctx = get_context()
    idx32 = None if ctx.is_full else ctx.idx_salient_row32
    if idx32 is not None and idx32.numel():
        y, res_out, packed = layer.input_layernorm.forward_with_rows(hidden_states, residual, idx32, ctx.num_salient_dev)
        if residual is None:      # first layer: the residual stream starts as the embedding
            res_out = hidden_states if hidden_states.dim() == 2 else hidden_states.reshape(-1, hidden_states.size(-1))
        return y, res_out, packed
    if residual is None:
        return layer.input_layernorm(hidden_states), hidden_states, None
    y, res_out = layer.input_layernorm(hidden_states, residual)
    return y, res_out, None


def _post_attention(layer, hidden_states, residual):
    """Second half of a decoder layer (ref: llada.py:183-186): residual add + RMSNorm, then the FFN on all rows
    (dense step) or on the salient rows (sparse step).  In a sparse step only the salient rows are normalised:
    they come out packed in list order and go straight into the FFN's GEMMs."""
    ctx = get_context()
    if ctx.is_full:
        hidden_states, residual = layer.post_attention_layernorm(hidden_states, residual)
        return layer.mlp(hidden_states), residual
    if ctx.idx_salient_row32 is not None and ctx.idx_salient_row32.numel():
        staged, residual = layer.post_attention_layernorm.forward_rows(hidden_states, residual, ctx.idx_salient_row32,
                                                                       ctx.num_salient_dev)
        return layer.mlp.forward_salient(staged, staged=True), residual
    hidden_states, residual = layer.post_attention_layernorm(hidden_states, residual)
    return layer.mlp.forward_salient(hidden_states), residual


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
        hidden_states, residual, packed = _input_norm(self, hidden_states, residual)
        hidden_states = self.self_attn(positions, hidden_states, packed)
        return _post_attention(self, hidden_states, residual)


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


# --------------------------------------------------------------------------------------------------
# Dream (ref: dyllm/model_executor/models/dream.py): grouped-query attention with biased q/k/v projections
# --------------------------------------------------------------------------------------------------
@dataclass
class DreamShape:
    """The fields of the reference's ``DreamConfig`` that the decoder reads (ref: dyllm/configs/dream.py);
    defaults are the Dream-7B shape."""

    hidden_size: int = 3584
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: int = 128
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    vocab_size: int = 152064
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    max_position_embeddings: int = 4096
    mask_token_id: int = 151666


class DreamAttention(LLaDAAttention):
    """ref: dyllm/model_executor/models/dream.py:46-144 (same data flow as the LLaDA block; qkv bias on)."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, max_position: int, head_dim: int,
                 rms_norm_eps: float = 1e-06, qkv_bias: bool = True, rope_theta: float = 1000000.0,
                 rope_scaling: tuple | None = None, threshold: float = 0.99, rotary_emb: RotaryEmbedding | None = None):
        super().__init__(hidden_size, num_heads, num_kv_heads, max_position, head_dim, rms_norm_eps, qkv_bias,
                         rope_theta, rope_scaling, threshold, rotary_emb)


class DreamMLP(LLaDAMLP):
    """ref: dyllm/model_executor/models/dream.py:26-43."""


class _DecoderLayer(nn.Module):
    """Residual wiring shared by the decoder layers (ref: llada.py:173-187, dream.py:168-182,
    lladamoe.py:266-280): add-RMSNorm, attention, add-RMSNorm, FFN on all rows (dense step) or on the salient
    rows through the step's index list (sparse step)."""

    def forward(self, positions, hidden_states, residual=None):
        hidden_states, residual, packed = _input_norm(self, hidden_states, residual)
        hidden_states = self.self_attn(positions, hidden_states, packed)
        return _post_attention(self, hidden_states, residual)


class DreamDecoderLayer(_DecoderLayer):
    def __init__(self, config: DreamShape, threshold: float, rotary_emb: RotaryEmbedding | None = None) -> None:
        super().__init__()
        self.self_attn = DreamAttention(
            hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
            num_kv_heads=config.num_key_value_heads, max_position=config.max_position_embeddings,
            rms_norm_eps=config.rms_norm_eps, qkv_bias=True, head_dim=getattr(config, "head_dim", None),
            rope_theta=getattr(config, "rope_theta", 1000000.0), threshold=threshold, rotary_emb=rotary_emb)
        self.mlp = DreamMLP(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)


class _DecoderStack(nn.Module):
    def _finish_init(self) -> None:
        # every layer's output goes straight into an RMSNorm of this package, which reads a block of every
        # sequence out of the FFN-output cache in place
        for layer in self.layers:
            layer.mlp.cache_update.block_view = True

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        hidden_states = self.embed_tokens(input_ids)
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(positions, hidden_states, residual)
        hidden_states, _ = self.norm(hidden_states, residual)
        return hidden_states


class DreamModel(_DecoderStack):
    def __init__(self, config: DreamShape, threshold: float):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        rope = RotaryEmbedding(config.head_dim, config.head_dim, config.max_position_embeddings, config.rope_theta)
        self.layers = nn.ModuleList([DreamDecoderLayer(config, threshold, rope) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self._finish_init()


class DreamForDLM(nn.Module):
    """ref: dyllm/model_executor/models/dream.py:201-234.  ``shift_logits``: the reference's Dream sampler reads
    the logits of the row before each candidate (sampler.py, ``DreamSampler.adjust_logits``)."""

    shift_logits = True

    def __init__(self, config: DreamShape, threshold: float):
        super().__init__()
        self.config = config
        self.model = DreamModel(config, threshold)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    def forward(self, input_ids, positions):
        return self.model(input_ids, positions)

    def compute_logits(self, hidden_states):
        return self.lm_head(hidden_states)


# --------------------------------------------------------------------------------------------------
# LLaDA-MoE (ref: dyllm/model_executor/models/lladamoe.py): per-head q/k RMSNorm, mixture-of-experts FFN
# --------------------------------------------------------------------------------------------------
@dataclass
class LLaDAMoEShape:
    """The fields of the LLaDA-MoE configuration that the decoder reads; defaults are LLaDA-MoE-7B-A1B."""

    hidden_size: int = 2048
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    head_dim: int = 128
    num_experts: int = 64
    num_experts_per_tok: int = 8
    expert_intermediate_size: int = 1024
    norm_topk_prob: bool = False
    num_hidden_layers: int = 16
    vocab_size: int = 157184
    rms_norm_eps: float = 1e-5
    rope_theta: float = 50000.0
    max_position_embeddings: int = 4096
    qk_layernorm: bool = True
    attention_bias: bool = False
    mask_token_id: int = 156895


class LLaDAMoEAttention(LLaDAAttention):
    """ref: dyllm/model_executor/models/lladamoe.py:145-242."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, max_position: int, head_dim: int,
                 rms_norm_eps: float = 1e-05, qkv_bias: bool = False, rope_theta: float = 50000.0,
                 rope_scaling: tuple | None = None, qk_layernorm: bool = True, threshold: float = 0.99,
                 rotary_emb: RotaryEmbedding | None = None):
        super().__init__(hidden_size, num_heads, num_kv_heads, max_position, head_dim, rms_norm_eps, qkv_bias,
                         rope_theta, rope_scaling, threshold, rotary_emb, qk_layernorm=qk_layernorm)


class LLaDAMoEDecoderLayer(_DecoderLayer):
    def __init__(self, config: LLaDAMoEShape, threshold: float, expert_parallel_size: int = 1,
                 rotary_emb: RotaryEmbedding | None = None) -> None:
        super().__init__()
        head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.self_attn = LLaDAMoEAttention(
            hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
            num_kv_heads=config.num_key_value_heads, max_position=config.max_position_embeddings, head_dim=head_dim,
            rms_norm_eps=config.rms_norm_eps, qkv_bias=getattr(config, "attention_bias", False),
            rope_theta=getattr(config, "rope_theta", 50000), qk_layernorm=bool(getattr(config, "qk_layernorm", False)),
            threshold=threshold, rotary_emb=rotary_emb)
        self.mlp = LLaDAMoESparseBlock(config, expert_parallel_size)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)


class LLaDAMoEModel(_DecoderStack):
    def __init__(self, config: LLaDAMoEShape, threshold: float, expert_parallel_size: int = 1):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        rope = RotaryEmbedding(config.head_dim, config.head_dim, config.max_position_embeddings, config.rope_theta)
        self.layers = nn.ModuleList([LLaDAMoEDecoderLayer(config, threshold, expert_parallel_size, rope)
                                     for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self._finish_init()


class LLaDAMoEForDLM(nn.Module):
    """ref: dyllm/model_executor/models/lladamoe.py:301-315.  ``expert_parallel_size`` is 1 (every expert
    sharded over the tensor-parallel ranks) or the tensor-parallel size (whole experts per rank)."""

    def __init__(self, config: LLaDAMoEShape, threshold: float, expert_parallel_size: int = 1):
        super().__init__()
        self.config = config
        self.model = LLaDAMoEModel(config, threshold, expert_parallel_size)
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
