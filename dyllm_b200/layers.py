"""Host-side mirror of the reference's ``model_executor`` layer interfaces for the saliency path.

Same class names, constructor arguments and ``forward`` signatures as the reference
(ref: dyllm/model_executor/layers/{attention,linear,layernorm,rotary_embedding,activations,mlp_cache_manage}.py,
dyllm/distributed/parallel_state.py, dyllm/model_executor/models/llada.py); the bodies call the sm_100a
kernels through the C ABI instead of flash-attn / cuBLAS-on-gathered-copies / the reference's extension.
Projections that run on every row (q_proj, o_proj, lm_head) stay ``F.linear``.
"""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from . import ops, profiling
from .attention_ops import attention_salient_rows, attention_sparse_varlen
from .cache_manager import CacheManager
from .context import get_context, get_metadata


# --------------------------------------------------------------------------------------------------
# distributed helpers (ref: dyllm/distributed/parallel_state.py)
# --------------------------------------------------------------------------------------------------
_replicated_depth = 0     # > 0 while modules are being built (or run) as if there were a single rank


def _world_size() -> int:
    if _replicated_depth:
        return 1
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _rank() -> int:
    if _replicated_depth:
        return 0
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


@contextlib.contextmanager
def replicated():
    """Modules built inside this scope are unsharded: every rank holds their complete weights."""
    global _replicated_depth
    _replicated_depth += 1
    try:
        yield
    finally:
        _replicated_depth -= 1


# How the work of a step is spread over the ranks.
#   "tensor"    the reference's layout (dyllm/model_executor/layers/linear.py): every rank sees every row;
#               attention heads and FFN columns are sharded; three all-reduces per sparse layer.
#   "sequence"  every rank owns whole sequences of the batch and runs the all-row work (projections, norms,
#               attention, statistics, selection, caches) for them alone with replicated attention weights;
#               only the FFN / expert weights are sharded, and only the salient rows travel: they are
#               gathered from all ranks, pushed through the sharded FFN, and the partial outputs go back to
#               the rows' owners.  No [T_q, hidden] all-reduce and no statistics all-reduce exist.
_layout = "tensor"


def set_layout(name: str) -> None:
    global _layout
    if name not in ("tensor", "sequence"):
        raise ValueError(f"unknown layout {name!r}")
    _layout = name


def get_layout() -> str:
    return _layout


def attention_scope():
    """Scope in which a model builds its attention block: unsharded under the sequence layout."""
    return replicated() if _layout == "sequence" else contextlib.nullcontext()


def sequence_sharded() -> bool:
    return _layout == "sequence" and _world_size() > 1


# A step driver that captures the launches of a step into CUDA graphs installs a hook here: every SUM
# all-reduce of the layers goes through it, so that the driver can close the graph it is capturing, issue
# the collective outside any capture and open the next graph.
_all_reduce_hook = None


def set_all_reduce_hook(hook) -> None:
    global _all_reduce_hook
    _all_reduce_hook = hook


def all_reduce_sum(t: torch.Tensor) -> None:
    """In-place SUM all-reduce over the tensor-parallel group (NCCL)."""
    if _all_reduce_hook is not None:
        _all_reduce_hook(t)
    else:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)


# The peer-memory exchange (tp_comm.TpComm) of this rank, when one has been set up: it carries the two small
# all-reduces of a sparse layer whose size depends on the device-side salient count (statistics, FFN rows).
_tp_comm = None


def set_tp_comm(comm) -> None:
    global _tp_comm
    _tp_comm = comm


def get_tp_comm():
    return _tp_comm


def all_reduce_stats(stats: torch.Tensor) -> None:
    """SUM all-reduce of the ``[T_q, 3]`` fp32 statistics (12 bytes per token)."""
    if _tp_comm is not None and stats.is_cuda:
        _tp_comm.all_reduce_f32_(stats)
    else:
        all_reduce_sum(stats)


def all_reduce_salient_rows(y: torch.Tensor, count_dev, cache_manager, seq_ids, rows_k) -> None:
    """SUM all-reduce of the live rows of the compact ``[capacity, hidden]`` FFN output ``y`` and scatter of
    the sums into the FFN-output cache (ref: linear.py:216-220 followed by mlp_cache_manage.py:24-40).  With
    the peer-memory exchange only the live rows cross NVLink and the scatter is the reduce kernel's store;
    without it the dead rows are cleared and the whole buffer goes through NCCL."""
    ctx = get_context()
    if _tp_comm is not None:
        dest = ops.cache_dest_rows(rows_k, ctx.cu_seqlens_k, cache_manager.seq_start_gpu, seq_ids, count_dev)
        _tp_comm.all_reduce_rows(y, count_dev, out=cache_manager.cache, out_row_map=dest)
        return
    if count_dev is not None:
        dead = torch.arange(y.size(0), device=y.device).unsqueeze(1) >= count_dev
        y.masked_fill_(dead, 0.0)          # rows past the live count were never written
    all_reduce_sum(y)
    cache_manager.scatter_update(seq_ids, rows_k, y, count_dev)


def tensor_parallel_cosine_mask(stats: torch.Tensor, threshold: float) -> torch.Tensor:
    """SUM all-reduce of the 12-byte-per-token statistics, then ``cosine < threshold``.

    ref: dyllm/distributed/parallel_state.py:52-66.  The decision itself runs in the mask kernel when the
    statistics live on a GPU.
    """
    if _world_size() > 1:
        all_reduce_stats(stats)
    return ops.cosine_mask(stats, threshold)      # raises unless the statistics are fp32 [rows, 3] on a GPU


def _gathered_ffn(ffn_shard, x: torch.Tensor, idx32, cap_local: int, count_dev, hint: int, out=None, out_row_map=None,
                  region=None):
    """FFN of the sequence-sharded layout: the rows ``x[idx32[:count]]`` of every rank are gathered on all ranks
    (peer-memory stores), ``ffn_shard(matrix, idx_all, capacity, total_dev, hint)`` runs this rank's weight shard
    over all of them, and each partial output row returns to the rank that owns the row, which adds the ranks'
    partials in rank order and writes the sums to ``out[map[m]]`` (default: a packed ``[cap_local, hidden]``
    tensor, which is returned)."""
    comm = get_tp_comm()
    if comm is None:
        raise RuntimeError("the sequence-sharded layout needs the peer-memory exchange (layers.set_tp_comm)")
    # timed regions (when region timing is on): the two exchanges apart from the GEMMs between them
    row_bytes = float((hint or cap_local) * x.size(1) * 2 * comm.world)
    with profiling.region("ffn_gather_exchange", 0.0, row_bytes):
        mat, idx_all, prefix, total = comm.gather_rows(x, idx32, count_dev, cap_local)
    cap_total = idx_all.numel()
    with profiling.region(*region) if region else contextlib.nullcontext():
        y = ffn_shard(mat, idx_all, cap_total, total, hint * comm.world if hint else 0)
    if out is None:
        out = torch.empty((cap_local, x.size(1)), dtype=x.dtype, device=x.device)
    with profiling.region("ffn_scatter_exchange", 0.0, row_bytes):
        comm.scatter_reduce_rows(y, prefix, cap_total, count_dev, cap_local, out, out_row_map)
    return out


# Which GEMM runs the all-row projections (q_proj, o_proj, dense-step kv_proj): "cublas" (F.linear; plain library
# GEMMs, the default) or "tcgen05" (this package's gathered GEMM on every row, 256-row tiles).
_projection_backend = "cublas"


def set_projection_backend(name: str) -> None:
    global _projection_backend
    if name not in ("cublas", "tcgen05"):
        raise ValueError(f"unknown projection backend {name!r}")
    _projection_backend = name


def _project(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    if _projection_backend == "tcgen05" and x.is_cuda and x.dim() == 2 and x.size(0) > 0:
        y = ops.gathered_linear(x.contiguous(), weight, None, num_rows=x.size(0), rows_hint=x.size(0))
        if bias is not None:
            y += bias
        return y
    return F.linear(x, weight, bias)


def divide(numerator: int, denominator: int) -> int:
    assert numerator % denominator == 0
    return numerator // denominator


# --------------------------------------------------------------------------------------------------
# linear layers (ref: dyllm/model_executor/layers/linear.py)
# --------------------------------------------------------------------------------------------------
class LinearBase(nn.Module):
    def __init__(self, input_size: int, output_size: int, bias: bool = False, tp_dim: int | None = None):
        super().__init__()
        self.tp_dim = tp_dim
        self.tp_rank = _rank()
        self.tp_size = _world_size()
        self.weight = nn.Parameter(torch.empty(output_size, input_size))
        self.weight.weight_loader = self.weight_loader
        if bias:
            self.bias = nn.Parameter(torch.empty(output_size))
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

    def full_shape(self, param: nn.Parameter) -> tuple:
        """Shape of the unsharded checkpoint tensor behind ``param``."""
        shape = list(param.shape)
        if self.tp_dim is not None and param.dim() > self.tp_dim and not (param.dim() == 1 and self.tp_dim == 1):
            shape[self.tp_dim] *= self.tp_size
        return tuple(shape)

    def load_full(self, param: nn.Parameter, full: torch.Tensor) -> None:
        """Keeps this rank's shard of an unsharded tensor (what the loaders do shard by shard)."""
        self.weight_loader(param, full)


class ReplicatedLinear(LinearBase):
    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(loaded_weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias)


class ColumnParallelLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        super().__init__(input_size, divide(output_size, _world_size()), bias, 0)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        shard = param.data.size(self.tp_dim)
        param.data.copy_(loaded_weight.narrow(self.tp_dim, self.tp_rank * shard, shard))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _project(x, self.weight, self.bias)

    def forward_gathered(self, x: torch.Tensor, idx32: torch.Tensor | None, num_rows: int, num_rows_dev=None,
                         rows_hint: int = 0, split_col: int = 0, out=None):
        """``self(x[idx])`` on the tcgen05 GEMM; ``num_rows`` may be a capacity with the live count on the
        device.  ``idx32`` None: ``x`` already holds the rows packed in list order.  With ``split_col`` the
        output columns are returned as two tensors (K and V halves); ``out`` may bring them (a pair)."""
        n_out = self.weight.size(0)
        if out is not None:
            out, out2 = out if split_col else (out, None)
        elif split_col:
            out = torch.empty((num_rows, split_col), dtype=x.dtype, device=x.device)
            out2 = torch.empty((num_rows, n_out - split_col), dtype=x.dtype, device=x.device)
        else:
            out, out2 = torch.empty((num_rows, n_out), dtype=x.dtype, device=x.device), None
        ops.gathered_linear(x, self.weight, idx32, num_rows=num_rows, num_rows_dev=num_rows_dev, rows_hint=rows_hint,
                            out=out, out2=out2, split_col=split_col)
        if self.bias is not None:
            out += self.bias[: out.size(1)]
            if out2 is not None:
                out2 += self.bias[out.size(1):]
        return (out, out2) if split_col else out


class MergedColumnParallelLinear(ColumnParallelLinear):
    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False):
        self.output_sizes = output_sizes
        super().__init__(input_size, sum(output_sizes), bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: int):
        offset = sum(self.output_sizes[:loaded_shard_id]) // self.tp_size
        size = self.output_sizes[loaded_shard_id] // self.tp_size
        dst = param.data.narrow(self.tp_dim, offset, size)
        dst.copy_(loaded_weight.chunk(self.tp_size, self.tp_dim)[self.tp_rank])

    def load_full(self, param: nn.Parameter, full: torch.Tensor) -> None:
        pos = 0
        for i, size in enumerate(self.output_sizes):
            self.weight_loader(param, full.narrow(0, pos, size), i)
            pos += size


class KVParallelLinear(ColumnParallelLinear):
    def __init__(self, hidden_size: int, head_size: int, total_num_kv_heads: int, bias: bool = False):
        self.head_size = head_size
        self.num_kv_heads = divide(total_num_kv_heads, _world_size())
        super().__init__(hidden_size, 2 * total_num_kv_heads * head_size, bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: str):
        assert loaded_shard_id in ("k", "v")
        size = self.num_kv_heads * self.head_size
        offset = 0 if loaded_shard_id == "k" else size
        dst = param.data.narrow(self.tp_dim, offset, size)
        dst.copy_(loaded_weight.chunk(self.tp_size, self.tp_dim)[self.tp_rank])

    def load_full(self, param: nn.Parameter, full: torch.Tensor) -> None:
        half = full.size(0) // 2
        self.weight_loader(param, full.narrow(0, 0, half), "k")
        self.weight_loader(param, full.narrow(0, half, half), "v")


class RowParallelLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        super().__init__(divide(input_size, _world_size()), output_size, bias, 1)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        if param.dim() == 1:
            param.data.copy_(loaded_weight)
            return
        shard = param.data.size(self.tp_dim)
        param.data.copy_(loaded_weight.narrow(self.tp_dim, self.tp_rank * shard, shard))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = _project(x, self.weight, self.bias if self.tp_rank == 0 else None)
        if self.tp_size > 1:
            all_reduce_sum(y)
        return y


# --------------------------------------------------------------------------------------------------
# norm, rotary embedding, activation (ref: layernorm.py:6-53, rotary_embedding.py:8-67, activations.py)
# --------------------------------------------------------------------------------------------------
class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        # bf16 on a GPU only (ops.add_rms_norm raises otherwise).  A 3-D input is a view of equal blocks of
        # rows inside a cache: it is read in place and the outputs are packed.
        if x.dim() == 2:
            x = x.contiguous()
        return ops.add_rms_norm(x, self.weight, self.eps, residual)

    def forward_heads_(self, x: torch.Tensor, num_rows_dev=None) -> torch.Tensor:
        """In place over the last dimension of ``x [rows, heads, head_dim]`` (this module's size is head_dim):
        the per-head q / k norm (ref: dyllm/model_executor/models/lladamoe.py:195-207)."""
        return ops.head_rms_norm_(x, self.weight, self.eps, num_rows_dev)

    def forward_rows(self, x: torch.Tensor, residual: torch.Tensor, sel_idx32: torch.Tensor, sel_count_dev=None):
        """Residual add of every row, normalised values of the listed rows only, packed in list order:
        ``(y_sel, new_residual)``.  What a sparse step needs of the post-attention norm: its output feeds the
        FFN of the salient rows and nothing else (ref: dyllm/model_executor/models/llada.py:183-185)."""
        if x.dim() == 2:
            x = x.contiguous()
        y_sel, res_out, _ = ops.add_rms_norm_rows(x, self.weight, self.eps, residual, sel_idx32, sel_count_dev)
        return y_sel, res_out

    def forward_with_rows(self, x: torch.Tensor, residual: torch.Tensor | None, sel_idx32: torch.Tensor, sel_count_dev=None):
        """The full norm plus the listed rows packed in list order: ``(y, new_residual or None, y_sel)``.  What a
        sparse step needs of the input norm: every row feeds q_proj, the salient rows also feed kv_proj
        (ref: dyllm/model_executor/models/llada.py:103,108)."""
        if x.dim() == 2:
            x = x.contiguous()
        y_sel, res_out, y_all = ops.add_rms_norm_rows(x, self.weight, self.eps, residual, sel_idx32, sel_count_dev,
                                                      all_rows=True)
        return y_all, res_out, y_sel


class RotaryEmbedding(nn.Module):
    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float) -> None:
        super().__init__()
        assert rotary_dim == head_size
        inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
        t = torch.arange(max_position_embeddings, dtype=torch.float)
        freqs = torch.einsum("i,j -> ij", t, inv_freq)
        # kept out of the module's buffers: the table stays fp32 when the model is cast to bf16
        self._cos_sin_cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1).unsqueeze_(1)

    @property
    def cos_sin_cache(self) -> torch.Tensor:
        return self._cos_sin_cache

    def rotate(self, positions: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        if self._cos_sin_cache.device != x.device:
            self._cos_sin_cache = self._cos_sin_cache.to(x.device)
        # in place on the freshly projected [rows, heads, 128] bf16 tensor (the kernel wrapper raises otherwise)
        return ops.rope_neox_(x.contiguous(), positions, self._cos_sin_cache.view(-1, x.size(-1)))

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        return self.rotate(positions, query), self.rotate(positions, key)


class SiluAndMul(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a, b = x.chunk(2, -1)
        return F.silu(a) * b


# --------------------------------------------------------------------------------------------------
# FFN-output cache (ref: dyllm/model_executor/layers/mlp_cache_manage.py)
# --------------------------------------------------------------------------------------------------
class MLPcache(nn.Module):
    def __init__(self, hidden_dim: int = 0):
        super().__init__()
        self.cache_manager = CacheManager(hidden_dim=hidden_dim)
        # When set (by a model whose next operation is this package's RMSNorm), response-only steps return
        # a strided [batch, len_q, hidden] view of the cache instead of a packed copy.
        self.block_view = False

    def result(self) -> torch.Tensor:
        """The full ``[T_q, hidden]`` activation of the step after the cache has been updated."""
        ctx, md = get_context(), get_metadata()
        if not ctx.is_full and ctx.idx_salient_row_k is not None:
            # may be a strided [batch, len_q, hidden] view of the cache (the norm that follows reads it in place)
            return self.cache_manager.get_seqs_block(md.running_seqs_tensor, allow_view=self.block_view,
                                                     seq_ids_list=md.running_seqs)
        return self.cache_manager.get_seqs(md.running_seqs_tensor, allow_view=True, seq_ids_list=md.running_seqs)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx, md = get_context(), get_metadata()
        if ctx.is_full:
            self.cache_manager.reset_full(x, md.running_seqs_tensor, seq_ids_list=md.running_seqs)
        else:
            rows = ctx.idx_salient_row_k if ctx.idx_salient_row_k is not None else ctx.idx_salient_row
            self.cache_manager.scatter_update(md.running_seqs_tensor, rows, x)
        self.cache_manager.finish(md.finished_seqs)
        return self.result()


class LLaDAMLP(nn.Module):
    """ref: dyllm/model_executor/models/llada.py:26-43."""

    def __init__(self, hidden_size: int, intermediate_size: int) -> None:
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(hidden_size, [intermediate_size] * 2, bias=False)
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, bias=False)
        self.act_fn = SiluAndMul()
        self.cache_update = MLPcache(hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Reference calling convention: ``x`` holds the rows to process (all rows of a dense step, the
        gathered salient rows of a sparse step)."""
        if sequence_sharded():
            return self.cache_update(_gathered_ffn(self._ffn_shard, x, None, x.size(0), None, 0))
        y = ops.swiglu_ffn(x, self.gate_up_proj.weight, self.down_proj.weight)
        if self.down_proj.tp_size > 1:
            all_reduce_sum(y)
        return self.cache_update(y)

    def _ffn_shard(self, mat, idx_all, cap_total, total_dev, hint):
        return ops.swiglu_ffn(mat, self.gate_up_proj.weight, self.down_proj.weight, idx_all, num_rows=cap_total,
                              num_rows_dev=total_dev, rows_hint=hint)

    def forward_salient(self, hidden: torch.Tensor, staged: bool = False) -> torch.Tensor:
        """Sparse step on the full ``[T_q, hidden]`` activation: the salient rows are read through the step's
        index list (live count on the device) and the down projection scatters straight into the
        FFN-output cache (replaces gather_rows_2D + MLP + scatter_update,
        dyllm/model_executor/models/llada.py:184-186).  With ``staged`` the input already holds the salient
        rows alone, packed in list order (``RMSNorm.forward_rows``)."""
        ctx, md = get_context(), get_metadata()
        cap = ctx.idx_salient_row.numel()
        n_dev, hint = ctx.num_salient_dev, ctx.salient_hint
        cm = self.cache_update.cache_manager
        idx32 = None if staged else ctx.idx_salient_row32
        if cap:
            rows_k = ctx.idx_salient_row_k if ctx.idx_salient_row_k is not None else ctx.idx_salient_row
            rows = hint or cap
            width, inter = hidden.size(1), self.down_proj.weight.size(1)
            # algorithmic bytes: the three weight matrices (this rank's shards) once, the rows in and out
            nbytes = 3.0 * width * inter * 2 + 2.0 * rows * width * 2
            if sequence_sharded():
                dest = ops.cache_dest_rows(rows_k, ctx.cu_seqlens_k, cm.seq_start_gpu, md.running_seqs_tensor, n_dev)
                world = _world_size()
                _gathered_ffn(self._ffn_shard, hidden, idx32, cap, n_dev, hint, out=cm.cache, out_row_map=dest,
                              region=("swiglu_ffn", 6.0 * rows * world * width * inter, nbytes))
            elif self.down_proj.tp_size > 1:
                with profiling.region("swiglu_ffn", 6.0 * rows * width * inter, nbytes):
                    y = ops.swiglu_ffn(hidden, self.gate_up_proj.weight, self.down_proj.weight, idx32,
                                       num_rows=cap, num_rows_dev=n_dev, rows_hint=hint)
                with profiling.region("ffn_all_reduce", 0.0, 2.0 * rows * width * 2):
                    all_reduce_salient_rows(y, n_dev, cm, md.running_seqs_tensor, rows_k)
            else:
                dest = ops.cache_dest_rows(rows_k, ctx.cu_seqlens_k, cm.seq_start_gpu, md.running_seqs_tensor, n_dev)
                with profiling.region("swiglu_ffn", 6.0 * rows * width * inter, nbytes):
                    ops.swiglu_ffn(hidden, self.gate_up_proj.weight, self.down_proj.weight, idx32,
                                   num_rows=cap, num_rows_dev=n_dev, rows_hint=hint, out=cm.cache, out_row_map=dest)
        cm.finish(md.finished_seqs)
        return self.cache_update.result()


class LLaDAMoESparseBlock(nn.Module):
    """Sparse MoE feed-forward: softmax top-k router (no renormalisation unless the config asks for it),
    SiLU experts, expert tensor parallelism or expert parallelism with an all-reduce combine.
    ref: dyllm/model_executor/models/lladamoe.py:48-142."""

    def __init__(self, config, expert_parallel_size: int = 1) -> None:
        super().__init__()
        self.num_experts = config.num_experts
        self.top_k = config.num_experts_per_tok
        self.renormalize = bool(getattr(config, "norm_topk_prob", False))
        H, I = config.hidden_size, config.expert_intermediate_size
        self.hidden_size, self.intermediate_size = H, I
        world = _world_size()
        if expert_parallel_size not in (1, world):
            raise ValueError("expert_parallel_size must be 1 (expert tensor parallelism) or "
                             f"tensor_parallel_size ({world}); got {expert_parallel_size}")
        self.ep_size = expert_parallel_size
        self.ep_rank = _rank() if expert_parallel_size > 1 else 0
        self.expert_parallel = self.ep_size > 1
        if self.expert_parallel:
            if self.num_experts % self.ep_size != 0:
                raise ValueError(f"num_experts ({self.num_experts}) must be divisible by EP size ({self.ep_size})")
            self.num_local_experts = self.num_experts // self.ep_size
            self.expert_start = self.ep_rank * self.num_local_experts
            self.local_intermediate_size = I
        else:
            if I % world != 0:
                raise ValueError(f"expert_intermediate_size ({I}) must be divisible by TP size ({world})")
            self.num_local_experts = self.num_experts
            self.expert_start = 0
            self.local_intermediate_size = I // world
        self.gate = ReplicatedLinear(H, self.num_experts, bias=False)
        self.gate_up_proj = nn.Parameter(torch.empty(self.num_local_experts, 2 * self.local_intermediate_size, H))
        self.down_proj = nn.Parameter(torch.empty(self.num_local_experts, H, self.local_intermediate_size))
        self.cache_update = MLPcache(H)

    def full_shape(self, param: nn.Parameter) -> tuple:
        """Shape of the unsharded expert tensor behind ``gate_up_proj`` / ``down_proj``."""
        if param is self.gate_up_proj:
            return (self.num_experts, 2 * self.intermediate_size, self.hidden_size)
        if param is self.down_proj:
            return (self.num_experts, self.hidden_size, self.intermediate_size)
        return tuple(param.shape)

    def load_full(self, param: nn.Parameter, full: torch.Tensor) -> None:
        """This rank's share of an unsharded expert tensor: a contiguous range of experts under expert
        parallelism, else a slice of every expert's intermediate dimension (gate and up rows separately)
        (ref: dyllm/model_executor/models/lladamoe.py:69-83)."""
        if self.expert_parallel:
            param.data.copy_(full.narrow(0, self.expert_start, self.num_local_experts))
            return
        world, rank, I, Il = _world_size(), _rank(), self.intermediate_size, self.local_intermediate_size
        if param is self.gate_up_proj:
            param.data[:, :Il].copy_(full[:, rank * Il:(rank + 1) * Il])
            param.data[:, Il:].copy_(full[:, I + rank * Il: I + (rank + 1) * Il])
        elif param is self.down_proj:
            param.data.copy_(full[:, :, rank * Il:(rank + 1) * Il])
        else:
            param.data.copy_(full)

    def _experts(self, x, idx32, num_rows, n_dev, hint, out=None, out_row_map=None):
        w, ids = ops.moe_route(x, self.gate.weight, self.top_k, self.renormalize, idx32, num_rows, n_dev)
        return ops.moe_ffn(x, self.gate_up_proj, self.down_proj, w, ids, self.expert_start, idx32, num_rows, n_dev,
                           hint, out, out_row_map)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Reference calling convention: ``x`` holds the rows to process."""
        if sequence_sharded():
            return self.cache_update(_gathered_ffn(self._experts, x, None, x.size(0), None, 0))
        y = self._experts(x, None, x.size(0), None, 0)
        if _world_size() > 1:
            all_reduce_sum(y)
        return self.cache_update(y)

    def forward_salient(self, hidden: torch.Tensor, staged: bool = False) -> torch.Tensor:
        """Sparse step on the full activation: rows through the salient list, results scattered into the
        FFN-output cache (at TP/EP > 1 after the all-reduce).  With ``staged`` the input already holds the
        salient rows alone, packed in list order."""
        ctx, md = get_context(), get_metadata()
        cap = ctx.idx_salient_row.numel()
        n_dev, hint = ctx.num_salient_dev, ctx.salient_hint
        cm = self.cache_update.cache_manager
        idx32 = None if staged else ctx.idx_salient_row32
        if cap:
            rows_k = ctx.idx_salient_row_k if ctx.idx_salient_row_k is not None else ctx.idx_salient_row
            if sequence_sharded():
                dest = ops.cache_dest_rows(rows_k, ctx.cu_seqlens_k, cm.seq_start_gpu, md.running_seqs_tensor, n_dev)
                _gathered_ffn(self._experts, hidden, idx32, cap, n_dev, hint, out=cm.cache, out_row_map=dest)
            elif _world_size() > 1:
                y = self._experts(hidden, idx32, cap, n_dev, hint)
                all_reduce_salient_rows(y, n_dev, cm, md.running_seqs_tensor, rows_k)
            else:
                dest = ops.cache_dest_rows(rows_k, ctx.cu_seqlens_k, cm.seq_start_gpu, md.running_seqs_tensor, n_dev)
                self._experts(hidden, idx32, cap, n_dev, hint, out=cm.cache, out_row_map=dest)
        cm.finish(md.finished_seqs)
        return self.cache_update.result()


# --------------------------------------------------------------------------------------------------
# attention (ref: dyllm/model_executor/layers/attention.py)
# --------------------------------------------------------------------------------------------------
_dense_attention_backend = "sdpa"


def set_dense_attention_backend(name: str) -> None:
    """"sdpa" (the default): the dense steps' attention runs on torch's scaled_dot_product_attention, as the
    reference runs it on flash-attn; "tcgen05": on this package's exact-attention kernel with every row listed
    (built for few query rows per sequence: 0.24 ms against 0.07 ms at 16 x 512 rows, 32 heads)."""
    global _dense_attention_backend
    if name not in ("tcgen05", "sdpa"):
        raise ValueError(f"unknown dense attention backend {name!r}")
    _dense_attention_backend = name


_all_rows_cache: dict = {}


def _dense_attention(q, k, v, ctx, scale):
    """Non-causal varlen attention of a dense step (ref: dyllm/model_executor/layers/attention.py:39-52, a
    flash-attn call there): the exact-attention kernel of the salient rows with every query row listed."""
    H, Hkv = q.size(1), k.size(1)
    if _dense_attention_backend == "tcgen05" and q.size(2) == 128:
        rows = q.size(0)
        key = (rows, q.device)
        idx = _all_rows_cache.get(key)
        if idx is None:
            idx = _all_rows_cache[key] = torch.arange(rows, dtype=torch.int32, device=q.device)
        return attention_salient_rows(q, k, v, ctx.cu_seqlens_k, ctx.cu_seqlens_q, idx, max_rows_per_seq=ctx.max_seqlen_q,
                                      num_salient=rows)
    lens = ctx.context_lens_cpu
    if len(set(lens)) == 1:
        B, L = len(lens), lens[0]
        o = F.scaled_dot_product_attention(
            q.view(B, L, H, -1).transpose(1, 2), k.view(B, L, Hkv, -1).transpose(1, 2),
            v.view(B, L, Hkv, -1).transpose(1, 2), scale=scale, enable_gqa=H != Hkv)
        return o.transpose(1, 2).reshape(B * L, H, -1)
    outs, pos = [], 0
    for L in lens:
        o = F.scaled_dot_product_attention(
            q[pos : pos + L].transpose(0, 1)[None], k[pos : pos + L].transpose(0, 1)[None],
            v[pos : pos + L].transpose(0, 1)[None], scale=scale, enable_gqa=H != Hkv)
        outs.append(o[0].transpose(0, 1))
        pos += L
    return torch.cat(outs, dim=0)


class Attention(nn.Module):
    def __init__(self, num_heads, head_dim, scale, num_kv_heads, threshold: float = 0.99):
        super().__init__()
        if head_dim != 128 or abs(scale - head_dim ** -0.5) > 1e-6 * scale:
            # the sm_100a attention kernels are built for head_dim 128 and the reference kernel's own scale
            # (1/sqrt(head_dim), dyllm/csrc/attention/attention_ops_kernels_sm80.cu:166)
            raise ValueError(f"Attention supports head_dim 128 with scale head_dim**-0.5; got {head_dim}, {scale}")
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.threshold = threshold
        self.tp_size = _world_size()        # 1 under the sequence-sharded layout: this rank's rows are complete
        self.context_cache = CacheManager(self.num_heads * self.head_dim)
        self.v_cache = CacheManager(self.num_kv_heads * self.head_dim)
        self._hint_host = None      # pinned int32[1]: this layer's salient count, copied back without waiting
        self._hint_event = None
        self._hint = 0

    def _next_hint(self, count_dev: torch.Tensor, capacity: int, fixed: int = 0) -> int:
        """Estimate of the salient count this layer has just produced: its value from the previous step
        (read back asynchronously, never waited for), or the capacity when none has arrived yet.  The
        estimate only shapes launches; kernels take the true count from the device.  With ``fixed`` the
        estimate is that constant and no host state is touched (steps captured into a CUDA graph)."""
        if fixed:
            return min(fixed, capacity)
        if self._hint_host is None:
            self._hint_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._hint_event = torch.cuda.Event()
        elif self._hint_event.query():
            self._hint = int(self._hint_host[0])
            profiling.count("salient_rows", self._hint)
        else:
            return min(self._hint, capacity) if self._hint else capacity
        self._hint_host.copy_(count_dev, non_blocking=True)
        self._hint_event.record()
        return min(self._hint, capacity) if self._hint else capacity

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dv: torch.Tensor | None = None) -> torch.Tensor:
        """Dense step: q, k, v hold every row.  Sparse step: ``q`` every query row, ``k`` the packed full
        key tensor, ``v`` the new value rows of the step's salient tokens (reference convention).  ``dv``:
        the caller has already formed delta-V and updated the value cache (``ops.kv_cache_update``)."""
        ctx, md = get_context(), get_metadata()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        seq_t = md.running_seqs_tensor

        if ctx.is_full:
            o = _dense_attention(q, k, v, ctx, self.scale)
            self.context_cache.reset_full(o.flatten(-2, -1).contiguous(), seq_t, seq_ids_list=md.running_seqs)
            self.v_cache.reset_full(v.flatten(-2, -1), seq_t, seq_ids_list=md.running_seqs)
            self.context_cache.finish(md.finished_seqs)
            self.v_cache.finish(md.finished_seqs)
            return o

        is_q_pruned = ctx.idx_salient_row_k is not None
        rows_k = ctx.idx_salient_row_k if is_q_pruned else ctx.idx_salient_row
        idx_q32 = ctx.idx_salient_row32
        cap = idx_q32.numel()            # capacity of the salient lists; the live count may be on the device
        n_dev, hint = ctx.num_salient_dev, ctx.salient_hint
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim

        # delta-V and value-cache update in one pass over the salient rows (attention.py:67-74,89-96)
        if dv is None:
            dv = torch.empty((cap, Hkv, D), dtype=v.dtype, device=v.device)
            if cap:
                dest = ops.cache_dest_rows(rows_k, ctx.cu_seqlens_k, self.v_cache.seq_start_gpu, seq_t, n_dev)
                ops.delta_v_update(v.view(cap, Hkv * D), self.v_cache.cache, dest, dv.view(cap, Hkv * D), n_dev)
        v_full = self.v_cache.get_seqs(seq_t, allow_view=True, seq_ids_list=md.running_seqs).view(-1, Hkv, D)

        # exact attention of the salient query rows (attention.py:76-87)
        max_rows = max(min(ctx.max_salient_per_seq, ctx.max_seqlen_q), 1)
        with profiling.region("salient_attention", 4.0 * (hint or cap) * ctx.max_seqlen_k * H * D,
                              2.0 * ctx.total_seqlen_k * Hkv * D * 2 + 2.0 * (hint or cap) * H * D * 2):
            o_sal = attention_salient_rows(q, k, v_full, ctx.cu_seqlens_k, ctx.cu_salientlens, idx_q32,
                                           max_rows_per_seq=max_rows, num_salient=cap)

        stats = torch.empty((ctx.total_seqlen, 3), dtype=torch.float32, device=q.device)   # overwritten (v_layout bit 2)
        mask = torch.empty((ctx.total_seqlen,), dtype=torch.bool, device=q.device)
        # the previous context is read from, and the new one written back to, the cache arena itself
        c_arena = self.context_cache.cache.view(-1, H, D)
        rows_k32 = None      # response-only steps: the kernel derives the key rows from the query rows
        # algorithmic flops: Q K^T over all keys (sum over sequences of len_q * len_k, equal lengths here)
        flops = 2.0 * ctx.total_seqlen * ctx.max_seqlen_k * H * D
        # algorithmic bytes of the fused call: Q and the previous context (straight from the context cache) read, the
        # new context written twice (the packed tensor that o_proj reads, and the cache rows in place: the reference's
        # reset_block / reset_full copy after its kernel, attention.py:153,168), K read once
        nbytes = 4.0 * ctx.total_seqlen * H * D * 2 + ctx.total_seqlen_k * Hkv * D * 2
        with profiling.region("delta_attention", flops, nbytes):
            new_c = attention_sparse_varlen(q, k, dv, c_arena, o_sal, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                            ctx.max_seqlen_q, ctx.max_seqlen_k, ctx.total_seqlen, ctx.cu_salientlens,
                                            idx_q32, stats, mask, self.threshold, is_q_pruned, rows_k32, v_layout=7,
                                            num_salient_dev=n_dev,
                                            c_cache=(self.context_cache.seq_start_gpu, seq_t, True))

        # 12 B/token all-reduce, then mask + ordered compaction (+ K-space offsets) in one launch; the new
        # lists stay on the device together with their length
        if self.tp_size > 1:
            all_reduce_stats(stats)
        with profiling.region("salient_select", 0.0, 12.0 * ctx.total_seqlen):
            sel = ops.salient_select(stats, self.threshold, ctx.cu_seqlens_q,
                                     ctx.cu_promptlens if is_q_pruned else None)
        if is_q_pruned:
            ctx.idx_salient_row_k = sel.idx_k
        ctx.idx_salient_row = sel.idx
        ctx.idx_salient_row32 = sel.idx32
        ctx.cu_salientlens = sel.cu_salientlens
        ctx.num_salient_dev = sel.count
        ctx.max_salient_per_seq = ctx.max_seqlen_q
        ctx.salient_hint = self._next_hint(sel.count, ctx.total_seqlen, ctx.fixed_hint)

        self.v_cache.finish(md.finished_seqs)
        self.context_cache.finish(md.finished_seqs)
        return new_c.view(-1, H, D)
