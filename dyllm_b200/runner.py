"""Minimal step driver for the saliency path: builds the per-step ``Context`` exactly as the reference's
``ModelRunner.prepare_full`` / ``prepare_sparse`` do (ref: dyllm/engine/model_runner.py:140-298), runs the
model, and unmasks tokens with the confidence rule of the reference's sampler
(ref: dyllm/model_executor/layers/sampler.py:244-315) for batches of equal-length sequences.

It exists so that the path can be measured and tested end to end; request scheduling, tokenisation
and multi-process control of the reference engine are outside this package.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import List

import torch
import torch.distributed as dist

from . import _lib, ops, profiling
from .context import get_context, get_metadata, set_context, set_metadata

# Row-count estimate baked into the launches of a captured step: the common case is at most one 128-row
# tile of salient rows per layer; the kernels adapt to the true count on the device.
GRAPH_ROWS_HINT = 128


class _SegmentedCapture:
    """Captures a step that contains collectives as a chain of CUDA graphs with the collectives between
    them: a graph is closed at every all-reduce, the all-reduce is issued eagerly (outside any capture) and
    the next graph is opened.  Replay walks the chain; the host then makes one call per graph and per
    collective instead of one per kernel."""

    def __init__(self, pool):
        self.pool = pool
        self.items: list = []          # ("graph", CUDAGraph) | ("reduce", tensor)
        self.stream = torch.cuda.Stream()
        self._graph = None

    def _begin(self) -> None:
        self._graph = torch.cuda.CUDAGraph()
        self._graph.capture_begin(pool=self.pool)

    def _end(self) -> None:
        self._graph.capture_end()
        self.items.append(("graph", self._graph))
        self._graph = None

    def on_all_reduce(self, t: torch.Tensor) -> None:
        self._end()
        dist.all_reduce(t, op=dist.ReduceOp.SUM)     # keeps the ranks in step; the data is not meaningful yet
        self.items.append(("reduce", t))
        self._begin()

    def capture(self, fn) -> None:
        from . import layers

        torch.cuda.synchronize()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            layers.set_all_reduce_hook(self.on_all_reduce)
            self._begin()
            try:
                fn()
            finally:
                layers.set_all_reduce_hook(None)
                if self._graph is not None:
                    self._end()
        torch.cuda.current_stream().wait_stream(self.stream)

    def replay(self) -> None:
        for kind, obj in self.items:
            if kind == "graph":
                obj.replay()
            else:
                dist.all_reduce(obj, op=dist.ReduceOp.SUM)


def _multi_rank() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


@dataclass
class Sequence:
    """The per-request state the step preparation reads (ref: dyllm/engine/sequence.py:15-82)."""

    seq_id: int
    token_ids: List[int]
    num_prompt_tokens: int
    max_new_tokens: int
    processed_steps: int = 0
    last_token_pos: List[int] = field(default_factory=list)
    last_tokens: List[int] = field(default_factory=list)

    def __len__(self) -> int:
        return len(self.token_ids)


io_bytes = {"h2d": 0, "d2h": 0}  # host<->device traffic of the step driver, counted from the tensors copied


def _dev(values, dtype, device):
    t = torch.tensor(values, dtype=dtype)
    io_bytes["h2d"] += t.numel() * t.element_size()
    return t.pin_memory().to(device, non_blocking=True) if device.type == "cuda" else t.to(device)


def prepare_full(seqs: List[Sequence], device: torch.device):
    """ref: dyllm/engine/model_runner.py:140-184."""
    input_ids, positions, cu = [], [], [0]
    lens, seq_ids = [], []
    for seq in seqs:
        n = len(seq)
        input_ids.extend(seq.token_ids)
        positions.extend(range(n))
        cu.append(cu[-1] + n)
        lens.append(n)
        seq_ids.append(seq.seq_id)
    md = get_metadata()
    md.running_seqs = seq_ids
    md.running_seqs_tensor = _dev(seq_ids, torch.long, device)
    cu_t = _dev(cu, torch.int32, device)
    set_context(True, cu_seqlens_q=cu_t, cu_seqlens_q_cpu=cu, cu_seqlens_k=cu_t, max_seqlen_q=max(lens),
                max_seqlen_k=max(lens), context_lens=_dev(lens, torch.int32, device), context_lens_cpu=lens,
                total_seqlen=cu[-1], total_seqlen_k=cu[-1])
    return _dev(input_ids, torch.int64, device), _dev(positions, torch.int64, device)


def prepare_sparse(seqs: List[Sequence], device: torch.device, refresh_period: int = 4):
    """ref: dyllm/engine/model_runner.py:186-298.  ``refresh_period`` is the reference's hard-coded 4:
    a step with ``processed_steps > period and processed_steps % period != 0`` uses response-only
    queries, every other sparse step the full sequence.  ``processed_steps`` counts the current step too
    (the reference's scheduler increments it before the step runs, dyllm/engine/scheduler.py:43,69)."""
    input_ids, positions, positions_k = [], [], []
    idx_q, idx_k, idx_upd = [], [], []
    cu_q, cu_k, cu_p, cu_sal = [0], [0], [0], [0]
    lens, seq_ids = [], []
    pruned_flags = []
    for seq in seqs:
        n = len(seq)
        cu_p.append(seq.num_prompt_tokens + cu_p[-1])
        answer_start = n - seq.max_new_tokens
        kept = [p for p in seq.last_token_pos if p >= answer_start]
        pruned = seq.processed_steps > refresh_period and seq.processed_steps % refresh_period != 0
        pruned_flags.append(pruned)
        if pruned:
            input_ids.extend(seq.token_ids[-seq.max_new_tokens:])
            positions.extend(range(answer_start, n))
            idx_q.extend(p - seq.num_prompt_tokens + cu_q[-1] for p in kept)
            idx_k.extend(p + cu_k[-1] for p in kept)
            lq = seq.max_new_tokens
        else:
            input_ids.extend(seq.token_ids)
            positions.extend(range(n))
            idx_q.extend(p + cu_q[-1] for p in kept)
            lq = n
        positions_k.extend(kept)
        idx_upd.extend(p + cu_k[-1] for p in kept)
        cu_sal.append(len(kept) + cu_sal[-1])
        seq_ids.append(seq.seq_id)
        cu_q.append(cu_q[-1] + lq)
        cu_k.append(cu_k[-1] + n)
        lens.append(n)
    any_pruned = any(pruned_flags)
    if any_pruned and not all(pruned_flags):
        raise RuntimeError("sequences of one batch must be at the same refresh phase")
    md = get_metadata()
    md.running_seqs = seq_ids
    md.running_seqs_tensor = _dev(seq_ids, torch.long, device)
    max_sal = max((cu_sal[i + 1] - cu_sal[i] for i in range(len(seqs))), default=0)
    set_context(
        False, cu_seqlens_q=_dev(cu_q, torch.int32, device), cu_seqlens_q_cpu=cu_q,
        cu_seqlens_k=_dev(cu_k, torch.int32, device), cu_promptlens=_dev(cu_p, torch.int32, device),
        cu_updatedlens=_dev(cu_sal, torch.int32, device), cu_salientlens=_dev(cu_sal, torch.int32, device),
        max_seqlen_q=max(cu_q[i + 1] - cu_q[i] for i in range(len(seqs))), max_seqlen_k=max(lens),
        idx_updated_row=_dev(idx_upd, torch.int32, device), idx_salient_row=_dev(idx_q, torch.int64, device),
        idx_salient_row_k=_dev(idx_k, torch.int64, device) if any_pruned else None,
        idx_salient_row32=_dev(idx_q, torch.int32, device), max_salient_per_seq=max_sal,
        context_lens=_dev(lens, torch.int32, device), context_lens_cpu=lens, total_seqlen_k=cu_k[-1],
        total_seqlen=cu_q[-1], positions_k=_dev(positions_k, torch.int64, device))
    return _dev(input_ids, torch.int64, device), _dev(positions, torch.int64, device)


class StepRunner:
    """Runs denoising steps of a fixed batch: ``num_full_steps`` dense steps, then sparse steps."""

    def __init__(self, model, mask_id: int, block_length: int = 32, steps: int = 256, num_full_steps: int = 8,
                 refresh_period: int = 4, use_graphs: bool = True, full_logits: bool = False,
                 graphs_with_tp: bool | None = None, graph_rows_hint: int = GRAPH_ROWS_HINT):
        self.model = model
        self.mask_id = mask_id
        self.block_length = block_length
        self.steps = steps
        self.num_full_steps = num_full_steps
        self.refresh_period = refresh_period
        self.device = next(model.parameters()).device
        self.salient_counts: list[int] = []
        self.use_graphs = use_graphs
        # salient-row estimate baked into the launches of a captured step (any value is correct; the GEMMs are
        # shaped for it: narrow tiles and split-K up to a few hundred rows, wide and tall tiles above)
        self.graph_rows_hint = max(1, int(graph_rows_hint))
        # With several ranks a step is captured whole, NCCL all-reduces and peer-memory exchanges included
        # (DYLLM_TP_GRAPHS=whole, the default).  NCCL keeps a communicator alive for as long as a graph that
        # captured one of its collectives exists, and destroying the process group waits for that: call
        # release_graphs() before dist.destroy_process_group().  DYLLM_TP_GRAPHS=segmented captures a chain of
        # graphs cut at every NCCL all-reduce (issued eagerly between them); graphs_with_tp=False or
        # DYLLM_TP_GRAPHS=off launches every kernel eagerly.
        mode = os.environ.get("DYLLM_TP_GRAPHS", "whole")
        if graphs_with_tp is None:
            graphs_with_tp = mode != "off"
        self.graphs_with_tp = graphs_with_tp
        self.tp_graph_mode = mode if mode in ("whole", "segmented") else "whole"
        # The reference projects every query row onto the vocabulary and then indexes the rows of the
        # current block (model_runner.py:377, sampler.py:244-315); with full_logits False only the rows the
        # sampler reads are projected, which yields the same tokens.
        self.full_logits = full_logits
        self._states: dict = {}
        self._graphs: dict = {}
        self._warm: set = set()
        self._graph_pool = None
        self._geometry = 0          # the model's cache epoch this runner's graphs belong to
        # host-driven steps keep the last step's candidate positions, confidences and tokens here when set
        self.record_candidates = False
        self.last_candidates = None

    def _set_geometry(self, key) -> None:
        """Called at the start of every generation with (sequence lengths, generation length).  Sequence ids
        are reused from one generation to the next, so when the geometry changes the model's activation caches
        forget the previous batch (its ranges have other lengths).  The record of the geometry lives on the
        model, whose caches it describes; every runner of that model drops its captured graphs and state
        buffers when the caches have been cleared since it captured them: a graph holds the addresses and row
        offsets of the geometry it was captured for, and the cache arenas may move when they grow."""
        state = getattr(self.model, "_dyllm_cache_state", None)
        if state is None:
            state = self.model._dyllm_cache_state = {"key": None, "epoch": 0}
        if state["key"] is not None and state["key"] != key:
            from .cache_manager import CacheManager

            torch.cuda.synchronize(self.device)
            for module in self.model.modules():
                for value in vars(module).values():
                    if isinstance(value, CacheManager):
                        value.clear()
            state["epoch"] += 1
        state["key"] = key
        if self._geometry != state["epoch"]:
            self.release_graphs()
            self._states.clear()
            self._geometry = state["epoch"]

    def release_graphs(self) -> None:
        """Destroys every captured graph (needed before the process group is destroyed when the graphs
        hold collectives, and whenever the buffers they address go away)."""
        import gc

        self._graphs.clear()
        self._warm.clear()
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def new_batch(self, prompts: List[List[int]], max_new_tokens: int, first_seq_id: int = 0) -> List[Sequence]:
        seqs = []
        for i, p in enumerate(prompts):
            seqs.append(Sequence(first_seq_id + i, list(p) + [self.mask_id] * max_new_tokens, len(p), max_new_tokens))
        set_metadata([s.seq_id for s in seqs], [s.seq_id for s in seqs], [])
        return seqs

    @torch.inference_mode()
    def step(self, seqs: List[Sequence]) -> int:
        """One denoising step of every sequence; returns the number of tokens unmasked."""
        return sum(len(p) for p in self.step_picks(seqs))

    @torch.inference_mode()
    def step_picks(self, seqs: List[Sequence], forced=None):
        """One denoising step; returns, per sequence, the ``(position, token)`` pairs this package's path chose
        to unmask, ascending by position.  ``forced`` (same format) replaces them when the sequences are
        updated: a test can keep the state on a recorded trajectory while it compares every step's choice.
        The step counter follows the reference's scheduler (dyllm/engine/scheduler.py:29-75): it is
        incremented before the step, the first ``num_full_steps`` steps are dense."""
        for seq in seqs:
            seq.processed_steps += 1
        is_full = seqs[0].processed_steps <= self.num_full_steps
        if is_full:
            input_ids, positions = prepare_full(seqs, self.device)
        else:
            input_ids, positions = prepare_sparse(seqs, self.device, self.refresh_period)
        ctx = get_context()
        hidden = self.model(input_ids, positions)
        return self._unmask(seqs, hidden, ctx, forced)

    def generate(self, prompts: List[List[int]], max_new_tokens: int, device_state: bool = True) -> List[List[int]]:
        """Runs all denoising steps of one batch and returns the generated token ids (host lists).

        With ``device_state`` (equal-length prompts, and steps * tokens-per-step == max_new_tokens) the token
        matrix, the step layouts and the list of positions unmasked in the previous step stay on the device:
        the prompts go up once, the generated ids come back once, and no step waits for the host."""
        from . import layers

        sharded = layers.sequence_sharded()
        if sharded:
            # every rank generates for its own slice of the batch; the results are gathered at the end
            world, rank = dist.get_world_size(), dist.get_rank()
            if len(prompts) % world:
                raise RuntimeError(f"the sequence-sharded layout needs a batch ({len(prompts)}) divisible by the ranks ({world})")
            per = len(prompts) // world
            prompts = prompts[rank * per:(rank + 1) * per]
        lens = {len(p) for p in prompts}
        gen = max_new_tokens
        steps_per_block = max(1, self.steps * self.block_length // gen)
        num_transfer = max(1, self.block_length // steps_per_block)
        self._set_geometry((tuple(len(p) for p in prompts), gen))
        # the device-resident loop unmasks exactly num_transfer tokens per step: every block must be filled by
        # its own steps_per_block steps, and the blocks' steps must add up to the step count
        exact = (gen % self.block_length == 0 and steps_per_block * num_transfer == self.block_length
                 and steps_per_block * (gen // self.block_length) == self.steps)
        if device_state and len(lens) == 1 and exact:
            return self._generate_device(prompts, gen, steps_per_block, num_transfer, sharded)
        seqs = self.new_batch(prompts, max_new_tokens)
        for _ in range(self.steps):
            self.step(seqs)
        out = [s.token_ids[s.num_prompt_tokens:] for s in seqs]
        if sharded:
            parts = [None] * dist.get_world_size()
            dist.all_gather_object(parts, out)
            out = [row for part in parts for row in part]
        return out

    def _device_state(self, B: int, P: int, gen: int, steps_per_block: int, num_transfer: int):
        """Buffers of the device-resident loop for one batch geometry.  They are allocated once and reused
        by every generation of that geometry, so that captured graphs stay valid."""
        key = (B, P, gen, steps_per_block, num_transfer)
        st = self._states.get(key)
        if st is not None:
            return st
        dev, L, blk_len = self.device, P + gen, self.block_length
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        st = SimpleNamespace(
            key=key, B=B, P=P, gen=gen, L=L, steps_per_block=steps_per_block, num_transfer=num_transfer,
            tokens=torch.full((B, L), self.mask_id, dtype=torch.int64, device=dev),
            last_pos=torch.zeros((B, num_transfer), dtype=torch.int64, device=dev),
            step_t=torch.zeros((), dtype=torch.int64, device=dev),
            seq_t=torch.arange(B, dtype=torch.long, device=dev),
            # step layouts: dense / full-sequence sparse share one, response-only sparse has its own
            cu_full_l=[b * L for b in range(B + 1)], cu_ro_l=[b * gen for b in range(B + 1)],
            cu_prompt=i32([b * P for b in range(B + 1)]), cu_sal=i32([b * num_transfer for b in range(B + 1)]),
            lens_t=i32([L] * B), pos_full=torch.arange(L, device=dev).repeat(B),
            pos_ro=torch.arange(P, L, device=dev).repeat(B),
            row_base_full=(torch.arange(B, device=dev) * L).unsqueeze(1),
            row_base_ro=(torch.arange(B, device=dev) * gen).unsqueeze(1),
            blk_ar=torch.arange(blk_len, device=dev).unsqueeze(0), fixed_hint=0)
        st.cu_full, st.cu_ro = i32(st.cu_full_l), i32(st.cu_ro_l)
        self._states[key] = st
        return st

    def _device_step(self, st, kind: str) -> None:
        """One denoising step on the state buffers.  ``kind`` is "full" (dense), "sparse" (full-sequence
        queries) or "pruned" (response-only queries).  Everything that changes from step to step (the token
        matrix, the positions unmasked by the previous step, the step counter that selects the current
        block) lives on the device, so the same sequence of launches serves every step of a kind."""
        B, P, L, gen, blk_len = st.B, st.P, st.L, st.gen, self.block_length
        tokens = st.tokens
        if kind == "full":
            set_context(True, cu_seqlens_q=st.cu_full, cu_seqlens_q_cpu=st.cu_full_l, cu_seqlens_k=st.cu_full,
                        max_seqlen_q=L, max_seqlen_k=L, context_lens=st.lens_t, context_lens_cpu=[L] * B,
                        total_seqlen=B * L, total_seqlen_k=B * L)
            input_ids, positions = tokens.reshape(-1), st.pos_full
        else:
            pruned = kind == "pruned"
            idx_k = (st.last_pos + st.row_base_full).reshape(-1)
            idx_q = (st.last_pos - P + st.row_base_ro).reshape(-1) if pruned else idx_k
            set_context(False, cu_seqlens_q=st.cu_ro if pruned else st.cu_full,
                        cu_seqlens_q_cpu=st.cu_ro_l if pruned else st.cu_full_l, cu_seqlens_k=st.cu_full,
                        cu_promptlens=st.cu_prompt, cu_updatedlens=st.cu_sal, cu_salientlens=st.cu_sal,
                        max_seqlen_q=gen if pruned else L, max_seqlen_k=L, idx_salient_row=idx_q,
                        idx_salient_row_k=idx_k if pruned else None, idx_salient_row32=idx_q.to(torch.int32),
                        max_salient_per_seq=st.num_transfer, context_lens=st.lens_t, context_lens_cpu=[L] * B,
                        total_seqlen_k=B * L, total_seqlen=B * (gen if pruned else L), fixed_hint=st.fixed_hint)
            input_ids = tokens[:, P:].reshape(-1) if pruned else tokens.reshape(-1)
            positions = st.pos_ro if pruned else st.pos_full
        hidden = self.model(input_ids, positions)
        # confidence rule on the current block (ref: sampler.py:244-315), entirely on the device
        blk = torch.clamp(st.step_t // st.steps_per_block, max=gen // blk_len - 1)
        start = P + blk * blk_len                                    # 0-d device tensor
        if kind == "pruned":
            rows = st.row_base_ro + (start - P) + st.blk_ar
        else:
            rows = st.row_base_full + start + st.blk_ar
        conf, tok = self._confidence(self._block_logits(hidden, rows.reshape(-1)), B, blk_len)
        # masked candidates of the block -> the num_transfer most confident ones take their token (one kernel)
        ops.confidence_unmask_(conf, tok, tokens, st.step_t, st.steps_per_block, P, blk_len, st.num_transfer, self.mask_id,
                               picked_pos=st.last_pos)
        st.step_t.add_(1)

    def _run_step(self, st, kind: str) -> None:
        """Runs one step: eagerly the first time a kind of step is met (allocations, one-time kernel
        attributes), then captured into a CUDA graph and replayed.  Graphs are not used while region
        timing is on (events cannot be timed inside a graph).  With several ranks every rank runs the
        same sequence of eager steps, captures and replays, so the all-reduces inside a step line up."""
        if not self.use_graphs or profiling.enabled() or (_multi_rank() and not self.graphs_with_tp):
            self._device_step(st, kind)
            return
        key = (st.key, kind)
        entry = self._graphs.get(key)
        if entry is None:
            if key not in self._warm:
                # same launch shapes as the capture that follows, so that every kernel it needs is loaded
                self._warm.add(key)
                st.fixed_hint = self.graph_rows_hint
                try:
                    self._device_step(st, kind)
                finally:
                    st.fixed_hint = 0
                return
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = _lib.launch_count
            st.fixed_hint = self.graph_rows_hint
            try:
                if _multi_rank() and self.tp_graph_mode == "segmented":
                    graph = _SegmentedCapture(self._graph_pool)
                    graph.capture(lambda: self._device_step(st, kind))
                else:
                    graph = torch.cuda.CUDAGraph()
                    # thread-local: NCCL's watchdog thread may query events while this thread captures
                    with torch.cuda.graph(graph, pool=self._graph_pool,
                                          capture_error_mode="thread_local" if _multi_rank() else "global"):
                        self._device_step(st, kind)
            finally:
                st.fixed_hint = 0
            entry = self._graphs[key] = (graph, _lib.launch_count - before)
            _lib.launch_count = before
        entry[0].replay()
        _lib.launch_count += entry[1]

    @torch.inference_mode()
    def _generate_device(self, prompts, gen, steps_per_block, num_transfer, gather_ranks=False):
        B, P = len(prompts), len(prompts[0])
        st = self._device_state(B, P, gen, steps_per_block, num_transfer)
        prompt_t = torch.tensor(prompts, dtype=torch.int64)
        io_bytes["h2d"] += prompt_t.numel() * 8
        st.tokens.fill_(self.mask_id)
        st.tokens[:, :P] = prompt_t.pin_memory().to(self.device, non_blocking=True)
        st.step_t.zero_()
        seq_ids = list(range(B))
        set_metadata(seq_ids, seq_ids, [])
        get_metadata().running_seqs_tensor = st.seq_t
        for step in range(self.steps):
            done = step + 1     # the reference's processed_steps: incremented before the step runs
            if done <= self.num_full_steps:
                kind = "full"
            elif done > self.refresh_period and done % self.refresh_period != 0:
                kind = "pruned"
            else:
                kind = "sparse"
            self._run_step(st, kind)
        out = st.tokens[:, P:].contiguous()
        if gather_ranks:
            world = dist.get_world_size()
            full = torch.empty((world * B, gen), dtype=out.dtype, device=out.device)
            dist.all_gather_into_tensor(full, out)
            out = full
        out = out.cpu()
        io_bytes["d2h"] += out.numel() * 8
        return out.tolist()

    def _block_logits(self, hidden: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Logits of the given query rows.  A model with ``shift_logits`` (Dream) predicts the token of row r
        from row r - 1 of the packed batch (ref: sampler.py, ``DreamSampler.adjust_logits``)."""
        if getattr(self.model, "shift_logits", False):
            rows = (rows - 1).clamp_min(0)
        if self.full_logits:
            return self.model.compute_logits(hidden).index_select(0, rows)
        return self.model.compute_logits(hidden.index_select(0, rows))

    @staticmethod
    def _confidence(logits: torch.Tensor, B: int, blk_len: int):
        """Probability and id of the most likely token of every candidate row, as ``[B, blk_len]``
        (ref: sampler.py:286-288, softmax then max)."""
        conf, tok = ops.row_confidence(logits.contiguous())     # bf16 logits on a GPU; raises otherwise
        return conf.view(B, blk_len), tok.view(B, blk_len)

    def _unmask(self, seqs: List[Sequence], hidden: torch.Tensor, ctx, forced=None):
        B = len(seqs)
        gen = seqs[0].max_new_tokens
        steps_per_block = max(1, self.steps * self.block_length // gen)
        num_transfer = max(1, self.block_length // steps_per_block)
        cu_q = ctx.cu_seqlens_q_cpu
        rows, cand_pos = [], []
        for b, seq in enumerate(seqs):
            blk = min((seq.processed_steps - 1) // steps_per_block, gen // self.block_length - 1)
            start = seq.num_prompt_tokens + blk * self.block_length
            lq = cu_q[b + 1] - cu_q[b]
            off = start - (len(seq) - lq)  # position -> row inside this sequence's query rows
            rows.append(torch.arange(off, off + self.block_length) + cu_q[b])
            cand_pos.append(list(range(start, start + self.block_length)))
        rows_t = torch.stack(rows)
        io_bytes["h2d"] += rows_t.numel() * rows_t.element_size()
        rows_t = rows_t.to(self.device)
        conf, tok = self._confidence(self._block_logits(hidden, rows_t.flatten()), B, self.block_length)
        still_masked = torch.tensor(
            [[seq.token_ids[p] == self.mask_id for p in cand_pos[b]] for b, seq in enumerate(seqs)])
        io_bytes["h2d"] += still_masked.numel()
        still_masked = still_masked.to(self.device)
        conf = torch.where(still_masked, conf, torch.full_like(conf, -1.0))
        if self.record_candidates:
            self.last_candidates = (cand_pos, conf.cpu(), tok.cpu())
        top_conf, top_i = conf.topk(num_transfer, dim=-1)
        picked = torch.stack([top_i, tok.gather(1, top_i), (top_conf >= 0).long()], dim=-1).cpu()  # one D2H per step
        io_bytes["d2h"] += picked.numel() * picked.element_size()
        picks = []
        for b, seq in enumerate(seqs):
            chosen = []
            for j in range(num_transfer):
                i, t, ok = picked[b, j].tolist()
                if ok:
                    chosen.append((cand_pos[b][i], int(t)))
            chosen.sort()  # the kernels expect ascending row lists
            picks.append(chosen)
            applied = sorted(forced[b]) if forced is not None else chosen
            for p, t in applied:
                seq.token_ids[p] = t
            seq.last_token_pos = [p for p, _ in applied]
            seq.last_tokens = [t for _, t in applied]
        return picks
