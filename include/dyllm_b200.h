/*
 * dyllm_b200 — C ABI of the sm_100a implementation of DyLLM's per-denoising-step saliency path.
 *
 * Every entry point takes raw device pointers, plain sizes and a CUDA stream (as void*), launches on
 * that stream, never synchronises, never throws and returns an int status (0 = ok, < 0 = error; the
 * text of the last error of the calling thread is returned by dyllm_last_error()).  Unless a
 * function says otherwise it allocates nothing: outputs and workspaces are provided by the caller.
 *
 * Citations of the form "ref: path:line" name the file of the reference project (scale-snu/DyLLM)
 * whose behaviour the entry point reproduces.
 *
 * Conventions: bf16 tensors are row-major and contiguous; "rows" are token rows of the packed
 * (varlen) batch; cu_* arrays are int32 prefix sums of length batch + 1.
 */
#ifndef DYLLM_B200_H_
#define DYLLM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DYLLM_OK 0
#define DYLLM_ERR_INVALID_ARGUMENT (-1)
#define DYLLM_ERR_UNSUPPORTED (-2)
#define DYLLM_ERR_CUDA (-3)
#define DYLLM_ERR_WORKSPACE (-4)
#define DYLLM_ERR_DEVICE_TIMEOUT (-5)

/* Library version (major * 10000 + minor * 100 + patch). */
int dyllm_version(void);
/* Message of the last failing call made by the calling thread ("" when none). */
const char* dyllm_last_error(void);
/* Reads and clears the per-device status word that kernels with bounded waits set when a wait ran
 * out.  Synchronises the device.  Returns 0 when no kernel gave up, else a positive site code. */
int dyllm_device_status(void);

/* ------------------------------------------------------------------------------------------------
 * Salient-token selection: statistics, mask, compaction
 * ---------------------------------------------------------------------------------------------- */

/* Per-row additive cosine statistics between the previous and the current attention context:
 * stats[r] = { sum(new*old), sum(new^2), sum(old^2) } over `width` bf16 elements, fp32 accumulation in
 * a fixed order (run-to-run identical).  When accumulate != 0 the three sums are added to the values
 * already in `stats` (one call per tensor-parallel head shard held on the same device); otherwise
 * they overwrite them.
 * ref: dyllm/csrc/attention/attention_ops_kernels_sm80.cu:407-481 (epilogue statistics),
 *      dyllm/csrc/attention/attention_aux_kernels.cu:34-71 (bf16 rows). */
int dyllm_context_stats(const void* c_old, const void* c_new, float* stats, int rows, int width,
                        int accumulate, void* stream);

/* mask[r] = dot * rsqrt(max(a, 1e-8)) * rsqrt(max(b, 1e-8)) < threshold, one byte per row.
 * ref: dyllm/csrc/attention/attention_aux_kernels.cu:10-20,138-146;
 *      dyllm/distributed/parallel_state.py:52-66. */
int dyllm_cosine_mask(const float* stats, uint8_t* mask, int rows, float threshold, void* stream);

/* Bytes of scratch memory dyllm_salient_select needs for `rows` rows. */
size_t dyllm_salient_select_workspace_bytes(int rows);

/* Fused mask + compaction.  From the (already all-reduced) statistics of `rows` query rows it writes
 *   idx_out[0..n)            ascending row numbers with cosine < threshold      (int64)
 *   idx32_out[0..n)          the same list as int32, nullable
 *   idx_k_out[0..n)          idx + cu_promptlens[b + 1], b = sequence of the row (int64, nullable;
 *                            requires cu_promptlens)
 *   cu_salientlens_out[b]    number of selected rows below cu_seqlens_q[b], b = 0..batch (int32)
 *   count_out[0]             n                                                   (int32)
 *   mask_out[r]              the per-row decision, nullable                       (uint8)
 * in one launch, without a host synchronisation.  `workspace` must hold
 * dyllm_salient_select_workspace_bytes(rows) bytes; its content on entry is irrelevant.
 * ref: dyllm/distributed/parallel_state.py:52-66 (mask rule),
 *      dyllm/model_executor/layers/attention.py:147-150,172-173 (nonzero + searchsorted),
 *      dyllm/csrc/attention/attention_aux_kernels.cu:112-128 (K-space offsets). */
int dyllm_salient_select(const float* stats, int rows, float threshold, const int32_t* cu_seqlens_q,
                         int batch, const int32_t* cu_promptlens, int64_t* idx_out, int32_t* idx32_out,
                         int64_t* idx_k_out, int32_t* cu_salientlens_out, int32_t* count_out,
                         uint8_t* mask_out, void* workspace, size_t workspace_bytes, void* stream);

/* Selection for callers that may not allocate.  Same inputs, outputs and results as
 * dyllm_salient_select, but the scratch memory is a fixed array inside the library (about 16 KB, held
 * by every GPU that loads the library until the process exits), so the caller passes no workspace and
 * neither this call nor anything it uses calls cudaMalloc, cudaFree or another allocating routine.
 * It is meant for hosts that have handed all device memory to a pool of their own before serving
 * starts, or whose steady-state step must not touch the CUDA allocator because an allocation there
 * would stall every stream of the device.  This entry point has no counterpart in the reference.
 *   - rows may be at most dyllm_salient_select_static_max_rows() (4 Mi rows); larger inputs are
 *     rejected with DYLLM_ERR_UNSUPPORTED and an error text that names the limit.
 *   - The first call on a device looks up the array's device address (once per device, with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array, which keeps the previous call's content; each call
 *     clears the part it uses on its stream before its kernel runs.  Two calls whose kernels can overlap
 *     on the GPU (different streams without an ordering between them) race on the array and give
 *     undefined results: issue them on one stream or order them with events. */
int dyllm_salient_select_static(const float* stats, int rows, float threshold, const int32_t* cu_seqlens_q,
                                int batch, const int32_t* cu_promptlens, int64_t* idx_out, int32_t* idx32_out,
                                int64_t* idx_k_out, int32_t* cu_salientlens_out, int32_t* count_out,
                                uint8_t* mask_out, void* stream);
/* Largest `rows` dyllm_salient_select_static accepts. */
int dyllm_salient_select_static_max_rows(void);

/* out[t] = idxs[t] + cu_promptlens[g + 1] for t < *num_idxs, g = group with
 * cu_salientlens[g] <= t < cu_salientlens[g + 1]; at most max_threads entries are written.
 * ref: dyllm/csrc/attention/attention_aux_kernels.cu:112-128,173-200 (fused_offset_launch). */
int dyllm_fused_offset(const int32_t* idxs, const int32_t* num_idxs, const int32_t* cu_promptlens,
                       const int32_t* cu_salientlens, int num_groups, int64_t* out, int max_threads,
                       void* stream);

/* ------------------------------------------------------------------------------------------------
 * Per-sequence activation cache (rows of `width` elements of `elem_bytes` bytes each;
 * width * elem_bytes must be a multiple of 16).  seq_starts[seq_ids[b]] is the first cache row of
 * batch entry b.
 * ---------------------------------------------------------------------------------------------- */

/* out[cu[b] + i] = cache[seq_starts[seq_ids[b]] + i], i < cu[b+1] - cu[b].
 * ref: dyllm/csrc/cache/cache_kernels.cu:18-108 (get_seqs_cuda). */
int dyllm_cache_get_seqs(const void* cache, void* out, const int64_t* seq_starts, const int32_t* cu_seqlens,
                         const int64_t* seq_ids, int batch, int total_rows, int width, int elem_bytes,
                         void* stream);
/* out[cu_q[b] + i] = cache[seq_starts[seq_ids[b]] + len_k(b) - len_q(b) + i]: the last len_q rows.
 * ref: dyllm/csrc/cache/cache_kernels.cu:249-294 (get_block_cuda). */
int dyllm_cache_get_block(const void* cache, void* out, const int64_t* seq_starts, const int32_t* cu_seqlens_k,
                          const int32_t* cu_seqlens_q, const int64_t* seq_ids, int batch, int total_rows,
                          int width, int elem_bytes, void* stream);
/* cache[seq_starts[seq_ids[b]] + i] = in[cu[b] + i].
 * ref: dyllm/csrc/cache/cache_kernels.cu:110-198 (reset_full_cuda). */
int dyllm_cache_reset_full(void* cache, const void* in, const int64_t* seq_starts, const int32_t* cu_seqlens,
                           const int64_t* seq_ids, int batch, int total_rows, int width, int elem_bytes,
                           void* stream);
/* cache[seq_starts[seq_ids[b]] + len_k(b) - len_q(b) + i] = in[cu_q[b] + i].
 * ref: dyllm/csrc/cache/cache_kernels.cu:296-386 (reset_block_cuda). */
int dyllm_cache_reset_block(void* cache, const void* in, const int64_t* seq_starts, const int32_t* cu_seqlens_k,
                            const int32_t* cu_seqlens_q, const int64_t* seq_ids, int batch, int total_rows,
                            int width, int elem_bytes, void* stream);
/* cache[seq_starts[seq_ids[b]] + row_idx[m] - cu[b]] = new_rows[m], b = sequence containing packed
 * row row_idx[m].  `num_rows_dev`, when not null, is a device int32 that bounds m from above
 * (m < min(num_rows, *num_rows_dev)).  cu_is_int64 selects the element type of cu_seqlens.
 * ref: dyllm/csrc/cache/cache_kernels.cu:388-459 (scatter_update_cuda). */
int dyllm_cache_scatter_update(void* cache, const void* new_rows, const int64_t* row_idx, const void* cu_seqlens,
                               int cu_is_int64, const int64_t* seq_starts, const int64_t* seq_ids, int batch,
                               int num_rows, const int32_t* num_rows_dev, int width, int elem_bytes,
                               void* stream);

/* ------------------------------------------------------------------------------------------------
 * Gathered tensor-core GEMMs (tcgen05 / TMEM).  Weights are bf16 [out, in] row-major as in
 * torch.nn.Linear.  The live row count may be given on the device (num_rows_dev, nullable): then
 * num_rows is only an upper bound that sizes buffers, rows_hint (<= 0: none) is the expected count
 * used to shape the launch, and no host synchronisation is needed.  a_mode selects how activation
 * rows reach the tensor cores: 0 = the indexed rows are first staged into a compact buffer of the
 * workspace and then loaded as plain TMA boxes (default when negative), 1 = TMA gather4 straight from
 * x.  tile_n = 64, 128, 256 (plain product with many rows only) or 0 (choose).
 * ---------------------------------------------------------------------------------------------- */

/* Bytes of workspace dyllm_gathered_linear needs for up to max_rows rows (row staging + split-K
 * partial sums).  Without a workspace the call still works with a_mode 1 or idx == null. */
size_t dyllm_gathered_linear_workspace_bytes(int max_rows, int in_features, int out_features);

/* out[map[m]] = scale[m] * (x[idx[m]] W^T), m < min(num_rows, *num_rows_dev).  idx null = identity,
 * out_row_map null = m (negative entries drop the row), row_scale null = 1.  When out2 is not null,
 * output columns >= split_col (a multiple of 128) go to out2[.., column - split_col] instead (used to
 * write K and V of the fused K/V projection into two tensors).  in_features % 64 == 0,
 * out_features % 64 == 0.  Few rows and few column tiles switch on a deterministic split-K: the k range is
 * cut into at most 4 parts whose fp32 partial sums go to the workspace, and the CTA that finishes an output
 * tile last adds them in split order inside the same launch (arrival counters live in a small array inside
 * the library, so two split-K calls on one device must not overlap on the GPU: issue them on one stream).
 * ref: dyllm/model_executor/models/llada.py:108 (kv_proj(hidden_states[idx_salient_row])),
 *      dyllm/model_executor/layers/linear.py:50-51. */
int dyllm_gathered_linear(const void* x, int x_rows, int in_features, int64_t ldx, const int32_t* idx,
                          int num_rows, const int32_t* num_rows_dev, int rows_hint, const void* weight,
                          int out_features, void* out, int64_t ldo, void* out2, int64_t ldo2, int split_col,
                          const int32_t* out_row_map, const float* row_scale, void* workspace,
                          size_t workspace_bytes, int a_mode, int tile_n, void* stream);

/* Bytes of workspace dyllm_swiglu_ffn needs for up to max_rows gathered rows. */
size_t dyllm_swiglu_ffn_workspace_bytes(int max_rows, int hidden, int inter);

/* out[map[m]] = down( silu(x[idx[m]] Wg^T) * (x[idx[m]] Wu^T) ) for the gathered rows: w_gate_up is
 * [2 * inter, hidden] with the gate rows first, w_down is [hidden, inter].  The SiLU product is fused
 * into the first GEMM's epilogue, the row scatter into the second's.  workspace: 16-byte aligned,
 * dyllm_swiglu_ffn_workspace_bytes(num_rows, hidden, inter) bytes.
 * ref: dyllm/model_executor/models/llada.py:38-43,184-185 (gather + MLP),
 *      dyllm/model_executor/layers/activations.py:9-14, dyllm/model_executor/layers/linear.py:76-93,195-220,
 *      dyllm/model_executor/layers/mlp_cache_manage.py:24-40 (scatter into the FFN-output cache). */
int dyllm_swiglu_ffn(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                     const int32_t* num_rows_dev, int rows_hint, const void* w_gate_up, const void* w_down,
                     int inter, void* out, int64_t ldo, const int32_t* out_row_map, void* workspace,
                     size_t workspace_bytes, int a_mode, int tile_n, void* stream);

/* dest_rows[m] = seq_starts[seq_ids[b]] + row_idx[m] - cu_seqlens[b] (the cache row that
 * dyllm_cache_scatter_update would write) for m < min(num_rows, *num_rows_dev), -1 for the rest;
 * feeds out_row_map of the GEMMs above.  ref: dyllm/csrc/cache/cache_kernels.cu:398-421. */
int dyllm_cache_dest_rows(const int64_t* row_idx, const int32_t* cu_seqlens, const int64_t* seq_starts,
                          const int64_t* seq_ids, int batch, int num_rows, const int32_t* num_rows_dev,
                          int32_t* dest_rows, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Approximate (delta) attention of a sparse step, head_dim 128
 * ---------------------------------------------------------------------------------------------- */

/* Bytes of scratch memory dyllm_attention_sparse_varlen needs (per-head partial statistics). */
size_t dyllm_attention_sparse_workspace_bytes(int total_q, int num_heads);

/* out[r] = bf16( c[r] + softmax(q_r K^T / sqrt(D)) V ) for all total_q query rows, where V is the
 * delta-V tensor of the step: it must be zero on every key row that is not listed in
 * idx_salient_row_k (the reference's caller builds it that way; only the listed rows are read).
 * Rows listed in idx_salient_row_q take the o_sal row as their new value instead, and
 *   cosine_stats[r] += {dot(new, c), |new|^2, |c|^2}   (caller zero-fills; new is the fp32 value before
 *                      rounding, or the bf16 o_sal row for the replaced rows)
 *   cosine_out[r]    = cosine(cosine_stats[r]) < threshold
 * q, c, out: [total_q, num_heads, 128]; k, v: [total_k, num_kv_heads, 128]; o_sal: [num_salient,
 * num_heads, 128]; all bf16.  idx_salient_row_q (query space) and idx_salient_row_k (key space) hold
 * num_salient ascending rows each, grouped by sequence through cu_salientlens; pass the same list
 * twice when queries are not pruned.  idx_salient_row_k may be null: the key row of a listed query row is
 * then taken to be the row at the same distance from the end of its sequence (the queries of a sequence
 * are its last len_q rows, as the reference's response-only steps build them).  num_salient_dev (nullable) is a device int32 holding the live list
 * length; num_salient is then only the capacity of the lists (the per-sequence counts always come from
 * cu_salientlens on the device).  The softmax scale is 1/sqrt(128).  Statistics are reduced over
 * heads in a fixed order.  v_layout is a bit set: bit 0 selects how the delta-V tile is fed to the
 * tensor cores (1 = as gathered, MN-major descriptor; 0 = transposed while gathering; results are
 * identical); bit 1 set means v is compact, [num_salient, num_kv_heads, 128] with row i belonging to
 * key idx_salient_row_k[i], instead of the zero-padded [total_k, ...] tensor (no memset, no scatter);
 * bit 2 set means cosine_stats is overwritten instead of added to (the caller need not zero-fill it).
 * Cache-resident context (c_seq_starts and c_seq_ids not null): c is then the context cache arena
 * [cache_rows, num_heads, 128] itself and the old context of query row r of batch entry b is cache row
 * c_seq_starts[c_seq_ids[b]] + len_k(b) - len_q(b) + (r - cu_seqlens_q[b]) (the last len_q rows of the
 * sequence), which removes the caller's gather copy; with c_update_in_place != 0 the new context is also
 * written back to those rows, which removes the caller's write-back copy (the reference's
 * get_seqs / get_block and reset_full / reset_block around this call, layers/attention.py:107-111,152-170).
 * ref: dyllm/csrc/attention/attention.cpp:64-179 (attention_sparse_varlen),
 *      dyllm/csrc/attention/attention_ops_kernels_sm80.cu:44-590,
 *      dyllm/csrc/attention/attention_aux_kernels.cu:10-110. */
int dyllm_attention_sparse_varlen(const void* q, const void* k, const void* v, const void* c, const void* o_sal,
                                  void* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                                  int max_seqlen_q, int max_seqlen_k, int total_q, int total_k, int num_heads,
                                  int num_kv_heads, int head_dim, const int32_t* cu_salientlens,
                                  const int32_t* idx_salient_row_q, const int32_t* idx_salient_row_k,
                                  int num_salient, const int32_t* num_salient_dev, float* cosine_stats,
                                  uint8_t* cosine_out, float threshold, void* workspace, size_t workspace_bytes,
                                  int v_layout, const int64_t* c_seq_starts, const int64_t* c_seq_ids,
                                  int c_update_in_place, void* stream);


/* Delta-V of the step and value-cache update in one pass over the salient rows:
 *   dv[i] = v_new[i] - cache[rows[i]];  cache[rows[i]] = v_new[i]       i < min(num_rows, *num_rows_dev)
 * (bf16, the difference rounded once).  rows are int32 row numbers of `cache`; width % 8 == 0.
 * ref: dyllm/model_executor/layers/attention.py:67-74,89-96 (v_delta, cache update, v_delta_sparse). */
int dyllm_delta_v_update(const void* v_new, void* cache, const int32_t* rows, int num_rows,
                         const int32_t* num_rows_dev, int width, void* dv, void* stream);

/* Exact attention of the salient query rows against the whole K / V of their sequence (non-causal):
 * o_sal[i] = softmax(q[idx_salient_row_q[i]] K^T / sqrt(128)) V, i grouped by sequence through
 * cu_salientlens.  q: [total_q, num_heads, 128], k, v: [total_k, num_kv_heads, 128], o_sal:
 * [num_salient, num_heads, 128], bf16.  max_rows_per_seq is an upper bound of the salient rows of one
 * sequence (it sizes the grid; the device-side counts decide the work).
 * ref: dyllm/model_executor/layers/attention.py:76-87 (flash_attn_varlen_func on q[idx_salient_row]). */
int dyllm_attention_salient_rows(const void* q, const void* k, const void* v, void* o_sal,
                                 const int32_t* cu_seqlens_k, int batch, int max_rows_per_seq, int total_q,
                                 int total_k, int num_heads, int num_kv_heads, int head_dim,
                                 const int32_t* cu_salientlens, const int32_t* idx_salient_row_q, void* stream);

/* Launch resources of the main attention kernel: [registers, local bytes, static shared bytes,
 * dynamic shared bytes, threads per block, resident blocks per SM, query rows per block, keys per
 * tile, head-dim split, ok].  ref: dyllm/csrc/attention/attention.cpp:184-208. */
int dyllm_attention_kernel_info(int dim, int64_t* info10);

/* ------------------------------------------------------------------------------------------------
 * Mixture-of-experts FFN on salient rows (softmax top-k router + expert-grouped tcgen05 GEMMs)
 * ---------------------------------------------------------------------------------------------- */

/* Router: for row m < min(num_rows, *num_rows_dev) of x[idx[m]] (idx null = identity) the fp32 logits
 * x . router_weight^T, softmax over the experts, the top_k probabilities (optionally renormalised to
 * sum 1; rounded to bf16 as the reference hands them on) and their expert ids, best first.
 * router_weight: bf16 [num_experts, hidden]; topk_weights: fp32 [num_rows, top_k]; topk_ids: int32.
 * ref: dyllm/model_executor/layers/fused_moe.py:375-407 (moe_gate), lladamoe.py:90-91. */
int dyllm_moe_route(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                    const int32_t* num_rows_dev, const void* router_weight, int num_experts, int top_k,
                    int renormalize, float* topk_weights, int32_t* topk_ids, void* stream);

/* Bytes of workspace dyllm_moe_ffn needs. */
size_t dyllm_moe_ffn_workspace_bytes(int max_rows, int top_k, int num_local_experts, int hidden, int inter);

/* out[map[m]] = sum over the slots j of row m whose expert e = topk_ids[m, j] - expert_start is local
 * (0 <= e < num_local_experts) of  topk_weights[m, j] * down_e( silu(x Wg_e^T) * (x Wu_e^T) ),
 * x = x[idx[m]].  w1: bf16 [num_local_experts, 2 * inter, hidden] (gate rows first), w2: bf16
 * [num_local_experts, hidden, inter].  Rows without a local expert get zeros.  The (row, slot) pairs are
 * grouped by expert on the device, each group padded to 128-row tiles; the routing weight is applied
 * in the down projection's epilogue and the slot sum runs in fp32 in slot order.  With
 * expert_start = 0 and all experts local this is the reference's fused_experts; a contiguous expert
 * range gives one rank's share under expert parallelism (the caller all-reduces the outputs).
 * ref: dyllm/model_executor/layers/fused_moe.py:37-85,269-335 (moe_align_block_size, fused_experts),
 *      dyllm/model_executor/models/lladamoe.py:107-142 (expert-parallel selection). */
int dyllm_moe_ffn(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                  const int32_t* num_rows_dev, int rows_hint, const float* topk_weights, const int32_t* topk_ids,
                  int top_k, const void* w1, const void* w2, int num_local_experts, int expert_start, int inter,
                  void* out, int64_t ldo, const int32_t* out_row_map, void* workspace, size_t workspace_bytes,
                  void* stream);

/* ------------------------------------------------------------------------------------------------
 * Row-wise kernels around the path (every query row, HBM-bound)
 * ---------------------------------------------------------------------------------------------- */

/* Everything between the K/V projection of the salient rows and the attention kernels, in one launch:
 *   k_cache[row_k(i)] = rope_neox(k_new[i], positions[pos_idx ? pos_idx[i] : i])
 *   dv[i] = v_new[i] - v_cache[row_v(i)];  v_cache[row_v(i)] = v_new[i]
 * k_new, v_new, dv: [num_rows, kv_heads, 128] bf16; rows_k: packed K-space rows (as for scatter_update);
 * row_x(i) = x_seq_starts[seq_ids[b]] + (rows_k[i] - cu_seqlens_k[b]) for the sequence b that holds the row;
 * cos_sin: fp32 [max_pos, 128]; num_rows_dev (nullable) bounds the rows on the device.
 * ref: dyllm/model_executor/models/llada.py:108-118 (rotary embedding of the new keys, k_cache.scatter_update)
 * and dyllm/model_executor/layers/attention.py:67-74,89-96 (delta-V, v_cache.scatter_update). */
int dyllm_kv_cache_update(const void* k_new, const void* v_new, const int64_t* rows_k, const int64_t* positions,
                          const int64_t* pos_idx, const float* cos_sin, int max_pos, const int32_t* cu_seqlens_k,
                          const int64_t* k_seq_starts, const int64_t* v_seq_starts, const int64_t* seq_ids, int batch,
                          int num_rows, const int32_t* num_rows_dev, int kv_heads, int head_dim, void* k_cache,
                          void* v_cache, void* dv, void* stream);

/* RMSNorm with the residual add fused in (bf16 in / out, fp32 statistics):
 *   s = x + residual_in (residual_in null = 0);  residual_out = bf16(s) (nullable);
 *   y = bf16( bf16(s * rsqrt(mean(s^2) + eps)) * weight ).
 * width % 8 == 0, width <= 8192.  y may alias x, residual_out may alias residual_in.
 * ref: dyllm/model_executor/layers/layernorm.py:17-53 (RMSNorm.rms_forward / add_rms_forward). */
int dyllm_add_rms_norm(const void* x, const void* residual_in, const void* weight, float eps, void* y,
                       void* residual_out, int rows, int width, void* stream);

/* The same with x given as equal segments: packed row r is row
 * (r / x_seg_rows) * x_seg_pitch_rows + r % x_seg_rows of x.  This reads a block of every sequence (for
 * example the response rows) straight out of an activation cache whose sequences have equal lengths,
 * instead of a packed copy made by dyllm_cache_get_block.  residual_in, y, residual_out are packed. */
int dyllm_add_rms_norm_segmented(const void* x, int x_seg_rows, int64_t x_seg_pitch_rows, const void* residual_in,
                                 const void* weight, float eps, void* y, void* residual_out, int rows, int width,
                                 void* stream);

/* The add-RMSNorm with the listed rows' normalised values also written packed in list order (the input of a
 * gathered GEMM of a sparse step, which then needs no row-staging launch):
 *   residual_out[r] = bf16(x[r] + residual_in[r])                 every row r < rows (nullable)
 *   y_all[r]        = the RMSNorm of row r, as dyllm_add_rms_norm     every row (nullable: the post-attention norm of
 *                     a sparse step feeds the FFN of the salient rows and nothing else)
 *   y_sel[m]        = the RMSNorm of row sel_idx[m]                   m < min(sel_max, *sel_count_dev)
 * y_sel is a packed [sel_max, width] tensor.  x may be segmented as for dyllm_add_rms_norm_segmented.
 * ref: dyllm/model_executor/models/llada.py:176-185 (both norms of a layer, hidden_states[idx_salient_row] and
 *      gather_rows_2D after them). */
int dyllm_add_rms_norm_rows(const void* x, int x_seg_rows, int64_t x_seg_pitch_rows, const void* residual_in,
                            const void* weight, float eps, void* y_all, void* residual_out, int rows, int width,
                            const int32_t* sel_idx, int sel_max, const int32_t* sel_count_dev, void* y_sel,
                            void* stream);

/* RMSNorm over the head_dim values of every (row, head) of x [rows, heads, 128] (bf16), in place:
 * x = bf16( bf16(x * rsqrt(mean(x^2) + eps)) * weight ), weight bf16 [128].  num_rows_dev (nullable) bounds the
 * rows on the device.  The per-head q / k normalisation of LLaDA-MoE.
 * ref: dyllm/model_executor/models/lladamoe.py:175-176,195-207 (q_norm / k_norm on reshape(-1, head_dim)),
 *      dyllm/model_executor/layers/layernorm.py:17-29. */
int dyllm_head_rms_norm(void* x, const void* weight, float eps, int rows, const int32_t* num_rows_dev, int heads,
                        int head_dim, void* stream);

/* Confidence of the most likely token per row of bf16 logits [rows, vocab] (row pitch in elements,
 * multiple of 8): conf[r] = max_j softmax(logits[r])_j in fp32, token[r] = the first j attaining the maximum.
 * Replaces softmax + max over fp32 copies of the candidate logits.
 * ref: dyllm/model_executor/layers/sampler.py:286-288 (F.softmax, probs.max). */
int dyllm_row_confidence(const void* logits, int rows, int vocab, int64_t pitch, float* conf, int64_t* token,
                         void* stream);

/* The unmasking rule of the confidence sampler for the current block of every sequence, on the device:
 * block = min(*step_counter / steps_per_block, num_blocks - 1) (step_counter null = block 0), candidates =
 * the block's positions prompt_len + block * block_len + i, i < block_len, that still hold mask_id in
 * tokens [batch, seq_pitch] (int64); conf / best_token [batch, block_len] are their confidences and most likely
 * tokens (dyllm_row_confidence).  The num_transfer most confident candidates (ties: the lowest position) get
 * their token written into `tokens`; their positions go to picked_pos [batch, num_transfer] in ascending order
 * (-1 padding when fewer masked candidates were left) and their number to picked_count [batch] (nullable).
 * block_len <= 1024, num_transfer <= 64.  Replaces the gather / compare / where / top-k / sort / scatter sequence
 * of torch kernels a step driver would issue.
 * ref: dyllm/model_executor/layers/sampler.py:244-315 (scores sorted per sequence, the first num_transfer kept;
 *      the Triton helpers ragged_to_dense_kernel / filter_and_count_kernel, sampler.py:43-175),
 *      dyllm/engine/sequence.py:69-75 (update_token). */
int dyllm_confidence_unmask(const float* conf, const int64_t* best_token, int64_t* tokens, int batch,
                            int64_t seq_pitch, const int64_t* step_counter, int steps_per_block, int num_blocks,
                            int prompt_len, int block_len, int num_transfer, int64_t mask_id, int64_t* picked_pos,
                            int32_t* picked_count, void* stream);

/* NeoX-style rotary embedding applied in place to x [rows, heads, 128] (bf16): row r uses the angle
 * table row of positions[pos_idx ? pos_idx[r] : r], clamped to [0, max_pos); cos_sin is fp32
 * [max_pos, 128] = cos(64) | sin(64).  num_rows_dev (nullable) bounds the rows on the device.
 * ref: dyllm/model_executor/layers/rotary_embedding.py:8-54. */
int dyllm_rope_neox(void* x, const int64_t* positions, const int64_t* pos_idx, const float* cos_sin, int rows,
                    const int32_t* num_rows_dev, int heads, int head_dim, int max_pos, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Tensor-parallel SUM exchange of the small per-layer tensors over peer memory (NVLink)
 *
 * One communicator per rank (process) and GPU.  Every rank owns a region of
 * 1024 + 2 * world * slot_bytes bytes; all regions are mapped into every process (CUDA IPC), or handed
 * over as plain pointers when several ranks are emulated inside one process.  An exchange is a `push`
 * (each rank stores its partial tensor into its slot of every rank's region and raises a flag there; only
 * stores cross NVLink) followed by a `reduce` (each rank waits for the flags of its own region and adds
 * the slots in rank order in fp32, so that all ranks hold bit-identical results).  Both are ordinary
 * kernels on the caller's stream: they read the live row count on the device and can be captured into a
 * CUDA graph.  Every rank must issue the same sequence of exchanges.  A flag wait gives up after a time
 * limit (default 2 s): the kernel then skips its sums, dyllm_device_status() reports 0x7E00 + the rank
 * whose flag was missing, and the device stays usable.
 * ---------------------------------------------------------------------------------------------- */

/* Creates the communicator of `rank` (0 <= rank < world <= 8) on the current device and allocates its
 * region (set-up time; this is the one call of this group that allocates).  slot_bytes (multiple of 256)
 * bounds the bytes one rank contributes to one exchange. */
int dyllm_tp_comm_create(int rank, int world, size_t slot_bytes, void** comm_out);
/* Size and device address of the local region. */
size_t dyllm_tp_comm_region_bytes(void* comm);
void* dyllm_tp_comm_region(void* comm);
/* 64-byte CUDA IPC handle of the local region, to be sent to the other ranks (any transport). */
int dyllm_tp_comm_ipc_handle(void* comm, void* handle64);
/* Maps the other ranks' regions from their handles (world * 64 bytes, indexed by rank).  All ranks must
 * synchronise with each other after this call and before their first exchange. */
int dyllm_tp_comm_open_ipc(void* comm, const void* handles);
/* The same for ranks that live in one process: regions[r] = dyllm_tp_comm_region(comm of rank r). */
int dyllm_tp_comm_open_local(void* comm, void* const* regions);
/* Time limit of a flag wait. */
int dyllm_tp_comm_set_wait_ms(void* comm, int milliseconds);
/* Synchronises the device, unmaps the peers' regions and frees the local one. */
int dyllm_tp_comm_destroy(void* comm);

/* SUM all-reduce of the live rows [row_offset, min(row_offset + max_rows, *count_dev)) of a compact bf16
 * [rows, width] tensor whose first row is row `row_offset` (count_dev null = max_rows rows), written to
 * out[map[row_offset + m]] (out_row_map null = row_offset + m; negative entries drop the row; ldo = row
 * pitch of out in elements).  width % 8 == 0, max_rows * width * 2 <= slot_bytes.  The count must be the
 * same on every rank.  dyllm_tp_allreduce_rows = dyllm_tp_push_rows + dyllm_tp_reduce_rows.
 * ref: dyllm/model_executor/layers/linear.py:216-220 (all_reduce after the row-parallel down projection),
 *      dyllm/model_executor/models/lladamoe.py:103-104,141 (expert outputs),
 *      dyllm/model_executor/layers/mlp_cache_manage.py:24-40 (scatter into the FFN-output cache). */
int dyllm_tp_push_rows(void* comm, const void* src, int width, int max_rows, const int32_t* count_dev,
                       int row_offset, void* stream);
int dyllm_tp_reduce_rows(void* comm, int width, int max_rows, const int32_t* count_dev, int row_offset, void* out,
                         int64_t ldo, const int32_t* out_row_map, void* stream);
int dyllm_tp_allreduce_rows(void* comm, const void* src, int width, int max_rows, const int32_t* count_dev,
                            int row_offset, void* out, int64_t ldo, const int32_t* out_row_map, void* stream);

/* Row gather of the sequence-sharded layout (every rank runs attention and the all-row projections for its
 * own sequences; the FFN / expert weights are sharded over the ranks).  Every rank contributes the rows
 * x[idx[m]] (idx null = identity), m < min(max_rows, *count_dev), of its bf16 [x_rows, width] activation
 * (row pitch ldx); afterwards every rank holds all contributions, ordered by rank, in the data area of its
 * region (dyllm_tp_comm_data: a bf16 matrix of 2 * world * (slot_bytes / (2 * width)) rows of `width`), and
 *   idx_all[0..total)   row numbers of the gathered rows inside that matrix (feed them, with the matrix as
 *                       x, to dyllm_swiglu_ffn / dyllm_moe_route / dyllm_moe_ffn as their index list)
 *   prefix[0..world]    number of rows contributed by the ranks before r
 *   total_out[0]        prefix[world]
 * The counts may differ from rank to rank.  slot_bytes must be a whole number of rows >= max_rows.
 * dyllm_tp_gather_rows = dyllm_tp_gather_push + dyllm_tp_gather_finish (the split form lets a test run
 * several emulated ranks one after the other).  No counterpart in the reference, whose tensor-parallel
 * ranks all hold every row (dyllm/model_executor/models/llada.py:184-186 gathers locally). */
int dyllm_tp_gather_rows(void* comm, const void* x, int x_rows, int width, int64_t ldx, const int32_t* idx,
                         int max_rows, const int32_t* count_dev, int32_t* idx_all, int32_t* prefix,
                         int32_t* total_out, void* stream);
int dyllm_tp_gather_push(void* comm, const void* x, int x_rows, int width, int64_t ldx, const int32_t* idx,
                         int max_rows, const int32_t* count_dev, void* stream);
int dyllm_tp_gather_finish(void* comm, int width, int32_t* idx_all, int32_t* prefix, int32_t* total_out,
                           void* stream);
void* dyllm_tp_comm_data(void* comm);
/* The way back: y holds one partial output row per gathered row (same order); row m goes to the rank that
 * contributed it (prefix from the gather), into the pushing rank's slot there.  The owner then calls
 * dyllm_tp_reduce_rows with its own count to add the world slots in rank order and scatter the sums.
 * ref: dyllm/model_executor/layers/linear.py:216-220 (SUM over the ranks' partial down projections). */
int dyllm_tp_scatter_push(void* comm, const void* y, int width, int max_rows, const int32_t* prefix, void* stream);

/* In-place SUM all-reduce of n fp32 values (the [rows, 3] cosine statistics, 12 bytes per token).
 * ref: dyllm/distributed/parallel_state.py:60-61. */
int dyllm_tp_push_f32(void* comm, const float* src, int n, void* stream);
int dyllm_tp_reduce_f32(void* comm, float* out, int n, void* stream);
int dyllm_tp_allreduce_f32(void* comm, float* inout, int n, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* DYLLM_B200_H_ */
