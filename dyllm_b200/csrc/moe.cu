// Mixture-of-experts FFN on salient rows: softmax top-k router, expert-sorted grouped GEMMs on the
// tcgen05 kernel of gemm.cuh (one weight block per 128-row tile), routing weight folded into the
// down-projection epilogue, per-token sum over the top-k slots.
//
//   route    logits = x[idx[m]] . Wr^T (fp32), softmax over experts, top-k           (one block per row)
//   align    (row, slot) pairs grouped by expert, every group padded to 128 rows  (one block)
//   GEMM 1   h = silu(x Wg_e^T) * (x Wu_e^T) for the rows of each tile's expert
//   GEMM 2   y[pair] = w_pair * (h Wd_e^T)
//   combine  out[map[m]] = sum over the owned slots of row m of y[m * k + j]
#include "gemm.cuh"

namespace dyllm {

int launch_gathered_gemm(bool swiglu, int a_mode, int tile_n, const GemmParams& p_in, int64_t lda, const void* b,
                         int64_t b_total_rows, int n, int rows_hint, float* partial, cudaStream_t stream);
int stage_rows(const void* x, int64_t ldx, const int32_t* idx, int x_rows, void* compact, int width, int num_rows,
               const int32_t* num_rows_dev, int rows_hint, cudaStream_t stream);

namespace {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 16;

// One block (256 threads) per row: 8 warps split the experts, lanes split the hidden dimension.
__global__ void __launch_bounds__(256)
moe_route_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const int32_t* __restrict__ idx, int x_rows,
                 int num_rows, const int32_t* __restrict__ num_rows_dev, const __nv_bfloat16* __restrict__ wr,
                 int hidden, int num_experts, int top_k, int renormalize, float* __restrict__ topk_w,
                 int32_t* __restrict__ topk_ids) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  __shared__ float s_logits[kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int m = blockIdx.x; m < n; m += gridDim.x) {
    const int r = idx ? min(max(idx[m], 0), x_rows - 1) : m;
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(r) * ldx);
    const int vecs = hidden / 8;
    for (int e = warp; e < num_experts; e += 8) {
      const uint4* w = reinterpret_cast<const uint4*>(wr + static_cast<int64_t>(e) * hidden);
      float acc = 0.f;
      for (int v = lane; v < vecs; v += 32) {
        const uint4 a = __ldg(xr + v), b = __ldg(w + v);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fa = __bfloat1622float2(a2[i]), fb = __bfloat1622float2(b2[i]);
          acc = fmaf(fa.x, fb.x, acc);
          acc = fmaf(fa.y, fb.y, acc);
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (lane == 0)
        s_logits[e] = acc;
    }
    __syncthreads();
    if (warp == 0) {
      // softmax over the experts, then top-k by repeated arg-max (lowest index wins ties)
      float mx = -3.0e38f;
      for (int e = lane; e < num_experts; e += 32)
        mx = fmaxf(mx, s_logits[e]);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      float sum = 0.f;
      for (int e = lane; e < num_experts; e += 32) {
        const float pe = expf(s_logits[e] - mx);
        s_logits[e] = pe;
        sum += pe;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
      __syncwarp();
      const float inv = 1.0f / sum;
      float picked_w = 0.f, total = 0.f;
      int picked_e = 0;
      for (int j = 0; j < top_k; ++j) {
        float best = -1.f;
        int best_e = 0x7fffffff;
        for (int e = lane; e < num_experts; e += 32) {
          const float v = s_logits[e];
          if (v > best) {
            best = v;
            best_e = e;
          }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, off);
          const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
          if (ob > best || (ob == best && oe < best_e)) {
            best = ob;
            best_e = oe;
          }
        }
        if (lane == 0)
          s_logits[best_e] = -1.f;  // taken
        __syncwarp();
        if (lane == j) {
          picked_w = best * inv;
          picked_e = best_e;
        }
        total += best * inv;
      }
      if (lane < top_k) {
        const float w = renormalize ? picked_w / total : picked_w;
        // the reference hands the routing weights on in the activation dtype (bf16)
        topk_w[static_cast<int64_t>(m) * top_k + lane] = __bfloat162float(__float2bfloat16(w));
        topk_ids[static_cast<int64_t>(m) * top_k + lane] = picked_e;
      }
    }
    __syncthreads();
  }
}

// Single block: groups the owned (row, slot) pairs by local expert, pads every group to 128 rows and
// writes, per padded position, the source row, the destination pair and the routing weight.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w, int num_rows,
                 const int32_t* __restrict__ num_rows_dev, int top_k, int expert_start, int num_local_experts,
                 const int32_t* __restrict__ row_src, int32_t* __restrict__ a_idx, int32_t* __restrict__ pair_idx,
                 float* __restrict__ pair_w, int32_t* __restrict__ tile_expert, int32_t* __restrict__ m_total,
                 int capacity) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  __shared__ int s_count[kMaxExperts];
  __shared__ int s_start[kMaxExperts + 1];
  __shared__ int s_fill[kMaxExperts];
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  const int pairs = n * top_k;
  for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x) {
    s_count[e] = 0;
    s_fill[e] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i] - expert_start;
    if (e >= 0 && e < num_local_experts)
      atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int pos = 0;
    for (int e = 0; e < num_local_experts; ++e) {
      s_start[e] = pos;
      pos += (s_count[e] + kGemmBM - 1) / kGemmBM * kGemmBM;
    }
    s_start[num_local_experts] = pos;
    *m_total = pos < capacity ? pos : capacity;
  }
  __syncthreads();
  const int total = min(s_start[num_local_experts], capacity);
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    a_idx[i] = -1;
    pair_idx[i] = -1;
    pair_w[i] = 0.f;
  }
  for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x)
    for (int t = s_start[e] / kGemmBM; t < s_start[e + 1] / kGemmBM; ++t)
      tile_expert[t] = e;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i] - expert_start;
    if (e < 0 || e >= num_local_experts)
      continue;
    const int pos = s_start[e] + atomicAdd(&s_fill[e], 1);
    if (pos >= capacity)
      continue;
    const int row = i / top_k;
    a_idx[pos] = row_src ? row_src[row] : row;
    pair_idx[pos] = i;
    pair_w[pos] = topk_w[i];
  }
}

// out[map[m]] = bf16( sum over the owned slots j of y[m * k + j] ), fp32 accumulation in slot order.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ topk_ids, int num_rows,
                   const int32_t* __restrict__ num_rows_dev, int top_k, int expert_start, int num_local_experts,
                   int hidden, __nv_bfloat16* __restrict__ out, int64_t ldo, const int32_t* __restrict__ out_row_map) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  const int vecs = hidden / 8;
  for (int m = blockIdx.x; m < n; m += gridDim.x) {
    const int dst_row = out_row_map ? out_row_map[m] : m;
    if (dst_row < 0)
      continue;
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < top_k; ++j) {
        const int e = topk_ids[static_cast<int64_t>(m) * top_k + j] - expert_start;
        if (e < 0 || e >= num_local_experts)
          continue;
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(y + (static_cast<int64_t>(m) * top_k + j) * hidden) + v);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(a2[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
      uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                           pack_bf16x2(acc[6], acc[7]));
      reinterpret_cast<uint4*>(out + static_cast<int64_t>(dst_row) * ldo)[v] = o;
    }
  }
}

size_t align_up_sz(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct MoeLayout {
  int capacity;        // padded (row, slot) positions
  size_t off_a_idx, off_pair_idx, off_pair_w, off_tile_expert, off_m_total, off_staged, off_inter, off_y, total;
};

MoeLayout moe_layout(int max_rows, int top_k, int num_local_experts, int hidden, int inter) {
  MoeLayout l;
  const int64_t pairs = static_cast<int64_t>(max_rows) * top_k;
  const int64_t cap = (pairs + static_cast<int64_t>(num_local_experts) * (kGemmBM - 1) + kGemmBM - 1) / kGemmBM * kGemmBM;
  l.capacity = static_cast<int>(cap);
  size_t off = 0;
  l.off_a_idx = off;       off = align_up_sz(off + cap * 4, 1024);
  l.off_pair_idx = off;    off = align_up_sz(off + cap * 4, 1024);
  l.off_pair_w = off;      off = align_up_sz(off + cap * 4, 1024);
  l.off_tile_expert = off; off = align_up_sz(off + (cap / kGemmBM) * 4, 1024);
  l.off_m_total = off;     off = align_up_sz(off + 16, 1024);
  l.off_staged = off;      off = align_up_sz(off + cap * static_cast<size_t>(hidden) * 2, 1024);
  l.off_inter = off;       off = align_up_sz(off + cap * static_cast<size_t>(inter) * 2, 1024);
  l.off_y = off;           off = align_up_sz(off + static_cast<size_t>(pairs) * hidden * 2, 1024);
  l.total = off;
  return l;
}

}  // namespace
}  // namespace dyllm

using namespace dyllm;

extern "C" {

int dyllm_moe_route(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                    const int32_t* num_rows_dev, const void* router_weight, int num_experts, int top_k,
                    int renormalize, float* topk_weights, int32_t* topk_ids, void* stream) {
  DYLLM_REQUIRE(x_rows >= 0 && num_rows >= 0 && hidden > 0, DYLLM_ERR_INVALID_ARGUMENT, "moe_route: rows %d hidden %d",
                num_rows, hidden);
  DYLLM_REQUIRE(num_experts > 0 && num_experts <= kMaxExperts && top_k > 0 && top_k <= kMaxTopK && top_k <= num_experts,
                DYLLM_ERR_UNSUPPORTED, "moe_route: %d experts (max %d), top-%d (max %d)", num_experts, kMaxExperts,
                top_k, kMaxTopK);
  DYLLM_REQUIRE(hidden % 8 == 0 && ldx % 8 == 0, DYLLM_ERR_UNSUPPORTED, "moe_route: hidden and pitch must be multiples of 8");
  if (num_rows == 0 || x_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && router_weight && topk_weights && topk_ids, DYLLM_ERR_INVALID_ARGUMENT, "moe_route: null pointer");
  const int blocks = min(num_rows, sm_count() * 8);
  DYLLM_LAUNCH(moe_route_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), ldx, idx, x_rows, num_rows, num_rows_dev,
      static_cast<const __nv_bfloat16*>(router_weight), hidden, num_experts, top_k, renormalize, topk_weights, topk_ids);
  return check_launch("moe_route");
}

size_t dyllm_moe_ffn_workspace_bytes(int max_rows, int top_k, int num_local_experts, int hidden, int inter) {
  if (max_rows <= 0 || top_k <= 0 || num_local_experts <= 0 || hidden <= 0 || inter <= 0)
    return 0;
  return moe_layout(max_rows, top_k, num_local_experts, hidden, inter).total;
}

int dyllm_moe_ffn(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                  const int32_t* num_rows_dev, int rows_hint, const float* topk_weights, const int32_t* topk_ids,
                  int top_k, const void* w1, const void* w2, int num_local_experts, int expert_start, int inter,
                  void* out, int64_t ldo, const int32_t* out_row_map, void* workspace, size_t workspace_bytes,
                  void* stream) {
  DYLLM_REQUIRE(x_rows >= 0 && num_rows >= 0 && hidden > 0 && inter > 0, DYLLM_ERR_INVALID_ARGUMENT,
                "moe_ffn: rows %d hidden %d inter %d", num_rows, hidden, inter);
  DYLLM_REQUIRE(num_local_experts > 0 && num_local_experts <= kMaxExperts && top_k > 0 && top_k <= kMaxTopK,
                DYLLM_ERR_UNSUPPORTED, "moe_ffn: %d local experts (max %d), top-%d (max %d)", num_local_experts,
                kMaxExperts, top_k, kMaxTopK);
  DYLLM_REQUIRE(hidden % 64 == 0 && inter % 64 == 0 && ldx % 8 == 0 && ldo % 8 == 0, DYLLM_ERR_UNSUPPORTED,
                "moe_ffn: hidden and inter must be multiples of 64, pitches of 8");
  if (num_rows == 0 || x_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && topk_weights && topk_ids && w1 && w2 && out && workspace, DYLLM_ERR_INVALID_ARGUMENT,
                "moe_ffn: null pointer");
  const MoeLayout l = moe_layout(num_rows, top_k, num_local_experts, hidden, inter);
  DYLLM_REQUIRE(workspace_bytes >= l.total && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0, DYLLM_ERR_WORKSPACE,
                "moe_ffn: needs a 16-byte aligned workspace of %zu bytes (got %zu)", l.total, workspace_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* a_idx = reinterpret_cast<int32_t*>(ws + l.off_a_idx);
  int32_t* pair_idx = reinterpret_cast<int32_t*>(ws + l.off_pair_idx);
  float* pair_w = reinterpret_cast<float*>(ws + l.off_pair_w);
  int32_t* tile_expert = reinterpret_cast<int32_t*>(ws + l.off_tile_expert);
  int32_t* m_total = reinterpret_cast<int32_t*>(ws + l.off_m_total);
  void* staged = ws + l.off_staged;
  __nv_bfloat16* inter_buf = reinterpret_cast<__nv_bfloat16*>(ws + l.off_inter);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(ws + l.off_y);

  DYLLM_LAUNCH(moe_align_kernel, 1, 1024, 0, s, topk_ids, topk_weights, num_rows, num_rows_dev, top_k, expert_start,
                                      num_local_experts, idx, a_idx, pair_idx, pair_w, tile_expert, m_total, l.capacity);
  int rc = check_launch("moe_align");
  if (rc != DYLLM_OK)
    return rc;
  const int hint_rows = rows_hint > 0 && rows_hint < num_rows ? rows_hint : num_rows;
  int64_t hint64 = static_cast<int64_t>(hint_rows) * top_k + static_cast<int64_t>(num_local_experts) * (kGemmBM / 2);
  const int hint = hint64 < l.capacity ? static_cast<int>(hint64) : l.capacity;

  // rows of x for every padded position (padding reads row 0), then plain TMA boxes
  rc = stage_rows(x, ldx, a_idx, x_rows, staged, hidden, l.capacity, m_total, hint, s);
  if (rc != DYLLM_OK)
    return rc;
  GemmParams g1 = {};
  g1.a = static_cast<const __nv_bfloat16*>(staged);
  g1.a_rows = l.capacity;
  g1.m_count_dev = m_total;
  g1.tile_expert = tile_expert;
  g1.M = l.capacity;
  g1.K = hidden;
  g1.b_rows_per_expert = 2 * inter;
  g1.up_row_offset = inter;
  g1.out = inter_buf;
  g1.ldc = inter;
  rc = launch_gathered_gemm(true, 0, 0, g1, hidden, w1, static_cast<int64_t>(num_local_experts) * 2 * inter, inter, hint,
                            nullptr, s);
  if (rc != DYLLM_OK)
    return rc;
  GemmParams g2 = {};
  g2.a = inter_buf;
  g2.a_rows = l.capacity;
  g2.m_count_dev = m_total;
  g2.tile_expert = tile_expert;
  g2.M = l.capacity;
  g2.K = inter;
  g2.b_rows_per_expert = hidden;
  g2.out = y;
  g2.ldc = hidden;
  g2.out_row_map = pair_idx;
  g2.row_scale = pair_w;
  rc = launch_gathered_gemm(false, 0, 0, g2, inter, w2, static_cast<int64_t>(num_local_experts) * hidden, hidden, hint,
                            nullptr, s);
  if (rc != DYLLM_OK)
    return rc;
  const int blocks = min(hint_rows, sm_count() * 8);
  DYLLM_LAUNCH(moe_combine_kernel, blocks < 1 ? 1 : blocks, 256, 0, s, y, topk_ids, num_rows, num_rows_dev, top_k, expert_start,
                                                            num_local_experts, hidden, static_cast<__nv_bfloat16*>(out),
                                                            ldo, out_row_map);
  return check_launch("moe_combine");
}

}  // extern "C"
