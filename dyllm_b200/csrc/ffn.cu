// Gathered linear layers and the SwiGLU FFN on salient rows:
//   out[map[m]] = down( silu(x[idx[m]] Wg^T) * (x[idx[m]] Wu^T) )
// built from the tcgen05 GEMM in gemm.cuh: gate/up with the activation fused in the epilogue, then the
// down projection whose epilogue scatters rows to their destination.  Activation rows reach the GEMM
// either through a small staging copy (rows gathered once into a compact buffer, then plain TMA boxes)
// or directly by TMA gather4.  Launch shapes are chosen from a row-count hint; the live row count is
// read on the device, so no host synchronisation is needed.
#include <atomic>

#include "gemm.cuh"

namespace dyllm {

constexpr int kSplitRows = 512;   // split-K partial sums are kept for at most this many live rows
constexpr int kMaxSplits = 4;

namespace {

template <int BNH, bool SWIGLU, int A_MODE, int STAGES, int MINB, int MT = 1>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BNH, SWIGLU, STAGES, MT>;
  auto kernel = gathered_gemm_kernel<BNH, SWIGLU, A_MODE, STAGES, MINB, MT>;
  // one flag per kernel instantiation and device: the opt-in shared-memory size is a per-function attribute
  static std::atomic<bool> smem_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev < 0 || dev >= 64) ? 0 : dev;
  if (!smem_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(Cfg::SMEM_BYTES)) != cudaSuccess)
      return set_error(DYLLM_ERR_CUDA, "cudaFuncSetAttribute(%u bytes of shared memory) failed: %s", Cfg::SMEM_BYTES,
                       cudaGetErrorString(cudaGetLastError()));
    smem_set[dev].store(true, std::memory_order_release);
  }
  DYLLM_LAUNCH(kernel, grid, kGemmThreads, Cfg::SMEM_BYTES, stream, ta, tb, p);
  return check_launch("gathered_gemm");
}

template <int BNH, bool SWIGLU, int STAGES, int MINB = 1>
int launch_mode(int a_mode, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, dim3 grid,
                cudaStream_t stream) {
  if (a_mode == 0)
    return launch_one<BNH, SWIGLU, 0, STAGES, MINB>(ta, tb, p, grid, stream);
  return launch_one<BNH, SWIGLU, 1, STAGES, MINB>(ta, tb, p, grid, stream);
}

// compact[m] = x[idx[m]] for the live rows; one warp per row, 16-byte accesses.
__global__ void __launch_bounds__(256)
stage_rows_kernel(const uint4* __restrict__ x, int64_t x_pitch_vecs, const int32_t* __restrict__ idx, int x_rows,
                  uint4* __restrict__ compact, int vecs, int num_rows, const int32_t* __restrict__ num_rows_dev) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int m = blockIdx.x * 8 + warp; m < n; m += gridDim.x * 8) {
    const int r = min(max(idx[m], 0), x_rows - 1);
    const uint4* src = x + static_cast<int64_t>(r) * x_pitch_vecs;
    uint4* dst = compact + static_cast<int64_t>(m) * vecs;
    int v = lane;
    for (; v + 96 < vecs; v += 128) {
      const uint4 a = __ldg(src + v), b = __ldg(src + v + 32), c = __ldg(src + v + 64), d = __ldg(src + v + 96);
      dst[v] = a;
      dst[v + 32] = b;
      dst[v + 64] = c;
      dst[v + 96] = d;
    }
    for (; v < vecs; v += 32)
      dst[v] = __ldg(src + v);
  }
}

struct Plan {
  int tile_n;
  int splits;
  bool two_per_sm;   // narrow tiles, half-depth pipeline, two CTAs per SM (weight-streaming regime)
  bool tall;         // 256-row tiles (two accumulators per weight tile) for many rows
  int slots;         // CTAs resident at once
  dim3 grid;
};

// Launch shape from the row-count hint: tile width so that the expected tiles fill the SMs, split-K
// when even the narrow tiles leave most SMs idle, one grid row per expected row tile.
Plan make_plan(bool swiglu, int M, int hint, int n, int K, int tile_n, bool can_split, bool allow_tall) {
  const int sms = sm_count();
  const int h = (hint > 0 && hint < M) ? hint : M;
  const int mt_h = cdiv_i(h, kGemmBM);
  Plan plan;
  if (tile_n == 0) {
    tile_n = (n % 128 == 0 && mt_h * (n / 128) >= sms * 3 / 4) ? 128 : 64;
    // Many rows, plain product: 256 x 256 tiles.  The MMA warp issues one tcgen05.mma per ~68 clocks, which is
    // what an N = 128 product keeps the tensor pipe busy for; N = 256 doubles the work per instruction, and the
    // tile moves 62 B/clk of operands from L2 where 256 x 128 moves 94.
    if (!swiglu && allow_tall && n % 256 == 0 && h > 256 && cdiv_i(h, 2 * kGemmBM) * (n / 256) >= sms * 3 / 4)
      tile_n = 256;
  }
  plan.tile_n = tile_n;
  const int n_tiles = n / tile_n;
  // many rows: the 128-row tile is limited by weight traffic from L2; 256-row tiles halve it
  plan.tall = allow_tall && h > 256 &&
              ((tile_n == 128 && cdiv_i(h, 2 * kGemmBM) * n_tiles >= sms) ||
               (tile_n == 256 && cdiv_i(h, 2 * kGemmBM) * n_tiles >= sms * 3 / 4));
  plan.two_per_sm = tile_n == 64 && mt_h <= 2;
  plan.slots = plan.two_per_sm ? 2 * sms : sms;
  // the grid carries the splits a single live row tile would use; CTAs of splits that the live count
  // does not need return at once
  plan.splits = 1;
  if (!swiglu && can_split && !plan.tall && h <= kSplitRows)
    plan.splits = effective_splits(1, n_tiles, plan.slots, kMaxSplits, K / kGemmBK);
  const int bm = plan.tall ? 2 * kGemmBM : kGemmBM;
  int m_groups = cdiv_i(h, bm);
  // a count above the hint is served by extra grid rows (they return at once when not needed) before
  // CTAs have to walk over several row tiles
  if (h <= kSplitRows && m_groups < kSplitRows / kGemmBM)
    m_groups = kSplitRows / kGemmBM;
  const int mt_all = cdiv_i(M, bm);
  m_groups = m_groups > mt_all ? mt_all : m_groups;
  plan.grid = dim3(n_tiles, plan.splits, m_groups < 1 ? 1 : m_groups);   // row groups last: see gemm.cuh
  return plan;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t padded_rows(int rows) { return static_cast<size_t>(cdiv_i(rows, kGemmBM)) * kGemmBM; }

// dest[m] = seq_starts[seq_ids[b]] + (row_idx[m] - cu[b]) for m < n, -1 beyond the live rows.
__global__ void cache_dest_rows_kernel(const int64_t* __restrict__ row_idx, const int32_t* __restrict__ cu,
                                       const int64_t* __restrict__ seq_starts, const int64_t* __restrict__ seq_ids,
                                       int batch, int num_rows, const int32_t* __restrict__ num_rows_dev,
                                       int32_t* __restrict__ dest) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  for (int m = blockIdx.x * blockDim.x + threadIdx.x; m < num_rows; m += gridDim.x * blockDim.x) {
    if (m >= n) {
      dest[m] = -1;
      continue;
    }
    const int64_t r = row_idx[m];
    int lo = 0, hi = batch;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (cu[mid + 1] <= r)
        lo = mid + 1;
      else
        hi = mid;
    }
    const int b = lo < batch ? lo : batch - 1;
    dest[m] = static_cast<int32_t>(seq_starts[seq_ids[b]] + (r - cu[b]));
  }
}

}  // namespace

// a_mode: 0 = A rows m0..m0+127 by one TMA box (A dense or already staged), 1 = TMA gather4 through
// p.a_idx.  n is the number of output columns per weight block (the intermediate size for SWIGLU).
// tile_n: 64, 128 or (many rows, no SwiGLU) 256 (0 = choose).  `partial` enables split-K for the non-SwiGLU GEMM.
int launch_gathered_gemm(bool swiglu, int a_mode, int tile_n, const GemmParams& p_in, int64_t lda, const void* b,
                         int64_t b_total_rows, int n, int rows_hint, float* partial, cudaStream_t stream) {
  GemmParams p = p_in;
  DYLLM_REQUIRE(p.K > 0 && p.K % kGemmBK == 0, DYLLM_ERR_UNSUPPORTED, "gemm: K = %d is not a multiple of 64", p.K);
  DYLLM_REQUIRE(n > 0 && n % 64 == 0, DYLLM_ERR_UNSUPPORTED, "gemm: N = %d is not a multiple of 64", n);
  DYLLM_REQUIRE(lda % 8 == 0 && p.ldc % 8 == 0 && p.ldc2 % 8 == 0, DYLLM_ERR_UNSUPPORTED,
                "gemm: row pitches must be multiples of 8");
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out2) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "gemm: operands must be 16-byte aligned");
  DYLLM_REQUIRE(a_mode == 0 || a_mode == 1, DYLLM_ERR_INVALID_ARGUMENT, "gemm: a_mode %d", a_mode);
  DYLLM_REQUIRE(!(a_mode == 0 && p.a_idx), DYLLM_ERR_INVALID_ARGUMENT, "gemm: a_mode 0 cannot gather");
  DYLLM_REQUIRE(!p.out2 || (p.split_col > 0 && p.split_col % 128 == 0 && p.split_col < n), DYLLM_ERR_INVALID_ARGUMENT,
                "gemm: split column %d must be a multiple of 128 inside (0, %d)", p.split_col, n);
  if (p.M <= 0)
    return DYLLM_OK;
  const Plan plan = make_plan(swiglu, p.M, rows_hint, n, p.K, tile_n, partial != nullptr,
                              a_mode == 0 && !p.tile_expert);
  DYLLM_REQUIRE((plan.tile_n == 64 || plan.tile_n == 128 || (plan.tile_n == 256 && plan.tall && !swiglu)) &&
                    n % plan.tile_n == 0,
                DYLLM_ERR_UNSUPPORTED,
                "gemm: tile_n %d does not divide N = %d", plan.tile_n, n);
  p.status_word = device_status_word();
  p.n_total = n;
  p.partial = plan.splits > 1 ? partial : nullptr;
  p.split_tickets = split_tickets();
  if (!p.split_tickets || static_cast<int64_t>(plan.grid.x) * (kSplitRows / kGemmBM) > kSplitTicketCount)
    p.partial = nullptr;   // no counters for this many tiles: every CTA runs its whole k range
  p.split_rows = kSplitRows;
  p.split_slots = plan.slots;

  CUtensorMap ta, tb;
  int rc;
  if (a_mode == 0)
    rc = encode_tmap_2d_bf16(&ta, p.a, p.a_rows, p.K, lda, plan.tall ? 2 * kGemmBM : kGemmBM, kGemmBK, true);
  else
    rc = encode_tmap_2d_bf16(&ta, p.a, p.a_rows, p.K, lda, 1, kGemmBK, true);
  if (rc != DYLLM_OK)
    return rc;
  rc = encode_tmap_2d_bf16(&tb, b, b_total_rows, p.K, p.K, plan.tile_n, kGemmBK, true);
  if (rc != DYLLM_OK)
    return rc;

  if (plan.tall) {
    if (swiglu)
      rc = launch_one<128, true, 0, 3, 1, 2>(ta, tb, p, plan.grid, stream);
    else if (plan.tile_n == 256)
      rc = launch_one<256, false, 0, 3, 1, 2>(ta, tb, p, plan.grid, stream);
    else
      rc = launch_one<128, false, 0, 4, 1, 2>(ta, tb, p, plan.grid, stream);
  } else if (swiglu) {
    if (plan.tile_n == 128)
      rc = launch_mode<128, true, 4>(a_mode, ta, tb, p, plan.grid, stream);
    else if (plan.two_per_sm)
      rc = launch_mode<64, true, 3, 2>(a_mode, ta, tb, p, plan.grid, stream);
    else
      rc = launch_mode<64, true, 6>(a_mode, ta, tb, p, plan.grid, stream);
  } else if (plan.tile_n == 128) {
    rc = launch_mode<128, false, 6>(a_mode, ta, tb, p, plan.grid, stream);
  } else if (plan.two_per_sm) {
    rc = launch_mode<64, false, 4, 2>(a_mode, ta, tb, p, plan.grid, stream);
  } else {
    rc = launch_mode<64, false, 8>(a_mode, ta, tb, p, plan.grid, stream);
  }
  return rc;
}

int stage_rows(const void* x, int64_t ldx, const int32_t* idx, int x_rows, void* compact, int width, int num_rows,
               const int32_t* num_rows_dev, int rows_hint, cudaStream_t stream) {
  const int h = (rows_hint > 0 && rows_hint < num_rows) ? rows_hint : num_rows;
  int blocks = cdiv_i(h, 8);
  const int cap = sm_count() * 8;
  blocks = blocks > cap ? cap : (blocks < 1 ? 1 : blocks);
  DYLLM_LAUNCH(stage_rows_kernel, blocks, 256, 0, stream, static_cast<const uint4*>(x), ldx / 8, idx, x_rows,
                                               static_cast<uint4*>(compact), width / 8, num_rows, num_rows_dev);
  return check_launch("stage_rows");
}

}  // namespace dyllm

using namespace dyllm;

extern "C" {

size_t dyllm_gathered_linear_workspace_bytes(int max_rows, int in_features, int out_features) {
  if (max_rows <= 0 || in_features <= 0 || out_features <= 0)
    return 0;
  return align_up(padded_rows(max_rows) * static_cast<size_t>(in_features) * 2, 1024) +
         static_cast<size_t>(kMaxSplits) * kSplitRows * out_features * sizeof(float);
}

size_t dyllm_swiglu_ffn_workspace_bytes(int max_rows, int hidden, int inter) {
  if (max_rows <= 0 || inter <= 0 || hidden <= 0)
    return 0;
  const size_t padded = padded_rows(max_rows);
  return align_up(padded * static_cast<size_t>(hidden) * 2, 1024) +
         align_up(padded * static_cast<size_t>(inter) * 2, 1024) +
         static_cast<size_t>(kMaxSplits) * kSplitRows * hidden * sizeof(float);
}

int dyllm_cache_dest_rows(const int64_t* row_idx, const int32_t* cu_seqlens, const int64_t* seq_starts,
                          const int64_t* seq_ids, int batch, int num_rows, const int32_t* num_rows_dev,
                          int32_t* dest_rows, void* stream) {
  DYLLM_REQUIRE(batch >= 0 && num_rows >= 0, DYLLM_ERR_INVALID_ARGUMENT, "cache_dest_rows: batch %d rows %d", batch,
                num_rows);
  if (num_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(row_idx && cu_seqlens && seq_starts && seq_ids && dest_rows && batch > 0, DYLLM_ERR_INVALID_ARGUMENT,
                "cache_dest_rows: null pointer or empty batch");
  const int blocks = min(cdiv_i(num_rows, 256), sm_count() * 4);
  DYLLM_LAUNCH(cache_dest_rows_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), 
      row_idx, cu_seqlens, seq_starts, seq_ids, batch, num_rows, num_rows_dev, dest_rows);
  return check_launch("cache_dest_rows");
}

int dyllm_gathered_linear(const void* x, int x_rows, int in_features, int64_t ldx, const int32_t* idx, int num_rows,
                          const int32_t* num_rows_dev, int rows_hint, const void* weight, int out_features, void* out,
                          int64_t ldo, void* out2, int64_t ldo2, int split_col, const int32_t* out_row_map,
                          const float* row_scale, void* workspace, size_t workspace_bytes, int a_mode, int tile_n,
                          void* stream) {
  DYLLM_REQUIRE(x_rows >= 0 && in_features > 0 && out_features > 0 && num_rows >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "gathered_linear: x_rows %d in %d out %d num_rows %d", x_rows, in_features, out_features, num_rows);
  if (num_rows == 0 || x_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && weight && out, DYLLM_ERR_INVALID_ARGUMENT, "gathered_linear: null pointer");
  if (a_mode < 0)
    a_mode = 0;
  DYLLM_REQUIRE(a_mode == 0 || a_mode == 1, DYLLM_ERR_INVALID_ARGUMENT,
                "gathered_linear: a_mode %d (0 = staged rows + TMA boxes, 1 = TMA gather4)", a_mode);
  DYLLM_REQUIRE(in_features % 8 == 0 && ldx % 8 == 0, DYLLM_ERR_UNSUPPORTED,
                "gathered_linear: pitches must be multiples of 8");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t stage_bytes = align_up(padded_rows(num_rows) * static_cast<size_t>(in_features) * 2, 1024);
  const size_t need = dyllm_gathered_linear_workspace_bytes(num_rows, in_features, out_features);
  const bool have_ws = workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0;
  DYLLM_REQUIRE(have_ws || a_mode == 1 || !idx, DYLLM_ERR_WORKSPACE,
                "gathered_linear: staging the gathered rows needs a 16-byte aligned workspace of %zu bytes (got %zu)",
                need, workspace_bytes);

  GemmParams g = {};
  g.a = static_cast<const __nv_bfloat16*>(x);
  g.a_rows = x_rows;
  int64_t lda = ldx;
  int mode = a_mode;
  if (idx && a_mode == 0) {
    int rc = stage_rows(x, ldx, idx, x_rows, workspace, in_features, num_rows, num_rows_dev, rows_hint, s);
    if (rc != DYLLM_OK)
      return rc;
    g.a = static_cast<const __nv_bfloat16*>(workspace);
    g.a_rows = static_cast<int>(padded_rows(num_rows));
    lda = in_features;
  } else if (idx) {
    g.a_idx = idx;
  } else {
    mode = 0;
  }
  g.m_count_dev = num_rows_dev;
  g.M = num_rows;
  g.K = in_features;
  g.b_rows_per_expert = out_features;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ldc = ldo;
  g.out2 = static_cast<__nv_bfloat16*>(out2);
  g.ldc2 = out2 ? ldo2 : 0;
  g.split_col = out2 ? split_col : 0;
  g.out_row_map = out_row_map;
  g.row_scale = row_scale;
  float* partial = have_ws ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + stage_bytes) : nullptr;
  return launch_gathered_gemm(false, mode, tile_n, g, lda, weight, out_features, out_features, rows_hint, partial, s);
}

int dyllm_swiglu_ffn(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                     const int32_t* num_rows_dev, int rows_hint, const void* w_gate_up, const void* w_down, int inter,
                     void* out, int64_t ldo, const int32_t* out_row_map, void* workspace, size_t workspace_bytes,
                     int a_mode, int tile_n, void* stream) {
  DYLLM_REQUIRE(x_rows >= 0 && hidden > 0 && inter > 0 && num_rows >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "swiglu_ffn: x_rows %d hidden %d inter %d num_rows %d", x_rows, hidden, inter, num_rows);
  if (num_rows == 0 || x_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && w_gate_up && w_down && out && workspace, DYLLM_ERR_INVALID_ARGUMENT, "swiglu_ffn: null pointer");
  DYLLM_REQUIRE(workspace_bytes >= dyllm_swiglu_ffn_workspace_bytes(num_rows, hidden, inter), DYLLM_ERR_WORKSPACE,
                "swiglu_ffn: workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
                dyllm_swiglu_ffn_workspace_bytes(num_rows, hidden, inter));
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "swiglu_ffn: workspace must be 16-byte aligned");
  DYLLM_REQUIRE(hidden % 8 == 0 && ldx % 8 == 0, DYLLM_ERR_UNSUPPORTED, "swiglu_ffn: pitches must be multiples of 8");
  if (a_mode < 0)
    a_mode = 0;
  DYLLM_REQUIRE(a_mode == 0 || a_mode == 1, DYLLM_ERR_INVALID_ARGUMENT,
                "swiglu_ffn: a_mode %d (0 = staged rows + TMA boxes, 1 = TMA gather4)", a_mode);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t padded = padded_rows(num_rows);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* staged = ws;
  uint8_t* inter_buf = ws + align_up(padded * static_cast<size_t>(hidden) * 2, 1024);
  float* partial = reinterpret_cast<float*>(inter_buf + align_up(padded * static_cast<size_t>(inter) * 2, 1024));

  GemmParams g1 = {};
  g1.a = static_cast<const __nv_bfloat16*>(x);
  g1.a_rows = x_rows;
  int64_t lda = ldx;
  int mode = a_mode;
  if (idx && a_mode == 0) {
    int rc = stage_rows(x, ldx, idx, x_rows, staged, hidden, num_rows, num_rows_dev, rows_hint, s);
    if (rc != DYLLM_OK)
      return rc;
    g1.a = static_cast<const __nv_bfloat16*>(staged);
    g1.a_rows = static_cast<int>(padded);
    lda = hidden;
  } else if (idx) {
    g1.a_idx = idx;
  } else {
    mode = 0;
  }
  g1.m_count_dev = num_rows_dev;
  g1.M = num_rows;
  g1.K = hidden;
  g1.b_rows_per_expert = 2 * inter;
  g1.up_row_offset = inter;
  g1.out = reinterpret_cast<__nv_bfloat16*>(inter_buf);
  g1.ldc = inter;
  int rc = launch_gathered_gemm(true, mode, tile_n, g1, lda, w_gate_up, 2 * static_cast<int64_t>(inter), inter,
                                rows_hint, nullptr, s);
  if (rc != DYLLM_OK)
    return rc;

  GemmParams g2 = {};
  g2.a = reinterpret_cast<const __nv_bfloat16*>(inter_buf);
  g2.m_count_dev = num_rows_dev;
  g2.M = num_rows;
  g2.K = inter;
  g2.a_rows = static_cast<int>(padded);
  g2.b_rows_per_expert = hidden;
  g2.out = static_cast<__nv_bfloat16*>(out);
  g2.ldc = ldo;
  g2.out_row_map = out_row_map;
  return launch_gathered_gemm(false, 0, tile_n, g2, inter, w_down, hidden, hidden, rows_hint, partial, s);
}

}  // extern "C"
