// Gathered SwiGLU FFN on salient rows:  out[map[m]] = down( silu(x[idx[m]] Wg^T) * (x[idx[m]] Wu^T) ).
// Two launches of the tcgen05 GEMM in gemm.cuh: gate/up with the activation fused in the epilogue, then
// the down projection whose epilogue scatters rows to their destination.
#include "gemm.cuh"

namespace dyllm {

namespace {

template <int BNH, bool SWIGLU, int A_MODE, int STAGES>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int n_tiles, cudaStream_t stream) {
  using Cfg = GemmCfg<BNH, SWIGLU, STAGES>;
  auto kernel = gathered_gemm_kernel<BNH, SWIGLU, A_MODE, STAGES>;
  // one flag per kernel instantiation and device: the opt-in shared-memory size is a per-function attribute
  static bool smem_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev < 0 || dev >= 64) ? 0 : dev;
  if (!smem_set[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(Cfg::SMEM_BYTES)) != cudaSuccess)
      return set_error(DYLLM_ERR_CUDA, "cudaFuncSetAttribute(%u bytes of shared memory) failed: %s", Cfg::SMEM_BYTES,
                       cudaGetErrorString(cudaGetLastError()));
    smem_set[dev] = true;
  }
  dim3 grid(cdiv_i(p.M, kGemmBM), n_tiles);
  kernel<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
  return check_launch("gathered_gemm");
}

template <int BNH, bool SWIGLU, int STAGES>
int launch_mode(int a_mode, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int n_tiles,
                cudaStream_t stream) {
  switch (a_mode) {
    case 0: return launch_one<BNH, SWIGLU, 0, STAGES>(ta, tb, p, n_tiles, stream);
    case 1: return launch_one<BNH, SWIGLU, 1, STAGES>(ta, tb, p, n_tiles, stream);
    default: return launch_one<BNH, SWIGLU, 2, STAGES>(ta, tb, p, n_tiles, stream);
  }
}

}  // namespace

// a_mode: 0 = rows m0..m0+127 of A by one TMA box (requires a_idx == null), 1 = TMA gather4, 2 = gather
// with 16-byte loads by the epilogue warps.  n is the number of output columns per weight block
// (the intermediate size for SWIGLU).  tile_n: 64 or 128 (0 = choose).
int launch_gathered_gemm(bool swiglu, int a_mode, int tile_n, const GemmParams& p_in, const void* b,
                         int64_t b_total_rows, int n, cudaStream_t stream) {
  GemmParams p = p_in;
  DYLLM_REQUIRE(p.K > 0 && p.K % kGemmBK == 0, DYLLM_ERR_UNSUPPORTED, "gemm: K = %d is not a multiple of 64", p.K);
  DYLLM_REQUIRE(n > 0 && n % 64 == 0, DYLLM_ERR_UNSUPPORTED, "gemm: N = %d is not a multiple of 64", n);
  DYLLM_REQUIRE(p.lda % 8 == 0 && p.ldc % 8 == 0, DYLLM_ERR_UNSUPPORTED, "gemm: row pitches must be multiples of 8");
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(p.out) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "gemm: operands must be 16-byte aligned");
  DYLLM_REQUIRE(a_mode >= 0 && a_mode <= 2, DYLLM_ERR_INVALID_ARGUMENT, "gemm: a_mode %d", a_mode);
  DYLLM_REQUIRE(!(a_mode == 0 && p.a_idx), DYLLM_ERR_INVALID_ARGUMENT, "gemm: a_mode 0 cannot gather");
  if (p.M <= 0)
    return DYLLM_OK;
  if (tile_n == 0) {
    const int tiles128 = cdiv_i(p.M, kGemmBM) * (n / 128);
    tile_n = (n % 128 == 0 && tiles128 >= sm_count() * 3 / 4) ? 128 : 64;
  }
  DYLLM_REQUIRE((tile_n == 64 || tile_n == 128) && n % tile_n == 0, DYLLM_ERR_UNSUPPORTED,
                "gemm: tile_n %d does not divide N = %d", tile_n, n);
  p.status_word = device_status_word();

  CUtensorMap ta, tb;
  int rc;
  if (a_mode == 0)
    rc = encode_tmap_2d_bf16(&ta, p.a, p.a_rows, p.K, p.lda, kGemmBM, kGemmBK, true);
  else
    rc = encode_tmap_2d_bf16(&ta, p.a, p.a_rows, p.K, p.lda, 1, kGemmBK, true);
  if (rc != DYLLM_OK)
    return rc;
  rc = encode_tmap_2d_bf16(&tb, b, b_total_rows, p.K, p.K, tile_n, kGemmBK, true);
  if (rc != DYLLM_OK)
    return rc;

  const int n_tiles = n / tile_n;
  if (swiglu) {
    if (tile_n == 128)
      return launch_mode<128, true, 4>(a_mode, ta, tb, p, n_tiles, stream);
    return launch_mode<64, true, 6>(a_mode, ta, tb, p, n_tiles, stream);
  }
  if (tile_n == 128)
    return launch_mode<128, false, 6>(a_mode, ta, tb, p, n_tiles, stream);
  return launch_mode<64, false, 8>(a_mode, ta, tb, p, n_tiles, stream);
}

namespace {

// dest[m] = seq_starts[seq_ids[b]] + (row_idx[m] - cu[b]) for m < n, -1 beyond the live rows.
__global__ void cache_dest_rows_kernel(const int64_t* __restrict__ row_idx, const int32_t* __restrict__ cu,
                                       const int64_t* __restrict__ seq_starts, const int64_t* __restrict__ seq_ids,
                                       int batch, int num_rows, const int32_t* __restrict__ num_rows_dev,
                                       int32_t* __restrict__ dest) {
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
}  // namespace dyllm

using namespace dyllm;

extern "C" {

size_t dyllm_swiglu_ffn_workspace_bytes(int max_rows, int inter) {
  if (max_rows <= 0 || inter <= 0)
    return 0;
  const size_t padded = static_cast<size_t>(cdiv_i(max_rows, kGemmBM)) * kGemmBM;
  return padded * static_cast<size_t>(inter) * 2;
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
  cache_dest_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      row_idx, cu_seqlens, seq_starts, seq_ids, batch, num_rows, num_rows_dev, dest_rows);
  return check_launch("cache_dest_rows");
}

int dyllm_gathered_linear(const void* x, int x_rows, int in_features, int64_t ldx, const int32_t* idx, int num_rows,
                          const int32_t* num_rows_dev, const void* weight, int out_features, void* out, int64_t ldo,
                          const int32_t* out_row_map, const float* row_scale, int a_mode, int tile_n, void* stream) {
  DYLLM_REQUIRE(x_rows >= 0 && in_features > 0 && out_features > 0 && num_rows >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "gathered_linear: x_rows %d in %d out %d num_rows %d", x_rows, in_features, out_features, num_rows);
  if (num_rows == 0 || x_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && weight && out, DYLLM_ERR_INVALID_ARGUMENT, "gathered_linear: null pointer");
  if (a_mode < 0)
    a_mode = 1;
  DYLLM_REQUIRE(a_mode == 1 || a_mode == 2, DYLLM_ERR_INVALID_ARGUMENT, "gathered_linear: a_mode %d", a_mode);
  GemmParams g = {};
  g.a = static_cast<const __nv_bfloat16*>(x);
  g.a_idx = idx;
  g.m_count_dev = num_rows_dev;
  g.M = num_rows;
  g.K = in_features;
  g.a_rows = x_rows;
  g.lda = ldx;
  g.b_rows_per_expert = out_features;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ldc = ldo;
  g.out_row_map = out_row_map;
  g.row_scale = row_scale;
  return launch_gathered_gemm(false, a_mode, tile_n, g, weight, out_features, out_features,
                              static_cast<cudaStream_t>(stream));
}

int dyllm_swiglu_ffn(const void* x, int x_rows, int hidden, int64_t ldx, const int32_t* idx, int num_rows,
                     const int32_t* num_rows_dev, const void* w_gate_up, const void* w_down, int inter, void* out,
                     int64_t ldo, const int32_t* out_row_map, void* workspace, size_t workspace_bytes, int a_mode,
                     int tile_n, void* stream) {
  DYLLM_REQUIRE(x_rows >= 0 && hidden > 0 && inter > 0 && num_rows >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "swiglu_ffn: x_rows %d hidden %d inter %d num_rows %d", x_rows, hidden, inter, num_rows);
  if (num_rows == 0 || x_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && w_gate_up && w_down && out && workspace, DYLLM_ERR_INVALID_ARGUMENT, "swiglu_ffn: null pointer");
  DYLLM_REQUIRE(workspace_bytes >= dyllm_swiglu_ffn_workspace_bytes(num_rows, inter), DYLLM_ERR_WORKSPACE,
                "swiglu_ffn: workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
                dyllm_swiglu_ffn_workspace_bytes(num_rows, inter));
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "swiglu_ffn: workspace must be 16-byte aligned");
  if (a_mode < 0)
    a_mode = 1;
  DYLLM_REQUIRE(a_mode == 1 || a_mode == 2, DYLLM_ERR_INVALID_ARGUMENT, "swiglu_ffn: a_mode %d (1 = TMA gather4, "
                "2 = vector-load gather)", a_mode);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int padded = cdiv_i(num_rows, kGemmBM) * kGemmBM;

  GemmParams g1 = {};
  g1.a = static_cast<const __nv_bfloat16*>(x);
  g1.a_idx = idx;
  g1.m_count_dev = num_rows_dev;
  g1.M = num_rows;
  g1.K = hidden;
  g1.a_rows = x_rows;
  g1.lda = ldx;
  g1.b_rows_per_expert = 2 * inter;
  g1.up_row_offset = inter;
  g1.out = static_cast<__nv_bfloat16*>(workspace);
  g1.ldc = inter;
  int rc = launch_gathered_gemm(true, a_mode, tile_n, g1, w_gate_up, 2 * static_cast<int64_t>(inter), inter, s);
  if (rc != DYLLM_OK)
    return rc;

  GemmParams g2 = {};
  g2.a = static_cast<const __nv_bfloat16*>(workspace);
  g2.m_count_dev = num_rows_dev;
  g2.M = num_rows;
  g2.K = inter;
  g2.a_rows = padded;
  g2.lda = inter;
  g2.b_rows_per_expert = hidden;
  g2.out = static_cast<__nv_bfloat16*>(out);
  g2.ldc = ldo;
  g2.out_row_map = out_row_map;
  return launch_gathered_gemm(false, 0, tile_n, g2, w_down, hidden, hidden, s);
}

}  // extern "C"
