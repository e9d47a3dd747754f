// Salient-token selection: additive cosine statistics, threshold mask, ordered compaction.
//
// All three are HBM-bound streaming kernels:
//   context_stats   reads 2 * width * 2 bytes per row, writes 12
//   cosine_mask     reads 12 bytes per row, writes 1
//   salient_select  reads 12 bytes per row once, writes 8 (+4, +8) bytes per selected row
#include "common.cuh"

namespace dyllm {
namespace {

// ----------------------------------------------------------------------------------------------
// context_stats: one warp per row, 16-byte loads, fixed reduction order
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void accum8(const uint4& a, const uint4& b, float& dot, float& na, float& nb) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(pa[i]);
    const float2 fb = __bfloat1622float2(pb[i]);
    dot = fmaf(fa.x, fb.x, dot);
    dot = fmaf(fa.y, fb.y, dot);
    na = fmaf(fa.x, fa.x, na);
    na = fmaf(fa.y, fa.y, na);
    nb = fmaf(fb.x, fb.x, nb);
    nb = fmaf(fb.y, fb.y, nb);
  }
}

constexpr int kStatsWarps = 8;

__global__ void __launch_bounds__(kStatsWarps * 32)
context_stats_kernel(const uint4* __restrict__ c_old, const uint4* __restrict__ c_new, float* __restrict__ stats,
                     int rows, int vecs_per_row, int accumulate) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * kStatsWarps + warp; row < rows; row += gridDim.x * kStatsWarps) {
    const uint4* po = c_old + static_cast<int64_t>(row) * vecs_per_row;
    const uint4* pn = c_new + static_cast<int64_t>(row) * vecs_per_row;
    float dot = 0.f, nn = 0.f, no = 0.f;
    int v = lane;
    // four independent 16-byte loads per tensor in flight per lane
    for (; v + 96 < vecs_per_row; v += 128) {
      const uint4 o0 = __ldg(po + v), o1 = __ldg(po + v + 32), o2 = __ldg(po + v + 64), o3 = __ldg(po + v + 96);
      const uint4 n0 = __ldg(pn + v), n1 = __ldg(pn + v + 32), n2 = __ldg(pn + v + 64), n3 = __ldg(pn + v + 96);
      accum8(n0, o0, dot, nn, no);
      accum8(n1, o1, dot, nn, no);
      accum8(n2, o2, dot, nn, no);
      accum8(n3, o3, dot, nn, no);
    }
    for (; v < vecs_per_row; v += 32) {
      const uint4 o0 = __ldg(po + v);
      const uint4 n0 = __ldg(pn + v);
      accum8(n0, o0, dot, nn, no);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      dot += __shfl_xor_sync(0xffffffffu, dot, off);
      nn += __shfl_xor_sync(0xffffffffu, nn, off);
      no += __shfl_xor_sync(0xffffffffu, no, off);
    }
    if (lane == 0) {
      float* s = stats + static_cast<int64_t>(row) * 3;
      if (accumulate) {
        s[0] += dot;
        s[1] += nn;
        s[2] += no;
      } else {
        s[0] = dot;
        s[1] = nn;
        s[2] = no;
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------
// cosine_mask
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ bool below_threshold(float dot, float a, float b, float threshold) {
  return dot * rsqrtf(fmaxf(a, 1e-8f)) * rsqrtf(fmaxf(b, 1e-8f)) < threshold;
}

__global__ void cosine_mask_kernel(const float* __restrict__ stats, uint8_t* __restrict__ mask, int rows,
                                   float threshold) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const float* s = stats + static_cast<int64_t>(r) * 3;
    mask[r] = below_threshold(s[0], s[1], s[2], threshold) ? 1 : 0;
  }
}

// ----------------------------------------------------------------------------------------------
// salient_select: warp-ballot flags + block scan + decoupled look-back across tiles
// ----------------------------------------------------------------------------------------------
constexpr int kSelWarps = 8;
constexpr int kSelChunks = 8;                                // 32-row chunks per warp
constexpr int kSelTileRows = kSelWarps * kSelChunks * 32;    // 2048 rows per tile
constexpr uint32_t kLookbackSpinLimit = 1u << 24;

// Workspace layout: [0] ticket counter (uint32), [1] padding, then one 64-bit descriptor per tile:
// bits 0-31 value, bits 32-33 state (0 = not ready, 1 = tile aggregate, 2 = inclusive prefix).
struct SelectWorkspace {
  unsigned int ticket;
  unsigned int pad;
  unsigned long long tiles[1];
};

__device__ __forceinline__ int lower_bound_i32(const int32_t* a, int n, int key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < key)
      lo = mid + 1;
    else
      hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(kSelWarps * 32)
salient_select_kernel(const float* __restrict__ stats, int rows, float threshold,
                      const int32_t* __restrict__ cu_seqlens_q, int batch, const int32_t* __restrict__ cu_promptlens,
                      int64_t* __restrict__ idx_out, int32_t* __restrict__ idx32_out, int64_t* __restrict__ idx_k_out,
                      int32_t* __restrict__ cu_salientlens_out, int32_t* __restrict__ count_out,
                      uint8_t* __restrict__ mask_out, SelectWorkspace* ws, int* status_word) {
  __shared__ uint32_t s_masks[kSelWarps * kSelChunks];
  __shared__ int s_warp_count[kSelWarps];
  __shared__ int s_tile;
  __shared__ int s_tile_prefix;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0)
    s_tile = static_cast<int>(atomicAdd(&ws->ticket, 1u));
  __syncthreads();
  const int tile = s_tile;
  const int tile_row0 = tile * kSelTileRows;

  // 1. flags: lane = row inside a 32-row chunk, ballot gives the chunk's bit mask
  uint32_t my_masks[kSelChunks];
  int warp_count = 0;
#pragma unroll
  for (int c = 0; c < kSelChunks; ++c) {
    const int r = tile_row0 + (warp * kSelChunks + c) * 32 + lane;
    bool flag = false;
    if (r < rows) {
      const float* s = stats + static_cast<int64_t>(r) * 3;
      flag = below_threshold(__ldg(s), __ldg(s + 1), __ldg(s + 2), threshold);
      if (mask_out)
        mask_out[r] = flag ? 1 : 0;
    }
    const uint32_t m = __ballot_sync(0xffffffffu, flag);
    my_masks[c] = m;
    warp_count += __popc(m);
  }
  if (lane == 0)
    s_warp_count[warp] = warp_count;
  if (lane < kSelChunks) {
    uint32_t m = 0;
#pragma unroll
    for (int c = 0; c < kSelChunks; ++c)
      m = (lane == c) ? my_masks[c] : m;
    s_masks[warp * kSelChunks + lane] = m;
  }
  __syncthreads();

  // 2. tile aggregate, then exclusive prefix over earlier tiles (decoupled look-back by warp 0)
  if (warp == 0) {
    int v = lane < kSelWarps ? s_warp_count[lane] : 0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      v += __shfl_xor_sync(0xffffffffu, v, off);
    const int aggregate = v;
    int exclusive = 0;
    if (lane == 0) {
      volatile unsigned long long* tiles = ws->tiles;
      if (tile == 0) {
        tiles[0] = (2ull << 32) | static_cast<unsigned int>(aggregate);
      } else {
        tiles[tile] = (1ull << 32) | static_cast<unsigned int>(aggregate);
        __threadfence();
        int look = tile - 1;
        uint32_t spins = 0;
        bool gave_up = false;
        while (look >= 0) {
          const unsigned long long d = tiles[look];
          const unsigned int state = static_cast<unsigned int>(d >> 32) & 3u;
          if (state == 0) {
            if (++spins > kLookbackSpinLimit) {
              gave_up = true;
              break;
            }
            continue;
          }
          exclusive += static_cast<int>(static_cast<unsigned int>(d));
          if (state == 2)
            break;
          --look;
        }
        if (gave_up && status_word)
          atomicCAS(status_word, 0, 101);
        tiles[tile] = (2ull << 32) | static_cast<unsigned int>(exclusive + aggregate);
      }
      __threadfence();
      s_tile_prefix = exclusive;
    }
  }
  __syncthreads();
  const int tile_prefix = s_tile_prefix;

  // 3. ordered writes
  int base = tile_prefix;
  for (int w = 0; w < warp; ++w)
    base += s_warp_count[w];
#pragma unroll
  for (int c = 0; c < kSelChunks; ++c) {
    const uint32_t m = my_masks[c];
    if ((m >> lane) & 1u) {
      const int r = tile_row0 + (warp * kSelChunks + c) * 32 + lane;
      const int pos = base + __popc(m & ((1u << lane) - 1u));
      idx_out[pos] = r;
      if (idx32_out)
        idx32_out[pos] = r;
      if (idx_k_out) {
        // sequence b with cu_q[b] <= r < cu_q[b + 1]
        const int b = lower_bound_i32(cu_seqlens_q, batch + 1, r + 1) - 1;
        idx_k_out[pos] = static_cast<int64_t>(r) + cu_promptlens[b + 1];
      }
    }
    base += __popc(m);
  }

  // 4. per-sequence prefix counts for the sequence boundaries that fall inside this tile
  const int tile_row1 = min(tile_row0 + kSelTileRows, rows);
  const int b_lo = lower_bound_i32(cu_seqlens_q, batch + 1, tile_row0);
  const int b_hi = lower_bound_i32(cu_seqlens_q, batch + 1, tile_row1);
  for (int b = b_lo + threadIdx.x; b < b_hi; b += blockDim.x) {
    const int local = cu_seqlens_q[b] - tile_row0;  // in [0, kSelTileRows)
    int cnt = tile_prefix;
    const int full_words = local >> 5;
    for (int w = 0; w < full_words; ++w)
      cnt += __popc(s_masks[w]);
    const int rem = local & 31;
    if (rem)
      cnt += __popc(s_masks[full_words] & ((1u << rem) - 1u));
    cu_salientlens_out[b] = cnt;
  }
  if (tile_row1 == rows) {  // last tile: boundaries at or beyond the end, and the total
    int total = tile_prefix;
    for (int w = 0; w < kSelWarps; ++w)
      total += s_warp_count[w];
    for (int b = b_hi + threadIdx.x; b <= batch; b += blockDim.x)
      cu_salientlens_out[b] = total;
    if (threadIdx.x == 0)
      count_out[0] = total;
  }
}

__global__ void select_empty_kernel(int32_t* cu_salientlens_out, int32_t* count_out, int batch) {
  for (int b = threadIdx.x; b <= batch; b += blockDim.x)
    cu_salientlens_out[b] = 0;
  if (threadIdx.x == 0)
    count_out[0] = 0;
}

// ----------------------------------------------------------------------------------------------
// fused_offset (stand-alone form of the K-space offset step)
// ----------------------------------------------------------------------------------------------
__global__ void fused_offset_kernel(const int32_t* __restrict__ idxs, const int32_t* __restrict__ num_idxs,
                                    const int32_t* __restrict__ cu_promptlens,
                                    const int32_t* __restrict__ cu_salientlens, int num_groups,
                                    int64_t* __restrict__ out, int max_threads) {
  const int n = min(*num_idxs, max_threads);
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
    int left = 0, right = num_groups;
    while (left < right) {
      const int mid = left + (right - left) / 2;
      if (cu_salientlens[mid + 1] <= t)
        left = mid + 1;
      else
        right = mid;
    }
    out[t] = static_cast<int64_t>(idxs[t]) + cu_promptlens[left + 1];
  }
}

}  // namespace

size_t select_workspace_bytes(int rows) {
  const int tiles = rows > 0 ? cdiv_i(rows, kSelTileRows) : 1;
  return sizeof(unsigned int) * 2 + sizeof(unsigned long long) * static_cast<size_t>(tiles);
}

// Shared by the caller-workspace entry point and by variants that bring their own scratch memory.
int launch_salient_select(const float* stats, int rows, float threshold, const int32_t* cu_seqlens_q, int batch,
                          const int32_t* cu_promptlens, int64_t* idx_out, int32_t* idx32_out, int64_t* idx_k_out,
                          int32_t* cu_salientlens_out, int32_t* count_out, uint8_t* mask_out, void* workspace,
                          cudaStream_t stream) {
  if (rows == 0) {
    select_empty_kernel<<<1, 128, 0, stream>>>(cu_salientlens_out, count_out, batch);
    return check_launch("salient_select(empty)");
  }
  const int tiles = cdiv_i(rows, kSelTileRows);
  if (cudaMemsetAsync(workspace, 0, select_workspace_bytes(rows), stream) != cudaSuccess)
    return set_error(DYLLM_ERR_CUDA, "salient_select: clearing the workspace failed");
  salient_select_kernel<<<tiles, kSelWarps * 32, 0, stream>>>(
      stats, rows, threshold, cu_seqlens_q, batch, cu_promptlens, idx_out, idx32_out, idx_k_out,
      cu_salientlens_out, count_out, mask_out, static_cast<SelectWorkspace*>(workspace), device_status_word());
  return check_launch("salient_select");
}

// ----------------------------------------------------------------------------------------------
// Selection without any caller- or library-allocated scratch memory.
//
// The look-back descriptors of salient_select live in this fixed array, which every device that loads
// the library holds until the process exits (kStaticSelectMaxRows / 2048 descriptors of 8 bytes plus
// the ticket: about 16 KB).  In host code the array's name is only a handle for the runtime, not a
// device address; its address on the current device is looked up once per device with
// cudaGetSymbolAddress and that pointer is what the kernel receives.
// ----------------------------------------------------------------------------------------------
constexpr int kStaticSelectMaxRows = 4 * 1024 * 1024;
constexpr size_t kStaticSelectBytes =
    sizeof(unsigned int) * 2 + sizeof(unsigned long long) * (kStaticSelectMaxRows / kSelTileRows);
static __device__ __align__(256) unsigned char g_static_select_scratch[kStaticSelectBytes];

namespace {
void* g_static_select_ptr[64] = {nullptr};
}

// Returns the device address of the static scratch array on the current device (set up on first use).
int static_select_scratch(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return set_error(DYLLM_ERR_CUDA, "salient_select_static: no usable current device");
  if (!g_static_select_ptr[dev]) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_select_scratch);
    if (err != cudaSuccess || !ptr)
      return set_error(DYLLM_ERR_CUDA, "salient_select_static: cudaGetSymbolAddress failed: %s",
                       cudaGetErrorString(err));
    g_static_select_ptr[dev] = ptr;
  }
  *out = g_static_select_ptr[dev];
  return DYLLM_OK;
}

}  // namespace dyllm

using namespace dyllm;

extern "C" {

int dyllm_context_stats(const void* c_old, const void* c_new, float* stats, int rows, int width, int accumulate,
                        void* stream) {
  DYLLM_REQUIRE(rows >= 0 && width > 0, DYLLM_ERR_INVALID_ARGUMENT, "context_stats: rows %d width %d", rows, width);
  DYLLM_REQUIRE(width % 8 == 0, DYLLM_ERR_UNSUPPORTED, "context_stats: width %d is not a multiple of 8", width);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(c_old && c_new && stats, DYLLM_ERR_INVALID_ARGUMENT, "context_stats: null pointer");
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(c_old) & 15) == 0 && (reinterpret_cast<uintptr_t>(c_new) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "context_stats: inputs must be 16-byte aligned");
  const int blocks = min(cdiv_i(rows, kStatsWarps), sm_count() * 8);
  context_stats_kernel<<<blocks, kStatsWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(c_old), static_cast<const uint4*>(c_new), stats, rows, width / 8, accumulate);
  return check_launch("context_stats");
}

int dyllm_cosine_mask(const float* stats, uint8_t* mask, int rows, float threshold, void* stream) {
  DYLLM_REQUIRE(rows >= 0, DYLLM_ERR_INVALID_ARGUMENT, "cosine_mask: rows %d", rows);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(stats && mask, DYLLM_ERR_INVALID_ARGUMENT, "cosine_mask: null pointer");
  const int blocks = min(cdiv_i(rows, 256), sm_count() * 8);
  cosine_mask_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(stats, mask, rows, threshold);
  return check_launch("cosine_mask");
}

size_t dyllm_salient_select_workspace_bytes(int rows) { return select_workspace_bytes(rows < 0 ? 0 : rows); }

int dyllm_salient_select(const float* stats, int rows, float threshold, const int32_t* cu_seqlens_q, int batch,
                         const int32_t* cu_promptlens, int64_t* idx_out, int32_t* idx32_out, int64_t* idx_k_out,
                         int32_t* cu_salientlens_out, int32_t* count_out, uint8_t* mask_out, void* workspace,
                         size_t workspace_bytes, void* stream) {
  DYLLM_REQUIRE(rows >= 0 && batch >= 0, DYLLM_ERR_INVALID_ARGUMENT, "salient_select: rows %d batch %d", rows, batch);
  DYLLM_REQUIRE(cu_seqlens_q && cu_salientlens_out && count_out, DYLLM_ERR_INVALID_ARGUMENT,
                "salient_select: null pointer");
  DYLLM_REQUIRE(rows == 0 || (stats && idx_out), DYLLM_ERR_INVALID_ARGUMENT, "salient_select: null pointer");
  DYLLM_REQUIRE(!idx_k_out || cu_promptlens, DYLLM_ERR_INVALID_ARGUMENT,
                "salient_select: idx_k_out needs cu_promptlens");
  DYLLM_REQUIRE(rows == 0 || (workspace && workspace_bytes >= select_workspace_bytes(rows)), DYLLM_ERR_WORKSPACE,
                "salient_select: workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
                select_workspace_bytes(rows));
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 7) == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "salient_select: workspace must be 8-byte aligned");
  return launch_salient_select(stats, rows, threshold, cu_seqlens_q, batch, cu_promptlens, idx_out, idx32_out,
                               idx_k_out, cu_salientlens_out, count_out, mask_out, workspace,
                               static_cast<cudaStream_t>(stream));
}

int dyllm_salient_select_static_max_rows(void) { return kStaticSelectMaxRows; }

int dyllm_salient_select_static(const float* stats, int rows, float threshold, const int32_t* cu_seqlens_q, int batch,
                                const int32_t* cu_promptlens, int64_t* idx_out, int32_t* idx32_out,
                                int64_t* idx_k_out, int32_t* cu_salientlens_out, int32_t* count_out,
                                uint8_t* mask_out, void* stream) {
  DYLLM_REQUIRE(rows >= 0 && batch >= 0, DYLLM_ERR_INVALID_ARGUMENT, "salient_select_static: rows %d batch %d", rows,
                batch);
  DYLLM_REQUIRE(rows <= kStaticSelectMaxRows, DYLLM_ERR_UNSUPPORTED,
                "salient_select_static: %d rows exceed the built-in scratch capacity of %d rows; use "
                "dyllm_salient_select with a caller-provided workspace",
                rows, kStaticSelectMaxRows);
  DYLLM_REQUIRE(cu_seqlens_q && cu_salientlens_out && count_out, DYLLM_ERR_INVALID_ARGUMENT,
                "salient_select_static: null pointer");
  DYLLM_REQUIRE(rows == 0 || (stats && idx_out), DYLLM_ERR_INVALID_ARGUMENT, "salient_select_static: null pointer");
  DYLLM_REQUIRE(!idx_k_out || cu_promptlens, DYLLM_ERR_INVALID_ARGUMENT,
                "salient_select_static: idx_k_out needs cu_promptlens");
  void* scratch = nullptr;
  const int rc = static_select_scratch(&scratch);
  if (rc != DYLLM_OK)
    return rc;
  // launch_salient_select clears the descriptors it is going to use (the array keeps the previous
  // call's content) before the kernel starts, on the same stream
  return launch_salient_select(stats, rows, threshold, cu_seqlens_q, batch, cu_promptlens, idx_out, idx32_out,
                               idx_k_out, cu_salientlens_out, count_out, mask_out, scratch,
                               static_cast<cudaStream_t>(stream));
}

int dyllm_fused_offset(const int32_t* idxs, const int32_t* num_idxs, const int32_t* cu_promptlens,
                       const int32_t* cu_salientlens, int num_groups, int64_t* out, int max_threads, void* stream) {
  DYLLM_REQUIRE(max_threads >= 0 && num_groups >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "fused_offset: max_threads %d num_groups %d", max_threads, num_groups);
  if (max_threads == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(idxs && num_idxs && cu_promptlens && cu_salientlens && out, DYLLM_ERR_INVALID_ARGUMENT,
                "fused_offset: null pointer");
  const int blocks = min(cdiv_i(max_threads, 256), sm_count() * 8);
  fused_offset_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(idxs, num_idxs, cu_promptlens,
                                                                           cu_salientlens, num_groups, out,
                                                                           max_threads);
  return check_launch("fused_offset");
}

}  // extern "C"
