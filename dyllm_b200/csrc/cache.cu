// Per-sequence activation cache: row copies between the packed step buffers and the cache.
//
// One warp moves one row with 16-byte accesses, four independent loads in flight per lane; the
// sequence of a packed row is found by binary search in the prefix-sum array.  All kernels are
// HBM-bound: 2 * width * elem_bytes bytes per row (one read, one write).
#include "common.cuh"

namespace dyllm {
namespace {

constexpr int kCopyWarps = 8;

__device__ __forceinline__ void copy_row_vec16(const uint4* __restrict__ src, uint4* __restrict__ dst, int vecs,
                                               int lane) {
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

template <typename T>
__device__ __forceinline__ int seq_of_row(const T* __restrict__ cu, int batch, int64_t row) {
  // largest b in [0, batch) with cu[b] <= row
  int lo = 0, hi = batch;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(cu[mid + 1]) <= row)
      lo = mid + 1;
    else
      hi = mid;
  }
  return lo < batch ? lo : batch - 1;
}

// TO_CACHE = false: packed[p] = cache[...]; true: cache[...] = packed[p].
// cu_k == nullptr: rows of sequence b start at the first cache row of the sequence;
// otherwise at its last (cu_pack[b+1] - cu_pack[b]) rows.
template <bool TO_CACHE>
__global__ void __launch_bounds__(kCopyWarps * 32)
cache_rows_kernel(uint4* __restrict__ cache, uint4* __restrict__ packed, const int64_t* __restrict__ seq_starts,
                  const int32_t* __restrict__ cu_pack, const int32_t* __restrict__ cu_k,
                  const int64_t* __restrict__ seq_ids, int batch, int packed_rows, int vecs) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int live_rows = min(packed_rows, cu_pack[batch]);
  for (int p = blockIdx.x * kCopyWarps + warp; p < live_rows; p += gridDim.x * kCopyWarps) {
    const int b = seq_of_row(cu_pack, batch, p);
    const int first = cu_pack[b];
    if (p < first)
      continue;  // rows below cu_pack[0]
    int64_t cache_row = seq_starts[seq_ids[b]] + (p - first);
    if (cu_k)
      cache_row += (cu_k[b + 1] - cu_k[b]) - (cu_pack[b + 1] - first);
    uint4* c = cache + cache_row * vecs;
    uint4* q = packed + static_cast<int64_t>(p) * vecs;
    if (TO_CACHE)
      copy_row_vec16(q, c, vecs, lane);
    else
      copy_row_vec16(c, q, vecs, lane);
  }
}

template <typename CuT>
__global__ void __launch_bounds__(kCopyWarps * 32)
scatter_rows_kernel(uint4* __restrict__ cache, const uint4* __restrict__ new_rows,
                    const int64_t* __restrict__ row_idx, const CuT* __restrict__ cu,
                    const int64_t* __restrict__ seq_starts, const int64_t* __restrict__ seq_ids, int batch,
                    int num_rows, const int32_t* __restrict__ num_rows_dev, int vecs) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  for (int m = blockIdx.x * kCopyWarps + warp; m < n; m += gridDim.x * kCopyWarps) {
    const int64_t r = row_idx[m];
    const int b = seq_of_row(cu, batch, r);
    const int64_t dest = seq_starts[seq_ids[b]] + (r - static_cast<int64_t>(cu[b]));
    copy_row_vec16(new_rows + static_cast<int64_t>(m) * vecs, cache + dest * vecs, vecs, lane);
  }
}

// Everything that follows the K/V projection of the salient rows, in one pass (8 threads per row and
// head, two 16-byte chunks of K and of V each):
//   k_cache[row] = rope(k_new[i], position)      (NeoX halves of 64, fp32 table)
//   dv[i] = v_new[i] - v_cache[row];  v_cache[row] = v_new[i]
// with row = first cache row of the sequence + (rows_k[i] - cu_k[b]) in each cache.
__global__ void __launch_bounds__(256)
kv_cache_update_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new,
                       const int64_t* __restrict__ rows_k, const int64_t* __restrict__ positions,
                       const int64_t* __restrict__ pos_idx, const float* __restrict__ cos_sin, int max_pos,
                       const int32_t* __restrict__ cu_k, const int64_t* __restrict__ k_starts,
                       const int64_t* __restrict__ v_starts, const int64_t* __restrict__ seq_ids, int batch,
                       int num_rows, const int32_t* __restrict__ num_rows_dev, int heads,
                       uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, uint4* __restrict__ dv) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  const int64_t total = static_cast<int64_t>(n) * heads * 8;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int part = static_cast<int>(t & 7);          // which 8 of the 64 rotation pairs
    const int64_t rh = t >> 3;
    const int i = static_cast<int>(rh / heads);
    const int h = static_cast<int>(rh - static_cast<int64_t>(i) * heads);
    const int64_t r = rows_k[i];
    const int b = seq_of_row(cu_k, batch, r);
    const int64_t off = r - static_cast<int64_t>(cu_k[b]);
    const int64_t sid = seq_ids[b];
    int64_t pos = positions[pos_idx ? pos_idx[i] : i];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + pos * 128;
    const int64_t src = rh * 16;                                   // 128 bf16 = 16 vectors per head
    const int64_t kdst = ((k_starts[sid] + off) * heads + h) * 16;
    const int64_t vdst = ((v_starts[sid] + off) * heads + h) * 16;
    {
      const uint4 a = __ldg(k_new + src + part), bb = __ldg(k_new + src + part + 8);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bb);
      uint4 oa, ob;
      __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
      __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x1 = __bfloat1622float2(a2[j]);
        const float2 x2 = __bfloat1622float2(b2[j]);
        const int d = part * 8 + 2 * j;
        const float c0 = __ldg(cs + d), c1 = __ldg(cs + d + 1), s0 = __ldg(cs + 64 + d), s1 = __ldg(cs + 64 + d + 1);
        oa2[j] = __floats2bfloat162_rn(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
        ob2[j] = __floats2bfloat162_rn(x2.x * c0 + x1.x * s0, x2.y * c1 + x1.y * s1);
      }
      k_cache[kdst + part] = oa;
      k_cache[kdst + part + 8] = ob;
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int v = part + 8 * c;
      const uint4 nv = __ldg(v_new + src + v);
      const uint4 ov = v_cache[vdst + v];
      uint4 out;
      const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nv);
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
      __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(n2[j]);
        const float2 y = __bfloat1622float2(o2[j]);
        d2[j] = __floats2bfloat162_rn(x.x - y.x, x.y - y.y);
      }
      dv[src + v] = out;
      v_cache[vdst + v] = nv;
    }
  }
}

// dv[i] = v_new[i] - cache[rows[i]]; cache[rows[i]] = v_new[i]; one warp per row.
__global__ void __launch_bounds__(kCopyWarps * 32)
delta_v_update_kernel(const uint4* __restrict__ v_new, uint4* __restrict__ cache, const int32_t* __restrict__ rows,
                      int num_rows, const int32_t* __restrict__ num_rows_dev, int vecs, uint4* __restrict__ dv) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n = num_rows_dev ? min(num_rows, *num_rows_dev) : num_rows;
  for (int i = blockIdx.x * kCopyWarps + warp; i < n; i += gridDim.x * kCopyWarps) {
    const int64_t r = rows[i];
    if (r < 0)
      continue;
    uint4* crow = cache + r * vecs;
    const uint4* nrow = v_new + static_cast<int64_t>(i) * vecs;
    uint4* drow = dv + static_cast<int64_t>(i) * vecs;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 nv = __ldg(nrow + v);
      const uint4 ov = crow[v];
      uint4 out;
      const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nv);
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
      __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(n2[j]);
        const float2 b = __bfloat1622float2(o2[j]);
        d2[j] = __floats2bfloat162_rn(a.x - b.x, a.y - b.y);
      }
      drow[v] = out;
      crow[v] = nv;
    }
  }
}

int check_common(const char* name, const void* cache, const void* other, const int64_t* seq_starts,
                 const void* cu, const int64_t* seq_ids, int batch, int rows, int width, int elem_bytes) {
  DYLLM_REQUIRE(batch >= 0 && rows >= 0 && width > 0 && elem_bytes > 0, DYLLM_ERR_INVALID_ARGUMENT,
                "%s: batch %d rows %d width %d elem_bytes %d", name, batch, rows, width, elem_bytes);
  DYLLM_REQUIRE((static_cast<int64_t>(width) * elem_bytes) % 16 == 0, DYLLM_ERR_UNSUPPORTED,
                "%s: row size %lld bytes is not a multiple of 16", name,
                static_cast<long long>(width) * elem_bytes);
  if (rows == 0 || batch == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(cache && other && seq_starts && cu && seq_ids, DYLLM_ERR_INVALID_ARGUMENT, "%s: null pointer", name);
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(other) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "%s: buffers must be 16-byte aligned", name);
  return DYLLM_OK;
}

template <bool TO_CACHE>
int launch_rows(const char* name, void* cache, void* packed, const int64_t* seq_starts, const int32_t* cu_pack,
                const int32_t* cu_k, const int64_t* seq_ids, int batch, int rows, int width, int elem_bytes,
                void* stream) {
  int rc = check_common(name, cache, packed, seq_starts, cu_pack, seq_ids, batch, rows, width, elem_bytes);
  if (rc != DYLLM_OK || rows == 0 || batch == 0)
    return rc;
  const int vecs = static_cast<int>(static_cast<int64_t>(width) * elem_bytes / 16);
  const int blocks = min(cdiv_i(rows, kCopyWarps), sm_count() * 8);
  DYLLM_LAUNCH(cache_rows_kernel<TO_CACHE>, blocks, kCopyWarps * 32, 0, static_cast<cudaStream_t>(stream), 
      static_cast<uint4*>(cache), static_cast<uint4*>(packed), seq_starts, cu_pack, cu_k, seq_ids, batch, rows,
      vecs);
  return check_launch(name);
}

}  // namespace
}  // namespace dyllm

using namespace dyllm;

extern "C" {

int dyllm_cache_get_seqs(const void* cache, void* out, const int64_t* seq_starts, const int32_t* cu_seqlens,
                         const int64_t* seq_ids, int batch, int total_rows, int width, int elem_bytes,
                         void* stream) {
  return launch_rows<false>("cache_get_seqs", const_cast<void*>(cache), out, seq_starts, cu_seqlens, nullptr,
                            seq_ids, batch, total_rows, width, elem_bytes, stream);
}

int dyllm_cache_get_block(const void* cache, void* out, const int64_t* seq_starts, const int32_t* cu_seqlens_k,
                          const int32_t* cu_seqlens_q, const int64_t* seq_ids, int batch, int total_rows, int width,
                          int elem_bytes, void* stream) {
  DYLLM_REQUIRE(batch == 0 || total_rows == 0 || cu_seqlens_k, DYLLM_ERR_INVALID_ARGUMENT,
                "cache_get_block: null cu_seqlens_k");
  return launch_rows<false>("cache_get_block", const_cast<void*>(cache), out, seq_starts, cu_seqlens_q,
                            cu_seqlens_k, seq_ids, batch, total_rows, width, elem_bytes, stream);
}

int dyllm_cache_reset_full(void* cache, const void* in, const int64_t* seq_starts, const int32_t* cu_seqlens,
                           const int64_t* seq_ids, int batch, int total_rows, int width, int elem_bytes,
                           void* stream) {
  return launch_rows<true>("cache_reset_full", cache, const_cast<void*>(in), seq_starts, cu_seqlens, nullptr,
                           seq_ids, batch, total_rows, width, elem_bytes, stream);
}

int dyllm_cache_reset_block(void* cache, const void* in, const int64_t* seq_starts, const int32_t* cu_seqlens_k,
                            const int32_t* cu_seqlens_q, const int64_t* seq_ids, int batch, int total_rows,
                            int width, int elem_bytes, void* stream) {
  DYLLM_REQUIRE(batch == 0 || total_rows == 0 || cu_seqlens_k, DYLLM_ERR_INVALID_ARGUMENT,
                "cache_reset_block: null cu_seqlens_k");
  return launch_rows<true>("cache_reset_block", cache, const_cast<void*>(in), seq_starts, cu_seqlens_q,
                           cu_seqlens_k, seq_ids, batch, total_rows, width, elem_bytes, stream);
}

int dyllm_delta_v_update(const void* v_new, void* cache, const int32_t* rows, int num_rows,
                         const int32_t* num_rows_dev, int width, void* dv, void* stream) {
  DYLLM_REQUIRE(num_rows >= 0 && width > 0, DYLLM_ERR_INVALID_ARGUMENT, "delta_v_update: rows %d width %d", num_rows,
                width);
  DYLLM_REQUIRE(width % 8 == 0, DYLLM_ERR_UNSUPPORTED, "delta_v_update: width %d is not a multiple of 8", width);
  if (num_rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(v_new && cache && rows && dv, DYLLM_ERR_INVALID_ARGUMENT, "delta_v_update: null pointer");
  DYLLM_REQUIRE(((reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(cache) |
                  reinterpret_cast<uintptr_t>(dv)) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "delta_v_update: buffers must be 16-byte aligned");
  const int blocks = min(cdiv_i(num_rows, kCopyWarps), sm_count() * 8);
  DYLLM_LAUNCH(delta_v_update_kernel, blocks, kCopyWarps * 32, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint4*>(v_new), static_cast<uint4*>(cache), rows, num_rows, num_rows_dev, width / 8,
      static_cast<uint4*>(dv));
  return check_launch("delta_v_update");
}

int dyllm_kv_cache_update(const void* k_new, const void* v_new, const int64_t* rows_k, const int64_t* positions,
                          const int64_t* pos_idx, const float* cos_sin, int max_pos, const int32_t* cu_seqlens_k,
                          const int64_t* k_seq_starts, const int64_t* v_seq_starts, const int64_t* seq_ids, int batch,
                          int num_rows, const int32_t* num_rows_dev, int kv_heads, int head_dim, void* k_cache,
                          void* v_cache, void* dv, void* stream) {
  DYLLM_REQUIRE(head_dim == 128, DYLLM_ERR_UNSUPPORTED, "kv_cache_update: head_dim %d (only 128 is built)", head_dim);
  DYLLM_REQUIRE(batch >= 0 && num_rows >= 0 && kv_heads > 0 && max_pos > 0, DYLLM_ERR_INVALID_ARGUMENT,
                "kv_cache_update: batch %d rows %d heads %d", batch, num_rows, kv_heads);
  if (num_rows == 0 || batch == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(k_new && v_new && rows_k && positions && cos_sin && cu_seqlens_k && k_seq_starts && v_seq_starts &&
                    seq_ids && k_cache && v_cache && dv,
                DYLLM_ERR_INVALID_ARGUMENT, "kv_cache_update: null pointer");
  DYLLM_REQUIRE(((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) |
                  reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                  reinterpret_cast<uintptr_t>(dv)) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "kv_cache_update: buffers must be 16-byte aligned");
  const int64_t total = static_cast<int64_t>(num_rows) * kv_heads * 8;
  const int64_t want = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  DYLLM_LAUNCH(kv_cache_update_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new), rows_k, positions, pos_idx, cos_sin, max_pos,
      cu_seqlens_k, k_seq_starts, v_seq_starts, seq_ids, batch, num_rows, num_rows_dev, kv_heads,
      static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache), static_cast<uint4*>(dv));
  return check_launch("kv_cache_update");
}

int dyllm_cache_scatter_update(void* cache, const void* new_rows, const int64_t* row_idx, const void* cu_seqlens,
                               int cu_is_int64, const int64_t* seq_starts, const int64_t* seq_ids, int batch,
                               int num_rows, const int32_t* num_rows_dev, int width, int elem_bytes, void* stream) {
  int rc = check_common("cache_scatter_update", cache, new_rows, seq_starts, cu_seqlens, seq_ids, batch, num_rows,
                        width, elem_bytes);
  if (rc != DYLLM_OK || num_rows == 0 || batch == 0)
    return rc;
  DYLLM_REQUIRE(row_idx, DYLLM_ERR_INVALID_ARGUMENT, "cache_scatter_update: null row_idx");
  const int vecs = static_cast<int>(static_cast<int64_t>(width) * elem_bytes / 16);
  const int blocks = min(cdiv_i(num_rows, kCopyWarps), sm_count() * 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cu_is_int64)
    DYLLM_LAUNCH(scatter_rows_kernel<int64_t>, blocks, kCopyWarps * 32, 0, s, 
        static_cast<uint4*>(cache), static_cast<const uint4*>(new_rows), row_idx,
        static_cast<const int64_t*>(cu_seqlens), seq_starts, seq_ids, batch, num_rows, num_rows_dev, vecs);
  else
    DYLLM_LAUNCH(scatter_rows_kernel<int32_t>, blocks, kCopyWarps * 32, 0, s, 
        static_cast<uint4*>(cache), static_cast<const uint4*>(new_rows), row_idx,
        static_cast<const int32_t*>(cu_seqlens), seq_starts, seq_ids, batch, num_rows, num_rows_dev, vecs);
  return check_launch("cache_scatter_update");
}

}  // extern "C"
