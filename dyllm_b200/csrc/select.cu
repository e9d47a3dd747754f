// Salient-token selection: additive cosine statistics, threshold mask, ordered compaction.
//
// All three are HBM-bound streaming kernels:
//   context_stats   reads 2 * width * 2 bytes per row, writes 12
//   cosine_mask     reads 12 bytes per row, writes 1
//   salient_select  reads 12 bytes per row once, writes 8 (+4, +8) bytes per selected row
#include <atomic>

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
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
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
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const float* s = stats + static_cast<int64_t>(r) * 3;
    mask[r] = below_threshold(s[0], s[1], s[2], threshold) ? 1 : 0;
  }
}

// ----------------------------------------------------------------------------------------------
// salient_select: warp-ballot flags + block scan + decoupled look-back across tiles
// ----------------------------------------------------------------------------------------------
constexpr int kSelWarps = 8;
constexpr int kSelTileRowsSmall = kSelWarps * 2 * 128;   // 2048 rows per tile (workspace is sized for these)
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

// Each thread owns 4 consecutive rows of a 128-row group (48 contiguous bytes = three 16-byte loads),
// so a warp reads 1536 contiguous bytes per group; a warp takes SUPER groups, a tile 8 * SUPER * 128
// rows.  Flags become a 4-bit nibble per thread; positions come from a warp prefix sum of the nibble
// popcounts, a block scan over the warps and a decoupled look-back over the tiles (32 predecessors per
// step).  The prefix front moves a bounded number of tiles per microsecond, which is what small inputs
// (up to 64 Ki rows, SUPER = 2) want: many small tiles in flight.  Larger inputs take
// salient_select_ranges_kernel below.
template <int SUPER>
__global__ void __launch_bounds__(kSelWarps * 32)
salient_select_kernel(const float* __restrict__ stats, int rows, float threshold,
                      const int32_t* __restrict__ cu_seqlens_q, int batch, const int32_t* __restrict__ cu_promptlens,
                      int64_t* __restrict__ idx_out, int32_t* __restrict__ idx32_out, int64_t* __restrict__ idx_k_out,
                      int32_t* __restrict__ cu_salientlens_out, int32_t* __restrict__ count_out,
                      uint8_t* __restrict__ mask_out, SelectWorkspace* ws, int* status_word) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  constexpr int kTileRows = kSelWarps * SUPER * 128;
  __shared__ int s_excl[kSelWarps * SUPER * 32];       // per thread and group: flags of the tile before its rows
  __shared__ uint8_t s_nib[kSelWarps * SUPER * 32];    // per thread and group: its 4 flags
  __shared__ int s_warp_count[kSelWarps];
  __shared__ int s_tile;
  __shared__ int s_tile_prefix;
  __shared__ int s_b_range[2];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0)
    s_tile = static_cast<int>(atomicAdd(&ws->ticket, 1u));
  __syncthreads();
  const int tile = s_tile;
  const int tile_row0 = tile * kTileRows;
  const int tile_row1 = min(tile_row0 + kTileRows, rows);
  // sequence boundaries inside this tile: two binary searches by two threads, under the loads below
  if (threadIdx.x == 32)
    s_b_range[0] = lower_bound_i32(cu_seqlens_q, batch + 1, tile_row0);
  if (threadIdx.x == 64)
    s_b_range[1] = lower_bound_i32(cu_seqlens_q, batch + 1, tile_row1);

  // 1. loads (all issued before any use), flags, warp-level exclusive positions
  float4 v[SUPER][3];
  int row0[SUPER];
#pragma unroll
  for (int g = 0; g < SUPER; ++g) {
    row0[g] = tile_row0 + (warp * SUPER + g) * 128 + lane * 4;
    if (row0[g] + 3 < rows) {
      const float4* src = reinterpret_cast<const float4*>(stats + static_cast<int64_t>(row0[g]) * 3);
      v[g][0] = __ldg(src);
      v[g][1] = __ldg(src + 1);
      v[g][2] = __ldg(src + 2);
    } else {
      float t[12];
#pragma unroll
      for (int i = 0; i < 12; ++i) {
        const int64_t e = static_cast<int64_t>(row0[g]) * 3 + i;
        t[i] = e < static_cast<int64_t>(rows) * 3 ? __ldg(stats + e) : 0.f;
      }
      v[g][0] = make_float4(t[0], t[1], t[2], t[3]);
      v[g][1] = make_float4(t[4], t[5], t[6], t[7]);
      v[g][2] = make_float4(t[8], t[9], t[10], t[11]);
    }
  }
  uint32_t nib[SUPER];
  int excl[SUPER];   // flags of this warp that precede this thread's first row of the group
  int warp_count = 0;
#pragma unroll
  for (int g = 0; g < SUPER; ++g) {
    const float4 a = v[g][0], b = v[g][1], c = v[g][2];
    uint32_t f = 0;
    if (row0[g] + 0 < rows && below_threshold(a.x, a.y, a.z, threshold)) f |= 1u;
    if (row0[g] + 1 < rows && below_threshold(a.w, b.x, b.y, threshold)) f |= 2u;
    if (row0[g] + 2 < rows && below_threshold(b.z, b.w, c.x, threshold)) f |= 4u;
    if (row0[g] + 3 < rows && below_threshold(c.y, c.z, c.w, threshold)) f |= 8u;
    nib[g] = f;
    if (mask_out) {
      if (row0[g] + 3 < rows) {
        *reinterpret_cast<uchar4*>(mask_out + row0[g]) = make_uchar4(f & 1u, (f >> 1) & 1u, (f >> 2) & 1u, (f >> 3) & 1u);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (row0[g] + j < rows)
            mask_out[row0[g] + j] = (f >> j) & 1u;
      }
    }
    const int cnt = __popc(f);
    int incl = cnt;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off)
        incl += o;
    }
    excl[g] = warp_count + incl - cnt;
    warp_count += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0)
    s_warp_count[warp] = warp_count;
  __syncthreads();

  // 2. tile aggregate, then exclusive prefix over earlier tiles: decoupled look-back by warp 0, whose
  // 32 lanes inspect 32 predecessors at a time
  if (warp == 0) {
    int t = lane < kSelWarps ? s_warp_count[lane] : 0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      t += __shfl_xor_sync(0xffffffffu, t, off);
    const int aggregate = t;
    volatile unsigned long long* tiles = ws->tiles;
    if (lane == 0) {
      tiles[tile] = ((tile == 0 ? 2ull : 1ull) << 32) | static_cast<unsigned int>(aggregate);
      __threadfence();
    }
    int exclusive = 0;
    bool gave_up = false;
    for (int base = tile - 1; base >= 0 && !gave_up; base -= 32) {
      const int look = base - lane;
      unsigned long long d = 2ull << 32;   // before the first tile: inclusive prefix 0
      uint32_t spins = 0;
      for (;;) {
        if (look >= 0)
          d = tiles[look];
        const bool ready = ((d >> 32) & 3ull) != 0;
        if (__all_sync(0xffffffffu, ready))
          break;
        if (++spins > kLookbackSpinLimit) {
          gave_up = true;
          break;
        }
      }
      gave_up = __any_sync(0xffffffffu, gave_up);
      const uint32_t inclusive_mask = __ballot_sync(0xffffffffu, ((d >> 32) & 3ull) == 2);
      const int first = inclusive_mask ? __ffs(inclusive_mask) - 1 : 31;   // nearest predecessor with a full prefix
      int contrib = lane <= first ? static_cast<int>(static_cast<unsigned int>(d)) : 0;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        contrib += __shfl_xor_sync(0xffffffffu, contrib, off);
      exclusive += contrib;
      if (inclusive_mask)
        break;
    }
    if (lane == 0) {
      if (gave_up && status_word)
        atomicCAS(status_word, 0, 101);
      if (tile != 0)
        tiles[tile] = (2ull << 32) | static_cast<unsigned int>(exclusive + aggregate);
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
  for (int g = 0; g < SUPER; ++g) {
    const int slot = (warp * SUPER + g) * 32 + lane;
    s_excl[slot] = base + excl[g] - tile_prefix;   // relative to the tile
    s_nib[slot] = static_cast<uint8_t>(nib[g]);
    int pos = base + excl[g];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if ((nib[g] >> j) & 1u) {
        const int r = row0[g] + j;
        idx_out[pos] = r;
        if (idx32_out)
          idx32_out[pos] = r;
        if (idx_k_out) {
          // sequence b with cu_q[b] <= r < cu_q[b + 1]
          const int b = lower_bound_i32(cu_seqlens_q, batch + 1, r + 1) - 1;
          idx_k_out[pos] = static_cast<int64_t>(r) + cu_promptlens[b + 1];
        }
        ++pos;
      }
    }
  }
  __syncthreads();

  // 4. per-sequence prefix counts for the sequence boundaries that fall inside this tile
  const int b_lo = s_b_range[0];
  const int b_hi = s_b_range[1];
  for (int b = b_lo + threadIdx.x; b < b_hi; b += blockDim.x) {
    const int local = cu_seqlens_q[b] - tile_row0;  // in [0, kTileRows)
    const int slot = local >> 2;                    // owner thread slot: 4 rows each, in row order
    const int j = local & 3;
    cu_salientlens_out[b] = tile_prefix + s_excl[slot] + __popc(static_cast<uint32_t>(s_nib[slot]) & ((1u << j) - 1u));
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

// Large inputs: one pass over contiguous row ranges.  The grid holds as many CTAs as the device runs at once;
// CTA number c (by arrival) owns rows [c * rows_per_cta, (c + 1) * rows_per_cta).  It streams the statistics of
// its range once (twelve 16-byte loads in flight per thread), writes the mask bytes and keeps the flags of the
// range in shared memory (one nibble per four rows).  Then every thread counts 32 rows at a time from those
// flags, a block scan turns the counts into positions, the CTA publishes the count of its range, adds the counts
// of the ranges before it (each belongs to a CTA that arrived earlier, so the wait cannot deadlock, and it is
// bounded) and writes its part of the lists.  No chain of dependent tiles: one exchange of ~600 counts for the
// whole input, and the statistics are read exactly once.
constexpr int kRangeGroups = 4;             // 128-row groups per warp and iteration (twelve loads per thread)
constexpr int kRangeMaxRows = 64 * 1024;    // rows of one range (16 KB of flags)
constexpr int kRangeThreads = kSelWarps * 32;

__global__ void __launch_bounds__(kRangeThreads, 4)
salient_select_ranges_kernel(const float* __restrict__ stats, int rows, float threshold,
                             const int32_t* __restrict__ cu_seqlens_q, int batch,
                             const int32_t* __restrict__ cu_promptlens, int64_t* __restrict__ idx_out,
                             int32_t* __restrict__ idx32_out, int64_t* __restrict__ idx_k_out,
                             int32_t* __restrict__ cu_salientlens_out, int32_t* __restrict__ count_out,
                             uint8_t* __restrict__ mask_out, SelectWorkspace* ws, int rows_per_cta, int* status_word) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  __shared__ __align__(8) uint8_t s_nib[kRangeMaxRows / 4];   // flags of four consecutive rows per byte
  __shared__ int s_pre[kRangeMaxRows / 32];                    // flags of the range before each 32-row chunk
  __shared__ int s_warp_sum[2][kSelWarps];
  __shared__ int s_cta;
  __shared__ int s_prefix;
  __shared__ int s_b_range[2];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0)
    s_cta = static_cast<int>(atomicAdd(&ws->ticket, 1u));
  __syncthreads();
  const int cta = s_cta;
  const int64_t r0_64 = static_cast<int64_t>(cta) * rows_per_cta;
  if (r0_64 >= rows)
    return;   // not reached: the grid holds exactly the ranges of the input
  const int range0 = static_cast<int>(r0_64);
  const int range1 = static_cast<int>(min(r0_64 + rows_per_cta, static_cast<int64_t>(rows)));
  const int n_groups = (range1 - range0 + 127) >> 7;
  const int iters = (n_groups + kSelWarps * kRangeGroups - 1) / (kSelWarps * kRangeGroups);
  if (threadIdx.x == 32)
    s_b_range[0] = lower_bound_i32(cu_seqlens_q, batch + 1, range0);
  if (threadIdx.x == 64)
    s_b_range[1] = lower_bound_i32(cu_seqlens_q, batch + 1, range1);

  // 1. one pass over the statistics: flags to shared memory, mask bytes out.  A group that lies completely
  // inside the range (every group but the last one of the input) takes the branch-free path: the test is
  // uniform over the warp.
  for (int it = 0; it < iters; ++it) {
    float4 v[kRangeGroups][3];
    const int grp0 = (it * kSelWarps + warp) * kRangeGroups;
#pragma unroll
    for (int g = 0; g < kRangeGroups; ++g) {
      const int grp = grp0 + g;
      const int row0 = range0 + grp * 128 + lane * 4;
      if (grp < n_groups && range0 + grp * 128 + 128 <= range1) {
        const float4* src = reinterpret_cast<const float4*>(stats + static_cast<int64_t>(row0) * 3);
        v[g][0] = __ldg(src);
        v[g][1] = __ldg(src + 1);
        v[g][2] = __ldg(src + 2);
      } else if (grp < n_groups) {
        float t[12];
#pragma unroll
        for (int i = 0; i < 12; ++i) {
          const int64_t e = static_cast<int64_t>(row0) * 3 + i;
          t[i] = e < static_cast<int64_t>(rows) * 3 ? __ldg(stats + e) : 0.f;
        }
        v[g][0] = make_float4(t[0], t[1], t[2], t[3]);
        v[g][1] = make_float4(t[4], t[5], t[6], t[7]);
        v[g][2] = make_float4(t[8], t[9], t[10], t[11]);
      }
    }
#pragma unroll
    for (int g = 0; g < kRangeGroups; ++g) {
      const int grp = grp0 + g;
      if (grp >= n_groups)
        continue;   // uniform over the warp
      const int row0 = range0 + grp * 128 + lane * 4;
      const float4 a = v[g][0], b = v[g][1], c = v[g][2];
      uint32_t f = (below_threshold(a.x, a.y, a.z, threshold) ? 1u : 0u) |
                   (below_threshold(a.w, b.x, b.y, threshold) ? 2u : 0u) |
                   (below_threshold(b.z, b.w, c.x, threshold) ? 4u : 0u) |
                   (below_threshold(c.y, c.z, c.w, threshold) ? 8u : 0u);
      if (range0 + grp * 128 + 128 <= range1) {
        if (mask_out)   // bits 0..3 of f to bytes 0..3
          *reinterpret_cast<uint32_t*>(mask_out + row0) = (f | (f << 7) | (f << 14) | (f << 21)) & 0x01010101u;
      } else {
        const int left = range1 - row0;   // rows of this thread inside the input
        f &= left >= 4 ? 15u : (left > 0 ? (1u << left) - 1u : 0u);
        if (mask_out) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (j < left)
              mask_out[row0 + j] = (f >> j) & 1u;
        }
      }
      s_nib[grp * 32 + lane] = static_cast<uint8_t>(f);
    }
  }
  __syncthreads();

  // 2. positions inside the range: pass p gives thread t the 32 rows of chunk p * 256 + t (eight flag bytes);
  // a block scan per pass.  The chunk's flags stay in a register for the writes below.
  const int n_chunks = n_groups * 4;
  const int passes = (n_chunks + kRangeThreads - 1) / kRangeThreads;
  unsigned long long bits[kRangeMaxRows / 32 / kRangeThreads];
  int running = 0;   // flags of the passes so far (the same value in every thread)
#pragma unroll
  for (int ps = 0; ps < kRangeMaxRows / 32 / kRangeThreads; ++ps) {
    bits[ps] = 0ull;
    if (ps >= passes)
      continue;   // uniform over the block
    const int chunk = ps * kRangeThreads + threadIdx.x;
    if (chunk < n_chunks)
      bits[ps] = *reinterpret_cast<const unsigned long long*>(s_nib + chunk * 8) & 0x0f0f0f0f0f0f0f0full;
    const int mine = __popcll(bits[ps]);
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off)
        incl += o;
    }
    if (lane == 31)
      s_warp_sum[ps & 1][warp] = incl;
    __syncthreads();
    int before = running, total = 0;
#pragma unroll
    for (int w = 0; w < kSelWarps; ++w) {
      const int ws_w = s_warp_sum[ps & 1][w];
      before += w < warp ? ws_w : 0;
      total += ws_w;
    }
    if (chunk < n_chunks)
      s_pre[chunk] = before + incl - mine;
    running += total;
  }
  // 3. count of this range out, counts of the earlier ranges in
  if (warp == 0) {
    volatile unsigned long long* tiles = ws->tiles;
    if (lane == 0) {
      tiles[cta] = (1ull << 32) | static_cast<unsigned int>(running);
      __threadfence();
    }
    int before = 0;
    bool gave_up = false;
    for (int pr = lane; pr < cta; pr += 32) {
      unsigned long long d = 0;
      uint32_t spins = 0;
      while ((((d = tiles[pr]) >> 32) & 3ull) == 0) {
        if (++spins > kLookbackSpinLimit) {
          gave_up = true;
          break;
        }
      }
      before += static_cast<int>(static_cast<unsigned int>(d));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      before += __shfl_xor_sync(0xffffffffu, before, off);
    gave_up = __any_sync(0xffffffffu, gave_up);
    if (lane == 0) {
      if (gave_up && status_word)
        atomicCAS(status_word, 0, 102);
      s_prefix = before;
      if (range1 == rows)
        count_out[0] = before + running;
    }
  }
  __syncthreads();
  const int prefix = s_prefix;

  // 4. ordered writes: every thread walks over the set flags of its chunks
#pragma unroll
  for (int ps = 0; ps < kRangeMaxRows / 32 / kRangeThreads; ++ps) {
    unsigned long long x = bits[ps];
    if (x == 0ull)
      continue;
    const int chunk = ps * kRangeThreads + threadIdx.x;
    int pos = prefix + s_pre[chunk];
    const int row_base = range0 + chunk * 32;
    while (x) {
      const int i = __ffsll(static_cast<long long>(x)) - 1;   // bit 8 * byte + j: row 4 * byte + j of the chunk
      x &= x - 1;
      const int r = row_base + ((i >> 3) << 2) + (i & 7);
      idx_out[pos] = r;
      if (idx32_out)
        idx32_out[pos] = r;
      if (idx_k_out) {
        const int b = lower_bound_i32(cu_seqlens_q, batch + 1, r + 1) - 1;   // sequence with cu_q[b] <= r < cu_q[b + 1]
        idx_k_out[pos] = static_cast<int64_t>(r) + cu_promptlens[b + 1];
      }
      ++pos;
    }
  }
  // 5. per-sequence prefix counts for the sequence boundaries inside this range
  const int b_lo = s_b_range[0];
  const int b_hi = s_b_range[1];
  for (int b = b_lo + threadIdx.x; b < b_hi; b += blockDim.x) {
    const int local = cu_seqlens_q[b] - range0;   // in [0, rows of the range)
    const int chunk = local >> 5, within = local & 31;
    unsigned long long x = *reinterpret_cast<const unsigned long long*>(s_nib + chunk * 8) & 0x0f0f0f0f0f0f0f0full;
    // rows before `within`: whole bytes below byte within / 4, then the low bits of that byte
    const int byte = within >> 2, j = within & 3;
    const unsigned long long below = byte == 0 ? 0ull : (~0ull >> (64 - 8 * byte));
    const unsigned long long part = ((1ull << j) - 1ull) << (8 * byte);
    cu_salientlens_out[b] = prefix + s_pre[chunk] + __popcll(x & (below | part));
  }
  if (range1 == rows) {  // last range: boundaries at or beyond the end
    const int total = prefix + running;
    for (int b = b_hi + threadIdx.x; b <= batch; b += blockDim.x)
      cu_salientlens_out[b] = total;
  }
}

__global__ void select_empty_kernel(int32_t* cu_salientlens_out, int32_t* count_out, int batch) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
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
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
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
  const int tiles = rows > 0 ? cdiv_i(rows, kSelTileRowsSmall) : 1;
  return sizeof(unsigned int) * 2 + sizeof(unsigned long long) * static_cast<size_t>(tiles);
}

// Shared by the caller-workspace entry point and by variants that bring their own scratch memory.
int launch_salient_select(const float* stats, int rows, float threshold, const int32_t* cu_seqlens_q, int batch,
                          const int32_t* cu_promptlens, int64_t* idx_out, int32_t* idx32_out, int64_t* idx_k_out,
                          int32_t* cu_salientlens_out, int32_t* count_out, uint8_t* mask_out, void* workspace,
                          cudaStream_t stream) {
  if (rows == 0) {
    DYLLM_LAUNCH(select_empty_kernel, 1, 128, 0, stream, cu_salientlens_out, count_out, batch);
    return check_launch("salient_select(empty)");
  }
  if (cudaMemsetAsync(workspace, 0, select_workspace_bytes(rows), stream) != cudaSuccess)
    return set_error(DYLLM_ERR_CUDA, "salient_select: clearing the workspace failed");
  SelectWorkspace* w = static_cast<SelectWorkspace*>(workspace);
  if (rows > 64 * 1024) {
    // contiguous ranges, one per CTA the device runs at once (four per SM: 63 registers, 18 KB of shared memory)
    const int64_t resident = 4ll * sm_count();
    int64_t per = (static_cast<int64_t>(rows) + resident - 1) / resident;
    per = (per + 127) / 128 * 128;   // whole 128-row groups; the ranges stay balanced over the SMs
    per = per < kSelTileRowsSmall ? kSelTileRowsSmall : per;   // the workspace holds one descriptor per 2048 rows
    per = per > kRangeMaxRows ? kRangeMaxRows : per;
    const int rows_per_cta = static_cast<int>(per);
    DYLLM_LAUNCH(salient_select_ranges_kernel, cdiv_i(rows, rows_per_cta), kSelWarps * 32, 0, stream,
        stats, rows, threshold, cu_seqlens_q, batch, cu_promptlens, idx_out, idx32_out, idx_k_out,
        cu_salientlens_out, count_out, mask_out, w, rows_per_cta, device_status_word());
  } else
    DYLLM_LAUNCH(salient_select_kernel<2>, cdiv_i(rows, kSelTileRowsSmall), kSelWarps * 32, 0, stream, 
        stats, rows, threshold, cu_seqlens_q, batch, cu_promptlens, idx_out, idx32_out, idx_k_out,
        cu_salientlens_out, count_out, mask_out, w, device_status_word());
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
    sizeof(unsigned int) * 2 + sizeof(unsigned long long) * (kStaticSelectMaxRows / kSelTileRowsSmall);
static __device__ __align__(256) unsigned char g_static_select_scratch[kStaticSelectBytes];

namespace {
// written once per device; atomic so that host threads may make their first call at the same time
std::atomic<void*> g_static_select_ptr[64];
}

// Returns the device address of the static scratch array on the current device (set up on first use).
int static_select_scratch(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return set_error(DYLLM_ERR_CUDA, "salient_select_static: no usable current device");
  void* ptr = g_static_select_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_select_scratch);
    if (err != cudaSuccess || !ptr)
      return set_error(DYLLM_ERR_CUDA, "salient_select_static: cudaGetSymbolAddress failed: %s",
                       cudaGetErrorString(err));
    g_static_select_ptr[dev].store(ptr, std::memory_order_release);  // every thread finds the same address
  }
  *out = ptr;
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
  DYLLM_LAUNCH(context_stats_kernel, blocks, kStatsWarps * 32, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint4*>(c_old), static_cast<const uint4*>(c_new), stats, rows, width / 8, accumulate);
  return check_launch("context_stats");
}

int dyllm_cosine_mask(const float* stats, uint8_t* mask, int rows, float threshold, void* stream) {
  DYLLM_REQUIRE(rows >= 0, DYLLM_ERR_INVALID_ARGUMENT, "cosine_mask: rows %d", rows);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(stats && mask, DYLLM_ERR_INVALID_ARGUMENT, "cosine_mask: null pointer");
  const int blocks = min(cdiv_i(rows, 256), sm_count() * 8);
  DYLLM_LAUNCH(cosine_mask_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), stats, mask, rows, threshold);
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
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(stats) & 15) == 0 && (reinterpret_cast<uintptr_t>(mask_out) & 3) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "salient_select: stats must be 16-byte and mask_out 4-byte aligned");
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
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(stats) & 15) == 0 && (reinterpret_cast<uintptr_t>(mask_out) & 3) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "salient_select_static: stats must be 16-byte and mask_out 4-byte aligned");
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
  DYLLM_LAUNCH(fused_offset_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), idxs, num_idxs, cu_promptlens,
                                                                           cu_salientlens, num_groups, out,
                                                                           max_threads);
  return check_launch("fused_offset");
}

}  // extern "C"
