// Row-gathered bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), shared by the dense
// SwiGLU FFN, the K/V projection of salient rows and the MoE expert FFN.
//
//   D[m, n] = sum_k A[a_idx[m], k] * B[b_row0(m_tile) + n, k]          (fp32 accumulation in TMEM)
//
// The number of live rows is read on the device (m_count_dev), so a launch needs no host knowledge of
// it: the grid is (n tiles, k splits, row groups) and every CTA walks over the row tiles
// blockIdx.z, blockIdx.z + gridDim.z, ... that lie below the live count.  The row groups come last in the grid so
// that the CTAs of the first row tile, all splits, are dispatched before the CTAs of row groups that usually find
// nothing to do (they return at once, but each takes a turn in an SM slot first).
//
// Warp roles (6 warps):
//   warp 0      producer: weight tiles by TMA (128-byte swizzle); activation rows by one TMA box per
//               stage (A_MODE 0: A is dense or was staged into a compact buffer) or by TMA gather4
//               through the index list (A_MODE 1, one copy of 4 rows per lane)
//   warp 1      allocates tensor memory (two accumulators), issues tcgen05.mma, commits to mbarriers
//   warps 2..5  epilogue of row tile i while the main loop of tile i+1 runs: tcgen05.ld, SiLU(gate)*up
//               or scale, bf16 stores with row scatter / column split, or fp32 split-K partials
// Every wait is bounded; a wait that runs out raises the CTA's abort flag and the device status word.
#pragma once

#include "common.cuh"

namespace dyllm {

struct GemmParams {
  const __nv_bfloat16* a;      // activation matrix
  const int32_t* a_idx;        // [M] source row of A for logical row m (A_MODE 1); null = identity
  const int32_t* m_count_dev;  // device scalar bounding the live logical rows; null = M
  const int32_t* tile_expert;  // [ceil(M/128)] weight block per row tile; null = block 0
  int M;                       // upper bound of logical rows
  int K;                       // contraction length, multiple of 64
  int a_rows;                  // rows of the activation matrix (for clamping)
  int b_rows_per_expert;       // rows of B per weight block
  int up_row_offset;           // SwiGLU: row distance from the gate rows to the up rows
  __nv_bfloat16* out;          // output matrix
  int64_t ldc;                 // row pitch of the output in elements
  const int32_t* out_row_map;  // [M] destination row per logical row (negative = drop); null = m
  const float* row_scale;      // [M] multiplier per logical row; null = 1
  __nv_bfloat16* out2;         // columns >= split_col go here (column - split_col); null = no split
  int64_t ldc2;
  int split_col;
  float* partial;              // split-K: fp32 [gridDim.y][split_rows][n_total]; null = no split-K
  int* split_tickets;          // split-K: arrival counter per (row tile, column tile), zero between launches
  int split_rows;              // split-K is used only while the live row count is <= split_rows
  int split_slots;             // CTAs the device runs at once; the live split count is derived from it
  int n_total;                 // output columns (row pitch of `partial`)
  int* status_word;
};

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 192;

// MT = 1: 128-row tiles, two accumulators alternate between consecutive row tiles (the epilogue of one
// tile overlaps the main loop of the next).  MT = 2: 256-row tiles made of two 128-row accumulators that
// share every weight tile in shared memory, which halves the weight traffic from L2 per flop (the
// limit at many rows); the epilogue is then not overlapped.
template <int BNH, bool SWIGLU, int STAGES, int MT = 1>
struct GemmCfg {
  static constexpr int BN = SWIGLU ? 2 * BNH : BNH;  // UMMA N
  static constexpr uint32_t A_BYTES = MT * kGemmBM * kGemmBK * 2;
  static constexpr uint32_t B_BYTES = BN * kGemmBK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + alignment slack
  static constexpr uint32_t TMEM_COLS = 2 * BN < 64 ? 64 : 2 * BN;     // two accumulators
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M = 128");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "tensor memory columns");
};

// Number of K splits for `live_tiles` row tiles: as many as keep every CTA slot busy, at most
// `max_splits` (the grid's z extent) and the number of k tiles.  The GEMM and the reduction kernel both
// derive it from the device-side row count, so one launch shape serves every count.
__host__ __device__ __forceinline__ int effective_splits(int live_tiles, int n_tiles, int slots, int max_splits,
                                                         int num_kt) {
  const int ctas = (live_tiles < 1 ? 1 : live_tiles) * n_tiles;
  if (ctas * 2 > slots)
    return 1;
  int s = slots / ctas;
  s = s > max_splits ? max_splits : s;
  s = s > num_kt ? num_kt : s;
  return s < 1 ? 1 : s;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// MINB = 2 (with half the pipeline depth) lets two CTAs share an SM: used when few row tiles are live and
// the kernel is bound by streaming the weights, so that every SM has loads in flight in a single wave.
template <int BNH, bool SWIGLU, int A_MODE, int STAGES, int MINB, int MT = 1>
__global__ void __launch_bounds__(kGemmThreads, MINB)
gathered_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const GemmParams p) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  using Cfg = GemmCfg<BNH, SWIGLU, STAGES, MT>;
  constexpr int BM = kGemmBM * MT, BK = kGemmBK, BN = Cfg::BN;
  static_assert(MT == 1 || A_MODE == 0, "256-row tiles take their rows as one TMA box");

  const int n_tile = blockIdx.x;
  const int m_count = p.m_count_dev ? min(*p.m_count_dev, p.M) : p.M;
  if (static_cast<int>(blockIdx.z) * BM >= m_count)
    return;
  // split-K only while the live rows fit the partial buffer; otherwise split 0 runs the whole K range
  const int num_kt_all = p.K / BK;
  int kt_begin = 0, kt_end = num_kt_all;
  bool write_partial = false;
  int splits = 1;
  if (p.partial != nullptr) {
    splits = m_count <= p.split_rows
                 ? effective_splits((m_count + BM - 1) / BM, gridDim.x, p.split_slots, gridDim.y, num_kt_all)
                 : 1;
    if (static_cast<int>(blockIdx.y) >= splits)
      return;
    if (splits > 1) {
      const int per = (num_kt_all + splits - 1) / splits;
      kt_begin = min(static_cast<int>(blockIdx.y) * per, num_kt_all);
      kt_end = min(kt_begin + per, num_kt_all);
      write_partial = true;
    }
  }
  const int num_kt = kt_end - kt_begin;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int last_split;   // split-K: this CTA was the last to finish the current output tile

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 128);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int it = 0;
    for (int mt = blockIdx.z; mt * BM < m_count; mt += gridDim.z) {
      const int m0 = mt * BM;
      const int b_row0 = (p.tile_expert ? p.tile_expert[mt] : 0) * p.b_rows_per_expert + n_tile * BNH;
      int rows4[4] = {0, 0, 0, 0};
      if (A_MODE == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int m = m0 + lane * 4 + j;
          int r = 0;
          if (m < m_count)
            r = p.a_idx ? p.a_idx[m] : m;
          rows4[j] = min(max(r, 0), p.a_rows - 1);
        }
      }
      for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, p.status_word, 201);
        uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
        uint8_t* b_dst = a_dst + Cfg::A_BYTES;
        if (lane == 0) {
          mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          tma_load_2d(b_dst, &tmap_b, &full_bar[s], kt * BK, b_row0);
          if (SWIGLU)
            tma_load_2d(b_dst + BNH * BK * 2, &tmap_b, &full_bar[s], kt * BK, b_row0 + p.up_row_offset);
          if (A_MODE == 0)
            tma_load_2d(a_dst, &tmap_a, &full_bar[s], kt * BK, m0);
        }
        __syncwarp();
        if (A_MODE == 1)
          tma_gather4_2d(a_dst + lane * 512, &tmap_a, &full_bar[s], kt * BK, rows4[0], rows4[1], rows4[2], rows4[3]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(kGemmBM, BN, 0, 0);
    int it = 0, ti = 0;
    for (int mt = blockIdx.z; mt * BM < m_count; mt += gridDim.z, ++ti) {
      // MT = 1: accumulators alternate; MT = 2: both belong to this tile and barrier 0 guards them
      const int acc = MT == 1 ? (ti & 1) : 0;
      const uint32_t use = MT == 1 ? (ti >> 1) : ti;
      mbar_wait(&tmem_empty_bar[acc], (use & 1) ^ 1, &abort_flag, p.status_word, 205);
      tc_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + acc * BN;
      for (int kt = 0; kt < num_kt; ++kt, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        mbar_wait(&full_bar[s], ph, &abort_flag, p.status_word, 202);
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          const uint64_t a_desc = umma_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = umma_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_ss(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt | k) != 0 ? 1u : 0u);
            if (MT == 2)   // second 128 rows (16 KB further in the A stage) against the same weight tile
              umma_ss(tmem_acc + BN, a_desc + 1024 + 2 * k, b_desc + 2 * k, idesc, (kt | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          if (kt == num_kt - 1)
            umma_commit(&tmem_full_bar[acc]);
        }
        __syncwarp();
      }
      if (num_kt == 0 && lane == 0)
        mbar_arrive(&tmem_full_bar[acc]);  // empty k range: nothing was issued
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;            // tensor-memory lane quarter this warp may read
    const int row = q * 32 + lane;     // accumulator row == logical row m0 + row
    int ti = 0;
    for (int mt = blockIdx.z; mt * BM < m_count; mt += gridDim.z, ++ti) {
      const int acc = MT == 1 ? (ti & 1) : 0;
      const uint32_t use = MT == 1 ? (ti >> 1) : ti;
      mbar_wait(&tmem_full_bar[acc], use & 1, &abort_flag, p.status_word, 204);
      tc_fence_after_sync();
#pragma unroll 1
      for (int sub = 0; sub < MT; ++sub) {
      const int m = mt * BM + sub * kGemmBM + row;
      const bool live = m < m_count;
      const uint32_t t_row = tmem_base + (MT == 1 ? acc : sub) * BN + (static_cast<uint32_t>(q * 32) << 16);
      int out_row = m;
      if (p.out_row_map && live)
        out_row = p.out_row_map[m];
      const bool store = live && out_row >= 0;
      const float scale = (p.row_scale && live) ? p.row_scale[m] : 1.0f;
      const int n0 = n_tile * BNH;
      __nv_bfloat16* dst;
      if (p.out2 && n0 >= p.split_col)
        dst = p.out2 + static_cast<int64_t>(store ? out_row : 0) * p.ldc2 + (n0 - p.split_col);
      else
        dst = p.out + static_cast<int64_t>(store ? out_row : 0) * p.ldc + n0;
      float* pdst = nullptr;
      if (write_partial)
        pdst = p.partial + (static_cast<int64_t>(blockIdx.y) * p.split_rows + (live ? m : 0)) * p.n_total + n0;

#pragma unroll 1
      for (int c0 = 0; c0 < BNH; c0 += 32) {
        uint32_t g[32];
        tmem_ld_32x32(t_row + c0, g);
        if (SWIGLU) {
          uint32_t u[32];
          uint32_t packed[16];
          tmem_ld_32x32(t_row + BNH + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float h0 = silu_f(__uint_as_float(g[2 * i])) * __uint_as_float(u[2 * i]);
            const float h1 = silu_f(__uint_as_float(g[2 * i + 1])) * __uint_as_float(u[2 * i + 1]);
            packed[i] = pack_bf16x2(h0, h1);
          }
          if (store) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + c0);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              d4[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          }
        } else {
          tmem_ld_wait();
          if (num_kt == 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              g[i] = 0u;
          }
          if (write_partial) {
            if (live) {
              uint4* d4 = reinterpret_cast<uint4*>(pdst + c0);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                d4[i] = make_uint4(g[4 * i], g[4 * i + 1], g[4 * i + 2], g[4 * i + 3]);
            }
          } else if (store) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + c0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                w[j] = pack_bf16x2(__uint_as_float(g[8 * i + 2 * j]) * scale,
                                   __uint_as_float(g[8 * i + 2 * j + 1]) * scale);
              d4[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      if (!SWIGLU && MT == 1 && write_partial) {
        // Split-K: the CTA that finishes an output tile last adds the splits' partial sums in split order
        // (the same order whichever CTA is last: deterministic) and writes the tile.
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          int* ticket = p.split_tickets + mt * gridDim.x + n_tile;
          const int t = atomicAdd(ticket, 1);
          last_split = (t == splits - 1) ? 1 : 0;
          if (t == splits - 1)
            *ticket = 0;   // every split has arrived: ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (last_split) {
          // all 128 epilogue threads share the live rows: 8 threads per row (32 bytes of fp32 each), 16 rows per
          // pass, the splits' loads of a pass all in flight at once
          __threadfence();
          const int t = threadIdx.x - 64;
          const int cg = (t & 7) * 8, r0 = t >> 3;
          const int rows_live = min(kGemmBM, m_count - mt * BM);
          const int64_t zstride = static_cast<int64_t>(p.split_rows) * p.n_total;
          for (int r = r0; r < rows_live; r += 16) {
            const int mr = mt * BM + r;
            const int orow = p.out_row_map ? p.out_row_map[mr] : mr;
            if (orow < 0)
              continue;
            const float sc = p.row_scale ? p.row_scale[mr] : 1.0f;
            __nv_bfloat16* drow = (p.out2 && n0 >= p.split_col)
                                      ? p.out2 + static_cast<int64_t>(orow) * p.ldc2 + (n0 - p.split_col)
                                      : p.out + static_cast<int64_t>(orow) * p.ldc + n0;
            const float* srow = p.partial + static_cast<int64_t>(mr) * p.n_total + n0;
#pragma unroll
            for (int c0 = 0; c0 < BNH; c0 += 64) {
              float4 va[4], vb[4];
#pragma unroll
              for (int z = 0; z < 4; ++z) {
                if (z < splits) {
                  const float4* src = reinterpret_cast<const float4*>(srow + z * zstride + c0 + cg);
                  va[z] = __ldcg(src);
                  vb[z] = __ldcg(src + 1);
                } else {
                  va[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                  vb[z] = va[z];
                }
              }
              float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int z = 0; z < 4; ++z) {   // split order: the same sum whichever CTA arrives last
                acc8[0] += va[z].x; acc8[1] += va[z].y; acc8[2] += va[z].z; acc8[3] += va[z].w;
                acc8[4] += vb[z].x; acc8[5] += vb[z].y; acc8[6] += vb[z].z; acc8[7] += vb[z].w;
              }
              *reinterpret_cast<uint4*>(drow + c0 + cg) =
                  make_uint4(pack_bf16x2(acc8[0] * sc, acc8[1] * sc), pack_bf16x2(acc8[2] * sc, acc8[3] * sc),
                             pack_bf16x2(acc8[4] * sc, acc8[5] * sc), pack_bf16x2(acc8[6] * sc, acc8[7] * sc));
            }
          }
        }
      }
      }
      // the accumulator may be overwritten by the tile after next (MT = 2: by the next tile)
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty_bar[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace dyllm
