// Row-gathered bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), shared by the dense
// SwiGLU FFN and the MoE expert FFN.
//
//   D[m, n] = sum_k A[a_idx[m], k] * B[b_row0(m_tile) + n, k]          (fp32 accumulation in TMEM)
//
// One CTA computes one 128 x BN output tile.  Warp roles (6 warps):
//   warp 0      producer: weight tiles by TMA (128-byte swizzle); activation rows by TMA gather4
//               (A_MODE 1), by a plain TMA box (A_MODE 0, no gather) or not at all (A_MODE 2)
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits to mbarriers
//   warps 2..5  epilogue: tcgen05.ld of the accumulator, SiLU(gate) * up or scale, bf16 stores, row
//               scatter; in A_MODE 2 they first gather the activation rows with 16-byte loads into the
//               swizzled tile (generic-proxy writes + fence.proxy.async)
// Every wait is bounded; a wait that runs out raises the CTA's abort flag and the device status word.
#pragma once

#include "common.cuh"

namespace dyllm {

struct GemmParams {
  const __nv_bfloat16* a;      // activation matrix (A_MODE 2 reads it directly)
  const int32_t* a_idx;        // [M] source row of A for logical row m; null = identity
  const int32_t* m_count_dev;  // device scalar bounding the live logical rows; null = M
  const int32_t* tile_expert;  // [ceil(M/128)] weight block per row tile; null = block 0
  int M;                       // upper bound of logical rows (grid is sized for it)
  int K;                       // contraction length, multiple of 64
  int a_rows;                  // rows of the activation matrix (for clamping)
  int64_t lda;                 // row pitch of A in elements
  int b_rows_per_expert;       // rows of B per weight block
  int up_row_offset;           // SwiGLU: row distance from the gate rows to the up rows
  __nv_bfloat16* out;          // output matrix
  int64_t ldc;                 // row pitch of the output in elements
  const int32_t* out_row_map;  // [M] destination row per logical row (negative = drop); null = m
  const float* row_scale;      // [M] multiplier per logical row; null = 1
  int* status_word;
};

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 192;

template <int BNH, bool SWIGLU, int STAGES>
struct GemmCfg {
  static constexpr int BN = SWIGLU ? 2 * BNH : BNH;  // UMMA N
  static constexpr uint32_t A_BYTES = kGemmBM * kGemmBK * 2;
  static constexpr uint32_t B_BYTES = BN * kGemmBK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + alignment slack
  static constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M = 128");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "tensor memory columns must be a power of two");
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int BNH, bool SWIGLU, int A_MODE, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gathered_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const GemmParams p) {
  using Cfg = GemmCfg<BNH, SWIGLU, STAGES>;
  constexpr int BM = kGemmBM, BK = kGemmBK, BN = Cfg::BN;

  const int m_tile = blockIdx.x;
  const int n_tile = blockIdx.y;
  const int m0 = m_tile * BM;
  const int m_count = p.m_count_dev ? min(*p.m_count_dev, p.M) : p.M;
  if (m0 >= m_count)
    return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kt = p.K / BK;
  const int b_row0 = (p.tile_expert ? p.tile_expert[m_tile] : 0) * p.b_rows_per_expert + n_tile * BNH;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], A_MODE == 2 ? 1 + 128 : 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    fence_mbar_init();
    if (A_MODE != 2)
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
  const uint32_t tmem_acc = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
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
    for (int kt = 0; kt < num_kt; ++kt) {
      const int s = kt % STAGES;
      const uint32_t ph = (kt / STAGES) & 1;
      mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, p.status_word, 201);
      uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
      uint8_t* b_dst = a_dst + Cfg::A_BYTES;
      if (lane == 0) {
        mbar_arrive_expect_tx(&full_bar[s], A_MODE == 2 ? Cfg::B_BYTES : Cfg::STAGE_BYTES);
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
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, 0);
    for (int kt = 0; kt < num_kt; ++kt) {
      const int s = kt % STAGES;
      const uint32_t ph = (kt / STAGES) & 1;
      mbar_wait(&full_bar[s], ph, &abort_flag, p.status_word, 202);
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint32_t b_addr = a_addr + Cfg::A_BYTES;
        const uint64_t a_desc = umma_smem_desc_sw128(a_addr, 16, 1024);
        const uint64_t b_desc = umma_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_ss(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt | k) != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);
        if (kt == num_kt - 1)
          umma_commit(&tmem_full_bar);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ gather (A_MODE 2) + epilogue
    const int q = warp & 3;            // tensor-memory lane quarter this warp may read
    const int row = q * 32 + lane;     // accumulator row == logical row m0 + row
    const int m = m0 + row;
    const bool live = m < m_count;

    if (A_MODE == 2) {
      int src = 0;
      if (live)
        src = p.a_idx ? p.a_idx[m] : m;
      src = min(max(src, 0), p.a_rows - 1);
      const uint4* src_row = reinterpret_cast<const uint4*>(p.a + static_cast<int64_t>(src) * p.lda);
      for (int kt = 0; kt < num_kt; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        uint4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          v[c] = __ldg(src_row + kt * 8 + c);
        mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, p.status_word, 203);
        uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(a_dst + sw128_offset(row, c)) = v[c];
        fence_proxy_async_smem();
        mbar_arrive(&full_bar[s]);
      }
    }

    mbar_wait(&tmem_full_bar, 0, &abort_flag, p.status_word, 204);
    tc_fence_after_sync();
    const uint32_t t_row = tmem_acc + (static_cast<uint32_t>(q * 32) << 16);
    int out_row = m;
    if (p.out_row_map && live)
      out_row = p.out_row_map[m];
    const bool store = live && out_row >= 0;
    __nv_bfloat16* dst = p.out + static_cast<int64_t>(store ? out_row : 0) * p.ldc + n_tile * BNH;
    const float scale = (p.row_scale && live) ? p.row_scale[m] : 1.0f;

#pragma unroll 1
    for (int c0 = 0; c0 < BNH; c0 += 32) {
      uint32_t g[32];
      uint32_t packed[16];
      tmem_ld_32x32(t_row + c0, g);
      if (SWIGLU) {
        uint32_t u[32];
        tmem_ld_32x32(t_row + BNH + c0, u);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float h0 = silu_f(__uint_as_float(g[2 * i])) * __uint_as_float(u[2 * i]);
          const float h1 = silu_f(__uint_as_float(g[2 * i + 1])) * __uint_as_float(u[2 * i + 1]);
          packed[i] = pack_bf16x2(h0, h1);
        }
      } else {
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i)
          packed[i] = pack_bf16x2(__uint_as_float(g[2 * i]) * scale, __uint_as_float(g[2 * i + 1]) * scale);
      }
      if (store) {
        uint4* d4 = reinterpret_cast<uint4*>(dst + c0);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          d4[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_acc, Cfg::TMEM_COLS);
  }
}

}  // namespace dyllm
