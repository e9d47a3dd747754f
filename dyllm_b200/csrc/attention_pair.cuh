// Approximate (delta) attention, second decomposition: one CTA per SM works on PAIRS of 128-row query tiles of
// one (sequence, head) and splits the phases of an item over different warps, so that the phases of consecutive
// items overlap instead of following one another on the same eight warps:
//
//   warp 0        TMA producer: the two Q tiles of the pair, K tiles of 128 keys through a two-stage ring
//                 (both tiles of the pair share every K tile)
//   warp 1        tensor memory owner and MMA issuer: S_s = Q_s K^T per stream s (N = 128, one S buffer per stream:
//                 while the softmax threads of one stream read theirs the other stream's product is issued), the
//                 logits of the salient keys in chunks of 16, O_s += P_s dV
//   warp 2        TMA of the context tiles: previous context in, updated tile out (output tensor and, in place,
//                 the context cache)
//   warps 4-11, 12-19  softmax threads of stream 0 / 1, two per query row (64 of the 128 keys of a step each): running
//                 maximum and sum over all keys (pass A), P = exp2(s c - m c) of the salient keys as bf16 into
//                 shared memory (pass B); stream 0 also gathers the salient K / dV rows.  Four softmax warps per
//                 scheduler keep the exponential unit busy while others wait for tensor memory or reduce maxima.
//   warps 20-23, 24-27 epilogue threads of stream 0 / 1, one per query row: new = old + O / rowsum (salient query
//                 rows take the exactly attended row), statistics, bf16 tile back to shared memory
//
// The softmax threads start the next pair as soon as they have handed (1 / rowsum) to the epilogue threads, so the
// exponentials of pair i + 1 run while pair i's context update is computed and stored.  Tensor memory: per stream
// a 128-column S buffer and a 128-column O accumulator (512 columns, one CTA per SM).  Shared memory: 2 x 32 KB
// Q, 2 x 32 KB K, 2 x 32 KB context tiles, 16 KB P, 8 KB salient K / dV = 216 KB.
//
// Every wait is bounded (mbar_wait); a wait that runs out raises the CTA's abort flag and the device status word.
// Included by attention.cu inside namespace dyllm { namespace { ... } }.
#pragma once

constexpr int kPairThreads = 896;
constexpr int kPairKeys = 128;                                 // keys per K stage and per product (N = 128: the MMA
                                                               // warp issues one tcgen05.mma per ~68 clocks, so narrower
                                                               // products would leave the tensor pipe waiting for it)
constexpr int kPairKStages = 2;
constexpr uint32_t kPairKStageBytes = kPairKeys * 128 * 2;     // two swizzled halves [128 keys][64 d]
constexpr uint32_t kPairKHalfBytes = kPairKeys * 64 * 2;
constexpr uint32_t kPairPBytes = 128 * 64 * 2;                 // one swizzled half tile [128 rows][64 columns]: stream s
                                                               // uses columns 16 s .. 16 s + 15 (32 bytes per row)
constexpr uint32_t kPairSmem =
    2 * kTileBytes + kPairKStages * kPairKStageBytes + 2 * kTileBytes + kPairPBytes + 2 * kSalBytes + 1024;
constexpr uint32_t kPairTmemCols = 512;

#ifdef DYLLM_ATTN_TRACE
#define DYLLM_PTRACE(cond, slot)                                                                  \
  do {                                                                                            \
    if (p.trace && (cond) && item < 1024)                                                         \
      p.trace[item * 16 + (slot)] = (slot) == 0 || (slot) == 15 ? global_ns() : (unsigned long long)clock64(); \
  } while (0)
#else
#define DYLLM_PTRACE(cond, slot) do { } while (0)
#endif

// One arrival per warp (the barriers count warps, not threads).  Every lane has done its fences before the
// __syncwarp.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0)
    mbar_arrive(bar);
}

struct PairItem {
  int h, hk, sal_begin, n_sal, q_end, q0, k_begin, len_k, num_kt, n_chunks;
  int k_shift;       // K row of a query row listed in idx_q when no K-space list is given: idx_q[i] + k_shift
  int64_t c_delta;   // C_old row of query row r: r + c_delta (cache-resident context)
  bool live1;        // the pair's second tile holds query rows
  bool tile_tma[2];  // the tile lies completely inside the sequence: context through shared memory
};

// Work item `item` = (sequence, head, pair of query tiles), pairs fastest; false when it holds no query rows.
__device__ __forceinline__ bool decode_pair(const AttnParams& p, int item, PairItem& it) {
  const int n_pairs = (p.n_qtiles + 1) >> 1;
  const int pair = item % n_pairs;
  it.h = (item / n_pairs) % p.H;
  const int b = item / (n_pairs * p.H);
  it.sal_begin = p.cu_sal[b];
  it.n_sal = p.cu_sal[b + 1] - it.sal_begin;
  const int q_begin = p.cu_q[b];
  it.q_end = p.cu_q[b + 1];
  it.q0 = q_begin + pair * 2 * kBQ;
  if (it.q0 >= it.q_end)
    return false;
  it.k_begin = p.cu_k[b];
  it.len_k = p.cu_k[b + 1] - it.k_begin;
  it.num_kt = (it.len_k + kPairKeys - 1) / kPairKeys;
  it.hk = it.h / (p.H / p.Hkv);
  it.n_chunks = (it.n_sal + kFastSal - 1) / kFastSal;
  // the queries of a sequence are its last len_q rows
  it.k_shift = it.k_begin + it.len_k - (it.q_end - q_begin) - q_begin;
  it.c_delta = p.c_seq_starts ? p.c_seq_starts[p.c_seq_ids[b]] + (it.len_k - (it.q_end - q_begin)) - q_begin : 0;
  it.live1 = it.q0 + kBQ < it.q_end;
  it.tile_tma[0] = it.q0 + kBQ <= it.q_end;
  it.tile_tma[1] = it.q0 + 2 * kBQ <= it.q_end;
  return true;
}

__global__ void __launch_bounds__(kPairThreads, 1)
delta_attention_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_c,
                            const AttnParams p) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;                                             // [2] Q tiles
  uint8_t* k_smem = q_smem + 2 * kTileBytes;                          // [3] K stages
  uint8_t* c_smem = k_smem + kPairKStages * kPairKStageBytes;         // [2] context tiles
  uint8_t* p_smem = c_smem + 2 * kTileBytes;                          // P of both streams (salient keys of one chunk)
  uint8_t* ks_smem = p_smem + kPairPBytes;                            // gathered salient K rows of one chunk
  uint8_t* dvs_smem = ks_smem + kSalBytes;                            // gathered dV rows of one chunk
  __shared__ uint64_t q_full, q_free, k_full[kPairKStages], k_empty[kPairKStages];
  __shared__ uint64_t s_full[2], s_empty[2], b_full, b_free, p_full[2], pv_done[2], o_free[2], epi_ready[2];
  __shared__ uint64_t c_full[2], c_stored[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float s_invl[2][128];         // 1 / rowsum, softmax threads -> epilogue threads
  __shared__ float2 s_ml[2][2][128];       // (max, sum) of the two column halves of each query row
  __shared__ uint16_t s_sal_pos[2][128];   // 1 + position in the sequence's salient list of a query row, 0 = not salient

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    mbar_init(&q_free, 1);
    for (int i = 0; i < kPairKStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 8);
      mbar_init(&p_full[s], 8);
      mbar_init(&pv_done[s], 1);
      mbar_init(&o_free[s], 4);
      mbar_init(&epi_ready[s], 4);
      mbar_init(&c_full[s], 1);
      mbar_init(&c_stored[s], 4);
    }
    mbar_init(&b_full, 8);
    mbar_init(&b_free, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_c);
    tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kPairTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;   // stream s: S at s * 256, O at s * 256 + 128

  if (warp == 0) {
    // ---------------------------------------------------------------- producer: Q tiles of the pair, K ring
    int n_items = 0, ku = 0;
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      PairItem it;
      if (!decode_pair(p, item, it))
        continue;
      // The first K tiles go out before the Q tiles: their stages have been free since the end of the previous
      // pair's pass A, while Q is only released by that pair's last product with it.
      auto load_k = [&](int kt) {
        const int st = ku % kPairKStages;
        mbar_wait(&k_empty[st], ((ku / kPairKStages) & 1) ^ 1, &abort_flag, p.status_word, 402);
        if (lane == 0) {
          uint8_t* dst = k_smem + st * kPairKStageBytes;
          mbar_arrive_expect_tx(&k_full[st], kPairKStageBytes);
          tma_load_2d(dst, &tmap_k, &k_full[st], it.hk * kD, it.k_begin + kt * kPairKeys);
          tma_load_2d(dst + kPairKHalfBytes, &tmap_k, &k_full[st], it.hk * kD + 64, it.k_begin + kt * kPairKeys);
        }
        __syncwarp();
        ++ku;
      };
      int kt = 0;
      for (; kt < it.num_kt && kt < kPairKStages; ++kt)
        load_k(kt);
      if (n_items > 0)
        mbar_wait(&q_free, (n_items - 1) & 1, &abort_flag, p.status_word, 401);
      if (lane == 0) {
        mbar_arrive_expect_tx(&q_full, it.live1 ? 2 * kTileBytes : kTileBytes);
        for (int s = 0; s < (it.live1 ? 2 : 1); ++s) {
          tma_load_2d(q_smem + s * kTileBytes, &tmap_q, &q_full, it.h * kD, it.q0 + s * kBQ);
          tma_load_2d(q_smem + s * kTileBytes + kHalfBytes, &tmap_q, &q_full, it.h * kD + 64, it.q0 + s * kBQ);
        }
        // the Q tiles of this CTA's next pair into L2: they are read from HBM for the first time
        PairItem nx;
        const int next = item + gridDim.x;
        if (next < p.num_items && decode_pair(p, next, nx)) {
          for (int s = 0; s < (nx.live1 ? 2 : 1); ++s) {
            tma_prefetch_2d(&tmap_q, nx.h * kD, nx.q0 + s * kBQ);
            tma_prefetch_2d(&tmap_q, nx.h * kD + 64, nx.q0 + s * kBQ);
          }
        }
      }
      __syncwarp();
      for (; kt < it.num_kt; ++kt)
        load_k(kt);
      ++n_items;
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = umma_idesc_bf16(128, kPairKeys, 0, 0);
    constexpr uint32_t idesc_sal = umma_idesc_bf16(128, kFastSal, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);   // dV rows as loaded: MN-major B operand
    int n_items = 0, kc = 0, n_b = 0;
    int use[2] = {0, 0};                // how often each stream's S buffer has been handed to the softmax threads
    int n_p[2] = {0, 0};                // P chunks consumed per stream
    int n_live[2] = {0, 0};             // items in which the stream held rows
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      PairItem it;
      if (!decode_pair(p, item, it))
        continue;
      const int ns = it.live1 ? 2 : 1;
      mbar_wait(&q_full, n_items & 1, &abort_flag, p.status_word, 403);
      DYLLM_PTRACE(lane == 0, 12);
      for (int kt = 0; kt < it.num_kt; ++kt, ++kc) {
        const int st = kc % kPairKStages;
        mbar_wait(&k_full[st], (kc / kPairKStages) & 1, &abort_flag, p.status_word, 404);
        const uint32_t kb_addr = smem_u32(k_smem + st * kPairKStageBytes);
        for (int s = 0; s < ns; ++s) {
          const int u = use[s]++;
          mbar_wait(&s_empty[s], (u & 1) ^ 1, &abort_flag, p.status_word, 405);
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t q_addr = smem_u32(q_smem + s * kTileBytes);
            const uint32_t tmem_s = tmem_base + s * 256;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const uint64_t a_desc = umma_smem_desc_sw128(q_addr + half * kHalfBytes, 16, 1024);
              const uint64_t b_desc = umma_smem_desc_sw128(kb_addr + half * kPairKHalfBytes, 16, 1024);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_ss(tmem_s, a_desc + 2 * kk, b_desc + 2 * kk, idesc_qk, (half | kk) != 0 ? 1u : 0u);
            }
            umma_commit(&s_full[s]);
          }
          __syncwarp();
        }
        if (lane == 0)
          umma_commit(&k_empty[st]);
        __syncwarp();
        if (kt == 0)
          DYLLM_PTRACE(lane == 0, 13);
        if (kt == 1)
          DYLLM_PTRACE(lane == 0, 14);
      }
      if (it.n_chunks == 0 && lane == 0)
        umma_commit(&q_free);   // the last product with Q has been issued
      for (int ch = 0; ch < it.n_chunks; ++ch) {
        mbar_wait(&b_full, (n_b++) & 1, &abort_flag, p.status_word, 406);
        for (int s = 0; s < ns; ++s) {
          const int u = use[s]++;
          mbar_wait(&s_empty[s], (u & 1) ^ 1, &abort_flag, p.status_word, 407);
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t q_addr = smem_u32(q_smem + s * kTileBytes);
            const uint32_t tmem_s = tmem_base + s * 256;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const uint64_t a_desc = umma_smem_desc_sw128(q_addr + half * kHalfBytes, 16, 1024);
              const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(ks_smem) + half * kSalHalfBytes, 16, 1024);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_ss(tmem_s, a_desc + 2 * kk, b_desc + 2 * kk, idesc_sal, (half | kk) != 0 ? 1u : 0u);
            }
            umma_commit(&s_full[s]);
          }
          __syncwarp();
        }
        if (ch == it.n_chunks - 1 && lane == 0)
          umma_commit(&q_free);
        for (int s = 0; s < ns; ++s) {
          mbar_wait(&p_full[s], (n_p[s]++) & 1, &abort_flag, p.status_word, 408);
          if (ch == 0 && n_live[s] > 0)   // the epilogue of the stream's previous item has read O
            mbar_wait(&o_free[s], (n_live[s] - 1) & 1, &abort_flag, p.status_word, 409);
          tc_fence_after_sync();
          if (lane == 0) {
            const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(p_smem) + s * 32, 16, 1024);
            const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(dvs_smem), kSalHalfBytes, 1024);
            umma_ss(tmem_base + s * 256 + 128, a_desc, b_desc, idesc_pv, ch != 0 ? 1u : 0u);
          }
          __syncwarp();
        }
        if (lane == 0) {
          umma_commit(&b_free);   // the chunk's K / dV rows and both P buffers have been read
          if (ch == it.n_chunks - 1) {
            umma_commit(&pv_done[0]);
            if (ns == 2)
              umma_commit(&pv_done[1]);
          }
        }
        __syncwarp();
      }
      for (int s = 0; s < ns; ++s)
        ++n_live[s];
      ++n_items;
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- context tiles in and out
    int n_cs[2] = {0, 0};
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      PairItem it;
      if (!decode_pair(p, item, it))
        continue;
      const int ns = it.live1 ? 2 : 1;
      if (lane == 0) {
        for (int s = 0; s < ns; ++s)
          if (it.tile_tma[s]) {
            uint8_t* dst = c_smem + s * kTileBytes;
            const int crow = static_cast<int>(it.q0 + s * kBQ + it.c_delta);
            mbar_arrive_expect_tx(&c_full[s], kTileBytes);
            tma_load_2d(dst, &tmap_c, &c_full[s], it.h * kD, crow);
            tma_load_2d(dst + kHalfBytes, &tmap_c, &c_full[s], it.h * kD + 64, crow);
          }
      }
      __syncwarp();
      for (int s = 0; s < ns; ++s)
        if (it.tile_tma[s]) {
          mbar_wait(&c_stored[s], (n_cs[s]++) & 1, &abort_flag, p.status_word, 410);
          if (lane == 0) {
            const uint8_t* src = c_smem + s * kTileBytes;
            const int orow = it.q0 + s * kBQ;
            tma_store_2d(&tmap_out, src, it.h * kD, orow);
            tma_store_2d(&tmap_out, src + kHalfBytes, it.h * kD + 64, orow);
            if (p.c_cache) {
              const int crow = static_cast<int>(orow + it.c_delta);
              tma_store_2d(&tmap_c, src, it.h * kD, crow);
              tma_store_2d(&tmap_c, src + kHalfBytes, it.h * kD + 64, crow);
            }
            tma_store_commit();
          }
          __syncwarp();
        }
      if (lane == 0)
        tma_store_wait_read();   // the tiles may be overwritten by the next item's loads
      __syncwarp();
    }
    if (lane == 0)
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else if (warp >= 4 && warp < 20) {
    // ---------------------------------------------------------------- softmax threads, two per query row
    const int s = (warp - 4) >> 3;
    const int half = ((warp - 4) >> 2) & 1;  // which 64 of the 128 keys of a step
    const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
    const int row = qd * 32 + lane;          // query row inside the stream's tile
    const int tid_s = ((warp - 4) & 7) * 32 + lane;   // 0..255 among the stream's softmax threads
    const uint32_t t_lane = static_cast<uint32_t>(qd * 32) << 16;
    const float c = p.scale_log2;
    int use = 0;             // how often the stream's S buffer has been read
    int chunks_done = 0;     // salient chunks of this CTA so far (phases of b_free)
    int n_live = 0;
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      PairItem it;
      if (!decode_pair(p, item, it))
        continue;
      if (s == 1 && !it.live1) {
        chunks_done += it.n_chunks;
        continue;
      }
      const int q0s = it.q0 + s * kBQ;
      const bool warp_live = q0s + qd * 32 < it.q_end;
      DYLLM_PTRACE(s == 0 && tid_s == 0, 0);
      DYLLM_PTRACE(s == 0 && tid_s == 0, 1);
      // stream 0: the K / dV rows of the first salient chunk (16 rows x 16 pieces of 16 bytes, one per thread)
      // are requested now and written after pass A
      uint4 ek = make_uint4(0, 0, 0, 0), ev = make_uint4(0, 0, 0, 0);
      if (s == 0 && it.n_chunks > 0) {
        const int r = tid_s >> 4, ch16 = tid_s & 15;
        if (r < it.n_sal) {
          const int src = p.idx_k ? p.idx_k[it.sal_begin + r] : p.idx_q[it.sal_begin + r] + it.k_shift;
          ek = __ldg(reinterpret_cast<const uint4*>(p.k + (static_cast<int64_t>(src) * p.Hkv + it.hk) * kD) + ch16);
          const int64_t vrow = p.v_compact ? static_cast<int64_t>(it.sal_begin + r) : src;
          ev = __ldg(reinterpret_cast<const uint4*>(p.v + (vrow * p.Hkv + it.hk) * kD) + ch16);
        }
      }
      // pass A: running maximum and sum over this thread's 64 of the 128 keys of every step
      float m = kNegBig, l = 0.f;
      for (int kt = 0; kt < it.num_kt; ++kt) {
        const int u = use++;
        mbar_wait(&s_full[s], u & 1, &abort_flag, p.status_word, 411);
        tc_fence_after_sync();
        if (kt == 0)
          DYLLM_PTRACE(s == 0 && tid_s == 0, 2);
        if (kt == 1)
          DYLLM_PTRACE(s == 0 && tid_s == 0, 3);
        const int valid = it.len_k - kt * kPairKeys;   // keys of this tile that belong to the sequence
        if (!warp_live) {
          tc_fence_before_sync();
          warp_arrive(&s_empty[s], lane);
          continue;
        }
#pragma unroll 1
        for (int cc = 0; cc < 64; cc += 32) {
          const int c0 = half * 64 + cc;
          uint32_t sr[32];
          tmem_ld_32x32(tmem_base + s * 256 + t_lane + c0, sr);
          tmem_ld_wait();
          if (cc == 32) {  // last chunk read: the MMA warp may overwrite the S buffer
            tc_fence_before_sync();
            warp_arrive(&s_empty[s], lane);
          }
          if (valid < kPairKeys) {   // keys past the end of the sequence
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c0 + i >= valid)
                sr[i] = __float_as_uint(kNegBig);
          }
          // maximum of the 32 values as four independent chains
          float mx0 = fmax3(__uint_as_float(sr[0]), __uint_as_float(sr[1]), __uint_as_float(sr[2]));
          float mx1 = fmax3(__uint_as_float(sr[8]), __uint_as_float(sr[9]), __uint_as_float(sr[10]));
          float mx2 = fmax3(__uint_as_float(sr[16]), __uint_as_float(sr[17]), __uint_as_float(sr[18]));
          float mx3 = fmax3(__uint_as_float(sr[24]), __uint_as_float(sr[25]), __uint_as_float(sr[26]));
          mx0 = fmax3(mx0, __uint_as_float(sr[3]), __uint_as_float(sr[4]));
          mx1 = fmax3(mx1, __uint_as_float(sr[11]), __uint_as_float(sr[12]));
          mx2 = fmax3(mx2, __uint_as_float(sr[19]), __uint_as_float(sr[20]));
          mx3 = fmax3(mx3, __uint_as_float(sr[27]), __uint_as_float(sr[28]));
          mx0 = fmax3(mx0, __uint_as_float(sr[5]), __uint_as_float(sr[6]));
          mx1 = fmax3(mx1, __uint_as_float(sr[13]), __uint_as_float(sr[14]));
          mx2 = fmax3(mx2, __uint_as_float(sr[21]), __uint_as_float(sr[22]));
          mx3 = fmax3(mx3, __uint_as_float(sr[29]), __uint_as_float(sr[30]));
          mx0 = fmax3(mx0, __uint_as_float(sr[7]), mx1);
          mx2 = fmax3(mx2, __uint_as_float(sr[15]), mx3);
          const float cmax = fmax3(fmax3(mx0, mx2, __uint_as_float(sr[23])), __uint_as_float(sr[31]), kNegBig);
          const float m_new = fmaxf(m, cmax);
          const float mc = m_new * c;
          const float2 c2 = make_float2(c, c), nmc2 = make_float2(-mc, -mc);
          float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 x0 =
                ffma2(make_float2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), c2, nmc2);
            const float2 x1 =
                ffma2(make_float2(__uint_as_float(sr[2 * i + 2]), __uint_as_float(sr[2 * i + 3])), c2, nmc2);
            acc0 = fadd2(acc0, make_float2(ex2(x0.x), ex2(x0.y)));
            acc1 = fadd2(acc1, make_float2(ex2(x1.x), ex2(x1.y)));
          }
          const float sum = (acc0.x + acc1.x) + (acc0.y + acc1.y);
          l = l * ex2((m - m_new) * c) + sum;
          m = m_new;
        }
      }
      // merge the two column halves of each row: m = max, l rescaled to the common maximum
      s_ml[s][half][row] = make_float2(m, l);
      if (s == 0)
        asm volatile("bar.sync 1, 256;" ::: "memory");
      else
        asm volatile("bar.sync 2, 256;" ::: "memory");
      {
        const float2 other = s_ml[s][half ^ 1][row];
        const float m_all = fmaxf(m, other.x);
        l = l * ex2((m - m_all) * c) + other.y * ex2((other.x - m_all) * c);
        m = m_all;
      }
      const float mc = m * c;
      DYLLM_PTRACE(s == 0 && tid_s == 0, 4);
      // pass B: the salient keys in chunks of 16; this thread computes 8 of a row's 16 probabilities
      for (int ch = 0; ch < it.n_chunks; ++ch, ++chunks_done) {
        if (s == 0 && ch > 0) {
          const int r = ch * kFastSal + (tid_s >> 4), ch16 = tid_s & 15;
          ek = ev = make_uint4(0, 0, 0, 0);
          if (r < it.n_sal) {
            const int src = p.idx_k ? p.idx_k[it.sal_begin + r] : p.idx_q[it.sal_begin + r] + it.k_shift;
            ek = __ldg(reinterpret_cast<const uint4*>(p.k + (static_cast<int64_t>(src) * p.Hkv + it.hk) * kD) + ch16);
            const int64_t vrow = p.v_compact ? static_cast<int64_t>(it.sal_begin + r) : src;
            ev = __ldg(reinterpret_cast<const uint4*>(p.v + (vrow * p.Hkv + it.hk) * kD) + ch16);
          }
        }
        // the previous chunk's products have read the gathered rows and the P buffer
        if (chunks_done > 0)
          mbar_wait(&b_free, (chunks_done - 1) & 1, &abort_flag, p.status_word, 412);
        if (s == 0) {
          const int r = tid_s >> 4, ch16 = tid_s & 15;
          *reinterpret_cast<uint4*>(ks_smem + (ch16 >> 3) * kSalHalfBytes + sw128_offset(r, ch16 & 7)) = ek;
          *reinterpret_cast<uint4*>(dvs_smem + (ch16 >> 3) * kSalHalfBytes + sw128_offset(r, ch16 & 7)) = ev;
          fence_proxy_async_smem();
          warp_arrive(&b_full, lane);
        }
        const int u = use++;
        mbar_wait(&s_full[s], u & 1, &abort_flag, p.status_word, 413);
        tc_fence_after_sync();
        DYLLM_PTRACE(s == 0 && tid_s == 0 && ch == 0, 5);
        uint32_t sr[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          sr[i] = 0u;
        if (warp_live) {
          tmem_ld_32x16(tmem_base + s * 256 + t_lane, sr);
          tmem_ld_wait();
        }
        tc_fence_before_sync();
        warp_arrive(&s_empty[s], lane);
        const int n_valid = min(kFastSal, it.n_sal - ch * kFastSal);
        uint32_t pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j0 = half * 8 + 2 * i;
          const float x0 = half ? __uint_as_float(sr[8 + 2 * i]) : __uint_as_float(sr[2 * i]);
          const float x1 = half ? __uint_as_float(sr[9 + 2 * i]) : __uint_as_float(sr[2 * i + 1]);
          const float p0 = (warp_live && j0 < n_valid) ? ex2(fmaf(x0, c, -mc)) : 0.f;
          const float p1 = (warp_live && j0 + 1 < n_valid) ? ex2(fmaf(x1, c, -mc)) : 0.f;
          __nv_bfloat162 v2 = __floats2bfloat162_rn(p0, p1);
          pk[i] = *reinterpret_cast<uint32_t*>(&v2);
        }
        *reinterpret_cast<uint4*>(p_smem + sw128_offset(row, 2 * s + half)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        fence_proxy_async_smem();
        warp_arrive(&p_full[s], lane);
      }
      // hand 1 / rowsum to the epilogue threads (they have finished the stream's previous item first)
      if (half == 0) {
        if (n_live > 0)
          mbar_wait(&o_free[s], (n_live - 1) & 1, &abort_flag, p.status_word, 414);
        s_invl[s][row] = l > 0.f ? 1.0f / l : 0.f;
        warp_arrive(&epi_ready[s], lane);
      }
      DYLLM_PTRACE(s == 0 && tid_s == 0, 6);
      ++n_live;
    }
  } else if (warp >= 20) {
    // ---------------------------------------------------------------- epilogue threads, one per query row
    const int s = (warp - 20) >> 2;
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int tid_s = ((warp - 20) & 3) * 32 + lane;
    const uint32_t t_lane = static_cast<uint32_t>(qd * 32) << 16;
    const uint32_t tmem_o = tmem_base + s * 256 + 128;
    int n_live = 0, n_pv = 0, n_c = 0;
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      PairItem it;
      if (!decode_pair(p, item, it))
        continue;
      if (s == 1 && !it.live1)
        continue;
      const int h = it.h;
      const int q0s = it.q0 + s * kBQ;
      const int r = q0s + row;
      const bool live = r < it.q_end;
      const bool tile = it.tile_tma[s];
      // mark the query rows of this tile that are salient (they take the exactly attended values)
      s_sal_pos[s][row] = 0;
      if (s == 0)
        asm volatile("bar.sync 3, 128;" ::: "memory");
      else
        asm volatile("bar.sync 4, 128;" ::: "memory");
      for (int j = tid_s; j < it.n_sal; j += 128) {
        const int rr = p.idx_q[it.sal_begin + j] - q0s;
        if (rr >= 0 && rr < kBQ)
          s_sal_pos[s][rr] = static_cast<uint16_t>(j + 1);
      }
      if (s == 0)
        asm volatile("bar.sync 3, 128;" ::: "memory");
      else
        asm volatile("bar.sync 4, 128;" ::: "memory");
      DYLLM_PTRACE(s == 0 && tid_s == 0, 7);
      mbar_wait(&epi_ready[s], n_live & 1, &abort_flag, p.status_word, 415);
      const float inv_l = s_invl[s][row];
      DYLLM_PTRACE(s == 0 && tid_s == 0, 8);
      if (tile)
        mbar_wait(&c_full[s], (n_c++) & 1, &abort_flag, p.status_word, 416);
      DYLLM_PTRACE(s == 0 && tid_s == 0, 9);
      if (it.n_chunks > 0) {
        mbar_wait(&pv_done[s], (n_pv++) & 1, &abort_flag, p.status_word, 417);
        tc_fence_after_sync();
      }
      DYLLM_PTRACE(s == 0 && tid_s == 0, 10);
      const int64_t row_off = (static_cast<int64_t>(live ? r : q0s) * p.H + h) * kD;
      const int64_t c_off = (((live ? r : q0s) + it.c_delta) * p.H + h) * kD;
      __nv_bfloat16* dst = p.out + row_off;
      __nv_bfloat16* cdst = p.c_cache ? p.c_cache + c_off : nullptr;
      uint8_t* c_tile = c_smem + s * kTileBytes;
      const int sal_pos = s_sal_pos[s][row];
      const uint4* sal_src = nullptr;
      if (sal_pos && live)
        sal_src = reinterpret_cast<const uint4*>(
            p.o_sal + (static_cast<int64_t>(it.sal_begin + sal_pos - 1) * p.H + h) * kD);
      float dot = 0.f, nn = 0.f, no = 0.f;
#pragma unroll 1
      for (int cc = 0; cc < 128; cc += 16) {
        uint32_t orr[16];
        if (it.n_chunks > 0) {
          tmem_ld_32x16(tmem_o + t_lane + cc, orr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            orr[i] = 0u;
        }
        uint8_t* c_half = c_tile + (cc >> 6) * kHalfBytes;
        const int chunk0 = (cc & 63) >> 3;
        uint4 old_row[2];
        if (tile) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            old_row[j] = *reinterpret_cast<const uint4*>(c_half + sw128_offset(row, chunk0 + j));
        } else {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            old_row[j] = live ? __ldg(reinterpret_cast<const uint4*>(p.c_old + c_off + cc) + j) : make_uint4(0, 0, 0, 0);
        }
        if (live) {
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(old_row);
          uint32_t pk[8];
          float2 d2 = make_float2(0.f, 0.f), n2 = make_float2(0.f, 0.f), q2 = make_float2(0.f, 0.f);
          if (!sal_src) {
            const float2 il2 = make_float2(inv_l, inv_l);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 of = __bfloat1622float2(o2[i]);
              const float2 nv = ffma2(make_float2(__uint_as_float(orr[2 * i]), __uint_as_float(orr[2 * i + 1])), il2, of);
              d2 = ffma2(nv, of, d2);
              n2 = ffma2(nv, nv, n2);
              q2 = ffma2(of, of, q2);
              __nv_bfloat162 v2 = __floats2bfloat162_rn(nv.x, nv.y);
              pk[i] = *reinterpret_cast<uint32_t*>(&v2);
            }
          } else {
            // salient query row (a few per sequence): the exactly attended row is the new value
            uint4 sal_row[2];
#pragma unroll
            for (int j = 0; j < 2; ++j)
              sal_row[j] = __ldg(sal_src + cc / 8 + j);
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(sal_row);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 of = __bfloat1622float2(o2[i]);
              const float2 nv = __bfloat1622float2(x2[i]);
              d2 = ffma2(nv, of, d2);
              n2 = ffma2(nv, nv, n2);
              q2 = ffma2(of, of, q2);
              pk[i] = reinterpret_cast<const uint32_t*>(sal_row)[i];
            }
          }
          dot += d2.x + d2.y;
          nn += n2.x + n2.y;
          no += q2.x + q2.y;
          if (tile) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              *reinterpret_cast<uint4*>(c_half + sw128_offset(row, chunk0 + j)) =
                  make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              reinterpret_cast<uint4*>(dst + cc)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            if (cdst) {
#pragma unroll
              for (int j = 0; j < 2; ++j)
                reinterpret_cast<uint4*>(cdst + cc)[j] =
                    make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            }
          }
        }
      }
      DYLLM_PTRACE(s == 0 && tid_s == 0, 11);
      // O and 1 / rowsum of this item have been read: the stream's next item may overwrite them
      tc_fence_before_sync();
      warp_arrive(&o_free[s], lane);
      if (tile) {
        fence_proxy_async_smem();   // the updated tile is read by the TMA stores of warp 2
        warp_arrive(&c_stored[s], lane);
      }
      if (live) {
        float* ps = p.partial + (static_cast<int64_t>(h) * p.Tq + r) * 3;
        ps[0] = dot;
        ps[1] = nn;
        ps[2] = no;
      }
      ++n_live;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_slot, kPairTmemCols);
  }
}
