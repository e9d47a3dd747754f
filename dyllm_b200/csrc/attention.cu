// Approximate (delta) attention for a sparse denoising step, head_dim 128:
//
//   O[r] = bf16( C_old[r] + sum_k softmax_k(q_r . k_k / sqrt(D)) * dV_k )      for every query row r
//
// dV is non-zero only on the salient key rows of the step, so the work splits into
//   pass A  row maximum and row sum of exp over ALL keys of the sequence: S = Q K^T on the tensor cores
//           (tcgen05, accumulator in tensor memory), online max/sum by four softmax warps (one thread
//           per query row);
//   pass B  the salient keys only: their K rows and dV rows are gathered into swizzled shared-memory
//           tiles, S2 = Q Ksal^T, P = exp2(S2*c - m*c) as bf16, O += P dVsal on the tensor cores;
//   epilogue  new = C_old + O / rowsum, bf16 store, per-head partial cosine statistics from the fp32
//           value before rounding.
// A second small kernel adds the per-head partials in head order (run-to-run identical results),
// overwrites the salient query rows with the exactly attended rows and writes the threshold mask.
//
// One CTA = (sequence, query head, 128 query rows); 10 warps: TMA producer, MMA issuer, 8 softmax warps
// (two per 32-row lane quarter, each taking half of the columns).  96 KB of shared memory and 256
// tensor-memory columns per CTA, so two CTAs share an SM and one CTA's tensor-core work overlaps the
// other's exponentials.
#include "common.cuh"

namespace dyllm {

namespace {

constexpr int kD = 128;          // head dimension
constexpr int kBQ = 128;         // query rows per CTA
constexpr int kBKeys = 128;      // keys per tile
constexpr int kAttnThreads = 320;          // TMA producer warp, MMA warp, eight softmax warps
constexpr uint32_t kTileBytes = 128 * 128 * 2;   // one [128][128] bf16 tile = two [128][64] swizzled halves
constexpr uint32_t kHalfBytes = 128 * 64 * 2;
constexpr uint32_t kAttnSmem = 3 * kTileBytes + 1024;
// Tensor memory: two S buffers (columns 0..127 and 128..255) during pass A, so that the product of
// key tile t+1 runs while tile t is being reduced; in pass B the second buffer holds O.
constexpr uint32_t kAttnTmemCols = 256;
constexpr float kNegBig = -1.0e30f;

struct AttnParams {
  const __nv_bfloat16* q;        // [Tq, H, D] (EXACT: rows gathered through idx_q)
  const int32_t* idx_q;          // EXACT: salient query rows (Q space), grouped by sequence
  __nv_bfloat16* o_sal;          // EXACT: [num_salient, H, D] output
  const __nv_bfloat16* k;        // [Tk, Hkv, D]
  const __nv_bfloat16* v;        // [Tk, Hkv, D] delta-V (non-zero on salient key rows only)
  const __nv_bfloat16* c_old;    // [Tq, H, D], or the context cache arena when c_seq_starts is set
  __nv_bfloat16* c_cache;        // cache arena to update in place (same memory as c_old), or null
  const int64_t* c_seq_starts;   // first cache row of every sequence id; null = c_old is packed like Q
  const int64_t* c_seq_ids;      // [B] sequence id of every batch entry
  __nv_bfloat16* out;            // [Tq, H, D]
  float* partial;                // [H, Tq, 3] per-head statistics
  const int32_t* cu_q;           // [B + 1]
  const int32_t* cu_k;           // [B + 1]
  const int32_t* cu_sal;         // [B + 1] prefix counts of the salient key list
  const int32_t* idx_k;          // salient key rows (K space), ascending, grouped by sequence
  int H, Hkv, Tq, Tk, n_qtiles;
  float scale_log2;              // log2(e) / sqrt(D)
  int v_mn_major;                // 1: dV tile kept [keys][d] (MN-major operand); 0: transposed while gathering
  int v_compact;                 // 1: v holds one row per salient key, in list order; 0: v is [Tk, Hkv, D]
  unsigned long long* trace;     // optional [256][8] phase timestamps (ns) of the first 256 CTAs; null = off
  int* status_word;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

#define DYLLM_TRACE(slot)                                                  \
  do {                                                                     \
    if (p.trace && blockIdx.x < 256 && threadIdx.x == 64)                  \
      p.trace[blockIdx.x * 8 + (slot)] = global_ns();                      \
  } while (0)

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// EXACT = false: the delta attention described at the top of this file.
// EXACT = true: plain softmax attention of the salient query rows against the full K / V of their
// sequence, o_sal[i] = softmax(q[idx_q[i]] K^T / sqrt(D)) V: the query tile is gathered through idx_q,
// pass B walks over all key tiles (K and V tiles by TMA; V is used as loaded, as an MN-major operand)
// and the epilogue stores O / rowsum.
template <bool EXACT>
__global__ void __launch_bounds__(kAttnThreads, 2)
attention_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  const int q_tile = blockIdx.x % p.n_qtiles;
  const int h = (blockIdx.x / p.n_qtiles) % p.H;
  const int b = blockIdx.x / (p.n_qtiles * p.H);
  const int sal_begin = p.cu_sal[b];
  const int n_sal = p.cu_sal[b + 1] - sal_begin;
  const int q_begin = EXACT ? 0 : p.cu_q[b];
  const int q_end = EXACT ? n_sal : p.cu_q[b + 1];   // EXACT: rows are positions in the salient list
  const int q0 = q_begin + q_tile * kBQ;
  if (q0 >= q_end)
    return;
  const int k_begin = p.cu_k[b], k_end = p.cu_k[b + 1];
  const int len_k = k_end - k_begin;
  const int num_kt = (len_k + kBKeys - 1) / kBKeys;
  const int hk = h / (p.H / p.Hkv);
  const int num_st = EXACT ? num_kt : (n_sal + kBKeys - 1) / kBKeys;   // tiles of pass B
  // C_old row of query row r: r + c_delta (cache-resident context: the last len_q rows of the sequence)
  int64_t c_delta = 0;
  if (!EXACT && p.c_seq_starts)
    c_delta = p.c_seq_starts[p.c_seq_ids[b]] + (len_k - (q_end - q_begin)) - q_begin;
  const bool v_mn_major = EXACT ? true : (p.v_mn_major != 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;                      // Q tile
  uint8_t* kv_smem0 = smem + kTileBytes;       // K stage 0 / gathered Ksal, later P
  uint8_t* kv_smem1 = smem + 2 * kTileBytes;   // K stage 1 / gathered dV
  __shared__ uint64_t q_full, k_full[2], k_empty[2], s_full[2], s_empty[2], b_full, p_full, pv_done, a_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int s_src[128];        // source row of each gather slot (-1 = none)
  __shared__ float2 s_ml[2][128];   // (max, sum) of the two column halves of each query row
  __shared__ float4 s_st[128];      // statistics of the second half of each row

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, EXACT ? 256 : 1);
    mbar_init(&k_full[0], 1);
    mbar_init(&k_full[1], 1);
    mbar_init(&k_empty[0], 1);
    mbar_init(&k_empty[1], 1);
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&s_empty[0], 256);
    mbar_init(&s_empty[1], 256);
    mbar_init(&b_full, EXACT ? 1 : 256);
    mbar_init(&p_full, 256);
    mbar_init(&pv_done, 1);
    mbar_init(&a_done, 1);
    fence_mbar_init();
    if (!EXACT)
      tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    if (EXACT)
      tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kAttnTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s0 = tmem_slot;
  const uint32_t tmem_o = tmem_slot + 128;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer: Q once, K tiles
    if (!EXACT && lane == 0) {
      mbar_arrive_expect_tx(&q_full, kTileBytes);
      tma_load_2d(q_smem, &tmap_q, &q_full, h * kD, q0);
      tma_load_2d(q_smem + kHalfBytes, &tmap_q, &q_full, h * kD + 64, q0);
    }
    for (int kt = 0; kt < num_kt; ++kt) {
      const int s = kt & 1;
      mbar_wait(&k_empty[s], ((kt >> 1) & 1) ^ 1, &abort_flag, p.status_word, 301);
      if (lane == 0) {
        uint8_t* dst = s ? kv_smem1 : kv_smem0;
        mbar_arrive_expect_tx(&k_full[s], kTileBytes);
        tma_load_2d(dst, &tmap_k, &k_full[s], hk * kD, k_begin + kt * kBKeys);
        tma_load_2d(dst + kHalfBytes, &tmap_k, &k_full[s], hk * kD + 64, k_begin + kt * kBKeys);
      }
      __syncwarp();
    }
    if (EXACT) {
      // pass B: K tile into buffer 0 and V tile into buffer 1 once both are free
      for (int st = 0; st < num_st; ++st) {
        if (st == 0)
          mbar_wait(&a_done, 0, &abort_flag, p.status_word, 311);
        else
          mbar_wait(&pv_done, (st - 1) & 1, &abort_flag, p.status_word, 312);
        if (lane == 0) {
          mbar_arrive_expect_tx(&b_full, 2 * kTileBytes);
          tma_load_2d(kv_smem0, &tmap_k, &b_full, hk * kD, k_begin + st * kBKeys);
          tma_load_2d(kv_smem0 + kHalfBytes, &tmap_k, &b_full, hk * kD + 64, k_begin + st * kBKeys);
          tma_load_2d(kv_smem1, &tmap_v, &b_full, hk * kD, k_begin + st * kBKeys);
          tma_load_2d(kv_smem1 + kHalfBytes, &tmap_v, &b_full, hk * kD + 64, k_begin + st * kBKeys);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, v_mn_major ? 1 : 0);
    const uint32_t q_addr = smem_u32(q_smem);
    mbar_wait(&q_full, 0, &abort_flag, p.status_word, 302);
    int uses[2] = {0, 0};   // how often each S buffer has been handed to the softmax warps
    for (int t = 0; t < num_kt + num_st; ++t) {
      const bool sal_tile = t >= num_kt;
      const int st = t - num_kt;
      const int sb = sal_tile ? 0 : (t & 1);   // pass B keeps to buffer 0: buffer 1 holds O then
      const int use = uses[sb]++;
      const uint32_t tmem_s = tmem_s0 + sb * 128;
      uint32_t kb_addr;
      if (!sal_tile) {
        const int s = t & 1;
        mbar_wait(&k_full[s], (t >> 1) & 1, &abort_flag, p.status_word, 303);
        kb_addr = smem_u32(s ? kv_smem1 : kv_smem0);
      } else {
        mbar_wait(&b_full, st & 1, &abort_flag, p.status_word, 304);
        kb_addr = smem_u32(kv_smem0);
      }
      mbar_wait(&s_empty[sb], (use & 1) ^ 1, &abort_flag, p.status_word, 305);
      tc_fence_after_sync();
      if (lane == 0) {
        // S = Q K^T: contraction over d in two swizzled halves of 64, four K = 16 steps each
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint64_t a_desc = umma_smem_desc_sw128(q_addr + half * kHalfBytes, 16, 1024);
          const uint64_t b_desc = umma_smem_desc_sw128(kb_addr + half * kHalfBytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem_s, a_desc + 2 * kk, b_desc + 2 * kk, idesc_qk, (half | kk) != 0 ? 1u : 0u);
        }
        if (!sal_tile)
          umma_commit(&k_empty[t & 1]);
        umma_commit(&s_full[sb]);
        if (EXACT && t == num_kt - 1)
          umma_commit(&a_done);
      }
      __syncwarp();
      if (sal_tile) {
        // O += P dV over the 128 (zero padded) salient keys of this tile
        mbar_wait(&p_full, st & 1, &abort_flag, p.status_word, 306);
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t p_addr = smem_u32(kv_smem0);
          const uint32_t v_addr = smem_u32(kv_smem1);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a_desc =
                umma_smem_desc_sw128(p_addr + (kk >> 2) * kHalfBytes + (kk & 3) * 32, 16, 1024);
            uint64_t b_desc;
            if (v_mn_major)  // [keys][d]: 16 keys = 2048 bytes per step, d halves 16 KB apart
              b_desc = umma_smem_desc_sw128(v_addr + kk * 2048, kHalfBytes, 1024);
            else               // [d][keys]: key halves 16 KB apart, 32 bytes per step inside a half
              b_desc = umma_smem_desc_sw128(v_addr + (kk >> 2) * kHalfBytes + (kk & 3) * 32, 16, 1024);
            umma_ss(tmem_o, a_desc, b_desc, idesc_pv, (st | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&pv_done);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / gather / epilogue
    // Eight warps: two warps share each tensor-memory lane quarter (= 32 query rows) and split the
    // columns of every tile in halves, so a thread owns one query row and 64 of 128 columns.
    const int sw = warp - 2;                 // 0..7
    const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
    const int half = sw >> 2;                // which 64 columns of a tile / of the head dimension
    const int row = qd * 32 + lane;          // query row inside the tile
    const int st_tid = sw * 32 + lane;       // 0..255 among the softmax threads
    const uint32_t t_lane = static_cast<uint32_t>(qd * 32) << 16;
    const int col0 = half * 64;
    const float c = p.scale_log2;
    float m = kNegBig, l = 0.f;
    DYLLM_TRACE(0);

    if (!EXACT && q0 + row < q_end) {
      // bring this thread's half of the C_old row (128 bytes) into L2 now; the epilogue reads it much later
      const char* crow =
          reinterpret_cast<const char*>(p.c_old + ((q0 + row + c_delta) * p.H + h) * kD + col0);
      asm volatile("prefetch.global.L2 [%0];" ::"l"(crow));
    }
    // source rows of the first gather (salient key rows, or the query rows of the EXACT variant)
    if (half == 0) {
      int src = -1;
      if (EXACT) {
        if (q0 + row < q_end)
          src = p.idx_q[sal_begin + q0 + row];
      } else if (row < n_sal) {
        src = p.idx_k[sal_begin + row];
      }
      s_src[row] = src;
    }
    if (EXACT) {
      // cooperative gather of the query rows (zeros past the list) into the swizzled Q tile
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int item = it * 256 + st_tid;
        const int r = item >> 4, ch = item & 15;
        const int src = s_src[r];
        const uint4 qv = src >= 0
            ? __ldg(reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(src) * p.H + h) * kD) + ch) : zero;
        *reinterpret_cast<uint4*>(q_smem + (ch >> 3) * kHalfBytes + sw128_offset(r, ch & 7)) = qv;
      }
      fence_proxy_async_smem();
      mbar_arrive(&q_full);
    }

    // pass A: running maximum and sum over this thread's half of the columns of every key tile
    int uses[2] = {0, 0};
    for (int kt = 0; kt < num_kt; ++kt) {
      const int sb = kt & 1;
      const int use = uses[sb]++;
      const uint32_t tmem_s = tmem_s0 + sb * 128;
      mbar_wait(&s_full[sb], use & 1, &abort_flag, p.status_word, 307);
      tc_fence_after_sync();
      if (kt == 0)
        DYLLM_TRACE(7);
      const int valid = len_k - kt * kBKeys;   // keys of this tile that belong to the sequence
#pragma unroll 1
      for (int cc = 0; cc < 64; cc += 32) {
        const int c0 = col0 + cc;
        uint32_t sr[32];
        tmem_ld_32x32(tmem_s + t_lane + c0, sr);
        tmem_ld_wait();
        if (cc == 32) {  // last chunk read: the MMA warp may overwrite this S buffer
          tc_fence_before_sync();
          mbar_arrive(&s_empty[sb]);
        }
        float cmax = kNegBig;
        if (valid >= kBKeys) {   // whole tile inside the sequence: no masking
#pragma unroll
          for (int i = 0; i < 32; ++i)
            cmax = fmaxf(cmax, __uint_as_float(sr[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float s = __uint_as_float(sr[i]);
            s = (c0 + i < valid) ? s : kNegBig;
            sr[i] = __float_as_uint(s);
            cmax = fmaxf(cmax, s);
          }
        }
        const float m_new = fmaxf(m, cmax);
        const float mc = m_new * c;
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          sum += ex2(fmaf(__uint_as_float(sr[i]), c, -mc));
        l = l * ex2((m - m_new) * c) + sum;
        m = m_new;
      }
    }
    // merge the two column halves of each row: m = max, l rescaled to the common maximum
    s_ml[half][row] = make_float2(m, l);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
      const float2 other = s_ml[half ^ 1][row];
      const float m_all = fmaxf(m, other.x);
      l = l * ex2((m - m_all) * c) + other.y * ex2((other.x - m_all) * c);
      m = m_all;
    }

    // pass B: salient keys (EXACT: all keys again, with their values)
    DYLLM_TRACE(1);
    const float mc = m * c;
    for (int st = 0; st < num_st; ++st) {
      // The buffers are free for tile 0 once the last Q K^T product is complete: s_full of the last
      // key tile was observed above and is committed after every earlier MMA.  Later tiles wait for the
      // previous P dV product.
      if (!EXACT && st > 0) {
        mbar_wait(&pv_done, (st - 1) & 1, &abort_flag, p.status_word, 308);
        if (half == 0) {
          const int j = st * kBKeys + row;
          s_src[row] = j < n_sal ? p.idx_k[sal_begin + j] : -1;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      const int n_tile = min(kBKeys, (EXACT ? len_k : n_sal) - st * kBKeys);
      if (!EXACT) {
        // cooperative gather: 128 slots x 16 chunks of the K rows and of the dV rows, zeros past the list
        const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int item = it * 256 + st_tid;
          const int r = item >> 4, ch = item & 15;
          const int src = s_src[r];
          const bool have = src >= 0;
          const uint4 kv = have
              ? __ldg(reinterpret_cast<const uint4*>(p.k + (static_cast<int64_t>(src) * p.Hkv + hk) * kD) + ch) : zero;
          *reinterpret_cast<uint4*>(kv_smem0 + (ch >> 3) * kHalfBytes + sw128_offset(r, ch & 7)) = kv;
          const int64_t vrow = p.v_compact ? static_cast<int64_t>(sal_begin + st * kBKeys + r) : src;
          const uint4 vv = have
              ? __ldg(reinterpret_cast<const uint4*>(p.v + (vrow * p.Hkv + hk) * kD) + ch) : zero;
          if (v_mn_major) {
            *reinterpret_cast<uint4*>(kv_smem1 + (ch >> 3) * kHalfBytes + sw128_offset(r, ch & 7)) = vv;
          } else {
            // transposed tile [d][key]: element (d, key = r)
            uint8_t* base = kv_smem1 + (r >> 6) * kHalfBytes + ((r & 7) << 1);
            const uint32_t key_chunk = (r & 63) >> 3;
            const uint16_t* e = reinterpret_cast<const uint16_t*>(&vv);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t d = ch * 8 + i;
              *reinterpret_cast<uint16_t*>(base + d * 128u + ((key_chunk ^ (d & 7u)) << 4)) = e[i];
            }
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&b_full);
      }
      // P = exp2(S2 * c - m * c) for the live columns of this thread's half
      DYLLM_TRACE(2);
      const int use = uses[0]++;
      mbar_wait(&s_full[0], use & 1, &abort_flag, p.status_word, 309);
      tc_fence_after_sync();
      DYLLM_TRACE(3);
#pragma unroll 1
      for (int cc = 0; cc < 64; cc += 32) {
        const int c0 = col0 + cc;
        uint32_t sr[32];
        tmem_ld_32x32(tmem_s0 + t_lane + c0, sr);
        tmem_ld_wait();
        if (cc == 32) {
          tc_fence_before_sync();
          mbar_arrive(&s_empty[0]);
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = (c0 + 2 * i < n_tile) ? ex2(fmaf(__uint_as_float(sr[2 * i]), c, -mc)) : 0.f;
          const float p1 = (c0 + 2 * i + 1 < n_tile) ? ex2(fmaf(__uint_as_float(sr[2 * i + 1]), c, -mc)) : 0.f;
          __nv_bfloat162 v2 = __floats2bfloat162_rn(p0, p1);
          pk[i] = *reinterpret_cast<uint32_t*>(&v2);
        }
        uint8_t* pdst = kv_smem0 + (c0 >> 6) * kHalfBytes;
        const uint32_t chunk0 = (c0 & 63) >> 3;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(pdst + sw128_offset(row, chunk0 + j)) =
              make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&p_full);
      DYLLM_TRACE(4);
    }
    if (num_st > 0) {
      mbar_wait(&pv_done, (num_st - 1) & 1, &abort_flag, p.status_word, 310);
      tc_fence_after_sync();
    }
    DYLLM_TRACE(5);

    // epilogue: new = old + O / rowsum for this thread's 64 of the 128 head dimensions; bf16 store;
    // partial statistics of this head.  The tensor-memory loads are warp-collective, so every lane issues
    // them; only the global-memory traffic is predicated on the row being inside the sequence.
    const int r = q0 + row;
    const bool live = r < q_end;
    const float inv_l = l > 0.f ? 1.0f / l : 0.f;
    const int64_t off = (static_cast<int64_t>((live ? r : q0) + (EXACT ? sal_begin : 0)) * p.H + h) * kD + col0;
    const int64_t c_off = (((live ? r : q0) + c_delta) * p.H + h) * kD + col0;
    const __nv_bfloat16* cold = EXACT ? nullptr : p.c_old + c_off;
    __nv_bfloat16* dst = (EXACT ? p.o_sal : p.out) + off;
    // in-place cache update: salient rows are left alone (their old value is still needed, and they are
    // overwritten with the exactly attended row afterwards)
    __nv_bfloat16* cdst = nullptr;
    if (!EXACT && p.c_cache && live) {
      int lo = 0, hi = n_sal;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (p.idx_q[sal_begin + mid] < r)
          lo = mid + 1;
        else
          hi = mid;
      }
      if (!(lo < n_sal && p.idx_q[sal_begin + lo] == r))
        cdst = p.c_cache + c_off;
    }
    float dot = 0.f, nn = 0.f, no = 0.f;
    uint4 old_row[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      old_row[j] = (EXACT || !live) ? make_uint4(0, 0, 0, 0) : __ldg(reinterpret_cast<const uint4*>(cold) + j);
#pragma unroll
    for (int cc = 0; cc < 64; cc += 32) {
      uint32_t orr[32];
      if (num_st > 0) {
        tmem_ld_32x32(tmem_o + t_lane + col0 + cc, orr);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          orr[i] = 0u;
      }
      if (live) {
        const uint4* oldv = old_row + cc / 8;
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(oldv);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 of = __bfloat1622float2(o2[i]);
          const float n0 = of.x + __uint_as_float(orr[2 * i]) * inv_l;
          const float n1 = of.y + __uint_as_float(orr[2 * i + 1]) * inv_l;
          dot = fmaf(n0, of.x, dot);
          dot = fmaf(n1, of.y, dot);
          nn = fmaf(n0, n0, nn);
          nn = fmaf(n1, n1, nn);
          no = fmaf(of.x, of.x, no);
          no = fmaf(of.y, of.y, no);
          __nv_bfloat162 v2 = __floats2bfloat162_rn(n0, n1);
          pk[i] = *reinterpret_cast<uint32_t*>(&v2);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          reinterpret_cast<uint4*>(dst + cc)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        if (cdst) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(cdst + cc)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
      }
    }
    if (!EXACT) {
      // the two halves of a row add their statistics in a fixed order (half 0 + half 1)
      if (half == 1)
        s_st[row] = make_float4(dot, nn, no, 0.f);
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0 && live) {
        const float4 o = s_st[row];
        float* ps = p.partial + (static_cast<int64_t>(h) * p.Tq + r) * 3;
        ps[0] = dot + o.x;
        ps[1] = nn + o.y;
        ps[2] = no + o.z;
      }
    }
    DYLLM_TRACE(6);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_slot, kAttnTmemCols);
  }
}

// ----------------------------------------------------------------------------------------------
// finalize: head-ordered reduction of the partial statistics + mask (part A, one thread per row);
// salient rows take the exactly attended values and statistics recomputed from bf16 (part B, one
// block per salient row).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ bool mask_rule(float dot, float a, float b, float threshold) {
  return dot * rsqrtf(fmaxf(a, 1e-8f)) * rsqrtf(fmaxf(b, 1e-8f)) < threshold;
}

__global__ void __launch_bounds__(256)
attention_finalize_kernel(const float* __restrict__ partial, int H, int Tq, const int32_t* __restrict__ idx_q,
                          int num_salient, const __nv_bfloat16* __restrict__ c_old,
                          const __nv_bfloat16* __restrict__ o_sal, __nv_bfloat16* __restrict__ out,
                          float* __restrict__ stats, uint8_t* __restrict__ mask, float threshold, int width,
                          int row_blocks, const int32_t* __restrict__ num_salient_dev,
                          __nv_bfloat16* __restrict__ c_cache, const int64_t* __restrict__ c_seq_starts,
                          const int64_t* __restrict__ c_seq_ids, const int32_t* __restrict__ cu_q,
                          const int32_t* __restrict__ cu_k, int batch) {
  if (num_salient_dev)
    num_salient = min(num_salient, *num_salient_dev);
  if (static_cast<int>(blockIdx.x) < row_blocks) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= Tq)
      return;
    // salient rows are written by part B
    int lo = 0, hi = num_salient;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (idx_q[mid] < r)
        lo = mid + 1;
      else
        hi = mid;
    }
    if (lo < num_salient && idx_q[lo] == r)
      return;
    float s0 = stats[r * 3 + 0], s1 = stats[r * 3 + 1], s2 = stats[r * 3 + 2];
    for (int h = 0; h < H; ++h) {
      const float* ps = partial + (static_cast<int64_t>(h) * Tq + r) * 3;
      s0 += ps[0];
      s1 += ps[1];
      s2 += ps[2];
    }
    stats[r * 3 + 0] = s0;
    stats[r * 3 + 1] = s1;
    stats[r * 3 + 2] = s2;
    mask[r] = mask_rule(s0, s1, s2, threshold) ? 1 : 0;
    return;
  }
  const int i = blockIdx.x - row_blocks;
  if (i >= num_salient)
    return;
  const int r = idx_q[i];
  int64_t c_row = r;
  if (c_seq_starts) {
    // sequence b with cu_q[b] <= r < cu_q[b + 1]; its context rows are the last len_q rows in the cache
    int lo = 0, hi = batch;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (cu_q[mid + 1] <= r)
        lo = mid + 1;
      else
        hi = mid;
    }
    const int b = lo < batch ? lo : batch - 1;
    c_row = c_seq_starts[c_seq_ids[b]] + ((cu_k[b + 1] - cu_k[b]) - (cu_q[b + 1] - cu_q[b])) + (r - cu_q[b]);
  }
  const uint4* old_row = reinterpret_cast<const uint4*>(c_old + c_row * width);
  const uint4* new_row = reinterpret_cast<const uint4*>(o_sal + static_cast<int64_t>(i) * width);
  uint4* out_row = reinterpret_cast<uint4*>(out + static_cast<int64_t>(r) * width);
  uint4* cache_row = c_cache ? reinterpret_cast<uint4*>(c_cache + c_row * width) : nullptr;
  float dot = 0.f, nn = 0.f, no = 0.f;
  for (int v = threadIdx.x; v < width / 8; v += blockDim.x) {
    const uint4 ov = old_row[v];
    const uint4 nv = __ldg(new_row + v);
    out_row[v] = nv;
    if (cache_row)
      cache_row[v] = nv;
    const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
    const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 of = __bfloat1622float2(o2[j]);
      const float2 nf = __bfloat1622float2(n2[j]);
      dot = fmaf(nf.x, of.x, dot);
      dot = fmaf(nf.y, of.y, dot);
      nn = fmaf(nf.x, nf.x, nn);
      nn = fmaf(nf.y, nf.y, nn);
      no = fmaf(of.x, of.x, no);
      no = fmaf(of.y, of.y, no);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    dot += __shfl_xor_sync(0xffffffffu, dot, off);
    nn += __shfl_xor_sync(0xffffffffu, nn, off);
    no += __shfl_xor_sync(0xffffffffu, no, off);
  }
  __shared__ float red[8][3];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red[warp][0] = dot;
    red[warp][1] = nn;
    red[warp][2] = no;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, bsum = 0.f, cs = 0.f;
    for (int w = 0; w < 8; ++w) {
      a += red[w][0];
      bsum += red[w][1];
      cs += red[w][2];
    }
    stats[r * 3 + 0] = a;
    stats[r * 3 + 1] = bsum;
    stats[r * 3 + 2] = cs;
    mask[r] = mask_rule(a, bsum, cs, threshold) ? 1 : 0;
  }
}

bool g_attn_smem_set[2][64] = {{false}, {false}};
unsigned long long* g_attn_trace = nullptr;

template <bool EXACT>
int launch_attention(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                     int64_t blocks, cudaStream_t s) {
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev < 0 || dev >= 64) ? 0 : dev;
  if (!g_attn_smem_set[EXACT ? 1 : 0][dev]) {
    if (cudaFuncSetAttribute(attention_kernel<EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kAttnSmem)) != cudaSuccess)
      return set_error(DYLLM_ERR_CUDA, "attention: cudaFuncSetAttribute failed: %s",
                       cudaGetErrorString(cudaGetLastError()));
    g_attn_smem_set[EXACT ? 1 : 0][dev] = true;
  }
  DYLLM_REQUIRE(blocks > 0 && blocks < (1ll << 31), DYLLM_ERR_UNSUPPORTED, "attention: grid of %lld blocks",
                static_cast<long long>(blocks));
  attention_kernel<EXACT><<<static_cast<unsigned>(blocks), kAttnThreads, kAttnSmem, s>>>(tq, tk, tv, p);
  return check_launch(EXACT ? "salient_attention" : "delta_attention");
}

}  // namespace
}  // namespace dyllm

using namespace dyllm;

extern "C" {

size_t dyllm_attention_sparse_workspace_bytes(int total_q, int num_heads) {
  if (total_q <= 0 || num_heads <= 0)
    return 0;
  return static_cast<size_t>(total_q) * num_heads * 3 * sizeof(float);
}

int dyllm_attention_sparse_varlen(const void* q, const void* k, const void* v, const void* c, const void* o_sal,
                                  void* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                                  int max_seqlen_q, int max_seqlen_k, int total_q, int total_k, int num_heads,
                                  int num_kv_heads, int head_dim, const int32_t* cu_salientlens,
                                  const int32_t* idx_salient_row_q, const int32_t* idx_salient_row_k,
                                  int num_salient, const int32_t* num_salient_dev, float* cosine_stats,
                                  uint8_t* cosine_out, float threshold, void* workspace, size_t workspace_bytes,
                                  int v_layout, const int64_t* c_seq_starts, const int64_t* c_seq_ids,
                                  int c_update_in_place, void* stream) {
  const int v_mn_major = (v_layout & 1) ? 1 : 0;
  const int v_compact = (v_layout & 2) ? 1 : 0;
  DYLLM_REQUIRE(head_dim == 128, DYLLM_ERR_UNSUPPORTED, "attention_sparse_varlen: head_dim %d (only 128 is built)",
                head_dim);
  DYLLM_REQUIRE(batch > 0 && total_q > 0 && total_k > 0, DYLLM_ERR_INVALID_ARGUMENT,
                "attention_sparse_varlen: Q and K/V token dimensions must be non-empty (batch %d, Tq %d, Tk %d)", batch,
                total_q, total_k);
  DYLLM_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "attention_sparse_varlen: local query heads (%d) must be a positive multiple of local KV heads (%d)",
                num_heads, num_kv_heads);
  DYLLM_REQUIRE(max_seqlen_q > 0 && max_seqlen_q <= total_q && max_seqlen_k > 0 && max_seqlen_k <= total_k,
                DYLLM_ERR_INVALID_ARGUMENT, "attention_sparse_varlen: maximum sequence lengths must be positive and fit");
  DYLLM_REQUIRE(num_salient >= 0 && num_salient <= total_q && num_salient <= total_k, DYLLM_ERR_INVALID_ARGUMENT,
                "attention_sparse_varlen: salient index count %d out of range", num_salient);
  DYLLM_REQUIRE(q && k && c && out && cu_seqlens_q && cu_seqlens_k && cu_salientlens && cosine_stats &&
                    cosine_out && workspace,
                DYLLM_ERR_INVALID_ARGUMENT, "attention_sparse_varlen: null pointer");
  DYLLM_REQUIRE(num_salient == 0 || (v && o_sal && idx_salient_row_q && idx_salient_row_k), DYLLM_ERR_INVALID_ARGUMENT,
                "attention_sparse_varlen: salient rows without delta-V / o_sal / index lists");
  DYLLM_REQUIRE(workspace_bytes >= dyllm_attention_sparse_workspace_bytes(total_q, num_heads), DYLLM_ERR_WORKSPACE,
                "attention_sparse_varlen: workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
                dyllm_attention_sparse_workspace_bytes(total_q, num_heads));
  for (const void* ptr16 : {q, k, v, c, o_sal, static_cast<const void*>(out)})
    DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(ptr16) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT,
                  "attention_sparse_varlen: tensors must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  CUtensorMap tq, tk;
  int rc = encode_tmap_2d_bf16(&tq, q, total_q, static_cast<uint64_t>(num_heads) * kD,
                               static_cast<uint64_t>(num_heads) * kD, kBQ, 64, true);
  if (rc != DYLLM_OK)
    return rc;
  rc = encode_tmap_2d_bf16(&tk, k, total_k, static_cast<uint64_t>(num_kv_heads) * kD,
                           static_cast<uint64_t>(num_kv_heads) * kD, kBKeys, 64, true);
  if (rc != DYLLM_OK)
    return rc;

  AttnParams p = {};
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  DYLLM_REQUIRE((c_seq_starts == nullptr) == (c_seq_ids == nullptr) && (!c_update_in_place || c_seq_starts),
                DYLLM_ERR_INVALID_ARGUMENT,
                "attention_sparse_varlen: a cache-resident context needs c_seq_starts and c_seq_ids");
  p.c_old = static_cast<const __nv_bfloat16*>(c);
  p.c_cache = c_update_in_place ? const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(c)) : nullptr;
  p.c_seq_starts = c_seq_starts;
  p.c_seq_ids = c_seq_ids;
  p.idx_q = idx_salient_row_q;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.partial = static_cast<float*>(workspace);
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.cu_sal = cu_salientlens;
  p.idx_k = idx_salient_row_k;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  p.Tq = total_q;
  p.Tk = total_k;
  p.n_qtiles = cdiv_i(max_seqlen_q, kBQ);
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(kD));
  p.v_mn_major = v_mn_major;
  p.v_compact = v_compact;
  p.trace = g_attn_trace;
  p.status_word = device_status_word();
  const int64_t blocks = static_cast<int64_t>(batch) * num_heads * p.n_qtiles;
  rc = launch_attention<false>(tq, tk, tk, p, blocks, s);
  if (rc != DYLLM_OK)
    return rc;

  const int row_blocks = cdiv_i(total_q, 256);
  attention_finalize_kernel<<<row_blocks + num_salient, 256, 0, s>>>(
      p.partial, num_heads, total_q, idx_salient_row_q, num_salient, p.c_old,
      static_cast<const __nv_bfloat16*>(o_sal), p.out, cosine_stats, cosine_out, threshold, num_heads * kD, row_blocks,
      num_salient_dev, p.c_cache, c_seq_starts, c_seq_ids, cu_seqlens_q, cu_seqlens_k, batch);
  return check_launch("attention_finalize");
}

int dyllm_attention_salient_rows(const void* q, const void* k, const void* v, void* o_sal,
                                 const int32_t* cu_seqlens_k, int batch, int max_rows_per_seq, int total_q,
                                 int total_k, int num_heads, int num_kv_heads, int head_dim,
                                 const int32_t* cu_salientlens, const int32_t* idx_salient_row_q, void* stream) {
  DYLLM_REQUIRE(head_dim == 128, DYLLM_ERR_UNSUPPORTED, "attention_salient_rows: head_dim %d (only 128 is built)",
                head_dim);
  DYLLM_REQUIRE(batch > 0 && total_q > 0 && total_k > 0 && max_rows_per_seq >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "attention_salient_rows: batch %d Tq %d Tk %d max rows %d", batch, total_q, total_k, max_rows_per_seq);
  DYLLM_REQUIRE(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "attention_salient_rows: query heads (%d) must be a positive multiple of KV heads (%d)", num_heads,
                num_kv_heads);
  if (max_rows_per_seq == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(q && k && v && o_sal && cu_seqlens_k && cu_salientlens && idx_salient_row_q,
                DYLLM_ERR_INVALID_ARGUMENT, "attention_salient_rows: null pointer");
  for (const void* ptr16 : {q, k, v, static_cast<const void*>(o_sal)})
    DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(ptr16) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT,
                  "attention_salient_rows: tensors must be 16-byte aligned");
  CUtensorMap tk, tv;
  int rc = encode_tmap_2d_bf16(&tk, k, total_k, static_cast<uint64_t>(num_kv_heads) * kD,
                               static_cast<uint64_t>(num_kv_heads) * kD, kBKeys, 64, true);
  if (rc != DYLLM_OK)
    return rc;
  rc = encode_tmap_2d_bf16(&tv, v, total_k, static_cast<uint64_t>(num_kv_heads) * kD,
                           static_cast<uint64_t>(num_kv_heads) * kD, kBKeys, 64, true);
  if (rc != DYLLM_OK)
    return rc;
  AttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.idx_q = idx_salient_row_q;
  p.o_sal = static_cast<__nv_bfloat16*>(o_sal);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.cu_q = cu_salientlens;
  p.cu_k = cu_seqlens_k;
  p.cu_sal = cu_salientlens;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  p.Tq = total_q;
  p.Tk = total_k;
  p.n_qtiles = cdiv_i(max_rows_per_seq, kBQ);
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(kD));
  p.v_mn_major = 1;
  p.status_word = device_status_word();
  const int64_t blocks = static_cast<int64_t>(batch) * num_heads * p.n_qtiles;
  return launch_attention<true>(tk, tk, tv, p, blocks, static_cast<cudaStream_t>(stream));
}

int dyllm_attention_trace(void* device_buffer) {
  g_attn_trace = static_cast<unsigned long long*>(device_buffer);
  return DYLLM_OK;
}

int dyllm_attention_kernel_info(int dim, int64_t* info10) {
  DYLLM_REQUIRE(info10, DYLLM_ERR_INVALID_ARGUMENT, "attention_kernel_info: null output");
  DYLLM_REQUIRE(dim == 128, DYLLM_ERR_UNSUPPORTED, "attention_kernel_info: head_dim %d (only 128 is built)", dim);
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, attention_kernel<false>) != cudaSuccess)
    return set_error(DYLLM_ERR_CUDA, "attention_kernel_info: %s", cudaGetErrorString(cudaGetLastError()));
  int blocks_per_sm = 0;
  cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(kAttnSmem));
  const bool ok = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, attention_kernel<false>, kAttnThreads,
                                                                kAttnSmem) == cudaSuccess;
  info10[0] = attr.numRegs;
  info10[1] = static_cast<int64_t>(attr.localSizeBytes);
  info10[2] = static_cast<int64_t>(attr.sharedSizeBytes);
  info10[3] = kAttnSmem;
  info10[4] = kAttnThreads;
  info10[5] = blocks_per_sm;
  info10[6] = kBQ;
  info10[7] = kBKeys;
  info10[8] = 1;
  info10[9] = ok ? 1 : 0;
  return DYLLM_OK;
}

}  // extern "C"
