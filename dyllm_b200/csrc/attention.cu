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
// Salient query rows take the exactly attended row (o_sal) as their new value in the same epilogue.
// A second small kernel adds the per-head partials in head order (run-to-run identical results) and
// writes the threshold mask.
//
// One CTA = (sequence, query head, 128 query rows); 10 warps: TMA producer, MMA issuer, 8 softmax warps
// (two per 32-row lane quarter, each taking half of the columns).  104 KB of shared memory and 256
// tensor-memory columns per CTA, so two CTAs share an SM and one CTA's tensor-core work overlaps the
// other's exponentials.
//
// Pass B works on the salient keys rounded up to a multiple of 16 (the MMA shapes are chosen at run
// time).  With at most 16 salient keys in the sequence (the common case) their K and dV rows are requested
// at the start of the item and land in a small dedicated buffer right after pass A, so pass B starts as
// soon as pass A ends and nothing of the item's set-up delays the first logits.  The new context tile of a
// full tile is stored (TMA) by the otherwise idle producer warp once the softmax threads have written it.
#include "common.cuh"

namespace dyllm {

namespace {

constexpr int kD = 128;          // head dimension
constexpr int kBQ = 128;         // query rows per CTA
constexpr int kBKeys = 128;      // keys per tile
constexpr int kAttnThreads = 320;          // TMA producer warp, MMA warp, eight softmax warps
constexpr uint32_t kTileBytes = 128 * 128 * 2;   // one [128][128] bf16 tile = two [128][64] swizzled halves
constexpr uint32_t kHalfBytes = 128 * 64 * 2;
constexpr int kFastSal = 16;                      // salient keys served by the early gather
constexpr int kSmallRows = 16;                    // salient query rows per sequence served by salient_rows_small_kernel
constexpr int kSmallMaxTiles = 15;                // ... 15 * 16 columns of S^T + 16 of O^T = 256 tensor-memory columns
constexpr uint32_t kSalHalfBytes = kFastSal * 128;   // one 64-column half of a 16-row tile
constexpr uint32_t kSalBytes = 2 * kSalHalfBytes;
constexpr uint32_t kAttnSmem = 3 * kTileBytes + 2 * kSalBytes + 1024;
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
  int H, Hkv, Tq, Tk, n_qtiles, batch, num_items;
  int skip_small;                // EXACT: sequences with few salient rows are left to salient_rows_small_kernel
  float scale_log2;              // log2(e) / sqrt(D)
  int v_mn_major;                // 1: dV tile kept [keys][d] (MN-major operand); 0: transposed while gathering
  int v_compact;                 // 1: v holds one row per salient key, in list order; 0: v is [Tk, Hkv, D]
  unsigned long long* trace;     // optional [1024][16] phase timestamps (ns) of 1024 CTAs from trace_first on; null = off
  unsigned trace_first;
  int* status_word;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Phase tracer (development aid): compiled in only with -DDYLLM_ATTN_TRACE, which also exports
// dyllm_attention_trace(buffer) to register a device buffer of 1024 * 16 uint64 time stamps.
#ifdef DYLLM_ATTN_TRACE
#define DYLLM_TRACE(slot)                                                  \
  do {                                                                     \
    if (p.trace && item >= static_cast<int>(p.trace_first) && item < static_cast<int>(p.trace_first) + 1024 && \
        threadIdx.x == 64)                                                 \
      p.trace[(item - p.trace_first) * 16 + (slot)] = global_ns();         \
  } while (0)
#else
#define DYLLM_TRACE(slot) do { } while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two-wide fp32 arithmetic (one instruction per pair) and a three-input maximum: the softmax warps are
// bound by instruction issue and by the exponential unit, not by arithmetic throughput.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
      " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n"
      " add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// (2^x0, 2^x1) through the two-wide half-precision exponential: one pass of the exponential unit for
// two values.  Used for the row sums of pass A only (arguments <= 0; the relative error of a term is
// below 3e-3 and far smaller for the terms near the maximum that dominate the sum); the probabilities
// that enter the P dV product are computed in fp32.
__device__ __forceinline__ float2 ex2_pair_f16(float x0, float x1) {
  uint32_t h;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(x1), "f"(x0));
  asm("ex2.approx.f16x2 %0, %0;" : "+r"(h));
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

constexpr bool kPassAHalfExp = false;   // measured: no faster than fp32 exponentials here

// Sequences whose salient query rows are handled by salient_rows_small_kernel.
__device__ __forceinline__ bool small_rows_item(int n_sal, int num_kt) {
  return n_sal > 0 && n_sal <= kSmallRows && num_kt <= kSmallMaxTiles;
}

// One unit of work: (sequence, query head, tile of 128 query rows).
struct AttnItem {
  int h, hk, sal_begin, n_sal, q_end, q0, k_begin, len_k, num_kt, num_st;
  int k_shift;       // K row of a query row listed in idx_q when no K-space list is given: idx_q[i] + k_shift
  int64_t c_delta;   // C_old row of query row r: r + c_delta (cache-resident context)
  bool tile_tma;     // the tile lies completely inside the sequence: context through shared memory
  bool fast;         // at most kFastSal salient keys: gathered early into their own buffers
};

// Decodes work item `item`; false when it holds no query rows.  The delta kernel orders items
// (sequence, head, tile) so that the tiles of one head run at the same time and share its keys in L2;
// the EXACT kernel puts the tile index first, because most sequences fill only their first tile and
// items are dealt out to CTAs round-robin.
template <bool EXACT>
__device__ __forceinline__ bool decode_item(const AttnParams& p, int item, AttnItem& it) {
  int q_tile, b;
  if (EXACT) {
    const int bh = p.batch * p.H;
    q_tile = item / bh;
    it.h = item % p.H;
    b = (item % bh) / p.H;
  } else {
    q_tile = item % p.n_qtiles;
    it.h = (item / p.n_qtiles) % p.H;
    b = item / (p.n_qtiles * p.H);
  }
  it.sal_begin = p.cu_sal[b];
  it.n_sal = p.cu_sal[b + 1] - it.sal_begin;
  const int q_begin = EXACT ? 0 : p.cu_q[b];
  it.q_end = EXACT ? it.n_sal : p.cu_q[b + 1];   // EXACT: rows are positions in the salient list
  it.q0 = q_begin + q_tile * kBQ;
  if (it.q0 >= it.q_end)
    return false;
  it.k_begin = p.cu_k[b];
  it.len_k = p.cu_k[b + 1] - it.k_begin;
  it.num_kt = (it.len_k + kBKeys - 1) / kBKeys;
  if (EXACT && p.skip_small && small_rows_item(it.n_sal, it.num_kt))
    return false;   // salient_rows_small_kernel takes this sequence
  it.hk = it.h / (p.H / p.Hkv);
  it.num_st = EXACT ? it.num_kt : (it.n_sal + kBKeys - 1) / kBKeys;   // tiles of pass B
  // the queries of a sequence are its last len_q rows
  it.k_shift = EXACT ? 0 : it.k_begin + it.len_k - (it.q_end - q_begin) - q_begin;
  it.c_delta = 0;
  if (!EXACT && p.c_seq_starts)
    it.c_delta = p.c_seq_starts[p.c_seq_ids[b]] + (it.len_k - (it.q_end - q_begin)) - q_begin;
  it.tile_tma = !EXACT && it.q0 + kBQ <= it.q_end;
  it.fast = !EXACT && p.v_mn_major != 0 && it.n_sal > 0 && it.n_sal <= kFastSal;
  return true;
}

#include "attention_pair.cuh"

// EXACT = false: the delta attention described at the top of this file.
// EXACT = true: plain softmax attention of the salient query rows against the full K / V of their
// sequence, o_sal[i] = softmax(q[idx_q[i]] K^T / sqrt(D)) V: the query tile is gathered through idx_q,
// pass B walks over all key tiles (K and V tiles by TMA; V is used as loaded, as an MN-major operand)
// and the epilogue stores O / rowsum.
//
// The kernel is persistent: the grid holds as many CTAs as the device runs at once and CTA i takes the
// work items i, i + gridDim.x, ...  Tensor memory and the barriers live for the whole kernel; every
// role counts how often it has used each barrier to know the phase it waits for.
template <bool EXACT>
__global__ void __launch_bounds__(kAttnThreads, 2)
attention_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_out,
                 const __grid_constant__ CUtensorMap tmap_c, const AttnParams p) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;                      // Q tile
  uint8_t* kv_smem0 = smem + kTileBytes;       // K stage 0 / gathered Ksal, later P
  uint8_t* kv_smem1 = smem + 2 * kTileBytes;   // K stage 1 / gathered dV, later the context tile
  uint8_t* ks_smem = smem + 3 * kTileBytes;    // early-gathered salient K rows (at most kFastSal)
  uint8_t* dvs_smem = ks_smem + kSalBytes;     // early-gathered dV rows
  __shared__ uint64_t q_full, k_full[2], k_empty[2], s_full[2], s_empty[2], b_full, p_full, pv_done, a_done, c_full;
  // delta kernel: buffers handed back to the producer / the MMA warp while the item is still in its epilogue
  __shared__ uint64_t q_free, kv0_free, kv1_free, o_free;
  // delta kernel, full tiles: the softmax threads have written the new context tile; the producer stores it
  __shared__ uint64_t c_stored;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int s_src[128];        // source row of each gather slot (-1 = none)
  __shared__ float2 s_ml[2][128];   // (max, sum) of the two column halves of each query row
  __shared__ float4 s_st[128];      // statistics of the second half of each row
  __shared__ uint16_t s_sal_pos[128];  // 1 + position in the sequence's salient list of this query row, 0 = not salient

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool v_mn_major = EXACT ? true : (p.v_mn_major != 0);

  if (EXACT && p.skip_small) {
    // usually every sequence has few salient rows and the other kernel has done all the work: leave
    // before any set-up
    int any = 0;
    for (int b = threadIdx.x; b < p.batch; b += blockDim.x) {
      const int n = p.cu_sal[b + 1] - p.cu_sal[b];
      const int kt = (p.cu_k[b + 1] - p.cu_k[b] + kBKeys - 1) / kBKeys;
      any |= (n > 0 && !small_rows_item(n, kt)) ? 1 : 0;
    }
    if (!__syncthreads_or(any))
      return;
  }

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
    mbar_init(&c_full, 1);
    mbar_init(&q_free, 1);
    mbar_init(&kv0_free, 1);
    mbar_init(&kv1_free, 1);
    mbar_init(&o_free, 256);
    mbar_init(&c_stored, 256);
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
    // ---------------------------------------------------------------- producer: Q (delta kernel), K tiles,
    // and for the EXACT kernel the K / V tiles of pass B
    int n_items = 0;            // items started so far
    int kuse[2] = {0, 0};       // loads issued into each K stage
    int n_pv = 0;               // P V products waited for (EXACT)
    int n_kv1 = 0, n_cst = 0;   // phases of kv1_free and c_stored waited for
    AttnItem prev_it;           // the previous item of this CTA (its context tile may still have to be stored)
    prev_it.tile_tma = false;
    // K stage 1 of the previous item becomes free.  A full tile's new context sits there: once the softmax
    // threads have written it, this warp stores it (out and, with an in-place cache, the cache rows) and waits
    // until the stores have read shared memory.  Otherwise the softmax threads signal kv1_free themselves.
    auto release_stage1 = [&]() {
      if (prev_it.tile_tma) {
        mbar_wait(&c_stored, (n_cst++) & 1, &abort_flag, p.status_word, 320);
        if (lane == 0) {
          tma_store_2d(&tmap_out, kv_smem1, prev_it.h * kD, prev_it.q0);
          tma_store_2d(&tmap_out, kv_smem1 + kHalfBytes, prev_it.h * kD + 64, prev_it.q0);
          if (p.c_cache) {
            tma_store_2d(&tmap_c, kv_smem1, prev_it.h * kD, static_cast<int>(prev_it.q0 + prev_it.c_delta));
            tma_store_2d(&tmap_c, kv_smem1 + kHalfBytes, prev_it.h * kD + 64, static_cast<int>(prev_it.q0 + prev_it.c_delta));
          }
          tma_store_commit();
          tma_store_wait_read();
        }
        __syncwarp();
      } else {
        mbar_wait(&kv1_free, (n_kv1++) & 1, &abort_flag, p.status_word, 316);
      }
    };
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      AttnItem it;
      if (!decode_item<EXACT>(p, item, it))
        continue;
      // Delta kernel: the softmax warps hand the buffers back one by one while the previous item is still
      // in its epilogue (Q after the last product with Q, K stage 0 after the last P dV product, K stage 1
      // after the stores of the context tile), so the first tiles of this item are in flight early.
      // EXACT kernel: its last P V product was awaited below.
      const uint32_t prev = (n_items - 1) & 1;
      if (!EXACT && n_items > 0)
        mbar_wait(&q_free, prev, &abort_flag, p.status_word, 314);
      if (lane == 0) {
        if (!EXACT) {
          mbar_arrive_expect_tx(&q_full, kTileBytes);
          tma_load_2d(q_smem, &tmap_q, &q_full, it.h * kD, it.q0);
          tma_load_2d(q_smem + kHalfBytes, &tmap_q, &q_full, it.h * kD + 64, it.q0);
          // the query tile of this CTA's next item
          AttnItem nx;
          const int next = item + gridDim.x;
          if (next < p.num_items && decode_item<EXACT>(p, next, nx)) {
            tma_prefetch_2d(&tmap_q, nx.h * kD, nx.q0);
            tma_prefetch_2d(&tmap_q, nx.h * kD + 64, nx.q0);
          }
        } else {
          // the value tiles are read once, late, and nothing else has touched them: bring them into L2 now
          for (int st = 0; st < it.num_st; ++st) {
            tma_prefetch_2d(&tmap_v, it.hk * kD, it.k_begin + st * kBKeys);
            tma_prefetch_2d(&tmap_v, it.hk * kD + 64, it.k_begin + st * kBKeys);
          }
        }
      }
      for (int kt = 0; kt < it.num_kt; ++kt) {
        const int s = kt & 1;
        const int u = kuse[s]++;
        if (!EXACT && n_items > 0 && kt == 0)
          mbar_wait(&kv0_free, prev, &abort_flag, p.status_word, 316);
        if (!EXACT && n_items > 0 && kt == 1)
          release_stage1();
        mbar_wait(&k_empty[s], (u & 1) ^ 1, &abort_flag, p.status_word, 301);
        if (lane == 0) {
          uint8_t* dst = s ? kv_smem1 : kv_smem0;
          mbar_arrive_expect_tx(&k_full[s], kTileBytes);
          tma_load_2d(dst, &tmap_k, &k_full[s], it.hk * kD, it.k_begin + kt * kBKeys);
          tma_load_2d(dst + kHalfBytes, &tmap_k, &k_full[s], it.hk * kD + 64, it.k_begin + kt * kBKeys);
        }
        __syncwarp();
      }
      if (EXACT) {
        // pass B: K tile into buffer 0 and V tile into buffer 1 once both are free
        for (int st = 0; st < it.num_st; ++st) {
          if (st == 0)
            mbar_wait(&a_done, n_items & 1, &abort_flag, p.status_word, 311);
          else
            mbar_wait(&pv_done, (n_pv++) & 1, &abort_flag, p.status_word, 312);
          if (lane == 0) {
            mbar_arrive_expect_tx(&b_full, 2 * kTileBytes);
            tma_load_2d(kv_smem0, &tmap_k, &b_full, it.hk * kD, it.k_begin + st * kBKeys);
            tma_load_2d(kv_smem0 + kHalfBytes, &tmap_k, &b_full, it.hk * kD + 64, it.k_begin + st * kBKeys);
            tma_load_2d(kv_smem1, &tmap_v, &b_full, it.hk * kD, it.k_begin + st * kBKeys);
            tma_load_2d(kv_smem1 + kHalfBytes, &tmap_v, &b_full, it.hk * kD + 64, it.k_begin + st * kBKeys);
          }
          __syncwarp();
        }
        if (it.num_st > 0)   // the last product has read both buffers: the next item may load into them
          mbar_wait(&pv_done, (n_pv++) & 1, &abort_flag, p.status_word, 315);
      } else if (n_items > 0 && it.num_kt < 2) {
        release_stage1();   // no second key tile: the previous item's context tile still has to go out
      }
      prev_it = it;
      ++n_items;
    }
    if (!EXACT && n_items > 0 && prev_it.tile_tma) {
      release_stage1();   // context tile of the last item
      if (lane == 0)
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, v_mn_major ? 1 : 0);
    const uint32_t q_addr = smem_u32(q_smem);
    int n_items = 0;
    int kuse[2] = {0, 0};   // K stages consumed
    int uses[2] = {0, 0};   // how often each S buffer has been handed to the softmax warps
    int n_sal_tiles = 0;    // pass-B tiles so far (phases of b_full and p_full)
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      AttnItem it;
      if (!decode_item<EXACT>(p, item, it))
        continue;
      // pass B of the delta kernel: keys of the tile rounded up to the MMA granularity
      const uint32_t k_half_stride = it.fast ? kSalHalfBytes : kHalfBytes;
      mbar_wait(&q_full, n_items & 1, &abort_flag, p.status_word, 302);
      bool o_waited = EXACT || n_items == 0;
      for (int t = 0; t < it.num_kt + it.num_st; ++t) {
        const bool sal_tile = t >= it.num_kt;
        const int st = t - it.num_kt;
        const int sb = sal_tile ? 0 : (t & 1);   // pass B keeps to buffer 0: buffer 1 holds O then
        const int use = uses[sb]++;
        if (!o_waited && (sb == 1 || sal_tile)) {
          // columns 128..255 still hold the previous item's O until its epilogue has read them
          mbar_wait(&o_free, (n_items - 1) & 1, &abort_flag, p.status_word, 318);
          o_waited = true;
        }
        const uint32_t tmem_s = tmem_s0 + sb * 128;
        uint32_t kb_addr;
        uint32_t idesc_s = idesc_qk;
        int n16 = kBKeys;
        if (!sal_tile) {
          const int s = t & 1;
          mbar_wait(&k_full[s], (kuse[s]++) & 1, &abort_flag, p.status_word, 303);
          kb_addr = smem_u32(s ? kv_smem1 : kv_smem0);
        } else {
          mbar_wait(&b_full, n_sal_tiles & 1, &abort_flag, p.status_word, 304);
          kb_addr = smem_u32(it.fast ? ks_smem : kv_smem0);
          if (!EXACT) {
            n16 = (min(kBKeys, it.n_sal - st * kBKeys) + 15) & ~15;
            idesc_s = umma_idesc_bf16(128, n16, 0, 0);
          }
        }
        mbar_wait(&s_empty[sb], (use & 1) ^ 1, &abort_flag, p.status_word, 305);
        tc_fence_after_sync();
        if (lane == 0) {
          // S = Q K^T: contraction over d in two swizzled halves of 64, four K = 16 steps each
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint64_t a_desc = umma_smem_desc_sw128(q_addr + half * kHalfBytes, 16, 1024);
            const uint64_t b_desc =
                umma_smem_desc_sw128(kb_addr + half * (sal_tile ? k_half_stride : kHalfBytes), 16, 1024);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ss(tmem_s, a_desc + 2 * kk, b_desc + 2 * kk, idesc_s, (half | kk) != 0 ? 1u : 0u);
          }
          if (!sal_tile)
            umma_commit(&k_empty[t & 1]);
          umma_commit(&s_full[sb]);
          if (EXACT && t == it.num_kt - 1)
            umma_commit(&a_done);
        }
        __syncwarp();
        if (sal_tile) {
          // O += P dV over the salient keys of this tile (zero padded to n16)
          mbar_wait(&p_full, n_sal_tiles & 1, &abort_flag, p.status_word, 306);
          ++n_sal_tiles;
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t p_addr = smem_u32(kv_smem0);
            const uint32_t v_addr = smem_u32(it.fast ? dvs_smem : kv_smem1);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              if (kk >= n16 / 16)
                break;
              const uint64_t a_desc =
                  umma_smem_desc_sw128(p_addr + (kk >> 2) * kHalfBytes + (kk & 3) * 32, 16, 1024);
              uint64_t b_desc;
              if (v_mn_major)  // [keys][d]: 16 keys = 2048 bytes per step, d halves one half-tile apart
                b_desc = umma_smem_desc_sw128(v_addr + kk * 2048, k_half_stride, 1024);
              else               // [d][keys]: key halves 16 KB apart, 32 bytes per step inside a half
                b_desc = umma_smem_desc_sw128(v_addr + (kk >> 2) * kHalfBytes + (kk & 3) * 32, 16, 1024);
              umma_ss(tmem_o, a_desc, b_desc, idesc_pv, (st | kk) != 0 ? 1u : 0u);
            }
            umma_commit(&pv_done);
          }
          __syncwarp();
        }
      }
      if (!o_waited)
        mbar_wait(&o_free, (n_items - 1) & 1, &abort_flag, p.status_word, 319);   // keep in step
      ++n_items;
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
    int uses[2] = {0, 0};   // S buffers read so far
    int n_pv = 0;           // P V products waited for
    int n_c = 0;            // context tiles loaded
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      AttnItem it;
      if (!decode_item<EXACT>(p, item, it))
        continue;
      const int h = it.h, hk = it.hk, q0 = it.q0, q_end = it.q_end, sal_begin = it.sal_begin, n_sal = it.n_sal;
      const int num_kt = it.num_kt, num_st = it.num_st, len_k = it.len_k, k_shift = it.k_shift;
      const int64_t c_delta = it.c_delta;
      const bool tile_tma = it.tile_tma, fast = it.fast;
      float m = kNegBig, l = 0.f;
      DYLLM_TRACE(0);
#ifdef DYLLM_ATTN_TRACE
      if (p.trace && item >= static_cast<int>(p.trace_first) && item < static_cast<int>(p.trace_first) + 1024 &&
          threadIdx.x == 64) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.trace[(item - p.trace_first) * 16 + 14] = smid;
      }
#endif

      if (!EXACT && q0 + row < q_end) {
        // bring this thread's half of the C_old row (128 bytes) into L2 now; the epilogue reads it much later
        const char* crow =
            reinterpret_cast<const char*>(p.c_old + ((q0 + row + c_delta) * p.H + h) * kD + col0);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(crow));
      }
      // a warp whose 32 query rows all lie past the end of the sequence keeps the barrier protocol going
      // but computes nothing
      const bool warp_live = q0 + qd * 32 < q_end;
      // Delta kernel, few salient keys: their K and dV rows (16 slots x 16 chunks of 16 bytes, one per thread,
      // zeros past the list) are requested now and written to shared memory after pass A, so that nothing of
      // the item's set-up stands between the softmax threads and the first logits.
      uint4 early_k = make_uint4(0, 0, 0, 0), early_v = make_uint4(0, 0, 0, 0);
      if (!EXACT && fast) {
        const int r = st_tid >> 4, ch = st_tid & 15;
        if (r < n_sal) {
          const int src = p.idx_k ? p.idx_k[sal_begin + r] : p.idx_q[sal_begin + r] + k_shift;
          early_k = __ldg(reinterpret_cast<const uint4*>(p.k + (static_cast<int64_t>(src) * p.Hkv + hk) * kD) + ch);
          const int64_t vrow = p.v_compact ? static_cast<int64_t>(sal_begin + r) : src;
          early_v = __ldg(reinterpret_cast<const uint4*>(p.v + (vrow * p.Hkv + hk) * kD) + ch);
        }
      }
      if (EXACT) {
        // source rows of the query gather
        if (half == 0)
          s_src[row] = q0 + row < q_end ? p.idx_q[sal_begin + q0 + row] : -1;
        // cooperative gather of the query rows (zeros past the list) into the swizzled Q tile
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int gi = 0; gi < 8; ++gi) {
          const int slot = gi * 256 + st_tid;
          const int r = slot >> 4, ch = slot & 15;
          const int src = s_src[r];
          const uint4 qv = src >= 0
              ? __ldg(reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(src) * p.H + h) * kD) + ch) : zero;
          *reinterpret_cast<uint4*>(q_smem + (ch >> 3) * kHalfBytes + sw128_offset(r, ch & 7)) = qv;
        }
        fence_proxy_async_smem();
        mbar_arrive(&q_full);
      }

      // pass A: running maximum and sum over this thread's half of the columns of every key tile
      for (int kt = 0; kt < num_kt; ++kt) {
        const int sb = kt & 1;
        const int use = uses[sb]++;
        const uint32_t tmem_s = tmem_s0 + sb * 128;
        mbar_wait(&s_full[sb], use & 1, &abort_flag, p.status_word, 307);
        tc_fence_after_sync();
        if (kt == 0)
          DYLLM_TRACE(7);
        const int valid = len_k - kt * kBKeys;   // keys of this tile that belong to the sequence
        if (!warp_live) {
          tc_fence_before_sync();
          mbar_arrive(&s_empty[sb]);
          continue;
        }
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
          if (valid < kBKeys) {   // keys past the end of the sequence
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c0 + i >= valid)
                sr[i] = __float_as_uint(kNegBig);
          }
          float cmax = kNegBig;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            cmax = fmax3(cmax, __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
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
            if (kPassAHalfExp) {
              acc0 = fadd2(acc0, ex2_pair_f16(x0.x, x0.y));
              acc1 = fadd2(acc1, ex2_pair_f16(x1.x, x1.y));
            } else {
              acc0 = fadd2(acc0, make_float2(ex2(x0.x), ex2(x0.y)));
              acc1 = fadd2(acc1, make_float2(ex2(x1.x), ex2(x1.y)));
            }
          }
          const float sum = (acc0.x + acc1.x) + (acc0.y + acc1.y);
          l = l * ex2((m - m_new) * c) + sum;
          m = m_new;
        }
      }
      if (!EXACT) {
        if (fast) {
          const int r = st_tid >> 4, ch = st_tid & 15;
          *reinterpret_cast<uint4*>(ks_smem + (ch >> 3) * kSalHalfBytes + sw128_offset(r, ch & 7)) = early_k;
          *reinterpret_cast<uint4*>(dvs_smem + (ch >> 3) * kSalHalfBytes + sw128_offset(r, ch & 7)) = early_v;
          fence_proxy_async_smem();
          mbar_arrive(&b_full);
        }
        if (half == 0) {
          // source rows of the first gathered tile of pass B (more than kFastSal salient keys)
          s_src[row] = row < n_sal ? (p.idx_k ? p.idx_k[sal_begin + row] : p.idx_q[sal_begin + row] + k_shift) : -1;
          s_sal_pos[row] = 0;
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
      if (!EXACT) {
        // mark the query rows of this tile that are salient (they take the exactly attended values); the
        // epilogue reads the marks after the P dV product, which every thread's arrival on p_full precedes
        for (int j = st_tid; j < n_sal; j += 256) {
          const int rr = p.idx_q[sal_begin + j] - q0;
          if (rr >= 0 && rr < kBQ)
            s_sal_pos[rr] = static_cast<uint16_t>(j + 1);
        }
      }

      // pass B: salient keys (EXACT: all keys again, with their values)
      DYLLM_TRACE(1);
      const float mc = m * c;
      // K stage 1 is not used by pass B when the salient rows were gathered early (or there are none):
      // the previous context tile can already come in.  Otherwise it follows the last P dV product.
      const bool c_early = fast || num_st == 0;
      if (!EXACT && st_tid == 0) {
        if (tile_tma && c_early) {
          mbar_arrive_expect_tx(&c_full, kTileBytes);
          tma_load_2d(kv_smem1, &tmap_c, &c_full, h * kD, static_cast<int>(q0 + c_delta));
          tma_load_2d(kv_smem1 + kHalfBytes, &tmap_c, &c_full, h * kD + 64, static_cast<int>(q0 + c_delta));
        }
        if (num_st == 0) {   // no product reads Q or P any more
          mbar_arrive(&q_free);
          mbar_arrive(&kv0_free);
          if (!tile_tma)
            mbar_arrive(&kv1_free);
        }
      }
      for (int st = 0; st < num_st; ++st) {
        // The buffers are free for tile 0 once the last Q K^T product is complete: s_full of the last
        // key tile was observed above and is committed after every earlier MMA.  Later tiles wait for the
        // previous P dV product.
        if (!EXACT && st > 0) {
          mbar_wait(&pv_done, (n_pv++) & 1, &abort_flag, p.status_word, 308);
          if (half == 0) {
            const int j = st * kBKeys + row;
            s_src[row] = j < n_sal ? (p.idx_k ? p.idx_k[sal_begin + j] : p.idx_q[sal_begin + j] + k_shift) : -1;
          }
          asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        if (EXACT && st > 0)
          mbar_wait(&pv_done, (n_pv++) & 1, &abort_flag, p.status_word, 308);
        const int n_tile = min(kBKeys, (EXACT ? len_k : n_sal) - st * kBKeys);
        const int n16 = EXACT ? kBKeys : (n_tile + 15) & ~15;   // columns the MMAs of this tile cover
        if (!EXACT && !fast) {
          // cooperative gather of the first n16 slots x 16 chunks of the K rows and of the dV rows, zeros
          // past the list; slots beyond n16 are read by no MMA
          const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 1
          for (int gi = 0; gi < n16 / 16; ++gi) {
            const int slot = gi * 256 + st_tid;
            const int r = slot >> 4, ch = slot & 15;
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
        if (!EXACT && st == num_st - 1 && st_tid == 0)
          mbar_arrive(&q_free);   // the last product that reads the query tile is complete
#pragma unroll 1
        for (int cc = 0; cc < 64; cc += 32) {
          const int c0 = col0 + cc;
          if (c0 >= n16 || !warp_live)
            continue;   // uniform over the warp: no MMA reads these columns (or these rows are unused)
          uint32_t sr[32];
          tmem_ld_32x32(tmem_s0 + t_lane + c0, sr);
          tmem_ld_wait();
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
        tc_fence_before_sync();
        mbar_arrive(&s_empty[0]);
        fence_proxy_async_smem();
        mbar_arrive(&p_full);
        DYLLM_TRACE(4);
      }
      if (num_st > 0) {
        mbar_wait(&pv_done, (n_pv++) & 1, &abort_flag, p.status_word, 310);
        tc_fence_after_sync();
        if (!EXACT && st_tid == 0) {
          mbar_arrive(&kv0_free);   // P has been read
          if (tile_tma && !c_early) {
            mbar_arrive_expect_tx(&c_full, kTileBytes);
            tma_load_2d(kv_smem1, &tmap_c, &c_full, h * kD, static_cast<int>(q0 + c_delta));
            tma_load_2d(kv_smem1 + kHalfBytes, &tmap_c, &c_full, h * kD + 64, static_cast<int>(q0 + c_delta));
          }
          if (!tile_tma)
            mbar_arrive(&kv1_free);   // dV has been read and no context tile will use the buffer
        }
      }
      DYLLM_TRACE(5);

      // epilogue: new = old + O / rowsum for this thread's 64 of the 128 head dimensions (salient rows take
      // the exactly attended row instead); bf16 store; partial statistics of this head.  The tensor-memory
      // loads are warp-collective, so every lane issues them; global-memory traffic is predicated on the row
      // being inside the sequence.
      const int r = q0 + row;
      const bool live = r < q_end;
      const float inv_l = l > 0.f ? 1.0f / l : 0.f;
      const int64_t off = (static_cast<int64_t>((live ? r : q0) + (EXACT ? sal_begin : 0)) * p.H + h) * kD + col0;
      const int64_t c_off = (((live ? r : q0) + c_delta) * p.H + h) * kD + col0;
      __nv_bfloat16* dst = (EXACT ? p.o_sal : p.out) + off;
      __nv_bfloat16* cdst = (!EXACT && p.c_cache) ? p.c_cache + c_off : nullptr;
      uint8_t* c_tile = kv_smem1 + half * kHalfBytes;   // tile_tma: this thread's half of the context tile
      float dot = 0.f, nn = 0.f, no = 0.f;
      uint4 old_row[8];
      if (tile_tma) {
        mbar_wait(&c_full, (n_c++) & 1, &abort_flag, p.status_word, 313);
        DYLLM_TRACE(8);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          old_row[j] = *reinterpret_cast<const uint4*>(c_tile + sw128_offset(row, j));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          old_row[j] = (EXACT || !live) ? make_uint4(0, 0, 0, 0)
                                        : __ldg(reinterpret_cast<const uint4*>(p.c_old + c_off) + j);
      }
      // salient query row: its new value is the exactly attended row
      const int sal_pos = EXACT ? 0 : s_sal_pos[row];
      const uint4* sal_src = nullptr;
      if (!EXACT && sal_pos && live)
        sal_src = reinterpret_cast<const uint4*>(
            p.o_sal + (static_cast<int64_t>(sal_begin + sal_pos - 1) * p.H + h) * kD + col0);
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
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(old_row + cc / 8);
          uint32_t pk[16];
          float2 d2 = make_float2(0.f, 0.f), n2 = make_float2(0.f, 0.f), q2 = make_float2(0.f, 0.f);
          if (!sal_src) {
            const float2 il2 = make_float2(inv_l, inv_l);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
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
            uint4 sal_row[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              sal_row[j] = __ldg(sal_src + cc / 8 + j);
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(sal_row);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
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
          if (tile_tma) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(c_tile + sw128_offset(row, cc / 8 + j)) =
                  make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(dst + cc)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            if (cdst) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(cdst + cc)[j] =
                    make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            }
          }
        }
      }
      if (!EXACT) {
        // this thread has read its part of O: the MMA warp may reuse the columns once all have
        tc_fence_before_sync();
        mbar_arrive(&o_free);
        // the two halves of a row add their statistics in a fixed order (half 0 + half 1)
        if (half == 1)
          s_st[row] = make_float4(dot, nn, no, 0.f);
        if (tile_tma) {
          fence_proxy_async_smem();   // the updated tile is read by the TMA stores that the producer warp issues
          mbar_arrive(&c_stored);
        }
        DYLLM_TRACE(9);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        DYLLM_TRACE(10);
        if (half == 0 && live) {
          const float4 o = s_st[row];
          float* ps = p.partial + (static_cast<int64_t>(h) * p.Tq + r) * 3;
          ps[0] = dot + o.x;
          ps[1] = nn + o.y;
          ps[2] = no + o.z;
        }
      }
      // end of the item: every softmax thread is done with the tensor-memory accumulator and with the
      // small shared arrays; then the producer may refill the tile buffers
      tc_fence_before_sync();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      DYLLM_TRACE(6);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_slot, kAttnTmemCols);
  }
}

// ----------------------------------------------------------------------------------------------
// Exact attention of a FEW salient query rows (at most 16 per sequence, the common case):
//   o_sal[i] = softmax(q[idx_q[i]] K^T / sqrt(D)) V
// With so few rows a 128-row query tile is almost empty, so the products are transposed: one CTA per
// (sequence, head) computes S^T = K Q^T tile by tile (M = 128 keys, N = 16 rows) and keeps S^T of the whole
// sequence in tensor memory (16 columns per key tile); the key and value tiles stream once through a
// three-slot TMA ring (values follow the keys, so they arrive while the row maxima are being reduced);
// a thread owns one key of a tile: the maximum over keys is a warp-shuffle + shared-memory reduction,
// P^T = exp2(S^T c - m c) goes to shared memory as the [16 rows][128 keys] K-major operand of
// O^T += V^T P^T (V tile used as loaded, as the MN-major A operand; M = 128 head dimensions, N = 16),
// and O^T / rowsum leaves with 64-byte row segments per warp.  Sequences with more rows or more than
// kSmallMaxTiles key tiles are left to attention_kernel<true>.
// ----------------------------------------------------------------------------------------------
constexpr int kSmallStages = 3;
constexpr uint32_t kSmallSmem = kSmallStages * kTileBytes + 3 * kSalBytes + 1024;   // ring, Q, two P slots

__global__ void __launch_bounds__(kAttnThreads, 2)
salient_rows_small_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                          const AttnParams p) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int sal_begin = p.cu_sal[b];
  const int n_sal = p.cu_sal[b + 1] - sal_begin;
  const int k_begin = p.cu_k[b];
  const int len_k = p.cu_k[b + 1] - k_begin;
  const int num_kt = (len_k + kBKeys - 1) / kBKeys;
  if (!small_rows_item(n_sal, num_kt))
    return;
  const int hk = h / (p.H / p.Hkv);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem + kSmallStages * kTileBytes;   // [16 rows][128 d], two 64-column halves
  uint8_t* p_smem = q_smem + kSalBytes;                 // two slots of [16 rows][128 keys]
  __shared__ uint64_t full[kSmallStages], empty[kSmallStages], q_full, s_done, p_full[2], p_empty[2], o_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float s_red[8][kSmallRows];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < kSmallStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&q_full, 256);
    mbar_init(&s_done, 1);
    mbar_init(&p_full[0], 128);
    mbar_init(&p_full[1], 128);
    mbar_init(&p_empty[0], 1);
    mbar_init(&p_empty[1], 1);
    mbar_init(&o_done, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kAttnTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_st = tmem_slot;                       // S^T of key tile t: columns [16 t, 16 t + 16)
  const uint32_t tmem_ot = tmem_slot + num_kt * kSmallRows;   // O^T: 16 columns

  if (warp == 0) {
    // ---------------------------------------------------------------- producer: K tiles, then V tiles
    for (int i = 0; i < 2 * num_kt; ++i) {
      const int slot = i % kSmallStages;
      mbar_wait(&empty[slot], ((i / kSmallStages) & 1) ^ 1, &abort_flag, p.status_word, 331);
      if (lane == 0) {
        const CUtensorMap* map = i < num_kt ? &tmap_k : &tmap_v;
        const int t = i < num_kt ? i : i - num_kt;
        uint8_t* dst = smem + slot * kTileBytes;
        mbar_arrive_expect_tx(&full[slot], kTileBytes);
        tma_load_2d(dst, map, &full[slot], hk * kD, k_begin + t * kBKeys);
        tma_load_2d(dst + kHalfBytes, map, &full[slot], hk * kD + 64, k_begin + t * kBKeys);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = umma_idesc_bf16(128, kSmallRows, 0, 0);    // K tile (K-major) x Q (K-major)
    constexpr uint32_t idesc_o = umma_idesc_bf16(128, kSmallRows, 1, 0);    // V tile (MN-major) x P (K-major)
    const uint32_t q_addr = smem_u32(q_smem);
    mbar_wait(&q_full, 0, &abort_flag, p.status_word, 332);
    for (int t = 0; t < num_kt; ++t) {
      const int slot = t % kSmallStages;
      mbar_wait(&full[slot], (t / kSmallStages) & 1, &abort_flag, p.status_word, 333);
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(smem + slot * kTileBytes);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint64_t a_desc = umma_smem_desc_sw128(k_addr + half * kHalfBytes, 16, 1024);
          const uint64_t b_desc = umma_smem_desc_sw128(q_addr + half * kSalHalfBytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem_st + t * kSmallRows, a_desc + 2 * kk, b_desc + 2 * kk, idesc_s, (half | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[slot]);
        if (t == num_kt - 1)
          umma_commit(&s_done);
      }
      __syncwarp();
    }
    for (int t = 0; t < num_kt; ++t) {
      const int i = num_kt + t;
      const int slot = i % kSmallStages;
      mbar_wait(&full[slot], (i / kSmallStages) & 1, &abort_flag, p.status_word, 334);
      mbar_wait(&p_full[t & 1], (t >> 1) & 1, &abort_flag, p.status_word, 335);
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(smem + slot * kTileBytes);
        const uint32_t p_addr = smem_u32(p_smem + (t & 1) * kSalBytes);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 keys per step: V rows [keys][d] (2048 bytes per step, d halves one half-tile apart),
          // P rows [16][keys] (32 bytes per step inside a 64-key half)
          const uint64_t a_desc = umma_smem_desc_sw128(v_addr + kk * 2048, kHalfBytes, 1024);
          const uint64_t b_desc =
              umma_smem_desc_sw128(p_addr + (kk >> 2) * kSalHalfBytes + (kk & 3) * 32, 16, 1024);
          umma_ss(tmem_ot, a_desc, b_desc, idesc_o, (t | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[slot]);
        umma_commit(&p_empty[t & 1]);
        if (t == num_kt - 1)
          umma_commit(&o_done);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- softmax over keys / epilogue
    const int sw = warp - 2;                 // 0..7
    const int qd = warp & 3;                 // tensor-memory lane quarter: keys (or head dims) 32 qd .. 32 qd + 31
    const int half = sw >> 2;                // key tiles t with t % 2 == half; P slot `half`
    const int st_tid = sw * 32 + lane;
    const int kl = qd * 32 + lane;           // key inside a tile / head dimension in the epilogue
    const uint32_t t_lane = static_cast<uint32_t>(qd * 32) << 16;
    const float c = p.scale_log2;

    {  // gather the query rows: 16 rows x 16 chunks of 16 bytes, one per thread, zeros past the list
      const int r = st_tid >> 4, ch = st_tid & 15;
      uint4 qv = make_uint4(0, 0, 0, 0);
      if (r < n_sal) {
        const int src = p.idx_q[sal_begin + r];
        qv = __ldg(reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(src) * p.H + h) * kD) + ch);
      }
      *reinterpret_cast<uint4*>(q_smem + (ch >> 3) * kSalHalfBytes + sw128_offset(r, ch & 7)) = qv;
      fence_proxy_async_smem();
      mbar_arrive(&q_full);
    }

    // row maxima over all keys
    mbar_wait(&s_done, 0, &abort_flag, p.status_word, 336);
    tc_fence_after_sync();
    float m[kSmallRows];
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r)
      m[r] = kNegBig;
    for (int t = half; t < num_kt; t += 2) {
      uint32_t sr[kSmallRows];
      tmem_ld_32x16(tmem_st + t_lane + t * kSmallRows, sr);
      tmem_ld_wait();
      if (t * kBKeys + kl < len_k) {
#pragma unroll
        for (int r = 0; r < kSmallRows; ++r)
          m[r] = fmaxf(m[r], __uint_as_float(sr[r]));
      }
    }
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        m[r] = fmaxf(m[r], __shfl_xor_sync(0xffffffffu, m[r], off));
    }
    if (lane < kSmallRows) {
      // lane r publishes row r (a select chain instead of dynamic register indexing)
      float v = m[0];
#pragma unroll
      for (int r = 1; r < kSmallRows; ++r)
        v = lane == r ? m[r] : v;
      s_red[sw][lane] = v;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r) {
      float v = s_red[0][r];
#pragma unroll
      for (int w = 1; w < 8; ++w)
        v = fmaxf(v, s_red[w][r]);
      m[r] = v * c;   // from here on m holds max * c
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");   // s_red is reused for the sums

    // P^T tile by tile (unnormalised), row sums on the side
    float l[kSmallRows];
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r)
      l[r] = 0.f;
    uint8_t* p_slot = p_smem + half * kSalBytes;
    for (int t = half, n = 0; t < num_kt; t += 2, ++n) {
      uint32_t sr[kSmallRows];
      tmem_ld_32x16(tmem_st + t_lane + t * kSmallRows, sr);
      tmem_ld_wait();
      const bool valid = t * kBKeys + kl < len_k;
      mbar_wait(&p_empty[half], (n & 1) ^ 1, &abort_flag, p.status_word, 337);
      // element (row r, key kl): 64-key half kl / 64, 16-byte chunk (kl % 64) / 8, 2 bytes at kl % 8
      uint8_t* base = p_slot + (kl >> 6) * kSalHalfBytes + ((kl & 7) << 1);
      const uint32_t chunk = (kl & 63) >> 3;
#pragma unroll
      for (int r = 0; r < kSmallRows; ++r) {
        const float e = valid ? ex2(fmaf(__uint_as_float(sr[r]), c, -m[r])) : 0.f;
        l[r] += e;
        *reinterpret_cast<__nv_bfloat16*>(base + r * 128u + ((chunk ^ (r & 7u)) << 4)) = __float2bfloat16_rn(e);
      }
      fence_proxy_async_smem();
      mbar_arrive(&p_full[half]);
    }
    // row sums over all keys
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], off);
    }
    if (lane < kSmallRows) {
      float v = l[0];
#pragma unroll
      for (int r = 1; r < kSmallRows; ++r)
        v = lane == r ? l[r] : v;
      s_red[sw][lane] = v;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    // epilogue: thread = head dimension kl; the two halves share the rows (8 each)
    mbar_wait(&o_done, 0, &abort_flag, p.status_word, 338);
    tc_fence_after_sync();
    uint32_t orr[kSmallRows];
    tmem_ld_32x16(tmem_ot + t_lane, orr);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < kSmallRows / 2; ++j) {
      const int r = half * (kSmallRows / 2) + j;
      if (r < n_sal) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w)
          sum += s_red[w][r];
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        // orr is indexed with a compile-time constant in each half
        const float o = half == 0 ? __uint_as_float(orr[j]) : __uint_as_float(orr[kSmallRows / 2 + j]);
        p.o_sal[(static_cast<int64_t>(sal_begin + r) * p.H + h) * kD + kl] = __float2bfloat16_rn(o * inv);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_slot, kAttnTmemCols);
  }
}

// ----------------------------------------------------------------------------------------------
// finalize: head-ordered reduction of the partial statistics + threshold mask, one thread per row.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ bool mask_rule(float dot, float a, float b, float threshold) {
  return dot * rsqrtf(fmaxf(a, 1e-8f)) * rsqrtf(fmaxf(b, 1e-8f)) < threshold;
}

__global__ void __launch_bounds__(256)
attention_finalize_kernel(const float* __restrict__ partial, int H, int Tq, float* __restrict__ stats,
                          uint8_t* __restrict__ mask, float threshold, int accumulate) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= Tq)
    return;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f;
  if (accumulate) {
    s0 = stats[r * 3 + 0];
    s1 = stats[r * 3 + 1];
    s2 = stats[r * 3 + 2];
  }
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
}

bool g_attn_smem_set[2][64] = {{false}, {false}};
unsigned long long* g_attn_trace = nullptr;

template <bool EXACT>
int launch_attention(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tout,
                     const CUtensorMap& tc, const AttnParams& p_in, int64_t items, cudaStream_t s) {
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
  DYLLM_REQUIRE(items > 0 && items < (1ll << 31), DYLLM_ERR_UNSUPPORTED, "attention: %lld work items",
                static_cast<long long>(items));
  AttnParams p = p_in;
  p.num_items = static_cast<int>(items);
  // persistent grid: as many CTAs as the device runs at once (two per SM)
  const int64_t resident = 2ll * sm_count();
  const unsigned blocks = static_cast<unsigned>(items < resident ? items : resident);
  DYLLM_LAUNCH(attention_kernel<EXACT>, blocks, kAttnThreads, kAttnSmem, s, tq, tk, tv, tout, tc, p);
  return check_launch(EXACT ? "salient_attention" : "delta_attention");
}

bool g_pair_smem_set[64] = {};

// Pair decomposition of the delta attention (attention_pair.cuh): one CTA per SM; the default when dV arrives as
// rows ([keys][d]).  DYLLM_ATTN_PAIR=0 selects the two-CTAs-per-SM kernel above instead.
bool pair_kernel_enabled() {
  static const bool on = [] {
    const char* e = getenv("DYLLM_ATTN_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

int launch_delta_pair(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tout, const CUtensorMap& tc,
                      const AttnParams& p_in, cudaStream_t s) {
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev < 0 || dev >= 64) ? 0 : dev;
  if (!g_pair_smem_set[dev]) {
    if (cudaFuncSetAttribute(delta_attention_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kPairSmem)) != cudaSuccess)
      return set_error(DYLLM_ERR_CUDA, "attention: cudaFuncSetAttribute failed: %s",
                       cudaGetErrorString(cudaGetLastError()));
    g_pair_smem_set[dev] = true;
  }
  AttnParams p = p_in;
  const int64_t items = static_cast<int64_t>(p.batch) * p.H * ((p.n_qtiles + 1) / 2);
  DYLLM_REQUIRE(items > 0 && items < (1ll << 31), DYLLM_ERR_UNSUPPORTED, "attention: %lld work items",
                static_cast<long long>(items));
  p.num_items = static_cast<int>(items);
  const int64_t resident = sm_count();
  const unsigned blocks = static_cast<unsigned>(items < resident ? items : resident);
  DYLLM_LAUNCH(delta_attention_pair_kernel, blocks, kPairThreads, kPairSmem, s, tq, tk, tout, tc, p);
  return check_launch("delta_attention(pair)");
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
  DYLLM_REQUIRE(num_salient == 0 || (v && o_sal && idx_salient_row_q), DYLLM_ERR_INVALID_ARGUMENT,
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
  p.o_sal = const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(o_sal));
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
  p.batch = batch;
  const int64_t blocks = static_cast<int64_t>(batch) * num_heads * p.n_qtiles;
  p.trace_first = blocks > 1536 ? 512u : 0u;   // the middle of the launch when it has several waves
  // context tiles: the new context [Tq, H*D], and the previous one (packed like Q, or the cache arena,
  // whose extent this call does not know: full tiles never leave the rows of their sequence)
  CUtensorMap tout, tc;
  rc = encode_tmap_2d_bf16(&tout, out, total_q, static_cast<uint64_t>(num_heads) * kD,
                           static_cast<uint64_t>(num_heads) * kD, kBQ, 64, true);
  if (rc != DYLLM_OK)
    return rc;
  rc = encode_tmap_2d_bf16(&tc, c, c_seq_starts ? (1ull << 30) : static_cast<uint64_t>(total_q),
                           static_cast<uint64_t>(num_heads) * kD, static_cast<uint64_t>(num_heads) * kD, kBQ, 64, true);
  if (rc != DYLLM_OK)
    return rc;
  if (v_mn_major && pair_kernel_enabled()) {
    rc = launch_delta_pair(tq, tk, tout, tc, p, s);
  } else {
    rc = launch_attention<false>(tq, tk, tk, tout, tc, p, blocks, s);
  }
  if (rc != DYLLM_OK)
    return rc;
  DYLLM_LAUNCH(attention_finalize_kernel, cdiv_i(total_q, 256), 256, 0, s, p.partial, num_heads, total_q, cosine_stats,
                                                                 cosine_out, threshold, (v_layout & 4) ? 0 : 1);
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
  p.batch = batch;
  // sequences with at most kSmallRows salient rows (and not too many key tiles): transposed kernel, one
  // CTA per (sequence, head); the general kernel skips them
  {
    static bool smem_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    if (!smem_set[dev]) {
      if (cudaFuncSetAttribute(salient_rows_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kSmallSmem)) != cudaSuccess)
        return set_error(DYLLM_ERR_CUDA, "attention_salient_rows: cudaFuncSetAttribute failed: %s",
                         cudaGetErrorString(cudaGetLastError()));
      smem_set[dev] = true;
    }
    DYLLM_LAUNCH(salient_rows_small_kernel, static_cast<unsigned>(batch) * num_heads, kAttnThreads, kSmallSmem, static_cast<cudaStream_t>(stream), tk, tv, p);
    rc = check_launch("salient_rows_small");
    if (rc != DYLLM_OK)
      return rc;
  }
  p.skip_small = 1;
  const int64_t blocks = static_cast<int64_t>(batch) * num_heads * p.n_qtiles;
  return launch_attention<true>(tk, tk, tv, tk, tk, p, blocks, static_cast<cudaStream_t>(stream));
}

#ifdef DYLLM_ATTN_TRACE
int dyllm_attention_trace(void* device_buffer) {
  g_attn_trace = static_cast<unsigned long long*>(device_buffer);
  return DYLLM_OK;
}
#endif

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
