// Row-wise kernels that surround the saliency path in a decoder layer: RMSNorm with the residual add
// fused in, and the NeoX-style rotary embedding.  Both are HBM-bound: each element is read once and
// written once.
#include "common.cuh"

namespace dyllm {
namespace {

constexpr int kNormThreads = 256;

// y = bf16( bf16((x + r) * rsqrt(mean((x + r)^2) + eps)) * w ), r_out = bf16(x + r); fp32 statistics.
// One block per row; VPT 16-byte vectors per thread are kept in registers between the two passes.
// yr null = only the residual sum is wanted; ror null = only the normalised row.
template <int VPT>
__device__ __forceinline__ void norm_one_row(const uint4* __restrict__ xr, const uint4* __restrict__ rr,
                                             const uint4* __restrict__ w, uint4* __restrict__ yr,
                                             uint4* __restrict__ ror, int vecs, float inv_width, float eps) {
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < vecs) {
      const uint4 xv = __ldg(xr + v);
      const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
      uint4 rv = make_uint4(0, 0, 0, 0);
      if (rr)
        rv = __ldg(rr + v);
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
      uint4 ro;
      __nv_bfloat162* ro2 = reinterpret_cast<__nv_bfloat162*>(&ro);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(x2[i]);
        const float2 b = __bfloat1622float2(r2[i]);
        const float s0 = a.x + b.x, s1 = a.y + b.y;
        vals[j][2 * i] = s0;
        vals[j][2 * i + 1] = s1;
        ss = fmaf(s0, s0, ss);
        ss = fmaf(s1, s1, ss);
        ro2[i] = __floats2bfloat162_rn(s0, s1);
      }
      if (ror)
        ror[v] = ro;
    }
  }
  if (!yr)
    return;      // uniform over the block
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    ss += __shfl_xor_sync(0xffffffffu, ss, off);
  __shared__ float red[kNormThreads / 32];
  __shared__ float s_scale;
  __syncthreads();   // a block that normalises several rows reuses the two shared words
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < kNormThreads / 32; ++i)
      t += red[i];
    s_scale = rsqrtf(t * inv_width + eps);
  }
  __syncthreads();
  const float scale = s_scale;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < vecs) {
      const uint4 wv = __ldg(w + v);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // two roundings, as the bf16 module does: normalise -> bf16, times weight -> bf16
        const __nv_bfloat162 n = __floats2bfloat162_rn(vals[j][2 * i] * scale, vals[j][2 * i + 1] * scale);
        o2[i] = __hmul2(n, w2[i]);
      }
      yr[v] = o;
    }
  }
}

template <int VPT>
__global__ void __launch_bounds__(kNormThreads)
add_rms_norm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res_in, const uint4* __restrict__ w,
                    uint4* __restrict__ y, uint4* __restrict__ res_out, int vecs, float inv_width, float eps,
                    int x_seg_rows, int64_t x_seg_pitch_rows) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int64_t row = blockIdx.x;
  // x may consist of equal segments of rows that lie x_seg_pitch_rows apart (a block of every sequence
  // read straight out of a cache); everything else is packed
  const int64_t x_row = (row / x_seg_rows) * x_seg_pitch_rows + row % x_seg_rows;
  norm_one_row<VPT>(x + x_row * vecs, res_in ? res_in + row * vecs : nullptr, w, y + row * vecs,
                    res_out ? res_out + row * vecs : nullptr, vecs, inv_width, eps);
}

// The same arithmetic with the listed rows' normalised values also (or only) written packed in list order:
// blocks [0, rows) handle their row (residual sum; normalised row when y_all is given), the remaining blocks
// walk the list and write the normalised row sel_idx[m] to y_sel[m], ready to be the packed input of a
// gathered GEMM (the FFN of a sparse step reads the salient rows alone; its K/V projection likewise).
template <int VPT>
__global__ void __launch_bounds__(kNormThreads)
add_rms_norm_rows_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res_in, const uint4* __restrict__ w,
                         uint4* __restrict__ y_all, uint4* __restrict__ y_sel, uint4* __restrict__ res_out, int rows,
                         int vecs, float inv_width,
                         float eps, int x_seg_rows, int64_t x_seg_pitch_rows, const int32_t* __restrict__ sel_idx,
                         int sel_max, const int32_t* __restrict__ sel_count_dev) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  if (static_cast<int>(blockIdx.x) < rows) {
    const int64_t row = blockIdx.x;
    const int64_t x_row = (row / x_seg_rows) * x_seg_pitch_rows + row % x_seg_rows;
    norm_one_row<VPT>(x + x_row * vecs, res_in ? res_in + row * vecs : nullptr, w, y_all ? y_all + row * vecs : nullptr,
                      res_out ? res_out + row * vecs : nullptr, vecs, inv_width, eps);
    return;
  }
  const int count = sel_count_dev ? min(sel_max, *sel_count_dev) : sel_max;
  for (int m = static_cast<int>(blockIdx.x) - rows; m < count; m += static_cast<int>(gridDim.x) - rows) {
    int64_t row = sel_idx[m];
    row = row < 0 ? 0 : (row >= rows ? rows - 1 : row);
    const int64_t x_row = (row / x_seg_rows) * x_seg_pitch_rows + row % x_seg_rows;
    norm_one_row<VPT>(x + x_row * vecs, res_in ? res_in + row * vecs : nullptr, w, y_sel + static_cast<int64_t>(m) * vecs,
                      nullptr, vecs, inv_width, eps);
  }
}

// RMSNorm over the 128 values of every (row, head), in place: one warp per head vector, 8 bytes per lane.
// y = bf16( bf16(x * rsqrt(mean(x^2) + eps)) * w ), the arithmetic of add_rms_norm without a residual.
__global__ void __launch_bounds__(256)
head_rms_norm_kernel(uint2* __restrict__ x, const uint2* __restrict__ w, int rows, int heads, float eps,
                     const int32_t* __restrict__ num_rows_dev) {
  pdl_wait();
  pdl_trigger();
  const int n = num_rows_dev ? min(rows, *num_rows_dev) : rows;
  const int64_t total = static_cast<int64_t>(n) * heads;
  const int lane = threadIdx.x & 31;
  const uint2 wv = __ldg(w + lane);
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5); v < total;
       v += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
    uint2* p = x + v * 32 + lane;
    const uint2 xv = *p;
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
    const float2 a = __bfloat1622float2(x2[0]), b = __bfloat1622float2(x2[1]);
    float ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float scale = rsqrtf(ss * (1.0f / 128.0f) + eps);
    uint2 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
    o2[0] = __hmul2(__floats2bfloat162_rn(a.x * scale, a.y * scale), w2[0]);
    o2[1] = __hmul2(__floats2bfloat162_rn(b.x * scale, b.y * scale), w2[1]);
    *p = o;
  }
}

// x[r, h, :] rotated in place by the angle table row of positions[pos_idx ? pos_idx[r] : r]:
// (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin), halves of 64; 8 threads per (row, head).
__global__ void __launch_bounds__(256)
rope_neox_kernel(uint4* __restrict__ x, const int64_t* __restrict__ positions, const int64_t* __restrict__ pos_idx,
                 const float* __restrict__ cos_sin, int rows, int heads, int max_pos,
                 const int32_t* __restrict__ num_rows_dev) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const int n = num_rows_dev ? min(rows, *num_rows_dev) : rows;
  const int64_t total = static_cast<int64_t>(n) * heads * 8;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int part = static_cast<int>(t & 7);          // which 8 of the 64 rotation pairs
    const int64_t rh = t >> 3;
    const int r = static_cast<int>(rh / heads);
    int64_t pos = positions[pos_idx ? pos_idx[r] : r];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + pos * 128;
    uint4* base = x + rh * 16;                          // 128 bf16 = 16 vectors
    const uint4 a = base[part], b = base[part + 8];
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 oa, ob;
    __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x1 = __bfloat1622float2(a2[i]);
      const float2 x2 = __bfloat1622float2(b2[i]);
      const int d = part * 8 + 2 * i;
      const float c0 = __ldg(cs + d), c1 = __ldg(cs + d + 1), s0 = __ldg(cs + 64 + d), s1 = __ldg(cs + 64 + d + 1);
      oa2[i] = __floats2bfloat162_rn(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
      ob2[i] = __floats2bfloat162_rn(x2.x * c0 + x1.x * s0, x2.y * c1 + x1.y * s1);
    }
    base[part] = oa;
    base[part + 8] = ob;
  }
}

// Confidence of the most likely token of every row of logits: conf = max_j softmax(x)_j = 1 / sum_j
// exp(x_j - max), token = the first j that attains the maximum.  One CTA per row, one pass over the row
// with 16-byte loads: every thread keeps a running (max, sum, argmax) and rescales its sum when its
// maximum grows; the block then merges the 256 triples.
// Confidence rule of the sampler for one block of candidates per sequence (ref: sampler.py:244-315): among the
// block's positions that still hold the mask token, the num_transfer most confident ones (ties: the lowest
// position) take their best token.  One CTA per sequence; the chosen positions come out ascending.
constexpr int kUnmaskThreads = 128;
constexpr int kUnmaskMaxBlock = 1024;
constexpr int kUnmaskMaxPicks = 64;

__global__ void __launch_bounds__(kUnmaskThreads)
confidence_unmask_kernel(const float* __restrict__ conf, const int64_t* __restrict__ best_token,
                         int64_t* __restrict__ tokens, int64_t seq_pitch, const int64_t* __restrict__ step_counter,
                         int steps_per_block, int num_blocks, int prompt_len, int block_len, int num_transfer,
                         int64_t mask_id, int64_t* __restrict__ picked_pos, int32_t* __restrict__ picked_count) {
  pdl_wait();
  pdl_trigger();
  __shared__ float s_conf[kUnmaskMaxBlock];
  __shared__ float s_best[kUnmaskThreads / 32];
  __shared__ int s_arg[kUnmaskThreads / 32];
  __shared__ int s_pick[kUnmaskMaxPicks];
  __shared__ int s_n;
  const int b = blockIdx.x;
  int64_t blk = step_counter ? *step_counter / steps_per_block : 0;
  blk = blk > num_blocks - 1 ? num_blocks - 1 : blk;
  const int start = prompt_len + static_cast<int>(blk) * block_len;
  int64_t* row = tokens + static_cast<int64_t>(b) * seq_pitch;
  for (int i = threadIdx.x; i < block_len; i += kUnmaskThreads)
    s_conf[i] = row[start + i] == mask_id ? conf[static_cast<int64_t>(b) * block_len + i] : -1.0f;
  if (threadIdx.x == 0)
    s_n = 0;
  __syncthreads();
  for (int pick = 0; pick < num_transfer; ++pick) {
    float best = -1.0f;
    int arg = 0x7fffffff;
    for (int i = threadIdx.x; i < block_len; i += kUnmaskThreads) {
      const float c = s_conf[i];
      if (c > best || (c == best && c >= 0.f && i < arg)) {
        best = c;
        arg = i;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    if ((threadIdx.x & 31) == 0) {
      s_best[threadIdx.x >> 5] = best;
      s_arg[threadIdx.x >> 5] = arg;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kUnmaskThreads / 32; ++w)
        if (s_best[w] > best || (s_best[w] == best && s_arg[w] < arg)) {
          best = s_best[w];
          arg = s_arg[w];
        }
      if (best >= 0.f) {         // a masked candidate is left
        s_pick[s_n++] = arg;
        s_conf[arg] = -2.0f;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const int n = s_n;
    for (int i = 1; i < n; ++i) {   // ascending positions (the kernels that follow expect sorted row lists)
      const int v = s_pick[i];
      int j = i - 1;
      while (j >= 0 && s_pick[j] > v) {
        s_pick[j + 1] = s_pick[j];
        --j;
      }
      s_pick[j + 1] = v;
    }
    for (int i = 0; i < n; ++i) {
      const int pos = start + s_pick[i];
      row[pos] = best_token[static_cast<int64_t>(b) * block_len + s_pick[i]];
      picked_pos[static_cast<int64_t>(b) * num_transfer + i] = pos;
    }
    for (int i = n; i < num_transfer; ++i)
      picked_pos[static_cast<int64_t>(b) * num_transfer + i] = -1;
    if (picked_count)
      picked_count[b] = n;
  }
}

constexpr int kConfThreads = 256;

__global__ void __launch_bounds__(kConfThreads)
row_confidence_kernel(const __nv_bfloat16* __restrict__ logits, int vocab, int64_t pitch,
                      float* __restrict__ conf, int64_t* __restrict__ token) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const __nv_bfloat16* row = logits + static_cast<int64_t>(blockIdx.x) * pitch;
  float m = -INFINITY, l = 0.f;
  int arg = 0;
  const int vecs = vocab / 8;
  const uint4* row4 = reinterpret_cast<const uint4*>(row);
  for (int v = threadIdx.x; v < vecs; v += kConfThreads) {
    const uint4 u = __ldg(row4 + v);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
    float x[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
    float vm = x[0];
    int va = 0;
#pragma unroll
    for (int i = 1; i < 8; ++i)
      if (x[i] > vm) {
        vm = x[i];
        va = i;
      }
    if (vm > m) {
      l *= __expf(m - vm);   // exp(-inf) = 0 on the first vector
      m = vm;
      arg = v * 8 + va;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      l += __expf(x[i] - m);
  }
  for (int j = vecs * 8 + threadIdx.x; j < vocab; j += kConfThreads) {   // tail when vocab % 8 != 0
    const float x = __bfloat162float(row[j]);
    if (x > m) {
      l *= __expf(m - x);
      m = x;
      arg = j;
    }
    l += __expf(x - m);
  }
  // merge: larger maximum wins, equal maxima keep the smaller index; sums are rescaled to the winner
  auto merge = [](float& m1, float& l1, int& a1, float m2, float l2, int a2) {
    if (m2 > m1 || (m2 == m1 && a2 < a1)) {
      const float t = m1; m1 = m2; m2 = t;
      const float tl = l1; l1 = l2; l2 = tl;
      a1 = a2;
    }
    l1 += (m2 == -INFINITY) ? 0.f : l2 * __expf(m2 - m1);
  };
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
    const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
    const int a2 = __shfl_xor_sync(0xffffffffu, arg, off);
    merge(m, l, arg, m2, l2, a2);
  }
  __shared__ float sm[kConfThreads / 32], sl[kConfThreads / 32];
  __shared__ int sa[kConfThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sm[warp] = m;
    sl[warp] = l;
    sa[warp] = arg;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kConfThreads / 32; ++w)
      merge(m, l, arg, sm[w], sl[w], sa[w]);
    conf[blockIdx.x] = l > 0.f ? 1.0f / l : 0.f;
    token[blockIdx.x] = arg;
  }
}

}  // namespace
}  // namespace dyllm

using namespace dyllm;

extern "C" {

int dyllm_add_rms_norm(const void* x, const void* residual_in, const void* weight, float eps, void* y,
                       void* residual_out, int rows, int width, void* stream) {
  return dyllm_add_rms_norm_segmented(x, rows > 0 ? rows : 1, rows > 0 ? rows : 1, residual_in, weight, eps, y,
                                      residual_out, rows, width, stream);
}

int dyllm_add_rms_norm_segmented(const void* x, int x_seg_rows, int64_t x_seg_pitch_rows, const void* residual_in,
                                 const void* weight, float eps, void* y, void* residual_out, int rows, int width,
                                 void* stream) {
  DYLLM_REQUIRE(rows >= 0 && width > 0, DYLLM_ERR_INVALID_ARGUMENT, "add_rms_norm: rows %d width %d", rows, width);
  DYLLM_REQUIRE(x_seg_rows > 0 && x_seg_pitch_rows >= x_seg_rows, DYLLM_ERR_INVALID_ARGUMENT,
                "add_rms_norm: segments of %d rows, %lld rows apart", x_seg_rows,
                static_cast<long long>(x_seg_pitch_rows));
  DYLLM_REQUIRE(width % 8 == 0 && width <= 8 * kNormThreads * 4, DYLLM_ERR_UNSUPPORTED,
                "add_rms_norm: width %d must be a multiple of 8 and at most %d", width, 8 * kNormThreads * 4);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && weight && y, DYLLM_ERR_INVALID_ARGUMENT, "add_rms_norm: null pointer");
  DYLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual_in) |
                  reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y) |
                  reinterpret_cast<uintptr_t>(residual_out)) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "add_rms_norm: buffers must be 16-byte aligned");
  const int vecs = width / 8;
  const int vpt = cdiv_i(vecs, kNormThreads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* xp = static_cast<const uint4*>(x);
  const uint4* rp = static_cast<const uint4*>(residual_in);
  const uint4* wp = static_cast<const uint4*>(weight);
  uint4* yp = static_cast<uint4*>(y);
  uint4* rop = static_cast<uint4*>(residual_out);
  const float inv = 1.0f / static_cast<float>(width);
  switch (vpt) {
    case 1: DYLLM_LAUNCH(add_rms_norm_kernel<1>, rows, kNormThreads, 0, s, xp, rp, wp, yp, rop, vecs, inv, eps, x_seg_rows, x_seg_pitch_rows); break;
    case 2: DYLLM_LAUNCH(add_rms_norm_kernel<2>, rows, kNormThreads, 0, s, xp, rp, wp, yp, rop, vecs, inv, eps, x_seg_rows, x_seg_pitch_rows); break;
    case 3: DYLLM_LAUNCH(add_rms_norm_kernel<3>, rows, kNormThreads, 0, s, xp, rp, wp, yp, rop, vecs, inv, eps, x_seg_rows, x_seg_pitch_rows); break;
    default: DYLLM_LAUNCH(add_rms_norm_kernel<4>, rows, kNormThreads, 0, s, xp, rp, wp, yp, rop, vecs, inv, eps, x_seg_rows, x_seg_pitch_rows); break;
  }
  return check_launch("add_rms_norm");
}

int dyllm_add_rms_norm_rows(const void* x, int x_seg_rows, int64_t x_seg_pitch_rows, const void* residual_in,
                            const void* weight, float eps, void* y_all, void* residual_out, int rows, int width,
                            const int32_t* sel_idx, int sel_max, const int32_t* sel_count_dev, void* y_sel,
                            void* stream) {
  DYLLM_REQUIRE(rows >= 0 && width > 0 && sel_max >= 0, DYLLM_ERR_INVALID_ARGUMENT, "add_rms_norm_rows: rows %d width %d",
                rows, width);
  DYLLM_REQUIRE(x_seg_rows > 0 && x_seg_pitch_rows >= x_seg_rows, DYLLM_ERR_INVALID_ARGUMENT,
                "add_rms_norm_rows: segments of %d rows, %lld rows apart", x_seg_rows,
                static_cast<long long>(x_seg_pitch_rows));
  DYLLM_REQUIRE(width % 8 == 0 && width <= 8 * kNormThreads * 4, DYLLM_ERR_UNSUPPORTED,
                "add_rms_norm_rows: width %d must be a multiple of 8 and at most %d", width, 8 * kNormThreads * 4);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && weight && (y_all || residual_out) && (sel_max == 0 || (sel_idx && y_sel)),
                DYLLM_ERR_INVALID_ARGUMENT, "add_rms_norm_rows: null pointer");
  DYLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual_in) |
                  reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y_sel) |
                  reinterpret_cast<uintptr_t>(y_all) | reinterpret_cast<uintptr_t>(residual_out)) & 15) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "add_rms_norm_rows: buffers must be 16-byte aligned");
  const int vecs = width / 8;
  const int vpt = cdiv_i(vecs, kNormThreads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* xp = static_cast<const uint4*>(x);
  const uint4* rp = static_cast<const uint4*>(residual_in);
  const uint4* wp = static_cast<const uint4*>(weight);
  uint4* yp = static_cast<uint4*>(y_sel);
  uint4* yap = static_cast<uint4*>(y_all);
  uint4* rop = static_cast<uint4*>(residual_out);
  const float inv = 1.0f / static_cast<float>(width);
  // the list is walked by at most 1024 blocks (each takes the entries blockIdx, blockIdx + n, ...)
  const int sel_blocks = sel_max < 1024 ? sel_max : 1024;
  const unsigned grid = static_cast<unsigned>(rows + sel_blocks);
#define DYLLM_NORM_ROWS(V)                                                                                         \
  DYLLM_LAUNCH(add_rms_norm_rows_kernel<V>, grid, kNormThreads, 0, s, xp, rp, wp, yap, yp, rop, rows, vecs, inv, eps,       \
                                                            x_seg_rows, x_seg_pitch_rows, sel_idx, sel_max,       \
                                                            sel_count_dev)
  switch (vpt) {
    case 1: DYLLM_NORM_ROWS(1); break;
    case 2: DYLLM_NORM_ROWS(2); break;
    case 3: DYLLM_NORM_ROWS(3); break;
    default: DYLLM_NORM_ROWS(4); break;
  }
#undef DYLLM_NORM_ROWS
  return check_launch("add_rms_norm_rows");
}

int dyllm_head_rms_norm(void* x, const void* weight, float eps, int rows, const int32_t* num_rows_dev, int heads,
                        int head_dim, void* stream) {
  DYLLM_REQUIRE(head_dim == 128, DYLLM_ERR_UNSUPPORTED, "head_rms_norm: head_dim %d (only 128 is built)", head_dim);
  DYLLM_REQUIRE(rows >= 0 && heads > 0, DYLLM_ERR_INVALID_ARGUMENT, "head_rms_norm: rows %d heads %d", rows, heads);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && weight, DYLLM_ERR_INVALID_ARGUMENT, "head_rms_norm: null pointer");
  DYLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight)) & 7) == 0,
                DYLLM_ERR_INVALID_ARGUMENT, "head_rms_norm: buffers must be 8-byte aligned");
  const int64_t vectors = static_cast<int64_t>(rows) * heads;
  const int64_t want = (vectors + 7) / 8;
  const int cap = sm_count() * 16;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  DYLLM_LAUNCH(head_rms_norm_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), static_cast<uint2*>(x),
               static_cast<const uint2*>(weight), rows, heads, eps, num_rows_dev);
  return check_launch("head_rms_norm");
}

int dyllm_rope_neox(void* x, const int64_t* positions, const int64_t* pos_idx, const float* cos_sin, int rows,
                    const int32_t* num_rows_dev, int heads, int head_dim, int max_pos, void* stream) {
  DYLLM_REQUIRE(head_dim == 128, DYLLM_ERR_UNSUPPORTED, "rope_neox: head_dim %d (only 128 is built)", head_dim);
  DYLLM_REQUIRE(rows >= 0 && heads > 0 && max_pos > 0, DYLLM_ERR_INVALID_ARGUMENT, "rope_neox: rows %d heads %d", rows,
                heads);
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(x && positions && cos_sin, DYLLM_ERR_INVALID_ARGUMENT, "rope_neox: null pointer");
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "rope_neox: x must be 16-byte aligned");
  const int64_t total = static_cast<int64_t>(rows) * heads * 8;
  int64_t want = cdiv_l(total, 256);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  DYLLM_LAUNCH(rope_neox_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), static_cast<uint4*>(x), positions, pos_idx,
                                                                        cos_sin, rows, heads, max_pos, num_rows_dev);
  return check_launch("rope_neox");
}

int dyllm_row_confidence(const void* logits, int rows, int vocab, int64_t pitch, float* conf, int64_t* token,
                         void* stream) {
  DYLLM_REQUIRE(rows >= 0 && vocab > 0 && pitch >= vocab, DYLLM_ERR_INVALID_ARGUMENT,
                "row_confidence: rows %d vocab %d pitch %lld", rows, vocab, static_cast<long long>(pitch));
  if (rows == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(logits && conf && token, DYLLM_ERR_INVALID_ARGUMENT, "row_confidence: null pointer");
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(logits) & 15) == 0 && pitch % 8 == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "row_confidence: rows must start on 16-byte boundaries");
  DYLLM_LAUNCH(row_confidence_kernel, rows, kConfThreads, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(logits), vocab, pitch, conf, token);
  return check_launch("row_confidence");
}

int dyllm_confidence_unmask(const float* conf, const int64_t* best_token, int64_t* tokens, int batch,
                            int64_t seq_pitch, const int64_t* step_counter, int steps_per_block, int num_blocks,
                            int prompt_len, int block_len, int num_transfer, int64_t mask_id, int64_t* picked_pos,
                            int32_t* picked_count, void* stream) {
  DYLLM_REQUIRE(batch >= 0 && block_len > 0 && block_len <= kUnmaskMaxBlock && num_transfer > 0 &&
                    num_transfer <= kUnmaskMaxPicks && num_transfer <= block_len,
                DYLLM_ERR_INVALID_ARGUMENT, "confidence_unmask: batch %d block %d (<= %d) picks %d (<= %d)", batch,
                block_len, kUnmaskMaxBlock, num_transfer, kUnmaskMaxPicks);
  DYLLM_REQUIRE(steps_per_block > 0 && num_blocks > 0 && prompt_len >= 0 &&
                    seq_pitch >= static_cast<int64_t>(prompt_len) + static_cast<int64_t>(num_blocks) * block_len,
                DYLLM_ERR_INVALID_ARGUMENT, "confidence_unmask: the blocks do not fit the token rows");
  if (batch == 0)
    return DYLLM_OK;
  DYLLM_REQUIRE(conf && best_token && tokens && picked_pos, DYLLM_ERR_INVALID_ARGUMENT, "confidence_unmask: null pointer");
  DYLLM_LAUNCH(confidence_unmask_kernel, batch, kUnmaskThreads, 0, static_cast<cudaStream_t>(stream), conf, best_token,
               tokens, seq_pitch, step_counter, steps_per_block, num_blocks, prompt_len, block_len, num_transfer, mask_id,
               picked_pos, picked_count);
  return check_launch("confidence_unmask");
}

}  // extern "C"
