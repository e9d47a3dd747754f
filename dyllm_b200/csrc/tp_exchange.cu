// Tensor-parallel SUM exchange over peer memory (NVLink): the small all-reduces of a sparse step.
//
// The reference all-reduces three tensors per sparse layer with NCCL: the 12-byte-per-token statistics
// (dyllm/distributed/parallel_state.py:60-61), the row-parallel o_proj output and the row-parallel
// down-projection / expert output of the salient rows (dyllm/model_executor/layers/linear.py:216-220,
// dyllm/model_executor/models/lladamoe.py:103-104,141).  The first and the last are small and their
// size is only known on the device (the salient count), so here they are exchanged by two kernels that
// read the count themselves and can sit inside a captured CUDA graph:
//
//   push    every rank stores its partial rows into its own slot of EVERY rank's region (plain 16-byte
//           stores through peer pointers; no loads from peer memory, no multicast), then raises its flag
//           in every region;
//   reduce  every rank waits (bounded) for all flags of its own region, adds the world_size slots of its
//           region in rank order in fp32 (so every rank computes bit-identical sums) and writes the rows
//           to their destination (optionally scattered through a row map: the FFN-output cache).
//
// Region of one rank (same layout everywhere; `slot` = slot_bytes):
//   [0]     uint32 epoch        number of completed exchanges (local use only)
//   [4]     uint32 push ticket  [8] uint32 reduce ticket
//   [64]    uint32 flags[2][8]  flags[parity][source rank] = epoch + 1 of the exchange whose data is complete
//   [128]   int32 counts[2][8]  rows the source rank contributed (row gathers only)
//   [1024]  data[2][world][slot]
// Exchange e uses the buffers of parity e & 1.  A rank can start pushing exchange e + 2 (same parity) only
// after it has finished reducing e + 1, for which every rank had to push e + 1, which each of them does
// after it finished reducing e: so nobody still reads the buffer that is being overwritten.
//
// Sequence-sharded layout (every rank runs attention and the all-row projections for its own sequences, the
// FFN weights are sharded over the ranks): two more exchanges built from the same pieces.
//   gather   every rank stores its salient (normed) rows and their count into its slot of every region; a
//            one-block kernel then waits for the flags and writes the list of all gathered rows in rank order
//            (as row numbers of the data area, so that the gathered GEMM reads them in place), the per-rank
//            prefix counts and the total;
//   scatter  every rank stores each partial FFN output row into its slot of the OWNER's region only; the
//            owner adds the slots in rank order (the reduce kernel above) and scatters into its cache.
#include <cstring>

#include "common.cuh"

namespace dyllm {
namespace {

constexpr int kTpMaxWorld = 8;
constexpr size_t kTpHeaderBytes = 1024;
constexpr size_t kTpFlagsOffset = 64;
constexpr size_t kTpCountsOffset = 128;
constexpr int kTpThreads = 256;
constexpr int kTpStatusBase = 0x7E00;   // device status code of a flag wait that ran out: base + source rank

struct TpComm {
  int rank = 0, world = 1, device = 0;
  size_t slot_bytes = 0, region_bytes = 0;
  unsigned char* local = nullptr;
  unsigned char* peers[kTpMaxWorld] = {nullptr};
  bool ipc_opened[kTpMaxWorld] = {false};
  unsigned char** peers_dev = nullptr;   // device copy of peers[]
  unsigned long long wait_ns = 2000000000ull;   // a flag wait gives up after this long
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ size_t data_offset(uint32_t parity, int world, int src_rank, size_t slot_bytes) {
  return kTpHeaderBytes + (static_cast<size_t>(parity) * world + src_rank) * slot_bytes;
}

__device__ __forceinline__ int live_rows(const int32_t* count_dev, int row_offset, int max_rows) {
  if (!count_dev)
    return max_rows;
  const int n = *count_dev - row_offset;
  return n < 0 ? 0 : (n > max_rows ? max_rows : n);
}

// VecT = uint4 (rows of bf16, row_vecs 16-byte vectors each) or uint32_t (a flat fp32 vector).
template <typename VecT>
__global__ void __launch_bounds__(kTpThreads)
tp_push_kernel(unsigned char* const* __restrict__ peers, int rank, int world, size_t slot_bytes,
               const VecT* __restrict__ src, int row_vecs, int max_rows, const int32_t* __restrict__ count_dev,
               int row_offset) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  unsigned char* local = peers[rank];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(local);
  const uint32_t parity = epoch & 1u;
  const int rows = live_rows(count_dev, row_offset, max_rows);
  const int64_t total = static_cast<int64_t>(rows) * row_vecs;
  const size_t off = data_offset(parity, world, rank, slot_bytes);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const VecT v = src[i];
#pragma unroll 1
    for (int k = 0; k < world; ++k) {
      int p = rank + 1 + k;          // start with the next rank so that the ranks do not all hit one peer first
      p = p >= world ? p - world : p;
      reinterpret_cast<VecT*>(peers[p] + off)[i] = v;
    }
  }
  // publish: all stores of the grid, then the flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* ticket = reinterpret_cast<uint32_t*>(local + 4);
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      *ticket = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        st_release_sys(reinterpret_cast<uint32_t*>(peers[p] + kTpFlagsOffset) + parity * kTpMaxWorld + rank, epoch + 1u);
    }
  }
}

// Waits until every source rank's flag of this exchange is up.  Returns false if a wait ran out.
__device__ __forceinline__ bool wait_flags(unsigned char* local, uint32_t parity, uint32_t want, int world,
                                           unsigned long long wait_ns, int* status_word) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0)
    ok_sh = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(local + kTpFlagsOffset) + parity * kTpMaxWorld + threadIdx.x;
    const unsigned long long t0 = now_ns();
    bool up = false;
    for (uint32_t spin = 0; spin < (1u << 30); ++spin) {
      if (ld_acquire_sys(flag) == want) {
        up = true;
        break;
      }
      if ((spin & 63u) == 63u && now_ns() - t0 > wait_ns)
        break;
      __nanosleep(64);
    }
    if (!up) {
      ok_sh = 0;
      if (status_word)
        atomicCAS(status_word, 0, kTpStatusBase + static_cast<int>(threadIdx.x));
    }
  }
  __syncthreads();
  return ok_sh != 0;
}

__device__ __forceinline__ void finish_exchange(unsigned char* local, uint32_t epoch) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ticket = reinterpret_cast<uint32_t*>(local + 8);
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      *ticket = 0;
      *reinterpret_cast<volatile uint32_t*>(local) = epoch + 1u;
    }
  }
}

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__global__ void __launch_bounds__(kTpThreads)
tp_reduce_rows_kernel(unsigned char* local, int world, size_t slot_bytes, int row_vecs, int max_rows,
                      const int32_t* __restrict__ count_dev, int row_offset, uint4* __restrict__ out, int64_t ldo_vecs,
                      const int32_t* __restrict__ out_row_map, unsigned long long wait_ns, int* status_word) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(local);
  const uint32_t parity = epoch & 1u;
  const bool ok = wait_flags(local, parity, epoch + 1u, world, wait_ns, status_word);
  if (ok) {
    const int rows = live_rows(count_dev, row_offset, max_rows);
    const int64_t total = static_cast<int64_t>(rows) * row_vecs;
    const unsigned char* base = local + data_offset(parity, world, 0, slot_bytes);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int m = static_cast<int>(i / row_vecs);
      const int c = static_cast<int>(i - static_cast<int64_t>(m) * row_vecs);
      const int dst = out_row_map ? out_row_map[row_offset + m] : row_offset + m;
      if (dst < 0)
        continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < world; ++p)     // rank order: the same sum on every rank
        add8(acc, reinterpret_cast<const uint4*>(base + static_cast<size_t>(p) * slot_bytes)[i]);
      uint4 r;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        q[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      out[static_cast<int64_t>(dst) * ldo_vecs + c] = r;
    }
  }
  finish_exchange(local, epoch);
}

// Gather push: row m of the local list (x[idx[m]], idx null = identity) goes to slot `rank` of every region,
// together with the number of rows.
__global__ void __launch_bounds__(kTpThreads)
tp_gather_push_kernel(unsigned char* const* __restrict__ peers, int rank, int world, size_t slot_bytes,
                      const uint4* __restrict__ x, int64_t ldx_vecs, const int32_t* __restrict__ idx, int x_rows,
                      int row_vecs, int max_rows, const int32_t* __restrict__ count_dev) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  unsigned char* local = peers[rank];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(local);
  const uint32_t parity = epoch & 1u;
  const int rows = live_rows(count_dev, 0, max_rows);
  const int64_t total = static_cast<int64_t>(rows) * row_vecs;
  const size_t off = data_offset(parity, world, rank, slot_bytes);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / row_vecs);
    const int c = static_cast<int>(i - static_cast<int64_t>(m) * row_vecs);
    int r = idx ? idx[m] : m;
    r = r < 0 ? 0 : (r >= x_rows ? x_rows - 1 : r);
    const uint4 v = x[static_cast<int64_t>(r) * ldx_vecs + c];
#pragma unroll 1
    for (int k = 0; k < world; ++k) {
      int p = rank + 1 + k;
      p = p >= world ? p - world : p;
      reinterpret_cast<uint4*>(peers[p] + off)[i] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* ticket = reinterpret_cast<uint32_t*>(local + 4);
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      *ticket = 0;
      for (int p = 0; p < world; ++p)
        reinterpret_cast<volatile int32_t*>(peers[p] + kTpCountsOffset)[parity * kTpMaxWorld + rank] = rows;
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        st_release_sys(reinterpret_cast<uint32_t*>(peers[p] + kTpFlagsOffset) + parity * kTpMaxWorld + rank, epoch + 1u);
    }
  }
}

// One block: waits for every rank's rows, then writes prefix[0..world] (rows of the ranks before r), the total
// and, for every gathered row in rank order, its row number inside the data area (both parities form one
// [2 * world * slot_rows, width] matrix that starts right after the header).
__global__ void __launch_bounds__(kTpThreads)
tp_gather_finish_kernel(unsigned char* local, int world, size_t slot_bytes, int slot_rows, int32_t* __restrict__ idx_all,
                        int32_t* __restrict__ prefix, int32_t* __restrict__ total_out, unsigned long long wait_ns,
                        int* status_word) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  __shared__ int pre[kTpMaxWorld + 1];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(local);
  const uint32_t parity = epoch & 1u;
  const bool ok = wait_flags(local, parity, epoch + 1u, world, wait_ns, status_word);
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int r = 0; r < world; ++r) {
      pre[r] = acc;
      int c = ok ? reinterpret_cast<volatile int32_t*>(local + kTpCountsOffset)[parity * kTpMaxWorld + r] : 0;
      c = c < 0 ? 0 : (c > slot_rows ? slot_rows : c);
      acc += c;
    }
    pre[world] = acc;
    for (int r = 0; r <= world; ++r)
      prefix[r] = pre[r];
    *total_out = acc;
  }
  __syncthreads();
  for (int r = 0; r < world; ++r) {
    const int n = pre[r + 1] - pre[r];
    const int base = (static_cast<int>(parity) * world + r) * slot_rows;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
      idx_all[pre[r] + j] = base + j;
  }
  finish_exchange(local, epoch);
}

// Scatter push: row m of y (a row of rank r = the rank whose prefix range holds m) goes to slot `rank` of
// rank r's region, at its position inside r's own list.
__global__ void __launch_bounds__(kTpThreads)
tp_scatter_push_kernel(unsigned char* const* __restrict__ peers, int rank, int world, size_t slot_bytes,
                       const uint4* __restrict__ y, int row_vecs, int max_rows, const int32_t* __restrict__ prefix) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  unsigned char* local = peers[rank];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(local);
  const uint32_t parity = epoch & 1u;
  __shared__ int pre[kTpMaxWorld + 1];
  if (threadIdx.x <= world)
    pre[threadIdx.x] = prefix[threadIdx.x];
  __syncthreads();
  int rows = pre[world];
  rows = rows > max_rows ? max_rows : rows;
  const int64_t total = static_cast<int64_t>(rows) * row_vecs;
  const size_t off = data_offset(parity, world, rank, slot_bytes);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / row_vecs);
    const int c = static_cast<int>(i - static_cast<int64_t>(m) * row_vecs);
    int owner = 0;
    while (owner + 1 < world && pre[owner + 1] <= m)
      ++owner;
    const int64_t j = static_cast<int64_t>(m - pre[owner]) * row_vecs + c;
    reinterpret_cast<uint4*>(peers[owner] + off)[j] = y[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* ticket = reinterpret_cast<uint32_t*>(local + 4);
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      *ticket = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        st_release_sys(reinterpret_cast<uint32_t*>(peers[p] + kTpFlagsOffset) + parity * kTpMaxWorld + rank, epoch + 1u);
    }
  }
}

__global__ void __launch_bounds__(kTpThreads)
tp_reduce_f32_kernel(unsigned char* local, int world, size_t slot_bytes, float* __restrict__ out, int n,
                     unsigned long long wait_ns, int* status_word) {
  pdl_wait();      // programmatic dependent launch: nothing before this reads an earlier kernel's data
  pdl_trigger();
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(local);
  const uint32_t parity = epoch & 1u;
  const bool ok = wait_flags(local, parity, epoch + 1u, world, wait_ns, status_word);
  if (ok) {
    const unsigned char* base = local + data_offset(parity, world, 0, slot_bytes);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
      float acc = 0.f;
      for (int p = 0; p < world; ++p)
        acc += reinterpret_cast<const float*>(base + static_cast<size_t>(p) * slot_bytes)[i];
      out[i] = acc;
    }
  }
  finish_exchange(local, epoch);
}

TpComm* as_comm(void* c) { return static_cast<TpComm*>(c); }

int upload_peers(TpComm* c) {
  if (cudaMemcpy(c->peers_dev, c->peers, sizeof(c->peers), cudaMemcpyHostToDevice) != cudaSuccess)
    return set_error(DYLLM_ERR_CUDA, "tp_comm: copying the peer table failed: %s", cudaGetErrorString(cudaGetLastError()));
  return DYLLM_OK;
}

int grid_for(int64_t items) {
  // at most one resident wave: the tickets assume that every block of a launch gets to run
  const int64_t blocks = (items + kTpThreads - 1) / kTpThreads;
  const int cap = sm_count() * 4;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace dyllm

using namespace dyllm;

extern "C" {

int dyllm_tp_comm_create(int rank, int world, size_t slot_bytes, void** comm_out) {
  DYLLM_REQUIRE(comm_out, DYLLM_ERR_INVALID_ARGUMENT, "tp_comm_create: null output");
  DYLLM_REQUIRE(world >= 1 && world <= kTpMaxWorld && rank >= 0 && rank < world, DYLLM_ERR_INVALID_ARGUMENT,
                "tp_comm_create: rank %d of %d (at most %d ranks)", rank, world, kTpMaxWorld);
  DYLLM_REQUIRE(slot_bytes >= 16 && slot_bytes % 256 == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "tp_comm_create: slot_bytes %zu must be a positive multiple of 256", slot_bytes);
  TpComm* c = new TpComm();
  c->rank = rank;
  c->world = world;
  c->slot_bytes = slot_bytes;
  c->region_bytes = kTpHeaderBytes + 2 * static_cast<size_t>(world) * slot_bytes;
  cudaGetDevice(&c->device);
  cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&c->local), c->region_bytes);
  if (err == cudaSuccess)
    err = cudaMemset(c->local, 0, kTpHeaderBytes);
  if (err == cudaSuccess)
    err = cudaMalloc(reinterpret_cast<void**>(&c->peers_dev), sizeof(c->peers));
  if (err == cudaSuccess)
    err = cudaDeviceSynchronize();
  if (err != cudaSuccess) {
    const int rc = set_error(DYLLM_ERR_CUDA, "tp_comm_create: allocating %zu bytes failed: %s", c->region_bytes,
                             cudaGetErrorString(err));
    cudaFree(c->local);
    cudaFree(c->peers_dev);
    delete c;
    return rc;
  }
  c->peers[rank] = c->local;
  *comm_out = c;
  return DYLLM_OK;
}

size_t dyllm_tp_comm_region_bytes(void* comm) { return comm ? as_comm(comm)->region_bytes : 0; }

void* dyllm_tp_comm_region(void* comm) { return comm ? as_comm(comm)->local : nullptr; }

int dyllm_tp_comm_ipc_handle(void* comm, void* handle64) {
  DYLLM_REQUIRE(comm && handle64, DYLLM_ERR_INVALID_ARGUMENT, "tp_comm_ipc_handle: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
  cudaIpcMemHandle_t h;
  const cudaError_t err = cudaIpcGetMemHandle(&h, as_comm(comm)->local);
  DYLLM_REQUIRE(err == cudaSuccess, DYLLM_ERR_CUDA, "tp_comm_ipc_handle: cudaIpcGetMemHandle failed: %s",
                cudaGetErrorString(err));
  memcpy(handle64, &h, 64);
  return DYLLM_OK;
}

int dyllm_tp_comm_open_ipc(void* comm, const void* handles) {
  DYLLM_REQUIRE(comm && handles, DYLLM_ERR_INVALID_ARGUMENT, "tp_comm_open_ipc: null pointer");
  TpComm* c = as_comm(comm);
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank)
      continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const unsigned char*>(handles) + 64 * p, 64);
    void* ptr = nullptr;
    const cudaError_t err = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    DYLLM_REQUIRE(err == cudaSuccess && ptr, DYLLM_ERR_CUDA, "tp_comm_open_ipc: opening the region of rank %d failed: %s",
                  p, cudaGetErrorString(err));
    c->peers[p] = static_cast<unsigned char*>(ptr);
    c->ipc_opened[p] = true;
  }
  return upload_peers(c);
}

int dyllm_tp_comm_open_local(void* comm, void* const* regions) {
  DYLLM_REQUIRE(comm && regions, DYLLM_ERR_INVALID_ARGUMENT, "tp_comm_open_local: null pointer");
  TpComm* c = as_comm(comm);
  for (int p = 0; p < c->world; ++p) {
    DYLLM_REQUIRE(regions[p], DYLLM_ERR_INVALID_ARGUMENT, "tp_comm_open_local: region %d is null", p);
    if (p != c->rank)
      c->peers[p] = static_cast<unsigned char*>(regions[p]);
  }
  return upload_peers(c);
}

int dyllm_tp_comm_set_wait_ms(void* comm, int milliseconds) {
  DYLLM_REQUIRE(comm && milliseconds > 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_comm_set_wait_ms: bad argument");
  as_comm(comm)->wait_ns = static_cast<unsigned long long>(milliseconds) * 1000000ull;
  return DYLLM_OK;
}

int dyllm_tp_comm_destroy(void* comm) {
  if (!comm)
    return DYLLM_OK;
  TpComm* c = as_comm(comm);
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p)
    if (c->ipc_opened[p])
      cudaIpcCloseMemHandle(c->peers[p]);
  cudaFree(c->peers_dev);
  cudaFree(c->local);
  delete c;
  return DYLLM_OK;
}

int dyllm_tp_push_rows(void* comm, const void* src, int width, int max_rows, const int32_t* count_dev,
                       int row_offset, void* stream) {
  DYLLM_REQUIRE(comm && src, DYLLM_ERR_INVALID_ARGUMENT, "tp_push_rows: null pointer");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(width > 0 && width % 8 == 0 && max_rows >= 0 && row_offset >= 0, DYLLM_ERR_INVALID_ARGUMENT,
                "tp_push_rows: width %d (multiple of 8) max_rows %d row_offset %d", width, max_rows, row_offset);
  DYLLM_REQUIRE(static_cast<size_t>(max_rows) * width * 2 <= c->slot_bytes, DYLLM_ERR_WORKSPACE,
                "tp_push_rows: %d rows of %d bf16 exceed the slot of %zu bytes", max_rows, width, c->slot_bytes);
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_push_rows: src must be 16-byte aligned");
  const int row_vecs = width / 8;
  DYLLM_LAUNCH(tp_push_kernel<uint4>, grid_for(static_cast<int64_t>(max_rows) * row_vecs), kTpThreads, 0, static_cast<cudaStream_t>(stream), c->peers_dev, c->rank, c->world, c->slot_bytes,
                                                                static_cast<const uint4*>(src), row_vecs, max_rows,
                                                                count_dev, row_offset);
  return check_launch("tp_push_rows");
}

int dyllm_tp_reduce_rows(void* comm, int width, int max_rows, const int32_t* count_dev, int row_offset, void* out,
                         int64_t ldo, const int32_t* out_row_map, void* stream) {
  DYLLM_REQUIRE(comm && out, DYLLM_ERR_INVALID_ARGUMENT, "tp_reduce_rows: null pointer");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(width > 0 && width % 8 == 0 && ldo % 8 == 0 && ldo >= width && max_rows >= 0 && row_offset >= 0,
                DYLLM_ERR_INVALID_ARGUMENT, "tp_reduce_rows: width %d ldo %lld max_rows %d", width,
                static_cast<long long>(ldo), max_rows);
  DYLLM_REQUIRE(static_cast<size_t>(max_rows) * width * 2 <= c->slot_bytes, DYLLM_ERR_WORKSPACE,
                "tp_reduce_rows: %d rows of %d bf16 exceed the slot of %zu bytes", max_rows, width, c->slot_bytes);
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_reduce_rows: out must be 16-byte aligned");
  const int row_vecs = width / 8;
  DYLLM_LAUNCH(tp_reduce_rows_kernel, grid_for(static_cast<int64_t>(max_rows) * row_vecs), kTpThreads, 0, static_cast<cudaStream_t>(stream), c->local, c->world, c->slot_bytes, row_vecs, max_rows,
                                                                count_dev, row_offset, static_cast<uint4*>(out), ldo / 8,
                                                                out_row_map, c->wait_ns, device_status_word());
  return check_launch("tp_reduce_rows");
}

int dyllm_tp_allreduce_rows(void* comm, const void* src, int width, int max_rows, const int32_t* count_dev,
                            int row_offset, void* out, int64_t ldo, const int32_t* out_row_map, void* stream) {
  const int rc = dyllm_tp_push_rows(comm, src, width, max_rows, count_dev, row_offset, stream);
  if (rc != DYLLM_OK)
    return rc;
  return dyllm_tp_reduce_rows(comm, width, max_rows, count_dev, row_offset, out, ldo, out_row_map, stream);
}

int dyllm_tp_gather_rows(void* comm, const void* x, int x_rows, int width, int64_t ldx, const int32_t* idx,
                         int max_rows, const int32_t* count_dev, int32_t* idx_all, int32_t* prefix,
                         int32_t* total_out, void* stream) {
  DYLLM_REQUIRE(comm && x && idx_all && prefix && total_out, DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_rows: null pointer");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(width > 0 && width % 8 == 0 && ldx % 8 == 0 && ldx >= width && max_rows >= 0 && x_rows > 0,
                DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_rows: width %d ldx %lld max_rows %d x_rows %d", width,
                static_cast<long long>(ldx), max_rows, x_rows);
  const size_t row_bytes = static_cast<size_t>(width) * 2;
  DYLLM_REQUIRE(c->slot_bytes % row_bytes == 0, DYLLM_ERR_INVALID_ARGUMENT,
                "tp_gather_rows: the slot of %zu bytes is not a whole number of %zu-byte rows", c->slot_bytes, row_bytes);
  DYLLM_REQUIRE(static_cast<size_t>(max_rows) * row_bytes <= c->slot_bytes, DYLLM_ERR_WORKSPACE,
                "tp_gather_rows: %d rows of %d bf16 exceed the slot of %zu bytes", max_rows, width, c->slot_bytes);
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_rows: x must be 16-byte aligned");
  const int row_vecs = width / 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DYLLM_LAUNCH(tp_gather_push_kernel, grid_for(static_cast<int64_t>(max_rows) * row_vecs), kTpThreads, 0, st, 
      c->peers_dev, c->rank, c->world, c->slot_bytes, static_cast<const uint4*>(x), ldx / 8, idx, x_rows, row_vecs,
      max_rows, count_dev);
  int rc = check_launch("tp_gather_push");
  if (rc != DYLLM_OK)
    return rc;
  DYLLM_LAUNCH(tp_gather_finish_kernel, 1, kTpThreads, 0, st, c->local, c->world, c->slot_bytes,
                                                   static_cast<int>(c->slot_bytes / row_bytes), idx_all, prefix,
                                                   total_out, c->wait_ns, device_status_word());
  return check_launch("tp_gather_finish");
}

int dyllm_tp_gather_push(void* comm, const void* x, int x_rows, int width, int64_t ldx, const int32_t* idx,
                         int max_rows, const int32_t* count_dev, void* stream) {
  DYLLM_REQUIRE(comm && x, DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_push: null pointer");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(width > 0 && width % 8 == 0 && ldx % 8 == 0 && ldx >= width && max_rows >= 0 && x_rows > 0 &&
                    static_cast<size_t>(max_rows) * width * 2 <= c->slot_bytes,
                DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_push: bad shape");
  const int row_vecs = width / 8;
  DYLLM_LAUNCH(tp_gather_push_kernel, grid_for(static_cast<int64_t>(max_rows) * row_vecs), kTpThreads, 0, static_cast<cudaStream_t>(stream), c->peers_dev, c->rank, c->world, c->slot_bytes,
                                                                static_cast<const uint4*>(x), ldx / 8, idx, x_rows,
                                                                row_vecs, max_rows, count_dev);
  return check_launch("tp_gather_push");
}

int dyllm_tp_gather_finish(void* comm, int width, int32_t* idx_all, int32_t* prefix, int32_t* total_out, void* stream) {
  DYLLM_REQUIRE(comm && idx_all && prefix && total_out && width > 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_finish: bad argument");
  TpComm* c = as_comm(comm);
  const size_t row_bytes = static_cast<size_t>(width) * 2;
  DYLLM_REQUIRE(c->slot_bytes % row_bytes == 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_gather_finish: slot is not a whole number of rows");
  DYLLM_LAUNCH(tp_gather_finish_kernel, 1, kTpThreads, 0, static_cast<cudaStream_t>(stream), 
      c->local, c->world, c->slot_bytes, static_cast<int>(c->slot_bytes / row_bytes), idx_all, prefix, total_out,
      c->wait_ns, device_status_word());
  return check_launch("tp_gather_finish");
}

void* dyllm_tp_comm_data(void* comm) { return comm ? as_comm(comm)->local + kTpHeaderBytes : nullptr; }

int dyllm_tp_scatter_push(void* comm, const void* y, int width, int max_rows, const int32_t* prefix, void* stream) {
  DYLLM_REQUIRE(comm && y && prefix, DYLLM_ERR_INVALID_ARGUMENT, "tp_scatter_push: null pointer");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(width > 0 && width % 8 == 0 && max_rows >= 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_scatter_push: width %d max_rows %d",
                width, max_rows);
  DYLLM_REQUIRE((reinterpret_cast<uintptr_t>(y) & 15) == 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_scatter_push: y must be 16-byte aligned");
  const int row_vecs = width / 8;
  DYLLM_LAUNCH(tp_scatter_push_kernel, grid_for(static_cast<int64_t>(max_rows) * row_vecs), kTpThreads, 0, static_cast<cudaStream_t>(stream), c->peers_dev, c->rank, c->world, c->slot_bytes,
                                                                 static_cast<const uint4*>(y), row_vecs, max_rows, prefix);
  return check_launch("tp_scatter_push");
}

int dyllm_tp_push_f32(void* comm, const float* src, int n, void* stream) {
  DYLLM_REQUIRE(comm && src && n >= 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_push_f32: bad argument");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(static_cast<size_t>(n) * 4 <= c->slot_bytes, DYLLM_ERR_WORKSPACE,
                "tp_push_f32: %d values exceed the slot of %zu bytes", n, c->slot_bytes);
  DYLLM_LAUNCH(tp_push_kernel<uint32_t>, grid_for(n), kTpThreads, 0, static_cast<cudaStream_t>(stream), 
      c->peers_dev, c->rank, c->world, c->slot_bytes, reinterpret_cast<const uint32_t*>(src), 1, n, nullptr, 0);
  return check_launch("tp_push_f32");
}

int dyllm_tp_reduce_f32(void* comm, float* out, int n, void* stream) {
  DYLLM_REQUIRE(comm && out && n >= 0, DYLLM_ERR_INVALID_ARGUMENT, "tp_reduce_f32: bad argument");
  TpComm* c = as_comm(comm);
  DYLLM_REQUIRE(static_cast<size_t>(n) * 4 <= c->slot_bytes, DYLLM_ERR_WORKSPACE,
                "tp_reduce_f32: %d values exceed the slot of %zu bytes", n, c->slot_bytes);
  DYLLM_LAUNCH(tp_reduce_f32_kernel, grid_for(n), kTpThreads, 0, static_cast<cudaStream_t>(stream), 
      c->local, c->world, c->slot_bytes, out, n, c->wait_ns, device_status_word());
  return check_launch("tp_reduce_f32");
}

int dyllm_tp_allreduce_f32(void* comm, float* inout, int n, void* stream) {
  const int rc = dyllm_tp_push_f32(comm, inout, n, stream);
  if (rc != DYLLM_OK)
    return rc;
  return dyllm_tp_reduce_f32(comm, inout, n, stream);
}

}  // extern "C"
