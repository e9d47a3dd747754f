// Host-side runtime pieces shared by every entry point: thread-local error text, per-device
// properties, the device status word written by bounded waits, and tensor-map encoding.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace dyllm {

namespace {
thread_local char g_error[512] = {0};
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
int* g_status_word[kMaxDevices] = {nullptr};
int* g_split_tickets_ptr[kMaxDevices] = {nullptr};
std::mutex g_mutex;
// One status word per device that loads this library (zero-initialised by the loader).
__device__ int g_device_status = 0;
// Arrival counters of the split-K GEMMs (one per output tile): zero between launches; the last CTA to
// arrive at a tile adds the splits' partial sums and resets the counter.
__device__ int g_split_tickets[kSplitTicketCount] = {0};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev < 0 || dev >= kMaxDevices ? 0 : dev;
}

EncodeTiledFn encode_fn() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_encode)
    return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("DYLLM_PDL");
    return v && v[0] == '1';
  }();
  return on;
}

int set_error(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(DYLLM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return DYLLM_OK;
}

int sm_count() {
  const int dev = current_device();
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

int* device_status_word() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status_word[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess)
      return nullptr;
    g_status_word[dev] = static_cast<int*>(p);
  }
  return g_status_word[dev];
}

int* split_tickets() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_split_tickets_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_split_tickets) != cudaSuccess)
      return nullptr;
    g_split_tickets_ptr[dev] = static_cast<int*>(p);
  }
  return g_split_tickets_ptr[dev];
}

int read_and_clear_device_status() {
  int* word = device_status_word();
  if (!word)
    return 0;
  int value = 0;
  if (cudaDeviceSynchronize() != cudaSuccess)
    return -1;
  cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost);
  if (value != 0)
    cudaMemset(word, 0, sizeof(int));
  return value;
}

int encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                        uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn)
    return set_error(DYLLM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                    elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return set_error(DYLLM_ERR_CUDA,
                     "cuTensorMapEncodeTiled(2d) failed with %d (base %p rows %llu cols %llu pitch %llu box %ux%u)",
                     static_cast<int>(res), base, (unsigned long long)rows, (unsigned long long)cols,
                     (unsigned long long)pitch_elems, box_rows, box_cols);
  return DYLLM_OK;
}

int encode_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1,
                        uint32_t box2, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn)
    return set_error(DYLLM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                    elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return set_error(DYLLM_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed with %d", static_cast<int>(res));
  return DYLLM_OK;
}

}  // namespace dyllm

extern "C" {

int dyllm_version(void) { return 100; }

const char* dyllm_last_error(void) { return dyllm::g_error; }

int dyllm_device_status(void) { return dyllm::read_and_clear_device_status(); }

}  // extern "C"
