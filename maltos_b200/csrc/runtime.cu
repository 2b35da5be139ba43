// Library runtime: per-device status word, launch counter, tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), last-error string.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "host.h"

namespace mb {

__device__ int g_status_words[4];

static std::atomic<unsigned long long> g_launches{0};
static char g_last_error[512] = {0};
static std::mutex g_mu;

void set_last_error(const char* msg) {
  std::lock_guard<std::mutex> lk(g_mu);
  std::snprintf(g_last_error, sizeof(g_last_error), "%s", msg ? msg : "");
}

void bind_context() {
  // Launchers may be entered from a thread that has made no runtime call yet (autograd worker threads): the
  // driver-level tensor-map encoder needs the primary context current on the calling thread.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

void count_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

int* status_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_words) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

static CUtensorMapDataType dtype_of(int elem_bytes) {
  return elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
}

bool encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                    uint32_t box0, uint32_t box1, int elem_bytes, bool swizzle128) {
  bind_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {stride1_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    std::snprintf(buf, sizeof(buf),
                  "cuTensorMapEncodeTiled(2d) failed: %d (base=%p dims=%llu,%llu stride=%llu box=%u,%u)",
                  static_cast<int>(r), base, (unsigned long long)dim0, (unsigned long long)dim1,
                  (unsigned long long)stride1_bytes, box0, box1);
    set_last_error(buf);
    return false;
  }
  return true;
}

bool encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                    uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                    int elem_bytes, bool swizzle128) {
  bind_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  cuuint64_t dims[3] = {dim0, dim1, dim2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    std::snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled(3d) failed: %d", static_cast<int>(r));
    set_last_error(buf);
    return false;
  }
  return true;
}

// 4-D tiled map, used for [batch, token, head, dim] activations: dim0 = head_dim (innermost), dim1 = heads, dim2 = tokens,
// dim3 = batch. A box of {64, 1, rows, 1} is one head's [rows x 64] tile; rows past the end of a batch read as zero.
bool encode_tmap_4d(CUtensorMap* out, const void* base, const uint64_t dims_in[4], const uint64_t strides_bytes[3],
                    const uint32_t box_in[4], int elem_bytes, bool swizzle128) {
  bind_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  cuuint64_t dims[4] = {dims_in[0], dims_in[1], dims_in[2], dims_in[3]};
  cuuint64_t strides[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t box[4] = {box_in[0], box_in[1], box_in[2], box_in[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes), 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    std::snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled(4d) failed: %d", static_cast<int>(r));
    set_last_error(buf);
    return false;
  }
  return true;
}

}  // namespace mb

// ------------------------------------------------------------------ exported C API
MB_API const char* mb_last_error() { return mb::g_last_error; }

MB_API unsigned long long mb_launch_count() { return mb::g_launches.load(std::memory_order_relaxed); }

// Reads the status word of the current device after synchronising `stream`, then clears it.
// out[0] = OR of error codes seen since the last call, out[1] = a block index, out[2] = detail.
MB_API int mb_status_fetch_and_clear(int* out4, cudaStream_t stream) {
  int* p = mb::status_ptr();
  if (!p) return -1;
  MB_CHECK_CUDA(cudaMemcpyAsync(out4, p, 4 * sizeof(int), cudaMemcpyDeviceToHost, stream));
  MB_CHECK_CUDA(cudaMemsetAsync(p, 0, 3 * sizeof(int), stream));   // word 3 holds the wait limit and is kept
  MB_CHECK_CUDA(cudaStreamSynchronize(stream));
  return 0;
}

// Limit of every bounded device-side wait in milliseconds on the current device (0 restores the default of 4 s).
MB_API int mb_set_wait_timeout_ms(int ms) {
  int* p = mb::status_ptr();
  if (!p) return -1;
  if (ms < 0) ms = 0;
  MB_CHECK_CUDA(cudaMemcpy(p + 3, &ms, sizeof(int), cudaMemcpyHostToDevice));
  return 0;
}

MB_API int mb_sm_count() { return mb::sm_count(); }
