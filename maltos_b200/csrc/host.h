// Host-side helpers shared by all launchers of the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MB_API extern "C" __attribute__((visibility("default")))

namespace mb {

// Device pointer to the status word of the CURRENT device (4 ints: code, block, detail, reserved).
int* status_ptr();
// Every launcher calls this once per kernel launch; exposed through mb_launch_count().
void count_launch(int n = 1);
// Makes the device's primary context current on the calling thread (first call per thread only).
void bind_context();
// Number of SMs of the current device (cached).
int sm_count();

// Encode a 2-D tiled bf16/fp32 tensor map (dim0 innermost). Returns false and records a message on failure.
bool encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                    uint32_t box0, uint32_t box1, int elem_bytes, bool swizzle128);
bool encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                    uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                    int elem_bytes, bool swizzle128);

bool encode_tmap_4d(CUtensorMap* out, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                    const uint32_t box[4], int elem_bytes, bool swizzle128);

void set_last_error(const char* msg);

}  // namespace mb

#define MB_CHECK_CUDA(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) {                                  \
      mb::set_last_error(cudaGetErrorString(_e));             \
      return static_cast<int>(_e);                            \
    }                                                         \
  } while (0)
