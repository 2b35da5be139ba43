// Contiguous copy between this GPU's memory and a peer's CUDA-IPC mapping (either side may be the peer) with plain
// 16-byte loads and stores, eight in flight per thread. Used where a whole remote block is fetched while other work
// runs on another stream (ring attention pulls the next K/V block, pushes its dK/dV contribution to the owner's slot).
// The kernel never waits on another GPU; callers order it with stream-ordered group barriers.
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 8;

__global__ void __launch_bounds__(kCopyThreads)
peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec, unsigned char* dst_tail,
                 const unsigned char* src_tail, int tail_bytes) {
  const long long stride = static_cast<long long>(gridDim.x) * kCopyThreads;
  long long i = static_cast<long long>(blockIdx.x) * kCopyThreads + threadIdx.x;
  for (; i + (kCopyUnroll - 1) * stride < nvec; i += kCopyUnroll * stride) {
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < nvec; i += stride) dst[i] = src[i];
  if (blockIdx.x == 0 && threadIdx.x < tail_bytes) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

// Gather: `world` equally sized pieces, piece r read from srcs.p[r] (this GPU's or a peer's memory), written back to
// back into dst. blockIdx.y = piece. Used by the sharded-parameter gather: every rank pulls the other ranks' shards
// straight from where their optimizers keep them, without a rendezvous.
struct GatherSrcs {
  const void* p[16];
};
__global__ void __launch_bounds__(kCopyThreads)
peer_gather_kernel(uint4* __restrict__ dst, GatherSrcs srcs, long long vec_each) {
  const uint4* __restrict__ src = static_cast<const uint4*>(srcs.p[blockIdx.y]);
  uint4* out = dst + static_cast<long long>(blockIdx.y) * vec_each;
  const long long stride = static_cast<long long>(gridDim.x) * kCopyThreads;
  long long i = static_cast<long long>(blockIdx.x) * kCopyThreads + threadIdx.x;
  for (; i + (kCopyUnroll - 1) * stride < vec_each; i += kCopyUnroll * stride) {
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) out[i + u * stride] = v[u];
  }
  for (; i < vec_each; i += stride) out[i] = src[i];
}

}  // namespace mb

// dst[r * bytes_each ...] <- srcs[r][0 .. bytes_each) for r < world; bytes_each a multiple of 16, all addresses 16-byte aligned.
MB_API int mb_peer_gather(void* dst, const void* const* srcs, int world, long long bytes_each, cudaStream_t stream) {
  using namespace mb;
  if (world < 1 || world > 16 || (bytes_each & 15) || (reinterpret_cast<uintptr_t>(dst) & 15u)) {
    set_last_error("mb_peer_gather: needs 1 <= world <= 16, 16-byte aligned pieces");
    return -1;
  }
  if (bytes_each == 0) return 0;
  GatherSrcs g{};
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(srcs[r]) & 15u) {
      set_last_error("mb_peer_gather: sources must be 16-byte aligned");
      return -1;
    }
    g.p[r] = srcs[r];
  }
  const long long vec_each = bytes_each >> 4;
  long long bx = (vec_each + kCopyThreads * kCopyUnroll - 1) / (kCopyThreads * kCopyUnroll);
  const long long cap = (static_cast<long long>(sm_count()) * 4 + world - 1) / world;
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  peer_gather_kernel<<<dim3(static_cast<unsigned>(bx), static_cast<unsigned>(world)), kCopyThreads, 0, stream>>>(
      static_cast<uint4*>(dst), g, vec_each);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// dst, src: 16-byte aligned device addresses (local or peer); any byte count.
MB_API int mb_peer_copy(void* dst, const void* src, long long nbytes, int max_blocks, cudaStream_t stream) {
  using namespace mb;
  if ((reinterpret_cast<uintptr_t>(dst) & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u) || nbytes < 0) {
    set_last_error("mb_peer_copy: addresses must be 16-byte aligned");
    return -1;
  }
  if (nbytes == 0) return 0;
  const long long nvec = nbytes >> 4;
  const int tail = static_cast<int>(nbytes & 15);
  long long blocks = (nvec + kCopyThreads * kCopyUnroll - 1) / (kCopyThreads * kCopyUnroll);
  const long long cap = max_blocks > 0 ? max_blocks : static_cast<long long>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  peer_copy_kernel<<<static_cast<unsigned>(blocks), kCopyThreads, 0, stream>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src), nvec, static_cast<unsigned char*>(dst) + (nvec << 4),
      static_cast<const unsigned char*>(src) + (nvec << 4), tail);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
