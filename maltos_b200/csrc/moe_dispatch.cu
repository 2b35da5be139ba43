// Expert-parallel token transport over peer memory (NVLink, CUDA-IPC mappings) for sm_100a.
//
// The source rank of a routed token knows, from the all-gathered per-expert counts, the exact row the token occupies in
// the destination rank's expert-major buffer. `push` gathers the token rows by index and stores them straight into the
// destination ranks' buffers; `pull` reads rows of the destination ranks' output buffers back into assignment order.
// Dispatch = push, combine = pull, and their gradients are the opposite transfers, so the four variable-split
// all-to-alls of the reference layer (runtime/layers/moe.py:112-150: tokens, gates, expert ids, results) become two
// one-sided row copies; gates and expert ids never travel because rows arrive sorted by expert and the gate is applied
// on the source side.
//
// A destination rank of -1 marks an assignment dropped by the capacity limit (skipped by a push, zeros from a pull), so
// the row count of a transfer is static and no host ever reads how many assignments survived.
// One warp moves one row with 16-byte accesses, four in flight per lane. The kernels never wait on another GPU; the
// callers separate them from the peers' reads and writes with stream-ordered group barriers.
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kRowWarps = 8;

// rows: row_bytes % 16 == 0, all bases 16-byte aligned, strides in bytes (multiples of 16).
// local_row == nullptr means "row j of the local tensor".
template <bool kPush>
__global__ void __launch_bounds__(32 * kRowWarps)
peer_rows_kernel(unsigned char* __restrict__ local, long long local_stride, const long long* __restrict__ local_row,
                 const long long* __restrict__ peer_base, long long peer_offset, long long peer_stride,
                 const int* __restrict__ peer_rank, const long long* __restrict__ peer_row, long long rows, int row_bytes,
                 int world, long long peer_rows_cap, long long local_rows_cap, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int chunks = row_bytes >> 4;
  for (long long j = static_cast<long long>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5); j < rows;
       j += static_cast<long long>(gridDim.x) * kRowWarps) {
    const int r = peer_rank[j];
    const long long pr = peer_row[j];
    const long long lr = local_row ? local_row[j] : j;
    if (r == -1) {
      // an assignment that was dropped by the capacity limit: nothing is sent; a pull delivers a row of zeros
      if (!kPush && lr >= 0 && lr < local_rows_cap) {
        uint4* mine = reinterpret_cast<uint4*>(local + lr * local_stride);
        for (int c = lane; c < chunks; c += 32) mine[c] = make_uint4(0u, 0u, 0u, 0u);
      }
      continue;
    }
    if (r < 0 || r >= world || pr < 0 || pr >= peer_rows_cap || lr < 0 || lr >= local_rows_cap) {
      // a bad index is recorded and the row skipped: nothing is read or written outside the buffers
      if (lane == 0) atomicOr(status, MB_ERR_BAD_INDEX);
      continue;
    }
    uint4* remote = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(peer_base[r]) + peer_offset + pr * peer_stride);
    uint4* mine = reinterpret_cast<uint4*>(local + lr * local_stride);
    const uint4* from = kPush ? mine : remote;
    uint4* to = kPush ? remote : mine;
    for (int c = lane; c < chunks; c += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c + 32 * u < chunks) v[u] = from[c + 32 * u];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c + 32 * u < chunks) to[c + 32 * u] = v[u];
    }
  }
}

static int rows_grid(long long rows) {
  long long b = (rows + kRowWarps - 1) / kRowWarps;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

static int check_rows_args(const void* local, long long local_stride, long long peer_offset, long long peer_stride, int row_bytes, int world) {
  if (row_bytes <= 0 || (row_bytes & 15) || (local_stride & 15) || (peer_stride & 15) || (peer_offset & 15) ||
      (reinterpret_cast<uintptr_t>(local) & 15u) || world < 1) {
    set_last_error("peer row transfer: rows, strides and bases must be multiples of 16 bytes");
    return -1;
  }
  return 0;
}

}  // namespace mb

// peer[peer_rank[j]] + peer_offset + peer_row[j] * peer_stride  <-  local + local_row[j] * local_stride   (row_bytes each)
MB_API int mb_peer_push_rows(const void* local, long long local_stride, const long long* local_row, long long local_rows_cap,
                             const long long* peer_base, long long peer_offset, long long peer_stride, long long peer_rows_cap,
                             const int* peer_rank, const long long* peer_row, long long rows, int row_bytes, int world, cudaStream_t stream) {
  using namespace mb;
  if (check_rows_args(local, local_stride, peer_offset, peer_stride, row_bytes, world)) return -1;
  if (rows <= 0) return 0;
  peer_rows_kernel<true><<<rows_grid(rows), 32 * kRowWarps, 0, stream>>>(
      static_cast<unsigned char*>(const_cast<void*>(local)), local_stride, local_row, peer_base, peer_offset, peer_stride, peer_rank,
      peer_row, rows, row_bytes, world, peer_rows_cap, local_rows_cap, status_ptr());
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// local + local_row[j] * local_stride  <-  peer[peer_rank[j]] + peer_offset + peer_row[j] * peer_stride
MB_API int mb_peer_pull_rows(void* local, long long local_stride, const long long* local_row, long long local_rows_cap,
                             const long long* peer_base, long long peer_offset, long long peer_stride, long long peer_rows_cap,
                             const int* peer_rank, const long long* peer_row, long long rows, int row_bytes, int world, cudaStream_t stream) {
  using namespace mb;
  if (check_rows_args(local, local_stride, peer_offset, peer_stride, row_bytes, world)) return -1;
  if (rows <= 0) return 0;
  peer_rows_kernel<false><<<rows_grid(rows), 32 * kRowWarps, 0, stream>>>(
      static_cast<unsigned char*>(local), local_stride, local_row, peer_base, peer_offset, peer_stride, peer_rank, peer_row, rows,
      row_bytes, world, peer_rows_cap, local_rows_cap, status_ptr());
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
