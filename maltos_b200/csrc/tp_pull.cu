// Sequence-parallel collectives of the tensor-parallel layers as one-sided PULL kernels over NVLink peer memory
// (CUDA-IPC mappings of every rank's symmetric buffers), used where the in-GEMM push does not pay (groups above four
// ranks: a GEMM block that also pushes moves ~190 GB/s, a whole grid of pulling threads ~700 GB/s):
//
//  * pull_reduce_scatter_kernel: every rank's GEMM leaves its bf16 partial result [B, S, N] in its own symmetric
//    buffer; the kernel publishes "my partial of call `seq` is complete" in every peer's signal pad, waits (bounded) for
//    the same word from every peer, then the OWNER of a sequence slice reads that slice from all ranks (16-byte peer
//    loads, all ranks' loads in flight before the first add), sums in fp32 in rank order and writes its [B, S/T, N] rows.
//    Replaces NCCL reduce-scatter after the row-parallel GEMMs (reference runtime/layers/functional.py:273-366).
//  * pull_all_gather_kernel: every rank copies its [B, S/T, K] rows into its symmetric buffer (and into its own slot of
//    the gathered tensor), the last block to finish publishes the flag, then every block pulls the peers' rows, peers
//    visited in ring order starting at rank + 1, one load per peer in flight per thread.
//    Replaces NCCL all-gather in front of the column-parallel GEMMs (reference runtime/layers/functional.py:369-486).
//
// Both buffers are double-buffered by call parity. That is enough for safe reuse without a second flag: a rank passes
// the wait of call n + 1 only after every peer has STARTED call n + 1, which on the peer's stream is after its call n
// kernel (the reader of this rank's parity-n buffer) has finished; this rank's call n + 2 (the next writer of that
// buffer) comes later still. Signal-pad words (uint32): [256 + buf*8 + src] partial of `src` complete (reduce-scatter),
// [272 + buf*8 + src] rows of `src` published (all-gather), [288] finished copy blocks of the running all-gather (local).
// Every wait is bounded by %globaltimer; a wait that runs out sets the "peer flag wait timed out" status bit and the
// kernel returns without touching peer memory.
#include "host.h"
#include "ptx.cuh"

namespace mb {

#ifdef MB_FLASH_PROBE
__device__ unsigned long long g_pull_probe[16];
#define MB_PULL_STAMP(cond, slot) do { if (cond) g_pull_probe[slot] = globaltimer_ns(); } while (0)
#else
#define MB_PULL_STAMP(cond, slot) do { } while (0)
#endif

constexpr int kPullThreads = 256;
constexpr int kPullMaxWorld = 8;

struct PullPtrs {
  unsigned long long data[kPullMaxWorld];   // per rank: base of its symmetric buffer half used by this call
  unsigned long long pads[kPullMaxWorld];   // per rank: base of its signal pad
};

__device__ __forceinline__ unsigned pull_ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void pull_st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Thread 0 of the block waits until the `world` words at `flags` have all reached `seq`; returns (to all threads of the
// block) whether they did. On a timeout the peer whose word was missing is recorded.
__device__ __forceinline__ bool pull_wait_all(const unsigned* flags, int world, int self, unsigned seq, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const int ms = status[3];
    const uint64_t limit = ms > 0 ? static_cast<uint64_t>(ms) * 1000000ull : kWaitTimeoutNs;
    const uint64_t t0 = globaltimer_ns();
    int ok = 1;
    for (int r = 0; r < world && ok; ++r) {
      if (r == self) continue;
      while (static_cast<int>(pull_ld_acquire_sys(flags + r) - seq) < 0) {
        if (globaltimer_ns() - t0 > limit) {
          ok = 0;
          atomicOr(&status[0], MB_ERR_PEER_TIMEOUT);
          status[1] = static_cast<int>(blockIdx.x);
          status[2] = r;
          break;
        }
        __nanosleep(100);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void bf16x8_accumulate(const uint4& v, float* acc) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    acc[2 * i] += t.x;
    acc[2 * i + 1] += t.y;
  }
}

// partial buffers: [B, T * rows, N] bf16 on every rank; out: [B, rows, N]. vec_per_slice = rows * N / 8.
template <int WORLD>
__global__ void __launch_bounds__(kPullThreads)
pull_reduce_scatter_kernel(PullPtrs pp, int rank, unsigned seq, int batches, long long vec_per_slice, uint4* __restrict__ out,
                           int* status) {
  const int buf = static_cast<int>(seq & 1u);
  if (blockIdx.x == 0 && threadIdx.x < WORLD && static_cast<int>(threadIdx.x) != rank) {
    __threadfence_system();   // the GEMM that wrote the partial ran before this kernel on the stream
    pull_st_release_sys(reinterpret_cast<unsigned*>(pp.pads[threadIdx.x]) + 256 + buf * 8 + rank, seq);
  }
  const unsigned* my_flags = reinterpret_cast<const unsigned*>(pp.pads[rank]) + 256 + buf * 8;
  if (!pull_wait_all(my_flags, WORLD, rank, seq, status)) return;
  const long long total = static_cast<long long>(batches) * vec_per_slice;
  const long long stride = static_cast<long long>(gridDim.x) * kPullThreads;
  constexpr int UNROLL = WORLD >= 8 ? 1 : (WORLD == 4 ? 2 : 4);     // loads in flight per thread: UNROLL x WORLD
  auto reduce_store = [&](const uint4 (&raw)[WORLD], long long v) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < WORLD; ++r) bf16x8_accumulate(raw[r], acc);     // rank order: the same bits on every owner
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]), o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]), o.w = pack_bf16x2(acc[6], acc[7]);
    out[v] = o;
  };
  auto src_of = [&](long long v) {
    const long long b = v / vec_per_slice, off = v - b * vec_per_slice;
    return (b * WORLD + rank) * vec_per_slice + off;                      // this rank's slice inside batch b
  };
  long long v = static_cast<long long>(blockIdx.x) * kPullThreads + threadIdx.x;
  for (; v + (UNROLL - 1) * stride < total; v += UNROLL * stride) {
    uint4 raw[UNROLL][WORLD];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long so = src_of(v + u * stride);
#pragma unroll
      for (int r = 0; r < WORLD; ++r) raw[u][r] = reinterpret_cast<const uint4*>(pp.data[r])[so];
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) reduce_store(raw[u], v + u * stride);
  }
  for (; v < total; v += stride) {
    const long long so = src_of(v);
    uint4 raw[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) raw[r] = reinterpret_cast<const uint4*>(pp.data[r])[so];
    reduce_store(raw, v);
  }
}

// x_local: [B, rows, K] contiguous bf16; pp.data[r]: rank r's symmetric publish buffer (same layout); gathered: local
// [B, T * rows, K]. vec_per_slice = rows * K / 8.
template <int WORLD>
__global__ void __launch_bounds__(kPullThreads)
pull_all_gather_kernel(PullPtrs pp, int rank, unsigned seq, int batches, long long vec_per_slice, const uint4* __restrict__ x_local,
                       uint4* __restrict__ gathered, int* status) {
  const int buf = static_cast<int>(seq & 1u);
  const long long total = static_cast<long long>(batches) * vec_per_slice;
  const long long stride = static_cast<long long>(gridDim.x) * kPullThreads;
  const long long tid = static_cast<long long>(blockIdx.x) * kPullThreads + threadIdx.x;
  unsigned* my_pad = reinterpret_cast<unsigned*>(pp.pads[rank]);
  MB_PULL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 0);
  // phase A: publish this rank's rows (no waiting here, so every block always gets through it)
  {
    uint4* pub = reinterpret_cast<uint4*>(pp.data[rank]);
    for (long long v = tid; v < total; v += stride) {
      const uint4 q = x_local[v];
      const long long b = v / vec_per_slice, off = v - b * vec_per_slice;
      pub[v] = q;
      gathered[(b * WORLD + rank) * vec_per_slice + off] = q;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    MB_PULL_STAMP(blockIdx.x == 0, 1);
    const unsigned done = atomicAdd(my_pad + 288, 1u);
    if (done == gridDim.x - 1) {
      atomicExch(my_pad + 288, 0u);
      __threadfence_system();
      MB_PULL_STAMP(true, 2);
      for (int r = 0; r < WORLD; ++r)
        if (r != rank) pull_st_release_sys(reinterpret_cast<unsigned*>(pp.pads[r]) + 272 + buf * 8 + rank, seq);
      MB_PULL_STAMP(true, 3);
    }
  }
  // phase B: pull the peers' rows; the grid is no larger than what is resident at once, so the blocks that spin here
  // never keep a phase-A block of this GPU from running
  if (!pull_wait_all(my_pad + 272 + buf * 8, WORLD, rank, seq, status)) return;
  MB_PULL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 4);
  // Remote loads need many requests in flight to fill the link (8 per thread reach ~735 GB/s, 3 only ~390): every thread
  // keeps UNROLL vectors x (WORLD - 1) peers outstanding, peers taken in ring order from rank + 1 so that the readers of
  // one source are spread over time.
  constexpr int UNROLL = WORLD >= 8 ? 2 : (WORLD == 4 ? 3 : 8);
  long long v = tid;
  for (; v + (UNROLL - 1) * stride < total; v += UNROLL * stride) {
    uint4 q[UNROLL][WORLD - 1];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int step = 1; step < WORLD; ++step) q[u][step - 1] = reinterpret_cast<const uint4*>(pp.data[(rank + step) % WORLD])[v + u * stride];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long vv = v + u * stride;
      const long long b = vv / vec_per_slice, off = vv - b * vec_per_slice;
#pragma unroll
      for (int step = 1; step < WORLD; ++step) gathered[(b * WORLD + (rank + step) % WORLD) * vec_per_slice + off] = q[u][step - 1];
    }
  }
  for (; v < total; v += stride) {
    const long long b = v / vec_per_slice, off = v - b * vec_per_slice;
#pragma unroll
    for (int step = 1; step < WORLD; ++step) {
      const int r = (rank + step) % WORLD;
      gathered[(b * WORLD + r) * vec_per_slice + off] = reinterpret_cast<const uint4*>(pp.data[r])[v];
    }
  }
  MB_PULL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 5);
  MB_PULL_STAMP(blockIdx.x == gridDim.x - 1 && threadIdx.x == 0, 6);
}

static int fill_ptrs(PullPtrs* pp, const unsigned long long* data, const unsigned long long* pads, int world, const char* what) {
  if (world < 2 || world > kPullMaxWorld || (world & (world - 1))) {
    set_last_error(what);
    return -1;
  }
  for (int r = 0; r < kPullMaxWorld; ++r) {
    pp->data[r] = r < world ? data[r] : 0ull;
    pp->pads[r] = r < world ? pads[r] : 0ull;
    if (r < world && ((data[r] & 15ull) || !pads[r] || !data[r])) {
      set_last_error(what);
      return -1;
    }
  }
  return 0;
}

}  // namespace mb

#ifdef MB_FLASH_PROBE
MB_API int mb_pull_probe_read(unsigned long long* host_out) {
  return static_cast<int>(cudaMemcpyFromSymbol(host_out, mb::g_pull_probe, sizeof(unsigned long long) * 16));
}
#endif

// out[B, rows, N] = sum over ranks of partial_r[B, rank-th slice of T * rows, N]. `partials[r]`: address, as mapped in
// this process, of the buffer half of rank r that holds its partial of this call; `pads[r]`: its signal pad. `seq`
// counts the calls of this protocol on the group (1, 2, ...). rows * N must be a multiple of 8.
MB_API int mb_pull_reduce_scatter_bf16(const unsigned long long* partials, const unsigned long long* pads, void* out, int batches,
                                       long long rows, long long n_cols, int rank, int world, unsigned seq, cudaStream_t stream) {
  using namespace mb;
  PullPtrs pp;
  if (fill_ptrs(&pp, partials, pads, world, "mb_pull_reduce_scatter_bf16: needs a power-of-two group of 2..8 ranks and 16-byte aligned buffers"))
    return -1;
  if (batches < 1 || rows < 1 || (rows * n_cols) % 8 || (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_last_error("mb_pull_reduce_scatter_bf16: rows * n_cols must be a multiple of 8 and out 16-byte aligned");
    return -2;
  }
  int* status = status_ptr();
  if (!status) return -4;
  const long long vec_per_slice = rows * n_cols / 8;
  const long long total = vec_per_slice * batches;
  long long blocks = (total + kPullThreads - 1) / kPullThreads;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  uint4* o = static_cast<uint4*>(out);
  const unsigned g = static_cast<unsigned>(blocks);
  switch (world) {
    case 2: pull_reduce_scatter_kernel<2><<<g, kPullThreads, 0, stream>>>(pp, rank, seq, batches, vec_per_slice, o, status); break;
    case 4: pull_reduce_scatter_kernel<4><<<g, kPullThreads, 0, stream>>>(pp, rank, seq, batches, vec_per_slice, o, status); break;
    default: pull_reduce_scatter_kernel<8><<<g, kPullThreads, 0, stream>>>(pp, rank, seq, batches, vec_per_slice, o, status); break;
  }
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// gathered[B, T * rows, K] (local) <- every rank's x_local[B, rows, K]. `publish[r]`: address, as mapped here, of the
// buffer half rank r publishes its rows in for this call (at least B * rows * K bf16). rows * K a multiple of 8.
MB_API int mb_pull_all_gather_bf16(const void* x_local, const unsigned long long* publish, const unsigned long long* pads,
                                   void* gathered, int batches, long long rows, long long k_cols, int rank, int world, unsigned seq,
                                   cudaStream_t stream) {
  using namespace mb;
  PullPtrs pp;
  if (fill_ptrs(&pp, publish, pads, world, "mb_pull_all_gather_bf16: needs a power-of-two group of 2..8 ranks and 16-byte aligned buffers"))
    return -1;
  if (batches < 1 || rows < 1 || (rows * k_cols) % 8 ||
      ((reinterpret_cast<uintptr_t>(x_local) | reinterpret_cast<uintptr_t>(gathered)) & 15)) {
    set_last_error("mb_pull_all_gather_bf16: rows * k_cols must be a multiple of 8 and tensors 16-byte aligned");
    return -2;
  }
  int* status = status_ptr();
  if (!status) return -4;
  const long long vec_per_slice = rows * k_cols / 8;
  const long long total = vec_per_slice * batches;
  long long blocks = (total + kPullThreads - 1) / kPullThreads;
  // the blocks that spin in phase B must never keep a phase-A block of the same launch from running: the grid is capped at
  // what the occupancy calculator says is resident at once for this instance
  int per_sm = 0;
  cudaError_t occ = world == 2   ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pull_all_gather_kernel<2>, kPullThreads, 0)
                    : world == 4 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pull_all_gather_kernel<4>, kPullThreads, 0)
                                 : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pull_all_gather_kernel<8>, kPullThreads, 0);
  if (occ != cudaSuccess || per_sm < 1) per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  if (blocks > cap) blocks = cap;
  const unsigned g = static_cast<unsigned>(blocks);
  const uint4* x = static_cast<const uint4*>(x_local);
  uint4* o = static_cast<uint4*>(gathered);
  switch (world) {
    case 2: pull_all_gather_kernel<2><<<g, kPullThreads, 0, stream>>>(pp, rank, seq, batches, vec_per_slice, x, o, status); break;
    case 4: pull_all_gather_kernel<4><<<g, kPullThreads, 0, stream>>>(pp, rank, seq, batches, vec_per_slice, x, o, status); break;
    default: pull_all_gather_kernel<8><<<g, kPullThreads, 0, stream>>>(pp, rank, seq, batches, vec_per_slice, x, o, status); break;
  }
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
