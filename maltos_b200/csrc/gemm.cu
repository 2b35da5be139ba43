// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] (+)= op(A) * op(B) (+ bias)          fp32 accumulation in tensor memory
//
// Roles inside one CTA (one CTA per SM, tiles handed out round-robin in an L2-friendly order):
//   warp 0     : TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, STAGES-deep smem ring)
//   warp 1     : MMA issuer    (one elected thread, tcgen05.mma 128 x BN x 16, accumulators in TMEM)
//   warps 2..5 : epilogue      (tcgen05.ld -> registers -> bias / accumulate / convert -> global)
// TMEM holds two BN-column accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand layouts (both without any transpose pass):
//   a_mn = 0 : A is [M,K] row-major ("K-major").      a_mn = 1 : A is stored as [K,M] row-major.
//   b_mn = 0 : B is [N,K] row-major ("K-major").      b_mn = 1 : B is stored as [K,N] row-major.
// which covers forward (x W^T), dgrad (dy W) and wgrad (dy^T x) of a linear layer.
#include <cstdlib>
#include <mutex>

#include "host.h"
#include "ptx.cuh"

// Timing probes (cycle counters per k-block, "MMAs without data" / "loads without math" modes) exist only in builds
// with -DMB_GEMM_PROBE; in the default build the macros below fold every probe branch away at compile time.
#ifdef MB_GEMM_PROBE
#define MB_DEBUG_MODE(p) ((p).debug_mode)
#define MB_TRACE(p) ((p).trace)
#define MB_CLOCK() clock64()
#else
#define MB_DEBUG_MODE(p) 0
#define MB_TRACE(p) (static_cast<long long*>(nullptr))
#define MB_CLOCK() 0ll
#endif

namespace mb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kEpiWarps = 4;
constexpr int kFirstPushWarp = 2 + kEpiWarps;
constexpr int kGemmThreads = 32 * kFirstPushWarp;        // warp 0 TMA, 1 MMA, 2..5 epilogue
constexpr int kWideThreads = kGemmThreads + 32 * kEpiWarps;   // 256x512 kernel: warps 6..9 are a second epilogue group
constexpr int kMaxPushThreads = 128;  // extra warps per block that copy rows to peers in the fused all-gather launch
constexpr int kGroupM = 8;  // tiles of one N column are visited for 8 consecutive M blocks (L2 reuse of B)

// Reduce-scatter fused into the GEMM epilogue (row-parallel layers; sequence-parallel output). Output row m belongs to
// rank owner(m) = (m % s_rows) / rows_per_chunk; instead of C, the bf16 partial tile is stored straight into slot
// `rank` of the owner's staging buffer over NVLink while later tiles are still being computed; the owner's reduce
// kernel (rs_reduce_kernel) sums the `world` slots once every writer's flag has arrived. Signal-pad words (uint32):
//   [64 + buf*8 + src]   partial of `src` is complete in my staging buffer `buf`          (written by src)
//   [96 + buf*8 + owner] `owner` has finished reducing ITS staging buffer `buf`           (written by owner)
//   [128] finished GEMM blocks of the running call (local)    [129] finished reduce blocks (local)
struct ScatterArgs {
  int enabled;
  int rank, world;
  int rows_per_chunk;     // S / T
  int s_rows;             // S
  unsigned seq;
  unsigned long long slot_base[8];   // per owner: address of slot `rank` in the owner's staging buffer of this call
  unsigned long long pads[8];
};

struct GemmArgs {
  void* C;
  const __nv_bfloat16* bias;  // [N] or nullptr
  long long ldc;
  int M, N, K;
  int a_mn, b_mn;
  int out_fp32;    // 0: C is bf16, 1: C is fp32
  int accumulate;  // 1: C += result
  int tiles_m, tiles_n, k_blocks;
  // UMMA shared-memory descriptor geometry in bytes (see make_smem_desc_sw128).
  unsigned a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep;
  int* status;
  int group_m;        // M blocks per rasterisation group (CTA-pair kernel)
  int stages;         // debug: ring depth used by the CTA-pair kernel (0 = all)
  int debug_mode;     // 0 normal; 1 = MMAs without waiting for data (producer idle); 2 = loads without MMAs (timing probes)
  long long* trace;   // debug: per-CTA cycle counters {mma total, wait full, wait tempty, producer wait empty} or nullptr
  int quad_epilogue;  // 1: interior bf16 tiles of the CTA-pair kernels are written with the line-coalesced epilogue
  // Split tail (256x512 kernel, plain launches): when the tiles left for the last wave occupy at most half of the CTA
  // pairs, each of them is computed by `tail_split` pairs over disjoint k ranges. Every epilogue warp writes its fp32
  // partial block to `tail_ws`, then counts itself on `tail_cnt`; the warp that arrives last sums the partials and
  // runs the normal epilogue. Nobody waits: the reduction is done by whoever finishes last.
  int tail_split;         // 1 = off
  float* tail_ws;         // [tail tiles][tail_split][2 CTAs][128 rows][512 cols] fp32
  unsigned* tail_cnt;     // [tail tiles][2 CTAs][8 warps], zeroed before the launch
  ScatterArgs sc;
};

// Sequence-parallel all-gather fused into the GEMM (A operand = rows gathered from all ranks of the TP group).
// `push_ctas` extra warps of every block copy this rank's rows into every peer's gathered buffer over NVLink and
// publish a per-source flag; the GEMM blocks start with this rank's own rows and visit the other sources in ring
// order, waiting (bounded) for a source's flag only when they reach its rows. Signal-pad words (uint32):
//   [buf*8 + src]        arrived : rows of `src` are complete in my gathered buffer `buf`      (written by src)
//   [16 + buf*8 + rank]  consumed: `rank` has finished reading ITS gathered buffer `buf`       (written by rank)
//   [32]                 finished GEMM blocks of the running call (local)   [40 + dst] finished push blocks (local)
constexpr int kMaxPeers = 8;
struct GatherArgs {
  int enabled;
  int push_ctas;          // push warps per block
  int bulk;               // 1: push with bulk async copies through a shared-memory staging buffer (one thread per block)
  int rank, world;
  int batches;            // B
  int rows_per_chunk;     // S / T rows of one rank per batch
  const __nv_bfloat16* x_local;   // [B * rows_per_chunk, K] (row stride x_ld)
  long long x_ld;
  unsigned seq;           // sequence number of this call (1, 2, ...); buffer = seq & 1
  long long buf_elems;    // elements of one gathered buffer (B * S * K)
  unsigned long long gathered[kMaxPeers];   // base address of every rank's gathered buffers, as mapped here
  unsigned long long pads[kMaxPeers];       // base address of every rank's signal pad, as mapped here
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Wait until *flag has reached `want` (sequence numbers, wrap-safe). Bounded: false after the deadline.
__device__ __forceinline__ bool wait_flag_reached(const unsigned* flag, unsigned want, volatile int* abort_flag) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t limit = wait_limit_ns(abort_flag);
#pragma unroll 1
  while (true) {
    if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
    if (abort_flag && *abort_flag) return false;
    if (globaltimer_ns() - t0 > limit) return false;
    __nanosleep(200);
  }
}

// Body of a push block: copies x_local into slot `rank` of every rank's gathered buffer, local copy first.
__device__ void gather_push_role(const GatherArgs& g, int K, int* status, int n_ctas, int first_thread = kGemmThreads) {
  __shared__ int s_ok;
  const int tid = static_cast<int>(threadIdx.x) - first_thread;          // push warps sit behind the GEMM warps
  const int nthr = static_cast<int>(blockDim.x) - first_thread;
  auto push_sync = [nthr]() { asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory"); };
  const int buf = static_cast<int>(g.seq & 1u);
  const long long vec_per_row = K >> 3;
  const long long rows_local = static_cast<long long>(g.batches) * g.rows_per_chunk;
  const long long s_rows = static_cast<long long>(g.rows_per_chunk) * g.world;   // rows of one batch in the gathered buffer
  unsigned* my_pad = reinterpret_cast<unsigned*>(g.pads[g.rank]);
  for (int step = 0; step < g.world; ++step) {
    // Destinations in descending ring order: every rank's GEMM visits the sources as rank, rank+1, rank+2, ..., so
    // rank r needs the rows of r+1 first - which r+1 delivers first when it starts with destination (r+1)-1.
    const int dst = (g.rank - step + g.world) % g.world;
    if (tid == 0) {
      // the destination must have finished the call that last used this buffer (two calls ago)
      bool ok = step == 0 ? true : wait_flag_reached(my_pad + 16 + buf * 8 + dst, g.seq - 2u, nullptr);
      if (step == 0) ok = wait_flag_reached(my_pad + 16 + buf * 8 + g.rank, g.seq - 2u, nullptr);
      if (!ok) {
        atomicOr(&status[0], MB_ERR_PEER_TIMEOUT);
        status[2] = dst;
      }
      s_ok = ok ? 1 : 0;
    }
    push_sync();
    if (!s_ok) return;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(g.gathered[dst]) + static_cast<long long>(buf) * g.buf_elems;
    // Row-wise copy, 4 rows per pass: every thread keeps several independent 16-byte loads in flight before the
    // (posted) NVLink stores - a dependent load->store chain per thread would make the copy latency-bound.
    constexpr int kRows = 4;
    const int vpr = static_cast<int>(vec_per_row);
    for (long long r0 = static_cast<long long>(blockIdx.x) * kRows; r0 < rows_local; r0 += static_cast<long long>(n_ctas) * kRows) {
      for (int c0 = tid; c0 < vpr; c0 += nthr * 2) {
        uint4 vals[kRows][2];
        const int c1 = c0 + nthr;
#pragma unroll
        for (int rr = 0; rr < kRows; ++rr) {
          const long long row = r0 + rr;
          if (row < rows_local) {
            const __nv_bfloat16* src = g.x_local + row * g.x_ld;
            vals[rr][0] = *reinterpret_cast<const uint4*>(src + c0 * 8);
            if (c1 < vpr) vals[rr][1] = *reinterpret_cast<const uint4*>(src + c1 * 8);
          }
        }
#pragma unroll
        for (int rr = 0; rr < kRows; ++rr) {
          const long long row = r0 + rr;
          if (row < rows_local) {
            const long long b = row / g.rows_per_chunk, i = row - b * g.rows_per_chunk;
            __nv_bfloat16* drow = out + (b * s_rows + static_cast<long long>(g.rank) * g.rows_per_chunk + i) * K;
            *reinterpret_cast<uint4*>(drow + c0 * 8) = vals[rr][0];
            if (c1 < vpr) *reinterpret_cast<uint4*>(drow + c1 * 8) = vals[rr][1];
          }
        }
      }
    }
    __threadfence_system();
    push_sync();
    if (tid == 0) {
      const unsigned done = atomicAdd(my_pad + 40 + dst, 1u);
      if (done == static_cast<unsigned>(n_ctas - 1)) {   // last block to finish this destination publishes the flag
        atomicExch(my_pad + 40 + dst, 0u);
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned*>(g.pads[dst]) + buf * 8 + g.rank, g.seq);
      }
    }
    push_sync();
  }
}

// Bulk variant of the push role: ONE thread per block moves 16 KB pieces global -> shared (bulk load, mbarrier) ->
// destination (bulk store into local or peer memory). No registers or issue slots of the other warps are used and the
// NVLink writes leave as large bursts. `stage` is 128-byte aligned: two mbarriers, then two 16 KB buffers.
constexpr uint32_t kBulkPiece = 16384;
constexpr uint32_t kPushSmemBytes = 128 + 2 * kBulkPiece;

__device__ void gather_push_role_bulk(const GatherArgs& g, int K, int* status, int n_ctas, uint8_t* stage, volatile int* abort_flag) {
  uint64_t* bar = reinterpret_cast<uint64_t*>(stage);
  uint8_t* buf_smem = stage + 128;
  mbar_init(&bar[0], 1);
  mbar_init(&bar[1], 1);
  fence_barrier_init();
  fence_proxy_async_smem();
  const int gbuf = static_cast<int>(g.seq & 1u);
  const long long chunk_bytes = static_cast<long long>(g.rows_per_chunk) * K * 2;      // one batch's rows of this rank
  const long long pieces_per_chunk = (chunk_bytes + kBulkPiece - 1) / kBulkPiece;
  const long long n_pieces = pieces_per_chunk * g.batches;
  const long long s_rows = static_cast<long long>(g.rows_per_chunk) * g.world;
  unsigned* my_pad = reinterpret_cast<unsigned*>(g.pads[g.rank]);
  const uint8_t* src_base = reinterpret_cast<const uint8_t*>(g.x_local);
  uint32_t use[2] = {0u, 0u};     // completed uses of each staging buffer (mbarrier phase)
  for (int step = 0; step < g.world; ++step) {
    const int dst = (g.rank - step + g.world) % g.world;
    if (!wait_flag_reached(my_pad + 16 + gbuf * 8 + dst, g.seq - 2u, abort_flag)) {
      atomicOr(&status[0], MB_ERR_PEER_TIMEOUT);
      status[2] = dst;
      return;
    }
    uint8_t* out = reinterpret_cast<uint8_t*>(g.gathered[dst]) + static_cast<long long>(gbuf) * g.buf_elems * 2;
    auto piece_bytes = [&](long long pc) -> uint32_t {
      const long long within = (pc % pieces_per_chunk) * kBulkPiece;
      const long long left = chunk_bytes - within;
      return static_cast<uint32_t>(left < kBulkPiece ? left : kBulkPiece);
    };
    auto issue_load = [&](long long pc, int b) {
      const long long batch = pc / pieces_per_chunk, within = (pc % pieces_per_chunk) * kBulkPiece;
      const uint32_t bytes = piece_bytes(pc);
      mbar_arrive_expect_tx(&bar[b], bytes);
      bulk_load(buf_smem + b * kBulkPiece, src_base + batch * chunk_bytes + within, bytes, &bar[b]);
    };
    long long pc = blockIdx.x;
    int b = 0;
    if (pc < n_pieces) issue_load(pc, 0);
    bool ok = true;
    for (; pc < n_pieces; pc += n_ctas, b ^= 1) {
      const long long next = pc + n_ctas;
      if (next < n_pieces) {
        tma_store_wait_read<0>();            // the other buffer's previous store has finished reading it
        issue_load(next, b ^ 1);
      }
      if (!mbar_wait(&bar[b], use[b] & 1u, abort_flag)) {
        ok = false;
        break;
      }
      ++use[b];
      const long long batch = pc / pieces_per_chunk, within = (pc % pieces_per_chunk) * kBulkPiece;
      uint8_t* drow = out + ((batch * s_rows + static_cast<long long>(g.rank) * g.rows_per_chunk) * K) * 2 + within;
      bulk_store(drow, buf_smem + b * kBulkPiece, piece_bytes(pc));
      tma_store_commit();
    }
    tma_store_wait_all<0>();                 // every store of this destination is complete
    if (!ok) return;
    fence_proxy_async_global();
    __threadfence_system();
    const unsigned done = atomicAdd(my_pad + 40 + dst, 1u);
    if (done == static_cast<unsigned>(n_ctas - 1)) {
      atomicExch(my_pad + 40 + dst, 0u);
      __threadfence_system();
      st_release_sys(reinterpret_cast<unsigned*>(g.pads[dst]) + gbuf * 8 + g.rank, g.seq);
    }
  }
}

// The push as a launch of its own (same stream, in front of the GEMM launch): 256-thread blocks doing nothing but the
// row copies reach the NVLink rate of a plain copy kernel (~680 GB/s measured with 64 blocks), which the push warps
// inside a GEMM block do not (~190 GB/s: they share the SM with spinning producer / MMA / epilogue warps). The GEMM
// launch that follows only waits for the peers' flags.
constexpr int kPushKernelThreads = 256;
__global__ void __launch_bounds__(kPushKernelThreads)
ag_push_kernel(const __grid_constant__ GatherArgs g, int K, int* status) {
  gather_push_role(g, K, status, static_cast<int>(gridDim.x), 0);
}

// First M block a rank visits: with a fused all-gather its own rows (already local), with a fused reduce-scatter the
// rows of the next rank (remote partials leave first, the rank's own rows need no transfer and come last).
__device__ __forceinline__ int tile_rotation(const GatherArgs& g, const ScatterArgs& sc, int tile_m) {
  if (g.enabled) return (g.rank * g.rows_per_chunk) / tile_m;
  if (sc.enabled) return (((sc.rank + 1) % sc.world) * sc.rows_per_chunk) / tile_m;
  return 0;
}

// Fused reduce-scatter, start of the kernel (one thread): every owner must have finished reducing the call that last
// used this staging buffer (two calls ago) before its slot is overwritten. Bounded; false on timeout.
__device__ bool scatter_wait_owners(const ScatterArgs& sc, int* status) {
  const unsigned* my_pad = reinterpret_cast<const unsigned*>(sc.pads[sc.rank]);
  const int buf = static_cast<int>(sc.seq & 1u);
  for (int r = 0; r < sc.world; ++r) {
    if (!wait_flag_reached(my_pad + 96 + buf * 8 + r, sc.seq - 2u, nullptr)) {
      atomicOr(&status[0], MB_ERR_PEER_TIMEOUT);
      status[2] = r;
      return false;
    }
  }
  return true;
}

// Fused reduce-scatter, end of the kernel (one thread per block, after a block-wide barrier that follows every thread's
// __threadfence_system): the last block tells every owner that this rank's partial is complete.
__device__ void scatter_publish(const ScatterArgs& sc, unsigned n_blocks) {
  unsigned* my_pad = reinterpret_cast<unsigned*>(sc.pads[sc.rank]);
  const unsigned done = atomicAdd(my_pad + 128, 1u);
  if (done == n_blocks - 1) {
    atomicExch(my_pad + 128, 0u);
    __threadfence_system();
    const int buf = static_cast<int>(sc.seq & 1u);
    for (int r = 0; r < sc.world; ++r) st_release_sys(reinterpret_cast<unsigned*>(sc.pads[r]) + 64 + buf * 8 + sc.rank, sc.seq);
  }
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& m_blk, int& n_blk, int group_m = kGroupM) {
  const int kGroupM = group_m;
  const int per_group = kGroupM * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsz = min(tiles_m - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

// Epilogue of one accumulator chunk: 32 consecutive fp32 columns of one output row (+bias, optional accumulate)
// written as bf16 or fp32 with 16-byte stores where the alignment allows.
__device__ __forceinline__ void epilogue_store32(const GemmArgs& p, int row, int col0, const uint32_t (&r)[32], bool vec_ok) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  if (p.bias) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        if (p.accumulate) {
          const float4 old = *reinterpret_cast<const float4*>(dst + i);
          o.x += old.x, o.y += old.y, o.z += old.z, o.w += old.w;
        }
        *reinterpret_cast<float4*>(dst + i) = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < p.N; ++i) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (p.sc.enabled) {   // fused reduce-scatter: the row goes to its owner's staging slot (peer memory)
      const int b = row / p.sc.s_rows, s = row - b * p.sc.s_rows;
      const int owner = s / p.sc.rows_per_chunk;
      const long long local = static_cast<long long>(b) * p.sc.rows_per_chunk + (s - owner * p.sc.rows_per_chunk);
      dst = reinterpret_cast<__nv_bfloat16*>(p.sc.slot_base[owner]) + local * p.ldc + col0;
    }
    if (vec_ok && !p.accumulate && col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
      // 64 contiguous bytes of one row as two 32-byte stores
#pragma unroll
      for (int i = 0; i < 32; i += 16) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + i),
                     "r"(pack_bf16x2(v[i], v[i + 1])), "r"(pack_bf16x2(v[i + 2], v[i + 3])), "r"(pack_bf16x2(v[i + 4], v[i + 5])),
                     "r"(pack_bf16x2(v[i + 6], v[i + 7])), "r"(pack_bf16x2(v[i + 8], v[i + 9])),
                     "r"(pack_bf16x2(v[i + 10], v[i + 11])), "r"(pack_bf16x2(v[i + 12], v[i + 13])),
                     "r"(pack_bf16x2(v[i + 14], v[i + 15]))
                     : "memory");
      }
    } else if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        if (p.accumulate) {
          const uint4 old = *reinterpret_cast<const uint4*>(dst + i);
          const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(ob[j]);
            v[i + 2 * j] += f.x;
            v[i + 2 * j + 1] += f.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(v[i], v[i + 1]);
        o.y = pack_bf16x2(v[i + 2], v[i + 3]);
        o.z = pack_bf16x2(v[i + 4], v[i + 5]);
        o.w = pack_bf16x2(v[i + 6], v[i + 7]);
        *reinterpret_cast<uint4*>(dst + i) = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < p.N; ++i) {
        const float o = p.accumulate ? v[i] + __bfloat162float(dst[i]) : v[i];
        dst[i] = __float2bfloat16(o);
      }
    }
  }
}

// Line-coalesced bf16 epilogue of a 16-row x 64-column accumulator block loaded with tmem_ld_16x256b_x8: after packing
// to bf16 pairs the four threads of a quad exchange 2-register blocks (a 4x4 transpose in two xor-shuffle stages) so
// that thread q of the quad holds columns 16q..16q+15 of its row; one 32-byte store per thread then makes every warp
// store instruction cover 8 rows x 128 contiguous bytes (8 lines) instead of 32 rows x 32 bytes (32 lines).
// `dst` points at (first row of the block, first column of the block); rows g and g+8 of the block are written.
__device__ __forceinline__ void epilogue_store_quad(__nv_bfloat16* dst, long long ldc, const uint32_t (&r)[32], int lane) {
  const int qd = lane & 3, g = lane >> 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {   // h = 0: row g, h = 1: row g + 8
    uint32_t x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = pack_bf16x2(__uint_as_float(r[4 * i + 2 * h]), __uint_as_float(r[4 * i + 2 * h + 1]));
    // block j = (x[2j], x[2j+1]) = columns 16j + 2qd (+1) and 16j + 8 + 2qd (+1); transpose blocks across the quad
#pragma unroll
    for (int s = 1; s <= 2; s <<= 1) {
      const bool upper = (qd & s) != 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j & s) continue;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t lo = x[2 * j + e], hi = x[2 * (j ^ s) + e];
          const uint32_t got = __shfl_xor_sync(0xffffffffu, upper ? lo : hi, s);
          if (upper) x[2 * j + e] = got;
          else x[2 * (j ^ s) + e] = got;
        }
      }
    }
    // now block j came from quad thread j: x[2j] = columns 16qd + 2j (+1), x[2j+1] = columns 16qd + 8 + 2j (+1)
    __nv_bfloat16* out = dst + static_cast<long long>(g + 8 * h) * ldc + 16 * qd;
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out), "r"(x[0]), "r"(x[2]), "r"(x[4]), "r"(x[6]),
                 "r"(x[1]), "r"(x[3]), "r"(x[5]), "r"(x[7])
                 : "memory");
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads + kMaxPushThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs p,
                 const __grid_constant__ GatherArgs g) {
  const int cta = static_cast<int>(blockIdx.x);
  const int n_ctas = static_cast<int>(gridDim.x);
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BN * kBK * 2;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + STAGES * B_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], kEpiWarps);
    }
    abort_flag[1] = p.status[3];   // wait limit in ms (0 = default)
    *abort_flag = (p.sc.enabled && !scatter_wait_owners(p.sc, p.status)) ? 1 : 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    constexpr bool is_a = true;
    if (lane == 0 && MB_DEBUG_MODE(p) != 1) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int s_rows = g.enabled ? g.rows_per_chunk * g.world : 1;
      const int m_rot = tile_rotation(g, p.sc, kBM);
      const int gbuf = static_cast<int>(g.seq & 1u);
      const unsigned* my_pad = g.enabled ? reinterpret_cast<const unsigned*>(g.pads[g.rank]) : nullptr;
      for (int tile = cta; ok && tile < total_tiles; tile += n_ctas) {
        int m_blk, n_blk;
        tile_coords(tile, p.tiles_m, p.tiles_n, m_blk, n_blk);
        m_blk = (m_blk + m_rot) % p.tiles_m;   // gather: own rows first; scatter: the next rank's rows first
        if (g.enabled && is_a) {
          // wait for a source only when its rows are needed
          const int row_lo = m_blk * kBM, row_hi = min(row_lo + kBM, p.M) - 1;
          const int src_lo = (row_lo % s_rows) / g.rows_per_chunk, src_hi = (row_hi % s_rows) / g.rows_per_chunk;
          bool ready = wait_flag_reached(my_pad + gbuf * 8 + src_lo, g.seq, abort_flag);
          if (ready && src_hi != src_lo) ready = wait_flag_reached(my_pad + gbuf * 8 + src_hi, g.seq, abort_flag);
          if (!ready) {
            *abort_flag = 1;
            atomicOr(&p.status[0], MB_ERR_PEER_TIMEOUT);
            p.status[2] = src_lo;
            ok = false;
            break;
          }
          fence_proxy_async_global();   // peers' generic-proxy stores -> this thread's TMA (async proxy) reads
        }
        const int m0 = m_blk * kBM, n0 = n_blk * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const int k0 = kb * kBK;
          {
            mbar_arrive_expect_tx(&full_bar[stage], A_BYTES + B_BYTES);
            uint8_t* a_dst = sA + stage * A_BYTES;
            if (!p.a_mn) {
              tma_load_2d(a_dst, &tmA, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[stage], m0 + 64 * j, k0);
            }
            uint8_t* b_dst = sB + stage * B_BYTES;
            if (!p.b_mn) {
              tma_load_2d(b_dst, &tmB, &full_bar[stage], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[stage], n0 + 64 * j, k0);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kBM, BN, p.a_mn, p.b_mn);
      // K-major: 8-row groups 1024 B apart, a k-step of 16 elements is 32 B inside the swizzle atom.
      // MN-major: 8-k groups 1024 B apart, 64-wide mn atoms 8192 B apart, a k-step of 16 is two groups.
      const uint32_t a_lbo = p.a_lbo, b_lbo = p.b_lbo, a_kstep = p.a_kstep, b_kstep = p.b_kstep;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; ok && tile < total_tiles; tile += n_ctas) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (MB_DEBUG_MODE(p) != 1 && !mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          if (MB_DEBUG_MODE(p) == 2) {   // timing probe: consume the stage without math
            mbar_arrive(&empty_bar[stage]);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + kk * a_kstep, a_lbo, p.a_sbo);
            const uint64_t bdesc = make_smem_desc_sw128(b_addr + kk * b_kstep, b_lbo, p.b_sbo);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete -> epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else if (warp >= kFirstPushWarp) {
    // ------------------------------------------------------------ all-gather push (fused launches only)
    // Every block carries push warps, so the copy is spread over all SMs and no block of the persistent GEMM is
    // delayed behind a copy-only block.
    if (g.bulk) {
      if (threadIdx.x == kGemmThreads)
        gather_push_role_bulk(g, p.K, p.status, n_ctas, smem + STAGES * (A_BYTES + B_BYTES) + 256, abort_flag);
    } else {
      gather_push_role(g, p.K, p.status, n_ctas);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = p.out_fp32 ? ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                   : ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const int m_rot_e = tile_rotation(g, p.sc, kBM);
    for (int tile = cta; tile < total_tiles; tile += n_ctas) {
      int m_blk, n_blk;
      tile_coords(tile, p.tiles_m, p.tiles_n, m_blk, n_blk);
      m_blk = (m_blk + m_rot_e) % p.tiles_m;
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_blk * kBM + q * 32 + lane;
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row < p.M && col0 < p.N) epilogue_store32(p, row, col0, r, vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  if (p.sc.enabled) __threadfence_system();   // this thread's partial-tile stores to peer memory
  __syncthreads();
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before the CTA's shared memory goes away.
    __nanosleep(50000);
    if (threadIdx.x == 0) {
      atomicOr(&p.status[0], MB_ERR_MBAR_TIMEOUT);
      p.status[1] = static_cast<int>(blockIdx.x);
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.sc.enabled && threadIdx.x == 0 && !*abort_flag) scatter_publish(p.sc, gridDim.x);
  if (g.enabled && threadIdx.x == 0 && !*abort_flag) {
    // the last GEMM block to finish tells every rank that this rank's gathered buffer may be overwritten
    unsigned* my_pad = reinterpret_cast<unsigned*>(g.pads[g.rank]);
    const unsigned done = atomicAdd(my_pad + 32, 1u);
    if (done == static_cast<unsigned>(n_ctas - 1)) {
      atomicExch(my_pad + 32, 0u);
      __threadfence_system();
      const int gbuf = static_cast<int>(g.seq & 1u);
      for (int r = 0; r < g.world; ++r) st_release_sys(reinterpret_cast<unsigned*>(g.pads[r]) + 16 + gbuf * 8 + g.rank, g.seq);
    }
  }
}

// ---------------------------------------------------------------------------------------------- CTA-pair kernel
// 256x256 output tiles computed by a cluster of two CTAs with ONE tcgen05.mma.cta_group::2 stream: CTA r of the pair
// stages rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the B tile (its half of N) in its
// own shared memory, the even CTA issues M=256 x N=256 UMMAs that read both CTAs' shared memory, and each CTA's TMEM
// receives its 128 output rows. Per CTA and k-block that is 32 KB of shared-memory operand traffic for 8.4 MFLOP,
// half the bytes per FLOP of the single-CTA 128x256 tile, which is what lifts the kernel off the shared-memory
// bandwidth limit. Barriers: full[s] lives in the leader and counts the TMA bytes of both CTAs; empty[s] and
// tfull[a] exist in both CTAs and are signalled by one commit addressed to both; tempty[a] lives in the leader and
// collects the epilogue warps of both CTAs.
#ifdef MB_GEMM_PROBE
static int g_debug_max_pairs = 0;   // probe builds: cap on the number of CTA pairs (0 = all)
#else
constexpr int g_debug_max_pairs = 0;
#endif
static int g_push_split = [] {       // 1: the all-gather push runs as its own launch in front of the GEMM
  const char* e = getenv("MALTOS_B200_PUSH_SPLIT");
  return e ? atoi(e) : 0;
}();
static int g_tail_split = [] {
  const char* e = getenv("MALTOS_B200_GEMM_TAIL_SPLIT");
  return e ? atoi(e) : 1;
}();

// Workspace of the split tail, one per (device, stream) so that launches on different streams never share partials.
// At most 74 tail tiles x slices of 512 KB each; allocated on first use and kept.
struct TailWorkspace {
  int dev;
  cudaStream_t stream;
  float* partials;
  unsigned* counters;
};
constexpr size_t kTailPartialBytes = 74ull * 2 * 128 * 512 * sizeof(float);
// Number of k slices for the tiles of the last wave (1 = no split): see GemmArgs::tail_split and the cost note in the
// launcher. `total` tiles on `pairs` CTA pairs, `k_blocks` k-blocks per tile.
static int tail_slices(int total, int pairs, int k_blocks) {
  if (!g_tail_split || pairs <= 0) return 1;
  const int rem = total % pairs;
  int s = rem > 0 ? pairs / rem : 1;
  if (s > 4) s = 4;
  while (s > 1 && k_blocks / s < 8) --s;
  if (s > 1 && k_blocks * 1080.0 * (1.0 - 1.0 / s) - 70000.0 <= 0.0) s = 1;
  return s;
}
static TailWorkspace g_tail_ws[16];
static int g_tail_ws_count = 0;
static std::mutex g_tail_ws_mutex;
static TailWorkspace* tail_workspace(int dev, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_tail_ws_mutex);
  for (int i = 0; i < g_tail_ws_count; ++i)
    if (g_tail_ws[i].dev == dev && g_tail_ws[i].stream == stream) return &g_tail_ws[i];
  if (g_tail_ws_count == 16) return nullptr;
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) return nullptr;
  TailWorkspace w{dev, stream, nullptr, nullptr};
  if (cudaMalloc(&w.partials, kTailPartialBytes) != cudaSuccess) return nullptr;
  if (cudaMalloc(&w.counters, 74 * 16 * sizeof(unsigned)) != cudaSuccess) {
    cudaFree(w.partials);
    return nullptr;
  }
  g_tail_ws[g_tail_ws_count] = w;
  return &g_tail_ws[g_tail_ws_count++];
}
constexpr int kPairStages = 6;
constexpr int kPairTile = 256;
constexpr int kWideStages = 4;   // 256x512 tiles: 48 KB per stage and CTA

// One unit of work of a CTA pair: a whole tile, or (split tail) one k range of a tile of the last wave.
struct WorkUnit {
  int tile;        // -1: nothing left
  int kb0, kb1;    // k-block range
  int slice;       // index of the k range, 0 when the tile is not split
  int tail_idx;    // index among the tail tiles (for the workspace), -1 when not split
};
__device__ __forceinline__ WorkUnit work_unit(int it, int pair, int n_pairs, int total_tiles, int k_blocks, int split) {
  WorkUnit u{-1, 0, k_blocks, 0, -1};
  if (split <= 1) {
    const int tile = pair + it * n_pairs;
    if (tile < total_tiles) u.tile = tile;
    return u;
  }
  const int full_iters = total_tiles / n_pairs, rem = total_tiles - full_iters * n_pairs;
  if (it < full_iters) {
    u.tile = pair + it * n_pairs;
  } else if (it == full_iters && pair < rem * split) {
    u.tail_idx = pair % rem;
    u.slice = pair / rem;
    u.tile = full_iters * n_pairs + u.tail_idx;
    u.kb0 = static_cast<int>(static_cast<long long>(k_blocks) * u.slice / split);
    u.kb1 = static_cast<int>(static_cast<long long>(k_blocks) * (u.slice + 1) / split);
  }
  return u;
}

template <bool WIDE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((WIDE ? kWideThreads : kGemmThreads) + kMaxPushThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs p,
                      const __grid_constant__ GatherArgs g) {
  // WIDE: the tile is 256x512 - every k-step issues two N=256 UMMAs that share the A stage, each CTA stages 256 rows
  // of B, and the single 512-column accumulator fills TMEM (the epilogue is then not overlapped with the next tile).
  // Per FLOP this moves a third less data through shared memory (TMA writes + UMMA operand reads share its bandwidth,
  // which is what limits the 256x256 and the single-CTA kernels).
  constexpr int STAGES = WIDE ? kWideStages : kPairStages;
  constexpr int B_ROWS = WIDE ? 256 : 128;          // rows of B staged per CTA
  constexpr int TILE_N = 2 * B_ROWS;
  constexpr int N_ACC = WIDE ? 1 : 2;               // accumulator buffers in TMEM
  constexpr int EPI_WARPS = WIDE ? 2 * kEpiWarps : kEpiWarps;   // WIDE: two groups of four, each drains 256 columns
  constexpr int FIRST_PUSH_THREAD = WIDE ? kWideThreads : kGemmThreads;
  constexpr int A_BYTES = 128 * kBK * 2;
  constexpr int B_BYTES = B_ROWS * kBK * 2;
  constexpr uint32_t TMEM_COLS = 512;   // two 256-column fp32 accumulators, or one of 512 columns
  const uint32_t cta_rank = cluster_cta_rank();
  const bool leader = cta_rank == 0;
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  const int n_pairs = static_cast<int>(gridDim.x) >> 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + STAGES * B_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;   // in 256x256 tiles
  const int n_stages = (p.stages > 0 && p.stages < STAGES) ? p.stages : STAGES;   // ring depth actually used (debug)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 2 * EPI_WARPS);
    }
    abort_flag[1] = p.status[3];   // wait limit in ms (0 = default)
    *abort_flag = (p.sc.enabled && !scatter_wait_owners(p.sc, p.status)) ? 1 : 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);   // the whole TMEM of this SM: both CTAs of the pair get base column 0
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // barriers of both CTAs are initialised before any remote arrive / TMA completion targets them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tmem_base != 0 && threadIdx.x == 0) {   // the pair's UMMA needs the same TMEM address in both CTAs
    *abort_flag = 1;
    atomicOr(&p.status[0], MB_ERR_BAD_INDEX);
  }
  __syncthreads();

  const int m_rot = tile_rotation(g, p.sc, kPairTile);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    constexpr bool is_a = true;
    if (lane == 0 && !*abort_flag && MB_DEBUG_MODE(p) != 1) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int s_rows = g.enabled ? g.rows_per_chunk * g.world : 1;
      const int gbuf = static_cast<int>(g.seq & 1u);
      const unsigned* my_pad = g.enabled ? reinterpret_cast<const unsigned*>(g.pads[g.rank]) : nullptr;
      uint32_t full_addr[STAGES];
#pragma unroll
      for (int s = 0; s < STAGES; ++s) full_addr[s] = mapa_u32(&full_bar[s], 0);
      long long t_empty = 0;
      int n_issued = 0;
      for (int it = 0; ok; ++it) {
        const WorkUnit wu = work_unit(it, pair, n_pairs, total_tiles, p.k_blocks, p.tail_split);
        if (wu.tile < 0) break;
        int m_blk, n_blk;
        tile_coords(wu.tile, p.tiles_m, p.tiles_n, m_blk, n_blk, p.group_m);
        m_blk = (m_blk + m_rot) % p.tiles_m;
        const int m0 = m_blk * kPairTile + static_cast<int>(cta_rank) * 128;
        const int n0 = n_blk * TILE_N + static_cast<int>(cta_rank) * B_ROWS;
        if (is_a && g.enabled && m0 < p.M) {
          const int row_hi = min(m0 + 128, p.M) - 1;
          const int src_lo = (m0 % s_rows) / g.rows_per_chunk, src_hi = (row_hi % s_rows) / g.rows_per_chunk;
          bool ready = wait_flag_reached(my_pad + gbuf * 8 + src_lo, g.seq, abort_flag);
          if (ready && src_hi != src_lo) ready = wait_flag_reached(my_pad + gbuf * 8 + src_hi, g.seq, abort_flag);
          if (!ready) {
            *abort_flag = 1;
            atomicOr(&p.status[0], MB_ERR_PEER_TIMEOUT);
            p.status[2] = src_lo;
            break;
          }
          fence_proxy_async_global();
        }
        for (int kb = wu.kb0; kb < wu.kb1; ++kb) {
          const long long t0 = MB_CLOCK();
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          t_empty += MB_CLOCK() - t0;
          if (is_a && MB_TRACE(p) && n_issued < 64) MB_TRACE(p)[4 * gridDim.x + blockIdx.x * 256 + n_issued] = MB_CLOCK();   // stage free seen / TMA issue
          ++n_issued;
          const int k0 = kb * kBK;
          {
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * (A_BYTES + B_BYTES));
            uint8_t* a_dst = sA + stage * A_BYTES;
            if (!p.a_mn) {
              tma_load_2d_pair(a_dst, &tmA, full_addr[stage], k0, m0);
            } else {
              tma_load_2d_pair(a_dst, &tmA, full_addr[stage], m0, k0);
              tma_load_2d_pair(a_dst + 8192, &tmA, full_addr[stage], m0 + 64, k0);
            }
            uint8_t* b_dst = sB + stage * B_BYTES;
            if (!p.b_mn) {
              tma_load_2d_pair(b_dst, &tmB, full_addr[stage], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < B_ROWS / 64; ++j) tma_load_2d_pair(b_dst + j * 8192, &tmB, full_addr[stage], n0 + 64 * j, k0);
            }
          }
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (is_a && MB_TRACE(p)) MB_TRACE(p)[4 * blockIdx.x + 3] = t_empty;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0 && !*abort_flag) {
      const uint32_t idesc = make_idesc_bf16(kPairTile, kPairTile, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_lbo, b_lbo = p.b_lbo, a_kstep = p.a_kstep, b_kstep = p.b_kstep;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      long long t_full = 0, t_tempty = 0;
      int n_seen = 0;
      const long long t_begin = MB_CLOCK();
      for (int it = 0; ok; ++it) {
        const WorkUnit wu = work_unit(it, pair, n_pairs, total_tiles, p.k_blocks, p.tail_split);
        if (wu.tile < 0) break;
        long long t0 = MB_CLOCK();
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) break;
        t_tempty += MB_CLOCK() - t0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPairTile);
        for (int kb = wu.kb0; kb < wu.kb1; ++kb) {
          t0 = MB_CLOCK();
          if (MB_DEBUG_MODE(p) != 1 && !mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          t_full += MB_CLOCK() - t0;
          if (MB_TRACE(p) && n_seen < 64) MB_TRACE(p)[4 * gridDim.x + blockIdx.x * 256 + 64 + n_seen] = MB_CLOCK();      // data seen
          ++n_seen;
          if (MB_DEBUG_MODE(p) == 2) {   // consume the stage without math: release it in both CTAs
            mbar_arrive(&empty_bar[stage]);
            mbar_arrive_cluster(mapa_u32(&empty_bar[stage], 1));
            if (++stage == n_stages) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + kk * a_kstep, a_lbo, p.a_sbo);
            const uint64_t bdesc = make_smem_desc_sw128(b_addr + kk * b_kstep, b_lbo, p.b_sbo);
            const uint32_t accumulate = (kb != wu.kb0 || kk != 0) ? 1u : 0u;
            umma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, accumulate);
            if (WIDE) {   // second half of the tile: rows 128..255 of this CTA's B stage, accumulator columns 256..511
              const uint64_t bdesc2 = make_smem_desc_sw128(b_addr + 16384 + kk * b_kstep, b_lbo, p.b_sbo);
              umma_bf16_ss_pair(d_tmem + 256, adesc, bdesc2, idesc, accumulate);
            }
          }
          umma_commit_pair(&empty_bar[stage], 3);   // both CTAs may refill this stage
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc], 3);       // accumulator complete in both CTAs' TMEM
        if (++acc == N_ACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (MB_TRACE(p)) {
        long long* t = MB_TRACE(p) + 4 * blockIdx.x;
        t[0] = MB_CLOCK() - t_begin, t[1] = t_full, t[2] = t_tempty;
      }
    }
    __syncwarp();
  } else if (warp >= FIRST_PUSH_THREAD / 32) {
    if (g.bulk) {
      if (threadIdx.x == FIRST_PUSH_THREAD)
        gather_push_role_bulk(g, p.K, p.status, static_cast<int>(gridDim.x), smem + STAGES * (A_BYTES + B_BYTES) + 256, abort_flag);
    } else {
      gather_push_role(g, p.K, p.status, static_cast<int>(gridDim.x), FIRST_PUSH_THREAD);
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = p.out_fp32 ? ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                   : ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    // (fused reduce-scatter: slots are 256-byte aligned and a 16-row block must not straddle two owners)
    const bool quad_ok = WIDE && p.quad_epilogue && !p.out_fp32 && !p.accumulate && !p.bias && (p.ldc & 15) == 0 &&
                         (p.sc.enabled ? (p.sc.rows_per_chunk & 15) == 0 : (reinterpret_cast<uintptr_t>(p.C) & 31) == 0);
    const uint32_t tempty_leader[2] = {mapa_u32(&tempty_bar[0], 0), mapa_u32(&tempty_bar[1], 0)};
    for (int it = 0;; ++it) {
      const WorkUnit wu = work_unit(it, pair, n_pairs, total_tiles, p.k_blocks, p.tail_split);
      if (wu.tile < 0) break;
      int m_blk, n_blk;
      tile_coords(wu.tile, p.tiles_m, p.tiles_n, m_blk, n_blk, p.group_m);
      m_blk = (m_blk + m_rot) % p.tiles_m;
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_blk * kPairTile + static_cast<int>(cta_rank) * 128 + q * 32 + lane;
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * kPairTile) + (static_cast<uint32_t>(q * 32) << 16);
      // Two chunks of 32 columns are kept in flight: the TMEM load of the next chunk is issued before the current one
      // is converted and stored. In the 256x512 kernel warps 2..5 drain columns 0..255 and warps 6..9 columns 256..511.
      const int c_begin = (WIDE && warp >= kFirstPushWarp) ? 8 : 0;
      const int c_end = WIDE ? c_begin + 8 : TILE_N / 32;
      auto out_col = [&](int c) {
        // accumulator columns -> output columns: each UMMA writes CTA 0's B rows first, then CTA 1's
        return WIDE ? n_blk * TILE_N + ((c & 4) ? 256 : 0) + (c >> 3) * 128 + (c & 3) * 32 : n_blk * kPairTile + c * 32;
      };
      uint32_t ra[32], rb[32];
      const int tile_row0 = m_blk * kPairTile + static_cast<int>(cta_rank) * 128;
      const int tile_col0 = n_blk * (WIDE ? TILE_N : kPairTile);
      if (WIDE && wu.tail_idx >= 0) {
        // ---- split tail: fp32 partial of this warp's 32 rows x 256 columns -> workspace; the last arriver reduces
        const int ew = warp - 2;                                     // 0..7: lane quarter q, column half ew / 4
        const long long blk_elems = 128ll * 512;                     // one CTA's share of a tile
        float* ws_tile = p.tail_ws + (static_cast<long long>(wu.tail_idx) * p.tail_split * 2) * blk_elems;
        float* mine = ws_tile + (static_cast<long long>(wu.slice) * 2 + cta_rank) * blk_elems + static_cast<long long>(q * 32 + lane) * 512;
        for (int c = c_begin; c < c_end; ++c) {
          tmem_ld_32x32b_x32(t_row + c * 32, ra);
          tmem_ld_wait();
          float4* dst = reinterpret_cast<float4*>(mine + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(ra[4 * i]), __uint_as_float(ra[4 * i + 1]), __uint_as_float(ra[4 * i + 2]),
                                 __uint_as_float(ra[4 * i + 3]));
        }
        // the accumulator is free again as soon as it has been read
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader[acc]);
        __threadfence();
        __syncwarp();
        unsigned arrived = 0;
        if (lane == 0) arrived = atomicAdd(p.tail_cnt + (wu.tail_idx * 2 + static_cast<int>(cta_rank)) * 8 + ew, 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == static_cast<unsigned>(p.tail_split - 1)) {
          __threadfence();
          for (int c = c_begin; c < c_end; ++c) {
            float acc32[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc32[i] = 0.f;
            for (int sl = 0; sl < p.tail_split; ++sl) {
              const float4* src = reinterpret_cast<const float4*>(ws_tile + (static_cast<long long>(sl) * 2 + cta_rank) * blk_elems +
                                                                  static_cast<long long>(q * 32 + lane) * 512 + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 v = __ldcg(src + i);
                acc32[4 * i] += v.x, acc32[4 * i + 1] += v.y, acc32[4 * i + 2] += v.z, acc32[4 * i + 3] += v.w;
              }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(acc32[i]);
            const int col0 = out_col(c);
            if (row < p.M && col0 < p.N) epilogue_store32(p, row, col0, ra, vec_ok);
          }
        }
        if (++acc == N_ACC) {
          acc = 0;
          acc_phase ^= 1;
        }
        continue;
      }
      if (quad_ok && tile_row0 + 128 <= p.M && tile_col0 + (WIDE ? TILE_N : kPairTile) <= p.N) {
        // interior tile, plain bf16 output: 16-row x 64-column blocks, whole 128-byte lines per store instruction
        // first row of a 16-row block -> where it is stored: C, or (fused reduce-scatter) the owner's staging slot
        auto block_base = [&](int r0) -> __nv_bfloat16* {
          if (!p.sc.enabled) return reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(r0) * p.ldc;
          const int b = r0 / p.sc.s_rows, s = r0 - b * p.sc.s_rows;
          const int owner = s / p.sc.rows_per_chunk;
          const long long local = static_cast<long long>(b) * p.sc.rows_per_chunk + (s - owner * p.sc.rows_per_chunk);
          return reinterpret_cast<__nv_bfloat16*>(p.sc.slot_base[owner]) + local * p.ldc;
        };
        __nv_bfloat16* c_lo = block_base(tile_row0 + q * 32);
        __nv_bfloat16* c_hi = block_base(tile_row0 + q * 32 + 16);
        const uint32_t t_lo = tmem_base + static_cast<uint32_t>(acc * kPairTile) + (static_cast<uint32_t>(q * 32) << 16);
        const uint32_t t_hi = t_lo + (16u << 16);
        tmem_ld_16x256b_x8(t_lo + c_begin * 32, ra);
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {
          tmem_ld_wait();
          tmem_ld_16x256b_x8(t_hi + c * 32, rb);
          const int col = out_col(c);
          epilogue_store_quad(c_lo + col, p.ldc, ra, lane);
          tmem_ld_wait();
          if (c + 2 < c_end) tmem_ld_16x256b_x8(t_lo + (c + 2) * 32, ra);
          epilogue_store_quad(c_hi + col, p.ldc, rb, lane);
        }
      } else {
        tmem_ld_32x32b_x32(t_row + c_begin * 32, ra);
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x32b_x32(t_row + (c + 1) * 32, rb);
          int col0 = out_col(c);
          if (row < p.M && col0 < p.N) epilogue_store32(p, row, col0, ra, vec_ok);
          tmem_ld_wait();
          if (c + 2 < c_end) tmem_ld_32x32b_x32(t_row + (c + 2) * 32, ra);
          col0 = out_col(c + 1);
          if (row < p.M && col0 < p.N) epilogue_store32(p, row, col0, rb, vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader[acc]);
      if (++acc == N_ACC) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  if (p.sc.enabled) __threadfence_system();   // this thread's partial-tile stores to peer memory
  __syncthreads();
  // Neither CTA may leave while the other can still read its shared memory (UMMA operands) or signal its barriers.
  cluster_arrive();
  cluster_wait();
  if (*abort_flag) {
    __nanosleep(50000);
    if (threadIdx.x == 0) {
      atomicOr(&p.status[0], MB_ERR_MBAR_TIMEOUT);
      p.status[1] = static_cast<int>(blockIdx.x);
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.sc.enabled && threadIdx.x == 0 && !*abort_flag) scatter_publish(p.sc, gridDim.x);
  if (g.enabled && threadIdx.x == 0 && !*abort_flag) {
    unsigned* my_pad = reinterpret_cast<unsigned*>(g.pads[g.rank]);
    const unsigned done = atomicAdd(my_pad + 32, 1u);
    if (done == gridDim.x - 1) {
      atomicExch(my_pad + 32, 0u);
      __threadfence_system();
      const int gbuf = static_cast<int>(g.seq & 1u);
      for (int r = 0; r < g.world; ++r) st_release_sys(reinterpret_cast<unsigned*>(g.pads[r]) + 16 + gbuf * 8 + g.rank, g.seq);
    }
  }
}

template <bool WIDE>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& args, cudaStream_t stream,
                            const GatherArgs* gather = nullptr) {
  constexpr int stages = WIDE ? kWideStages : kPairStages;
  constexpr int tile_n = WIDE ? 512 : 256;
  constexpr size_t smem_base = 1024 + stages * ((128 + tile_n / 2) * kBK * 2) + 256;
  constexpr size_t smem_max = smem_base + kPushSmemBytes;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    MB_CHECK_CUDA(cudaFuncSetAttribute(gemm_bf16_pair_kernel<WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_max)));
    configured[dev & 63] = true;
  }
  args.tiles_m = (args.M + kPairTile - 1) / kPairTile;
  args.tiles_n = (args.N + tile_n - 1) / tile_n;
  const int total = args.tiles_m * args.tiles_n;
  GatherArgs g;
  if (gather) {
    g = *gather;
  } else {
    g.enabled = 0;
    g.push_ctas = 0;
    g.bulk = 0;
  }
  const int max_pairs = g_debug_max_pairs > 0 ? g_debug_max_pairs : sm_count() / 2;
  // Split tail: see GemmArgs. Worth it when the k range saved per pair outweighs writing and re-reading the fp32 partials
  // (about 70k cycles, measured on 8192x4096: K=6144 -2 %, K=7168 0 %, K=14336 +5 %, K=28672 +8 %): with s slices the last
  // wave shrinks by (1 - 1/s) of a tile's main loop.
  args.tail_split = 1;
  args.tail_ws = nullptr;
  args.tail_cnt = nullptr;
  int split_pairs = 0;
  if (WIDE && !g.enabled && !args.sc.enabled && g_tail_split && args.debug_mode == 0 && args.trace == nullptr) {
    const int rem = total % max_pairs;
    const int s = tail_slices(total, max_pairs, args.k_blocks);
    TailWorkspace* ws = s > 1 ? tail_workspace(dev, stream) : nullptr;
    if (ws) {
      args.tail_split = s;
      args.tail_ws = ws->partials;
      args.tail_cnt = ws->counters;
      split_pairs = max_pairs;
      MB_CHECK_CUDA(cudaMemsetAsync(ws->counters, 0, static_cast<size_t>(rem) * 16 * sizeof(unsigned), stream));
    }
  }
  const int grid = split_pairs > 0 ? 2 * split_pairs : 2 * (total < max_pairs ? total : max_pairs);
  const int base_threads = WIDE ? kWideThreads : kGemmThreads;
  const int threads = g.enabled ? base_threads + 32 * g.push_ctas : base_threads;
  const size_t smem = (g.enabled && g.bulk) ? smem_max : smem_base;
  gemm_bf16_pair_kernel<WIDE><<<grid, threads, smem, stream>>>(tmA, tmB, args, g);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Kernel choice. Relative throughputs per SM measured on B200 at K = 4096 (fraction of the math-only rate of the
// pipeline): 256x512 pair tiles ~0.9, 256x256 pair tiles and 128x256 single-CTA tiles ~0.7 (shared-memory bandwidth
// bound: TMA writes and UMMA operand reads share it), 128x128 tiles ~0.4. The estimate is waves x tile area / rate;
// wide tiles lose when the problem has too few of them to fill the 74 SM pairs.
enum GemmKind { kKindSingle128 = 128, kKindSingle256 = 256, kKindPair = 512, kKindWide = 1024 };

static GemmKind choose_gemm_kind(int M, int N, int K, bool plain = true) {   // plain: no fused collective in the launch
  // Estimated cycles = waves x cycles per tile. Per k-block of 64: 128x128 tiles ~640 cycles, 128x256 tiles ~850 (both
  // shared-memory bound, epilogue overlapped with the next tile's MMAs), 256x512 pair tiles ~1080 (tensor-pipe bound)
  // plus ~5000 cycles of epilogue that cannot overlap because the accumulator fills tensor memory. With few k-blocks
  // the 256x512 tile therefore loses to 128x256 (measured on 8192x4096: K=512 51 vs 45 us, K=1024 75 vs 75, K=1792 110
  // vs 120), and it loses when the problem has too few tiles to fill the 74 SM pairs.
  const int sms = sm_count(), pairs = sms / 2;
  const double kb = static_cast<double>((K + kBK - 1) / kBK);
  auto waves = [&](int tm, int tn, int slots) {
    const long long tiles = static_cast<long long>((M + tm - 1) / tm) * ((N + tn - 1) / tn);
    return static_cast<double>((tiles + slots - 1) / slots);
  };
  GemmKind best = kKindSingle128;
  double best_cost = waves(128, 128, sms) * (kb * 640.0 > 1500.0 ? kb * 640.0 : 1500.0);
  const double c256 = waves(128, 256, sms) * (kb * 850.0 > 3000.0 ? kb * 850.0 : 3000.0);
  if (c256 < best_cost) best = kKindSingle256, best_cost = c256;
  double cwide = waves(256, 512, pairs) * (kb * 1080.0 + 5000.0);
  {
    // with the split tail the last wave costs 1/slices of a main loop plus the partial exchange
    const int wide_tiles = ((M + 255) / 256) * ((N + 511) / 512);
    const int s = plain ? tail_slices(wide_tiles, pairs, static_cast<int>(kb)) : 1;
    if (s > 1) cwide = (wide_tiles / pairs) * (kb * 1080.0 + 5000.0) + kb * 1080.0 / s + 5000.0 + 70000.0;
  }
  if (cwide < best_cost) best = kKindWide, best_cost = cwide;
  return best;
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& args, cudaStream_t stream,
                       const GatherArgs* gather = nullptr) {
  constexpr size_t smem_base = 1024 + STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 256;
  constexpr size_t smem_max = smem_base + kPushSmemBytes;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    MB_CHECK_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_max)));
    configured[dev & 63] = true;
  }
  args.tiles_n = (args.N + BN - 1) / BN;
  const int total = args.tiles_m * args.tiles_n;
  GatherArgs g;
  if (gather) {
    g = *gather;
  } else {
    g.enabled = 0;
    g.push_ctas = 0;
    g.bulk = 0;
  }
  const int grid = total < sm_count() ? total : sm_count();
  const int threads = g.enabled ? kGemmThreads + 32 * g.push_ctas : kGemmThreads;
  const size_t smem = (g.enabled && g.bulk) ? smem_max : smem_base;
  gemm_bf16_kernel<BN, STAGES><<<grid, threads, smem, stream>>>(tmA, tmB, args, g);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Owner side of the fused reduce-scatter: out[r, :] = sum over sources of slot[src][r, :] (fp32 accumulation), after
// every source's flag for this call has arrived. One thread per block does the (bounded) waiting.
__global__ void __launch_bounds__(256)
rs_reduce_kernel(const __nv_bfloat16* __restrict__ stage, long long slot_elems, int world, int rank, unsigned seq,
                 const unsigned long long* __restrict__ pads_dev, unsigned long long my_pad_addr, __nv_bfloat16* __restrict__ out,
                 long long n_vec, int* status) {
  __shared__ int s_ok;
  unsigned* my_pad = reinterpret_cast<unsigned*>(my_pad_addr);
  const int buf = static_cast<int>(seq & 1u);
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int src = 0; ok && src < world; ++src) ok = wait_flag_reached(my_pad + 64 + buf * 8 + src, seq, nullptr);
    if (!ok) atomicOr(&status[0], MB_ERR_PEER_TIMEOUT);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (s_ok) {
    const uint4* base = reinterpret_cast<const uint4*>(stage);
    const long long slot_vec = slot_elems >> 3;
    for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int src = 0; src < world; ++src) {
        const uint4 q = base[src * slot_vec + v];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]), o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]), o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out)[v] = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(my_pad + 129, 1u);
    if (done == gridDim.x - 1) {   // staging buffer fully read: every writer may reuse its slot two calls from now
      atomicExch(my_pad + 129, 0u);
      __threadfence_system();
      for (int r = 0; r < world; ++r) st_release_sys(reinterpret_cast<unsigned*>(pads_dev[r]) + 96 + buf * 8 + rank, seq);
    }
  }
}

#ifdef MB_GEMM_PROBE
// Probe builds only: override of the descriptor geometry {lbo, sbo, kstep} per operand (negative = built-in value), cycle
// trace buffer, math-only / load-only modes, ring depth.
static int g_desc_override[6] = {-1, -1, -1, -1, -1, -1};
static long long* g_trace = nullptr;
static int g_debug_mode = 0;
static int g_debug_stages = 0;
#else
constexpr int g_desc_override[6] = {-1, -1, -1, -1, -1, -1};
constexpr long long* g_trace = nullptr;
constexpr int g_debug_mode = 0;
constexpr int g_debug_stages = 0;
#endif
static int g_pair_group_m = 8;
static int g_quad_epilogue = [] {
  const char* e = getenv("MALTOS_B200_QUAD_EPILOGUE");
  return e ? atoi(e) : 1;
}();
static int g_push_bulk = 0;      // fused all-gather: 1 = push with bulk async copies, 0 = push with the copy warps
static int g_scatter_kind = 0;   // tuning: kernel kind forced for the fused reduce-scatter GEMM (0 = cost model)

}  // namespace mb

#ifdef MB_GEMM_PROBE
// Device buffer of 4 int64 per CTA that the CTA-pair kernel fills with cycle counters (nullptr = off).
MB_API void mb_gemm_set_trace(long long* buf) { mb::g_trace = buf; }
// Timing probes of the CTA-pair kernel (results are meaningless): 1 = math only, 2 = loads only, 0 = normal.
MB_API void mb_gemm_set_debug_mode(int mode) { mb::g_debug_mode = mode; }
MB_API void mb_gemm_set_debug_stages(int stages) { mb::g_debug_stages = stages; }
// Cap the number of CTA pairs of the pair kernel (0 = one pair per two SMs).
MB_API void mb_gemm_set_debug_max_pairs(int pairs) { mb::g_debug_max_pairs = pairs; }
MB_API void mb_gemm_debug_descriptor(int a_lbo, int a_sbo, int a_kstep, int b_lbo, int b_sbo, int b_kstep) {
  int v[6] = {a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep};
  for (int i = 0; i < 6; ++i) mb::g_desc_override[i] = v[i];
}
#endif

// Tuning knob of the CTA-pair kernel: M blocks per rasterisation group. (An L2 prefetch stream ahead of the
// shared-memory ring was tried and removed: the extra L2 requests cost a third of the throughput.)
MB_API void mb_gemm_set_tuning(int group_m) {
  if (group_m > 0) mb::g_pair_group_m = group_m;
}
// 0 selects the row-per-thread epilogue everywhere, 1 the line-coalesced one where it applies
// (initial value: environment variable MALTOS_B200_QUAD_EPILOGUE, default 1).
MB_API void mb_gemm_set_quad_epilogue(int on) { mb::g_quad_epilogue = on ? 1 : 0; }
// 0 switches the split tail of the 256x512 kernel off (initial value: MALTOS_B200_GEMM_TAIL_SPLIT, default 1).
MB_API void mb_gemm_set_tail_split(int on) { mb::g_tail_split = on ? 1 : 0; }
MB_API void mb_gemm_set_scatter_kind(int kind) { mb::g_scatter_kind = kind; }
MB_API void mb_gemm_set_push_bulk(int on) { mb::g_push_bulk = on ? 1 : 0; }
MB_API void mb_gemm_set_push_split(int on) { mb::g_push_split = on ? 1 : 0; }
// C[M,N] (+)= op(A) op(B) (+bias). Leading dimensions are in elements; bf16 operands need them (and the base
// addresses) to be multiples of 8 elements / 16 bytes because the operands are fetched with TMA.
// block_n: 0 = choose; 128 or 256 = single-CTA kernel with that tile width; 512 = CTA-pair kernel (256x256 tiles);
// 1024 = CTA-pair kernel with 256x512 tiles.
MB_API int mb_gemm_bf16(const void* A, int a_mn, long long lda, const void* B, int b_mn, long long ldb, void* C,
                        long long ldc, int M, int N, int K, int out_fp32, int accumulate, const void* bias,
                        int block_n, cudaStream_t stream) {
  using namespace mb;
  if (M <= 0 || N <= 0 || K <= 0) {
    set_last_error("mb_gemm_bf16: empty problem");
    return -1;
  }
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) {
    set_last_error("mb_gemm_bf16: operands must be 16-byte aligned with leading dimensions multiple of 8");
    return -2;
  }
  int* status = status_ptr();
  if (!status) {
    set_last_error("mb_gemm_bf16: no status word");
    return -3;
  }
  GemmArgs args;
  args.C = C;
  args.bias = static_cast<const __nv_bfloat16*>(bias);
  args.ldc = ldc;
  args.M = M, args.N = N, args.K = K;
  args.a_mn = a_mn ? 1 : 0, args.b_mn = b_mn ? 1 : 0;
  args.out_fp32 = out_fp32, args.accumulate = accumulate;
  args.tiles_m = (M + kBM - 1) / kBM;
  args.k_blocks = (K + kBK - 1) / kBK;
  args.status = status;
  args.sc.enabled = 0;
  args.trace = g_trace;
  args.group_m = g_pair_group_m;
  args.debug_mode = g_debug_mode;
  args.quad_epilogue = g_quad_epilogue;
  args.stages = g_debug_stages;
  args.a_lbo = a_mn ? 8192u : 16u, args.a_sbo = 1024u, args.a_kstep = a_mn ? 2048u : 32u;
  args.b_lbo = b_mn ? 8192u : 16u, args.b_sbo = 1024u, args.b_kstep = b_mn ? 2048u : 32u;
  {
    unsigned* f[6] = {&args.a_lbo, &args.a_sbo, &args.a_kstep, &args.b_lbo, &args.b_sbo, &args.b_kstep};
    for (int i = 0; i < 6; ++i)
      if (g_desc_override[i] >= 0) *f[i] = static_cast<unsigned>(g_desc_override[i]);
  }

  const int kind = (block_n == 128 || block_n == 256 || block_n == 512 || block_n == 1024) ? block_n : choose_gemm_kind(M, N, K);
  const bool wide = kind == kKindWide, pair = wide || kind == kKindPair;
  const int bn = wide ? 256 : (pair ? 128 : kind);   // rows of B staged per CTA and k-block
  CUtensorMap tmA, tmB;
  bool ok;
  if (!a_mn)
    ok = encode_tmap_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kBK, kBM, 2, true);
  else
    ok = encode_tmap_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, kBK, 2, true);
  if (!ok) return -4;
  if (!b_mn)
    ok = encode_tmap_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, (uint32_t)bn, 2, true);
  else
    ok = encode_tmap_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kBK, 2, true);
  if (!ok) return -4;
  if (wide) return launch_gemm_pair<true>(tmA, tmB, args, stream);
  if (pair) return launch_gemm_pair<false>(tmA, tmB, args, stream);
  if (bn == 256) return launch_gemm<256, 4>(tmA, tmB, args, stream);
  return launch_gemm<128, 6>(tmA, tmB, args, stream);
}

// Sequence-parallel all-gather fused into a column-parallel GEMM:
//   C[B*S, N] = gather_over_ranks(x_local)[B*S, K] @ op(W),  op(W) = W[N, K]^T (b_mn = 0) or W[K, N] (b_mn = 1)
// x_local is this rank's [B * rows_per_chunk, K] slice (row stride x_ld). `gathered` / `pads` hold, for every rank of
// the group, the address at which that rank's double-buffered gathered buffer / signal pad is mapped in this process.
// `seq` is the call's sequence number (same on every rank, starting at 1, +1 per call on this context).
MB_API int mb_ag_gemm_bf16(const void* x_local, long long x_ld, int batches, int rows_per_chunk, const void* W, int b_mn,
                           long long ldb, void* C, long long ldc, int N, int K, int rank, int world, unsigned seq,
                           const unsigned long long* gathered, const unsigned long long* pads, long long buf_elems,
                           int push_ctas, cudaStream_t stream) {
  using namespace mb;
  if (world < 2 || world > kMaxPeers) {
    set_last_error("mb_ag_gemm_bf16: group size must be in [2, 8]");
    return -1;
  }
  if ((K & 7) || (x_ld & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(x_local) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15)) {
    set_last_error("mb_ag_gemm_bf16: operands must be 16-byte aligned with K and leading dimensions multiple of 8");
    return -2;
  }
  const long long M = static_cast<long long>(batches) * rows_per_chunk * world;
  if (M * K > buf_elems) {
    set_last_error("mb_ag_gemm_bf16: gathered buffer too small");
    return -3;
  }
  int* status = status_ptr();
  if (!status) return -4;
  GemmArgs args;
  args.C = C;
  args.bias = nullptr;
  args.ldc = ldc;
  args.M = static_cast<int>(M), args.N = N, args.K = K;
  args.a_mn = 0, args.b_mn = b_mn ? 1 : 0;
  args.out_fp32 = 0, args.accumulate = 0;
  args.tiles_m = (args.M + kBM - 1) / kBM;
  args.k_blocks = (K + kBK - 1) / kBK;
  args.status = status;
  args.sc.enabled = 0;
  args.trace = nullptr;
  args.group_m = g_pair_group_m;
  args.debug_mode = g_debug_mode;
  args.quad_epilogue = g_quad_epilogue;
  args.stages = g_debug_stages;
  args.a_lbo = 16u, args.a_sbo = 1024u, args.a_kstep = 32u;
  args.b_lbo = b_mn ? 8192u : 16u, args.b_sbo = 1024u, args.b_kstep = b_mn ? 2048u : 32u;
  GatherArgs g;
  g.enabled = 1;
  g.push_ctas = (push_ctas > 0 && push_ctas * 32 <= kMaxPushThreads) ? push_ctas : kMaxPushThreads / 32;
  g.bulk = (g_push_bulk && x_ld == K) ? 1 : 0;   // bulk copies need dense rows
  g.rank = rank, g.world = world;
  g.batches = batches, g.rows_per_chunk = rows_per_chunk;
  g.x_local = static_cast<const __nv_bfloat16*>(x_local);
  g.x_ld = x_ld;
  g.seq = seq;
  g.buf_elems = buf_elems;
  for (int r = 0; r < kMaxPeers; ++r) {
    g.gathered[r] = r < world ? gathered[r] : 0ull;
    g.pads[r] = r < world ? pads[r] : 0ull;
  }
  const __nv_bfloat16* a_base = reinterpret_cast<const __nv_bfloat16*>(gathered[rank]) + static_cast<long long>(seq & 1u) * buf_elems;
  const int kind = choose_gemm_kind(args.M, N, K, false);
  const bool wide = kind == kKindWide, pair = wide || kind == kKindPair;
  const int bn = wide ? 256 : (pair ? 128 : kind);
  CUtensorMap tmA, tmB;
  if (!encode_tmap_2d(&tmA, a_base, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kBM, 2, true)) return -5;
  if (!(b_mn ? encode_tmap_2d(&tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kBK, 2, true)
             : encode_tmap_2d(&tmB, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, (uint32_t)bn, 2, true)))
    return -5;
  if (g_push_split) {
    const long long rows_local = static_cast<long long>(batches) * rows_per_chunk;
    long long blocks = (rows_local + 3) / 4;
    if (blocks > 128) blocks = 128;
    ag_push_kernel<<<static_cast<unsigned>(blocks < 1 ? 1 : blocks), kPushKernelThreads, 0, stream>>>(g, K, status);
    count_launch();
    MB_CHECK_CUDA(cudaGetLastError());
    g.push_ctas = 0;      // the GEMM launch below has no push warps: it only waits for the flags
    g.bulk = 0;
  }
  if (wide) return launch_gemm_pair<true>(tmA, tmB, args, stream, &g);
  if (pair) return launch_gemm_pair<false>(tmA, tmB, args, stream, &g);
  if (bn == 256) return launch_gemm<256, 4>(tmA, tmB, args, stream, &g);
  return launch_gemm<128, 6>(tmA, tmB, args, stream, &g);
}

// Row-parallel GEMM fused with the sequence-parallel reduce-scatter:
//   out[B*S/T, N] = sum over ranks of (X[B*S, K_local] op(W))  restricted to this rank's rows
// op(W) = W[N, K]^T (b_mn = 0, forward of a row-parallel layer) or W[K, N] (b_mn = 1, input gradient of a column-parallel
// layer). `stage` / `pads`: for every rank, the address at which its double-buffered staging buffer (2 x world slots of
// B*S/T x N bf16) / signal pad is mapped here; `pads_dev` the same pad table in device memory. `seq` counts the calls
// of this entry point on the context (1, 2, ...), identical on all ranks.
MB_API int mb_gemm_rs_bf16(const void* X, long long lda, const void* W, int b_mn, long long ldb, void* out, int batches,
                           int rows_per_chunk, int N, int K, int rank, int world, unsigned seq,
                           const unsigned long long* stage, const unsigned long long* pads,
                           const unsigned long long* pads_dev, cudaStream_t stream) {
  using namespace mb;
  if (world < 2 || world > kMaxPeers) {
    set_last_error("mb_gemm_rs_bf16: group size must be in [2, 8]");
    return -1;
  }
  if ((N & 7) || (lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) {
    set_last_error("mb_gemm_rs_bf16: operands must be 16-byte aligned with N and leading dimensions multiple of 8");
    return -2;
  }
  int* status = status_ptr();
  if (!status) return -4;
  const long long rows_local = static_cast<long long>(batches) * rows_per_chunk;
  const long long M = rows_local * world;
  const long long slot_elems = rows_local * N;
  GemmArgs args;
  args.C = nullptr;
  args.bias = nullptr;
  args.ldc = N;
  args.M = static_cast<int>(M), args.N = N, args.K = K;
  args.a_mn = 0, args.b_mn = b_mn ? 1 : 0;
  args.out_fp32 = 0, args.accumulate = 0;
  args.tiles_m = (args.M + kBM - 1) / kBM;
  args.k_blocks = (K + kBK - 1) / kBK;
  args.status = status;
  args.trace = nullptr;
  args.group_m = g_pair_group_m;
  args.debug_mode = 0;
  args.quad_epilogue = g_quad_epilogue;
  args.stages = 0;
  args.a_lbo = 16u, args.a_sbo = 1024u, args.a_kstep = 32u;
  args.b_lbo = b_mn ? 8192u : 16u, args.b_sbo = 1024u, args.b_kstep = b_mn ? 2048u : 32u;
  ScatterArgs& sc = args.sc;
  sc.enabled = 1;
  sc.rank = rank, sc.world = world;
  sc.rows_per_chunk = rows_per_chunk, sc.s_rows = rows_per_chunk * world;
  sc.seq = seq;
  const long long buf_off = static_cast<long long>(seq & 1u) * world * slot_elems;
  for (int r = 0; r < kMaxPeers; ++r) {
    sc.slot_base[r] = r < world ? stage[r] + static_cast<unsigned long long>((buf_off + rank * slot_elems) * 2) : 0ull;
    sc.pads[r] = r < world ? pads[r] : 0ull;
  }
  int kind = choose_gemm_kind(args.M, N, K, false);
  if (g_scatter_kind > 0) kind = g_scatter_kind;
  const bool wide = kind == kKindWide, pair = wide || kind == kKindPair;
  const int bn = wide ? 256 : (pair ? 128 : kind);
  CUtensorMap tmA, tmB;
  if (!encode_tmap_2d(&tmA, X, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kBK, kBM, 2, true)) return -5;
  bool ok;
  if (!b_mn)
    ok = encode_tmap_2d(&tmB, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, (uint32_t)bn, 2, true);
  else
    ok = encode_tmap_2d(&tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kBK, 2, true);
  if (!ok) return -5;
  int rc;
  if (wide) rc = launch_gemm_pair<true>(tmA, tmB, args, stream);
  else if (pair) rc = launch_gemm_pair<false>(tmA, tmB, args, stream);
  else if (bn == 256) rc = launch_gemm<256, 4>(tmA, tmB, args, stream);
  else rc = launch_gemm<128, 6>(tmA, tmB, args, stream);
  if (rc != 0) return rc;
  const __nv_bfloat16* my_stage = reinterpret_cast<const __nv_bfloat16*>(stage[rank]) + buf_off;
  const long long n_vec = slot_elems >> 3;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 4LL * sm_count()) blocks = 4LL * sm_count();
  rs_reduce_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), 256, 0, stream>>>(
      my_stage, slot_elems, world, rank, seq, pads_dev, pads[rank], static_cast<__nv_bfloat16*>(out), n_vec, status);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
