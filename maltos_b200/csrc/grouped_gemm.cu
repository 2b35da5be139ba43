// Grouped bf16 GEMM on tcgen05 tensor cores for mixture-of-experts layers: ONE launch runs the GEMMs of all local
// experts, and how many rows each expert really has is read from DEVICE memory by the kernel's tile scheduler, so the
// host never learns the token counts (no synchronisation, static launch shapes, CUDA-graph friendly). The expert inputs
// sit in one capacity-bounded buffer [G, cap, .]; group g uses rows [g * cap, g * cap + count[g]).
//
//   mode 0 (forward)         C[g*cap + m, n] = sum_k A[g*cap + m, k] * B_g[n, k]        m < count[g]   (B_g: [N, K] weights)
//   mode 1 (input gradient)  C[g*cap + m, n] = sum_k A[g*cap + m, k] * B_g[k, n]        m < count[g]   (B_g: [K, N] weights)
//   mode 2 (weight gradient) C_g[m, n]       = sum_{r < count[g]} A[g*cap + r, m] * B[g*cap + r, n]     (C_g: [M, N] per group)
//
// Tiles whose rows lie beyond count[g] are skipped by all roles of the kernel; in mode 2 the reduction runs over
// ceil(count[g] / 64) row blocks (rows between count[g] and the block end must hold zeros in A, which the caller
// guarantees by clearing the gradient buffer before the rows are written). The per-expert operand of modes 0/1 has a
// tensor map of its own (the experts' weights need not be adjacent in memory), passed as a __grid_constant__ array.
// Persistent kernel, one CTA per SM: warp 0 = TMA producer (4-stage ring), warp 1 = UMMA issuer (128 x 256 tiles, two
// accumulators in TMEM so the epilogue of a tile runs under the MMAs of the next), warps 2..5 = epilogue.
// The reference runs one cuBLAS call per expert behind two host synchronisations (runtime/layers/moe.py:82-137).
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kGgBM = 128, kGgBN = 256, kGgBK = 64, kGgStages = 4;
constexpr int kGgThreads = 192;       // producer, MMA issuer, 4 epilogue warps
constexpr int kGgMaxGroups = 16;

struct GroupedMaps {
  CUtensorMap m[kGgMaxGroups];
};

struct GroupedArgs {
  int mode;
  int groups;
  int cap;                 // rows per group in the stacked activation buffers
  int M, N, K;             // per-group problem: modes 0/1: M = cap (bounded by count), mode 2: K = cap (bounded by count)
  int tiles_m, tiles_n, k_blocks;
  const int* counts;       // [groups] on the device
  void* c[kGgMaxGroups];   // mode 2: per-group outputs; modes 0/1: c[0] = stacked output [groups * cap, N]
  long long ldc;
  int out_fp32;
  int* status;
};

__global__ void __launch_bounds__(kGgThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB_single,
                    const __grid_constant__ GroupedMaps tmB, const GroupedArgs p) {
  constexpr int A_BYTES = kGgBM * kGgBK * 2;
  constexpr int B_BYTES = kGgBN * kGgBK * 2;
  constexpr uint32_t TMEM_COLS = 2 * kGgBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kGgStages * A_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + kGgStages * B_BYTES);
  uint64_t* empty_bar = full_bar + kGgStages;
  uint64_t* tfull_bar = empty_bar + kGgStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = static_cast<int>(blockIdx.x), n_ctas = static_cast<int>(gridDim.x);
  const int tiles_per_group = p.tiles_m * p.tiles_n;
  const int total_tiles = p.groups * tiles_per_group;
  const bool a_mn = p.mode == 2, b_mn = p.mode != 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGgStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    abort_flag[0] = 0;
    abort_flag[1] = p.status[3];
    fence_barrier_init();
    prefetch_tmap(&tmA);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The same schedule in all three roles: tile -> (group, m block, n block), skipped when the group has no rows there.
  // Returns the number of k blocks to run (0 in mode 2 = write zeros), or -1 to skip the tile.
  auto schedule = [&](int tile, int& grp, int& m_blk, int& n_blk) -> int {
    grp = tile / tiles_per_group;
    const int rem = tile - grp * tiles_per_group;
    n_blk = rem / p.tiles_m;
    m_blk = rem - n_blk * p.tiles_m;
    const int count = min(max(p.counts[grp], 0), p.cap);
    if (p.mode == 2) return (count + kGgBK - 1) / kGgBK;
    return m_blk * kGgBM < count ? p.k_blocks : -1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; ok && tile < total_tiles; tile += n_ctas) {
        int grp, m_blk, n_blk;
        const int kbn = schedule(tile, grp, m_blk, n_blk);
        if (kbn <= 0) continue;
        const CUtensorMap* mapB = p.mode == 2 ? &tmB_single : &tmB.m[grp];
        const int m0 = m_blk * kGgBM, n0 = n_blk * kGgBN, row0 = grp * p.cap;
        for (int kb = 0; kb < kbn; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const int k0 = kb * kGgBK;
          mbar_arrive_expect_tx(&full_bar[stage], A_BYTES + B_BYTES);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (!a_mn) {
            tma_load_2d(a_dst, &tmA, &full_bar[stage], k0, row0 + m0);                    // A[g*cap + m, k]
          } else {
#pragma unroll
            for (int j = 0; j < kGgBM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[stage], m0 + 64 * j, row0 + k0);   // A[g*cap + r, m]
          }
          if (!b_mn) {
            tma_load_2d(b_dst, mapB, &full_bar[stage], k0, n0);                          // B_g[n, k]
          } else {
            const int krow = p.mode == 2 ? row0 + k0 : k0;                                  // mode 2: B[g*cap + r, n]; mode 1: B_g[k, n]
#pragma unroll
            for (int j = 0; j < kGgBN / 64; ++j) tma_load_2d(b_dst + j * 8192, mapB, &full_bar[stage], n0 + 64 * j, krow);
          }
          if (++stage == kGgStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kGgBM, kGgBN, a_mn ? 1 : 0, b_mn ? 1 : 0);
      constexpr uint32_t hi = smem_desc_hi_sw128(1024);
      const uint32_t a_lbo = a_mn ? 8192u : 16u, b_lbo = b_mn ? 8192u : 16u;
      const uint32_t a_kstep = (a_mn ? 2048u : 32u) >> 4, b_kstep = (b_mn ? 2048u : 32u) >> 4;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = cta; ok && tile < total_tiles; tile += n_ctas) {
        int grp, m_blk, n_blk;
        const int kbn = schedule(tile, grp, m_blk, n_blk);
        if (kbn < 0) continue;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kGgBN);
        for (int kb = 0; kb < kbn; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = smem_desc_lo(smem_u32(sA + stage * A_BYTES), a_lbo);
          const uint32_t b_lo = smem_desc_lo(smem_u32(sB + stage * B_BYTES), b_lbo);
#pragma unroll
          for (int kk = 0; kk < kGgBK / 16; ++kk)
            umma_bf16_ss_lh(d_tmem, a_lo + kk * a_kstep, hi, b_lo + kk * b_kstep, hi, idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kGgStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);     // with no UMMA pending (empty group in mode 2) this arrives at once
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: lane = output row, 32 columns per TMEM load
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cta; tile < total_tiles; tile += n_ctas) {
      int grp, m_blk, n_blk;
      const int kbn = schedule(tile, grp, m_blk, n_blk);
      if (kbn < 0) continue;
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_blk * kGgBM + q * 32 + lane;                 // row inside the group
      const bool row_ok = row < p.M;
      void* base = p.mode == 2 ? p.c[grp] : p.c[0];
      const long long out_row = p.mode == 2 ? row : static_cast<long long>(grp) * p.cap + row;
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * kGgBN) + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kGgBN / 32; ++c) {
        uint32_t r[32];
        if (kbn > 0) {
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        const int col0 = n_blk * kGgBN + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        const int ncols = min(32, p.N - col0);
        if (p.out_fp32) {
          float* dst = static_cast<float*>(base) + out_row * p.ldc + col0;
          if (ncols == 32 && (p.ldc & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          } else {
            for (int i = 0; i < ncols; ++i) dst[i] = __uint_as_float(r[i]);
          }
        } else {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(base) + out_row * p.ldc + col0;
          if (ncols == 32 && (p.ldc & 7) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
              *reinterpret_cast<uint4*>(dst + i) = v;
            }
          } else {
            for (int i = 0; i < ncols; ++i) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(50000);
    if (threadIdx.x == 0) {
      atomicOr(&p.status[0], MB_ERR_MBAR_TIMEOUT);
      p.status[1] = static_cast<int>(blockIdx.x);
      p.status[2] = 2001;
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace mb

// Grouped GEMM (see the top of this file). `a`: stacked activations, row stride `lda` (elements). `b_ptrs[g]`: modes 0/1 the
// weights of group g ([N, K] row-major in mode 0, [K, N] row-major in mode 1, row stride `ldb`); mode 2: b_ptrs[0] is the
// second stacked activation buffer [groups * cap, N]. `c_ptrs`: modes 0/1 c_ptrs[0] = stacked output [groups * cap, N];
// mode 2 one [M, N] output per group. `counts`: int32 [groups] in device memory. All operands bf16, outputs bf16 or fp32.
// Pointers 16-byte aligned, row strides multiples of 8 elements.
MB_API int mb_grouped_gemm_bf16(int mode, const void* a, long long lda, const void* const* b_ptrs, long long ldb, void* const* c_ptrs,
                                long long ldc, const int* counts, int groups, int cap, int M, int N, int K, int out_fp32,
                                cudaStream_t stream) {
  using namespace mb;
  if (mode < 0 || mode > 2 || groups < 1 || groups > kGgMaxGroups || cap < 1 || M < 1 || N < 1 || K < 1 || !counts) {
    set_last_error("mb_grouped_gemm_bf16: bad mode / sizes (at most 16 groups per launch)");
    return -1;
  }
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(a) & 15)) {
    set_last_error("mb_grouped_gemm_bf16: operands must be 16-byte aligned with row strides multiple of 8");
    return -2;
  }
  if (mode != 2 && M != cap) {
    set_last_error("mb_grouped_gemm_bf16: modes 0 and 1 take M = cap");
    return -2;
  }
  if (mode == 2 && K != cap) {
    set_last_error("mb_grouped_gemm_bf16: mode 2 takes K = cap");
    return -2;
  }
  int* status = status_ptr();
  if (!status) return -4;
  GroupedArgs args{};
  args.mode = mode, args.groups = groups, args.cap = cap, args.M = M, args.N = N, args.K = K;
  args.tiles_m = (M + kGgBM - 1) / kGgBM, args.tiles_n = (N + kGgBN - 1) / kGgBN, args.k_blocks = (K + kGgBK - 1) / kGgBK;
  args.counts = counts, args.ldc = ldc, args.out_fp32 = out_fp32, args.status = status;
  const long long rows_total = static_cast<long long>(groups) * cap;
  CUtensorMap tmA, tmBs;
  GroupedMaps maps;
  bool ok;
  if (mode != 2) {
    ok = encode_tmap_2d(&tmA, a, (uint64_t)K, (uint64_t)rows_total, (uint64_t)lda * 2, kGgBK, kGgBM, 2, true);         // [rows, K], K-major
    for (int g = 0; ok && g < groups; ++g) {
      if (reinterpret_cast<uintptr_t>(b_ptrs[g]) & 15) ok = false;
      else if (mode == 0) ok = encode_tmap_2d(&maps.m[g], b_ptrs[g], (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kGgBK, kGgBN, 2, true);   // [N, K]
      else ok = encode_tmap_2d(&maps.m[g], b_ptrs[g], (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kGgBK, 2, true);                    // [K, N]
    }
    for (int g = groups; g < kGgMaxGroups; ++g) maps.m[g] = maps.m[0];
    tmBs = maps.m[0];
    args.c[0] = c_ptrs[0];
  } else {
    ok = encode_tmap_2d(&tmA, a, (uint64_t)M, (uint64_t)rows_total, (uint64_t)lda * 2, 64, kGgBK, 2, true);            // [rows, M], rows = reduction
    ok = ok && encode_tmap_2d(&tmBs, b_ptrs[0], (uint64_t)N, (uint64_t)rows_total, (uint64_t)ldb * 2, 64, kGgBK, 2, true);
    for (int g = 0; g < kGgMaxGroups; ++g) maps.m[g] = tmBs;
    for (int g = 0; g < groups; ++g) args.c[g] = c_ptrs[g];
  }
  if (!ok) return -5;
  constexpr size_t smem = 1024 + kGgStages * (kGgBM * kGgBK * 2 + kGgBN * kGgBK * 2) + 256;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    MB_CHECK_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured[dev & 63] = true;
  }
  const long long tiles = static_cast<long long>(groups) * args.tiles_m * args.tiles_n;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  grouped_gemm_kernel<<<grid, kGgThreads, smem, stream>>>(tmA, tmBs, maps, args);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
