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
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kEpiWarps = 4;
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);
constexpr int kGroupM = 8;  // tiles of one N column are visited for 8 consecutive M blocks (L2 reuse of B)

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
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& m_blk, int& n_blk) {
  const int per_group = kGroupM * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsz = min(tiles_m - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs p) {
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
    *abort_flag = 0;
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, p.tiles_m, p.tiles_n, m_blk, n_blk);
        const int m0 = m_blk * kBM, n0 = n_blk * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], A_BYTES + B_BYTES);
          const int k0 = kb * kBK;
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (!p.a_mn) {
            tma_load_2d(a_dst, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[stage], m0 + 64 * j, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(b_dst, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[stage], n0 + 64 * j, k0);
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
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
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
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = p.out_fp32 ? ((p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                   : ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, p.tiles_m, p.tiles_n, m_blk, n_blk);
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
        if (row < p.M && col0 < p.N) {
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
            if (vec_ok && col0 + 32 <= p.N) {
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
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& args, cudaStream_t stream) {
  constexpr size_t smem = 1024 + STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 256;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    MB_CHECK_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    configured[dev & 63] = true;
  }
  args.tiles_n = (args.N + BN - 1) / BN;
  const int total = args.tiles_m * args.tiles_n;
  const int grid = total < sm_count() ? total : sm_count();
  gemm_bf16_kernel<BN, STAGES><<<grid, kGemmThreads, smem, stream>>>(tmA, tmB, args);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Debug override of the descriptor geometry {lbo, sbo, kstep} per operand; negative = built-in value.
static int g_desc_override[6] = {-1, -1, -1, -1, -1, -1};

}  // namespace mb

MB_API void mb_gemm_debug_descriptor(int a_lbo, int a_sbo, int a_kstep, int b_lbo, int b_sbo, int b_kstep) {
  int v[6] = {a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep};
  for (int i = 0; i < 6; ++i) mb::g_desc_override[i] = v[i];
}

// C[M,N] (+)= op(A) op(B) (+bias). Leading dimensions are in elements; bf16 operands need them (and the base
// addresses) to be multiples of 8 elements / 16 bytes because the operands are fetched with TMA.
// block_n: 0 = choose, else 128 or 256.
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
  args.a_lbo = a_mn ? 8192u : 16u, args.a_sbo = 1024u, args.a_kstep = a_mn ? 2048u : 32u;
  args.b_lbo = b_mn ? 8192u : 16u, args.b_sbo = 1024u, args.b_kstep = b_mn ? 2048u : 32u;
  {
    unsigned* f[6] = {&args.a_lbo, &args.a_sbo, &args.a_kstep, &args.b_lbo, &args.b_sbo, &args.b_kstep};
    for (int i = 0; i < 6; ++i)
      if (g_desc_override[i] >= 0) *f[i] = static_cast<unsigned>(g_desc_override[i]);
  }

  int bn = block_n;
  if (bn != 128 && bn != 256) {
    const long long tiles256 = static_cast<long long>(args.tiles_m) * ((N + 255) / 256);
    bn = (N <= 128 || tiles256 < sm_count()) ? 128 : 256;
  }
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
  if (bn == 256) return launch_gemm<256, 4>(tmA, tmB, args, stream);
  return launch_gemm<128, 6>(tmA, tmB, args, stream);
}
