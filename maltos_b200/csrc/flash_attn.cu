// Flash-attention forward for sm_100a with tcgen05 tensor cores: S = Q K^T and O += P V run as UMMAs with S and O in
// tensor memory, the online softmax runs in registers (one thread per query row), K/V stream through a two-stage TMA
// ring. Native GQA (a query head reads K/V head h / group), head_dim 64 or 128, bf16 in / bf16 out + fp32 log-sum-exp
// (so partial results of ring attention can be merged). Visibility rules:
//   mode 0  every key is visible (blocks below the diagonal of ring attention);
//   mode 1  causal with offset: key j visible to query i  <=>  j <= i + (Sk - Sq);
//   mode 2  general: k_pos[j] <= q_pos[i] and k_seq[j] == q_seq[i] and k_seq[j] != -1 (packed documents, zigzag blocks);
//   mode 3  causal by index (as mode 1, so key blocks above the diagonal are skipped) and k_seq[j] == q_seq[i] != -1:
//           packed documents inside one row.
// One CTA handles 128 query rows of one (batch, head): warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-9 = softmax,
// rescale and output (two threads per query row, each owning half of the key columns). The reference gets this op from the flash-attn 2 package (utils/attention_backend.py:42-135).
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kFaBM = 128;          // query rows per CTA
constexpr int kFaBN = 128;          // keys per block
constexpr int kFaSoftmaxWarps = 8;   // two warps per TMEM lane quarter: each thread owns one query row and half of the key columns
constexpr int kFaThreads = 32 * (2 + kFaSoftmaxWarps);
constexpr float kLog2e = 1.4426950408889634f;

struct FlashArgs {
  __nv_bfloat16* out;       // [B, Sq, Hq, D]
  float* lse;               // [B, Hq, Sq]
  const int* q_pos;         // [B, Sq] or nullptr
  const int* k_pos;         // [B, Sk] or nullptr
  const int* q_seq;         // [B, Sq] or nullptr
  const int* k_seq;         // [B, Sk] or nullptr
  long long out_tstride;    // elements between tokens of out (>= Hq * D)
  int B, Sq, Sk, Hq, Hkv, D;
  int mode;
  float scale_log2;         // softmax scale * log2(e)
  int* status;
};

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled [rows x 64 bf16] atom
__device__ __forceinline__ float fast_exp2(float x) {   // x <= 0 here; one MUFU instruction
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
  return static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashArgs p) {
  constexpr int ATOMS = D / 64;                    // 64-wide swizzle atoms along head_dim
  constexpr int TILE_BYTES = kFaBM * D * 2;        // Q, K and V tiles: 128 rows x D bf16
  constexpr int P_BYTES = kFaBM * kFaBN * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, O_COL = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;                   // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;               // 2 stages
  uint8_t* sP = sV + 2 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;        // 2
  uint64_t* s_empty = bars + 7;       // 2
  uint64_t* p_full = bars + 9;        // 1
  uint64_t* o_full = bars + 10;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_xchg = reinterpret_cast<float*>(sP + P_BYTES + 256);   // exchange area: [2 parities][2 halves][128 rows] floats, then [2 halves][128 rows] int tags

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // long (late) tiles first under a causal mask
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = q_tile * kFaBM;
  const int causal_off = p.Sk - p.Sq;

  // number of key blocks this tile has to look at
  int n_blocks = (p.Sk + kFaBN - 1) / kFaBN;
  if (p.mode == 1 || p.mode == 3) {
    const int last_key = min(q0 + kFaBM - 1, p.Sq - 1) + causal_off;      // last key visible to the tile's last row
    n_blocks = last_key < 0 ? 0 : min(n_blocks, last_key / kFaBN + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], kFaSoftmaxWarps);
    }
    mbar_init(p_full, kFaSoftmaxWarps);
    mbar_init(o_full, 1);
    abort_flag[0] = 0;
    abort_flag[1] = p.status[3];
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  for (int i = threadIdx.x; i < 256; i += blockDim.x) reinterpret_cast<int*>(s_xchg + 768)[i] = 0;   // exchange tags
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_blocks > 0) {
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int a = 0; a < ATOMS; ++a) tma_load_4d(sQ + a * (kFaBM * 128), &tmQ, q_full, a * 64, head, q0, batch);
      for (int j = 0; j < n_blocks; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&kv_full[s], 2 * TILE_BYTES);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
          tma_load_4d(sK + s * TILE_BYTES + a * (kFaBN * 128), &tmK, &kv_full[s], a * 64, kv_head, j * kFaBN, batch);
          tma_load_4d(sV + s * TILE_BYTES + a * (kFaBN * 128), &tmV, &kv_full[s], a * 64, kv_head, j * kFaBN, batch);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_blocks > 0) {
      const uint32_t idesc_qk = make_idesc_bf16(kFaBM, kFaBN, 0, 0);      // S[128 q, 128 keys]: A = Q, B = K, both K-major over d
      const uint32_t idesc_pv = make_idesc_bf16(kFaBM, D, 0, 1);          // O[128 q, D]: A = P (K-major over keys), B = V (MN-major)
      constexpr uint32_t hi_k = smem_desc_hi_sw128(1024);
      const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16), p_lo = smem_desc_lo(smem_u32(sP), 16);
      auto issue_qk = [&](int j) {
        const int s = j & 1;
        const uint32_t k_lo = smem_desc_lo(smem_u32(sK + s * TILE_BYTES), 16);
        const uint32_t d_tmem = tmem_base + S_COL0 + static_cast<uint32_t>(s * kFaBN);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = static_cast<uint32_t>(((kk >> 2) * (kFaBM * 128) + (kk & 3) * 32) >> 4);
          umma_bf16_ss_lh(d_tmem, q_lo + off, hi_k, k_lo + off, hi_k, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&kv_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; ok && j < n_blocks; ++j) {
        if (j + 1 < n_blocks) {   // next block's scores while the softmax works on this one
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(&kv_full[s1], ((j + 1) >> 1) & 1, abort_flag) && mbar_wait(&s_empty[s1], (((j + 1) >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        if (!mbar_wait(p_full, j & 1, abort_flag)) break;
        tc_fence_after();
        const int s = j & 1;
        const uint32_t v_lo = smem_desc_lo(smem_u32(sV + s * TILE_BYTES), kFaBN * 128);   // MN-major: atoms kFaBN * 128 bytes apart
        const uint32_t acc0 = j != 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kFaBN / 16; ++kk) {
          const uint32_t off_p = static_cast<uint32_t>(((kk >> 2) * (kFaBM * 128) + (kk & 3) * 32) >> 4);
          umma_bf16_ss_lh(tmem_base + O_COL, p_lo + off_p, hi_k, v_lo + static_cast<uint32_t>(kk * 128), hi_k, idesc_pv, kk != 0 ? 1u : acc0);
        }
        umma_commit(&kv_empty[s]);   // K and V of this stage are free
        umma_commit(o_full);         // O holds blocks 0..j; the P tile may be overwritten
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax, rescale, output
    // Thread = (query row, half of the key columns): warps 2..5 take key columns 0..63 of every block, warps 6..9 columns
    // 64..127; the two threads of a row exchange their partial row maxima through shared memory. Two warps per
    // scheduler hide each other's instruction latencies, which a single warp per scheduler could not.
    const int qw = warp & 3;                       // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;              // 0: key columns [0, 64), 1: [64, 128)
    const int row = qw * 32 + lane;                // row inside the tile
    const int qi = q0 + row;                       // query index in the sequence
    const bool row_valid = qi < p.Sq;
    const uint32_t t_lane = static_cast<uint32_t>(qw * 32) << 16;
    const int my_pos = (p.mode == 2 && row_valid) ? p.q_pos[static_cast<long long>(batch) * p.Sq + qi] : 0;
    const int my_seq = (p.mode >= 2 && row_valid && p.q_seq) ? p.q_seq[static_cast<long long>(batch) * p.Sq + qi] : 0;
    // Pairwise exchange between the two threads of a row through shared memory: value, then a monotonically increasing
    // tag; the reader polls the partner's tag with the usual bound (no block-wide barrier, so an aborting warp cannot
    // strand the others).
    volatile int* x_tag = reinterpret_cast<volatile int*>(s_xchg + 768);     // [2 halves][128 rows]
    auto exchange = [&](float mine, int tag, float& theirs) -> bool {
      volatile float* val = s_xchg + (tag & 1) * 256;
      val[half * 128 + row] = mine;
      __threadfence_block();
      x_tag[half * 128 + row] = tag;
      const int partner = (half ^ 1) * 128 + row;
      const uint64_t t0 = globaltimer_ns();
      const uint64_t limit = wait_limit_ns(abort_flag);
      while (x_tag[partner] < tag) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > limit) {
          *abort_flag = 1;
          return false;
        }
      }
      theirs = val[partner];
      return true;
    };
    float m_run = -INFINITY, l_run = 0.f;          // l_run: this thread's half of the row sum
    bool ok = true;
    constexpr int HALF_N = kFaBN / 2;
    constexpr int HALF_D = D / 2;
    for (int j = 0; j < n_blocks; ++j) {
      const int s = j & 1;
      ok = mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_s = tmem_base + S_COL0 + static_cast<uint32_t>(s * kFaBN + half * HALF_N) + t_lane;
      const int key0 = j * kFaBN + half * HALF_N;  // first key of this thread's columns
      bool need_mask = j * kFaBN + kFaBN > p.Sk;
      if (p.mode == 1) need_mask = need_mask || (j * kFaBN + kFaBN - 1 > q0 + causal_off);
      if (p.mode >= 2) need_mask = true;
      auto visible = [&](int c) -> bool {          // c = column inside this thread's half
        const int kj = key0 + c;
        if (kj >= p.Sk) return false;
        if (p.mode == 1) return kj <= qi + causal_off;
        if (p.mode == 3 && kj > qi + causal_off) return false;
        if (p.mode >= 2) {
          const long long at = static_cast<long long>(batch) * p.Sk + kj;
          if (p.mode == 2 && p.k_pos[at] > my_pos) return false;
          if (p.k_seq) {
            const int ks = p.k_seq[at];
            if (ks == -1 || ks != my_seq) return false;
          }
        }
        return true;
      };
      // scores of this thread's 64 columns stay in registers for both passes
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(t_s, r0);
      tmem_ld_32x32b_x32(t_s + 32, r1);
      tmem_ld_wait();
      float m_part = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (!visible(i)) r0[i] = __float_as_uint(-INFINITY);
          if (!visible(32 + i)) r1[i] = __float_as_uint(-INFINITY);
        }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) m_part = fmaxf(m_part, fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
      float m_other = -INFINITY;
      ok = exchange(m_part, j + 1, m_other);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float m_blk = fmaxf(m_part, m_other) * p.scale_log2;   // scale > 0: max commutes with it
      const float m_new = fmaxf(m_run, m_blk);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = m_run == -INFINITY ? (m_new == -INFINITY ? 1.f : 0.f) : fast_exp2(m_run - m_new);
      // the previous P V product must be complete before O is rescaled or the P tile is overwritten
      if (j > 0) {
        ok = mbar_wait(o_full, (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {   // this thread rescales its half of the head dimension
          const uint32_t t_o = tmem_base + O_COL + static_cast<uint32_t>(half * HALF_D) + t_lane;
#pragma unroll 1
          for (int c0 = 0; c0 < HALF_D; c0 += 16) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(t_o + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x16(t_o + c0, r);
          }
          tmem_st_wait();
        }
      }
      // probabilities, partial row sum, this thread's atom of the P tile (bf16, 128-byte swizzled, K-major over keys)
      float l_blk = 0.f;
      uint8_t* atom = sP + half * (kFaBM * 128);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {             // 8 chunks of 8 keys
        float pr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float sc = __uint_as_float(ch < 4 ? r0[ch * 8 + i] : r1[(ch - 4) * 8 + i]);
          pr[i] = fast_exp2(sc * p.scale_log2 - m_safe);    // masked scores are -inf -> 0
          l_blk += pr[i];
        }
        uint4 v;
        v.x = pack_bf16x2(pr[0], pr[1]);
        v.y = pack_bf16x2(pr[2], pr[3]);
        v.z = pack_bf16x2(pr[4], pr[5]);
        v.w = pack_bf16x2(pr[6], pr[7]);
        *reinterpret_cast<uint4*>(atom + sw128_offset(row, ch)) = v;
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      fence_proxy_async_smem();                    // P stores (generic proxy) -> UMMA reads (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(p_full);
        mbar_arrive(&s_empty[s]);
      }
    }
    // ------------------------------------------------------------------ output
    if (ok && n_blocks > 0) {
      ok = mbar_wait(o_full, (n_blocks - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    // the two halves of a row add up their partial sums (all softmax warps reach this point, also after an abort)
    float l_other = 0.f;
    if (ok) {
      ok = exchange(l_run, n_blocks + 1, l_other);
      ok = __all_sync(0xffffffffu, ok);
    }
    const float l_tot = l_run + l_other;
    if (ok) {
      // TMEM loads are warp-collective: every lane takes part, only rows inside the sequence are stored
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<long long>(batch) * p.Sq + qi) * p.out_tstride + static_cast<long long>(head) * D + half * HALF_D;
      if (n_blocks > 0) {
        tc_fence_after();
        const uint32_t t_o = tmem_base + O_COL + static_cast<uint32_t>(half * HALF_D) + t_lane;
#pragma unroll 1
        for (int c0 = 0; c0 < HALF_D; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_o + c0, r);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c0 + i) = v;
            }
          }
        }
      } else if (row_valid) {
        for (int c = 0; c < HALF_D; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
      }
      if (row_valid && half == 0)
        p.lse[(static_cast<long long>(batch) * p.Hq + head) * p.Sq + qi] =
            l_tot > 0.f ? (m_run + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
    }
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
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
}

template <int D>
static int launch_flash_fwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FlashArgs& args,
                            cudaStream_t stream) {
  constexpr size_t smem = 1024 + 5 * (kFaBM * D * 2) + kFaBM * kFaBN * 2 + 256 + 4 * 1024;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    MB_CHECK_CUDA(cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured[dev & 63] = true;
  }
  dim3 grid((args.Sq + kFaBM - 1) / kFaBM, args.Hq, args.B);
  flash_fwd_kernel<D><<<grid, kFaThreads, smem, stream>>>(tmQ, tmK, tmV, args);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace mb

// q [B, Sq, Hq, D], k / v [B, Sk, Hkv, D] bf16 with element strides between tokens (`*_tstride`, heads contiguous inside a
// token, multiples of 8) and between batches; out [B, Sq, Hq, D] bf16, lse [B, Hq, Sq] fp32. mode / positions: see top.
MB_API int mb_flash_attn_fwd(const void* q, long long q_tstride, long long q_bstride, const void* k, const void* v,
                             long long kv_tstride, long long kv_bstride, void* out, long long out_tstride, float* lse,
                             const int* q_pos, const int* k_pos, const int* q_seq, const int* k_seq, int B, int Sq, int Sk,
                             int Hq, int Hkv, int D, int mode, float scale, cudaStream_t stream) {
  using namespace mb;
  if ((D != 64 && D != 128) || Hkv < 1 || Hq % Hkv != 0 || B < 1 || Sq < 1 || Sk < 1) {
    set_last_error("mb_flash_attn_fwd: head_dim must be 64 or 128, query heads a multiple of key/value heads");
    return -1;
  }
  if (mode < 0 || mode > 3 || (mode == 2 && (!q_pos || !k_pos)) || ((q_seq == nullptr) != (k_seq == nullptr)) ||
      (mode == 3 && !q_seq)) {
    set_last_error("mb_flash_attn_fwd: bad mask mode or missing position / sequence-id arrays");
    return -2;
  }
  if ((q_tstride & 7) || (kv_tstride & 7) || (q_bstride & 7) || (kv_bstride & 7) || (out_tstride & 7) ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
        reinterpret_cast<uintptr_t>(out)) & 15)) {
    set_last_error("mb_flash_attn_fwd: tensors must be 16-byte aligned with strides multiple of 8 elements");
    return -3;
  }
  int* status = status_ptr();
  if (!status) return -4;
  FlashArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.q_pos = q_pos, a.k_pos = k_pos, a.q_seq = q_seq, a.k_seq = k_seq;
  a.out_tstride = out_tstride;
  a.B = B, a.Sq = Sq, a.Sk = Sk, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
  a.mode = mode;
  a.scale_log2 = scale * kLog2e;
  a.status = status;
  CUtensorMap tmQ, tmK, tmV;
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(kFaBM), 1};
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hq, (uint64_t)Sq, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)q_tstride * 2, (uint64_t)q_bstride * 2};
    if (!encode_tmap_4d(&tmQ, q, dims, strides, box, 2, true)) return -5;
  }
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)Sk, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)kv_tstride * 2, (uint64_t)kv_bstride * 2};
    if (!encode_tmap_4d(&tmK, k, dims, strides, box, 2, true)) return -5;
    if (!encode_tmap_4d(&tmV, v, dims, strides, box, 2, true)) return -5;
  }
  return D == 128 ? launch_flash_fwd<128>(tmQ, tmK, tmV, a, stream) : launch_flash_fwd<64>(tmQ, tmK, tmV, a, stream);
}
