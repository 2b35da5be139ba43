// Flash-attention backward for sm_100a with tcgen05 tensor cores. Given q, k, v, the forward's output and log-sum-exp
// and the output gradient, it recomputes the probabilities block by block and produces dq, dk, dv:
//   P = exp(S * scale - lse),  dP = dO V^T,  dS = P * (dP - delta),  delta = rowsum(dO * O),
//   dV = P^T dO,  dK = scale * dS^T Q,  dQ = scale * dS K.
// Three launches:
//   flash_bwd_prep_kernel   delta and the log-sum-exp in the exp2 domain, padded to whole tiles (padding rows get
//                           lse = +inf so their probabilities are exactly zero), plus padded copies of the position /
//                           sequence-id arrays for the general mask;
//   flash_bwd_dkdv_kernel   one CTA per 128 keys of one (batch, key/value head): loops over the query heads of the group
//                           and over 64-row query sub-blocks. It forms the TRANSPOSED products S^T = K Q^T and
//                           dP^T = V dO^T (TMEM lane = key), so that P^T and dS^T - written back into tensor memory as
//                           bf16 over the scores they came from - are directly the A operands of dV += P^T dO and
//                           dK += dS^T Q: neither tile ever touches shared memory. Two TMEM slots alternate, so the
//                           arithmetic of one sub-block runs under the UMMAs of its neighbours;
//   flash_bwd_dq_kernel     one CTA per 128 query rows of one (batch, head): loops over 128-key blocks, S double-buffered
//                           in TMEM, dS written over S as the A operand of dQ += dS K.
// dK/dV and dQ are each owned by exactly one CTA: no atomics, results are deterministic. Masks and GQA as in the
// forward (mode 0 all visible, 1 causal with offset, 2 positions + sequence ids, 3 causal by index + same sequence id).
// Every wait is bounded (see ptx.cuh). The reference gets this op from the flash-attn 2 package
// (runtime/layers/flash_utils.py:218-260) or from autograd through SDPA.
#include <cstdlib>

#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kBwComputeWarps = 16;   // four warps per TMEM lane quarter: enough warps per scheduler to hide the latency of
                                      // the dependent exp / multiply / pack chains
constexpr int kBwThreads = 32 * (2 + kBwComputeWarps);   // warp 0 TMA producer, warp 1 UMMA issuer, warps 2..17 arithmetic
constexpr float kBwLog2e = 1.4426950408889634f;

struct FlashBwdArgs {
  void* dq;                 // [B, Sq, Hq, D]  bf16 or fp32
  void* dk;                 // [B, Sk, Hkv, D]
  void* dv;
  const float* lse2;        // [B * Hq, Sq_pad]  log-sum-exp * log2(e); +inf for rows that saw nothing and for padding
  const float* delta;       // [B * Hq, Sq_pad]
  const int* qpos;          // [B, Sq_pad]  (modes 2, 3)
  const int* qseq;
  const int* kpos;          // [B, Sk_pad]
  const int* kseq;          // padding keys carry sequence id -1
  long long dq_tstride;     // elements between tokens
  long long dkv_tstride;
  int B, Sq, Sk, Hq, Hkv, Sq_pad, Sk_pad;
  int mode;
  int out_fp32;             // 1: outputs are fp32
  int accumulate;           // 1 (fp32 outputs only): add to what the output holds
  float scale, scale_log2;
  int* status;
  int split;                // dK/dV kernel: the query heads of a group are divided over `split` CTAs (1 = no split)
  float* dk_tmp;            // split > 1: fp32 [B, Sk, Hkv, D] sums the CTAs add their parts to
  float* dv_tmp;
  int dbg;                  // probe builds only: bit 0 skip the S/dP UMMAs, bit 1 skip the accumulation UMMAs, bit 2 skip the arithmetic
};

#ifdef MB_FLASH_PROBE
// Timing probe (never part of the default build): clock64() stamps of the first CTA's issuing thread and of one arithmetic
// warp, 8 slots per iteration, read back with mb_flash_probe_read.
__device__ long long g_flash_probe[16 * 256];
#define MB_PROBE(cond, it, slot)                                                                  \
  do {                                                                                            \
    if ((cond) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (it) < 256) g_flash_probe[(it) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define MB_PROBE(cond, it, slot) do { } while (0)
#endif
#ifdef MB_FLASH_PROBE
#define MB_DBG(bit) ((p.dbg >> (bit)) & 1)
#else
#define MB_DBG(bit) 0
#endif

__device__ __forceinline__ float bw_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------- preprocessing
// One warp per (batch, head, query row): delta = sum_d out * dout; lse2 = lse * log2(e).
template <int D>
__global__ void flash_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                      long long o_tstride, long long o_bstride, long long do_tstride, long long do_bstride,
                                      const float* __restrict__ lse, float* __restrict__ lse2, float* __restrict__ delta,
                                      int B, int Sq, int Hq, int Sq_pad) {
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * Hq * Sq_pad;
  if (warp_global >= total) return;
  const int qi = static_cast<int>(warp_global % Sq_pad);
  const long long bh = warp_global / Sq_pad;
  const int h = static_cast<int>(bh % Hq), b = static_cast<int>(bh / Hq);
  float acc = 0.f, l2 = INFINITY;
  if (qi < Sq) {
    constexpr int PER = D / 32;   // 2 or 4 bf16 per lane
    const __nv_bfloat16* po = out + b * o_bstride + qi * o_tstride + static_cast<long long>(h) * D + lane * PER;
    const __nv_bfloat16* pd = dout + b * do_bstride + qi * do_tstride + static_cast<long long>(h) * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; i += 2) {
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(po + i);
      const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(pd + i);
      acc += __bfloat162float(a.x) * __bfloat162float(g.x) + __bfloat162float(a.y) * __bfloat162float(g.y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    const float l = lse[(static_cast<long long>(b) * Hq + h) * Sq + qi];
    l2 = (l == -INFINITY) ? INFINITY : l * kBwLog2e;
  }
  if (lane == 0) {
    lse2[warp_global] = l2;
    delta[warp_global] = acc;
  }
}

// Padded int copies of positions / sequence ids: [B, n_pad]; padding gets `pad_value`; a null source gives `null_value`.
__global__ void flash_bwd_pad_kernel(const int* __restrict__ src, int* __restrict__ dst, int B, int n, int n_pad, int null_value,
                                     int pad_value, int index_when_null) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(B) * n_pad) return;
  const int t = static_cast<int>(i % n_pad), b = static_cast<int>(i / n_pad);
  int v = pad_value;
  if (t < n) v = src ? src[static_cast<long long>(b) * n + t] : (index_when_null ? t : null_value);
  dst[i] = v;
}

// 16 consecutive output elements starting at elem_off
__device__ __forceinline__ void store_row_chunk(void* base, long long elem_off, const uint32_t (&r)[16], float mul, bool fp32,
                                                bool accumulate) {
  if (fp32) {
    float* dst = static_cast<float*>(base) + elem_off;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      float4 v = make_float4(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul, __uint_as_float(r[i + 2]) * mul,
                             __uint_as_float(r[i + 3]) * mul);
      if (accumulate) {
        const float4 o = *reinterpret_cast<const float4*>(dst + i);
        v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
      }
      *reinterpret_cast<float4*>(dst + i) = v;
    }
  } else {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(base) + elem_off;
#pragma unroll
    for (int i = 0; i < 16; i += 8) {
      uint4 v;
      v.x = pack_bf16x2(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
      v.y = pack_bf16x2(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
      v.z = pack_bf16x2(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
      v.w = pack_bf16x2(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
      *reinterpret_cast<uint4*>(dst + i) = v;
    }
  }
}

__device__ __forceinline__ void store_row_zero(void* base, long long elem_off, int n, bool fp32) {
  if (fp32) {
    float* dst = static_cast<float*>(base) + elem_off;
    for (int i = 0; i < n; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(base) + elem_off;
    for (int i = 0; i < n; i += 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// ---------------------------------------------------------------------------------------------- dK / dV
constexpr int kKvRows = 128;   // keys per CTA
constexpr int kQSub = 64;      // query rows per iteration
constexpr int kQStages = 4;

template <int D, int MODE>
__global__ void __launch_bounds__(kBwThreads, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const FlashBwdArgs p) {
  constexpr int ATOMS = D / 64;
  constexpr int KV_BYTES = kKvRows * D * 2;
  constexpr int Q_BYTES = kQSub * D * 2;
  constexpr int AUX_BYTES = 4 * kQSub * 4;          // lse2, delta, qpos, qseq of one stage
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t DV_COL = 256, DK_COL = 256 + D;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_BYTES;
  uint8_t* sQ = sV + KV_BYTES;                      // kQStages tiles
  uint8_t* sDO = sQ + kQStages * Q_BYTES;           // kQStages tiles
  uint8_t* sAux = sDO + kQStages * Q_BYTES;         // kQStages x AUX_BYTES
  uint64_t* bars = reinterpret_cast<uint64_t*>(sAux + kQStages * AUX_BYTES);
  uint64_t* kv_full = bars;                 // 1
  uint64_t* q_full = bars + 1;              // kQStages
  uint64_t* q_empty = q_full + kQStages;    // kQStages
  uint64_t* s_full = q_empty + kQStages;    // 2
  uint64_t* p_full = s_full + 2;            // 2
  uint64_t* acc_full = p_full + 2;          // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // With few key/value heads per GPU (tensor parallelism) one CTA per (key block, key/value head) would leave most SMs
  // idle: the query heads of the group are then divided over `split` CTAs, which add their parts into fp32 sums.
  const int kv_head = static_cast<int>(blockIdx.y) / p.split, part = static_cast<int>(blockIdx.y) % p.split, batch = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int heads_here = group / p.split;
  const int head0 = kv_head * group + part * heads_here;
  const int k0 = static_cast<int>(blockIdx.x) * kKvRows;
  const int causal_off = p.Sk - p.Sq;
  constexpr bool causal = MODE == 1 || MODE == 3;

  // query sub-blocks this key block has to visit
  const int n_qsub_all = (p.Sq + kQSub - 1) / kQSub;
  int qb_start = 0;
  if (causal) {
    const int first_q = k0 - causal_off;             // first query row that sees key k0
    qb_start = first_q <= 0 ? 0 : first_q / kQSub;
  }
  const int n_sub = qb_start < n_qsub_all ? n_qsub_all - qb_start : 0;
  const int n_iter = n_sub * heads_here;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], kBwComputeWarps);
    }
    mbar_init(acc_full, 1);
    abort_flag[0] = 0;
    abort_flag[1] = p.status[3];
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmDO);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * KV_BYTES);
#pragma unroll
      for (int a = 0; a < ATOMS; ++a) {
        tma_load_4d(sK + a * (kKvRows * 128), &tmK, kv_full, a * 64, kv_head, k0, batch);
        tma_load_4d(sV + a * (kKvRows * 128), &tmV, kv_full, a * 64, kv_head, k0, batch);
      }
      constexpr bool with_ids = MODE >= 2;
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % kQStages;
        if (!mbar_wait(&q_empty[st], ((it / kQStages) & 1) ^ 1, abort_flag)) break;
        const int head = head0 + it / n_sub;
        const int qrow0 = (qb_start + it % n_sub) * kQSub;
        mbar_arrive_expect_tx(&q_full[st], 2 * Q_BYTES + (with_ids ? 4 : 2) * kQSub * 4);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
          tma_load_4d(sQ + st * Q_BYTES + a * (kQSub * 128), &tmQ, &q_full[st], a * 64, head, qrow0, batch);
          tma_load_4d(sDO + st * Q_BYTES + a * (kQSub * 128), &tmDO, &q_full[st], a * 64, head, qrow0, batch);
        }
        uint8_t* aux = sAux + st * AUX_BYTES;
        const long long row = (static_cast<long long>(batch) * p.Hq + head) * p.Sq_pad + qrow0;
        bulk_load(aux, p.lse2 + row, kQSub * 4, &q_full[st]);
        bulk_load(aux + kQSub * 4, p.delta + row, kQSub * 4, &q_full[st]);
        if (with_ids) {
          const long long prow = static_cast<long long>(batch) * p.Sq_pad + qrow0;
          bulk_load(aux + 2 * kQSub * 4, p.qpos + prow, kQSub * 4, &q_full[st]);
          bulk_load(aux + 3 * kQSub * 4, p.qseq + prow, kQSub * 4, &q_full[st]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_s = make_idesc_bf16(kKvRows, kQSub, 0, 0);    // [128 keys, 64 q] = A(K-major over d) x B(K-major over d)
      const uint32_t idesc_acc = make_idesc_bf16(kKvRows, D, 0, 1);      // [128 keys, D]   = A(TMEM) x B(MN-major)
      constexpr uint32_t hi_k = smem_desc_hi_sw128(1024);               // both operand kinds: 8-row groups 1024 bytes apart
      const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 16), v_lo = smem_desc_lo(smem_u32(sV), 16);
      auto issue_sdp = [&](int it) {
        const int st = it % kQStages;
        const uint32_t slot = tmem_base + static_cast<uint32_t>(it & 1) * 128u;
        const uint32_t q_lo = smem_desc_lo(smem_u32(sQ + st * Q_BYTES), 16), do_lo = smem_desc_lo(smem_u32(sDO + st * Q_BYTES), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (MB_DBG(0)) break;
          const uint32_t off_a = static_cast<uint32_t>(((kk >> 2) * (kKvRows * 128) + (kk & 3) * 32) >> 4);
          const uint32_t off_b = static_cast<uint32_t>(((kk >> 2) * (kQSub * 128) + (kk & 3) * 32) >> 4);
          umma_bf16_ss_lh(slot, k_lo + off_a, hi_k, q_lo + off_b, hi_k, idesc_s, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (MB_DBG(0)) break;
          const uint32_t off_a = static_cast<uint32_t>(((kk >> 2) * (kKvRows * 128) + (kk & 3) * 32) >> 4);
          const uint32_t off_b = static_cast<uint32_t>(((kk >> 2) * (kQSub * 128) + (kk & 3) * 32) >> 4);
          umma_bf16_ss_lh(slot + 64u, v_lo + off_a, hi_k, do_lo + off_b, hi_k, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[it & 1]);
      };
      auto issue_acc = [&](int it) {
        const int st = it % kQStages;
        const uint32_t slot = tmem_base + static_cast<uint32_t>(it & 1) * 128u;
        // MN-major B operands: 64-wide atoms of the head dimension are kQSub * 128 bytes apart
        const uint32_t q_lo = smem_desc_lo(smem_u32(sQ + st * Q_BYTES), kQSub * 128), do_lo = smem_desc_lo(smem_u32(sDO + st * Q_BYTES), kQSub * 128);
        const uint32_t acc0 = it != 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kQSub / 16; ++kk) {
          if (MB_DBG(1)) break;
          // packed bf16 pairs: the 16 query rows of k-step kk sit in the first 8 of the 16 columns their scores had
          const uint32_t a_col = static_cast<uint32_t>(kk * 16);
          const uint32_t acc_on = kk != 0 ? 1u : acc0;
          umma_bf16_ts_lh(tmem_base + DV_COL, slot + a_col, do_lo + static_cast<uint32_t>(kk * 128), hi_k, idesc_acc, acc_on);
          umma_bf16_ts_lh(tmem_base + DK_COL, slot + 64u + a_col, q_lo + static_cast<uint32_t>(kk * 128), hi_k, idesc_acc, acc_on);
        }
        umma_commit(&q_empty[st]);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag) && mbar_wait(&q_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int it = 0; ok && it < n_iter; ++it) {
        if (it + 1 < n_iter) {
          ok = mbar_wait(&q_full[(it + 1) % kQStages], ((it + 1) / kQStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          MB_PROBE(true, it, 0);
          issue_sdp(it + 1);     // its slot was last read by the accumulation UMMAs of it - 1, issued before
          MB_PROBE(true, it, 1);
        }
        ok = mbar_wait(&p_full[it & 1], (it >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        MB_PROBE(true, it, 2);
        issue_acc(it);
        MB_PROBE(true, it, 3);
      }
      if (ok) umma_commit(acc_full);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ arithmetic: lane = key, 16 query columns per thread
    const int qw = warp & 3;                      // TMEM lane quarter this warp may touch
    const int grp = (warp - 2) >> 2;              // which 16 of the 64 query columns
    const int row = qw * 32 + lane;
    const int kj = k0 + row;
    const bool key_valid = kj < p.Sk;
    const uint32_t t_lane = static_cast<uint32_t>(qw * 32) << 16;
    int my_pos = 0, my_seq = 0;
    if (MODE >= 2) {
      const long long at = static_cast<long long>(batch) * p.Sk_pad + kj;   // padded: always in range
      my_pos = p.kpos[at];
      my_seq = p.kseq[at];
    }
    const float scale_log2 = p.scale_log2;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int st = it % kQStages;
      const uint32_t slot = static_cast<uint32_t>(it & 1) * 128u;
      ok = mbar_wait(&q_full[st], (it / kQStages) & 1, abort_flag) && mbar_wait(&s_full[it & 1], (it >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      MB_PROBE(warp == 2 && lane == 0, it, 4);
      if (MB_DBG(2)) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[it & 1]);
        continue;
      }
      const uint32_t t_s = tmem_base + slot + static_cast<uint32_t>(grp * 16) + t_lane;
      uint32_t s[16], dp[16];
      if (!MB_DBG(3)) {
        tmem_ld_32x32b_x16(t_s, s);
        tmem_ld_32x32b_x16(t_s + 64u, dp);
      } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) s[c] = dp[c] = static_cast<uint32_t>(it + c);
      }
      const uint8_t* aux = sAux + st * AUX_BYTES + grp * 64;
      float lse[16], dl[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(aux + i * 16);
        const float4 d = *reinterpret_cast<const float4*>(aux + kQSub * 4 + i * 16);
        lse[4 * i] = a.x, lse[4 * i + 1] = a.y, lse[4 * i + 2] = a.z, lse[4 * i + 3] = a.w;
        dl[4 * i] = d.x, dl[4 * i + 1] = d.y, dl[4 * i + 2] = d.z, dl[4 * i + 3] = d.w;
      }
      tmem_ld_wait();
      MB_PROBE(warp == 2 && lane == 0, it, 5);
      const int qsub0 = (qb_start + it % n_sub) * kQSub;      // first query row of the sub-block
      // does this sub-block contain a masked pair? (warp-uniform)
      bool need_mask = (k0 + kKvRows > p.Sk) || MODE >= 2;
      if (causal) need_mask = need_mask || (k0 + kKvRows - 1 > qsub0 + causal_off);
      float pr[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) pr[c] = MB_DBG(5) ? __uint_as_float(s[c]) : bw_exp2(fmaf(__uint_as_float(s[c]), scale_log2, -lse[c]));
      if (need_mask) {
        int qp[16], qs[16];
        if (MODE >= 2) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int4 a = *reinterpret_cast<const int4*>(aux + 2 * kQSub * 4 + i * 16);
            const int4 d = *reinterpret_cast<const int4*>(aux + 3 * kQSub * 4 + i * 16);
            qp[4 * i] = a.x, qp[4 * i + 1] = a.y, qp[4 * i + 2] = a.z, qp[4 * i + 3] = a.w;
            qs[4 * i] = d.x, qs[4 * i + 1] = d.y, qs[4 * i + 2] = d.z, qs[4 * i + 3] = d.w;
          }
        }
        const int q_first = qsub0 + grp * 16 + causal_off;     // key index visible up to (causal modes)
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          bool vis = key_valid;
          if (causal) vis = vis && (kj <= q_first + c);
          if (MODE == 2) vis = vis && (my_pos <= qp[c]);
          if (MODE >= 2) vis = vis && (my_seq == qs[c]) && (my_seq != -1);
          pr[c] = vis ? pr[c] : 0.f;
        }
      }
      uint32_t pk[8], dsk[8];
#pragma unroll
      for (int c = 0; c < 16; c += 2) {
        pk[c >> 1] = pack_bf16x2(pr[c], pr[c + 1]);
        dsk[c >> 1] = pack_bf16x2(pr[c] * (__uint_as_float(dp[c]) - dl[c]), pr[c + 1] * (__uint_as_float(dp[c + 1]) - dl[c + 1]));
      }
      MB_PROBE(warp == 2 && lane == 0, it, 6);
      if (!MB_DBG(4)) {
      tmem_st_32x32b_x8(t_s, pk);           // P^T over the first half of this thread's own score columns
      tmem_st_32x32b_x8(t_s + 64u, dsk);    // dS^T over its dP columns
      tmem_st_wait();
      } else if (pk[0] == 0x12345678u && dsk[3] == 0x9abcdef0u) {
        p.status[2] = 7;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[it & 1]);
      MB_PROBE(warp == 2 && lane == 0, it, 7);
    }
    // ------------------------------------------------------------------ epilogue: dV, dK rows of this key
    if (ok && n_iter > 0) {
      ok = mbar_wait(acc_full, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      constexpr int QUART_D = D / 4;                // columns of the head dimension per thread
      const long long off = (static_cast<long long>(batch) * p.Sk + kj) * p.dkv_tstride + static_cast<long long>(kv_head) * D + grp * QUART_D;
      const long long toff = ((static_cast<long long>(batch) * p.Sk + kj) * p.Hkv + kv_head) * D + grp * QUART_D;
      if (n_iter > 0) {
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < QUART_D; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_base + DV_COL + static_cast<uint32_t>(grp * QUART_D + c0) + t_lane, r);
          tmem_ld_wait();
          if (key_valid) {
            if (p.split > 1) {
#pragma unroll
              for (int i = 0; i < 16; ++i) atomicAdd(p.dv_tmp + toff + c0 + i, __uint_as_float(r[i]));
            } else {
              store_row_chunk(p.dv, off + c0, r, 1.f, p.out_fp32 != 0, p.accumulate != 0);
            }
          }
          tmem_ld_32x32b_x16(tmem_base + DK_COL + static_cast<uint32_t>(grp * QUART_D + c0) + t_lane, r);
          tmem_ld_wait();
          if (key_valid) {
            if (p.split > 1) {
#pragma unroll
              for (int i = 0; i < 16; ++i) atomicAdd(p.dk_tmp + toff + c0 + i, __uint_as_float(r[i]) * p.scale);
            } else {
              store_row_chunk(p.dk, off + c0, r, p.scale, p.out_fp32 != 0, p.accumulate != 0);
            }
          }
        }
      } else if (key_valid && !p.accumulate && p.split == 1) {
        store_row_zero(p.dv, off, QUART_D, p.out_fp32 != 0);
        store_row_zero(p.dk, off, QUART_D, p.out_fp32 != 0);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(50000);
    if (threadIdx.x == 0) {
      atomicOr(&p.status[0], MB_ERR_MBAR_TIMEOUT);
      p.status[1] = static_cast<int>(blockIdx.x);
      p.status[2] = 1001;
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// fp32 sums [tokens, hd] of a split dK/dV launch -> the caller's outputs (bf16 or fp32, token stride `tstride`).
__global__ void flash_bwd_finish_split_kernel(const float* __restrict__ dk_tmp, const float* __restrict__ dv_tmp, void* dk, void* dv,
                                              long long tokens, int hd, long long tstride, int out_fp32, int accumulate) {
  const long long i4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i4 >= tokens * hd) return;
  const long long t = i4 / hd;
  const int c = static_cast<int>(i4 - t * hd);
  const long long o = t * tstride + c;
  const float4 a = *reinterpret_cast<const float4*>(dk_tmp + i4), b = *reinterpret_cast<const float4*>(dv_tmp + i4);
  if (out_fp32) {
    float4* pk = reinterpret_cast<float4*>(static_cast<float*>(dk) + o);
    float4* pv = reinterpret_cast<float4*>(static_cast<float*>(dv) + o);
    float4 k = a, v = b;
    if (accumulate) {
      const float4 ok = *pk, ov = *pv;
      k.x += ok.x, k.y += ok.y, k.z += ok.z, k.w += ok.w;
      v.x += ov.x, v.y += ov.y, v.z += ov.z, v.w += ov.w;
    }
    *pk = k;
    *pv = v;
  } else {
    uint2 k, v;
    k.x = pack_bf16x2(a.x, a.y), k.y = pack_bf16x2(a.z, a.w);
    v.x = pack_bf16x2(b.x, b.y), v.y = pack_bf16x2(b.z, b.w);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(dk) + o) = k;
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(dv) + o) = v;
  }
}

// How many CTAs share the query heads of one key/value head in the dK/dV kernel: the smallest power of two that fills
// the GPU (or uses up the group).
static int dkdv_split(int B, int Sk, int Hq, int Hkv) {
  const long long ctas = static_cast<long long>((Sk + kKvRows - 1) / kKvRows) * Hkv * B;
  const int group = Hq / Hkv;
  int split = 1;
  while (split * 2 <= group && group % (split * 2) == 0 && ctas * split < sm_count()) split *= 2;
  return split;
}

// ---------------------------------------------------------------------------------------------- dQ
constexpr int kDqRows = 128;   // query rows per CTA
constexpr int kDqKeys = 128;   // keys per block

template <int D, int MODE>
__global__ void __launch_bounds__(kBwThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const FlashBwdArgs p) {
  constexpr int ATOMS = D / 64;
  constexpr int TILE_BYTES = 128 * D * 2;
  constexpr int AUX_BYTES = 2 * kDqKeys * 4;        // kpos, kseq of one stage
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t DP_COL = 256, DQ_COL = 384;

  // K and V have rings of their own: a V tile is free as soon as dP of its block is done, a K tile only after dQ, and
  // the tensor-map loads are slow enough (64 KB take ~1400 cycles) that K needs three stages to stay ahead. With Q and
  // dO resident that fills the shared memory of the SM, so the dynamic window must start 1024-byte aligned (checked).
  // (The masks that need per-key ids keep two K stages at head_dim 128: their id arrays take the remaining space.)
  constexpr int K_STAGES = (D == 128) ? (MODE >= 2 ? 2 : 3) : 4;
  constexpr int AUX_STAGES = MODE >= 2 ? K_STAGES : 0;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE_BYTES;
  uint8_t* sK = sDO + TILE_BYTES;                   // K_STAGES stages
  uint8_t* sV = sK + K_STAGES * TILE_BYTES;         // 2 stages
  uint8_t* sAux = sV + 2 * TILE_BYTES;              // AUX_STAGES x AUX_BYTES
  uint64_t* bars = reinterpret_cast<uint64_t*>(sAux + AUX_STAGES * AUX_BYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // K_STAGES (<= 4)
  uint64_t* k_empty = bars + 5;       // K_STAGES
  uint64_t* v_full = bars + 9;        // 2
  uint64_t* v_empty = bars + 11;      // 2
  uint64_t* s_full = bars + 13;       // 2
  uint64_t* dp_full = bars + 15;      // 1
  uint64_t* dp_free = bars + 16;      // 1 (count = arithmetic warps)
  uint64_t* ds_full = bars + 17;      // 1 (count = arithmetic warps)
  uint64_t* dq_full = bars + 18;      // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // long tiles first under a causal mask
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = q_tile * kDqRows;
  const int causal_off = p.Sk - p.Sq;
  constexpr bool causal = MODE == 1 || MODE == 3;

  int n_blocks = (p.Sk + kDqKeys - 1) / kDqKeys;
  if (causal) {
    const int last_key = min(q0 + kDqRows - 1, p.Sq - 1) + causal_off;
    n_blocks = last_key < 0 ? 0 : min(n_blocks, last_key / kDqKeys + 1);
  }

  if (smem_u32(smem_raw) & 1023u) {   // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0) {
      atomicOr(&p.status[0], MB_ERR_BAD_INDEX);
      p.status[2] = 1003;
    }
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < K_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(dp_full, 1);
    mbar_init(dp_free, kBwComputeWarps);
    mbar_init(ds_full, kBwComputeWarps);
    mbar_init(dq_full, 1);
    abort_flag[0] = 0;
    abort_flag[1] = p.status[3];
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmDO);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_blocks > 0) {
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int a = 0; a < ATOMS; ++a) {
        tma_load_4d(sQ + a * (kDqRows * 128), &tmQ, q_full, a * 64, head, q0, batch);
        tma_load_4d(sDO + a * (kDqRows * 128), &tmDO, q_full, a * 64, head, q0, batch);
      }
      constexpr bool with_ids = MODE >= 2;
      for (int j = 0; j < n_blocks; ++j) {
        const int ks = j % K_STAGES, vs = j & 1;
        if (!mbar_wait(&k_empty[ks], ((j / K_STAGES) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&k_full[ks], TILE_BYTES + (with_ids ? AUX_BYTES : 0));
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_4d(sK + ks * TILE_BYTES + a * (kDqKeys * 128), &tmK, &k_full[ks], a * 64, kv_head, j * kDqKeys, batch);
        if (with_ids) {
          const long long prow = static_cast<long long>(batch) * p.Sk_pad + j * kDqKeys;
          bulk_load(sAux + ks * AUX_BYTES, p.kpos + prow, kDqKeys * 4, &k_full[ks]);
          bulk_load(sAux + ks * AUX_BYTES + kDqKeys * 4, p.kseq + prow, kDqKeys * 4, &k_full[ks]);
        }
        if (!mbar_wait(&v_empty[vs], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&v_full[vs], TILE_BYTES);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_4d(sV + vs * TILE_BYTES + a * (kDqKeys * 128), &tmV, &v_full[vs], a * 64, kv_head, j * kDqKeys, batch);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0 && n_blocks > 0) {
      const uint32_t idesc_s = make_idesc_bf16(kDqRows, kDqKeys, 0, 0);   // [128 q, 128 keys]
      const uint32_t idesc_dq = make_idesc_bf16(kDqRows, D, 0, 1);         // [128 q, D] = A(TMEM) x B(K tile, MN-major)
      constexpr uint32_t hi_k = smem_desc_hi_sw128(1024);
      const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16), do_lo = smem_desc_lo(smem_u32(sDO), 16);
      auto issue_s = [&](int j) {
        const uint32_t k_lo = smem_desc_lo(smem_u32(sK + (j % K_STAGES) * TILE_BYTES), 16);
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(j & 1) * 128u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = static_cast<uint32_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);
          umma_bf16_ss_lh(d_tmem, q_lo + off, hi_k, k_lo + off, hi_k, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      auto issue_dp = [&](int j) {
        const uint32_t v_lo = smem_desc_lo(smem_u32(sV + (j & 1) * TILE_BYTES), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = static_cast<uint32_t>(((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4);
          umma_bf16_ss_lh(tmem_base + DP_COL, do_lo + off, hi_k, v_lo + off, hi_k, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
        umma_commit(&v_empty[j & 1]);   // this V tile is not read again
      };
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = mbar_wait(&v_full[0], 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(0);
      }
      // Issue order per block j: dQ of block j - 1 first (its dS has just been finished by the arithmetic warps, which
      // now start on block j), then dP and S of block j + 1. The only wait that can really block is the one on dS; the
      // loads and the "dP consumed" signal it waits for next arrive while dQ(j - 1) is being issued, so the tensor pipe
      // never idles behind this thread.
      auto issue_dq = [&](int j) {
        const uint32_t k_lo = smem_desc_lo(smem_u32(sK + (j % K_STAGES) * TILE_BYTES), kDqKeys * 128);   // MN-major B: atoms kDqKeys * 128 bytes apart
        const uint32_t s_col = tmem_base + static_cast<uint32_t>(j & 1) * 128u;
        const uint32_t acc0 = j != 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kDqKeys / 16; ++kk) {
          // packed bf16 pairs: the 32 keys of column group g sit in the first 16 of the 32 columns their scores had
          const uint32_t a_col = static_cast<uint32_t>((kk >> 1) * 32 + (kk & 1) * 8);
          umma_bf16_ts_lh(tmem_base + DQ_COL, s_col + a_col, k_lo + static_cast<uint32_t>(kk * 128), hi_k, idesc_dq, kk != 0 ? 1u : acc0);
        }
        umma_commit(&k_empty[j % K_STAGES]);
      };
      for (int j = 0; ok && j < n_blocks; ++j) {
        if (j > 0) {
          ok = mbar_wait(ds_full, (j - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          MB_PROBE(true, j, 4);
          issue_dq(j - 1);
          MB_PROBE(true, j, 5);
        }
        if (j + 1 < n_blocks) {
          ok = mbar_wait(dp_free, j & 1, abort_flag) &&   // block j's dP has been read
               mbar_wait(&v_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          MB_PROBE(true, j, 2);
          issue_dp(j + 1);
          MB_PROBE(true, j, 3);
          ok = mbar_wait(&k_full[(j + 1) % K_STAGES], ((j + 1) / K_STAGES) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          MB_PROBE(true, j, 0);
          issue_s(j + 1);           // its S buffer was last read by dQ of block j - 1, issued above
          MB_PROBE(true, j, 1);
        }
      }
      if (ok) {
        ok = mbar_wait(ds_full, (n_blocks - 1) & 1, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_dq(n_blocks - 1);
        }
      }
      if (ok) umma_commit(dq_full);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ arithmetic: lane = query row, 32 key columns per thread
    const int qw = warp & 3;
    const int grp = (warp - 2) >> 2;              // which 32 of the 128 key columns
    const int row = qw * 32 + lane;
    const int qi = q0 + row;
    const bool row_valid = qi < p.Sq;
    const uint32_t t_lane = static_cast<uint32_t>(qw * 32) << 16;
    const long long arow = (static_cast<long long>(batch) * p.Hq + head) * p.Sq_pad + qi;   // padded: always in range
    const float my_lse = p.lse2[arow];
    const float my_delta = p.delta[arow];
    int my_pos = 0, my_seq = 0;
    if (MODE >= 2) {
      const long long at = static_cast<long long>(batch) * p.Sq_pad + qi;
      my_pos = p.qpos[at];
      my_seq = p.qseq[at];
    }
    const float scale_log2 = p.scale_log2;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const int s = j & 1;
      ok = mbar_wait(&k_full[j % K_STAGES], (j / K_STAGES) & 1, abort_flag) && mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag) &&
           mbar_wait(dp_full, j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      MB_PROBE(warp == 2 && lane == 0, j, 8);
      const uint32_t t_s = tmem_base + static_cast<uint32_t>(s * 128 + grp * 32) + t_lane;
      const uint32_t t_dp = tmem_base + DP_COL + static_cast<uint32_t>(grp * 32) + t_lane;
      uint32_t sc[32], dp[32];
      tmem_ld_32x32b_x32(t_s, sc);
      tmem_ld_32x32b_x32(t_dp, dp);
      tmem_ld_wait();
      MB_PROBE(warp == 2 && lane == 0, j, 9);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dp_free);        // this warp's dP columns are in registers: the next block's dP may be issued
      const int key0 = j * kDqKeys + grp * 32;
      bool need_mask = (j * kDqKeys + kDqKeys > p.Sk) || MODE >= 2;
      if (causal) need_mask = need_mask || (j * kDqKeys + kDqKeys - 1 > q0 + causal_off);
      float pr[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) pr[c] = bw_exp2(fmaf(__uint_as_float(sc[c]), scale_log2, -my_lse));
      if (need_mask) {
        const uint8_t* aux = sAux + (j % K_STAGES) * AUX_BYTES + grp * 128;
        const int q_lim = qi + causal_off - key0;   // column c visible (causal modes) iff c <= q_lim
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          int4 kp = make_int4(0, 0, 0, 0), ks = make_int4(0, 0, 0, 0);
          if (MODE >= 2) {
            kp = *reinterpret_cast<const int4*>(aux + i * 16);
            ks = *reinterpret_cast<const int4*>(aux + kDqKeys * 4 + i * 16);
          }
          const int kpv[4] = {kp.x, kp.y, kp.z, kp.w}, ksv[4] = {ks.x, ks.y, ks.z, ks.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = 4 * i + u;
            bool vis = key0 + c < p.Sk;
            if (causal) vis = vis && (c <= q_lim);
            if (MODE == 2) vis = vis && (kpv[u] <= my_pos);
            if (MODE >= 2) vis = vis && (ksv[u] == my_seq) && (ksv[u] != -1);
            pr[c] = vis ? pr[c] : 0.f;
          }
        }
      }
      uint32_t dsp[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2)
        dsp[c >> 1] = pack_bf16x2(pr[c] * (__uint_as_float(dp[c]) - my_delta), pr[c + 1] * (__uint_as_float(dp[c + 1]) - my_delta));
      MB_PROBE(warp == 2 && lane == 0, j, 10);
      tmem_st_32x32b_x16(t_s, dsp);               // dS over the first half of this thread's own score columns
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      MB_PROBE(warp == 2 && lane == 0, j, 11);
    }
    // ------------------------------------------------------------------ epilogue
    if (ok && n_blocks > 0) {
      ok = mbar_wait(dq_full, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      constexpr int QUART_D = D / 4;
      const long long off = (static_cast<long long>(batch) * p.Sq + qi) * p.dq_tstride + static_cast<long long>(head) * D + grp * QUART_D;
      if (n_blocks > 0) {
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < QUART_D; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_base + DQ_COL + static_cast<uint32_t>(grp * QUART_D + c0) + t_lane, r);
          tmem_ld_wait();
          if (row_valid) store_row_chunk(p.dq, off + c0, r, p.scale, p.out_fp32 != 0, p.accumulate != 0);
        }
      } else if (row_valid && !p.accumulate) {
        store_row_zero(p.dq, off, QUART_D, p.out_fp32 != 0);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(50000);
    if (threadIdx.x == 0) {
      atomicOr(&p.status[0], MB_ERR_MBAR_TIMEOUT);
      p.status[1] = static_cast<int>(blockIdx.x);
      p.status[2] = 1002;
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, int MODE>
static int launch_flash_bwd(const void* q, long long q_tstride, long long q_bstride, const void* k, const void* v,
                            long long kv_tstride, long long kv_bstride, const void* out, long long o_tstride, long long o_bstride,
                            const void* dout, long long do_tstride, long long do_bstride, const float* lse, const int* q_pos,
                            const int* k_pos, const int* q_seq, const int* k_seq, float* scratch, FlashBwdArgs a,
                            cudaStream_t stream) {
  // scratch layout (floats / ints, 4 bytes each)
  const long long n_rows = static_cast<long long>(a.B) * a.Hq * a.Sq_pad;
  float* lse2 = scratch;
  float* delta = scratch + n_rows;
  int* qpos = reinterpret_cast<int*>(scratch + 2 * n_rows);
  int* qseq = qpos + static_cast<long long>(a.B) * a.Sq_pad;
  int* kpos = qseq + static_cast<long long>(a.B) * a.Sq_pad;
  int* kseq = kpos + static_cast<long long>(a.B) * a.Sk_pad;
  a.lse2 = lse2, a.delta = delta, a.qpos = qpos, a.qseq = qseq, a.kpos = kpos, a.kseq = kseq;
  a.split = dkdv_split(a.B, a.Sk, a.Hq, a.Hkv);
  const long long kv_elems = static_cast<long long>(a.B) * a.Sk * a.Hkv * D;
  if (a.split > 1) {
    a.dk_tmp = reinterpret_cast<float*>(kseq + static_cast<long long>(a.B) * a.Sk_pad);
    a.dv_tmp = a.dk_tmp + kv_elems;
    MB_CHECK_CUDA(cudaMemsetAsync(a.dk_tmp, 0, sizeof(float) * 2 * kv_elems, stream));
  }
  {
    const long long threads = n_rows * 32;
    const int block = 256;
    flash_bwd_prep_kernel<D><<<static_cast<unsigned>((threads + block - 1) / block), block, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), o_tstride, o_bstride, do_tstride,
        do_bstride, lse, lse2, delta, a.B, a.Sq, a.Hq, a.Sq_pad);
    count_launch();
  }
  if (MODE >= 2) {
    const int block = 256;
    const long long nq = static_cast<long long>(a.B) * a.Sq_pad, nk = static_cast<long long>(a.B) * a.Sk_pad;
    const unsigned gq = static_cast<unsigned>((nq + block - 1) / block), gk = static_cast<unsigned>((nk + block - 1) / block);
    flash_bwd_pad_kernel<<<gq, block, 0, stream>>>(q_pos, qpos, a.B, a.Sq, a.Sq_pad, 0, 0, 1);
    flash_bwd_pad_kernel<<<gq, block, 0, stream>>>(q_seq, qseq, a.B, a.Sq, a.Sq_pad, 0, 0, 0);
    flash_bwd_pad_kernel<<<gk, block, 0, stream>>>(k_pos, kpos, a.B, a.Sk, a.Sk_pad, 0, 0x7fffffff, 1);
    flash_bwd_pad_kernel<<<gk, block, 0, stream>>>(k_seq, kseq, a.B, a.Sk, a.Sk_pad, 0, -1, 0);
    count_launch(4);
  }
  MB_CHECK_CUDA(cudaGetLastError());

  CUtensorMap tmQ128, tmDO128, tmQ64, tmDO64, tmK, tmV;
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)a.Hq, (uint64_t)a.Sq, (uint64_t)a.B};
    const uint64_t sq[3] = {(uint64_t)D * 2, (uint64_t)q_tstride * 2, (uint64_t)q_bstride * 2};
    const uint64_t sdo[3] = {(uint64_t)D * 2, (uint64_t)do_tstride * 2, (uint64_t)do_bstride * 2};
    const uint32_t box128[4] = {64, 1, 128, 1}, box64[4] = {64, 1, 64, 1};
    if (!encode_tmap_4d(&tmQ128, q, dims, sq, box128, 2, true) || !encode_tmap_4d(&tmQ64, q, dims, sq, box64, 2, true) ||
        !encode_tmap_4d(&tmDO128, dout, dims, sdo, box128, 2, true) || !encode_tmap_4d(&tmDO64, dout, dims, sdo, box64, 2, true))
      return -5;
  }
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)a.Hkv, (uint64_t)a.Sk, (uint64_t)a.B};
    const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)kv_tstride * 2, (uint64_t)kv_bstride * 2};
    const uint32_t box128[4] = {64, 1, 128, 1};
    if (!encode_tmap_4d(&tmK, k, dims, strides, box128, 2, true) || !encode_tmap_4d(&tmV, v, dims, strides, box128, 2, true))
      return -5;
  }
  constexpr size_t smem_dkdv = 1024 + 2 * (kKvRows * D * 2) + 2 * kQStages * (kQSub * D * 2) + kQStages * (4 * kQSub * 4) + 256;
  constexpr int k_stages = (D == 128) ? (MODE >= 2 ? 2 : 3) : 4;
  constexpr size_t smem_dq = (4 + k_stages) * (128 * D * 2) + (MODE >= 2 ? k_stages : 0) * (2 * kDqKeys * 4) + 256;
  static bool configured[64] = {false};   // one flag set per (D, MODE) instantiation
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    MB_CHECK_CUDA(cudaFuncSetAttribute(flash_bwd_dkdv_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_dkdv)));
    MB_CHECK_CUDA(cudaFuncSetAttribute(flash_bwd_dq_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_dq)));
    configured[dev & 63] = true;
  }
  {
    dim3 grid((a.Sk + kKvRows - 1) / kKvRows, a.Hkv * a.split, a.B);
    flash_bwd_dkdv_kernel<D, MODE><<<grid, kBwThreads, smem_dkdv, stream>>>(tmQ64, tmDO64, tmK, tmV, a);
    count_launch();
    if (a.split > 1) {
      const long long quads = kv_elems / 4;
      flash_bwd_finish_split_kernel<<<static_cast<unsigned>((quads + 255) / 256), 256, 0, stream>>>(
          a.dk_tmp, a.dv_tmp, a.dk, a.dv, static_cast<long long>(a.B) * a.Sk, a.Hkv * D, a.dkv_tstride, a.out_fp32, a.accumulate);
      count_launch();
    }
  }
  {
    dim3 grid((a.Sq + kDqRows - 1) / kDqRows, a.Hq, a.B);
    flash_bwd_dq_kernel<D, MODE><<<grid, kBwThreads, smem_dq, stream>>>(tmQ128, tmDO128, tmK, tmV, a);
    count_launch();
  }
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace mb

#ifdef MB_FLASH_PROBE
MB_API int mb_flash_probe_read(long long* host_out) {
  return static_cast<int>(cudaMemcpyFromSymbol(host_out, mb::g_flash_probe, sizeof(long long) * 16 * 256));
}
#endif

// Number of 4-byte words of scratch memory mb_flash_attn_bwd needs for these sizes.
MB_API long long mb_flash_attn_bwd_scratch_words(int B, int Sq, int Sk, int Hq, int Hkv, int D) {
  const long long sq_pad = (static_cast<long long>(Sq) + 127) / 128 * 128, sk_pad = (static_cast<long long>(Sk) + 127) / 128 * 128;
  long long words = 2 * B * Hq * sq_pad + 2 * B * sq_pad + 2 * B * sk_pad;
  if (Hkv >= 1 && Hq % Hkv == 0 && mb::dkdv_split(B, Sk, Hq, Hkv) > 1) words += 2ll * B * Sk * Hkv * D;   // fp32 dK / dV sums
  return words;
}

// q, out, dout [B, Sq, Hq, D]; k, v [B, Sk, Hkv, D] bf16 (heads contiguous inside a token; token / batch strides in
// elements, multiples of 8); lse [B, Hq, Sq] fp32 from the forward. dq [B, Sq, Hq, D], dk / dv [B, Sk, Hkv, D]: bf16, or
// fp32 when out_fp32 (then `accumulate` adds to their contents). scratch: mb_flash_attn_bwd_scratch_words() words.
MB_API int mb_flash_attn_bwd(const void* q, long long q_tstride, long long q_bstride, const void* k, const void* v,
                             long long kv_tstride, long long kv_bstride, const void* out, long long o_tstride, long long o_bstride,
                             const void* dout, long long do_tstride, long long do_bstride, const float* lse, void* dq,
                             long long dq_tstride, void* dk, void* dv, long long dkv_tstride, const int* q_pos, const int* k_pos,
                             const int* q_seq, const int* k_seq, float* scratch, int B, int Sq, int Sk, int Hq, int Hkv, int D,
                             int mode, float scale, int out_fp32, int accumulate, cudaStream_t stream) {
  using namespace mb;
  if ((D != 64 && D != 128) || Hkv < 1 || Hq % Hkv != 0 || B < 1 || Sq < 1 || Sk < 1) {
    set_last_error("mb_flash_attn_bwd: head_dim must be 64 or 128, query heads a multiple of key/value heads");
    return -1;
  }
  if (mode < 0 || mode > 3 || (mode == 2 && (!q_pos || !k_pos)) || ((q_seq == nullptr) != (k_seq == nullptr)) ||
      (mode == 3 && !q_seq) || (accumulate && !out_fp32)) {
    set_last_error("mb_flash_attn_bwd: bad mask mode, missing position / sequence-id arrays, or accumulate without fp32 outputs");
    return -2;
  }
  const long long strides[] = {q_tstride, q_bstride, kv_tstride, kv_bstride, o_tstride, o_bstride, do_tstride, do_bstride,
                               dq_tstride, dkv_tstride};
  for (long long s : strides)
    if (s & 7) {
      set_last_error("mb_flash_attn_bwd: strides must be multiples of 8 elements");
      return -3;
    }
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) |
       reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(scratch)) & 15) {
    set_last_error("mb_flash_attn_bwd: tensors must be 16-byte aligned");
    return -3;
  }
  int* status = status_ptr();
  if (!status) return -4;
  FlashBwdArgs a{};
  a.dq = dq, a.dk = dk, a.dv = dv;
  a.dq_tstride = dq_tstride, a.dkv_tstride = dkv_tstride;
  a.B = B, a.Sq = Sq, a.Sk = Sk, a.Hq = Hq, a.Hkv = Hkv;
  a.Sq_pad = (Sq + 127) / 128 * 128, a.Sk_pad = (Sk + 127) / 128 * 128;
  a.mode = mode, a.out_fp32 = out_fp32, a.accumulate = accumulate;
  a.scale = scale, a.scale_log2 = scale * kBwLog2e;
  a.status = status;
#ifdef MB_FLASH_PROBE
  a.dbg = getenv("MB_FLASH_DBG") ? atoi(getenv("MB_FLASH_DBG")) : 0;
#endif
#define MB_BWD_ARGS q, q_tstride, q_bstride, k, v, kv_tstride, kv_bstride, out, o_tstride, o_bstride, dout, do_tstride, do_bstride, \
                    lse, q_pos, k_pos, q_seq, k_seq, scratch, a, stream
  if (D == 128) {
    switch (mode) {
      case 0: return launch_flash_bwd<128, 0>(MB_BWD_ARGS);
      case 1: return launch_flash_bwd<128, 1>(MB_BWD_ARGS);
      case 2: return launch_flash_bwd<128, 2>(MB_BWD_ARGS);
      default: return launch_flash_bwd<128, 3>(MB_BWD_ARGS);
    }
  }
  switch (mode) {
    case 0: return launch_flash_bwd<64, 0>(MB_BWD_ARGS);
    case 1: return launch_flash_bwd<64, 1>(MB_BWD_ARGS);
    case 2: return launch_flash_bwd<64, 2>(MB_BWD_ARGS);
    default: return launch_flash_bwd<64, 3>(MB_BWD_ARGS);
  }
#undef MB_BWD_ARGS
}
