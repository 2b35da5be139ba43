// MoE router for sm_100a: softmax over experts, top-k selection (optionally renormalised), per-expert assignment counts
// and per-expert probability sums (for the load-balance loss) in ONE pass over the router logits, and the matching
// backward. One warp per token; a lane holds up to 32 experts in registers, so up to 1024 experts are supported.
// The reference computes this with separate ATen softmax / argmax / gather / one_hot / mean launches
// (runtime/layers/moe.py:74-80,158-163); top-k > 1 and renormalisation go beyond its top-1 router.
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kRouterMaxPerLane = 32;
constexpr int kRouterWarps = 8;

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, long long i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits [N, E]; idx [N, k] int64; gate [N, k] fp32; rowmax/rowsum [N] fp32 (saved for backward);
// prob_sum [E] fp32 and counts [E] int32 are ACCUMULATED (caller zeroes them).
template <typename T>
__global__ void __launch_bounds__(32 * kRouterWarps)
moe_router_fwd_kernel(const T* __restrict__ logits, long long N, int E, int k, int renorm, long long* __restrict__ idx,
                      float* __restrict__ gate, float* __restrict__ rowmax, float* __restrict__ rowsum,
                      float* __restrict__ prob_sum, int* __restrict__ counts) {
  extern __shared__ float s_prob[];   // [E] per-block partial probability sums
  int* s_cnt = reinterpret_cast<int*>(s_prob + E);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    s_prob[e] = 0.f;
    s_cnt[e] = 0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_lane = (E + 31) / 32;
  for (long long t = static_cast<long long>(blockIdx.x) * kRouterWarps + warp; t < N;
       t += static_cast<long long>(gridDim.x) * kRouterWarps) {
    float p[kRouterMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      p[j] = (j < per_lane && e < E) ? load_as_float(logits, t * E + e) : -INFINITY;
      m = fmaxf(m, p[j]);
    }
    m = warp_max_f(m);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      p[j] = (j < per_lane && lane + 32 * j < E) ? __expf(p[j] - m) : 0.f;
      s += p[j];
    }
    s = warp_sum_f(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      p[j] *= inv;
      if (j < per_lane && lane + 32 * j < E) atomicAdd(&s_prob[lane + 32 * j], p[j]);
    }
    if (lane == 0) {
      rowmax[t] = m;
      rowsum[t] = s;
    }
    // top-k by k rounds of warp arg-max (ties: lower expert index), selected entries are masked out
    unsigned taken = 0u;
    float chosen_p[8];
    int chosen_e[8];
    float chosen_sum = 0.f;
    for (int r = 0; r < k; ++r) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        if (j < per_lane && e < E && !((taken >> j) & 1u) && (p[j] > best || (p[j] == best && e < best_e))) {
          best = p[j];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
      chosen_p[r] = best;
      chosen_e[r] = best_e;
      chosen_sum += best;
    }
    if (lane == 0) {
      const float scale = (renorm && k > 1) ? 1.f / chosen_sum : 1.f;
      for (int r = 0; r < k; ++r) {
        idx[t * k + r] = chosen_e[r];
        gate[t * k + r] = chosen_p[r] * scale;
        atomicAdd(&s_cnt[chosen_e[r]], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_prob[e] != 0.f) atomicAdd(&prob_sum[e], s_prob[e]);
    if (s_cnt[e] != 0) atomicAdd(&counts[e], s_cnt[e]);
  }
}

// dlogits[t, e] = p_e * (dLdp_e - sum_e' dLdp_e' p_e'), dLdp = (selected ? d gate -> d prob) + aux_w[e]
template <typename T>
__global__ void __launch_bounds__(32 * kRouterWarps)
moe_router_bwd_kernel(const T* __restrict__ logits, long long N, int E, int k, int renorm, const long long* __restrict__ idx,
                      const float* __restrict__ gate, const float* __restrict__ dgate, const float* __restrict__ rowmax,
                      const float* __restrict__ rowsum, const float* __restrict__ aux_w, T* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_lane = (E + 31) / 32;
  for (long long t = static_cast<long long>(blockIdx.x) * kRouterWarps + warp; t < N;
       t += static_cast<long long>(gridDim.x) * kRouterWarps) {
    const float m = rowmax[t], inv = 1.f / rowsum[t];
    // gradient with respect to the selected probabilities
    float sel_grad[8];
    int sel_e[8];
    float dot = 0.f, psel = 0.f;
    for (int r = 0; r < k; ++r) {
      sel_e[r] = static_cast<int>(idx[t * k + r]);
      dot += dgate[t * k + r] * gate[t * k + r];
      psel += __expf(load_as_float(logits, t * E + sel_e[r]) - m) * inv;
    }
    const bool rn = renorm && k > 1;
    for (int r = 0; r < k; ++r) sel_grad[r] = rn ? (dgate[t * k + r] - dot) / psel : dgate[t * k + r];
    float p[kRouterMaxPerLane], g[kRouterMaxPerLane];
    float c = 0.f;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      const bool in = j < per_lane && e < E;
      p[j] = in ? __expf(load_as_float(logits, t * E + e) - m) * inv : 0.f;
      float ge = (in && aux_w) ? aux_w[e] : 0.f;
      for (int r = 0; r < k; ++r)
        if (in && sel_e[r] == e) ge += sel_grad[r];
      g[j] = ge;
      c += ge * p[j];
    }
    c = warp_sum_f(c);
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < per_lane && e < E) {
        const float d = p[j] * (g[j] - c);
        if constexpr (sizeof(T) == 2) dlogits[t * E + e] = __float2bfloat16(d);
        else dlogits[t * E + e] = d;
      }
    }
  }
}

static int router_grid(long long N) {
  long long b = (N + kRouterWarps - 1) / kRouterWarps;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace mb

MB_API int mb_moe_router_fwd(const void* logits, int is_bf16, long long N, int E, int k, int renorm, long long* idx, float* gate,
                             float* rowmax, float* rowsum, float* prob_sum, int* counts, cudaStream_t stream) {
  using namespace mb;
  if (E < 1 || E > 32 * kRouterMaxPerLane || k < 1 || k > 8 || k > E) {
    set_last_error("mb_moe_router_fwd: needs 1 <= experts <= 1024 and 1 <= k <= min(8, experts)");
    return -1;
  }
  if (N <= 0) return 0;
  const size_t smem = static_cast<size_t>(E) * (sizeof(float) + sizeof(int));
  if (is_bf16)
    moe_router_fwd_kernel<__nv_bfloat16><<<router_grid(N), 32 * kRouterWarps, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), N, E, k, renorm, idx, gate, rowmax, rowsum, prob_sum, counts);
  else
    moe_router_fwd_kernel<float><<<router_grid(N), 32 * kRouterWarps, smem, stream>>>(
        static_cast<const float*>(logits), N, E, k, renorm, idx, gate, rowmax, rowsum, prob_sum, counts);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_moe_router_bwd(const void* logits, int is_bf16, long long N, int E, int k, int renorm, const long long* idx,
                             const float* gate, const float* dgate, const float* rowmax, const float* rowsum,
                             const float* aux_w, void* dlogits, cudaStream_t stream) {
  using namespace mb;
  if (E < 1 || E > 32 * kRouterMaxPerLane || k < 1 || k > 8) {
    set_last_error("mb_moe_router_bwd: needs 1 <= experts <= 1024 and 1 <= k <= 8");
    return -1;
  }
  if (N <= 0) return 0;
  if (is_bf16)
    moe_router_bwd_kernel<__nv_bfloat16><<<router_grid(N), 32 * kRouterWarps, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), N, E, k, renorm, idx, gate, dgate, rowmax, rowsum, aux_w,
        static_cast<__nv_bfloat16*>(dlogits));
  else
    moe_router_bwd_kernel<float><<<router_grid(N), 32 * kRouterWarps, 0, stream>>>(
        static_cast<const float*>(logits), N, E, k, renorm, idx, gate, dgate, rowmax, rowsum, aux_w, static_cast<float*>(dlogits));
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
