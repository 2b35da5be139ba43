// Cross-entropy (forward + in-place gradient), multi-tensor AdamW with fp32 masters, multi-tensor sum of
// squares and scaling. All for sm_100a; bandwidth-bound, 128-bit accesses where alignment allows.
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kCeThreads = 512;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) {
  return p[i];
}
template <typename T>
__device__ __forceinline__ void st_logit(T* p, long long i, float v);
template <>
__device__ __forceinline__ void st_logit<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}
template <>
__device__ __forceinline__ void st_logit<float>(float* p, long long i, float v) {
  p[i] = v;
}

// One block per row. loss_rows[row] = lse - logit[label] (0 for ignored rows); lse_out[row] = log-sum-exp.
// If grad_out != nullptr: grad_out[row, :] = (softmax - onehot) * scale_row, where
// scale_row = (label != ignore) * (*grad_scale_ptr). grad_out may BE logits (in place): every thread rewrites only the
// columns it read itself, and the target logit needed for the loss is captured during the first pass, before any
// column is overwritten. (logits is therefore not declared __restrict__.)
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const T* logits, long long row_stride, const long long* __restrict__ labels,
                     float* __restrict__ loss_rows, float* __restrict__ lse_out, T* grad_out,
                     const float* __restrict__ grad_scale_ptr, int V, long long ignore_index, int* status) {
  __shared__ float red_m[kCeThreads / 32], red_s[kCeThreads / 32];
  __shared__ float target_logit;
  const long long row = blockIdx.x;
  const T* lr = logits + row * row_stride;
  const long long label = labels[row];
  const bool active = label != ignore_index;
  if (active && (label < 0 || label >= V)) {
    if (threadIdx.x == 0) {
      atomicOr(&status[0], MB_ERR_BAD_INDEX);
      status[2] = static_cast<int>(label);
    }
  }
  // online max / sum
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < V; c += kCeThreads) {
    const float v = ld_logit<T>(lr, c);
    if (c == label) target_logit = v;      // exactly one thread of the block owns the target column
    if (v > m) {
      s = s * __expf(m - v) + 1.f;
      m = v;
    } else {
      s += __expf(v - m);
    }
  }
  // combine across the warp, then across warps
  {
    // a thread (or a whole warp, when V < block size) without elements has m = -inf: its term must be 0, not exp(nan)
    const float wm = warp_max(m);
    s = warp_add(m == -INFINITY ? 0.f : s * __expf(m - wm));
    m = wm;
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red_m[w] = m, red_s[w] = s;
  __syncthreads();
  if (w == 0) {
    float mm = l < kCeThreads / 32 ? red_m[l] : -INFINITY;
    float sv = l < kCeThreads / 32 ? red_s[l] : 0.f;
    const float gm = warp_max(mm);
    sv = warp_add(mm == -INFINITY ? 0.f : sv * __expf(mm - gm));
    if (l == 0) red_m[0] = gm, red_s[0] = sv;
  }
  __syncthreads();
  const float gmax = red_m[0], gsum = red_s[0];
  const float lse = gmax + __logf(gsum);
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[row] = lse;
    float lrow = 0.f;
    if (active && label >= 0 && label < V) lrow = lse - target_logit;
    loss_rows[row] = lrow;
  }
  if (grad_out) {
    T* gr = grad_out + row * row_stride;
    const float scale = active ? *grad_scale_ptr : 0.f;
    for (int c = threadIdx.x; c < V; c += kCeThreads) {
      float p = __expf(ld_logit<T>(lr, c) - lse);
      if (c == label) p -= 1.f;
      st_logit<T>(gr, c, p * scale);
    }
  }
}

// ------------------------------------------------------------------------------------------------ multi-tensor
// Table row layout (8 x int64 per tensor): master fp32*, grad*, exp_avg fp32*, exp_avg_sq fp32*, low-precision bf16* (or 0),
// numel, grad_is_bf16, first_chunk (prefix sum of chunk counts). hyper row (per tensor, 2 floats): bias corrections.
constexpr int kMtChunk = 8192;
constexpr int kMtThreads = 256;

struct MtEntry {
  long long master, grad, m, v, lowp, numel, grad_bf16, first_chunk;
};

__device__ __forceinline__ int find_tensor(const MtEntry* __restrict__ tab, int n, long long chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tab[mid].first_chunk <= chunk)
      lo = mid;
    else
      hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(kMtThreads)
adamw_mt_kernel(const MtEntry* __restrict__ tab, const float* __restrict__ bias_corr, int ntensors, float lr, float beta1,
                float beta2, float eps, float weight_decay, const float* __restrict__ grad_scale_ptr) {
  const long long chunk = blockIdx.x;
  const int t = find_tensor(tab, ntensors, chunk);
  const MtEntry e = tab[t];
  const long long start = (chunk - e.first_chunk) * kMtChunk;
  const long long end = min(start + kMtChunk, e.numel);
  float* p = reinterpret_cast<float*>(e.master);
  float* m = reinterpret_cast<float*>(e.m);
  float* v = reinterpret_cast<float*>(e.v);
  __nv_bfloat16* lp = reinterpret_cast<__nv_bfloat16*>(e.lowp);
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  const float bc1 = bias_corr[2 * t], bc2_sqrt = bias_corr[2 * t + 1];
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * weight_decay;
  for (long long i = start + threadIdx.x; i < end; i += kMtThreads) {
    float g = e.grad_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.grad)[i])
                          : reinterpret_cast<const float*>(e.grad)[i];
    g *= gs;
    float pv = p[i] * decay;
    const float mv = beta1 * m[i] + (1.f - beta1) * g;
    const float vv = beta2 * v[i] + (1.f - beta2) * g * g;
    const float denom = sqrtf(vv) / bc2_sqrt + eps;
    pv -= step_size * mv / denom;
    p[i] = pv, m[i] = mv, v[i] = vv;
    if (lp) lp[i] = __float2bfloat16(pv);
  }
}

// Table row for reductions/scaling: ptr, numel, is_bf16, first_chunk, weight (as double bits), pad...
struct MtVecEntry {
  long long ptr, numel, is_bf16, first_chunk;
  double weight;
  long long pad[3];
};

__global__ void __launch_bounds__(kMtThreads)
sumsq_mt_kernel(const MtVecEntry* __restrict__ tab, int ntensors, double* __restrict__ out) {
  __shared__ float red[kMtThreads / 32];
  const long long chunk = blockIdx.x;
  int lo = 0, hi = ntensors - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tab[mid].first_chunk <= chunk)
      lo = mid;
    else
      hi = mid - 1;
  }
  const MtVecEntry e = tab[lo];
  const long long start = (chunk - e.first_chunk) * kMtChunk;
  const long long end = min(start + kMtChunk, e.numel);
  float acc = 0.f;
  for (long long i = start + threadIdx.x; i < end; i += kMtThreads) {
    const float g = e.is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.ptr)[i])
                              : reinterpret_cast<const float*>(e.ptr)[i];
    acc += g * g;
  }
  acc = warp_add(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kMtThreads / 32 ? red[threadIdx.x] : 0.f;
    t = warp_add(t);
    if (threadIdx.x == 0) atomicAdd(out, static_cast<double>(t) * e.weight);
  }
}

__global__ void __launch_bounds__(kMtThreads)
scale_mt_kernel(const MtVecEntry* __restrict__ tab, int ntensors, const float* __restrict__ scale_ptr) {
  const float sc = *scale_ptr;
  if (sc == 1.f) return;
  const long long chunk = blockIdx.x;
  int lo = 0, hi = ntensors - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tab[mid].first_chunk <= chunk)
      lo = mid;
    else
      hi = mid - 1;
  }
  const MtVecEntry e = tab[lo];
  const long long start = (chunk - e.first_chunk) * kMtChunk;
  const long long end = min(start + kMtChunk, e.numel);
  for (long long i = start + threadIdx.x; i < end; i += kMtThreads) {
    if (e.is_bf16) {
      __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(e.ptr);
      p[i] = __float2bfloat16(__bfloat162float(p[i]) * sc);
    } else {
      reinterpret_cast<float*>(e.ptr)[i] *= sc;
    }
  }
}

// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)); norm_out = sqrt(sumsq)
__global__ void clip_coef_kernel(const double* sumsq, float max_norm, float* coef_out, float* norm_out) {
  const double n = sqrt(*sumsq);
  if (norm_out) *norm_out = static_cast<float>(n);
  float c = 1.f;
  if (max_norm > 0.f) {
    const double r = static_cast<double>(max_norm) / (n + 1e-6);
    c = r < 1.0 ? static_cast<float>(r) : 1.f;
  }
  *coef_out = c;
}

}  // namespace mb

using namespace mb;

MB_API int mb_cross_entropy(const void* logits, int logits_fp32, long long row_stride, const long long* labels,
                            float* loss_rows, float* lse_out, void* grad_out, const float* grad_scale, long long rows,
                            int V, long long ignore_index, cudaStream_t stream) {
  if (rows <= 0) return 0;
  int* status = status_ptr();
  if (logits_fp32)
    cross_entropy_kernel<float><<<static_cast<unsigned>(rows), kCeThreads, 0, stream>>>(
        static_cast<const float*>(logits), row_stride, labels, loss_rows, lse_out, static_cast<float*>(grad_out),
        grad_scale, V, ignore_index, status);
  else
    cross_entropy_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), kCeThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), row_stride, labels, loss_rows, lse_out,
        static_cast<__nv_bfloat16*>(grad_out), grad_scale, V, ignore_index, status);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_mt_chunk() { return kMtChunk; }

MB_API int mb_adamw_multi_tensor(const void* table, const float* bias_corr, int ntensors, long long total_chunks, float lr,
                                 float beta1, float beta2, float eps, float weight_decay, const float* grad_scale,
                                 cudaStream_t stream) {
  if (ntensors <= 0 || total_chunks <= 0) return 0;
  adamw_mt_kernel<<<static_cast<unsigned>(total_chunks), kMtThreads, 0, stream>>>(
      static_cast<const MtEntry*>(table), bias_corr, ntensors, lr, beta1, beta2, eps, weight_decay, grad_scale);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// out (double, device) must be zeroed by the caller; adds sum_t weight_t * ||x_t||^2.
MB_API int mb_sumsq_multi_tensor(const void* table, int ntensors, long long total_chunks, double* out,
                                 cudaStream_t stream) {
  if (ntensors <= 0 || total_chunks <= 0) return 0;
  sumsq_mt_kernel<<<static_cast<unsigned>(total_chunks), kMtThreads, 0, stream>>>(static_cast<const MtVecEntry*>(table),
                                                                                  ntensors, out);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_scale_multi_tensor(const void* table, int ntensors, long long total_chunks, const float* scale,
                                 cudaStream_t stream) {
  if (ntensors <= 0 || total_chunks <= 0) return 0;
  scale_mt_kernel<<<static_cast<unsigned>(total_chunks), kMtThreads, 0, stream>>>(static_cast<const MtVecEntry*>(table),
                                                                                  ntensors, scale);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_clip_coef(const double* sumsq, float max_norm, float* coef_out, float* norm_out, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, coef_out, norm_out);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
