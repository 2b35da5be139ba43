// Sharded-optimizer data paths over peer memory (NVLink, CUDA-IPC mappings) for sm_100a.
//
//  * peer_reduce_shard_kernel: the OWNER of a shard reads that slice of the flat gradient bucket from every rank of the
//    group (plain 16-byte peer loads, all issued before the first use), sums in fp32 in rank order, applies `scale`
//    (1/world x role correction), writes or accumulates the shard gradient and adds sum(g^2) of the result to a device
//    scalar. One pass replaces
//    reduce-scatter + cast + scale + accumulate + norm partial (reference runtime/plugins/zero1.py:183-231,
//    zero2.py:262-330 and runtime/plugins/grad_clip.py).
//  * adamw_push_kernel: AdamW on the fp32 master shard (clip coefficient read from device memory) and the bf16 result
//    stored straight into EVERY rank's flat parameter buffer (16-byte peer stores): optimizer step + cast + all-gather in
//    one pass (reference runtime/optim.py:43-104 + zero1.py:264-283).
//
// Neither kernel waits on another GPU: the callers order them against the peers' kernels with stream-ordered group
// barriers on the host side, so nothing here can spin.
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kZfThreads = 256;
constexpr int kZfMaxWorld = 16;

struct PeerPtrs {
  const void* p[kZfMaxWorld];
};
struct PeerDst {
  void* p[kZfMaxWorld];
};

__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// out_mode: 0 = write bf16, 1 = write fp32, 2 = accumulate into fp32, 3 = accumulate into bf16.
// `src.p[r]` points at element 0 of the shard inside rank r's bucket (bf16). `vec` = every pointer is 16-byte aligned.
template <bool kVec>
__global__ void __launch_bounds__(kZfThreads)
peer_reduce_shard_kernel(PeerPtrs src, int world, int rank, long long n, float scale, void* __restrict__ out, int out_mode,
                         double* __restrict__ sumsq) {
  float local_sq = 0.f;
  const long long tid = static_cast<long long>(blockIdx.x) * kZfThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kZfThreads;
  if constexpr (kVec) {
    const long long nvec = n >> 3;
    for (long long i = tid; i < nvec; i += nthreads) {
      uint4 raw[kZfMaxWorld];
      // every load is issued before the first use (up to 16 peer reads of 16 bytes in flight per thread)
#pragma unroll
      for (int r = 0; r < kZfMaxWorld; ++r)
        if (r < world) raw[r] = reinterpret_cast<const uint4*>(src.p[r])[i];
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // summed in RANK order so that the result does not depend on which rank owns the shard
#pragma unroll
      for (int r = 0; r < kZfMaxWorld; ++r)
        if (r < world) {
          float f[8];
          bf16x8_to_float(raw[r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= scale;
      if (out_mode == 0) {
        const uint4 o = float_to_bf16x8(acc);
        float f[8];
        bf16x8_to_float(o, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) local_sq += f[j] * f[j];
        reinterpret_cast<uint4*>(out)[i] = o;
      } else if (out_mode == 3) {
        float f[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(out)[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += acc[j];
        const uint4 o = float_to_bf16x8(f);
        bf16x8_to_float(o, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) local_sq += f[j] * f[j];
        reinterpret_cast<uint4*>(out)[i] = o;
      } else {
        float4* o = reinterpret_cast<float4*>(out) + 2 * i;
        float4 a = make_float4(acc[0], acc[1], acc[2], acc[3]), b = make_float4(acc[4], acc[5], acc[6], acc[7]);
        if (out_mode == 2) {
          const float4 pa = o[0], pb = o[1];
          a.x += pa.x, a.y += pa.y, a.z += pa.z, a.w += pa.w;
          b.x += pb.x, b.y += pb.y, b.z += pb.z, b.w += pb.w;
        }
        local_sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        o[0] = a;
        o[1] = b;
      }
    }
  }
  // scalar path: everything when unaligned, otherwise the tail of fewer than 8 elements
  const long long first = kVec ? (n & ~7ll) : 0;
  for (long long i = first + tid; i < n; i += nthreads) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src.p[r])[i]);
    acc *= scale;
    float res;
    if (out_mode == 0) {
      const __nv_bfloat16 o = __float2bfloat16(acc);
      reinterpret_cast<__nv_bfloat16*>(out)[i] = o;
      res = __bfloat162float(o);
    } else if (out_mode == 3) {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + i;
      const __nv_bfloat16 w = __float2bfloat16(__bfloat162float(*o) + acc);
      *o = w;
      res = __bfloat162float(w);
    } else {
      float* o = reinterpret_cast<float*>(out) + i;
      res = (out_mode == 2) ? *o + acc : acc;
      *o = res;
    }
    local_sq += res * res;
  }
  if (sumsq) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o);
    __shared__ float warp_sq[kZfThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_sq[threadIdx.x >> 5] = local_sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      double t = 0.0;
      for (int w = 0; w < kZfThreads / 32; ++w) t += static_cast<double>(warp_sq[w]);
      if (t != 0.0) atomicAdd(sumsq, t);
    }
  }
}

// AdamW over one contiguous fp32 master shard; the bf16 result is stored into `ndst` destinations, in the order given
// (each = element 0 of the shard inside some rank's flat parameter buffer; the caller lists the peers in ring order
// starting after itself, so that the ranks do not all write to the same GPU at once, and its own buffers last).
template <bool kVec>
__global__ void __launch_bounds__(kZfThreads)
adamw_push_kernel(float* __restrict__ master, const void* __restrict__ grad, int grad_bf16, float* __restrict__ m,
                  float* __restrict__ v, long long n, PeerDst dst, int ndst, float lr, float beta1, float beta2,
                  float eps, float weight_decay, float bc1, float bc2_sqrt, const float* __restrict__ grad_scale_ptr) {
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * weight_decay;
  const long long tid = static_cast<long long>(blockIdx.x) * kZfThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kZfThreads;
  auto update = [&](float g, float& pv, float& mv, float& vv) {
    g *= gs;
    pv *= decay;
    mv = beta1 * mv + (1.f - beta1) * g;
    vv = beta2 * vv + (1.f - beta2) * g * g;
    pv -= step_size * mv / (sqrtf(vv) / bc2_sqrt + eps);
  };
  if constexpr (kVec) {
    const long long nvec = n >> 3;
    for (long long i = tid; i < nvec; i += nthreads) {
      float g[8], p[8], mm[8], vv[8];
      if (grad_bf16) {
        bf16x8_to_float(reinterpret_cast<const uint4*>(grad)[i], g);
      } else {
        const float4 a = reinterpret_cast<const float4*>(grad)[2 * i], b = reinterpret_cast<const float4*>(grad)[2 * i + 1];
        g[0] = a.x, g[1] = a.y, g[2] = a.z, g[3] = a.w, g[4] = b.x, g[5] = b.y, g[6] = b.z, g[7] = b.w;
      }
      float4* p4 = reinterpret_cast<float4*>(master) + 2 * i;
      float4* m4 = reinterpret_cast<float4*>(m) + 2 * i;
      float4* v4 = reinterpret_cast<float4*>(v) + 2 * i;
      *reinterpret_cast<float4*>(p) = p4[0], *reinterpret_cast<float4*>(p + 4) = p4[1];
      *reinterpret_cast<float4*>(mm) = m4[0], *reinterpret_cast<float4*>(mm + 4) = m4[1];
      *reinterpret_cast<float4*>(vv) = v4[0], *reinterpret_cast<float4*>(vv + 4) = v4[1];
#pragma unroll
      for (int j = 0; j < 8; ++j) update(g[j], p[j], mm[j], vv[j]);
      p4[0] = *reinterpret_cast<float4*>(p), p4[1] = *reinterpret_cast<float4*>(p + 4);
      m4[0] = *reinterpret_cast<float4*>(mm), m4[1] = *reinterpret_cast<float4*>(mm + 4);
      v4[0] = *reinterpret_cast<float4*>(vv), v4[1] = *reinterpret_cast<float4*>(vv + 4);
      const uint4 o = float_to_bf16x8(p);
#pragma unroll
      for (int d = 0; d < kZfMaxWorld; ++d)
        if (d < ndst) reinterpret_cast<uint4*>(dst.p[d])[i] = o;
    }
  }
  const long long first = kVec ? (n & ~7ll) : 0;
  for (long long i = first + tid; i < n; i += nthreads) {
    const float g = grad_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i]) : reinterpret_cast<const float*>(grad)[i];
    float pv = master[i], mv = m[i], vv = v[i];
    update(g, pv, mv, vv);
    master[i] = pv, m[i] = mv, v[i] = vv;
    const __nv_bfloat16 o = __float2bfloat16(pv);
    for (int d = 0; d < ndst; ++d) reinterpret_cast<__nv_bfloat16*>(dst.p[d])[i] = o;
  }
}

// In-place all-reduce of flat gradient buckets over peer memory: the owner of a slice reads it from every rank's bucket,
// sums in fp32 in rank order, scales, and stores the result back into EVERY rank's bucket (16-byte peer loads and
// stores). Owners' slices are disjoint, so nobody reads what another block writes. One kernel replaces the
// all-reduce(AVG) of the data-parallel plugins (reference runtime/plugins/ddp.py:20-203); the callers bracket it with
// stream-ordered group barriers. T = __nv_bfloat16 (8 per 16 bytes) or float (4 per 16 bytes).
template <typename T>
__global__ void __launch_bounds__(kZfThreads)
peer_all_reduce_kernel(PeerDst bufs, int world, long long n, float scale) {
  constexpr int kPer = 16 / sizeof(T);
  const long long tid = static_cast<long long>(blockIdx.x) * kZfThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kZfThreads;
  const long long nvec = n / kPer;
  for (long long i = tid; i < nvec; i += nthreads) {
    uint4 raw[kZfMaxWorld];
#pragma unroll
    for (int r = 0; r < kZfMaxWorld; ++r)
      if (r < world) raw[r] = reinterpret_cast<const uint4*>(bufs.p[r])[i];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kZfMaxWorld; ++r)
      if (r < world) {
        if constexpr (sizeof(T) == 2) {
          float f[8];
          bf16x8_to_float(raw[r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        } else {
          const float* f = reinterpret_cast<const float*>(&raw[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] += f[j];
        }
      }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= scale;
    uint4 o;
    if constexpr (sizeof(T) == 2) o = float_to_bf16x8(acc);
    else o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
#pragma unroll
    for (int r = 0; r < kZfMaxWorld; ++r)
      if (r < world) reinterpret_cast<uint4*>(bufs.p[r])[i] = o;
  }
  for (long long i = nvec * kPer + tid; i < n; i += nthreads) {     // tail of fewer than 16 bytes
    float a = 0.f;
    for (int r = 0; r < world; ++r) {
      if constexpr (sizeof(T) == 2) a += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bufs.p[r])[i]);
      else a += reinterpret_cast<const float*>(bufs.p[r])[i];
    }
    a *= scale;
    for (int r = 0; r < world; ++r) {
      if constexpr (sizeof(T) == 2) reinterpret_cast<__nv_bfloat16*>(bufs.p[r])[i] = __float2bfloat16(a);
      else reinterpret_cast<float*>(bufs.p[r])[i] = a;
    }
  }
}

static int zf_grid(long long n) {
  long long blocks = (n / 8 + kZfThreads - 1) / kZfThreads;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mb

// srcs: `world` host pointers (device addresses, bf16), each at element 0 of the shard in that rank's bucket.
MB_API int mb_peer_reduce_shard(const void* const* srcs, int world, int rank, long long n, float scale, void* out, int out_mode,
                                double* sumsq, cudaStream_t stream) {
  using namespace mb;
  if (world < 1 || world > kZfMaxWorld || rank < 0 || rank >= world || out_mode < 0 || out_mode > 3) {
    set_last_error("mb_peer_reduce_shard: needs 1 <= world <= 16, 0 <= rank < world, out_mode in 0..3");
    return -1;
  }
  if (n <= 0) return 0;
  PeerPtrs src{};
  bool vec = aligned16(out);
  for (int r = 0; r < world; ++r) {
    src.p[r] = srcs[r];
    vec = vec && aligned16(srcs[r]);
  }
  if (vec)
    peer_reduce_shard_kernel<true><<<zf_grid(n), kZfThreads, 0, stream>>>(src, world, rank, n, scale, out, out_mode, sumsq);
  else
    peer_reduce_shard_kernel<false><<<zf_grid(n), kZfThreads, 0, stream>>>(src, world, rank, n, scale, out, out_mode, sumsq);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_adamw_push(float* master, const void* grad, int grad_bf16, float* m, float* v, long long n, void* const* dsts, int ndst,
                         float lr, float beta1, float beta2, float eps, float weight_decay, float bias_corr1,
                         float bias_corr2_sqrt, const float* grad_scale, cudaStream_t stream) {
  using namespace mb;
  if (ndst < 1 || ndst > kZfMaxWorld) {
    set_last_error("mb_adamw_push: needs 1 <= destinations <= 16");
    return -1;
  }
  if (n <= 0) return 0;
  PeerDst dst{};
  bool vec = aligned16(master) && aligned16(grad) && aligned16(m) && aligned16(v);
  for (int r = 0; r < ndst; ++r) {
    dst.p[r] = dsts[r];
    vec = vec && aligned16(dsts[r]);
  }
  if (vec)
    adamw_push_kernel<true><<<zf_grid(n), kZfThreads, 0, stream>>>(master, grad, grad_bf16, m, v, n, dst, ndst, lr, beta1, beta2,
                                                                   eps, weight_decay, bias_corr1, bias_corr2_sqrt, grad_scale);
  else
    adamw_push_kernel<false><<<zf_grid(n), kZfThreads, 0, stream>>>(master, grad, grad_bf16, m, v, n, dst, ndst, lr, beta1, beta2,
                                                                    eps, weight_decay, bias_corr1, bias_corr2_sqrt, grad_scale);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// bufs[r]: device address of THIS rank's slice (first element) inside rank r's bucket; 16-byte aligned. n elements.
MB_API int mb_peer_all_reduce(void* const* bufs, int world, long long n, int is_bf16, float scale, cudaStream_t stream) {
  using namespace mb;
  if (world < 1 || world > kZfMaxWorld) {
    set_last_error("mb_peer_all_reduce: needs 1 <= world <= 16");
    return -1;
  }
  if (n <= 0) return 0;
  PeerDst b{};
  for (int r = 0; r < world; ++r) {
    if (!aligned16(bufs[r])) {
      set_last_error("mb_peer_all_reduce: slices must start on a 16-byte boundary");
      return -2;
    }
    b.p[r] = bufs[r];
  }
  if (is_bf16)
    peer_all_reduce_kernel<__nv_bfloat16><<<zf_grid(n), kZfThreads, 0, stream>>>(b, world, n, scale);
  else
    peer_all_reduce_kernel<float><<<zf_grid(n / 2 + 1), kZfThreads, 0, stream>>>(b, world, n, scale);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
