// Memory-bound layer ops for sm_100a, bf16 in/out with fp32 math, 128-bit accesses:
//   RMSNorm forward (+fused residual add) / backward (+fused residual-gradient add, two-stage dw),
//   RoPE (interleaved pairs and rotate-half, forward and backward, in place, position gather),
//   SwiGLU forward / backward on separate or packed [gate | up] operands.
// Each kernel touches every byte once (HBM3e roofline is the target), so rows are kept in registers between
// the reduction and the write-back instead of being re-read.
#include "host.h"
#include "ptx.cuh"

namespace mb {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // 8 bf16 per vector -> rows up to 256*4*8 = 8192 elements stay in registers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]), v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]), v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

// y = w * (h * rsqrt(mean(h^2) + eps)), h = x (+ residual). Optionally writes h (the new residual stream).
// One block per row. H must be a multiple of 8.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + row * H) : nullptr;
  uint4* hr = h_out ? reinterpret_cast<uint4*>(h_out + row * H) : nullptr;
  float cache[kNormMaxVec][8];
  float ss = 0.f;
  const bool cached = nvec <= kNormThreads * kNormMaxVec;
#pragma unroll
  for (int j = 0; j < kNormMaxVec; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      float f[8];
      unpack8(xr[v], f);
      if (rr) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
        // the residual stream is stored in bf16: normalise exactly what later layers will read
        const uint4 packed = pack8(f);
        unpack8(packed, f);
        if (hr) hr[v] = packed;
      } else if (hr) {
        hr[v] = xr[v];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        cache[j][i] = f[i];
        ss += f[i] * f[i];
      }
    }
  }
  if (!cached) {
    for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
      float f[8];
      unpack8(xr[v], f);
      if (rr) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
        const uint4 packed = pack8(f);
        unpack8(packed, f);
        if (hr) hr[v] = packed;
      } else if (hr) {
        hr[v] = xr[v];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
  for (int j = 0; j < kNormMaxVec; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      float g[8], o[8];
      unpack8(wr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = cache[j][i] * rstd * g[i];
      yr[v] = pack8(o);
    }
  }
  if (!cached) {
    const uint4* src = hr ? reinterpret_cast<const uint4*>(h_out + row * H) : xr;  // h was written above when fused
    for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
      float f[8], g[8], o[8];
      unpack8(src[v], f);
      unpack8(wr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * g[i];
      yr[v] = pack8(o);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres);   dw_partial[block] += dy * xhat over the block's rows.
// Grid-stride over rows; each block owns one fp32 partial row of dw. H multiple of 8, H <= 8192 * k handled by loops.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, long long rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float dw_acc[kNormMaxVec][8];
#pragma unroll
  for (int j = 0; j < kNormMaxVec; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw_acc[j][i] = 0.f;
  float* my_partial = dw_partial + static_cast<long long>(blockIdx.x) * H;
  const bool wide = nvec > kNormThreads * kNormMaxVec;
  if (wide) {
    for (int c = threadIdx.x; c < H; c += kNormThreads) my_partial[c] = 0.f;
    __syncthreads();
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * H);
    const uint4* hr = reinterpret_cast<const uint4*>(h + row * H);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    float gy[kNormMaxVec][8], xh[kNormMaxVec][8];
#pragma unroll
    for (int j = 0; j < kNormMaxVec; ++j) {
      const int v = threadIdx.x + j * kNormThreads;
      if (v < nvec) {
        float a[8], b[8], g[8];
        unpack8(dyr[v], a);
        unpack8(hr[v], b);
        unpack8(wr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] = b[i] * rstd;
          dw_acc[j][i] += a[i] * xh[j][i];
          gy[j][i] = a[i] * g[i];
          dot += gy[j][i] * xh[j][i];
        }
      }
    }
    if (wide) {
      for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
        float a[8], b[8], g[8];
        unpack8(dyr[v], a);
        unpack8(hr[v], b);
        unpack8(wr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = b[i] * rstd;
          my_partial[v * 8 + i] += a[i] * xhat;
          dot += a[i] * g[i] * xhat;
        }
      }
    }
    dot = block_sum<kNormThreads>(dot, red);
    const float c = dot / static_cast<float>(H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
#pragma unroll
    for (int j = 0; j < kNormMaxVec; ++j) {
      const int v = threadIdx.x + j * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (gy[j][i] - xh[j][i] * c);
        if (drr) {
          float r[8];
          unpack8(drr[v], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        dxr[v] = pack8(o);
      }
    }
    if (wide) {
      for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
        float a[8], b[8], g[8], o[8];
        unpack8(dyr[v], a);
        unpack8(hr[v], b);
        unpack8(wr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (a[i] * g[i] - b[i] * rstd * c);
        if (drr) {
          float r[8];
          unpack8(drr[v], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        dxr[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kNormMaxVec; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) my_partial[v * 8 + i] = dw_acc[j][i];
    }
  }
}

// dw[c] (+)= sum_b partial[b][c]
__global__ void colsum_partials_kernel(const float* __restrict__ partial, int nblocks, int H,
                                       __nv_bfloat16* __restrict__ dw_bf16, float* __restrict__ dw_f32, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[static_cast<long long>(b) * H + c];
  if (dw_f32) dw_f32[c] = accumulate ? dw_f32[c] + s : s;
  if (dw_bf16) dw_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(dw_bf16[c]) + s : s);
}

// ------------------------------------------------------------------------------------------------ RoPE
// src/dst: [T, heads, D] with token strides in elements (heads*D contiguous inside a token); dst may equal src.
// pos: int64 [T] or nullptr (then position = pos_offset + t % seq_len). cos/sin: fp32 [max_pos, D/2].
// interleaved=1: pairs (2i, 2i+1); 0: pairs (i, i + D/2). sign = -1 gives the backward rotation.
// rotate=0 copies without rotating (used to move V into / out of a packed qkv buffer with the same launch shape).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ src, long long src_tstride, __nv_bfloat16* __restrict__ dst,
                            long long dst_tstride, long long T, int heads, int D, const long long* __restrict__ pos,
                            int pos_offset, int seq_len, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int max_pos, int interleaved, float sign, int rotate,
                            int* status) {
  const int half = D >> 1;
  const long long total = T * heads * half;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % half);
    const long long th = idx / half;
    const int hd = static_cast<int>(th % heads);
    const long long t = th / heads;
    float c = 1.f, s = 0.f;
    if (rotate) {
      long long p = pos ? pos[t] : (pos_offset + t % seq_len);
      if (p < 0 || p >= max_pos) {
        atomicOr(&status[0], MB_ERR_BAD_INDEX);
        status[2] = static_cast<int>(p);
        p = 0;
      }
      c = cos_t[p * half + i], s = sign * sin_t[p * half + i];
    }
    const __nv_bfloat16* in = src + t * src_tstride + static_cast<long long>(hd) * D;
    __nv_bfloat16* out = dst + t * dst_tstride + static_cast<long long>(hd) * D;
    if (interleaved) {
      const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(in)[i]);
      reinterpret_cast<__nv_bfloat162*>(out)[i] = __floats2bfloat162_rn(v.x * c - v.y * s, v.x * s + v.y * c);
    } else {
      const float a = __bfloat162float(in[i]), b = __bfloat162float(in[i + half]);
      out[i] = __float2bfloat16(a * c - b * s);
      out[i + half] = __float2bfloat16(a * s + b * c);
    }
  }
}

// ------------------------------------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                  long long in_stride, __nv_bfloat16* __restrict__ out, long long out_stride,
                                  long long T, int F) {
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / fv;
    const int v = static_cast<int>(idx % fv);
    float g[8], u[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(gate + t * in_stride)[v], g);
    unpack8(reinterpret_cast<const uint4*>(up + t * in_stride)[v], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    reinterpret_cast<uint4*>(out + t * out_stride)[v] = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, long long dout_stride,
                                  const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                  long long in_stride, __nv_bfloat16* __restrict__ dgate,
                                  __nv_bfloat16* __restrict__ dup, long long dstride, long long T, int F) {
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / fv;
    const int v = static_cast<int>(idx % fv);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(reinterpret_cast<const uint4*>(gate + t * in_stride)[v], g);
    unpack8(reinterpret_cast<const uint4*>(up + t * in_stride)[v], u);
    unpack8(reinterpret_cast<const uint4*>(dout + t * dout_stride)[v], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-g[i]));
      const float silu = g[i] * sg;
      du[i] = d[i] * silu;
      dg[i] = d[i] * u[i] * sg * (1.f + g[i] * (1.f - sg));
    }
    reinterpret_cast<uint4*>(dgate + t * dstride)[v] = pack8(dg);
    reinterpret_cast<uint4*>(dup + t * dstride)[v] = pack8(du);
  }
}

static inline int ew_grid(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace mb

using namespace mb;

MB_API int mb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd,
                          long long rows, int H, float eps, cudaStream_t stream) {
  if (H % 8 != 0) {
    set_last_error("mb_rmsnorm_fwd: hidden size must be a multiple of 8");
    return -1;
  }
  if (rows <= 0) return 0;
  rmsnorm_fwd_kernel<<<static_cast<unsigned>(rows), kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(h_out), rstd, H,
      eps);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Number of fp32 partial rows the backward needs as scratch: `mb_rmsnorm_bwd_blocks(rows) * H` floats.
MB_API int mb_rmsnorm_bwd_blocks(long long rows) {
  long long b = static_cast<long long>(sm_count()) * 2;
  if (b > rows) b = rows;
  return static_cast<int>(b < 1 ? 1 : b);
}

MB_API int mb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dx,
                          float* dw_partial, void* dw_bf16, float* dw_f32, int accumulate_dw, long long rows, int H,
                          cudaStream_t stream) {
  if (H % 8 != 0) {
    set_last_error("mb_rmsnorm_bwd: hidden size must be a multiple of 8");
    return -1;
  }
  if (rows <= 0) return 0;
  const int blocks = mb_rmsnorm_bwd_blocks(rows);
  rmsnorm_bwd_kernel<<<blocks, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w),
      rstd, static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), dw_partial, rows, H);
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_partial, blocks, H, static_cast<__nv_bfloat16*>(dw_bf16),
                                                              dw_f32, accumulate_dw);
  count_launch(2);
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_rope(const void* src, long long src_tstride, void* dst, long long dst_tstride, long long T, int heads,
                   int D, const long long* pos, int pos_offset, int seq_len, const float* cos_t, const float* sin_t,
                   int max_pos, int interleaved, int backward, int rotate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 2 != 0) {
    set_last_error("mb_rope: head_dim must be even");
    return -1;
  }
  int* status = status_ptr();
  const long long total = T * heads * (D / 2);
  rope_kernel<<<ew_grid(total, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(src), src_tstride, static_cast<__nv_bfloat16*>(dst), dst_tstride, T, heads, D,
      pos, pos_offset, seq_len > 0 ? seq_len : 1, cos_t, sin_t, max_pos, interleaved, backward ? -1.f : 1.f, rotate,
      status);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_swiglu_fwd(const void* gate, const void* up, long long in_stride, void* out, long long out_stride,
                         long long T, int F, cudaStream_t stream) {
  if (F % 8 != 0 || in_stride % 8 != 0 || out_stride % 8 != 0) {
    set_last_error("mb_swiglu_fwd: F and strides must be multiples of 8");
    return -1;
  }
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), in_stride,
      static_cast<__nv_bfloat16*>(out), out_stride, T, F);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MB_API int mb_swiglu_bwd(const void* dout, long long dout_stride, const void* gate, const void* up, long long in_stride,
                         void* dgate, void* dup, long long dstride, long long T, int F, cudaStream_t stream) {
  if (F % 8 != 0 || in_stride % 8 != 0 || dout_stride % 8 != 0 || dstride % 8 != 0) {
    set_last_error("mb_swiglu_bwd: F and strides must be multiples of 8");
    return -1;
  }
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dout), dout_stride, static_cast<const __nv_bfloat16*>(gate),
      static_cast<const __nv_bfloat16*>(up), in_stride, static_cast<__nv_bfloat16*>(dgate),
      static_cast<__nv_bfloat16*>(dup), dstride, T, F);
  count_launch();
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// RMSNorm backward whose partial-sum scratch is a file-scope device array instead of a caller-provided buffer, for
// hosts that must not allocate device memory around the call (see rmsnorm_bwd_static.h for limits and sharing rules).
#include "rmsnorm_bwd_static.h"

namespace mb {
static __device__ __align__(256) float g_rmsnorm_static_scratch[MB_RMSNORM_STATIC_MAX_BLOCKS * MB_RMSNORM_STATIC_MAX_H];
}

MB_API int mb_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                                 void* dx, void* dw_bf16, float* dw_f32, int accumulate_dw, long long rows, int H,
                                 cudaStream_t stream) {
  using namespace mb;
  if (H <= 0 || H % 8 != 0) {
    set_last_error("mb_rmsnorm_bwd_static: hidden size must be a positive multiple of 8");
    return -1;
  }
  if (rows <= 0) return 0;
  const int blocks = mb_rmsnorm_bwd_blocks(rows);
  if (H > MB_RMSNORM_STATIC_MAX_H || blocks > MB_RMSNORM_STATIC_MAX_BLOCKS) {
    set_last_error("mb_rmsnorm_bwd_static: problem exceeds the static scratch (H <= 8192, at most 304 row blocks)");
    return -2;
  }
  // Per-device address of the scratch array, resolved on the first call on that device.
  static float* scratch_of_device[64] = {nullptr};
  int dev = 0;
  MB_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_last_error("mb_rmsnorm_bwd_static: device index out of range");
    return -3;
  }
  float* scratch = scratch_of_device[dev];
  if (!scratch) {
    MB_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_rmsnorm_static_scratch));
    scratch_of_device[dev] = scratch;
  }
  rmsnorm_bwd_kernel<<<blocks, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w),
      rstd, static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), scratch, rows, H);
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(scratch, blocks, H, static_cast<__nv_bfloat16*>(dw_bf16),
                                                              dw_f32, accumulate_dw);
  count_launch(2);
  MB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
