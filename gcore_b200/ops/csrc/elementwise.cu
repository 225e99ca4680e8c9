// Bandwidth-bound kernels of the transformer block and the optimizer: RMSNorm (+residual) fwd/bwd, RoPE
// fwd/bwd, SwiGLU fwd/bwd, fused Adam on the distributed-optimizer shard, squared-L2 norm, casts.
// All use 128-bit accesses; H, D and F must be multiples of 8.
//
// These stand in for the TransformerEngine / apex fused ops the reference reaches through Megatron-Core
// (gpatch_v4/training_backend/megatron_backend/mixin.py:311-348, optimizer.py:53-111).
#include "host_utils.h"
#include <cuda_bf16.h>

namespace gk {

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ void unpack8(const bf16x8& a, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(a.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 a;
#pragma unroll
  for (int i = 0; i < 4; ++i) a.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return a;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffff, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffff, v, o));
  return v;
}
// Block-wide sum; `red` must hold 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------------------------------ RMSNorm
// y = (x [+ res]) * rstd * w ; optionally writes the summed residual stream to res_out.
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ res,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y,
                                                          __nv_bfloat16* __restrict__ res_out,
                                                          float* __restrict__ rstd_out, int T, int H, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int nv = H >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + static_cast<size_t>(row) * H);
    const bf16x8* rr = res ? reinterpret_cast<const bf16x8*>(res + static_cast<size_t>(row) * H) : nullptr;
    bf16x8* ro = res_out ? reinterpret_cast<bf16x8*>(res_out + static_cast<size_t>(row) * H) : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float f[8];
      unpack8(xr[i], f);
      if (rr) {
        float g[8];
        unpack8(rr[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        const bf16x8 s = pack8(f);
        if (ro) ro[i] = s;
        unpack8(s, f);  // normalise what the residual stream actually stores
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    const bf16x8* src = (rr && ro) ? reinterpret_cast<const bf16x8*>(ro) : xr;
    bf16x8* yr = reinterpret_cast<bf16x8*>(y + static_cast<size_t>(row) * H);
    const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float f[8], g[8];
      if (rr && !ro) {
        float a[8], b[8];
        unpack8(xr[i], a);
        unpack8(rr[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += b[j];
        unpack8(pack8(a), f);
      } else {
        unpack8(src[i], f);
      }
      unpack8(wv[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
      yr[i] = pack8(f);
    }
  }
}

// dx = rstd * (g*w - x * rstd^2 * mean(g*w*x)) [+ dres] ; partial dw per CTA (reduced by a second kernel).
constexpr int RMS_SLOTS = 4;  // H <= 256 * 8 * 4 = 8192
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ g,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const float* __restrict__ rstd,
                                                          const __nv_bfloat16* __restrict__ dres,
                                                          __nv_bfloat16* __restrict__ dx,
                                                          float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  const int nv = H >> 3;
  float dw[RMS_SLOTS][8];
#pragma unroll
  for (int s = 0; s < RMS_SLOTS; ++s)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[s][j] = 0.f;
  const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(g + static_cast<size_t>(row) * H);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + static_cast<size_t>(row) * H);
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int s = 0; s < RMS_SLOTS; ++s) {
      const int i = threadIdx.x + s * 256;
      if (i < nv) {
        float gf[8], xf[8], wf[8];
        unpack8(gr[i], gf);
        unpack8(xr[i], xf);
        unpack8(wv[i], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += gf[j] * wf[j] * xf[j];
          dw[s][j] += gf[j] * xf[j] * rs;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rs * rs / H;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + static_cast<size_t>(row) * H);
    const bf16x8* dr = dres ? reinterpret_cast<const bf16x8*>(dres + static_cast<size_t>(row) * H) : nullptr;
#pragma unroll
    for (int s = 0; s < RMS_SLOTS; ++s) {
      const int i = threadIdx.x + s * 256;
      if (i < nv) {
        float gf[8], xf[8], wf[8], o[8];
        unpack8(gr[i], gf);
        unpack8(xr[i], xf);
        unpack8(wv[i], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (gf[j] * wf[j] - xf[j] * c);
        if (dr) {
          float d[8];
          unpack8(dr[i], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += d[j];
        }
        dxr[i] = pack8(o);
      }
    }
  }
  float* out = dw_partial + static_cast<size_t>(blockIdx.x) * H;
#pragma unroll
  for (int s = 0; s < RMS_SLOTS; ++s) {
    const int i = threadIdx.x + s * 256;
    if (i < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[i * 8 + j] = dw[s][j];
    }
  }
}

__global__ void colsum_partial_kernel(const float* __restrict__ partial, float* __restrict__ out, int nparts, int H,
                                      int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= H) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<size_t>(p) * H + i];
  out[i] = accumulate ? out[i] + s : s;
}

// ------------------------------------------------------------------------------------------ RoPE
// In-place rotation of the first `rot` dims of every head (rotate-half / "neox" pairing: i <-> i + rot/2).
// x is [T, nheads, D] with token stride `stride_t` elements (so it can be a slice of a packed QKV buffer).
// sign = +1 forward, -1 backward (the transpose of a rotation is the rotation by the negated angle).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, int T, int nheads, int D,
                            int rot, long long stride_t, float theta, float sign, int interleaved) {
  const int half = rot >> 1;
  const long long total = static_cast<long long>(T) * nheads * half;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % half);
    const long long th = idx / half;
    const int h = static_cast<int>(th % nheads);
    const int t = static_cast<int>(th / nheads);
    const float inv = __powf(theta, -2.f * i / rot);
    float s, c;
    sincosf(pos[t] * inv, &s, &c);
    s *= sign;
    __nv_bfloat16* p = x + t * stride_t + static_cast<long long>(h) * D;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(p[i0]), b = __bfloat162float(p[i1]);
    p[i0] = __float2bfloat16(a * c - b * s);
    p[i1] = __float2bfloat16(b * c + a * s);
  }
}

// Same rotation with the angles given as tables cos / sin [T, rot / 2] (multi-axis rotary position ids of
// vision-language models: every frequency takes its angle from the temporal, height or width index of the token).
__global__ void rope_table_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs,
                                  const float* __restrict__ sn, int T, int nheads, int D, int rot, long long stride_t,
                                  float sign, int interleaved) {
  const int half = rot >> 1;
  const long long total = static_cast<long long>(T) * nheads * half;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % half);
    const long long th = idx / half;
    const int h = static_cast<int>(th % nheads);
    const int t = static_cast<int>(th / nheads);
    const float c = cs[static_cast<long long>(t) * half + i];
    const float s = sn[static_cast<long long>(t) * half + i] * sign;
    __nv_bfloat16* p = x + t * stride_t + static_cast<long long>(h) * D;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(p[i0]), b = __bfloat162float(p[i1]);
    p[i0] = __float2bfloat16(a * c - b * s);
    p[i1] = __float2bfloat16(b * c + a * s);
  }
}

// ------------------------------------------------------------------------------------------ SwiGLU
// in [T, 2F] = [gate | up]; out [T, F] = silu(gate) * up
// A thread's (row, 8-wide column vector) pair advances by the grid stride without a division per element: one 64-bit
// division at entry, then carries (a division per element made the kernel issue-bound: 99 us for 9216 x 1536 outputs).
struct RowColIter {
  long long t;
  int i, di, nv;
  long long dt;
  __device__ RowColIter(int nv_) : nv(nv_) {
    const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    t = idx / nv;
    i = static_cast<int>(idx - t * nv);
    dt = step / nv;
    di = static_cast<int>(step - dt * nv);
  }
  __device__ void next() {
    t += dt;
    i += di;
    if (i >= nv) { i -= nv; ++t; }
  }
};

// n_rows (device, optional): rows at or beyond *n_rows are left untouched (expert-sorted buffers sized for the worst
// case carry a device-side count of the rows in use).
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long T,
                                  int F, const int* __restrict__ n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int nv = F >> 3;
  if (n_rows && *n_rows < T) T = *n_rows;
  for (RowColIter it(nv); it.t < T; it.next()) {
    const long long t = it.t;
    const int i = it.i;
    const bf16x8* row = reinterpret_cast<const bf16x8*>(in + t * 2 * F);
    float g[8], u[8];
    unpack8(row[i], g);
    unpack8(row[nv + i], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<bf16x8*>(out + t * F)[i] = pack8(g);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ in,
                                  __nv_bfloat16* __restrict__ din, long long T, int F) {
  const int nv = F >> 3;
  for (RowColIter it(nv); it.t < T; it.next()) {
    const long long t = it.t;
    const int i = it.i;
    const bf16x8* row = reinterpret_cast<const bf16x8*>(in + t * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[i], g);
    unpack8(row[nv + i], u);
    unpack8(reinterpret_cast<const bf16x8*>(dout + t * F)[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
    }
    bf16x8* orow = reinterpret_cast<bf16x8*>(din + t * 2 * F);
    orow[i] = pack8(dg);
    orow[nv + i] = pack8(du);
  }
}

// ------------------------------------------------------------------------------------------ Adam
// One pass over the optimizer shard: unscale/clip the gradient, AdamW on the fp32 master, write the bf16
// parameter.  `scale_ptr` (device) holds the combined gradient multiplier (1/loss-scale * clip coefficient) so
// the clip coefficient never visits the host.
__global__ void adam_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                            const void* __restrict__ grad, int grad_fp32, __nv_bfloat16* __restrict__ param,
                            long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                            const float* __restrict__ scale_ptr, float scale_val) {
  const float scale = (scale_ptr ? *scale_ptr : 1.f) * scale_val;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = (grad_fp32 ? reinterpret_cast<const float*>(grad)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i])) * scale;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float p = master[i];
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * p;
    p -= lr * upd;
    master[i] = p;
    if (param) param[i] = __float2bfloat16(p);
  }
}

__global__ void __launch_bounds__(256) sumsq_kernel(const void* __restrict__ x, int is_fp32, long long n,
                                                    float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = is_fp32 ? reinterpret_cast<const float*>(x)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// dst(bf16 or fp32) (+)= scale * src
__global__ void axpy_cast_kernel(const void* __restrict__ src, int src_fp32, void* __restrict__ dst, int dst_fp32,
                                 long long n, float scale, int accumulate) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f = (src_fp32 ? reinterpret_cast<const float*>(src)[i]
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i])) * scale;
    if (dst_fp32) {
      float* d = reinterpret_cast<float*>(dst);
      d[i] = accumulate ? d[i] + f : f;
    } else {
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst);
      d[i] = __float2bfloat16(accumulate ? __bfloat162float(d[i]) + f : f);
    }
  }
}

inline int grid_for(long long work_items, int threads, int waves = 8) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * waves;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace gk

using namespace gk;

GK_EXPORT int gk_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd,
                             int T, int H, float eps, void* stream) {
  if (H % 8) return -1;
  const int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  launch_k(rmsnorm_fwd_kernel, dim3(grid > 0 ? grid : 1), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(res),
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(y),
      reinterpret_cast<__nv_bfloat16*>(res_out), rstd, T, H, eps);
  return launch_status();
}

// Per-head RMSNorm of the query and key heads of packed [q | k | v] rows, in place (decode / prefill of models with
// q / k layer norms): one warp per (token, head), D <= 256.  Replaces two norm launches over reshaped copies and the
// copies back into the packed rows.
__global__ void qk_headnorm_kernel(__nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                                   const __nv_bfloat16* __restrict__ wk, long long T, int Hq, int Hk, int D,
                                   long long stride_t, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int heads = Hq + Hk;
  const int nv = D >> 3;
  for (long long w = warp; w < T * heads; w += nwarps) {
    const long long t = w / heads;
    const int h = static_cast<int>(w - t * heads);
    bf16x8* row = reinterpret_cast<bf16x8*>(qkv + t * stride_t + static_cast<long long>(h) * D);
    const bf16x8* g = reinterpret_cast<const bf16x8*>(h < Hq ? wq : wk);
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float ss = 0.f;
    if (lane < nv) {
      unpack8(row[lane], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffff, ss, off);
    const float rstd = rsqrtf(ss / D + eps);
    if (lane < nv) {
      float gw[8];
      unpack8(g[lane], gw);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * gw[j];
      row[lane] = pack8(f);
    }
  }
}

GK_EXPORT int gk_qk_headnorm(void* qkv, const void* wq, const void* wk, long long T, int Hq, int Hk, int D,
                             long long stride_t, float eps, void* stream) {
  if (D % 8 || D > 256 || stride_t % 8) return -1;
  if (T == 0) return 0;
  launch_k(qk_headnorm_kernel, dim3(grid_for(T * (Hq + Hk) * 32, 256)), dim3(256), 0,
           reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<__nv_bfloat16*>(qkv),
           reinterpret_cast<const __nv_bfloat16*>(wq), reinterpret_cast<const __nv_bfloat16*>(wk), T, Hq, Hk, D, stride_t,
           eps);
  return launch_status();
}

GK_EXPORT int gk_rmsnorm_bwd_parts(int T) {
  const int cap = sm_count() * 2;
  return T < cap ? (T > 0 ? T : 1) : cap;
}

// dw_partial must hold gk_rmsnorm_bwd_parts(T) * H floats.
GK_EXPORT int gk_rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, const void* dres,
                             void* dx, float* dw_partial, float* dw, int dw_accumulate, int T, int H, void* stream) {
  if (H % 8 || H > 256 * 8 * RMS_SLOTS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int parts = gk_rmsnorm_bwd_parts(T);
  rmsnorm_bwd_kernel<<<parts, 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(g), reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<const __nv_bfloat16*>(dres),
      reinterpret_cast<__nv_bfloat16*>(dx), dw_partial, T, H);
  colsum_partial_kernel<<<(H + 255) / 256, 256, 0, st>>>(dw_partial, dw, parts, H, dw_accumulate);
  return launch_status();
}

GK_EXPORT int gk_rope(void* x, const int* pos, int T, int nheads, int D, int rot, long long stride_t, float theta,
                      int backward, int interleaved, void* stream) {
  if (rot % 2 || rot > D) return -1;
  const long long total = static_cast<long long>(T) * nheads * (rot / 2);
  if (total == 0) return 0;
  rope_kernel<<<grid_for(total, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(x), pos, T, nheads, D, rot, stride_t, theta, backward ? -1.f : 1.f,
      interleaved);
  return launch_status();
}

GK_EXPORT int gk_rope_table(void* x, const float* cs, const float* sn, int T, int nheads, int D, int rot,
                            long long stride_t, int backward, int interleaved, void* stream) {
  if (rot % 2 || rot > D) return -1;
  const long long total = static_cast<long long>(T) * nheads * (rot / 2);
  if (total == 0) return 0;
  rope_table_kernel<<<grid_for(total, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(x), cs, sn, T, nheads, D, rot, stride_t, backward ? -1.f : 1.f, interleaved);
  return launch_status();
}

static int swiglu_fwd_launch(const void* in, void* out, long long T, int F, const int* n_rows, void* stream) {
  if (F % 8) return -1;
  if (T == 0) return 0;
  launch_k(swiglu_fwd_kernel, dim3(grid_for(T * (F / 8), 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), T, F, n_rows);
  return launch_status();
}

GK_EXPORT int gk_swiglu_fwd(const void* in, void* out, long long T, int F, void* stream) {
  return swiglu_fwd_launch(in, out, T, F, nullptr, stream);
}

// rows at or beyond *n_rows (device) are not computed
GK_EXPORT int gk_swiglu_fwd_rows(const void* in, void* out, long long T, int F, const int* n_rows, void* stream) {
  return swiglu_fwd_launch(in, out, T, F, n_rows, stream);
}

GK_EXPORT int gk_swiglu_bwd(const void* dout, const void* in, void* din, long long T, int F, void* stream) {
  if (F % 8) return -1;
  if (T == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(in),
      reinterpret_cast<__nv_bfloat16*>(din), T, F);
  return launch_status();
}

GK_EXPORT int gk_adam(float* master, float* m, float* v, const void* grad, int grad_fp32, void* param, long long n,
                      float lr, float b1, float b2, float eps, float wd, int step, const float* scale_ptr,
                      float scale_val, void* stream) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, static_cast<float>(step));
  const float bc2 = 1.f - powf(b2, static_cast<float>(step));
  adam_kernel<<<grid_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, grad_fp32, reinterpret_cast<__nv_bfloat16*>(param), n, lr, b1, b2, eps, wd, bc1, bc2,
      scale_ptr, scale_val);
  return launch_status();
}

// out[0] += sum(x^2); the caller zeroes out[0].
GK_EXPORT int gk_sumsq(const void* x, int is_fp32, long long n, float* out, void* stream) {
  if (n == 0) return 0;
  sumsq_kernel<<<grid_for(n, 256, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, is_fp32, n, out);
  return launch_status();
}

GK_EXPORT int gk_axpy_cast(const void* src, int src_fp32, void* dst, int dst_fp32, long long n, float scale,
                           int accumulate, void* stream) {
  if (n == 0) return 0;
  axpy_cast_kernel<<<grid_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(src, src_fp32, dst,
                                                                                        dst_fp32, n, scale,
                                                                                        accumulate);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant of gk_rmsnorm_bwd (declared and documented in no_alloc.h).
#include "no_alloc.h"

namespace gk {
// Scratch for the per-CTA weight-gradient partials.  In host code this name is only a handle for the symbol: the
// device address has to be looked up (once per device) before it can be given to a kernel.
static __device__ __align__(256) float g_noalloc_rms_scratch[GK_NOALLOC_RMSNORM_MAX_PARTS * GK_NOALLOC_RMSNORM_MAX_H];
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_rms_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace gk

GK_EXPORT int gk_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, const void* dres,
                                     void* dx, float* dw, int dw_accumulate, int T, int H, void* stream) {
  if (H % 8) return -1;
  if (H > GK_NOALLOC_RMSNORM_MAX_H) {
    fprintf(stderr, "[gcore_b200] gk_rmsnorm_bwd_noalloc: H=%d exceeds the built-in scratch (max H %d)\n", H,
            GK_NOALLOC_RMSNORM_MAX_H);
    return -2;
  }
  if (T <= 0) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return -3;
  if (!g_noalloc_rms_ptr[dev]) {
    // first call on this device: resolve the device address of the file-scope array
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_rms_scratch);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "[gcore_b200] gk_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return -3;
    }
    g_noalloc_rms_ptr[dev] = p;
  }
  float* scratch = g_noalloc_rms_ptr[dev];
  int parts = gk_rmsnorm_bwd_parts(T);
  if (parts > GK_NOALLOC_RMSNORM_MAX_PARTS) parts = GK_NOALLOC_RMSNORM_MAX_PARTS;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  rmsnorm_bwd_kernel<<<parts, 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(g), reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<const __nv_bfloat16*>(dres),
      reinterpret_cast<__nv_bfloat16*>(dx), scratch, T, H);
  colsum_partial_kernel<<<(H + 255) / 256, 256, 0, st>>>(scratch, dw, parts, H, dw_accumulate);
  return launch_status();
}
