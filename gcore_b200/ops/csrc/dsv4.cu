// Kernels of the DeepSeek-V4-class attention stack: lightning-indexer scores (forward, and backward on the selected
// entries), top-k sparse multi-query attention with a shared key/value row and per-head sink (forward / backward), and
// the Walsh-Hadamard rotation of activations.  They replace the reference's TileLang kernels
// (gpatch_v4/models/deepseek_v4/kernel/tilelang_indexer_fwd.py:21-240, tilelang_indexer_bwd.py:21-143,
// tilelang_sparse_mla_fwd.py:25-155, tilelang_sparse_mla_bwd.py:19-267) and the library Hadamard transform
// (kernel/hadamard_transform.py:9-19).
//
// These are gather-bound kernels (every query reads its own set of key rows), written on CUDA cores with warp
// reductions: one warp per (query, head) for the attention, one thread per key for the indexer.  fp32 accumulation
// everywhere; the scatter of key gradients uses fp32 atomics (as the reference's backward does).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "host_utils.h"

namespace gkd {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float bf(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

// ---------------------------------------------------------------------------------------------- indexer forward
// score[t, s] = sum_h w[t, h] * relu(q[t, h, :] . k[s, :]) * scale   for ks[t] <= s < ke[t], else -inf
// q [S, H, D] bf16, k [T, D] bf16, w [S, H] fp32; D <= 256, H <= 128.
__global__ void indexer_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                   const float* __restrict__ w, const int* __restrict__ ks,
                                   const int* __restrict__ ke, float* __restrict__ out, int S, int T, int H, int D,
                                   float scale) {
  extern __shared__ uint8_t smem[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem);          // [H, D]
  float* sw = reinterpret_cast<float*>(smem + static_cast<size_t>(H) * D * 2);  // [H]
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) sq[i] = q[static_cast<long long>(t) * H * D + i];
  for (int i = threadIdx.x; i < H; i += blockDim.x) sw[i] = w[static_cast<long long>(t) * H + i];
  __syncthreads();
  const int lo = ks[t], hi = ke[t];
  for (int s = blockIdx.y * blockDim.x + threadIdx.x; s < T; s += gridDim.y * blockDim.x) {
    float r = -INFINITY;
    if (s >= lo && s < hi) {
      float acc = 0.f;
      const __nv_bfloat16* kr = k + static_cast<long long>(s) * D;
      for (int h = 0; h < H; ++h) {
        float dot = 0.f;
        const __nv_bfloat16* qr = sq + h * D;
        for (int d = 0; d < D; d += 2) {
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qr + d));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kr + d));
          dot += a.x * b.x + a.y * b.y;
        }
        acc += sw[h] * fmaxf(dot, 0.f);
      }
      r = acc * scale;
    }
    out[static_cast<long long>(t) * T + s] = r;
  }
}

// ---------------------------------------------------------------------------------------------- indexer backward
// Gradient through the selected entries only: ds [S, K] for indices idx [S, K] (-1 = none).
//   dq[t, h, :] += g * k[j, :],  dk[j, :] += g * q[t, h, :],  g = ds * scale * w[t, h] * (dot > 0)
//   dw[t, h]    += ds * scale * relu(dot)
// One block per query; dq is accumulated in shared memory, dk through fp32 atomics.
__global__ void indexer_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                   const float* __restrict__ w, const int* __restrict__ idx,
                                   const float* __restrict__ ds, float* __restrict__ dq, float* __restrict__ dk,
                                   float* __restrict__ dw, int S, int T, int H, int D, int K, float scale) {
  extern __shared__ uint8_t smem[];
  float* sdq = reinterpret_cast<float*>(smem);                                   // [H, D]
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(sdq + static_cast<size_t>(H) * D);  // [H, D]
  __nv_bfloat16* sk = sq + static_cast<size_t>(H) * D;                                     // [D]
  float* sg = reinterpret_cast<float*>(sk + D);                                            // [H]
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
    sq[i] = q[static_cast<long long>(t) * H * D + i];
    sdq[i] = 0.f;
  }
  __syncthreads();
  float dw_acc = 0.f;  // thread h < H owns head h
  for (int j = 0; j < K; ++j) {
    const int row = idx[static_cast<long long>(t) * K + j];
    if (row < 0 || row >= T) continue;  // uniform across the block
    const float g0 = ds[static_cast<long long>(t) * K + j] * scale;
    for (int d = threadIdx.x; d < D; d += blockDim.x) sk[d] = k[static_cast<long long>(row) * D + d];
    __syncthreads();
    if (threadIdx.x < H) {
      const int h = threadIdx.x;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot += __bfloat162float(sq[h * D + d]) * __bfloat162float(sk[d]);
      dw_acc += g0 * fmaxf(dot, 0.f);
      sg[h] = dot > 0.f ? g0 * w[static_cast<long long>(t) * H + h] : 0.f;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const float kd = __bfloat162float(sk[d]);
      float acc = 0.f;
      for (int h = 0; h < H; ++h) {
        const float g = sg[h];
        sdq[h * D + d] += g * kd;
        acc += g * __bfloat162float(sq[h * D + d]);
      }
      atomicAdd(dk + static_cast<long long>(row) * D + d, acc);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) dq[static_cast<long long>(t) * H * D + i] = sdq[i];
  if (threadIdx.x < H) dw[static_cast<long long>(t) * H + threadIdx.x] = dw_acc;
}

// ---------------------------------------------------------------------------------------------- sparse MQA forward
// out[t, h, :] = sum_j p[j] kv[idx[t, j], :],  p = softmax over {scale * q[t, h] . kv[idx[t, j]]} U {sink[h]}
// (the sink only enters the denominator).  One warp per (t, h); lane l owns elements l, l + 32, ... of the rows.
template <int EPL>  // elements per lane = D / 32
__global__ void sparse_mqa_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                                      const float* __restrict__ sinks, const int* __restrict__ idx,
                                      __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int S, int T, int H,
                                      int K, float scale) {
  const int warps = blockDim.x >> 5, wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * warps + wid;
  if (h >= H) return;
  const int D = EPL * 32;
  float qv[EPL], acc[EPL];
  const __nv_bfloat16* qr = q + (static_cast<long long>(t) * H + h) * D;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    qv[e] = bf(qr, lane + 32 * e) * scale;
    acc[e] = 0.f;
  }
  float m = sinks ? sinks[h] : -INFINITY, l = sinks ? 1.f : 0.f;  // the sink is a key with an all-zero value row
  for (int j = 0; j < K; ++j) {
    const int row = idx[static_cast<long long>(t) * K + j];
    if (row < 0 || row >= T) continue;
    const __nv_bfloat16* kr = kv + static_cast<long long>(row) * D;
    float kvv[EPL], dot = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kvv[e] = bf(kr, lane + 32 * e);
      dot += qv[e] * kvv[e];
    }
    dot = warp_sum(dot);
    const float mn = fmaxf(m, dot);
    const float c = __expf(m - mn), p = __expf(dot - mn);
    l = l * c + p;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * c + p * kvv[e];
    m = mn;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* orow = out + (static_cast<long long>(t) * H + h) * D;
#pragma unroll
  for (int e = 0; e < EPL; ++e) orow[lane + 32 * e] = __float2bfloat16(acc[e] * inv);
  if (lane == 0) lse[static_cast<long long>(t) * H + h] = l > 0.f ? m + __logf(l) : -INFINITY;
}

// ---------------------------------------------------------------------------------------------- sparse MQA backward
// p_j = exp(s_j - lse), delta = do . out, ds_j = p_j (do . kv_j - delta)
//   dq[t, h]  = scale * sum_j ds_j kv_j
//   dkv[row] += scale * ds_j q[t, h] + p_j do[t, h]        (keys and values are the same rows)
//   dsink[h] += -exp(sink - lse) * delta
template <int EPL>
__global__ void sparse_mqa_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                                      const float* __restrict__ sinks, const int* __restrict__ idx,
                                      const __nv_bfloat16* __restrict__ out, const float* __restrict__ lse,
                                      const __nv_bfloat16* __restrict__ dout, float* __restrict__ dq,
                                      float* __restrict__ dkv, float* __restrict__ dsinks, int S, int T, int H, int K,
                                      float scale) {
  const int warps = blockDim.x >> 5, wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * warps + wid;
  if (h >= H) return;
  const int D = EPL * 32;
  const long long base = (static_cast<long long>(t) * H + h) * D;
  float qv[EPL], dov[EPL], dqv[EPL];
  float delta = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    qv[e] = bf(q, base + lane + 32 * e);
    dov[e] = bf(dout, base + lane + 32 * e);
    delta += dov[e] * bf(out, base + lane + 32 * e);
    dqv[e] = 0.f;
  }
  delta = warp_sum(delta);
  const float L = lse[static_cast<long long>(t) * H + h];
  if (L == -INFINITY) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) dq[base + lane + 32 * e] = 0.f;
    return;
  }
  for (int j = 0; j < K; ++j) {
    const int row = idx[static_cast<long long>(t) * K + j];
    if (row < 0 || row >= T) continue;
    const __nv_bfloat16* kr = kv + static_cast<long long>(row) * D;
    float kvv[EPL], s = 0.f, dp = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kvv[e] = bf(kr, lane + 32 * e);
      s += qv[e] * kvv[e];
      dp += dov[e] * kvv[e];
    }
    s = warp_sum(s) * scale;
    dp = warp_sum(dp);
    const float p = __expf(s - L);
    const float dsj = p * (dp - delta);
    float* dk = dkv + static_cast<long long>(row) * D;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      dqv[e] += dsj * kvv[e];
      atomicAdd(dk + lane + 32 * e, scale * dsj * qv[e] + p * dov[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) dq[base + lane + 32 * e] = dqv[e] * scale;
  if (sinks && lane == 0) atomicAdd(dsinks + h, -__expf(sinks[h] - L) * delta);
}

// ---------------------------------------------------------------------------------------------- Hadamard rotation
// y = H_n x / sqrt(n) along the last dimension (n a power of two <= 4096); one block per row, butterflies in shared
// memory.  The transform is its own inverse, so the same kernel serves the backward pass.
__global__ void hadamard_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int n,
                                float scale) {
  extern __shared__ float sh[];
  const long long row = blockIdx.x;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sh[i] = __bfloat162float(x[row * n + i]);
  __syncthreads();
  for (int len = 1; len < n; len <<= 1) {
    for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
      const int a = (i / len) * (2 * len) + (i % len), b = a + len;
      const float u = sh[a], v = sh[b];
      sh[a] = u + v;
      sh[b] = u - v;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) y[row * n + i] = __float2bfloat16(sh[i] * scale);
}

}  // namespace gkd

using namespace gkd;

GK_EXPORT int gk_dsv4_indexer_fwd(const void* q, const void* k, const float* w, const int* ks, const int* ke,
                                  float* out, int S, int T, int H, int D, float scale, void* stream) {
  if (S <= 0 || T <= 0) return 0;
  if (D % 2 || D > 256 || H > 128) return -1;
  const size_t smem = static_cast<size_t>(H) * D * 2 + H * 4;
  static bool cfg = false;
  if (!cfg) {
    cudaFuncSetAttribute(indexer_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 256 * 2 + 512);
    cfg = true;
  }
  int gy = (T + 127) / 128;
  if (gy > 64) gy = 64;
  indexer_fwd_kernel<<<dim3(S, gy), 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k), w, ks, ke, out, S, T, H, D,
      scale);
  return gk::launch_status();
}

// dq [S, H, D], dk [T, D] (must be zeroed by the caller), dw [S, H]: fp32.
GK_EXPORT int gk_dsv4_indexer_bwd(const void* q, const void* k, const float* w, const int* idx, const float* ds,
                                  float* dq, float* dk, float* dw, int S, int T, int H, int D, int K, float scale,
                                  void* stream) {
  if (S <= 0) return 0;
  if (D > 256 || H > 128) return -1;
  const size_t smem = static_cast<size_t>(H) * D * 4 + static_cast<size_t>(H) * D * 2 + D * 2 + H * 4;
  static bool cfg = false;
  if (!cfg) {
    cudaFuncSetAttribute(indexer_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cfg = true;
  }
  if (smem > 200 * 1024) return -2;
  indexer_bwd_kernel<<<S, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k), w, idx, ds, dq, dk, dw, S, T,
      H, D, K, scale);
  return gk::launch_status();
}

#define GK_SPARSE_DISPATCH(KERNEL, ...)                                                        \
  switch (D / 32) {                                                                            \
    case 1: KERNEL<1><<<grid, 128, 0, st>>>(__VA_ARGS__); break;                               \
    case 2: KERNEL<2><<<grid, 128, 0, st>>>(__VA_ARGS__); break;                               \
    case 4: KERNEL<4><<<grid, 128, 0, st>>>(__VA_ARGS__); break;                               \
    case 8: KERNEL<8><<<grid, 128, 0, st>>>(__VA_ARGS__); break;                               \
    case 16: KERNEL<16><<<grid, 128, 0, st>>>(__VA_ARGS__); break;                             \
    default: return -1;                                                                        \
  }

// q [S, H, D], kv [T, D] bf16; sinks [H] fp32 or null; idx [S, K] int32 (-1 = none); D in {32, 64, 128, 256, 512}.
GK_EXPORT int gk_dsv4_sparse_mqa_fwd(const void* q, const void* kv, const float* sinks, const int* idx, void* out,
                                     float* lse, int S, int T, int H, int D, int K, float scale, void* stream) {
  if (S <= 0 || H <= 0) return 0;
  if (D % 32) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(S, (H + 3) / 4);
  GK_SPARSE_DISPATCH(sparse_mqa_fwd_kernel, reinterpret_cast<const __nv_bfloat16*>(q),
                     reinterpret_cast<const __nv_bfloat16*>(kv), sinks, idx, reinterpret_cast<__nv_bfloat16*>(out), lse,
                     S, T, H, K, scale)
  return gk::launch_status();
}

// dq [S, H, D] fp32 (written), dkv [T, D] fp32 and dsinks [H] fp32 (accumulated: zero them first).
GK_EXPORT int gk_dsv4_sparse_mqa_bwd(const void* q, const void* kv, const float* sinks, const int* idx,
                                     const void* out, const float* lse, const void* dout, float* dq, float* dkv,
                                     float* dsinks, int S, int T, int H, int D, int K, float scale, void* stream) {
  if (S <= 0 || H <= 0) return 0;
  if (D % 32) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(S, (H + 3) / 4);
  GK_SPARSE_DISPATCH(sparse_mqa_bwd_kernel, reinterpret_cast<const __nv_bfloat16*>(q),
                     reinterpret_cast<const __nv_bfloat16*>(kv), sinks, idx,
                     reinterpret_cast<const __nv_bfloat16*>(out), lse, reinterpret_cast<const __nv_bfloat16*>(dout), dq,
                     dkv, dsinks, S, T, H, K, scale)
  return gk::launch_status();
}

GK_EXPORT int gk_hadamard(const void* x, void* y, long long rows, int n, void* stream) {
  if (rows <= 0) return 0;
  if (n < 2 || n > 4096 || (n & (n - 1))) return -1;
  const int threads = n / 2 < 256 ? (n / 2 < 32 ? 32 : n / 2) : 256;
  hadamard_kernel<<<static_cast<unsigned>(rows), threads, n * 4, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y), n, rsqrtf(static_cast<float>(n)));
  return gk::launch_status();
}
