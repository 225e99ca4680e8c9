// Block-scaled low-precision quantisers (e4m3 1x128 activations, e4m3 128x128 weights, e2m1 1x32) with fp32 or
// power-of-two (ue8m0-representable) scales, plus the quantise->dequantise round trips used for QAT.
// Semantics follow the reference's TileLang kernels (gpatch_v4/kernel/quantize/qat.py:117-285,
// fused_quant_kernels.py:103-403) and their eager definitions (eager_quant_kernels.py:63-233).
#include "host_utils.h"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace gq {

constexpr float E4M3_MAX = 448.f;
constexpr float E2M1_MAX = 6.f;

__device__ __forceinline__ float pow2_ceil(float s) {
  // smallest power of two >= s (s > 0): what an e8m0 scale can represent
  int e;
  const float m = frexpf(s, &e);  // s = m * 2^e, m in [0.5, 1)
  return m == 0.5f ? ldexpf(1.f, e - 1) : ldexpf(1.f, e);
}
__device__ __forceinline__ float block_scale(float amax, float qmax, int pow2) {
  float s = fmaxf(amax, 1e-10f) / qmax;
  return pow2 ? pow2_ceil(s) : s;
}
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  __nv_fp8_e4m3 t;
  t.__x = b;
  return static_cast<float>(t);
}
// e2m1: values {0, .5, 1, 1.5, 2, 3, 4, 6} with a sign bit; round to nearest (ties to even code)
__device__ __forceinline__ uint8_t to_e2m1(float v) {
  const float a = fminf(fabsf(v), E2M1_MAX);
  uint8_t code;
  if (a <= 0.25f) code = 0;
  else if (a < 0.75f) code = 1;
  else if (a <= 1.25f) code = 2;
  else if (a < 1.75f) code = 3;
  else if (a <= 2.5f) code = 4;
  else if (a < 3.5f) code = 5;
  else if (a <= 5.f) code = 6;
  else code = 7;
  return code | (v < 0.f ? 8 : 0);
}
__device__ __forceinline__ float from_e2m1(uint8_t c) {
  const float tab[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float a = tab[c & 7];
  return (c & 8) ? -a : a;
}

// one warp per (row, 128-column block); lane holds 4 consecutive elements
__global__ void act_quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ scales, __nv_bfloat16* __restrict__ dq, long long M, int K,
                                       int pow2) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int kb = K / 128;
  if (warp >= M * kb) return;
  const long long row = warp / kb;
  const int b = static_cast<int>(warp - row * kb);
  const long long base = row * K + b * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(x[base + j]);
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, o));
  const float s = block_scale(amax, E4M3_MAX, pow2);
  const float inv = 1.f / s;
  if (lane == 0 && scales) scales[row * kb + b] = s;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint8_t c = to_e4m3(v[j] * inv);
    if (q) q[base + j] = c;
    if (dq) dq[base + j] = __float2bfloat16(from_e4m3(c) * s);
  }
}

// one CTA (256 threads) per 128x128 block
__global__ void __launch_bounds__(256) weight_quant_128x128_kernel(const __nv_bfloat16* __restrict__ w,
                                                                   uint8_t* __restrict__ q, float* __restrict__ scales,
                                                                   __nv_bfloat16* __restrict__ dq, int N, int K,
                                                                   int pow2) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int bn = blockIdx.y, bk = blockIdx.x;
  const int kblocks = (K + 127) / 128;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = bn * 128 + (i >> 7), c = bk * 128 + (i & 127);
    if (r < N && c < K) amax = fmaxf(amax, fabsf(__bfloat162float(w[static_cast<long long>(r) * K + c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, red[i]);
    s_scale = block_scale(m, E4M3_MAX, pow2);
    if (scales) scales[bn * kblocks + bk] = s_scale;
  }
  __syncthreads();
  const float s = s_scale, inv = 1.f / s_scale;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = bn * 128 + (i >> 7), c = bk * 128 + (i & 127);
    if (r < N && c < K) {
      const long long idx = static_cast<long long>(r) * K + c;
      const uint8_t code = to_e4m3(__bfloat162float(w[idx]) * inv);
      if (q) q[idx] = code;
      if (dq) dq[idx] = __float2bfloat16(from_e4m3(code) * s);
    }
  }
}

// e2m1 1x32: one thread per 32-element block; packed two codes per byte (low nibble = even element); scale is a
// power of two stored as its biased exponent (ue8m0) and as fp32
__global__ void fp4_quant_1x32_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ packed,
                                      uint8_t* __restrict__ scale_e8m0, float* __restrict__ scale_f32,
                                      __nv_bfloat16* __restrict__ dq, long long nblocks) {
  const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (b >= nblocks) return;
  const long long base = b * 32;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v[j] = __bfloat162float(x[base + j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const float s = pow2_ceil(fmaxf(amax, 1e-10f) / E2M1_MAX);
  int e;
  frexpf(s, &e);  // s = 0.5 * 2^e  ->  exponent of s is e - 1
  if (scale_e8m0) scale_e8m0[b] = static_cast<uint8_t>(min(max(e - 1 + 127, 0), 254));
  if (scale_f32) scale_f32[b] = s;
  const float inv = 1.f / s;
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const uint8_t c0 = to_e2m1(v[j] * inv), c1 = to_e2m1(v[j + 1] * inv);
    if (packed) packed[(base + j) >> 1] = c0 | (c1 << 4);
    if (dq) {
      dq[base + j] = __float2bfloat16(from_e2m1(c0) * s);
      dq[base + j + 1] = __float2bfloat16(from_e2m1(c1) * s);
    }
  }
}

}  // namespace gq

using namespace gq;

// q (uint8 e4m3 codes), scales (fp32) and dq (bf16 round trip) are each optional.
GK_EXPORT int gk_act_quant_1x128(const void* x, void* q, float* scales, void* dq, long long M, int K, int pow2,
                                 void* stream) {
  if (K % 128) return -1;
  const long long warps = M * (K / 128);
  if (warps == 0) return 0;
  const long long blocks = (warps * 32 + 255) / 256;
  act_quant_1x128_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), scales,
      reinterpret_cast<__nv_bfloat16*>(dq), M, K, pow2);
  return gk::launch_status();
}

GK_EXPORT int gk_weight_quant_128x128(const void* w, void* q, float* scales, void* dq, int N, int K, int pow2,
                                      void* stream) {
  dim3 grid((K + 127) / 128, (N + 127) / 128);
  weight_quant_128x128_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<uint8_t*>(q), scales,
      reinterpret_cast<__nv_bfloat16*>(dq), N, K, pow2);
  return gk::launch_status();
}

GK_EXPORT int gk_fp4_quant_1x32(const void* x, void* packed, void* scale_e8m0, float* scale_f32, void* dq,
                                long long numel, void* stream) {
  if (numel % 32) return -1;
  const long long nb = numel / 32;
  if (nb == 0) return 0;
  fp4_quant_1x32_kernel<<<static_cast<unsigned>((nb + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(packed),
      reinterpret_cast<uint8_t*>(scale_e8m0), scale_f32, reinterpret_cast<__nv_bfloat16*>(dq), nb);
  return gk::launch_status();
}
