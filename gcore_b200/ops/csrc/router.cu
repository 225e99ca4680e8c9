// Mixture-of-experts routing in one pass per token: softmax or sigmoid scores, optional selection bias, group-limited
// selection (the best `topk_group` of G expert groups by the sum of each group's two best scores), top-k, weight
// normalisation and scaling; and the matching backward from d(weights) to d(logits).
//
// One warp per token, the E scores of a token live in registers (lane l holds experts l, l + 32, ...).  Replaces the
// chain topk / scatter / masked_fill / topk / gather / sum / div of the PyTorch formulation (the semantics of the
// reference's routers: softmax top-k with renormalisation for the Qwen MoE families, sigmoid + bias + node-limited
// groups for the DeepSeek families, gpatch_v4/models/deepseek_v4/modeling_deepseek_v4.py:1120-1219).
// Ties go to the lower expert index.
#include "host_utils.h"
#include <cfloat>
#include <stdint.h>

namespace gkr {

constexpr int MAX_K = 16;
constexpr int MAX_G = 8;

struct RouterParams {
  const float* logits;      // [T, E]
  const float* bias;        // [E] or null (selection only)
  const long long* replay;  // [T, K] or null: forced expert ids
  long long* idx;           // [T, K]
  float* w;                 // [T, K]
  long long T;
  int E, K, G, topk_group;
  int sigmoid, norm;
  float scale;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

template <int VPT>
__global__ void __launch_bounds__(256) router_fwd_kernel(RouterParams p) {
  const long long t = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= p.T) return;
  const float* row = p.logits + t * p.E;
  float sc[VPT], sel[VPT];
  // ---- scores
  if (p.sigmoid) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) sc[i] = 1.f / (1.f + __expf(-row[lane + 32 * i]));
  } else {
    float m = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < VPT; ++i) { sc[i] = row[lane + 32 * i]; m = fmaxf(m, sc[i]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) { sc[i] = __expf(sc[i] - m); s += sc[i]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < VPT; ++i) sc[i] *= inv;
  }
  long long* out_idx = p.idx + t * p.K;
  float* out_w = p.w + t * p.K;
  float chosen_w[MAX_K];
  int chosen_i[MAX_K];
  if (p.replay) {
#pragma unroll
    for (int k = 0; k < MAX_K; ++k) {
      if (k >= p.K) break;
      const int e = static_cast<int>(p.replay[t * p.K + k]);
      float v = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        if (lane + 32 * i == e) v = sc[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      chosen_w[k] = v;
      chosen_i[k] = e;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) sel[i] = sc[i] + (p.bias ? p.bias[lane + 32 * i] : 0.f);
    if (p.G > 1) {
      // group score = sum of the two best selection scores inside the group
      const int gs = p.E / p.G;
      float gscore[MAX_G];
#pragma unroll
      for (int g = 0; g < MAX_G; ++g) {
        if (g >= p.G) break;
        float a = -FLT_MAX, b = -FLT_MAX;  // a >= b
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          if ((lane + 32 * i) / gs == g) {
            const float v = sel[i];
            if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
          const float na = fmaxf(a, oa);
          const float nb = fmaxf(fminf(a, oa), fmaxf(b, ob));
          a = na; b = nb;
        }
        gscore[g] = a + b;
      }
#pragma unroll
      for (int g = 0; g < MAX_G; ++g) {
        if (g >= p.G) break;
        int rank = 0;
#pragma unroll
        for (int h = 0; h < MAX_G; ++h)
          if (h < p.G) rank += (gscore[h] > gscore[g] || (gscore[h] == gscore[g] && h < g)) ? 1 : 0;
        if (rank >= p.topk_group) {
#pragma unroll
          for (int i = 0; i < VPT; ++i)
            if ((lane + 32 * i) / gs == g) sel[i] = -FLT_MAX;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < MAX_K; ++k) {
      if (k >= p.K) break;
      float bv = -FLT_MAX;
      int bi = 1 << 30;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        // strict > keeps the lowest index among a lane's equal values (indices grow with i)
        if (sel[i] > bv) { bv = sel[i]; bi = lane + 32 * i; }
      }
      if (bv == -FLT_MAX) bi = 1 << 30;
      float v = bv;
      int e = bi;
      warp_argmax(v, e);
      if (e >= p.E) e = k < p.E ? k : 0;  // fewer selectable experts than K: cannot happen with valid configurations
      float cw = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        if (lane + 32 * i == e) { cw = sc[i]; sel[i] = -FLT_MAX; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cw += __shfl_xor_sync(0xffffffffu, cw, o);
      chosen_w[k] = cw;
      chosen_i[k] = e;
    }
  }
  float denom = 1.f;
  if (p.norm) {
    denom = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_K; ++k)
      if (k < p.K) denom += chosen_w[k];
    denom = fmaxf(denom, 1e-20f);
  }
  if (lane < p.K) {
    // every lane holds all K results; lane k writes entry k
    float wv = 0.f;
    int iv = 0;
#pragma unroll
    for (int k = 0; k < MAX_K; ++k)
      if (k == lane) { wv = chosen_w[k]; iv = chosen_i[k]; }
    out_idx[lane] = iv;
    out_w[lane] = wv / denom * p.scale;
  }
}

struct RouterBwdParams {
  const float* logits;     // [T, E]
  const long long* idx;    // [T, K]
  const float* dw;         // [T, K]
  float* dlogits;          // [T, E]
  long long T;
  int E, K, sigmoid, norm;
  float scale;
};

template <int VPT>
__global__ void __launch_bounds__(256) router_bwd_kernel(RouterBwdParams p) {
  const long long t = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= p.T) return;
  const float* row = p.logits + t * p.E;
  float sc[VPT], g[VPT];
  if (p.sigmoid) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) sc[i] = 1.f / (1.f + __expf(-row[lane + 32 * i]));
  } else {
    float m = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < VPT; ++i) { sc[i] = row[lane + 32 * i]; m = fmaxf(m, sc[i]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) { sc[i] = __expf(sc[i] - m); s += sc[i]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < VPT; ++i) sc[i] *= inv;
  }
  // gradient w.r.t. the selected scores: w_k = scale * s_k / S (S = sum of selected scores, or 1 without normalisation)
#pragma unroll
  for (int i = 0; i < VPT; ++i) g[i] = 0.f;
  float S = 0.f, dot = 0.f;  // S = sum_k s_k,  dot = sum_k dw_k s_k
  for (int k = 0; k < p.K; ++k) {
    const int e = static_cast<int>(p.idx[t * p.K + k]);
    const float d = p.dw[t * p.K + k];
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (lane + 32 * i == e) { v = sc[i]; g[i] += d; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    S += v;
    dot += d * v;
  }
  if (p.norm) {
    S = fmaxf(S, 1e-20f);
    const float c = p.scale / S, shift = dot / S;
    for (int k = 0; k < p.K; ++k) {
      const int e = static_cast<int>(p.idx[t * p.K + k]);
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        if (lane + 32 * i == e) g[i] -= shift;  // once per occurrence of the expert in the list
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) g[i] *= c;
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) g[i] *= p.scale;
  }
  float* out = p.dlogits + t * p.E;
  if (p.sigmoid) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) out[lane + 32 * i] = g[i] * sc[i] * (1.f - sc[i]);
  } else {
    float gp = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) gp += g[i] * sc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gp += __shfl_xor_sync(0xffffffffu, gp, o);
#pragma unroll
    for (int i = 0; i < VPT; ++i) out[lane + 32 * i] = sc[i] * (g[i] - gp);
  }
}

template <typename P, typename F>
int dispatch_vpt(int E, const P& p, F launch) {
  switch (E / 32) {
    case 1: return launch(std::integral_constant<int, 1>{});
    case 2: return launch(std::integral_constant<int, 2>{});
    case 4: return launch(std::integral_constant<int, 4>{});
    case 8: return launch(std::integral_constant<int, 8>{});
    case 16: return launch(std::integral_constant<int, 16>{});
    default: return -2;
  }
}

}  // namespace gkr

using namespace gkr;

// E in {32, 64, 128, 256, 512}; K <= 16; G <= 8 and E % G == 0.  Returns -2 for an expert count without a kernel.
GK_EXPORT int gk_router_fwd(const float* logits, const float* bias, const long long* replay, long long* idx, float* w,
                            long long T, int E, int K, int G, int topk_group, int sigmoid, int norm, float scale,
                            void* stream) {
  if (T <= 0) return 0;
  if (E % 32 || K < 1 || K > MAX_K || K > E || G < 1 || G > MAX_G || E % G || (G > 1 && (topk_group < 1 || topk_group > G)))
    return -1;
  RouterParams p;
  p.logits = logits; p.bias = bias; p.replay = replay; p.idx = idx; p.w = w; p.T = T; p.E = E; p.K = K; p.G = G;
  p.topk_group = topk_group; p.sigmoid = sigmoid; p.norm = norm; p.scale = scale;
  const unsigned blocks = static_cast<unsigned>((T + 7) / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_vpt(E, p, [&](auto v) {
    router_fwd_kernel<decltype(v)::value><<<blocks, 256, 0, st>>>(p);
    return gk::launch_status();
  });
}

GK_EXPORT int gk_router_bwd(const float* logits, const long long* idx, const float* dw, float* dlogits, long long T,
                            int E, int K, int sigmoid, int norm, float scale, void* stream) {
  if (T <= 0) return 0;
  if (E % 32 || K < 1 || K > MAX_K) return -1;
  RouterBwdParams p;
  p.logits = logits; p.idx = idx; p.dw = dw; p.dlogits = dlogits; p.T = T; p.E = E; p.K = K; p.sigmoid = sigmoid;
  p.norm = norm; p.scale = scale;
  const unsigned blocks = static_cast<unsigned>((T + 7) / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_vpt(E, p, [&](auto v) {
    router_bwd_kernel<decltype(v)::value><<<blocks, 256, 0, st>>>(p);
    return gk::launch_status();
  });
}
