// Kernels over the vocabulary axis and the RL objective:
//   * log-prob + entropy of a [T, V] logits chunk in one pass (online max / sum-exp / sum p*z), producing either
//     final values or per-rank partials for vocab-parallel TP (one small all-gather replaces the three
//     all-reduces of gpatch_v4/training_backend/vocab_parallel_entropy.py:20-29);
//   * its backward, overwriting the logits chunk with d(logits);
//   * Gumbel-max sampling with a per-request counter-based random stream, returning the sampled token's log-prob
//     (per-request seed semantics of gpatch_v4/extended_model/llm.py:57-68);
//   * the GRPO / PPO-clip token objective with k3 KL, fwd + grad in one pass
//     (gpatch_v4/training_backend/loss/ppo_loss.py:232-346, gpatch_v4/utils/ppo_utils.py:151-193);
//   * the GAE reverse scan (gpatch_v4/core/advantage_impl.py:394-444).
#include "host_utils.h"
#include <cuda_bf16.h>
#include <float.h>

namespace gk {

__device__ __forceinline__ float load_logit(const void* p, int is_fp32, long long i) {
  return is_fp32 ? reinterpret_cast<const float*>(p)[i]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// Counter-based uniform in (0, 1): splitmix64 finaliser over (seed, step, token id).  Stateless, so the draw for a
// token does not depend on which thread, CTA or tensor-parallel rank evaluates it.
__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned long long step,
                                              unsigned long long idx) {
  unsigned long long x = seed * 0x9E3779B97F4A7C15ULL + step * 0xD1B54A32D192ED03ULL + idx * 0x2545F4914F6CDD1DULL +
                         0x632BE59BD9B4E019ULL;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ULL;
  x ^= x >> 27; x *= 0x94D049BB133111EBULL;
  x ^= x >> 31;
  return (static_cast<float>(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

struct Online {
  float m, s, sz;  // running max, sum exp(z-m), sum exp(z-m)*z
};
__device__ __forceinline__ void online_add(Online& o, float z) {
  if (z > o.m) {
    const float r = __expf(o.m - z);
    o.s = o.s * r + 1.f;
    o.sz = o.sz * r + z;
    o.m = z;
  } else {
    const float e = __expf(z - o.m);
    o.s += e;
    o.sz += e * z;
  }
}
__device__ __forceinline__ void online_merge(Online& a, const Online& b) {
  if (b.m == -FLT_MAX) return;
  if (a.m == -FLT_MAX) { a = b; return; }
  const float m = fmaxf(a.m, b.m);
  const float ra = __expf(a.m - m), rb = __expf(b.m - m);
  a.s = a.s * ra + b.s * rb;
  a.sz = a.sz * ra + b.sz * rb;
  a.m = m;
}
__device__ __forceinline__ Online block_online(Online o, Online* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    Online b;
    b.m = __shfl_xor_sync(0xffffffff, o.m, off);
    b.s = __shfl_xor_sync(0xffffffff, o.s, off);
    b.sz = __shfl_xor_sync(0xffffffff, o.sz, off);
    online_merge(o, b);
  }
  __syncthreads();
  if (lane == 0) red[w] = o;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  Online t;
  t.m = -FLT_MAX; t.s = 0.f; t.sz = 0.f;
  if (lane < nw) t = red[lane];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    Online b;
    b.m = __shfl_xor_sync(0xffffffff, t.m, off);
    b.s = __shfl_xor_sync(0xffffffff, t.s, off);
    b.sz = __shfl_xor_sync(0xffffffff, t.sz, off);
    online_merge(t, b);
  }
  return t;
}

// One CTA per row.  targets are global vocabulary ids; this rank owns [vocab_start, vocab_start + V).
// partial_out != nullptr: write (max, sumexp, sum e*z, target z or -inf) and skip the final values.
__global__ void __launch_bounds__(256) logprob_entropy_fwd_kernel(const void* __restrict__ logits, int is_fp32,
                                                                  long long ld, const long long* __restrict__ targets,
                                                                  float inv_temp, int vocab_start, int V,
                                                                  float* __restrict__ logp, float* __restrict__ ent,
                                                                  float* __restrict__ lse_out,
                                                                  float* __restrict__ partial_out) {
  __shared__ Online red[32];
  const long long row = blockIdx.x;
  const long long base = row * ld;
  Online o;
  o.m = -FLT_MAX; o.s = 0.f; o.sz = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) online_add(o, load_logit(logits, is_fp32, base + j) * inv_temp);
  o = block_online(o, red);
  if (threadIdx.x == 0) {
    const long long tg = targets ? targets[row] - vocab_start : -1;
    const bool mine = tg >= 0 && tg < V;
    const float zt = mine ? load_logit(logits, is_fp32, base + tg) * inv_temp : -FLT_MAX;
    if (partial_out) {
      float* p = partial_out + row * 4;
      p[0] = o.m; p[1] = o.s; p[2] = o.sz; p[3] = zt;
    } else {
      const float lse = o.m + __logf(o.s);
      if (lse_out) lse_out[row] = lse;
      if (logp) logp[row] = mine ? zt - lse : 0.f;
      if (ent) ent[row] = lse - o.sz / o.s;
    }
  }
}

// partials [R, T, 4] (R ranks) -> logp, entropy, lse
__global__ void logprob_entropy_combine_kernel(const float* __restrict__ partials, int R, long long T,
                                               float* __restrict__ logp, float* __restrict__ ent,
                                               float* __restrict__ lse_out) {
  const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (t >= T) return;
  Online o;
  o.m = -FLT_MAX; o.s = 0.f; o.sz = 0.f;
  float zt = -FLT_MAX;
  for (int r = 0; r < R; ++r) {
    const float* p = partials + (static_cast<long long>(r) * T + t) * 4;
    Online b;
    b.m = p[0]; b.s = p[1]; b.sz = p[2];
    online_merge(o, b);
    zt = fmaxf(zt, p[3]);
  }
  const float lse = o.m + __logf(o.s);
  if (lse_out) lse_out[t] = lse;
  if (logp) logp[t] = zt - lse;
  if (ent) ent[t] = lse - o.sz / o.s;
}

// d logit_j = inv_temp * [ g_lp * (1{j==y} - p_j) - g_H * p_j * (z_j - lse + H) ], written over the logits.
__global__ void __launch_bounds__(256) logprob_entropy_bwd_kernel(void* __restrict__ logits, int is_fp32, long long ld,
                                                                  const long long* __restrict__ targets,
                                                                  const float* __restrict__ lse,
                                                                  const float* __restrict__ ent,
                                                                  const float* __restrict__ g_lp,
                                                                  const float* __restrict__ g_ent, float inv_temp,
                                                                  int vocab_start, int V) {
  const long long row = blockIdx.x;
  const long long base = row * ld;
  const float l = lse[row];
  const float H = ent ? ent[row] : 0.f;
  const float gl = g_lp ? g_lp[row] : 0.f;
  const float gh = g_ent ? g_ent[row] : 0.f;
  const long long tg = targets[row] - vocab_start;
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    const float z = load_logit(logits, is_fp32, base + j) * inv_temp;
    const float p = __expf(z - l);
    float d = gl * ((j == tg ? 1.f : 0.f) - p);
    if (g_ent) d -= gh * p * (z - l + H);
    d *= inv_temp;
    if (is_fp32) reinterpret_cast<float*>(logits)[base + j] = d;
    else reinterpret_cast<__nv_bfloat16*>(logits)[base + j] = __float2bfloat16(d);
  }
}

// Gumbel-max: argmax_j (z_j + G_j) is a sample from softmax(z).  One CTA per request.
// The uniform for a token is a hash of (seeds[b], steps[b], global vocab id): the draw depends only on those three,
// so any TP / batching layout reproduces the same sample.
__global__ void __launch_bounds__(256) sample_kernel(const void* __restrict__ logits, int is_fp32, long long ld, int V,
                                                     int vocab_start, float inv_temp, int greedy,
                                                     const long long* __restrict__ seeds,
                                                     const int* __restrict__ steps, long long* __restrict__ tokens,
                                                     float* __restrict__ logp, float* __restrict__ partial_out) {
  __shared__ Online red[32];
  __shared__ float s_best[32];
  __shared__ int s_idx[32];
  __shared__ float s_bz[32];
  const long long row = blockIdx.x;
  const long long base = row * ld;
  Online o;
  o.m = -FLT_MAX; o.s = 0.f; o.sz = 0.f;
  float best = -FLT_MAX, bz = 0.f;
  int bidx = 0;
  const unsigned long long seed = static_cast<unsigned long long>(seeds ? seeds[row] : 0);
  const unsigned long long step = static_cast<unsigned long long>(steps ? steps[row] : 0);
  // gridDim.y CTAs share a row: each takes a contiguous slice of the vocabulary and writes a partial
  const int per = (V + gridDim.y - 1) / gridDim.y;
  const int j0 = blockIdx.y * per;
  const int j1 = j0 + per < V ? j0 + per : V;
  for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
    const float z = load_logit(logits, is_fp32, base + j) * inv_temp;
    online_add(o, z);
    float score = z;
    if (!greedy) {
      const float u = hash_uniform(seed, step, static_cast<unsigned long long>(vocab_start + j));  // (0, 1)
      score = z - __logf(-__logf(u));
    }
    if (score > best) { best = score; bidx = vocab_start + j; bz = z; }
  }
  o = block_online(o, red);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffff, best, off);
    const int oi = __shfl_xor_sync(0xffffffff, bidx, off);
    const float oz = __shfl_xor_sync(0xffffffff, bz, off);
    if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; bz = oz; }
  }
  if (lane == 0) { s_best[w] = best; s_idx[w] = bidx; s_bz[w] = bz; }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    for (int i = 1; i < nw; ++i)
      if (s_best[i] > best || (s_best[i] == best && s_idx[i] < bidx)) { best = s_best[i]; bidx = s_idx[i]; bz = s_bz[i]; }
    if (partial_out) {
      float* p = partial_out + (static_cast<long long>(blockIdx.y) * gridDim.x + row) * 6;
      p[0] = o.m; p[1] = o.s; p[2] = o.sz; p[3] = best; p[4] = __int_as_float(bidx); p[5] = bz;
    } else {
      tokens[row] = bidx;
      if (logp) logp[row] = bz - (o.m + __logf(o.s));
    }
  }
}

// partials [R, B, 6] -> token, logp
__global__ void sample_combine_kernel(const float* __restrict__ partials, int R, int B,
                                      long long* __restrict__ tokens, float* __restrict__ logp) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  Online o;
  o.m = -FLT_MAX; o.s = 0.f; o.sz = 0.f;
  float best = -FLT_MAX, bz = 0.f;
  int bidx = 0;
  for (int r = 0; r < R; ++r) {
    const float* p = partials + (static_cast<long long>(r) * B + b) * 6;
    Online t;
    t.m = p[0]; t.s = p[1]; t.sz = p[2];
    online_merge(o, t);
    const int idx = __float_as_int(p[4]);
    if (p[3] > best || (p[3] == best && idx < bidx)) { best = p[3]; bidx = idx; bz = p[5]; }
  }
  tokens[b] = bidx;
  if (logp) logp[b] = bz - (o.m + __logf(o.s));
}

struct GrpoArgs {
  float clip_low, clip_high, dual_clip_c, kl_beta, ratio_clamp, kl_clamp;
  int use_dual_clip, use_kl;
};

// loss = sum_t w_t * (L_clip(t) + beta * kl3(t));  dlogp_t = w_t * d/dlogp.  stats (atomics):
// [0] sum w*L_clip  [1] sum w*kl  [2] sum w  [3] sum w*1{clipped}  [4] sum w*ratio  [5] sum w*(old-new) (approx kl)
__global__ void __launch_bounds__(256) grpo_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_lp,
                                                        const float* __restrict__ ref_lp, const float* __restrict__ adv,
                                                        const float* __restrict__ weight, long long n, GrpoArgs a,
                                                        float* __restrict__ tok_loss, float* __restrict__ dlogp,
                                                        float* __restrict__ stats) {
  float acc[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float w = weight[i];
    const float lp = logp[i];
    const float olp = old_lp ? old_lp[i] : lp;
    const float A = adv[i];
    float d = lp - olp;
    bool d_in = true;
    if (a.ratio_clamp > 0.f) {
      if (d > a.ratio_clamp) { d = a.ratio_clamp; d_in = false; }
      if (d < -a.ratio_clamp) { d = -a.ratio_clamp; d_in = false; }
    }
    const float ratio = __expf(d);
    const float rc = fminf(fmaxf(ratio, 1.f - a.clip_low), 1.f + a.clip_high);
    const float l1 = -A * ratio, l2 = -A * rc;
    float L = fmaxf(l1, l2);
    // gradient flows through the unclipped branch, or through the clipped one only when it is not saturated
    float g = (l1 >= l2) ? (d_in ? -A * ratio : 0.f) : ((rc == ratio && d_in) ? -A * ratio : 0.f);
    bool clipped = l2 > l1;
    if (a.use_dual_clip && A < 0.f) {
      const float l3 = -A * a.dual_clip_c;
      if (l3 < L) { L = l3; g = 0.f; clipped = true; }
    }
    float kl = 0.f, gk = 0.f;
    if (a.use_kl && ref_lp) {
      const float dr = ref_lp[i] - lp;
      const float e = __expf(dr);
      kl = e - dr - 1.f;
      gk = 1.f - e;
      if (a.kl_clamp > 0.f && kl > a.kl_clamp) { kl = a.kl_clamp; gk = 0.f; }
    }
    const float tl = L + a.kl_beta * kl;
    if (tok_loss) tok_loss[i] = tl;
    if (dlogp) dlogp[i] = w * (g + a.kl_beta * gk);
    acc[0] += w * L; acc[1] += w * kl; acc[2] += w; acc[3] += clipped ? w : 0.f; acc[4] += w * ratio;
    acc[5] += w * (olp - lp);
  }
  __shared__ float red[6][32];
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 6; ++k) {
    float v = acc[k];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffff, v, off);
    if (lane == 0) red[k][wp] = v;
  }
  __syncthreads();
  if (threadIdx.x < 6) {
    float v = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) v += red[threadIdx.x][i];
    atomicAdd(&stats[threadIdx.x], v);
  }
}

// GAE: one thread per sequence; [B, S] row-major rewards/values/mask -> advantages, returns.
// Tokens with mask 0 are skipped by carrying next_value / last_gae through them.
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const float* __restrict__ mask, float* __restrict__ adv, float* __restrict__ ret, int B,
                           int S, float gamma, float lam) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const long long o = static_cast<long long>(b) * S;
  float next_v = 0.f, last = 0.f;
  for (int t = S - 1; t >= 0; --t) {
    const float mk = mask[o + t];
    if (mk > 0.f) {
      const float delta = rewards[o + t] + gamma * next_v - values[o + t];
      last = delta + gamma * lam * last;
      next_v = values[o + t];
      adv[o + t] = last;
      ret[o + t] = last + values[o + t];
    } else {
      adv[o + t] = 0.f;
      ret[o + t] = 0.f;
    }
  }
}

}  // namespace gk

using namespace gk;

GK_EXPORT int gk_logprob_entropy_fwd(const void* logits, int is_fp32, long long ld, const long long* targets,
                                     float inv_temp, int vocab_start, int V, long long T, float* logp, float* ent,
                                     float* lse, float* partial, void* stream) {
  if (T == 0) return 0;
  logprob_entropy_fwd_kernel<<<static_cast<unsigned>(T), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, is_fp32, ld, targets, inv_temp, vocab_start, V, logp, ent, lse, partial);
  return launch_status();
}

GK_EXPORT int gk_logprob_entropy_combine(const float* partials, int R, long long T, float* logp, float* ent,
                                         float* lse, void* stream) {
  if (T == 0) return 0;
  logprob_entropy_combine_kernel<<<static_cast<unsigned>((T + 255) / 256), 256, 0,
                                   reinterpret_cast<cudaStream_t>(stream)>>>(partials, R, T, logp, ent, lse);
  return launch_status();
}

GK_EXPORT int gk_logprob_entropy_bwd(void* logits, int is_fp32, long long ld, const long long* targets,
                                     const float* lse, const float* ent, const float* g_lp, const float* g_ent,
                                     float inv_temp, int vocab_start, int V, long long T, void* stream) {
  if (T == 0) return 0;
  logprob_entropy_bwd_kernel<<<static_cast<unsigned>(T), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, is_fp32, ld, targets, lse, ent, g_lp, g_ent, inv_temp, vocab_start, V);
  return launch_status();
}

// slices > 1: every row is shared by `slices` CTAs and `partial` receives [slices, B, 6] (merged by gk_sample_combine
// with R = slices, or R = ranks x slices after an all-gather); the draw does not depend on the slicing.
GK_EXPORT int gk_sample(const void* logits, int is_fp32, long long ld, int V, int vocab_start, float inv_temp,
                        int greedy, const long long* seeds, const int* steps, long long* tokens, float* logp,
                        float* partial, int B, int slices, void* stream) {
  if (B == 0) return 0;
  if (slices < 1 || (slices > 1 && !partial)) return -1;
  sample_kernel<<<dim3(B, slices), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, is_fp32, ld, V, vocab_start, inv_temp, greedy, seeds, steps, tokens, logp, partial);
  return launch_status();
}

GK_EXPORT int gk_sample_combine(const float* partials, int R, int B, long long* tokens, float* logp, void* stream) {
  if (B == 0) return 0;
  sample_combine_kernel<<<(B + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(partials, R, B, tokens,
                                                                                           logp);
  return launch_status();
}

GK_EXPORT int gk_grpo_loss(const float* logp, const float* old_lp, const float* ref_lp, const float* adv,
                           const float* weight, long long n, float clip_low, float clip_high, float dual_clip_c,
                           float kl_beta, float ratio_clamp, float kl_clamp, float* tok_loss, float* dlogp,
                           float* stats, void* stream) {
  if (n == 0) return 0;
  GrpoArgs a;
  a.clip_low = clip_low; a.clip_high = clip_high; a.dual_clip_c = dual_clip_c; a.kl_beta = kl_beta;
  a.ratio_clamp = ratio_clamp; a.kl_clamp = kl_clamp;
  a.use_dual_clip = dual_clip_c > 0.f; a.use_kl = kl_beta != 0.f;
  long long blocks = (n + 255) / 256;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  grpo_loss_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logp, old_lp, ref_lp, adv, weight, n, a, tok_loss, dlogp, stats);
  return launch_status();
}

GK_EXPORT int gk_gae(const float* rewards, const float* values, const float* mask, float* adv, float* ret, int B,
                     int S, float gamma, float lam, void* stream) {
  if (B == 0) return 0;
  gae_kernel<<<(B + 63) / 64, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(rewards, values, mask, adv, ret, B, S,
                                                                             gamma, lam);
  return launch_status();
}
