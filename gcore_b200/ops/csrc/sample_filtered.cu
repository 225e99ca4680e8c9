// Top-k / nucleus (top-p) / min-p sampling in one kernel per batch, without sorting the vocabulary.
//
// One CTA per row.  After the row maximum is known every logit is mapped to a 24-bit key, u = (zmax - z) / 40 * 2^24
// (smaller key = larger logit; logits more than 40 below the maximum carry less than 5e-18 of the mass and are
// outside every filter).  A three-level radix descent over 8-bit digits, with a count and a probability-mass histogram
// per level in shared memory, finds
//   * the key of the k-th largest logit                                  (top-k),
//   * the key of the last element of the shortest prefix of the descending order whose preceding mass is <= top_p of
//     the top-k-filtered mass                                             (top-p, applied after top-k),
// and min-p is a key bound by itself (p >= min_p * p_max  <=>  z >= zmax + ln(min_p)).  Logits whose keys coincide
// (closer than 2.4e-6) are kept or dropped together.  The draw is Gumbel-max over the kept set with the same
// counter-based random stream as the unfiltered sampler (vocab.cu), and the returned log-prob is that of the
// renormalised filtered distribution.  Filter semantics follow the sort-based definition in ops/vocab.py
// (apply_top_k_top_p), which is what the reference's serving engines apply (sampling parameters of
// gpatch_v4/generation_backend/infer_engine.py: top_k, top_p, min_p).
#include "host_utils.h"
#include <cuda_bf16.h>
#include <float.h>

namespace gks {

constexpr int THREADS = 1024;
constexpr float WINDOW = 40.f;
constexpr unsigned int KEY_MAX = (1u << 24) - 1u;

__device__ __forceinline__ float load_logit(const void* p, int is_fp32, long long i) {
  return is_fp32 ? reinterpret_cast<const float*>(p)[i]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned long long step,
                                              unsigned long long idx) {
  unsigned long long x = seed * 0x9E3779B97F4A7C15ULL + step * 0xD1B54A32D192ED03ULL + idx * 0x2545F4914F6CDD1DULL +
                         0x632BE59BD9B4E019ULL;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ULL;
  x ^= x >> 27; x *= 0x94D049BB133111EBULL;
  x ^= x >> 31;
  return (static_cast<float>(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}
// Scaled logit and its key; 0xFFFFFFFF = outside the window.  Explicitly rounded operations: the same element must map
// to the same key in every pass, so the compiler may not contract the scaling, the subtraction and the multiply into
// fused multiply-adds differently from one call site to the next.
__device__ __forceinline__ float scaled(const void* p, int is_fp32, long long i, float inv_temp) {
  return __fmul_rn(load_logit(p, is_fp32, i), inv_temp);
}
__device__ __forceinline__ unsigned int key_of(float z, float zmax) {
  const float q = __fmul_rn(__fsub_rn(zmax, z), 16777216.f / WINDOW);
  return q < 16777215.5f ? static_cast<unsigned int>(q) : 0xFFFFFFFFu;
}

struct Sel {
  unsigned int key;   // elements with key <= this are kept
  float mass;         // sum of exp(z - zmax) over the kept elements
  int found;
};

// Radix descent.  mode 0: smallest key with count(key' <= key) >= target_count.  mode 1: smallest key with
// mass(key' <= key) > target_mass.  Only elements with key <= limit take part.
__device__ Sel radix_select(const void* logits, int is_fp32, long long base, int V, float inv_temp, float zmax,
                            unsigned int limit, int mode, float target_count, float target_mass, float* hist_c,
                            float* hist_m, unsigned int* s_prefix, float* s_above, int* s_found) {
  unsigned int prefix = 0;  // resolved high digits
  float count_above = 0.f, mass_above = 0.f;
  for (int level = 0; level < 3; ++level) {
    const int shift = 16 - 8 * level;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { hist_c[i] = 0.f; hist_m[i] = 0.f; }
    __syncthreads();
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
      const float z = scaled(logits, is_fp32, base + j, inv_temp);
      const unsigned int u = key_of(z, zmax);
      if (u > limit) continue;
      if (level > 0 && (u >> (shift + 8)) != prefix) continue;
      const int d = (u >> shift) & 255;
      atomicAdd(&hist_c[d], 1.f);
      atomicAdd(&hist_m[d], __expf(z - zmax));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float c = count_above, m = mass_above;
      int pick = -1;
      for (int d = 0; d < 256; ++d) {
        const float nc = c + hist_c[d], nm = m + hist_m[d];
        const bool hit = mode == 0 ? (nc >= target_count) : (nm > target_mass);
        if (hit && hist_c[d] > 0.f) { pick = d; break; }
        c = nc; m = nm;
      }
      if (pick < 0 && level > 0) {
        // the parent bucket crossed the target; rounding of this level's partial sums must not lose the crossing:
        // it lies in the last occupied digit
        c = count_above; m = mass_above;
        int last = -1;
        for (int d = 0; d < 256; ++d)
          if (hist_c[d] > 0.f) last = d;
        for (int d = 0; d < last; ++d) { c += hist_c[d]; m += hist_m[d]; }
        pick = last;
      }
      if (pick < 0) {
        *s_found = 0;
        s_above[0] = c; s_above[1] = m;
      } else {
        *s_found = 1;
        *s_prefix = (prefix << 8) | static_cast<unsigned int>(pick);
        if (level == 2) { c += hist_c[pick]; m += hist_m[pick]; }  // the final key's own elements are kept
        s_above[0] = c; s_above[1] = m;
      }
    }
    __syncthreads();
    count_above = s_above[0];
    mass_above = s_above[1];
    if (!*s_found) {
      Sel r;
      r.key = limit; r.mass = mass_above; r.found = 0;  // fewer elements / less mass than asked: keep everything
      __syncthreads();
      return r;
    }
    prefix = *s_prefix;
    __syncthreads();
  }
  Sel r;
  r.key = prefix; r.mass = mass_above; r.found = 1;
  return r;
}

__global__ void __launch_bounds__(THREADS) sample_filtered_kernel(
    const void* __restrict__ logits, int is_fp32, long long ld, int V, float inv_temp, int top_k, float top_p,
    float min_p, int greedy, const long long* __restrict__ seeds, const int* __restrict__ steps,
    long long* __restrict__ tokens, float* __restrict__ logp, int* __restrict__ kept_out) {
  __shared__ float hist_c[256], hist_m[256];
  __shared__ float s_red[32], s_bz[32], s_above[2];
  __shared__ int s_idx[32], s_found;
  __shared__ unsigned int s_prefix;
  const long long row = blockIdx.x;
  const long long base = row * ld;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  // ---- row maximum
  float zmax = -FLT_MAX;
  for (int j = threadIdx.x; j < V; j += blockDim.x) zmax = fmaxf(zmax, scaled(logits, is_fp32, base + j, inv_temp));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
  if (lane == 0) s_red[w] = zmax;
  __syncthreads();
  zmax = s_red[0];
  for (int i = 1; i < nw; ++i) zmax = fmaxf(zmax, s_red[i]);
  __syncthreads();
  // ---- thresholds
  unsigned int limit = KEY_MAX;
  if (top_k > 0 && top_k < V) {
    const Sel k = radix_select(logits, is_fp32, base, V, inv_temp, zmax, limit, 0, static_cast<float>(top_k), 0.f, hist_c,
                               hist_m, &s_prefix, s_above, &s_found);
    if (k.key < limit) limit = k.key;
  }
  if (top_p < 1.f) {
    // mass of what is left after top-k / min-p
    float m = 0.f;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
      const float z = scaled(logits, is_fp32, base + j, inv_temp);
      if (key_of(z, zmax) <= limit) m += __expf(z - zmax);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m += __shfl_xor_sync(0xffffffffu, m, o);
    if (lane == 0) s_red[w] = m;
    __syncthreads();
    m = 0.f;
    for (int i = 0; i < nw; ++i) m += s_red[i];
    __syncthreads();
    const Sel p = radix_select(logits, is_fp32, base, V, inv_temp, zmax, limit, 1, 0.f, top_p * m, hist_c, hist_m,
                               &s_prefix, s_above, &s_found);
    if (p.key < limit) limit = p.key;
  }
  if (min_p > 0.f) {  // applied last, like the definition; the bound itself does not depend on the other filters
    const float q = -__logf(min_p) * (16777216.f / WINDOW);
    if (q < 16777215.f && static_cast<unsigned int>(q) < limit) limit = static_cast<unsigned int>(q);
  }
  // ---- draw among the kept elements
  const unsigned long long seed = static_cast<unsigned long long>(seeds ? seeds[row] : 0);
  const unsigned long long step = static_cast<unsigned long long>(steps ? steps[row] : 0);
  float best = -FLT_MAX, bz = 0.f, mass = 0.f;
  int bidx = 0, kept = 0;
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    const float z = scaled(logits, is_fp32, base + j, inv_temp);
    if (key_of(z, zmax) > limit) continue;
    mass += __expf(z - zmax);
    ++kept;
    float score = z;
    if (!greedy) score = z - __logf(-__logf(hash_uniform(seed, step, static_cast<unsigned long long>(j))));
    if (score > best) { best = score; bidx = j; bz = z; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
    const float oz = __shfl_xor_sync(0xffffffffu, bz, o);
    if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; bz = oz; }
    mass += __shfl_xor_sync(0xffffffffu, mass, o);
    kept += __shfl_xor_sync(0xffffffffu, kept, o);
  }
  if (lane == 0) { s_red[w] = best; s_idx[w] = bidx; s_bz[w] = bz; hist_m[w] = mass; hist_c[w] = static_cast<float>(kept); }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tm = 0.f, tk = 0.f;
    for (int i = 0; i < nw; ++i) {
      if (i > 0 && (s_red[i] > best || (s_red[i] == best && s_idx[i] < bidx))) { best = s_red[i]; bidx = s_idx[i]; bz = s_bz[i]; }
      tm += hist_m[i];
      tk += hist_c[i];
    }
    tokens[row] = bidx;
    if (logp) logp[row] = bz - zmax - __logf(tm);
    if (kept_out) kept_out[row] = static_cast<int>(tk);
  }
}

}  // namespace gks

// logits [B, V] (bf16 or fp32, row stride ld) hold the WHOLE vocabulary (tensor-parallel callers gather first).
// top_k <= 0, top_p >= 1, min_p <= 0 switch the respective filter off.  kept_out (optional) receives the size of the
// kept set per row.
GK_EXPORT int gk_sample_filtered(const void* logits, int is_fp32, long long ld, int V, float inv_temp, int top_k,
                                 float top_p, float min_p, int greedy, const long long* seeds, const int* steps,
                                 long long* tokens, float* logp, int* kept_out, int B, void* stream) {
  if (B == 0) return 0;
  if (V <= 0) return -1;
  gks::sample_filtered_kernel<<<B, gks::THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, is_fp32, ld, V, inv_temp, top_k, top_p, min_p, greedy, seeds, steps, tokens, logp, kept_out);
  return gk::launch_status();
}
