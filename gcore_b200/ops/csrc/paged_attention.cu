// Rollout-decoder attention: RoPE-fused KV-cache append and split-KV paged decode attention (GQA, optional
// sliding window and per-head sink logit).  Both are HBM-bandwidth bound: a CTA serves one (request, kv-head, KV split)
// and all query heads of the group so every K/V byte is read once (16-byte cp.async into swizzled shared memory); the
// scores run on mma.sync tiles (8 query heads are far below the 64-row minimum of a tcgen05 instruction), with a
// CUDA-core kernel for GQA groups wider than 8.  Stands in for the vLLM / SGLang attention back ends the reference drives
// (gpatch_v4/generation_backend/infer_engine.py:479-768).
#include "host_utils.h"
#include <cuda_bf16.h>
#include <float.h>

namespace gk {

constexpr int PD_THREADS = 128;
constexpr int PD_TILE = 32;     // tokens per shared-memory tile
constexpr int PD_MAX_GROUP = 16;
constexpr int PD_SPLIT = 128;   // tokens per KV split (the finest; the tensor-core kernel uses multiples)
inline int& paged_target_ctas() {
  static int n = 444;
  return n;
}

// qkv: [T, (Hq + 2*Hk) * D] as produced by the fused QKV projection ([q | k | v] per token).
// Rotates q and k in place (rotate-half pairing) and writes k, v to cache slot `slots[t]`
// (slot = block * block_size + offset; negative = skip the cache write).
__global__ void kv_append_rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                      const int* __restrict__ slots, __nv_bfloat16* __restrict__ kc,
                                      __nv_bfloat16* __restrict__ vc, int T, int Hq, int Hk, int D, int rot,
                                      float theta, int do_rope) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= T) return;
  const int half = rot >> 1;
  __nv_bfloat16* row = qkv + static_cast<long long>(t) * (Hq + 2 * Hk) * D;
  const int p = pos[t];
  if (do_rope) {
    const int nrot = (Hq + Hk) * half;
    for (int i = threadIdx.x; i < nrot; i += blockDim.x) {
      const int h = i / half, j = i - h * half;
      const float inv = __powf(theta, -2.f * j / rot);
      float s, c;
      sincosf(p * inv, &s, &c);
      __nv_bfloat16* x = row + h * D;
      const float a = __bfloat162float(x[j]), b = __bfloat162float(x[j + half]);
      x[j] = __float2bfloat16(a * c - b * s);
      x[j + half] = __float2bfloat16(b * c + a * s);
    }
    __syncthreads();
  }
  const long long slot = slots ? slots[t] : -1;
  if (slot < 0) return;
  const int nkv = Hk * D / 8;
  const uint4* ks = reinterpret_cast<const uint4*>(row + Hq * D);
  const uint4* vs = reinterpret_cast<const uint4*>(row + (Hq + Hk) * D);
  uint4* kd = reinterpret_cast<uint4*>(kc + slot * Hk * D);
  uint4* vd = reinterpret_cast<uint4*>(vc + slot * Hk * D);
  for (int i = threadIdx.x; i < nkv; i += blockDim.x) {
    kd[i] = ks[i];
    vd[i] = vs[i];
  }
}

// One CTA per (request b, kv head, split).  D == 128.  Writes either the final output (nsplit == 1) or
// partial (o unnormalised, m, l) to the scratch buffer for the combine kernel.
template <int D>
__global__ void __launch_bounds__(PD_THREADS, 4) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kc,
    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ ctx_len, const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
    float* __restrict__ scratch, int Hq, int Hk, int block_size, int window, float scale, int nsplit) {
  constexpr int DP = D + 8;  // padded row (bank-conflict free 16-byte accesses)
  __shared__ __align__(16) __nv_bfloat16 sk[PD_TILE][DP];
  __shared__ __align__(16) __nv_bfloat16 sv[PD_TILE][DP];
  __shared__ float sq[PD_MAX_GROUP][D];
  __shared__ float sp[PD_MAX_GROUP][PD_TILE];
  __shared__ float s_m[PD_MAX_GROUP], s_l[PD_MAX_GROUP], s_scale[PD_MAX_GROUP];

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hk;
  const int len = ctx_len[b];
  int start = 0;
  if (window > 0 && len > window) start = len - window;
  if (split > 0 && start + split * PD_SPLIT >= len) return;  // dead split: the combine kernel skips it
  const int s0 = start + split * PD_SPLIT;
  int s1 = s0 + PD_SPLIT;
  if (s1 > len) s1 = len;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < G * D; i += PD_THREADS) {
    const int g = i / D, d = i - g * D;
    sq[g][d] = __bfloat162float(q[b * q_stride + static_cast<long long>(kvh * G + g) * D + d]) * scale;
  }
  if (tid < PD_MAX_GROUP) { s_m[tid] = -FLT_MAX; s_l[tid] = 0.f; }
  float o[PD_MAX_GROUP];
#pragma unroll
  for (int g = 0; g < PD_MAX_GROUP; ++g) o[g] = 0.f;
  __syncthreads();

  for (int t0 = s0; t0 < s1; t0 += PD_TILE) {
    const int nt = s1 - t0 < PD_TILE ? s1 - t0 : PD_TILE;
    // ---- load K/V tile (16-byte coalesced)
    for (int i = tid; i < PD_TILE * (D / 8); i += PD_THREADS) {
      const int r = i / (D / 8), c = i - r * (D / 8);
      uint4 kk = make_uint4(0, 0, 0, 0), vv = kk;
      if (r < nt) {
        const int tok = t0 + r;
        const long long blk = block_table[static_cast<long long>(b) * max_blocks + tok / block_size];
        const long long slot = blk * block_size + tok % block_size;
        kk = reinterpret_cast<const uint4*>(kc + (slot * Hk + kvh) * D)[c];
        vv = reinterpret_cast<const uint4*>(vc + (slot * Hk + kvh) * D)[c];
      }
      *reinterpret_cast<uint4*>(&sk[r][c * 8]) = kk;
      *reinterpret_cast<uint4*>(&sv[r][c * 8]) = vv;
    }
    __syncthreads();
    // ---- scores: thread = (slot = tid / 32, token = lane); heads g = slot, slot + 4, ...
    for (int g = warp; g < G; g += PD_THREADS / 32) {
      float acc = 0.f;
#pragma unroll
      for (int d8 = 0; d8 < D / 8; ++d8) {
        const uint4 kk = *reinterpret_cast<const uint4*>(&sk[lane][d8 * 8]);
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kk);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 kf = __bfloat1622float2(k2[j]);
          acc += kf.x * sq[g][d8 * 8 + 2 * j] + kf.y * sq[g][d8 * 8 + 2 * j + 1];
        }
      }
      const float s = lane < nt ? acc : -FLT_MAX;
      float mx = s;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffff, mx, off));
      const float m_old = s_m[g];
      const float m_new = fmaxf(m_old, mx);
      const float p = lane < nt ? __expf(s - m_new) : 0.f;
      float ps = p;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffff, ps, off);
      sp[g][lane] = p;
      if (lane == 0) {
        const float sc = __expf(m_old - m_new);
        s_scale[g] = sc;
        s_l[g] = s_l[g] * sc + ps;
        s_m[g] = m_new;
      }
    }
    __syncthreads();
    // ---- O += P V : thread owns output dim d = tid
    if (tid < D) {
#pragma unroll
      for (int g = 0; g < PD_MAX_GROUP; ++g) {
        if (g < G) {
          float a = o[g] * s_scale[g];
          for (int r = 0; r < nt; ++r) a += sp[g][r] * __bfloat162float(sv[r][tid]);
          o[g] = a;
        }
      }
    }
    __syncthreads();
  }

  if (nsplit == 1) {
    if (tid < D) {
#pragma unroll
      for (int g = 0; g < PD_MAX_GROUP; ++g) {
        if (g < G) {
          float l = s_l[g];
          const int h = kvh * G + g;
          if (sinks) l += __expf(sinks[h] - s_m[g]);
          out[(static_cast<long long>(b) * Hq + h) * D + tid] = __float2bfloat16(l > 0.f ? o[g] / l : 0.f);
        }
      }
    }
  } else {
    // scratch layout: [b, h, split, D + 2]
#pragma unroll
    for (int g = 0; g < PD_MAX_GROUP; ++g) {
      if (g < G) {
        const int h = kvh * G + g;
        float* dst = scratch + ((static_cast<long long>(b) * Hq + h) * nsplit + split) * (D + 2);
        if (tid < D) dst[tid] = o[g];
        if (tid == 0) { dst[D] = s_m[g]; dst[D + 1] = s_l[g]; }
      }
    }
  }
}


constexpr int PD2_WARPS = 4;
constexpr int PD2_G = 8;
constexpr int PD2_TOK_PER_WARP = PD_SPLIT / PD2_WARPS;  // 32: one tile per warp

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core variant (GQA groups of up to 8 heads, D = 128).  The scalar kernels above spend ~128 FMAs per
// (head, token) pair and end up issue-bound long before HBM is saturated; here the group's heads are the (padded)
// M = 16 rows of mma.sync m16n8k16 tiles, so a 32-token tile costs 32 MMAs for Q K^T and 32 for P V per warp.
// (tcgen05 needs M >= 64 per instruction and a TMEM / mbarrier set-up per CTA, which does not pay for 8 query rows.)
//   * K and V tiles arrive with cp.async into chunk-swizzled shared memory (16-byte chunk c of row r at c ^ (r & 15)),
//     so ldmatrix is bank-conflict free without padding;
//   * S lives in the accumulator layout, P is re-packed in registers into the A-operand layout of the P V MMA;
//   * rows 8..15 of every tile are padding and are ignored.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(PD2_WARPS * 32, 3) paged_decode_mma_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kc,
    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ ctx_len, const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
    float* __restrict__ scratch, int Hq, int Hk, int block_size, int window, float scale, int nsplit,
    int split_tokens, int rot, float theta, const int* __restrict__ new_slots, __nv_bfloat16* __restrict__ kc_w,
    __nv_bfloat16* __restrict__ vc_w) {
  // rot > 0: q is the query part of packed [q | k | v] rows (row stride q_stride) that have not been rotated yet.
  // The kernel then does what kv_append_rope_kernel does for its (request, kv head): rotary embedding of the query
  // heads while they are staged, and, in the CTA whose split ends at the request's newest position, rotation of the
  // new key, its and the new value's store to cache slot new_slots[b], and their use from shared memory in this step
  // (the cache row the tile copy fetched for that position is stale and is overwritten in the tile).
  constexpr int D = 128;
  __shared__ __align__(16) uint8_t sq[16 * 256];  // Q tile, 16 rows (heads, zero padded) x 256 B, chunk-swizzled
  __shared__ float rope_s[64], rope_c[64];
  __shared__ long long slot_buf[PD2_WARPS][32];
  __shared__ float m_all[PD2_WARPS][PD2_G], l_all[PD2_WARPS][PD2_G];
  extern __shared__ __align__(16) uint8_t pd3_dyn[];  // K tiles | V tiles: 32 rows x 256 B per warp
  uint8_t* k_tile = pd3_dyn;
  uint8_t* v_tile = pd3_dyn + PD2_WARPS * 32 * 256;

  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hk;
  const int len = ctx_len[b];
  int start = 0;
  if (window > 0 && len > window) start = len - window;
  // A CTA owns `split_tokens` consecutive tokens of the request (the host sizes the splits so that the grid about
  // fills the GPU once: with many requests a CTA walks a request's whole context, and the per-CTA costs - context
  // length, block table, Q staging, merge, partial write - are paid once per request instead of once per 128 tokens).
  // Splits beyond this request's context have nothing to do (the combine kernel only reads the live ones).
  const int s0 = start + split * split_tokens;
  if (split > 0 && s0 >= len) return;
  int s1 = s0 + split_tokens;
  if (s1 > len) s1 = len;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ntiles = s1 > s0 ? (s1 - s0 + 31) / 32 : 0;

  uint8_t* kt = k_tile + warp * (32 * 256);
  uint8_t* vt = v_tile + warp * (32 * 256);
  const uint32_t kts = static_cast<uint32_t>(__cvta_generic_to_shared(kt));
  const uint32_t vts = static_cast<uint32_t>(__cvta_generic_to_shared(vt));

  // this warp's tiles are warp, warp + 4, ...: request the first one, stage Q while it is in flight
  auto tile_slot = [&](int t) -> long long {
    const int tok = s0 + t * 32 + lane;
    if (t >= ntiles || tok >= s1) return 0;
    return static_cast<long long>(block_table[static_cast<long long>(b) * max_blocks + tok / block_size]) * block_size +
           tok % block_size;
  };
  auto request_tile = [&](int t, long long slot_lane) {
    const int base_tok = s0 + t * 32;
    const int nt = s1 - base_tok < 32 ? s1 - base_tok : 32;
    slot_buf[warp][lane] = slot_lane;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = i * 32 + lane;
      const int row = idx >> 4, ch = idx & 15;
      const long long slot = slot_buf[warp][row];
      const uint32_t nbytes = row < nt ? 16u : 0u;  // rows past the end are zero-filled
      const uint32_t doff = static_cast<uint32_t>(row * 256 + ((ch ^ (row & 15)) << 4));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kts + doff),
                   "l"(kc + (slot * Hk + kvh) * D + ch * 8), "r"(nbytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vts + doff),
                   "l"(vc + (slot * Hk + kvh) * D + ch * 8), "r"(nbytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (warp < ntiles) request_tile(warp, tile_slot(warp));
  const int half = rot >> 1;
  if (rot > 0) {
    if (tid < half) {
      const float inv = __powf(theta, -2.f * tid / rot);
      sincosf((len - 1) * inv, &rope_s[tid], &rope_c[tid]);
    }
    __syncthreads();
  }
  // rotate-half pairing on 16-byte chunks: chunk c < half / 8 holds dims 8c .. 8c + 7, its partners sit half / 8
  // chunks further; dims at or beyond rot pass through
  auto rotate_pair = [&](uint4& lo, uint4& hi, int c) {
    __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&lo);
    __nv_bfloat16* bb = reinterpret_cast<__nv_bfloat16*>(&hi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sn = rope_s[c * 8 + e], cs = rope_c[c * 8 + e];
      const float x = __bfloat162float(a[e]), y = __bfloat162float(bb[e]);
      a[e] = __float2bfloat16(x * cs - y * sn);
      bb[e] = __float2bfloat16(y * cs + x * sn);
    }
  };
  const int hc = half >> 3;   // chunks per rotated half (0 without fused rotation)
  for (int i = tid; i < 16 * 16; i += PD2_WARPS * 32) {
    const int g = i >> 4, c = i & 15;
    if (rot > 0 && c >= hc && c < 2 * hc) continue;   // written together with its partner chunk
    const uint4* src = reinterpret_cast<const uint4*>(q + b * q_stride + static_cast<long long>(kvh * G + g) * D);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rot > 0 && c < hc) {
      uint4 w = make_uint4(0, 0, 0, 0);
      if (g < G) {
        v = src[c];
        w = src[c + hc];
        rotate_pair(v, w, c);
      }
      *reinterpret_cast<uint4*>(sq + g * 256 + (((c + hc) ^ (g & 15)) << 4)) = w;
    } else if (g < G) {
      v = src[c];
    }
    *reinterpret_cast<uint4*>(sq + g * 256 + ((c ^ (g & 15)) << 4)) = v;
  }
  __syncthreads();
  // the newest position of the request lies in the last tile of the split that ends at `len`
  const bool appends = rot > 0 && s1 == len && ntiles > 0;

  const int r0 = lane >> 2;        // this thread's accumulator row = head index inside the group
  const int cq = (lane & 3) * 2;   // first of its two columns inside an 8-wide tile
  float m_run = -FLT_MAX, l_run = 0.f;
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  if (warp < ntiles) {
    // Q as A fragments for the 8 k-steps (16 dims each)
    uint32_t qa[8][4];
    const uint32_t sqs = static_cast<uint32_t>(__cvta_generic_to_shared(sq));
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int ch = ks * 2 + (lane >> 4);
      ldsm_x4(qa[ks], sqs + row * 256 + ((ch ^ (row & 15)) << 4));
    }
#pragma unroll 1
    for (int t = warp; t < ntiles; t += PD2_WARPS) {
      const int base_tok = s0 + t * 32;
      const int nt = s1 - base_tok < 32 ? s1 - base_tok : 32;
      // the block-table entries of this warp's next tile are fetched while the current tile's K / V arrive
      const long long next_slot = tile_slot(t + PD2_WARPS);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
      if (appends && t == ntiles - 1) {
        const int row = len - 1 - base_tok;
        const long long slot = new_slots[b];
        const __nv_bfloat16* krow = q + b * q_stride + static_cast<long long>(Hq + kvh) * D;
        const __nv_bfloat16* vrow = q + b * q_stride + static_cast<long long>(Hq + Hk + kvh) * D;
        if (lane < 16) {          // the key: lanes below hc rotate a chunk pair, lanes of unrotated chunks copy
          const int c = lane;
          const bool lead = c < hc, partner = c >= hc && c < 2 * hc;
          if (!partner) {
            uint4 v = reinterpret_cast<const uint4*>(krow)[c];
            if (lead) {
              uint4 w = reinterpret_cast<const uint4*>(krow)[c + hc];
              rotate_pair(v, w, c);
              *reinterpret_cast<uint4*>(kt + row * 256 + (((c + hc) ^ (row & 15)) << 4)) = w;
              if (slot >= 0) reinterpret_cast<uint4*>(kc_w + (slot * Hk + kvh) * D)[c + hc] = w;
            }
            *reinterpret_cast<uint4*>(kt + row * 256 + ((c ^ (row & 15)) << 4)) = v;
            if (slot >= 0) reinterpret_cast<uint4*>(kc_w + (slot * Hk + kvh) * D)[c] = v;
          }
        } else {                  // the value
          const int c = lane - 16;
          const uint4 v = reinterpret_cast<const uint4*>(vrow)[c];
          *reinterpret_cast<uint4*>(vt + row * 256 + ((c ^ (row & 15)) << 4)) = v;
          if (slot >= 0) reinterpret_cast<uint4*>(vc_w + (slot * Hk + kvh) * D)[c] = v;
        }
        __syncwarp();
      }
      // ---- S = Q K^T : 4 token tiles of 8
      float sc[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {  // pairs of k-steps
          uint32_t kb[4];
          const int row = j * 8 + (lane & 7);
          const int ch = kp * 4 + (lane >> 3);
          ldsm_x4(kb, kts + row * 256 + ((ch ^ (row & 15)) << 4));
          mma_bf16_16816(sc[j], qa[2 * kp], kb[0], kb[1]);
          mma_bf16_16816(sc[j], qa[2 * kp + 1], kb[2], kb[3]);
        }
      }
      // ---- online softmax over this tile for row r0 (rows 8..15 are padding)
      float mx = -FLT_MAX;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int ti = j * 8 + cq + e;
          const float v = ti < nt ? sc[j][e] * scale : -FLT_MAX;
          sc[j][e] = v;
          mx = fmaxf(mx, v);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffff, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffff, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float resc = m_run == -FLT_MAX ? 0.f : __expf(m_run - m_new);
      m_run = m_new;
      l_run *= resc;
#pragma unroll
      for (int j = 0; j < 16; ++j) { o[j][0] *= resc; o[j][1] *= resc; }
      uint32_t pa[2][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p0 = sc[j][0] == -FLT_MAX ? 0.f : __expf(sc[j][0] - m_new);
        const float p1 = sc[j][1] == -FLT_MAX ? 0.f : __expf(sc[j][1] - m_new);
        l_run += p0 + p1;
        // A fragment of k-step j/2: regs {rows lo cols lo, rows hi cols lo, rows lo cols hi, rows hi cols hi}
        pa[j >> 1][(j & 1) * 2] = pack2_bf16(p0, p1);
        pa[j >> 1][(j & 1) * 2 + 1] = 0u;  // padding rows
      }
      // ---- O += P V : 2 k-steps of 16 tokens, 16 dim tiles of 8
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int np = 0; np < 8; ++np) {  // pairs of dim tiles
          uint32_t vb[4];
          const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int ch = np * 2 + (lane >> 4);
          ldsm_x4_trans(vb, vts + row * 256 + ((ch ^ (row & 15)) << 4));
          mma_bf16_16816(o[2 * np], pa[kk], vb[0], vb[1]);
          mma_bf16_16816(o[2 * np + 1], pa[kk], vb[2], vb[3]);
        }
      }
      __syncwarp();   // every lane is done with the tile before its storage is refilled
      if (t + PD2_WARPS < ntiles) request_tile(t + PD2_WARPS, next_slot);
    }
  }
  // ---- merge the four warps (K tiles are dead after the barrier: their storage carries the partial outputs)
  l_run += __shfl_xor_sync(0xffffffff, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffff, l_run, 2);
  __syncthreads();
  float (*o_all)[PD2_G][D] = reinterpret_cast<float (*)[PD2_G][D]>(k_tile);
  if ((lane & 3) == 0) { m_all[warp][r0] = m_run; l_all[warp][r0] = l_run; }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    *reinterpret_cast<float2*>(&o_all[warp][r0][j * 8 + cq]) = make_float2(o[j][0], o[j][1]);
  }
  __syncthreads();
  const int d = tid;  // 128 threads <-> 128 dims
  for (int g = 0; g < G; ++g) {
    float mm = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < PD2_WARPS; ++w) mm = fmaxf(mm, m_all[w][g]);
    float acc = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < PD2_WARPS; ++w) {
      const float f = m_all[w][g] == -FLT_MAX ? 0.f : __expf(m_all[w][g] - mm);
      acc += o_all[w][g][d] * f;
      ls += l_all[w][g] * f;
    }
    const int h = kvh * G + g;
    if (nsplit == 1) {
      if (sinks) ls += __expf(sinks[h] - mm);
      out[(static_cast<long long>(b) * Hq + h) * D + d] = __float2bfloat16(ls > 0.f ? acc / ls : 0.f);
    } else {
      float* dst = scratch + ((static_cast<long long>(b) * Hq + h) * nsplit + split) * (D + 2);
      dst[d] = acc;
      if (d == 0) { dst[D] = mm; dst[D + 1] = ls; }
    }
  }
}

template <int D>
__global__ void paged_decode_combine_kernel(const float* __restrict__ scratch, const float* __restrict__ sinks,
                                            const int* __restrict__ ctx_len, int window,
                                            __nv_bfloat16* __restrict__ out, int Hq, int nsplit_total,
                                            int split_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float* base = scratch + (static_cast<long long>(b) * Hq + h) * nsplit_total * (D + 2);
  int span = ctx_len[b];
  if (window > 0 && span > window) span = window;
  int nsplit = (span + split_tokens - 1) / split_tokens;  // live splits: the others were never written
  if (nsplit < 1) nsplit = 1;
  if (nsplit > nsplit_total) nsplit = nsplit_total;
  float m = -FLT_MAX;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, base[s * (D + 2) + D]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = base[s * (D + 2) + D];
    const float w = ms == -FLT_MAX ? 0.f : __expf(ms - m);
    l += base[s * (D + 2) + D + 1] * w;
    acc += base[s * (D + 2) + d] * w;
  }
  if (sinks) l += __expf(sinks[h] - m);
  out[(static_cast<long long>(b) * Hq + h) * D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace gk

using namespace gk;

GK_EXPORT int gk_kv_append_rope(void* qkv, const int* pos, const int* slots, void* kc, void* vc, int T, int Hq,
                                int Hk, int D, int rot, int do_rope, float theta, int reserved, void* stream) {
  (void)reserved;
  if (T == 0) return 0;
  if ((Hk * D) % 8) return -1;
  // ordinary launch: with programmatic serialization this 64-block kernel measured slower (8.2 us vs 5.7 us)
  kv_append_rope_kernel<<<T, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(qkv), pos, slots, reinterpret_cast<__nv_bfloat16*>(kc),
      reinterpret_cast<__nv_bfloat16*>(vc), T, Hq, Hk, D, rot, theta, do_rope);
  return launch_status();
}

// CTAs the tensor-core decode kernel aims for (three fit an SM); the host derives the split size from it
GK_EXPORT void gk_paged_set_target_ctas(int n) { paged_target_ctas() = n > 0 ? n : 444; }

GK_EXPORT void gk_paged_decode_scratch(int B, int Hq, int D, int max_ctx, long long* floats) {
  const long long ns = (max_ctx + PD_SPLIT - 1) / PD_SPLIT;
  *floats = static_cast<long long>(B) * Hq * ns * (D + 2);
}

// max_ctx bounds every ctx_len[b] (after windowing); it fixes the number of KV splits so the launch shape does
// not depend on device data (CUDA-graph friendly).
static int paged_decode_impl(const void* q, const void* kc, const void* vc, const int* block_table,
                             const int* ctx_len, const float* sinks, void* out, float* scratch, int B, int Hq,
                             int Hk, int D, int block_size, int max_blocks, int max_ctx, float scale, int window,
                             int q_stride, int rot, float theta, const int* new_slots, void* stream) {
  if (D != 128 || Hq % Hk || Hq / Hk > PD_MAX_GROUP) return -1;
  if (rot > 0 && (Hq / Hk > PD2_G || rot > D || rot % 16 || !new_slots)) return -4;
  if (B == 0) return 0;
  int span = max_ctx;
  if (window > 0 && window < span) span = window;
  const int nsplit_max = (span + PD_SPLIT - 1) / PD_SPLIT > 0 ? (span + PD_SPLIT - 1) / PD_SPLIT : 1;
  int nsplit = nsplit_max, split_tokens = PD_SPLIT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (Hq / Hk <= PD2_G) {
    // as many splits as give the GPU about one wave of CTAs (three fit an SM), never finer than 128 tokens
    const int pairs = B * Hk;
    int want = paged_target_ctas() / pairs;
    if (want < 1) want = 1;
    if (want < nsplit) nsplit = want;
    split_tokens = ((span + nsplit - 1) / nsplit + 31) / 32 * 32;
    if (split_tokens < PD_SPLIT) split_tokens = PD_SPLIT;
    nsplit = (span + split_tokens - 1) / split_tokens;
    if (nsplit < 1) nsplit = 1;
  }
  if (nsplit > 1 && !scratch) return -2;
  dim3 grid(B, Hk, nsplit);
  if (Hq / Hk <= PD2_G) {
    constexpr int PD2_SMEM = 2 * PD2_WARPS * 32 * 128 * 2;
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(paged_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PD2_SMEM);
      configured = true;
    }
    launch_k(paged_decode_mma_kernel, grid, dim3(PD2_WARPS * 32), PD2_SMEM, st,
        reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<const __nv_bfloat16*>(kc),
        reinterpret_cast<const __nv_bfloat16*>(vc), block_table, max_blocks, ctx_len, sinks,
        reinterpret_cast<__nv_bfloat16*>(out), scratch, Hq, Hk, block_size, window, scale, nsplit, split_tokens,
        rot, theta, new_slots, reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(kc)),
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(vc)));
  } else
  paged_decode_kernel<128><<<grid, PD_THREADS, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<const __nv_bfloat16*>(kc),
      reinterpret_cast<const __nv_bfloat16*>(vc), block_table, max_blocks, ctx_len, sinks,
      reinterpret_cast<__nv_bfloat16*>(out), scratch, Hq, Hk, block_size, window, scale, nsplit);
  if (nsplit > 1) {
    launch_k(paged_decode_combine_kernel<128>, dim3(B, Hq), dim3(128), 0, st, scratch, sinks, ctx_len, window,
                                                                  reinterpret_cast<__nv_bfloat16*>(out), Hq, nsplit,
                                                                  split_tokens);
  }
  return launch_status();
}

GK_EXPORT int gk_paged_decode(const void* q, const void* kc, const void* vc, const int* block_table,
                              const int* ctx_len, const float* sinks, void* out, float* scratch, int B, int Hq,
                              int Hk, int D, int block_size, int max_blocks, int max_ctx, float scale, int window,
                              int q_stride, void* stream) {
  return paged_decode_impl(q, kc, vc, block_table, ctx_len, sinks, out, scratch, B, Hq, Hk, D, block_size, max_blocks,
                           max_ctx, scale, window, q_stride, 0, 0.f, nullptr, stream);
}

// Decode attention straight on the packed, not yet rotated [q | k | v] rows of the QKV projection: rotary embedding,
// the append of the new key / value to the cache (slot new_slots[b], negative = no store) and the attention in one
// launch.  Tensor-core kernel only (GQA groups of up to 8 heads); rot = rotated dims (a multiple of 16, <= D).
GK_EXPORT int gk_paged_decode_append(void* qkv, void* kc, void* vc, const int* block_table, const int* ctx_len,
                                     const int* new_slots, const float* sinks, void* out, float* scratch, int B,
                                     int Hq, int Hk, int D, int block_size, int max_blocks, int max_ctx, float scale,
                                     int window, int q_stride, int rot, float theta, void* stream) {
  if (rot <= 0) return -4;
  return paged_decode_impl(qkv, kc, vc, block_table, ctx_len, sinks, out, scratch, B, Hq, Hk, D, block_size,
                           max_blocks, max_ctx, scale, window, q_stride, rot, theta, new_slots, stream);
}
