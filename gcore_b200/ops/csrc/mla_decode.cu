// Multi-head latent attention, one query token per request, on the paged latent cache (absorbed form): every cached
// token is one row [kv_lora | rope] shared by all heads, the query of a head is [q_nope W_uk | q_rope] and the output
// is the probability-weighted sum of the kv_lora part of the rows (the value up-projection follows outside).  A step
// reads kv_lora + rope values per cached token, whatever the head count, so the kernel is the multi-query case with
// a 576-wide score contraction and a 512-wide value: heads are the M rows of the tensor-core tiles.
//
// A CTA serves (request, group of 16 heads, KV split).  Per 32-token tile:
//   * the rows arrive with 16-byte cp.async through the block table into chunk-swizzled shared memory (two buffers:
//     the next tile streams in while this one is used);
//   * the score contraction is split over the four warps by k-step (the query fragments of a warp's k-steps stay in
//     registers for the whole kernel), the four partial 16 x 32 score tiles are summed through shared memory;
//   * every warp runs the online softmax on the summed tile (identical in all four: no exchange of running max / sum)
//     and multiplies the probabilities, re-packed in registers as an A operand, with its quarter of the value columns.
//     (Evaluating each exponential once and passing P through shared memory costs a third barrier per tile and
//     measured 5 % slower: the kernel is bound by issue latency at two warps per scheduler, not by the exponentials.)
// Stands in for the latent decode kernels the reference reaches through its serving engines and its own
// gpatch_v4/models/deepseek_v4/kernel/flash_mla_wrapper.py:56-160.
#include "host_utils.h"
#include <cuda_bf16.h>
#include <float.h>

namespace gkmla {

using gk::launch_k;
using gk::launch_status;
using gk::pdl_launch_dependents;
using gk::pdl_wait;

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int TILE = 32;        // tokens per shared-memory tile
constexpr int HEADS = 16;       // heads per CTA: the M rows of one mma.sync tile
constexpr int MIN_SPLIT = 128;  // finest KV split
constexpr int SP_STRIDE = 40;   // floats per row of the partial-score exchange (8 mod 32: conflict-free float2)

inline int& target_ctas() {
  static int n = 296;   // two CTAs fit an SM
  return n;
}

template <int CV, int DR>
struct Geo {
  static constexpr int ROW = CV + DR;
  static constexpr int CHUNKS = ROW / 8;                           // 16-byte chunks of a row
  static constexpr int ROW_BYTES = (ROW * 2 + 127) / 128 * 128;    // shared-memory row stride (swizzle stays inside)
  static constexpr int KSTEPS = ROW / 16;
  static constexpr int KS_PER_WARP = (KSTEPS + WARPS - 1) / WARPS;
  static constexpr int COLS_PER_WARP = CV / WARPS;
  static constexpr int NT = COLS_PER_WARP / 8;                     // 8-wide output tiles per warp
  static constexpr int Q_BYTES = HEADS * ROW_BYTES;
  static constexpr int TILE_BYTES = TILE * ROW_BYTES;
  static constexpr int SP_BYTES = WARPS * HEADS * SP_STRIDE * 4;
  static constexpr int SMEM = Q_BYTES + 2 * TILE_BYTES + SP_BYTES;
  static_assert(ROW % 16 == 0 && CV % 64 == 0 && DR % 8 == 0, "unsupported latent geometry");
};

// 16-byte chunk `ch` of row `row`: the low three chunk bits are xor-ed with the row so that the eight rows of an
// ldmatrix land in eight different 16-byte lanes of a 128-byte line
__device__ __forceinline__ uint32_t swz(int row, int ch, int row_bytes) {
  return static_cast<uint32_t>(row * row_bytes + (((ch & ~7) | ((ch ^ row) & 7)) << 4));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// q_lat [B, H, CV] and q_rope [B, H, DR] and out [B, H, CV] are addressed through (batch, head) strides in elements,
// so the batched projections around the kernel can keep their head-major layout.
template <int CV, int DR>
__global__ void __launch_bounds__(THREADS, 2) mla_paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q_lat, long long qs_b, long long qs_h, const __nv_bfloat16* __restrict__ q_rope,
    long long rs_b, long long rs_h, const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table,
    int max_blocks, const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, long long os_b, long long os_h,
    float* __restrict__ scratch, int H, int block_size, float scale, int nsplit, int split_tokens) {
  using G = Geo<CV, DR>;
  extern __shared__ __align__(128) uint8_t mla_smem[];
  uint8_t* sq = mla_smem;
  uint8_t* tiles = mla_smem + G::Q_BYTES;
  float* sp = reinterpret_cast<float*>(tiles + 2 * G::TILE_BYTES);

  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, hg = blockIdx.y, split = blockIdx.z;
  const int len = ctx_len[b];
  const int s0 = split * split_tokens;
  if (split > 0 && s0 >= len) return;   // the combine kernel reads the live splits only
  int s1 = s0 + split_tokens;
  if (s1 > len) s1 = len;
  const int ntiles = s1 > s0 ? (s1 - s0 + TILE - 1) / TILE : 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sqs = static_cast<uint32_t>(__cvta_generic_to_shared(sq));
  const uint32_t tls = static_cast<uint32_t>(__cvta_generic_to_shared(tiles));

  // a warp fetches rows 8*warp .. 8*warp+7 of a tile; lane r < 8 looks up the cache slot of row r
  auto tile_slot = [&](int t) -> long long {
    const int tok = s0 + t * TILE + warp * 8 + (lane & 7);
    if (t >= ntiles || tok >= s1) return -1;
    return static_cast<long long>(block_table[static_cast<long long>(b) * max_blocks + tok / block_size]) * block_size +
           tok % block_size;
  };
  auto request_tile = [&](int t, long long slot_lane) {
    const uint32_t base = tls + (t & 1) * G::TILE_BYTES;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const long long slot = __shfl_sync(0xffffffff, slot_lane, r);
      const int row = warp * 8 + r;
      const uint32_t nbytes = slot >= 0 ? 16u : 0u;   // rows past the end are zero-filled
      const __nv_bfloat16* src = cache + (slot >= 0 ? slot : 0) * G::ROW;
#pragma unroll
      for (int c0 = 0; c0 < G::CHUNKS; c0 += 32) {
        const int c = c0 + lane;
        if (c < G::CHUNKS) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(base + swz(row, c, G::ROW_BYTES)),
                       "l"(src + c * 8), "r"(nbytes) : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (ntiles > 0) request_tile(0, tile_slot(0));
  long long next_slot = tile_slot(1);

  // the query rows of this head group as one [16, CV + DR] tile (heads past H are zero rows)
  for (int i = tid; i < HEADS * G::CHUNKS; i += THREADS) {
    const int g = i / G::CHUNKS, c = i - g * G::CHUNKS;
    const int h = hg * HEADS + g;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h < H) {
      v = c < CV / 8 ? *reinterpret_cast<const uint4*>(q_lat + b * qs_b + h * qs_h + c * 8)
                     : *reinterpret_cast<const uint4*>(q_rope + b * rs_b + h * rs_h + (c - CV / 8) * 8);
    }
    *reinterpret_cast<uint4*>(sq + swz(g, c, G::ROW_BYTES)) = v;
  }
  __syncthreads();
  // this warp's k-steps are warp, warp + 4, ...: their A fragments stay in registers
  uint32_t qa[G::KS_PER_WARP][4];
#pragma unroll
  for (int i = 0; i < G::KS_PER_WARP; ++i) {
    const int ks = warp + i * WARPS;
    if (ks < G::KSTEPS) {
      const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
      ldsm_x4(qa[i], sqs + swz(row, ks * 2 + (lane >> 4), G::ROW_BYTES));
    } else {
      qa[i][0] = qa[i][1] = qa[i][2] = qa[i][3] = 0u;
    }
  }

  const int r0 = lane >> 2;        // accumulator rows r0 and r0 + 8
  const int cq = (lane & 3) * 2;   // first of the two columns inside an 8-wide tile
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};
  float o[G::NT][4];
#pragma unroll
  for (int j = 0; j < G::NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

#pragma unroll 1
  for (int t = 0; t < ntiles; ++t) {
    const int nt = s1 - (s0 + t * TILE) < TILE ? s1 - (s0 + t * TILE) : TILE;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();   // tile t is complete for every thread, and nobody still reads tile t - 1 or the exchange
    if (t + 1 < ntiles) request_tile(t + 1, next_slot);
    next_slot = tile_slot(t + 2);
    const uint32_t tb = tls + (t & 1) * G::TILE_BYTES;

    // ---- partial S = Q K^T over this warp's k-steps: 4 token tiles of 8
    float sc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
    for (int i = 0; i < G::KS_PER_WARP; ++i) {
      const int ks = warp + i * WARPS;
      if (ks < G::KSTEPS) {
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {   // pairs of token tiles
          uint32_t kb[4];
          const int id = lane >> 3;
          const int row = (jp * 2 + (id >> 1)) * 8 + (lane & 7);
          ldsm_x4(kb, tb + swz(row, ks * 2 + (id & 1), G::ROW_BYTES));
          mma_16816(sc[jp * 2], qa[i], kb[0], kb[1]);
          mma_16816(sc[jp * 2 + 1], qa[i], kb[2], kb[3]);
        }
      }
    }
    float* mine = sp + warp * HEADS * SP_STRIDE;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      *reinterpret_cast<float2*>(mine + r0 * SP_STRIDE + j * 8 + cq) = make_float2(sc[j][0], sc[j][1]);
      *reinterpret_cast<float2*>(mine + (r0 + 8) * SP_STRIDE + j * 8 + cq) = make_float2(sc[j][2], sc[j][3]);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* p = sp + w * HEADS * SP_STRIDE;
        const float2 a = *reinterpret_cast<const float2*>(p + r0 * SP_STRIDE + j * 8 + cq);
        const float2 c = *reinterpret_cast<const float2*>(p + (r0 + 8) * SP_STRIDE + j * 8 + cq);
        lo.x += a.x; lo.y += a.y; hi.x += c.x; hi.y += c.y;
      }
      sc[j][0] = lo.x; sc[j][1] = lo.y; sc[j][2] = hi.x; sc[j][3] = hi.y;
    }

    // ---- online softmax of rows r0 (elements 0, 1) and r0 + 8 (elements 2, 3)
    float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ti = j * 8 + cq + (e & 1);
        const float v = ti < nt ? sc[j][e] * scale : -FLT_MAX;
        sc[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float resc[2], m_new[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffff, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffff, mx[h], 2));
      m_new[h] = fmaxf(m_run[h], mx[h]);
      resc[h] = m_run[h] == -FLT_MAX ? 0.f : __expf(m_run[h] - m_new[h]);
      m_run[h] = m_new[h];
      l_run[h] *= resc[h];
    }
    // once the running maxima have settled (after the first tiles of a long context) no row of the warp moves and
    // the pass over the accumulators is skipped
    if (__any_sync(0xffffffff, resc[0] != 1.f || resc[1] != 1.f)) {
#pragma unroll
      for (int j = 0; j < G::NT; ++j) { o[j][0] *= resc[0]; o[j][1] *= resc[0]; o[j][2] *= resc[1]; o[j][3] *= resc[1]; }
    }
    uint32_t pa[2][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = sc[j][e] == -FLT_MAX ? 0.f : __expf(sc[j][e] - m_new[e >> 1]);
        l_run[e >> 1] += p[e];
      }
      // A fragment of k-step j / 2: {rows lo cols lo, rows hi cols lo, rows lo cols hi, rows hi cols hi}
      pa[j >> 1][(j & 1) * 2] = pack2(p[0], p[1]);
      pa[j >> 1][(j & 1) * 2 + 1] = pack2(p[2], p[3]);
    }

    // ---- O += P V on this warp's quarter of the value columns: 2 k-steps of 16 tokens
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int np = 0; np < G::NT / 2; ++np) {
        uint32_t vb[4];
        const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int ch = warp * (G::COLS_PER_WARP / 8) + np * 2 + (lane >> 4);
        ldsm_x4_trans(vb, tb + swz(row, ch, G::ROW_BYTES));
        mma_16816(o[2 * np], pa[kk], vb[0], vb[1]);
        mma_16816(o[2 * np + 1], pa[kk], vb[2], vb[3]);
      }
    }
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffff, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffff, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int head = hg * HEADS + r0 + h * 8;
    if (head >= H) continue;
    const int col0 = warp * G::COLS_PER_WARP + cq;
    if (nsplit == 1) {
      const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
      __nv_bfloat16* dst = out + b * os_b + head * os_h + col0;
#pragma unroll
      for (int j = 0; j < G::NT; ++j) {
        *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) =
            __floats2bfloat162_rn(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
      }
    } else {
      float* dst = scratch + ((static_cast<long long>(b) * H + head) * nsplit + split) * (CV + 2);
#pragma unroll
      for (int j = 0; j < G::NT; ++j) {
        *reinterpret_cast<float2*>(dst + col0 + j * 8) = make_float2(o[j][2 * h], o[j][2 * h + 1]);
      }
      if (warp == 0 && (lane & 3) == 0) { dst[CV] = m_run[h]; dst[CV + 1] = l_run[h]; }
    }
  }
}

// Merges the live KV splits of one (request, head): scratch rows are [CV values | running max | running sum].
__global__ void mla_decode_combine_kernel(const float* __restrict__ scratch, const int* __restrict__ ctx_len,
                                          __nv_bfloat16* __restrict__ out, long long os_b, long long os_h, int H,
                                          int CV, int nsplit_total, int split_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const float* base = scratch + (static_cast<long long>(b) * H + h) * nsplit_total * (CV + 2);
  int nsplit = (ctx_len[b] + split_tokens - 1) / split_tokens;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > nsplit_total) nsplit = nsplit_total;
  float m = -FLT_MAX;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, base[s * (CV + 2) + CV]);
  float l = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = base[s * (CV + 2) + CV];
    l += base[s * (CV + 2) + CV + 1] * (ms == -FLT_MAX ? 0.f : __expf(ms - m));
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < CV; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = base[s * (CV + 2) + CV];
      acc += base[s * (CV + 2) + d] * (ms == -FLT_MAX ? 0.f : __expf(ms - m));
    }
    out[b * os_b + h * os_h + d] = __float2bfloat16(acc * inv);
  }
}

// KV splits for a launch: about one wave of CTAs, never finer than MIN_SPLIT tokens.  Depends only on host values
// (the launch shape is fixed for a CUDA graph).
static void plan(int B, int H, int max_ctx, int* nsplit, int* split_tokens) {
  const int groups = B * ((H + HEADS - 1) / HEADS);
  int ns = (max_ctx + MIN_SPLIT - 1) / MIN_SPLIT;
  if (ns < 1) ns = 1;
  int want = target_ctas() / (groups > 0 ? groups : 1);
  if (want < 1) want = 1;
  if (want < ns) ns = want;
  int st = ((max_ctx + ns - 1) / ns + TILE - 1) / TILE * TILE;
  if (st < MIN_SPLIT) st = MIN_SPLIT;
  ns = (max_ctx + st - 1) / st;
  if (ns < 1) ns = 1;
  *nsplit = ns;
  *split_tokens = st;
}

template <int CV, int DR>
static int launch(const void* q_lat, long long qs_b, long long qs_h, const void* q_rope, long long rs_b,
                  long long rs_h, const void* cache, const int* block_table, int max_blocks, const int* ctx_len,
                  void* out, long long os_b, long long os_h, float* scratch, int B, int H, int block_size, float scale,
                  int nsplit, int split_tokens, cudaStream_t st) {
  using G = Geo<CV, DR>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(mla_paged_decode_kernel<CV, DR>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM);
    configured = true;
  }
  launch_k(mla_paged_decode_kernel<CV, DR>, dim3(B, (H + HEADS - 1) / HEADS, nsplit), dim3(THREADS), G::SMEM, st,
           reinterpret_cast<const __nv_bfloat16*>(q_lat), qs_b, qs_h, reinterpret_cast<const __nv_bfloat16*>(q_rope),
           rs_b, rs_h, reinterpret_cast<const __nv_bfloat16*>(cache), block_table, max_blocks, ctx_len,
           reinterpret_cast<__nv_bfloat16*>(out), os_b, os_h, scratch, H, block_size, scale, nsplit, split_tokens);
  return 0;
}

}  // namespace gkmla

using namespace gkmla;

GK_EXPORT void gk_mla_set_target_ctas(int n) { target_ctas() = n > 0 ? n : 296; }

// 1 when a kernel is built for this latent geometry
GK_EXPORT int gk_mla_decode_supported(int CV, int DR) {
  return (CV == 512 && DR == 64) || (CV == 256 && DR == 64) || (CV == 128 && DR == 32);
}

GK_EXPORT void gk_mla_decode_scratch(int B, int H, int CV, int max_ctx, long long* floats) {
  int ns, st;
  plan(B, H, max_ctx, &ns, &st);
  *floats = ns > 1 ? static_cast<long long>(B) * H * ns * (CV + 2) : 0;
}

// max_ctx bounds every ctx_len[b]; strides are in elements and must be multiples of 8 (16-byte query loads).
GK_EXPORT int gk_mla_paged_decode(const void* q_lat, long long qs_b, long long qs_h, const void* q_rope,
                                  long long rs_b, long long rs_h, const void* cache, const int* block_table,
                                  const int* ctx_len, void* out, long long os_b, long long os_h, float* scratch,
                                  int B, int H, int CV, int DR, int block_size, int max_blocks, int max_ctx,
                                  float scale, void* stream) {
  if (!gk_mla_decode_supported(CV, DR)) return -1;
  if ((qs_b | qs_h | rs_b | rs_h) % 8 || (os_b | os_h) % 2) return -3;
  if (B == 0 || H == 0) return 0;
  int nsplit, split_tokens;
  plan(B, H, max_ctx, &nsplit, &split_tokens);
  if (nsplit > 1 && !scratch) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define GK_MLA_ARGS q_lat, qs_b, qs_h, q_rope, rs_b, rs_h, cache, block_table, max_blocks, ctx_len, out, os_b, os_h, \
                    scratch, B, H, block_size, scale, nsplit, split_tokens, st
  if (CV == 512) launch<512, 64>(GK_MLA_ARGS);
  else if (CV == 256) launch<256, 64>(GK_MLA_ARGS);
  else launch<128, 32>(GK_MLA_ARGS);
#undef GK_MLA_ARGS
  if (nsplit > 1) {
    launch_k(mla_decode_combine_kernel, dim3(B, H), dim3(128), 0, st, static_cast<const float*>(scratch), ctx_len,
             reinterpret_cast<__nv_bfloat16*>(out), os_b, os_h, H, CV, nsplit, split_tokens);
  }
  return launch_status();
}
