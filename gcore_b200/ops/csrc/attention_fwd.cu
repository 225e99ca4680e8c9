// Flash-attention forward on tcgen05: varlen (cu_seqlens) GQA, causal or full, optional sliding window, optional
// learned per-head sink logit in the softmax denominator, prefix-K offset (q_offset = lk - lq).  Semantics follow
// the reference's TileLang kernels (gfused/myfa_varlen_sw_sinks.py:18-191, gfused/myfa_sw_sinks.py:21-190).
//
// One CTA = 128 query rows of one head.  S = Q K^T and O += P V run on the tensor core with fp32 accumulators in
// tensor memory; with M = 128 every TMEM lane is one query row, so each of the 128 softmax threads owns a whole
// row of S and needs no cross-thread reduction.
//
//   warps 0-3  softmax / O-correction / epilogue (thread t <-> query row t <-> TMEM lane t)
//   warp 4     TMA producer (Q once, then K_j / V_j into a 2-stage ring)
//   warp 5     MMA issuer: S_{j+1} is issued before P_j V_j so QK^T overlaps the softmax of the previous tile
//
// TMEM columns (256 allocated per CTA, two CTAs per SM): S buffers at [0,64) and [64,128), O at [128, 128 + D).
// With one CTA per SM the four softmax warps (one per scheduler) left every pipe under 35 % busy (ncu): the kernel was
// bound by the latency of each warp's dependent chain, so the tile is 64 keys wide and two CTAs interleave on an SM.
// P is written as bf16 into a 128-byte-swizzled K-major shared tile and consumed as the A operand of P V.
#include "ptx.cuh"
#include "host_utils.h"
#include <float.h>

namespace gk {

constexpr int FA_BM = 128;
constexpr int FA_BN = 64;   // keys per tile: 64 keeps a CTA at 112 KB of shared memory, so two CTAs share an SM
constexpr int FA_THREADS = 192;

struct FaParams {
  const int* cu_q;
  const int* cu_k;
  const float* sinks;   // [Hq] or null
  __nv_bfloat16* out;   // [Tq, Hq, D]
  long long o_stride_t;
  float* lse;           // [Hq, Tq_total]
  long long tq_total;
  int Hq, Hk;
  int causal, window;
  float scale;
  int* err;
};

// DQK = head dim of queries and keys, DV = head dim of values and of the output (equal except for multi-head latent
// attention expanded to per-head keys: 128 + 64 rotary dims against 128-wide values).
template <int DQK, int DV>
__global__ void __launch_bounds__(FA_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FaParams p) {
  constexpr int NCH = DQK / 64;            // 64-element (128-byte) chunks along the query / key head dim
  constexpr int NCHV = DV / 64;
  constexpr int TILE_BYTES = 128 * DQK * 2;    // the Q tile
  constexpr int K_BYTES = FA_BN * DQK * 2;     // one K tile
  constexpr int V_BYTES = FA_BN * DV * 2;      // one V tile
  constexpr int KV_CHUNK = FA_BN * 128;        // one 64-dim (128-byte) chunk of a K / V tile
  constexpr int P_BYTES = 128 * FA_BN * 2;
  // no alignment slack: two CTAs must fit in one SM.  The dynamic segment starts on a 1024-byte boundary when the
  // kernel has no static shared memory; checked below instead of assumed.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;    // 2 stages
  uint8_t* sV = sK + 2 * K_BYTES;   // 2 stages
  uint8_t* sP = sV + 2 * V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;         // 1
  uint64_t* k_full = bars + 1;     // 2
  uint64_t* v_full = bars + 3;     // 2
  uint64_t* kv_empty = bars + 5;   // 2
  uint64_t* s_full = bars + 7;     // 2
  uint64_t* s_empty = bars + 9;    // 2 (128 arrivals)
  uint64_t* p_full = bars + 11;    // 1 (128 arrivals)
  uint64_t* pv_done = bars + 12;   // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_beg = p.cu_q[b], lq = p.cu_q[b + 1] - q_beg;
  const int k_beg = p.cu_k[b], lk = p.cu_k[b + 1] - k_beg;
  const int q0 = qt * FA_BM;
  if (q0 >= lq) return;  // uniform across the CTA, before any allocation
  if (smem_u32(smem_raw) & 1023u) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_WAIT_MISC);
    return;
  }
  const int hk = h / (p.Hq / p.Hk);
  const int off = lk - lq;  // key index of query row i's diagonal is i + off
  const int q_hi = (q0 + FA_BM - 1 < lq - 1) ? q0 + FA_BM - 1 : lq - 1;
  int j_end = (lk + FA_BN - 1) / FA_BN;
  if (p.causal) {
    const int last_key = q_hi + off;
    const int je = last_key < 0 ? 0 : last_key / FA_BN + 1;
    if (je < j_end) j_end = je;
  }
  int j_beg = 0;
  if (p.window > 0) {
    const int first_key = q0 + off - p.window + 1;
    if (first_key > 0) j_beg = first_key / FA_BN;
  }
  const int ntiles = j_end > j_beg ? j_end - j_beg : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 5) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const uint32_t tmem_o = tmem_base + 2 * FA_BN;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (ntiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_3d(sQ + c * 16384, &tmQ, q_full, c * 64, h, q_beg + q0);
      }
      __syncwarp();
      bool ok = true;
      for (int it = 0; it < ntiles && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        ok = mbar_wait(&kv_empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          const int krow = k_beg + (j_beg + it) * FA_BN;
          mbar_expect_tx(&k_full[s], K_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c) tma_load_3d(sK + s * K_BYTES + c * KV_CHUNK, &tmK, &k_full[s], c * 64, hk, krow);
          mbar_expect_tx(&v_full[s], V_BYTES);
#pragma unroll
          for (int c = 0; c < NCHV; ++c) tma_load_3d(sV + s * V_BYTES + c * KV_CHUNK, &tmV, &v_full[s], c * 64, hk, krow);
        }
        __syncwarp();
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc(FA_BM, FA_BN, 1, 1, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(FA_BM, DV, 1, 1, 0, 1);
    bool ok = ntiles > 0;
    if (ok) ok = mbar_wait(q_full, 0, p.err, ERR_WAIT_FULL);
    auto issue_s = [&](int it) -> bool {
      const int s = it & 1;
      if (!mbar_wait(&k_full[s], (it >> 1) & 1, p.err, ERR_WAIT_FULL)) return false;
      if (it >= 2 && !mbar_wait(&s_empty[s], ((it - 2) >> 1) & 1, p.err, ERR_WAIT_TMEM_EMPTY)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + s * K_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < DQK / 16; ++k4) {
          const uint32_t oq = (k4 >> 2) * 16384 + (k4 & 3) * 32;     // Q chunks are 128 rows x 128 B apart
          const uint32_t okk = (k4 >> 2) * KV_CHUNK + (k4 & 3) * 32;  // K chunks FA_BN rows x 128 B
          umma_f16(tmem_base + s * FA_BN, make_smem_desc_sw128(qa + oq, 16, 1024),
                   make_smem_desc_sw128(ka + okk, 16, 1024), idesc_s, k4 > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_s(0);
    for (int it = 0; it < ntiles && ok; ++it) {
      const int s = it & 1;
      if (it + 1 < ntiles) {
        ok = issue_s(it + 1);
        if (!ok) break;
      }
      ok = mbar_wait(p_full, it & 1, p.err, ERR_WAIT_MISC);
      if (!ok) break;
      ok = mbar_wait(&v_full[s], (it >> 1) & 1, p.err, ERR_WAIT_FULL);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + s * V_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < FA_BN / 16; ++k4) {
          const uint64_t adesc = make_smem_desc_sw128(pa + (k4 >> 2) * 16384 + (k4 & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(va + k4 * 2048, KV_CHUNK, 1024);
          umma_f16(tmem_o, adesc, bdesc, idesc_pv, (it > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(pv_done);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int row = threadIdx.x;  // 0..127
    const int qi = q0 + row;      // query index inside the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    float m = -FLT_MAX, l = 0.f;
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int s = it & 1;
      ok = mbar_wait(&s_full[s], (it >> 1) & 1, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      float sv[FA_BN];
#pragma unroll
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_addr + s * FA_BN + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sv[c * 32 + j] = __uint_as_float(r[j]);
      }
      tc_fence_before();
      mbar_arrive(&s_empty[s]);
      // mask + row max
      const int kbase = (j_beg + it) * FA_BN;
      int hi = lk - 1;  // last visible key
      if (p.causal && qi + off < hi) hi = qi + off;
      int lo = 0;
      if (p.window > 0) { lo = qi + off - p.window + 1; if (lo < 0) lo = 0; }
      // row maximum of the raw scores; tiles that lie entirely inside this row's visible range skip the masking
      float mx = -FLT_MAX;
      if (kbase >= lo && kbase + FA_BN - 1 <= hi) {
#pragma unroll
        for (int j = 0; j < FA_BN; ++j) mx = fmaxf(mx, sv[j]);
      } else {
#pragma unroll
        for (int j = 0; j < FA_BN; ++j) {
          const int kj = kbase + j;
          const float v = (kj >= lo && kj <= hi) ? sv[j] : -FLT_MAX;
          sv[j] = v;
          mx = fmaxf(mx, v);
        }
      }
      mx = mx == -FLT_MAX ? -FLT_MAX : mx * sl2;  // to the log2 domain (sl2 > 0 keeps the ordering)
      // Lazy rescale: the running reference maximum only moves when the tile's maximum exceeds it by more than 2^8.
      // Probabilities then reach at most 256 (exact in fp32 accumulation, fine in bf16) and the read-scale-write of
      // the O accumulator in tensor memory, the most expensive step of the loop, is skipped on almost every tile.
      const float m_cand = fmaxf(m, mx);
      const bool grow = (m == -FLT_MAX) ? (m_cand != -FLT_MAX) : (m_cand > m + 8.f);
      const float m_new = grow ? m_cand : m;
      const float m_use = m_new == -FLT_MAX ? 0.f : m_new;
      const float corr = grow ? exp2f(m - m_use) : 1.f;  // m == -FLT_MAX on the first tile -> 0
      float ps = 0.f;
#pragma unroll
      for (int j = 0; j < FA_BN; ++j) {
        const float e = exp2f(fmaf(sv[j], sl2, -m_use));  // masked scores (-FLT_MAX) underflow to exactly 0
        sv[j] = e;
        ps += e;
      }
      l = l * corr + ps;
      const bool changed = grow;
      m = m_new;
      // previous P V must have retired before P is overwritten and O is rescaled
      if (it > 0) {
        ok = mbar_wait(pv_done, (it - 1) & 1, p.err, ERR_WAIT_MISC);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffff, changed)) {
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_o + lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
            tmem_st32(tmem_o + lane_addr + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // P (bf16) -> shared, K-major with the 128-byte swizzle: 16-byte unit u of row r sits at unit u ^ (r & 7)
#pragma unroll
      for (int c = 0; c < FA_BN / 64; ++c) {
        uint8_t* rowp = sP + c * 16384 + row * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          uint4 w;
          w.x = pack_bf16x2(sv[c * 64 + u * 8 + 0], sv[c * 64 + u * 8 + 1]);
          w.y = pack_bf16x2(sv[c * 64 + u * 8 + 2], sv[c * 64 + u * 8 + 3]);
          w.z = pack_bf16x2(sv[c * 64 + u * 8 + 4], sv[c * 64 + u * 8 + 5]);
          w.w = pack_bf16x2(sv[c * 64 + u * 8 + 6], sv[c * 64 + u * 8 + 7]);
          *reinterpret_cast<uint4*>(rowp + ((u ^ (row & 7)) << 4)) = w;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    // ---- epilogue
    if (ok && ntiles > 0) {
      ok = mbar_wait(pv_done, (ntiles - 1) & 1, p.err, ERR_WAIT_MISC);
      if (ok) tc_fence_after();
    }
    if (ok) {
      const float m_use = m == -FLT_MAX ? 0.f : m;
      if (p.sinks) l += exp2f(p.sinks[h] * 1.4426950408889634f - m_use);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool valid = qi < lq;
      __nv_bfloat16* orow = p.out + static_cast<long long>(q_beg + qi) * p.o_stride_t + static_cast<long long>(h) * DV;
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t r[32];
        if (ntiles > 0) {
          tmem_ld32(tmem_o + lane_addr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * inv, __uint_as_float(r[8 * j + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + j * 8) = w;
          }
        }
      }
      if (valid && p.lse) {
        p.lse[static_cast<long long>(h) * p.tq_total + q_beg + qi] =
            l > 0.f ? (m_use + log2f(l)) * 0.6931471805599453f : -FLT_MAX;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int DQK, int DV>
int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, dim3 grid,
              cudaStream_t st) {
  // 112 KB at 128 / 128 (two CTAs per SM), 144 KB at 192 / 128 (one)
  constexpr int SMEM = 128 * DQK * 2 + 2 * FA_BN * DQK * 2 + 2 * FA_BN * DV * 2 + 128 * FA_BN * 2 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<DQK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    // the whole L1 / shared array as shared memory, so that two CTAs fit
    cudaFuncSetAttribute(attn_fwd_kernel<DQK, DV>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  attn_fwd_kernel<DQK, DV><<<grid, FA_THREADS, SMEM, st>>>(tq, tk, tv, p);
  return launch_status();
}

}  // namespace gk

using namespace gk;

// q: [Tq, Hq, D], k: [Tk, Hk, D], v: [Tk, Hk, Dv] (token strides in elements, heads contiguous), out: [Tq, Hq, Dv].
// Dv = 0 means Dv = D; built geometries: 64 / 64, 128 / 128 and 192 / 128.
// cu_q / cu_k: int32 [B + 1] on device.  max_q bounds every sequence's query length (fixes the grid).
GK_EXPORT int gk_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q,
                          const int* cu_k, const float* sinks, int B, int Tq, int Tk, int Hq, int Hk, int D,
                          int max_q, int causal, float scale, int window, int Dv, void* strides,
                          void* stream_err) {
  // strides: long long[4] = {q_stride_t, k_stride_t, v_stride_t, o_stride_t}; stream_err: void*[2] = {stream, err}
  const long long* sd = reinterpret_cast<const long long*>(strides);
  void** se = reinterpret_cast<void**>(stream_err);
  if (Dv == 0) Dv = D;
  if (!((D == 64 && Dv == 64) || (D == 128 && Dv == 128) || (D == 192 && Dv == 128))) return -1;
  if (Hq % Hk) return -2;
  CUtensorMap tq, tk, tv;
  if (make_tmap_3d(&tq, q, 2, Tq, Hq, D, sd[0], D, 128, 1, 64, true)) return -3;
  if (make_tmap_3d(&tk, k, 2, Tk, Hk, D, sd[1], D, FA_BN, 1, 64, true)) return -4;
  if (make_tmap_3d(&tv, v, 2, Tk, Hk, Dv, sd[2], Dv, FA_BN, 1, 64, true)) return -5;
  FaParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.sinks = sinks;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.o_stride_t = sd[3];
  p.lse = lse; p.tq_total = Tq;
  p.Hq = Hq; p.Hk = Hk; p.causal = causal; p.window = window; p.scale = scale;
  p.err = reinterpret_cast<int*>(se[1]);
  dim3 grid((max_q + FA_BM - 1) / FA_BM, Hq, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(se[0]);
  if (D == 192) return launch_fa<192, 128>(tq, tk, tv, p, grid, st);
  if (D == 128) return launch_fa<128, 128>(tq, tk, tv, p, grid, st);
  return launch_fa<64, 64>(tq, tk, tv, p, grid, st);
}
