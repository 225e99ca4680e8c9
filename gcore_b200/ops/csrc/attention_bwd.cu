// Flash-attention backward on tcgen05, deterministic (no atomics): a delta pre-pass and two tensor-core kernels.
//
//   delta[h, t] = sum_d O[t, h, d] * dO[t, h, d]
//   dKdV kernel : one CTA per (128-key tile, query head, sequence), loops over 64-row query tiles
//                   S^T = K Q^T,  dP^T = V dO^T            (accumulators in TMEM, rows = keys)
//                   P^T = exp(S^T * scale - lse),  dS^T = P^T * (dP^T - delta)      (threads, one key row each)
//                   dV += P^T dO,  dK += dS^T Q            (A from shared memory, B = the same dO / Q tiles read
//                                                            MN-major)
//   dQ kernel   : one CTA per (128-query tile, head, sequence), loops over 64-key tiles
//                   S = Q K^T,  dP = dO V^T,  dS = P * (dP - delta),  dQ += dS K
//
// Gradients w.r.t. K and V are produced per query head ([Tk, Hq, D]) and summed over the GQA group by the caller,
// which keeps the result bit-reproducible (the reference's TileLang backward accumulates with fp32 atomics,
// gfused/myfa_varlen_sw_sinks.py:292-451).  Masking rules (causal, window, prefix offset) match the forward.
#include "ptx.cuh"
#include "host_utils.h"
#include <float.h>

namespace gk {

constexpr int FB_THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;

struct FbParams {
  const int* cu_q;
  const int* cu_k;
  const float* lse;     // [Hq, Tq]
  const float* delta;   // [Hq, Tq]
  __nv_bfloat16* dq;    // [Tq, Hq, D]
  __nv_bfloat16* dk;    // [Tk, Hq, D]  (per query head)
  __nv_bfloat16* dv;    // [Tk, Hq, D]
  long long tq_total;
  int Hq, Hk;
  int causal, window;
  float scale;
  int* err;
};

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_stride,
                                  const __nv_bfloat16* __restrict__ d_o, long long do_stride, float* __restrict__ delta,
                                  long long T, int Hq, int D) {
  // one warp per (token, head)
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * Hq) return;
  const long long t = w / Hq;
  const int h = static_cast<int>(w - t * Hq);
  const __nv_bfloat16* po = o + t * o_stride + static_cast<long long>(h) * D;
  const __nv_bfloat16* pd = d_o + t * do_stride + static_cast<long long>(h) * D;
  float s = 0.f;
  for (int i = lane; i < D; i += 32) s += __bfloat162float(po[i]) * __bfloat162float(pd[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffff, s, off);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

__device__ __forceinline__ bool visible(int qi, int kj, int off, int lq, int lk, int causal, int window) {
  if (qi >= lq || kj >= lk) return false;
  if (causal && kj > qi + off) return false;
  if (window > 0 && kj <= qi + off - window) return false;
  return true;
}

// Writes 32 consecutive bf16 values of row `row` (columns col0 .. col0+31, col0 in {0, 32}) into a K-major
// 128-byte-swizzled tile of 64 columns (row pitch 128 bytes).
__device__ __forceinline__ void store_row_chunk_sw128(uint8_t* tile, int row, int col0, const float (&v)[32]) {
  uint8_t* rowp = tile + row * 128;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    uint4 w;
    w.x = pack_bf16x2(v[u * 8 + 0], v[u * 8 + 1]);
    w.y = pack_bf16x2(v[u * 8 + 2], v[u * 8 + 3]);
    w.z = pack_bf16x2(v[u * 8 + 4], v[u * 8 + 5]);
    w.w = pack_bf16x2(v[u * 8 + 6], v[u * 8 + 7]);
    const int unit = (col0 >> 3) + u;
    *reinterpret_cast<uint4*>(rowp + ((unit ^ (row & 7)) << 4)) = w;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dK / dV.  Stationary: K, V tile of 128 keys.  Streamed: Q, dO tiles of 64 query rows (2 stages).
// DQK = head dim of Q / K / dK, DV = head dim of V / dO / dV.
// TMEM columns with equal head dims (<= 128): S^T buffers [0,64) [64,128), dP^T buffers [128,192) [192,256),
// dV [256, 256+DV), dK [384, 384+DQK).  The 192 / 128 instance has one S^T and one dP^T buffer (NT = 1), which is
// what fits beside a 192-column dK: S^T [0,64), dP^T [64,128), dV [128,256), dK [256,448); the scores of tile i+1
// are then issued once the threads have read tile i, and still overlap tile i's accumulate MMAs.
template <int DQK, int DV>
__global__ void __launch_bounds__(FB_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, FbParams p) {
  constexpr int NCH = DQK / 64;
  constexpr int NCHV = DV / 64;
  constexpr int NT = (256 + DV + DQK <= 512) ? 2 : 1;   // S^T / dP^T buffers in tensor memory
  constexpr int K_BYTES = 128 * DQK * 2;  // stationary tiles
  constexpr int V_BYTES = 128 * DV * 2;
  constexpr int Q_BYTES = 64 * DQK * 2;   // streamed tiles (64 rows): chunks of 8 KB
  constexpr int DO_BYTES = 64 * DV * 2;
  constexpr int PS_BYTES = 128 * 64 * 2;  // P^T / dS^T tile: 128 rows x 128 B
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + K_BYTES;
  uint8_t* sQ = sV + V_BYTES;            // 2 stages
  uint8_t* sDO = sQ + 2 * Q_BYTES;       // 2 stages
  uint8_t* sP = sDO + 2 * DO_BYTES;      // 2 buffers
  uint8_t* sDS = sP + 2 * PS_BYTES;      // 2 buffers
  float* s_lse = reinterpret_cast<float*>(sDS + 2 * PS_BYTES);  // [2][64]
  float* s_delta = s_lse + 128;                                  // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 128);
  uint64_t* kv_full = bars;        // 1
  uint64_t* qd_full = bars + 1;    // 2
  uint64_t* s_full = bars + 3;     // 2
  uint64_t* s_free = bars + 5;     // 2 (128 arrivals)
  uint64_t* pds_full = bars + 7;   // 2 (128 arrivals)
  uint64_t* acc_done = bars + 9;   // 2
  uint64_t* lse_full = bars + 11;  // 2 (64 arrivals)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_beg = p.cu_q[b], lq = p.cu_q[b + 1] - q_beg;
  const int k_beg = p.cu_k[b], lk = p.cu_k[b + 1] - k_beg;
  const int k0 = kt * 128;
  if (k0 >= lk) return;
  const int hk = h / (p.Hq / p.Hk);
  const int off = lk - lq;
  const int k1 = (k0 + 128 < lk) ? k0 + 128 : lk;
  // query tiles (64 rows) that can see this key tile
  int i_beg = 0, i_end = (lq + 63) / 64;
  if (p.causal) {
    const int first_q = k0 - off;
    if (first_q > 0) i_beg = first_q / 64;
  }
  if (p.window > 0) {
    const int last_q = (k1 - 1) - off + p.window - 1;  // largest query index that still sees key k1-1
    const int ie = last_q < 0 ? 0 : last_q / 64 + 1;
    if (ie < i_end) i_end = ie;
  }
  const int ntiles = i_end > i_beg ? i_end - i_beg : 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&pds_full[i], 128);
      mbar_init(&acc_done[i], 1);
      mbar_init(&lse_full[i], 64);
    }
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
  }
  if (warp == 5) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const uint32_t tmem_dp = tmem_base + NT * 64;
  const uint32_t tmem_dv = tmem_base + 2 * NT * 64, tmem_dk = tmem_dv + DV;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (ntiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(kv_full, K_BYTES + V_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_3d(sK + c * 16384, &tmK, kv_full, c * 64, hk, k_beg + k0);
#pragma unroll
        for (int c = 0; c < NCHV; ++c) tma_load_3d(sV + c * 16384, &tmV, kv_full, c * 64, hk, k_beg + k0);
      }
      __syncwarp();
      bool ok = true;
      for (int it = 0; it < ntiles && ok; ++it) {
        const int s = it & 1;
        if (it >= 2) ok = mbar_wait(&acc_done[s], ((it - 2) >> 1) & 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          const int qrow = q_beg + (i_beg + it) * 64;
          mbar_expect_tx(&qd_full[s], Q_BYTES + DO_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c) tma_load_3d(sQ + s * Q_BYTES + c * 8192, &tmQ, &qd_full[s], c * 64, h, qrow);
#pragma unroll
          for (int c = 0; c < NCHV; ++c)
            tma_load_3d(sDO + s * DO_BYTES + c * 8192, &tmDO, &qd_full[s], c * 64, h, qrow);
        }
        __syncwarp();
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_st = make_idesc(128, 64, 1, 1, 0, 0);  // [keys x q] = K-major x K-major
    constexpr uint32_t idesc_dv = make_idesc(128, DV, 1, 1, 0, 1);   // [keys x DV] = A(K-major over q) x B(MN-major)
    constexpr uint32_t idesc_dk = make_idesc(128, DQK, 1, 1, 0, 1);
    bool ok = ntiles > 0;
    if (ok) ok = mbar_wait(kv_full, 0, p.err, ERR_WAIT_FULL);
    auto issue_scores = [&](int it) -> bool {
      const int s = it & 1, ts = it % NT;
      if (!mbar_wait(&qd_full[s], (it >> 1) & 1, p.err, ERR_WAIT_FULL)) return false;
      if (it >= NT && !mbar_wait(&s_free[ts], ((it - NT) / NT) & 1, p.err, ERR_WAIT_TMEM_EMPTY)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
        const uint32_t qa = smem_u32(sQ + s * Q_BYTES), da = smem_u32(sDO + s * DO_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < DQK / 16; ++k4) {
          const uint32_t oa = (k4 >> 2) * 16384 + (k4 & 3) * 32;  // stationary tiles: 128-row chunks
          const uint32_t ob = (k4 >> 2) * 8192 + (k4 & 3) * 32;   // streamed tiles: 64-row chunks
          umma_f16(tmem_base + ts * 64, make_smem_desc_sw128(ka + oa, 16, 1024),
                   make_smem_desc_sw128(qa + ob, 16, 1024), idesc_st, k4 > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k4 = 0; k4 < DV / 16; ++k4) {
          const uint32_t oa = (k4 >> 2) * 16384 + (k4 & 3) * 32;
          const uint32_t ob = (k4 >> 2) * 8192 + (k4 & 3) * 32;
          umma_f16(tmem_dp + ts * 64, make_smem_desc_sw128(va + oa, 16, 1024),
                   make_smem_desc_sw128(da + ob, 16, 1024), idesc_st, k4 > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[ts]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_scores(0);
    for (int it = 0; it < ntiles && ok; ++it) {
      const int s = it & 1;
      if (it + 1 < ntiles) {
        ok = issue_scores(it + 1);
        if (!ok) break;
      }
      ok = mbar_wait(&pds_full[s], (it >> 1) & 1, p.err, ERR_WAIT_MISC);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t pa = smem_u32(sP + s * PS_BYTES), dsa = smem_u32(sDS + s * PS_BYTES);
        const uint32_t qa = smem_u32(sQ + s * Q_BYTES), da = smem_u32(sDO + s * DO_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < 64 / 16; ++k4) {  // contraction over the 64 query rows
          umma_f16(tmem_dv, make_smem_desc_sw128(pa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(da + k4 * 2048, 8192, 1024), idesc_dv, (it > 0 || k4 > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k4 = 0; k4 < 64 / 16; ++k4) {
          umma_f16(tmem_dk, make_smem_desc_sw128(dsa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(qa + k4 * 2048, 8192, 1024), idesc_dk, (it > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(&acc_done[s]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ P^T / dS^T (thread = key row) + epilogue
    const int row = threadIdx.x;
    const int kj = k0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int s = it & 1;
      const int q0 = (i_beg + it) * 64;
      if (it >= 2) {
        // tile it-2 is fully consumed once its accumulate MMAs retired: the P^T / dS^T buffer and the lse / delta
        // slots of this parity may be overwritten
        ok = mbar_wait(&acc_done[s], ((it - 2) >> 1) & 1, p.err, ERR_WAIT_MISC);
        if (!ok) break;
      }
      if (row < 64) {
        const int qi = q0 + row;
        const bool in = qi < lq;
        const long long idx = static_cast<long long>(h) * p.tq_total + q_beg + qi;
        // log2-domain lse; rows without any visible key (or past the sequence) get +FLT_MAX so that their
        // probabilities evaluate to exp2(-huge) = 0 without a branch
        const float l = in ? p.lse[idx] : -FLT_MAX;
        s_lse[s * 64 + row] = l != -FLT_MAX ? l * LOG2E : FLT_MAX;
        s_delta[s * 64 + row] = in ? p.delta[idx] : 0.f;
        mbar_arrive(&lse_full[s]);
      }
      ok = mbar_wait(&lse_full[s], (it >> 1) & 1, p.err, ERR_WAIT_MISC);
      if (!ok) break;
      const int ts = it % NT;
      ok = mbar_wait(&s_full[ts], (it / NT) & 1, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      // interior tile for this warp's 32 keys: every (query, key) pair is visible, no mask arithmetic needed
      const int kmin = k0 + warp * 32, kmax = kmin + 31;
      const bool interior = kmax < lk && q0 + 63 < lq && (!p.causal || kmax <= q0 + off) &&
                            (p.window <= 0 || kmin > q0 + 63 + off - p.window);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem_base + lane_addr + ts * 64 + c * 32, rs);
        tmem_ld32(tmem_dp + lane_addr + ts * 64 + c * 32, rp);
        tmem_ld_wait();
        float pv[32], dsv[32];
        const float4* l4 = reinterpret_cast<const float4*>(s_lse + s * 64 + c * 32);
        const float4* d4 = reinterpret_cast<const float4*>(s_delta + s * 64 + c * 32);
        if (interior) {
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 l = l4[j4], d = d4[j4];
            const float lv[4] = {l.x, l.y, l.z, l.w}, dv[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = j4 * 4 + u;
              const float pe = exp2f(fmaf(__uint_as_float(rs[j]), sl2, -lv[u]));
              pv[j] = pe;
              dsv[j] = pe * (__uint_as_float(rp[j]) - dv[u]);
            }
          }
        } else {
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 l = l4[j4], d = d4[j4];
            const float lv[4] = {l.x, l.y, l.z, l.w}, dv[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = j4 * 4 + u;
              const bool vis = visible(q0 + c * 32 + j, kj, off, lq, lk, p.causal, p.window);
              const float pe = vis ? exp2f(fmaf(__uint_as_float(rs[j]), sl2, -lv[u])) : 0.f;
              pv[j] = pe;
              dsv[j] = pe * (__uint_as_float(rp[j]) - dv[u]);
            }
          }
        }
        store_row_chunk_sw128(sP + s * PS_BYTES, row, c * 32, pv);
        store_row_chunk_sw128(sDS + s * PS_BYTES, row, c * 32, dsv);
      }
      tc_fence_before();
      mbar_arrive(&s_free[ts]);
      fence_proxy_async();
      mbar_arrive(&pds_full[s]);
    }
    if (ok && ntiles > 0) {
      ok = mbar_wait(&acc_done[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, p.err, ERR_WAIT_MISC);
      if (ok) tc_fence_after();
    }
    if (ok) {
      const bool valid = kj < lk;
      const long long orow = static_cast<long long>(k_beg + kj) * p.Hq + h;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = which == 0 ? p.dv + orow * DV : p.dk + orow * DQK;
        const uint32_t tbase = (which == 0 ? tmem_dv : tmem_dk) + lane_addr;
        const float mul = which == 0 ? 1.f : p.scale;
#pragma unroll
        for (int c = 0; c < (which == 0 ? DV : DQK) / 32; ++c) {
          uint32_t r[32];
          if (ntiles > 0) {
            tmem_ld32(tbase + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          if (valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * mul, __uint_as_float(r[8 * j + 1]) * mul);
              w.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * mul, __uint_as_float(r[8 * j + 3]) * mul);
              w.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * mul, __uint_as_float(r[8 * j + 5]) * mul);
              w.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * mul, __uint_as_float(r[8 * j + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dQ.  Stationary: Q, dO tile of 128 query rows.  Streamed: K, V tiles of 64 keys (2 stages).
// TMEM columns: S buffers [0,64) [64,128), dP buffers [128,192) [192,256), dQ [256, 256+DQK).
template <int DQK, int DV>
__global__ void __launch_bounds__(FB_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, FbParams p) {
  constexpr int NCH = DQK / 64;
  constexpr int NCHV = DV / 64;
  constexpr int Q_BYTES = 128 * DQK * 2;
  constexpr int DO_BYTES = 128 * DV * 2;
  constexpr int K_BYTES = 64 * DQK * 2;
  constexpr int V_BYTES = 64 * DV * 2;
  constexpr int DS_BYTES = 128 * 64 * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + Q_BYTES;
  uint8_t* sK = sDO + DO_BYTES;        // 2 stages
  uint8_t* sV = sK + 2 * K_BYTES;      // 2 stages
  uint8_t* sDS = sV + 2 * V_BYTES;     // 2 buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * DS_BYTES);
  uint64_t* q_full = bars;         // 1
  uint64_t* kv_full = bars + 1;    // 2
  uint64_t* s_full = bars + 3;     // 2
  uint64_t* s_free = bars + 5;     // 2 (128)
  uint64_t* ds_full = bars + 7;    // 2 (128)
  uint64_t* acc_done = bars + 9;   // 2
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_beg = p.cu_q[b], lq = p.cu_q[b + 1] - q_beg;
  const int k_beg = p.cu_k[b], lk = p.cu_k[b + 1] - k_beg;
  const int q0 = qt * 128;
  if (q0 >= lq) return;
  const int hk = h / (p.Hq / p.Hk);
  const int off = lk - lq;
  const int q_hi = (q0 + 127 < lq - 1) ? q0 + 127 : lq - 1;
  int j_end = (lk + 63) / 64;
  if (p.causal) {
    const int last_key = q_hi + off;
    const int je = last_key < 0 ? 0 : last_key / 64 + 1;
    if (je < j_end) j_end = je;
  }
  int j_beg = 0;
  if (p.window > 0) {
    const int first_key = q0 + off - p.window + 1;
    if (first_key > 0) j_beg = first_key / 64;
  }
  const int ntiles = j_end > j_beg ? j_end - j_beg : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&ds_full[i], 128);
      mbar_init(&acc_done[i], 1);
    }
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
  }
  if (warp == 5) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const uint32_t tmem_dq = tmem_base + 256;

  if (warp == 4) {
    if (ntiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, Q_BYTES + DO_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_3d(sQ + c * 16384, &tmQ, q_full, c * 64, h, q_beg + q0);
#pragma unroll
        for (int c = 0; c < NCHV; ++c) tma_load_3d(sDO + c * 16384, &tmDO, q_full, c * 64, h, q_beg + q0);
      }
      __syncwarp();
      bool ok = true;
      for (int it = 0; it < ntiles && ok; ++it) {
        const int s = it & 1;
        if (it >= 2) ok = mbar_wait(&acc_done[s], ((it - 2) >> 1) & 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          const int krow = k_beg + (j_beg + it) * 64;
          mbar_expect_tx(&kv_full[s], K_BYTES + V_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c) tma_load_3d(sK + s * K_BYTES + c * 8192, &tmK, &kv_full[s], c * 64, hk, krow);
#pragma unroll
          for (int c = 0; c < NCHV; ++c) tma_load_3d(sV + s * V_BYTES + c * 8192, &tmV, &kv_full[s], c * 64, hk, krow);
        }
        __syncwarp();
      }
    }
  } else if (warp == 5) {
    constexpr uint32_t idesc_s = make_idesc(128, 64, 1, 1, 0, 0);
    constexpr uint32_t idesc_dq = make_idesc(128, DQK, 1, 1, 0, 1);
    bool ok = ntiles > 0;
    if (ok) ok = mbar_wait(q_full, 0, p.err, ERR_WAIT_FULL);
    auto issue_scores = [&](int it) -> bool {
      const int s = it & 1;
      if (!mbar_wait(&kv_full[s], (it >> 1) & 1, p.err, ERR_WAIT_FULL)) return false;
      if (it >= 2 && !mbar_wait(&s_free[s], ((it - 2) >> 1) & 1, p.err, ERR_WAIT_TMEM_EMPTY)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t qa = smem_u32(sQ), da = smem_u32(sDO);
        const uint32_t ka = smem_u32(sK + s * K_BYTES), va = smem_u32(sV + s * V_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < DQK / 16; ++k4) {
          const uint32_t oa = (k4 >> 2) * 16384 + (k4 & 3) * 32;
          const uint32_t ob = (k4 >> 2) * 8192 + (k4 & 3) * 32;
          umma_f16(tmem_base + s * 64, make_smem_desc_sw128(qa + oa, 16, 1024),
                   make_smem_desc_sw128(ka + ob, 16, 1024), idesc_s, k4 > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k4 = 0; k4 < DV / 16; ++k4) {
          const uint32_t oa = (k4 >> 2) * 16384 + (k4 & 3) * 32;
          const uint32_t ob = (k4 >> 2) * 8192 + (k4 & 3) * 32;
          umma_f16(tmem_base + 128 + s * 64, make_smem_desc_sw128(da + oa, 16, 1024),
                   make_smem_desc_sw128(va + ob, 16, 1024), idesc_s, k4 > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_scores(0);
    for (int it = 0; it < ntiles && ok; ++it) {
      const int s = it & 1;
      if (it + 1 < ntiles) {
        ok = issue_scores(it + 1);
        if (!ok) break;
      }
      ok = mbar_wait(&ds_full[s], (it >> 1) & 1, p.err, ERR_WAIT_MISC);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t dsa = smem_u32(sDS + s * DS_BYTES), ka = smem_u32(sK + s * K_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < 64 / 16; ++k4) {  // contraction over the 64 keys
          umma_f16(tmem_dq, make_smem_desc_sw128(dsa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(ka + k4 * 2048, 8192, 1024), idesc_dq, (it > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(&acc_done[s]);
      }
      __syncwarp();
    }
  } else {
    const int row = threadIdx.x;
    const int qi = q0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    const bool in = qi < lq;
    const long long idx = static_cast<long long>(h) * p.tq_total + q_beg + qi;
    const float lse = in ? p.lse[idx] : -FLT_MAX;
    const float delta = in ? p.delta[idx] : 0.f;
    // rows without any visible key get +FLT_MAX: their probabilities evaluate to exp2(-huge) = 0
    const float lse2 = lse != -FLT_MAX ? lse * LOG2E : FLT_MAX;
    const int qmin = q0 + warp * 32, qmax = qmin + 31;
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int s = it & 1;
      const int kbase = (j_beg + it) * 64;
      if (it >= 2) {
        ok = mbar_wait(&acc_done[s], ((it - 2) >> 1) & 1, p.err, ERR_WAIT_MISC);
        if (!ok) break;
      }
      ok = mbar_wait(&s_full[s], (it >> 1) & 1, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      // interior tile for this warp's 32 queries: every pair visible, no mask arithmetic needed
      const bool interior = qmax < lq && kbase + 63 < lk && (!p.causal || kbase + 63 <= qmin + off) &&
                            (p.window <= 0 || kbase > qmax + off - p.window);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem_base + lane_addr + s * 64 + c * 32, rs);
        tmem_ld32(tmem_base + lane_addr + 128 + s * 64 + c * 32, rp);
        tmem_ld_wait();
        float dsv[32];
        if (interior) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float pe = exp2f(fmaf(__uint_as_float(rs[j]), sl2, -lse2));
            dsv[j] = pe * (__uint_as_float(rp[j]) - delta);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int kj = kbase + c * 32 + j;
            const bool vis = visible(qi, kj, off, lq, lk, p.causal, p.window);
            const float pe = vis ? exp2f(fmaf(__uint_as_float(rs[j]), sl2, -lse2)) : 0.f;
            dsv[j] = pe * (__uint_as_float(rp[j]) - delta);
          }
        }
        store_row_chunk_sw128(sDS + s * DS_BYTES, row, c * 32, dsv);
      }
      tc_fence_before();
      mbar_arrive(&s_free[s]);
      fence_proxy_async();
      mbar_arrive(&ds_full[s]);
    }
    if (ok && ntiles > 0) {
      ok = mbar_wait(&acc_done[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, p.err, ERR_WAIT_MISC);
      if (ok) tc_fence_after();
    }
    if (ok) {
      __nv_bfloat16* dst = p.dq + (static_cast<long long>(q_beg + qi) * p.Hq + h) * DQK;
#pragma unroll
      for (int c = 0; c < DQK / 32; ++c) {
        uint32_t r[32];
        if (ntiles > 0) {
          tmem_ld32(tmem_dq + lane_addr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (in) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * p.scale, __uint_as_float(r[8 * j + 1]) * p.scale);
            w.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * p.scale, __uint_as_float(r[8 * j + 3]) * p.scale);
            w.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * p.scale, __uint_as_float(r[8 * j + 5]) * p.scale);
            w.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * p.scale, __uint_as_float(r[8 * j + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DQK, int DV>
int launch_bwd(const CUtensorMap& q128, const CUtensorMap& q64, const CUtensorMap& k128, const CUtensorMap& k64,
               const CUtensorMap& v128, const CUtensorMap& v64, const CUtensorMap& do128, const CUtensorMap& do64,
               const FbParams& p, int B, int max_q, int max_k, cudaStream_t st) {
  // stationary + 2 streamed stages of each operand, P^T / dS^T buffers, lse / delta slots, alignment slack, barriers:
  // 226.25 KB for 192 / 128 (of 227 KB), 194.25 KB for 128 / 128
  constexpr int SMEM1 = (128 + 2 * 64) * (DQK + DV) * 2 + 4 * 128 * 64 * 2 + 1024 + 1024 + 256;
  constexpr int SMEM2 = (128 + 2 * 64) * (DQK + DV) * 2 + 2 * 128 * 64 * 2 + 1024 + 256;
  static_assert(SMEM1 <= 232448, "dK/dV kernel exceeds the shared memory of an SM");
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(attn_bwd_dkdv_kernel<DQK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM1);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_bwd_dq_kernel<DQK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 g1((max_k + 127) / 128, p.Hq, B);
  attn_bwd_dkdv_kernel<DQK, DV><<<g1, FB_THREADS, SMEM1, st>>>(q64, k128, v128, do64, p);
  dim3 g2((max_q + 127) / 128, p.Hq, B);
  attn_bwd_dq_kernel<DQK, DV><<<g2, FB_THREADS, SMEM2, st>>>(q128, k64, v64, do128, p);
  return launch_status();
}

}  // namespace gk

using namespace gk;

// q / k: [T, H, D], v / out: [T, H, Dv] with token strides given in `strides` = {q, k, v, out} (elements); `d_o` is
// contiguous ([Tq, Hq, Dv]).  dq [Tq, Hq, D], dk_h [Tk, Hq, D], dv_h [Tk, Hq, Dv] contiguous outputs; delta [Hq, Tq]
// scratch.  Dv = 0 means Dv = D; built geometries: 64 / 64, 128 / 128, 192 / 128.
// dsink is not computed here: it is -sum_t exp(sink_h - lse[h, t]) * delta[h, t], a reduction of the two arrays this
// call leaves behind.
GK_EXPORT int gk_attn_bwd_dv(const void* d_o, const void* q, const void* k, const void* v, const void* out,
                             const float* lse, float* delta, void* dq, void* dk_h, void* dv_h, const int* cu_q,
                             const int* cu_k, int B, int Tq, int Tk, int Hq, int Hk, int D, int Dv, int max_q,
                             int max_k, float scale, int causal, int window, void* strides, void* stream_err) {
  const long long* sd = reinterpret_cast<const long long*>(strides);
  void** se = reinterpret_cast<void**>(stream_err);
  if (Dv == 0) Dv = D;
  if (!((D == 64 && Dv == 64) || (D == 128 && Dv == 128) || (D == 192 && Dv == 128))) return -1;
  if (Hq % Hk) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(se[0]);
  {
    const long long warps = static_cast<long long>(Tq) * Hq;
    const long long blocks = (warps * 32 + 255) / 256;
    if (blocks > 0)
      attn_delta_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(out), sd[3], reinterpret_cast<const __nv_bfloat16*>(d_o),
          static_cast<long long>(Hq) * Dv, delta, Tq, Hq, Dv);
  }
  CUtensorMap q128, q64, k128, k64, v128, v64, do128, do64;
  const long long dos = static_cast<long long>(Hq) * Dv;
  if (make_tmap_3d(&q128, q, 2, Tq, Hq, D, sd[0], D, 128, 1, 64, true)) return -3;
  if (make_tmap_3d(&q64, q, 2, Tq, Hq, D, sd[0], D, 64, 1, 64, true)) return -3;
  if (make_tmap_3d(&k128, k, 2, Tk, Hk, D, sd[1], D, 128, 1, 64, true)) return -4;
  if (make_tmap_3d(&k64, k, 2, Tk, Hk, D, sd[1], D, 64, 1, 64, true)) return -4;
  if (make_tmap_3d(&v128, v, 2, Tk, Hk, Dv, sd[2], Dv, 128, 1, 64, true)) return -5;
  if (make_tmap_3d(&v64, v, 2, Tk, Hk, Dv, sd[2], Dv, 64, 1, 64, true)) return -5;
  if (make_tmap_3d(&do128, d_o, 2, Tq, Hq, Dv, dos, Dv, 128, 1, 64, true)) return -6;
  if (make_tmap_3d(&do64, d_o, 2, Tq, Hq, Dv, dos, Dv, 64, 1, 64, true)) return -6;
  FbParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.lse = lse; p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk_h);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv_h);
  p.tq_total = Tq; p.Hq = Hq; p.Hk = Hk; p.causal = causal; p.window = window; p.scale = scale;
  p.err = reinterpret_cast<int*>(se[1]);
  if (D == 192) return launch_bwd<192, 128>(q128, q64, k128, k64, v128, v64, do128, do64, p, B, max_q, max_k, st);
  if (D == 128) return launch_bwd<128, 128>(q128, q64, k128, k64, v128, v64, do128, do64, p, B, max_q, max_k, st);
  return launch_bwd<64, 64>(q128, q64, k128, k64, v128, v64, do128, do64, p, B, max_q, max_k, st);
}

GK_EXPORT int gk_attn_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* out,
                          const float* lse, float* delta, void* dq, void* dk_h, void* dv_h, const int* cu_q,
                          const int* cu_k, const float* sinks, float* dsink, int B, int Tq, int Tk, int Hq, int Hk,
                          int D, int max_q, int max_k, float scale, int causal, int window, void* strides,
                          void* stream_err) {
  (void)sinks; (void)dsink;
  return gk_attn_bwd_dv(d_o, q, k, v, out, lse, delta, dq, dk_h, dv_h, cu_q, cu_k, B, Tq, Tk, Hq, Hk, D, 0, max_q, max_k,
                        scale, causal, window, strides, stream_err);
}
