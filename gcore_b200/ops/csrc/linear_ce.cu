// Fused vocabulary projection + softmax statistics: the logits never leave the SM.
//
//   z[t, v] = inv_temp * (hidden[t, :] . weight[v, :])          hidden [T, K] bf16, weight [V, K] bf16
//   per row and vocabulary split:  (max z, sum exp(z - max), sum exp(z - max) * z, z[target] or -FLT_MAX)
//
// A work item is (128-row block, vocabulary split).  The CTA that owns it walks the split's 256-column tiles with the
// usual tcgen05 pipeline (TMA producer warp, one MMA-issuing thread, accumulators double-buffered in tensor memory);
// the four epilogue warps hold one row per thread and fold every finished tile into that row's running statistics
// while the tensor cores already work on the next tile.  Only `splits * T * 16` bytes are written; log-prob, entropy
// and log-sum-exp follow from the partials in the merge kernel of vocab.cu (which also merges tensor-parallel ranks'
// partials).  Same contract as the reference's linear cross-entropy forward (gpatch_v4/kernel/triton/
// linear_ce_kernels.py:174-340: per-split max / accumulate / entropy terms, merged in an epilogue kernel :735-768).
//
// Items are ordered row block fastest so that the CTAs running together read the same weight tiles from L2.
#include "ptx.cuh"
#include "host_utils.h"
#include <cfloat>

namespace gkl {
using namespace gk;

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 2 * BN;

struct CeParams {
  int T, V, K;
  int row_blocks, nt, splits, tiles_per_split;
  const long long* targets;  // [T] global vocabulary ids (may be null)
  int vocab_start;
  float inv_temp;
  float* partials;           // [splits, T, 4]
  int* err;
};

__global__ void __launch_bounds__(THREADS, 1)
linear_ce_fwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, CeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 128);
    }
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const int items = p.row_blocks * p.splits;
  const int kblocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int m0 = (item % p.row_blocks) * BM;
      const int sp = item / p.row_blocks;
      const int n_begin = sp * p.tiles_per_split;
      const int n_end = n_begin + p.tiles_per_split < p.nt ? n_begin + p.tiles_per_split : p.nt;
      for (int n = n_begin; n < n_end && ok; ++n) {
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
          if (!ok) break;
          if (lane == 0) {
            uint8_t* sa = smem + s * STAGE_BYTES;
            mbar_expect_tx(&full[s], STAGE_BYTES);
            tma_load_2d(sa, &tmA, &full[s], kb * BK, m0);
            tma_load_2d(sa + A_BYTES, &tmB, &full[s], kb * BK, n * BN);
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, 0, 0);
    int s = 0, acc = 0;
    uint32_t ph = 0, pacc = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int sp = item / p.row_blocks;
      const int n_begin = sp * p.tiles_per_split;
      const int n_end = n_begin + p.tiles_per_split < p.nt ? n_begin + p.tiles_per_split : p.nt;
      for (int n = n_begin; n < n_end && ok; ++n) {
        ok = mbar_wait(&tempty[acc], pacc ^ 1, p.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_base = smem_u32(smem + s * STAGE_BYTES);
            const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
              umma_f16(d_tmem, make_smem_desc_sw128(a_base + k4 * (UMMA_K * 2), 16, 1024),
                       make_smem_desc_sw128(b_base + k4 * (UMMA_K * 2), 16, 1024), idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
            }
            umma_commit(&empty[s]);
            if (kb == kblocks - 1) umma_commit(&tfull[acc]);
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        acc ^= 1;
        if (acc == 0) pacc ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ statistics (warps 2..5, one row per thread)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t pacc = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int row = (item % p.row_blocks) * BM + row_in_tile;
      const int sp = item / p.row_blocks;
      const int n_begin = sp * p.tiles_per_split;
      const int n_end = n_begin + p.tiles_per_split < p.nt ? n_begin + p.tiles_per_split : p.nt;
      long long tg = -1;
      if (p.targets && row < p.T) tg = p.targets[row] - p.vocab_start;
      const int tg_i = (tg >= 0 && tg < p.V) ? static_cast<int>(tg) : -(1 << 30);
      float m = -FLT_MAX, sum = 0.f, sz = 0.f, zt = -FLT_MAX;
      for (int n = n_begin; n < n_end && ok; ++n) {
        ok = mbar_wait(&tfull[acc], pacc, p.err, ERR_WAIT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = n * BN + c * 32;
          const int ncols = p.V - col0 < 32 ? p.V - col0 : 32;
          if (ncols <= 0) continue;
          float z[32];
          float cm = -FLT_MAX;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            z[j] = __uint_as_float(r[j]) * p.inv_temp;
            if (j < ncols) cm = fmaxf(cm, z[j]);
          }
          if (cm > m) {
            const float resc = __expf(m - cm);  // 0 on the first chunk (m = -FLT_MAX)
            sum *= resc;
            sz *= resc;
            m = cm;
          }
          const int d = tg_i - col0;  // position of the target inside this chunk, if any
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < ncols) {
              const float e = __expf(z[j] - m);
              sum += e;
              sz = fmaf(e, z[j], sz);
              zt = (j == d) ? z[j] : zt;
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&tempty[acc]);
        acc ^= 1;
        if (acc == 0) pacc ^= 1;
      }
      if (ok && row < p.T) {
        float4* out = reinterpret_cast<float4*>(p.partials) + static_cast<long long>(sp) * p.T + row;
        *out = make_float4(m, sum, sz, zt);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Tiles per split that keep the persistent CTAs evenly loaded: the makespan of a round-robin over `items` work items of
// `tps` tiles each is ceil(items / ctas) * tps; among the choices within 2 % of the best, the longest walk wins (fewer
// partials, fewer pipeline drains).
inline int choose_tiles_per_split(int row_blocks, int nt, int ctas) {
  double best = 0.0;
  for (int tps = 1; tps <= nt; ++tps) {
    const long long items = static_cast<long long>(row_blocks) * ((nt + tps - 1) / tps);
    const double eff = static_cast<double>(row_blocks) * nt / (static_cast<double>((items + ctas - 1) / ctas) * tps * ctas);
    if (eff > best) best = eff;
  }
  int pick = 1;
  for (int tps = 1; tps <= nt; ++tps) {
    const long long items = static_cast<long long>(row_blocks) * ((nt + tps - 1) / tps);
    const double eff = static_cast<double>(row_blocks) * nt / (static_cast<double>((items + ctas - 1) / ctas) * tps * ctas);
    if (eff >= best * 0.98) pick = tps;
  }
  return pick;
}

}  // namespace gkl

using namespace gkl;

// Number of vocabulary splits gk_linear_ce_fwd will use for this shape (the caller sizes `partials` [splits, T, 4]).
GK_EXPORT int gk_linear_ce_splits(int T, int V) {
  if (T <= 0 || V <= 0) return 0;
  const int row_blocks = (T + BM - 1) / BM, nt = (V + BN - 1) / BN;
  const int tps = choose_tiles_per_split(row_blocks, nt, gk::sm_count());
  return (nt + tps - 1) / tps;
}

GK_EXPORT int gk_linear_ce_fwd(const void* hidden, long long ldh, const void* weight, long long ldw,
                               const long long* targets, float inv_temp, int vocab_start, int T, int V, int K,
                               int splits, float* partials, int* err, void* stream) {
  if (T <= 0 || V <= 0 || K <= 0 || splits <= 0) return -10;
  if ((reinterpret_cast<uintptr_t>(hidden) & 15) || (reinterpret_cast<uintptr_t>(weight) & 15) || (ldh & 7) || (ldw & 7) ||
      (reinterpret_cast<uintptr_t>(partials) & 15))
    return -15;
  CeParams p;
  p.T = T; p.V = V; p.K = K;
  p.row_blocks = (T + BM - 1) / BM;
  p.nt = (V + BN - 1) / BN;
  p.splits = splits;
  p.tiles_per_split = (p.nt + splits - 1) / splits;
  p.targets = targets; p.vocab_start = vocab_start; p.inv_temp = inv_temp; p.partials = partials; p.err = err;
  CUtensorMap tmA, tmB;
  int rc = gk::make_tmap_2d(&tmA, hidden, 2, T, K, ldh, BM, 64, true);
  if (rc) return -20 + rc;
  rc = gk::make_tmap_2d(&tmB, weight, 2, V, K, ldw, BN, 64, true);
  if (rc) return -30 + rc;
  static bool configured = false;
  if (!configured) {
    const cudaError_t e =
        cudaFuncSetAttribute(linear_ce_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const long long items = static_cast<long long>(p.row_blocks) * splits;
  const int sms = gk::sm_count();
  const int grid = static_cast<int>(items < sms ? items : sms);
  linear_ce_fwd_kernel<<<grid, THREADS, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  return gk::launch_status();
}
