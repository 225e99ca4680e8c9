// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory), fed by a TMA
// shared-memory ring, as one persistent warp-specialised kernel:
//
//   warp 0      TMA producer   (waits empty[s], arms full[s] with the stage's byte count, issues the loads)
//   warp 1      MMA issuer     (waits full[s], one lane issues BK/16 tcgen05.mma, commits to empty[s];
//                               after the last k-block of a tile commits to tmem_full[acc])
//   warps 2-5   epilogue       (wait tmem_full[acc], tcgen05.ld their 32-lane quadrant, scale / bias /
//                               accumulate, store, arrive on tmem_empty[acc])
//
// Two accumulator buffers in TMEM (2*BN columns) let the epilogue of tile i overlap the main loop of tile i+1.
//
// C[M,N] = alpha * sum_k A[m,k] * B[n,k]  (+ bias) (+ C)
//   A is "K-major" ([M,K] row-major) or "MN-major" ([K,M] row-major); same for B ([N,K] or [K,N]).
//   These cover forward (x W^T), dgrad (dy W) and wgrad (dy^T x) of a linear layer without a transpose pass.
//
// Extra modes used by the rest of the library:
//   * transposed store  - writes C^T; the decode path calls the kernel with the weight as A (128-row tiles of
//                         the weight stream from HBM once) and the few tokens as B ("swap-AB").
//   * split-K           - each CTA reduces a K slice; partials go to a scratch buffer and the last CTA to
//                         arrive on a per-tile counter sums them in a fixed order (deterministic) and stores.
//   * ragged-M groups   - MoE expert GEMMs: rows of A are grouped by expert (segments padded to 128 rows),
//                         B holds one weight per group stacked along rows.
//   * ragged-K groups   - MoE wgrad: the contraction runs over each expert's row segment, one C per group.
//
// Replaces the reference's TileLang `gemm_impl` (gfused/mygemm_fp8.py:13-41) and the cuBLAS/TE GEMMs reached
// through Megatron-Core.
#include "ptx.cuh"
#include "host_utils.h"

namespace gk {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int MAX_GROUPS = 1024;

struct GemmParams {
  int M, N, K;
  int ksplit;
  int group_mode;  // 0 dense, 1 ragged-M, 2 ragged-K
  int num_groups;
  const int* group_offsets;  // [num_groups + 1], multiples of 128
  int b_group_rows;          // mode 1: rows added to B's row coordinate per group
  long long c_group_stride;  // mode 2: elements between consecutive groups' outputs
  void* C;
  long long ldc;
  int out_fp32;
  int transposed;
  int accumulate;
  const void* bias;
  int bias_fp32;
  int bias_along_m;
  float alpha;
  float* ws;
  int* counters;
  int* err;
  int stages;   // shared-memory ring depth actually used (<= Cfg::STAGES)
  int group_m;  // tile order of dense problems (host_utils.h: raster_tile)
  int a_early;  // operand A does not depend on the kernel before this one (decode: A is the weight): its first
                // tiles are requested before the programmatic-dependency wait, while the predecessor still runs
};

struct Tile {
  int m0, n0;       // output tile origin (GEMM coordinates)
  int k0;           // first contraction element
  int kblocks;      // number of BK blocks
  int b_y_off;      // added to B's row coordinate
  int m_limit;      // rows >= m_limit are not stored
  long long c_off;  // element offset into C
  int mn_index;     // index of the (m,n) tile for split-K bookkeeping
  int ks;           // split-K slice
};

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (192 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ +
                                    (MAX_GROUPS + 1) * 4;
};

__device__ __forceinline__ int total_tiles(const GemmParams& p, const int* s_prefix, int BN) {
  const int nt = (p.N + BN - 1) / BN;
  if (p.group_mode == 1) return s_prefix[p.num_groups] * nt;
  const int mt = (p.M + BM - 1) / BM;
  if (p.group_mode == 2) return p.num_groups * mt * nt;
  return mt * nt * p.ksplit;
}

__device__ __forceinline__ Tile decode_tile(const GemmParams& p, const int* s_prefix, int BN, int tile) {
  Tile t;
  const int nt = (p.N + BN - 1) / BN;
  t.ks = 0;
  t.b_y_off = 0;
  t.c_off = 0;
  if (p.group_mode == 1) {
    // tiles are ordered n-tile major inside a group so that CTAs running together share the group's weight
    const int total_m = s_prefix[p.num_groups];
    const int n_idx = tile / total_m;
    const int m_lin = tile - n_idx * total_m;
    int lo = 0, hi = p.num_groups;  // find g with prefix[g] <= m_lin < prefix[g+1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= m_lin) lo = mid; else hi = mid;
    }
    const int g = lo;
    t.m0 = p.group_offsets[g] + (m_lin - s_prefix[g]) * BM;
    t.n0 = n_idx * BN;
    t.k0 = 0;
    t.kblocks = (p.K + BK - 1) / BK;
    t.b_y_off = g * p.b_group_rows;
    t.m_limit = p.group_offsets[g + 1];
    t.mn_index = tile;
  } else if (p.group_mode == 2) {
    const int mt = (p.M + BM - 1) / BM;
    const int per_g = mt * nt;
    const int g = tile / per_g;
    const int r = tile - g * per_g;
    t.m0 = (r % mt) * BM;
    t.n0 = (r / mt) * BN;
    t.k0 = p.group_offsets[g];
    t.kblocks = (p.group_offsets[g + 1] - p.group_offsets[g] + BK - 1) / BK;
    t.m_limit = p.M;
    t.c_off = static_cast<long long>(g) * p.c_group_stride;
    t.mn_index = tile;
  } else {
    const int mt = (p.M + BM - 1) / BM;
    t.ks = tile % p.ksplit;
    const int r = tile / p.ksplit;
    int mi, ni;
    raster_tile(r, mt, nt, p.group_m, mi, ni);
    t.m0 = mi * BM;
    t.n0 = ni * BN;
    const int kb_total = (p.K + BK - 1) / BK;
    const int per = (kb_total + p.ksplit - 1) / p.ksplit;
    const int kb0 = t.ks * per;
    int kb1 = kb0 + per;
    if (kb1 > kb_total) kb1 = kb_total;
    t.k0 = kb0 * BK;
    t.kblocks = kb1 > kb0 ? kb1 - kb0 : 0;
    t.m_limit = p.M;
    t.mn_index = r;
  }
  return t;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Final store of 32 consecutive accumulator columns of one row.
__device__ __forceinline__ void store_chunk(const GemmParams& p, const Tile& t, float (&v)[32], int row, int col0) {
  if (row >= t.m_limit) return;
  const int ncols = p.N - col0 < 32 ? p.N - col0 : 32;
  if (ncols <= 0) return;
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
  if (p.bias) {
    if (p.bias_along_m) {
      const float b = p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[row]
                                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[row]);
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += b;
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols) {
          v[j] += p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[col0 + j]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + j]);
        }
      }
    }
  }
  if (p.transposed) {
    // C^T: element (row, col) lives at C[col * ldc + row]; lanes hold consecutive rows -> coalesced per column.
    if (p.out_fp32) {
      float* c = reinterpret_cast<float*>(p.C) + t.c_off;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols) {
          float* dst = c + static_cast<long long>(col0 + j) * p.ldc + row;
          *dst = p.accumulate ? *dst + v[j] : v[j];
        }
      }
    } else {
      __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + t.c_off;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols) {
          __nv_bfloat16* dst = c + static_cast<long long>(col0 + j) * p.ldc + row;
          *dst = __float2bfloat16(p.accumulate ? __bfloat162float(*dst) + v[j] : v[j]);
        }
      }
    }
    return;
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + t.c_off + static_cast<long long>(row) * p.ldc + col0;
    const bool vec = ncols == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
    if (vec) {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (p.accumulate) {
          const float4 c = d4[j];
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        d4[j] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* dst =
        reinterpret_cast<__nv_bfloat16*>(p.C) + t.c_off + static_cast<long long>(row) * p.ldc + col0;
    const bool vec = ncols == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
    if (vec) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.accumulate) {
          const uint4 c = d4[j];
          const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            v[8 * j + 2 * q] += bf16_bits_to_float(static_cast<uint16_t>(cw[q] & 0xFFFF));
            v[8 * j + 2 * q + 1] += bf16_bits_to_float(static_cast<uint16_t>(cw[q] >> 16));
          }
        }
        uint4 o;
        o.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
        o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
        o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
        o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
        d4[j] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = __float2bfloat16(p.accumulate ? __bfloat162float(dst[j]) + v[j] : v[j]);
    }
  }
}

// MINB = 2 is the decode instantiation: registers are capped so that two CTAs (of this kernel, or this one and the
// next GEMM of the chain) fit one SM's register file together.
template <int BN, bool A_MN, bool B_MN, int MINB = 1>
__global__ void __launch_bounds__(GEMM_THREADS, MINB)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using C = Cfg<BN>;
  const int STAGES = p.stages;  // ring depth of this launch; the barrier arrays are sized for the maximum
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tfull = empty + C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  int* s_flag = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_prefix = reinterpret_cast<int*>(smem + STAGES * C::STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();

  int pre = 0;  // k-blocks of this CTA's first tile whose A tiles were requested early (thread 0 only)
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
    if (p.a_early && p.group_mode == 0 && !A_MN) {
      // the weight tiles of the first output tile start streaming now; the stage barriers are armed for the whole
      // stage, the B halves follow after the dependency wait (producer loop below)
      if (static_cast<int>(blockIdx.x) < total_tiles(p, nullptr, BN)) {
        const Tile t = decode_tile(p, nullptr, BN, blockIdx.x);
        pre = t.kblocks < STAGES ? t.kblocks : STAGES;
        for (int kb = 0; kb < pre; ++kb) {
          mbar_expect_tx(&full[kb], C::STAGE_BYTES);
          tma_load_2d(smem + kb * C::STAGE_BYTES, &tmA, &full[kb], t.k0 + kb * BK, t.m0);
        }
      }
    }
    prefetch_tmap(&tmB);
    if (!p.a_early) prefetch_tmap(&tmA);
  }
  if (threadIdx.x == 32 && p.group_mode == 1) {
    pdl_wait();  // the group offsets come from the kernel before this one
    int acc = 0;
    s_prefix[0] = 0;
    for (int g = 0; g < p.num_groups; ++g) {
      acc += (p.group_offsets[g + 1] - p.group_offsets[g] + BM - 1) / BM;
      s_prefix[g + 1] = acc;
    }
  }
  if (warp == 2) {
    tmem_alloc(tmem_holder, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const int ntiles = total_tiles(p, s_prefix, BN);
  pdl_wait();  // barrier set-up, tensor-memory allocation and descriptor prefetch overlapped the previous kernel

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    pre = __shfl_sync(0xffffffffu, pre, 0);
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      const Tile t = decode_tile(p, s_prefix, BN, tile);
      for (int kb = 0; kb < t.kblocks; ++kb) {
        ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        const bool a_done = (tile == static_cast<int>(blockIdx.x)) && (kb < pre);  // requested before the wait
        if (lane == 0) {
          uint8_t* sa = smem + s * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          const int k = t.k0 + kb * BK;
          if (!a_done) mbar_expect_tx(&full[s], C::STAGE_BYTES);
          if (a_done) {
          } else if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, &full[s], t.m0 + i * 64, k);
          } else {
            tma_load_2d(sa, &tmA, &full[s], k, t.m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sb + i * 8192, &tmB, &full[s], t.n0 + i * 64, k + t.b_y_off);
          } else {
            tma_load_2d(sb, &tmB, &full[s], k, t.n0 + t.b_y_off);
          }
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
    int s = 0, acc = 0;
    uint32_t ph = 0, pacc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      const Tile t = decode_tile(p, s_prefix, BN, tile);
      if (t.kblocks == 0) continue;
      ok = mbar_wait(&tempty[acc], pacc ^ 1, p.err, ERR_WAIT_TMEM_EMPTY);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < t.kblocks; ++kb) {
        ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_base = a_base + C::A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_base + k4 * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(a_base + k4 * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k4 * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(b_base + k4 * (UMMA_K * 2), 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (kb == t.kblocks - 1) umma_commit(&tfull[acc]);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      acc ^= 1;
      if (acc == 0) pacc ^= 1;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // the TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t pacc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      const Tile t = decode_tile(p, s_prefix, BN, tile);
      const bool has_acc = t.kblocks > 0;
      if (has_acc) {
        ok = mbar_wait(&tfull[acc], pacc, p.err, ERR_WAIT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
      }
      const int row = t.m0 + row_in_tile;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        if (has_acc) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (p.ksplit > 1) {
          // partial, column-major inside the tile so that lanes are coalesced
          float* w = p.ws + (static_cast<long long>(t.mn_index) * p.ksplit + t.ks) * (BM * BN) +
                     static_cast<long long>(c * 32) * BM + row_in_tile;
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(w + j * BM, v[j]);
        } else {
          store_chunk(p, t, v, row, t.n0 + c * 32);
        }
      }
      if (has_acc) {
        tc_fence_before();
        mbar_arrive(&tempty[acc]);
        acc ^= 1;
        if (acc == 0) pacc ^= 1;
      }
      if (p.ksplit > 1) {
        __threadfence();
        epi_bar_sync();
        if (threadIdx.x == 64) {
          const int old = atomicAdd(&p.counters[t.mn_index], 1);
          *s_flag = (old == p.ksplit - 1) ? 1 : 0;
        }
        epi_bar_sync();
        if (*s_flag) {
          __threadfence();
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
            // several partials' loads are in flight together: the reduction costs ksplit / U trips to L2, not ksplit
            constexpr int U = MINB > 1 ? 2 : 4;
            for (int ks0 = 0; ks0 < p.ksplit; ks0 += U) {
              float part[U][32];
#pragma unroll
              for (int u = 0; u < U; ++u) {
                const int ks = ks0 + u < p.ksplit ? ks0 + u : ks0;  // a repeated slice is loaded but not added
                const float* w = p.ws + (static_cast<long long>(t.mn_index) * p.ksplit + ks) * (BM * BN) +
                                 static_cast<long long>(c * 32) * BM + row_in_tile;
#pragma unroll
                for (int j = 0; j < 32; ++j) part[u][j] = __ldcg(w + j * BM);
              }
#pragma unroll
              for (int u = 0; u < U; ++u) {
                if (ks0 + u < p.ksplit) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += part[u][j];
                }
              }
            }
            store_chunk(p, t, v, row, t.n0 + c * 32);
          }
          if (threadIdx.x == 64) p.counters[t.mn_index] = 0;
        }
        epi_bar_sync();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, int MINB>
int launch_gemm_q(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& q, int grid, cudaStream_t st) {
  using C = Cfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, A_MN, B_MN, MINB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int smem_bytes = q.stages * C::STAGE_BYTES + 1024 + 256 + (MAX_GROUPS + 1) * 4;
  launch_k(gemm_bf16_kernel<BN, A_MN, B_MN, MINB>, dim3(grid), dim3(GEMM_THREADS), smem_bytes, st, tmA, tmB, q);
  return launch_status();
}

template <int BN, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t st) {
  using C = Cfg<BN>;
  GemmParams q = p;
  q.stages = C::STAGES;
  q.a_early = 0;
  q.group_m = gk::raster_group_m();
  if constexpr (!A_MN && !B_MN && BN <= 128) {
    if (p.transposed && p.group_mode == 0) {
      // decode (swap-AB): A is the weight, which no earlier kernel of the chain writes: its first tiles are requested
      // before the dependency wait.  With a shared-memory budget set, a shallower ring and the register-capped
      // instantiation also leave room for the next kernel's CTA on the same SM.
      q.a_early = 1;
      if (decode_smem_cap() > 0) {
        int nst = (decode_smem_cap() - 1024 - 256 - (MAX_GROUPS + 1) * 4) / C::STAGE_BYTES;
        if (nst < 3) nst = 3;
        if (nst < C::STAGES) q.stages = nst;
        return launch_gemm_q<BN, A_MN, B_MN, 2>(tmA, tmB, q, grid, st);
      }
    }
  }
  return launch_gemm_q<BN, A_MN, B_MN, 1>(tmA, tmB, q, grid, st);
}

}  // namespace gk

using namespace gk;

// Shared-memory budget of decode-shaped (swap-AB) launches; 0 restores the full-depth ring and the late A loads.
GK_EXPORT void gk_gemm_set_decode_smem_cap(int bytes) { gk::decode_smem_cap() = bytes; }

// Tile rows per band of the dense GEMMs' tile order (host_utils.h: raster_group_m); 0 or 1 = row-fastest order.
GK_EXPORT void gk_gemm_set_raster(int group_m) { gk::raster_group_m() = group_m; }

// Scratch requirement of split-K for a given problem: floats of workspace and ints of counters.
GK_EXPORT void gk_gemm_splitk_scratch(int M, int N, int bn, int ksplit, long long* ws_floats, long long* counters) {
  const long long mt = (M + BM - 1) / BM, nt = (N + bn - 1) / bn;
  *ws_floats = ksplit > 1 ? mt * nt * ksplit * BM * bn : 0;
  *counters = ksplit > 1 ? mt * nt : 0;
}

// See the header comment for the semantics.  Returns 0 on success, a negative value for bad arguments or a
// positive cudaError_t.  `err` is a device int the kernel writes a non-zero code into if a bounded wait expires.
GK_EXPORT int gk_gemm_bf16(const void* A, long long lda, long long a_rows, int a_mn,  //
                           const void* B, long long ldb, long long b_rows, int b_mn,  //
                           void* C, long long ldc, int out_fp32, int transposed, int accumulate,
                           const void* bias, int bias_fp32, int bias_along_m, float alpha,  //
                           int M, int N, int K, int bn, int ksplit,                         //
                           int group_mode, int num_groups, const int* group_offsets, int b_group_rows,
                           long long c_group_stride, int max_tiles_hint,  //
                           float* ws, int* counters, int* err, void* stream) {
  if (M <= 0 || N <= 0 || K < 0) return -10;
  if (b_mn && bn < 64) return -11;
  if (num_groups > MAX_GROUPS) return -12;
  if (ksplit < 1) ksplit = 1;
  if (group_mode != 0 && ksplit != 1) return -13;
  if (ksplit > 1 && (!ws || !counters)) return -14;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return -15;
  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn) {  // [a_rows = contraction, cols = M]
    rc = make_tmap_2d(&tmA, A, 2, a_rows, M, lda, 64, 64, true);
  } else {     // [a_rows = M (total), cols = K]
    rc = make_tmap_2d(&tmA, A, 2, a_rows, K, lda, BM, 64, true);
  }
  if (rc) return -20 + rc;
  if (b_mn) {
    rc = make_tmap_2d(&tmB, B, 2, b_rows, N, ldb, 64, 64, true);
  } else {
    rc = make_tmap_2d(&tmB, B, 2, b_rows, K, ldb, bn, 64, true);
  }
  if (rc) return -30 + rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.ksplit = ksplit;
  p.group_mode = group_mode;
  p.num_groups = num_groups;
  p.group_offsets = group_offsets;
  p.b_group_rows = b_group_rows;
  p.c_group_stride = c_group_stride;
  p.C = C; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.transposed = transposed; p.accumulate = accumulate;
  p.bias = bias; p.bias_fp32 = bias_fp32; p.bias_along_m = bias_along_m;
  p.alpha = alpha;
  p.ws = ws; p.counters = counters; p.err = err;

  long long tiles;
  const long long mt = (M + BM - 1) / BM, nt = (N + bn - 1) / bn;
  if (group_mode == 1) tiles = max_tiles_hint > 0 ? static_cast<long long>(max_tiles_hint) * nt : sm_count();
  else if (group_mode == 2) tiles = static_cast<long long>(num_groups) * mt * nt;
  else tiles = mt * nt * ksplit;
  int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  if (grid < 1) grid = 1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

#define GK_DISPATCH(BN_)                                                                   \
  if (bn == BN_) {                                                                         \
    if (!a_mn && !b_mn) return launch_gemm<BN_, false, false>(tmA, tmB, p, grid, st);      \
    if (a_mn && !b_mn) return launch_gemm<BN_, true, false>(tmA, tmB, p, grid, st);        \
    if constexpr (BN_ >= 64) {                                                             \
      if (!a_mn && b_mn) return launch_gemm<BN_, false, true>(tmA, tmB, p, grid, st);      \
      if (a_mn && b_mn) return launch_gemm<BN_, true, true>(tmA, tmB, p, grid, st);        \
    }                                                                                      \
  }
  GK_DISPATCH(32)
  GK_DISPATCH(64)
  GK_DISPATCH(128)
  GK_DISPATCH(192)
  GK_DISPATCH(256)
  if (bn == 224 && !b_mn) {  // 224 is not a whole number of 64-column chunks, which the MN-major B loads need
    if (!a_mn) return launch_gemm<224, false, false>(tmA, tmB, p, grid, st);
    return launch_gemm<224, true, false>(tmA, tmB, p, grid, st);
  }
#undef GK_DISPATCH
  return -16;
}
