// Large dense bf16 GEMM with 256 x 256 output tiles per CTA.
//
// ncu on the 128 x 256 kernel (gemm_tcgen05.cu) at training shapes shows the tensor pipe busy 71.5 % of the time with
// shared memory as the limiter: per 64-deep k-block TMA writes (128 + 256) x 128 B into shared memory and the two
// operands are read back once by tcgen05.mma, 179 B / clock against a 128 B / clock shared-memory port.  A 256-row
// tile runs two M = 128 instructions against the SAME B tile: per k-block (256 + 256) x 128 B written and
// (256 + 2 x 256) x 128 B read for twice the FLOPs, 17 % less shared-memory traffic per FLOP.
//
// The two 128 x 256 fp32 accumulators fill all 512 TMEM columns, so they cannot be double-buffered; instead each half
// has its own "empty" barrier: the epilogue releases the upper half first and the MMA issuer of the next tile starts
// on it while the lower half is still being drained.
//
// Dense problems only (no groups, no split-K, no transposed store); all four operand layouts; bias along N, alpha,
// bf16 or fp32 output with optional accumulation.  Roles: warp 0 TMA, warp 1 MMA, warps 2-5 epilogue.
#include "ptx.cuh"
#include "host_utils.h"

namespace gkw {
using namespace gk;

constexpr int BMW = 256, BN = 256, BK = 64, UMMA_K = 16;
constexpr int EPI_WARPS = 8;       // two per TMEM lane quarter: each drains one 128-column half of an accumulator
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int THREADS = 64 + EPI_THREADS;
constexpr int STAGES = 3;
constexpr int A_BYTES = BMW * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
// Epilogue staging: every epilogue warp owns 32 rows x 128 bytes (64 bf16 or 32 fp32 columns of its TMEM lane
// quarter).  Values go from TMEM registers into that area row by row (16-byte units, XOR-swizzled by row so that the
// 32 lanes of a store hit 32 different banks groups) and leave it as whole 128-byte row segments, four rows per
// warp-wide store: every global store instruction then writes complete 128-byte lines instead of 32 separate
// 16-byte fragments.  The accumulators of this kernel are not double-buffered, so the time the epilogue needs to
// drain the first half of a tile is time the tensor cores wait.
constexpr int MAX_TAIL_KS = 4;      // K-slices of a tail tile (their partials are summed by one CTA)
constexpr int STAGE_ROW_BYTES = 128;
constexpr int EPI_STAGE_BYTES = EPI_WARPS * 32 * STAGE_ROW_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_BYTES + 1024 + 256;

struct WParams {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32, accumulate;
  const void* bias;
  int bias_fp32;
  float alpha;
  int* err;
  int group_m;
  int staged;   // C rows are 16-byte aligned (and no bf16 read-modify-write): the epilogue stores through shared memory
  // Tail split: a problem whose tile count is a little more than a whole number of waves would leave most SMs idle
  // during the last wave (448 tiles on 148 SMs: 3 waves and 4 tiles).  The tiles of that partial wave are cut along K
  // into `tail_ks` slices of `tail_per` k-blocks, each slice is a work item of its own, the slices leave fp32
  // partials in `ws` and the CTA that finishes a tile's last slice adds them up and stores the tile.
  int full_tiles;   // tiles [0, full_tiles) are whole work items; the others are split
  int tail_ks, tail_per;
  float* ws;        // [tail tiles][tail_ks][256 x 256] fp32
  int* counters;    // [tail tiles], zero between launches
};

struct Item {
  int tile, kb0, kb1, slice;
  bool split;
};
__device__ __forceinline__ Item work_item(const WParams& p, int w, int kblocks) {
  Item it;
  if (w < p.full_tiles) {
    it.tile = w; it.kb0 = 0; it.kb1 = kblocks; it.slice = 0; it.split = false;
  } else {
    const int r = w - p.full_tiles;
    it.tile = p.full_tiles + r / p.tail_ks;
    it.slice = r % p.tail_ks;
    it.kb0 = it.slice * p.tail_per;
    it.kb1 = it.kb0 + p.tail_per < kblocks ? it.kb0 + p.tail_per : kblocks;
    it.split = true;
  }
  return it;
}

// 32 consecutive accumulator columns of one output row
__device__ __forceinline__ void store32(const WParams& p, float (&v)[32], int row, int col0) {
  if (row >= p.M) return;
  const int ncols = p.N - col0 < 32 ? p.N - col0 : 32;
  if (ncols <= 0) return;
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < ncols) {
        v[j] += p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[col0 + j]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + j]);
      }
    }
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (ncols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
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
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (ncols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
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

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, WParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + EPI_STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;   // 1: both halves are complete
  uint64_t* tempty = tfull + 1;       // 2: upper / lower half drained (128 arrivals each)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  int* s_last = reinterpret_cast<int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(tfull, 1);
    mbar_init(&tempty[0], EPI_THREADS);
    mbar_init(&tempty[1], EPI_THREADS);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  pdl_wait();

  const int mt = (p.M + BMW - 1) / BMW, nt = (p.N + BN - 1) / BN;
  const int ntiles = mt * nt;
  const int kblocks = (p.K + BK - 1) / BK;
  const int nitems = p.full_tiles + (ntiles - p.full_tiles) * p.tail_ks;

  if (warp == 0) {
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
      const Item it = work_item(p, w, kblocks);
      int mi, ni;
      raster_tile(it.tile, mt, nt, p.group_m, mi, ni);
      const int m0 = mi * BMW, n0 = ni * BN;
      for (int kb = it.kb0; kb < it.kb1; ++kb) {
        ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const int k = kb * BK;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BMW / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, &full[s], m0 + i * 64, k);
          } else {
            tma_load_2d(sa, &tmA, &full[s], k, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, &full[s], n0 + i * 64, k);
          } else {
            tma_load_2d(sb, &tmB, &full[s], k, n0);
          }
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(128, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
    int s = 0;
    uint32_t ph = 0, pt = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
      const Item it = work_item(p, w, kblocks);
      for (int kb = it.kb0; kb < it.kb1 && ok; ++kb) {
        ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(smem + s * STAGE_BYTES);
        const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (kb == it.kb0) {  // the previous item's accumulator half must have been read out
            ok = mbar_wait(&tempty[half], pt ^ 1, p.err, ERR_WAIT_TMEM_EMPTY);
            if (!ok) break;
            tc_fence_after();
          }
          if (lane == 0) {
            // K-major A: rows 128..255 start 128 x 128 B further; MN-major A: two 64-column chunks further
            const uint32_t ah = a_base + half * 16384;
#pragma unroll
            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
              const uint64_t adesc = A_MN ? make_smem_desc_sw128(ah + k4 * (UMMA_K * 128), 8192, 1024)
                                          : make_smem_desc_sw128(ah + k4 * (UMMA_K * 2), 16, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k4 * (UMMA_K * 128), 8192, 1024)
                                          : make_smem_desc_sw128(b_base + k4 * (UMMA_K * 2), 16, 1024);
              umma_f16(tmem_base + half * BN, adesc, bdesc, idesc, (kb > it.kb0 || k4 > 0) ? 1u : 0u);
            }
          }
          __syncwarp();
        }
        if (!ok) break;
        if (lane == 0) {
          umma_commit(&empty[s]);
          if (kb == it.kb1 - 1) umma_commit(tfull);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      pt ^= 1;
    }
  } else {
    const int quad = warp & 3;            // the TMEM lane quarter a warp may read is fixed by its index
    const int chalf = (warp - 2) >> 2;    // which 128 columns of the 256
    uint32_t pt = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
      const Item it = work_item(p, w, kblocks);
      int mi, ni;
      raster_tile(it.tile, mt, nt, p.group_m, mi, ni);
      const int m0 = mi * BMW, n0 = ni * BN;
      if (kblocks > 0) {
        ok = mbar_wait(tfull, pt, p.err, ERR_WAIT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
      }
      if (it.split) {
        // ---- a K-slice of a tail tile: park the fp32 partial (column-major inside the tile: lanes hold consecutive
        // rows, so every store is one 128-byte line), release the accumulators, and let the CTA that brings the last
        // slice add everything up and store the tile
        const int tslot = it.tile - p.full_tiles;
        float* part = p.ws + (static_cast<long long>(tslot) * p.tail_ks + it.slice) * (BMW * BN);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + half * BN;
          const int rin = half * 128 + quad * 32 + lane;
#pragma unroll 1
          for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(part + static_cast<long long>(c * 32 + j) * BMW + rin, __uint_as_float(r[j]));
          }
          tc_fence_before();
          mbar_arrive(&tempty[half]);
        }
        pt ^= 1;
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 64) *s_last = atomicAdd(&p.counters[tslot], 1) == p.tail_ks - 1 ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        if (*s_last) {
          __threadfence();
          const float* base = p.ws + static_cast<long long>(tslot) * p.tail_ks * (BMW * BN);
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            const int rin = half * 128 + quad * 32 + lane;
#pragma unroll 1
            for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
              // all slices' loads of a chunk are in flight together (at most MAX_TAIL_KS x 32 per thread): the pass
              // costs one trip to L2 per chunk, not one per slice
              float part[MAX_TAIL_KS][32];
#pragma unroll
              for (int sl = 0; sl < MAX_TAIL_KS; ++sl) {
                const int s2 = sl < p.tail_ks ? sl : 0;   // a repeated slice is loaded but not added
                const float* src = base + static_cast<long long>(s2) * (BMW * BN) + static_cast<long long>(c * 32) * BMW + rin;
#pragma unroll
                for (int j = 0; j < 32; ++j) part[sl][j] = __ldcg(src + j * BMW);
              }
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = part[0][j];
#pragma unroll
              for (int sl = 1; sl < MAX_TAIL_KS; ++sl) {
                if (sl < p.tail_ks) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += part[sl][j];
                }
              }
              store32(p, v, m0 + rin, n0 + c * 32);
            }
          }
          if (threadIdx.x == 64) p.counters[tslot] = 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        continue;
      }
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        const int row = m0 + half * 128 + quad * 32 + lane;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + half * BN;
        if (p.staged) {
          uint8_t* st = epi_stage + (warp - 2) * (32 * STAGE_ROW_BYTES);
          const int esz = p.out_fp32 ? 4 : 2;
          const int group_cols = STAGE_ROW_BYTES / esz;          // 32 fp32 or 64 bf16 columns per pass
          const int row0 = m0 + half * 128 + quad * 32;           // first row of this warp
#pragma unroll 1
          for (int g0 = chalf * 128; g0 < chalf * 128 + 128; g0 += group_cols) {
#pragma unroll 1
            for (int c = g0 / 32; c < (g0 + group_cols) / 32; ++c) {
              float v[32];
              if (kblocks > 0) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
              }
              const int col0 = n0 + c * 32;
              if (p.bias) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (col0 + j < p.N)
                    v[j] += p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[col0 + j]
                                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + j]);
                }
              }
              if (p.out_fp32) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  *reinterpret_cast<float4*>(st + lane * STAGE_ROW_BYTES + ((j ^ (lane & 7)) << 4)) =
                      make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              } else {
                const int ubase = (c & 1) * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 o;
                  o.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
                  o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                  o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                  o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                  *reinterpret_cast<uint4*>(st + lane * STAGE_ROW_BYTES + (((ubase + j) ^ (lane & 7)) << 4)) = o;
                }
              }
            }
            __syncwarp();
            // drain: lane -> (row 4 i + lane / 8, unit lane % 8); one instruction = four rows x 128 bytes
            const int unit = lane & 7;
            const int ucols = 16 / esz;
            const int col = n0 + g0 + unit * ucols;
#pragma unroll 4
            for (int i = 0; i < 8; ++i) {
              const int rr = 4 * i + (lane >> 3);
              const int grow = row0 + rr;
              const uint4 w = *reinterpret_cast<const uint4*>(st + rr * STAGE_ROW_BYTES + ((unit ^ (rr & 7)) << 4));
              if (grow >= p.M || col >= p.N) continue;
              uint8_t* dst = reinterpret_cast<uint8_t*>(p.C) + (static_cast<long long>(grow) * p.ldc + col) * esz;
              if (col + ucols <= p.N) {
                if (p.out_fp32 && p.accumulate) {
                  const float4 c4 = *reinterpret_cast<const float4*>(dst);
                  float4 o = *reinterpret_cast<const float4*>(&w);
                  o.x += c4.x; o.y += c4.y; o.z += c4.z; o.w += c4.w;
                  *reinterpret_cast<float4*>(dst) = o;
                } else {
                  *reinterpret_cast<uint4*>(dst) = w;
                }
              } else if (p.out_fp32) {
                const float* e = reinterpret_cast<const float*>(&w);
                float* d = reinterpret_cast<float*>(dst);
                for (int j = 0; j < ucols; ++j)
                  if (col + j < p.N) d[j] = p.accumulate ? d[j] + e[j] : e[j];
              } else {
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&w);
                __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst);
                for (int j = 0; j < ucols; ++j)
                  if (col + j < p.N) d[j] = e[j];
              }
            }
            __syncwarp();   // the staging rows are free for the next pass
          }
        } else {
#pragma unroll 1
          for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
            float v[32];
            if (kblocks > 0) {
              uint32_t r[32];
              tmem_ld32(taddr + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
            store32(p, v, row, n0 + c * 32);
          }
        }
        tc_fence_before();
        mbar_arrive(&tempty[half]);
      }
      pt ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <bool A_MN, bool B_MN>
int launch_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const WParams& p, int grid, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_wide_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return -6;
    configured = true;
  }
  launch_k(gemm_wide_kernel<A_MN, B_MN>, dim3(grid), dim3(THREADS), SMEM_BYTES, st, tmA, tmB, p);
  return launch_status();
}

}  // namespace gkw

using namespace gkw;

// 0: per-thread row stores (A/B switch for the staged epilogue)
GK_EXPORT void gk_gemm_wide_set_staged(int on) { gk::wide_staged_epilogue() = on; }

// C[M,N] (+)= alpha * A . B^T (+ bias over N).  a_mn: A is [K, M] (M contiguous); b_mn: B is [K, N].
// 0: no K-split of the partial last wave (A/B switch)
GK_EXPORT void gk_gemm_wide_set_tail_split(int on) { gk::wide_tail_split() = on; }

// ws / counters (optional): scratch for the tail split, `ws_floats` floats and `counter_ints` zero-initialised ints.
GK_EXPORT int gk_gemm_wide(const void* A, long long lda, long long a_rows, int a_mn, const void* B, long long ldb,
                           long long b_rows, int b_mn, void* C, long long ldc, int out_fp32, int accumulate,
                           const void* bias, int bias_fp32, float alpha, int M, int N, int K, float* ws,
                           long long ws_floats, int* counters, int counter_ints, int* err, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -15;
  CUtensorMap tmA, tmB;
  int rc = a_mn ? gk::make_tmap_2d(&tmA, A, 2, a_rows, M, lda, 64, 64, true)
                : gk::make_tmap_2d(&tmA, A, 2, a_rows, K, lda, BMW, 64, true);
  if (rc) return -20 + rc;
  rc = b_mn ? gk::make_tmap_2d(&tmB, B, 2, b_rows, N, ldb, 64, 64, true)
            : gk::make_tmap_2d(&tmB, B, 2, b_rows, K, ldb, BN, 64, true);
  if (rc) return -30 + rc;
  WParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = bias; p.bias_fp32 = bias_fp32; p.alpha = alpha; p.err = err;
  p.group_m = gk::raster_group_m();
  const int esz = out_fp32 ? 4 : 2;
  p.staged = ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * esz) % 16 == 0 && (out_fp32 || !accumulate) &&
              gk::wide_staged_epilogue()) ? 1 : 0;
  const long long tiles = static_cast<long long>((M + BMW - 1) / BMW) * ((N + BN - 1) / BN);
  const int sms = gk::sm_count();
  int grid = static_cast<int>(tiles < sms ? tiles : sms);
  p.full_tiles = static_cast<int>(tiles); p.tail_ks = 1; p.tail_per = 0; p.ws = ws; p.counters = counters;
  const int kblocks = (K + BK - 1) / BK;
  const int tail = static_cast<int>(tiles % sms);
  if (ws && counters && gk::wide_tail_split() && tail > 0 && tail * 2 <= sms && kblocks >= 8) {
    // as many slices as fill the idle SMs of the partial wave, at least four k-blocks each
    int ks = sms / tail;
    if (ks > kblocks / 4) ks = kblocks / 4;
    if (ks > MAX_TAIL_KS) ks = MAX_TAIL_KS;
    const long long need = static_cast<long long>(tail) * ks * BMW * BN;
    if (ks >= 2 && need <= ws_floats && tail <= counter_ints) {
      const int per = (kblocks + ks - 1) / ks;
      p.tail_per = per;
      p.tail_ks = (kblocks + per - 1) / per;   // no empty slice
      p.full_tiles = static_cast<int>(tiles) - tail;
      if (tiles < sms) grid = static_cast<int>(tiles - tail + tail * p.tail_ks < sms ? tiles - tail + tail * p.tail_ks : sms);
    }
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch_wide<false, false>(tmA, tmB, p, grid, st);
  if (a_mn && !b_mn) return launch_wide<true, false>(tmA, tmB, p, grid, st);
  if (!a_mn && b_mn) return launch_wide<false, true>(tmA, tmB, p, grid, st);
  return launch_wide<true, true>(tmA, tmB, p, grid, st);
}
