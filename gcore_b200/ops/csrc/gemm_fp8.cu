// Block-scaled e4m3 GEMM on tcgen05 (kind::f8f6f4): C[M,N] = sum_kb sA[m,kb] * sB[n/128,kb] * (A_kb * B_kb^T),
// A [M,K] e4m3 with one fp32 scale per (row, 128-wide K block), B [N,K] e4m3 with one fp32 scale per 128x128 block
// (the DeepSeek-V3 recipe; the reference's TileLang version is gfused/mygemm_fp8.py:45-97).
//
// Two-level accumulation: every 128-deep K block is multiplied on the tensor core into a fresh TMEM accumulator
// (four buffers in rotation); eight promotion warps (two per TMEM lane quarter, 64 columns each) pull that partial
// product out of TMEM, apply sA * sB and add it into fp32 register accumulators while the tensor core already works
// on the next block.  The promotion has to keep up with ~270 tensor-core cycles per block, hence the eight warps,
// both TMEM loads of a thread in flight at once and the scales fetched one block ahead.  bf16 or fp32 output.
#include "ptx.cuh"
#include "host_utils.h"

namespace gk8 {
using namespace gk;

constexpr int BM = 128, BN = 128, BK = 128;  // BK bytes = 128 = one swizzle row of e4m3
constexpr int UMMA_K = 32;
constexpr int STAGES = 5;
constexpr int THREADS = 320;          // TMA warp, MMA warp, 8 promotion warps
constexpr int PROMO_THREADS = 256;
constexpr int HALF = BN / 2;           // columns per promotion warp
constexpr int NBUF = 4;                // TMEM accumulators in flight (4 x 128 columns = all of TMEM)
constexpr int STAGE_BYTES = (BM + BN) * BK;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct P8 {
  int M, N, K;
  const float* sA;  // [M, KB]
  const float* sB;  // [ceil(N/128), KB]
  void* C;
  long long ldc;
  int out_fp32;
  int* err;
  // ragged-M groups (experts): rows [offsets[g], offsets[g+1]) of A multiply group g's weight, stored at rows
  // [g * N, (g + 1) * N) of B with its scales at rows [g * ceil(N / 128), ...) of sB.  Offsets are multiples of 128
  // (device array, G + 1 entries); M is the capacity of A, tiles at or beyond offsets[G] are skipped.
  const int* group_offsets;
  int num_groups;
};

// group of the 128-row tile starting at row m0, or -1 when the tile lies beyond the last group
__device__ __forceinline__ int group_of(const P8& p, int m0) {
  if (m0 >= p.group_offsets[p.num_groups]) return -1;
  int lo = 0, hi = p.num_groups;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.group_offsets[mid] <= m0) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, P8 p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;   // NBUF
  uint64_t* tempty = tfull + NBUF;    // NBUF (one arrival per promotion thread)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + NBUF);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = (p.M + BM - 1) / BM;
  const int ntiles = mt * ((p.N + BN - 1) / BN);
  const int KB = (p.K + BK - 1) / BK;
  // persistent: CTA c works on tiles c, c + grid, ...; the three roles walk the same sequence, and the pipeline
  // (shared-memory stages, the two TMEM buffers) keeps running across tile boundaries, so the loads and MMAs of the
  // next tile overlap the promotion and the store of the current one

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < NBUF; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], PROMO_THREADS); }
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) { tmem_alloc(tmem_holder, NBUF * BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    bool ok = true;
    long long it = 0;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
      int b_row = n0;
      if (p.group_offsets) {
        const int g = group_of(p, m0);
        if (g < 0) continue;
        b_row += g * p.N;
      }
      for (int kb = 0; kb < KB && ok; ++kb, ++it) {
        const int s = static_cast<int>(it % STAGES);
        const uint32_t ph = static_cast<uint32_t>(it / STAGES) & 1;
        ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* sa = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full[s], kb * BK, m0);
          tma_load_2d(sa + BM * BK, &tmB, &full[s], kb * BK, b_row);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0, 0, 0);  // e4m3 x e4m3 -> f32
    bool ok = true;
    long long live = 0;  // tiles of this CTA that carry rows (all of them for a dense problem)
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x)
      live += (!p.group_offsets || (tile % mt) * BM < p.group_offsets[p.num_groups]) ? 1 : 0;
    const long long total = live * KB;
    for (long long it = 0; it < total && ok; ++it) {
      const int s = static_cast<int>(it % STAGES), a = static_cast<int>(it % NBUF);
      ok = mbar_wait(&tempty[a], (static_cast<uint32_t>(it / NBUF) & 1) ^ 1, p.err, ERR_WAIT_TMEM_EMPTY);
      if (!ok) break;
      ok = mbar_wait(&full[s], static_cast<uint32_t>(it / STAGES) & 1, p.err, ERR_WAIT_FULL);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t ab = smem_u32(smem + s * STAGE_BYTES), bb = ab + BM * BK;
#pragma unroll
        for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
          umma_f8(tmem_base + a * BN, make_smem_desc_sw128(ab + k4 * UMMA_K, 16, 1024),
                  make_smem_desc_sw128(bb + k4 * UMMA_K, 16, 1024), idesc, k4 > 0 ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        umma_commit(&tfull[a]);
      }
      __syncwarp();
    }
  } else {
    const int quad = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;          // which 64 columns of the tile
    bool ok = true;
    long long it = 0;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
    const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
    const int row = m0 + quad * 32 + lane;
    int nb = n0 / 128;
    if (p.group_offsets) {
      const int g = group_of(p, m0);
      if (g < 0) continue;
      nb += g * ((p.N + 127) / 128);
    }
    float acc[HALF];
#pragma unroll
    for (int j = 0; j < HALF; ++j) acc[j] = 0.f;
    const float* sa_row = p.sA + static_cast<long long>(row < p.M ? row : 0) * KB;
    const float* sb_row = p.sB + static_cast<long long>(nb) * KB;
    float sc_next = (row < p.M ? sa_row[0] : 0.f) * sb_row[0];
    for (int kb = 0; kb < KB && ok; ++kb, ++it) {
      const int a = static_cast<int>(it % NBUF);
      const float sc = sc_next;
      if (kb + 1 < KB) sc_next = (row < p.M ? sa_row[kb + 1] : 0.f) * sb_row[kb + 1];  // in flight during the wait
      ok = mbar_wait(&tfull[a], static_cast<uint32_t>(it / NBUF) & 1, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + a * BN + half * HALF;
      uint32_t r0[32], r1[32];
      tmem_ld32(taddr, r0);
      tmem_ld32(taddr + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&tempty[a]);                 // the values are in registers: the buffer can take the next block
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = fmaf(sc, __uint_as_float(r0[j]), acc[j]);
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(sc, __uint_as_float(r1[j]), acc[32 + j]);
    }
    if (ok && row < p.M) {
#pragma unroll
      for (int c = 0; c < HALF / 8; ++c) {
        const int col = n0 + half * HALF + c * 8;
        if (col + 8 <= p.N && (p.ldc & 7) == 0) {
          if (p.out_fp32) {
            float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col);
            d[0] = make_float4(acc[c * 8], acc[c * 8 + 1], acc[c * 8 + 2], acc[c * 8 + 3]);
            d[1] = make_float4(acc[c * 8 + 4], acc[c * 8 + 5], acc[c * 8 + 6], acc[c * 8 + 7]);
          } else {
            uint4 o;
            o.x = pack_bf16x2(acc[c * 8], acc[c * 8 + 1]);
            o.y = pack_bf16x2(acc[c * 8 + 2], acc[c * 8 + 3]);
            o.z = pack_bf16x2(acc[c * 8 + 4], acc[c * 8 + 5]);
            o.w = pack_bf16x2(acc[c * 8 + 6], acc[c * 8 + 7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col) = o;
          }
        } else {
          for (int j = 0; j < 8; ++j) {
            if (col + j < p.N) {
              if (p.out_fp32) reinterpret_cast<float*>(p.C)[static_cast<long long>(row) * p.ldc + col + j] = acc[c * 8 + j];
              else reinterpret_cast<__nv_bfloat16*>(p.C)[static_cast<long long>(row) * p.ldc + col + j] = __float2bfloat16(acc[c * 8 + j]);
            }
          }
        }
      }
    }
    }  // tiles
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, NBUF * BN); }
}

}  // namespace gk8

using namespace gk8;

// A [M,K] and B [N,K] are e4m3 bytes (row-major, K contiguous, K % 16 == 0); sA fp32 [M, ceil(K/128)],
// sB fp32 [ceil(N/128), ceil(K/128)].
GK_EXPORT int gk_gemm_fp8_blockscaled(const void* A, long long lda, const void* B, long long ldb, const float* sA,
                                      const float* sB, void* C, long long ldc, int out_fp32, int M, int N, int K,
                                      int* err, void* stream) {
  if ((lda & 15) || (ldb & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  CUtensorMap tmA, tmB;
  if (gk::make_tmap_2d(&tmA, A, 1, M, K, lda, BM, BK, true)) return -2;
  if (gk::make_tmap_2d(&tmB, B, 1, N, K, ldb, BN, BK, true)) return -3;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -4;
    configured = true;
  }
  P8 p;
  p.M = M; p.N = N; p.K = K; p.sA = sA; p.sB = sB; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.err = err;
  p.group_offsets = nullptr; p.num_groups = 0;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  gemm_fp8_kernel<<<tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  return gk::launch_status();
}

// Ragged-M grouped form (experts): A [M_cap, K] e4m3 with expert-sorted rows, group g = rows [offsets[g],
// offsets[g+1]) (multiples of 128, device array of G + 1 ints); B [G * N, K] e4m3, sB [G * ceil(N/128), ceil(K/128)].
// C [M_cap, N]: rows of group g hold A_g . B_g^T; rows beyond offsets[G] are not written.
GK_EXPORT int gk_gemm_fp8_grouped(const void* A, long long lda, const void* B, long long ldb, const float* sA,
                                  const float* sB, void* C, long long ldc, int out_fp32, int M_cap, int N, int K,
                                  const int* offsets, int num_groups, int* err, void* stream) {
  if ((lda & 15) || (ldb & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  if (num_groups < 1 || !offsets || M_cap % BM) return -5;
  CUtensorMap tmA, tmB;
  if (gk::make_tmap_2d(&tmA, A, 1, M_cap, K, lda, BM, BK, true)) return -2;
  if (gk::make_tmap_2d(&tmB, B, 1, static_cast<uint64_t>(num_groups) * N, K, ldb, BN, BK, true)) return -3;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -4;
    configured = true;
  }
  P8 p;
  p.M = M_cap; p.N = N; p.K = K; p.sA = sA; p.sB = sB; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.err = err;
  p.group_offsets = offsets; p.num_groups = num_groups;
  const int tiles = (M_cap / BM) * ((N + BN - 1) / BN);
  const int sms = gk::sm_count();
  gemm_fp8_kernel<<<tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  return gk::launch_status();
}
