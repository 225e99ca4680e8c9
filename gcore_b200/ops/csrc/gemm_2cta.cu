// bf16 GEMM on CTA pairs: two CTAs of a cluster (two SMs) compute one 256 x 256 output tile with
// `tcgen05.mma.cta_group::2`.  Each CTA stages its own 128 rows of A and its own 128 rows (half of N) of B; the tensor
// cores of both SMs read the two B halves from both shared memories, so every SM moves half the B bytes per FLOP of
// the one-CTA 128 x 256 kernel (gemm_tcgen05.cu), which is bound by shared-memory bandwidth at training shapes.
//
//   C[M,N] = A[m,k] . B[n,k]  (+ bias[n]) (+ C)      bf16 operands, fp32 accumulation, bf16 or fp32 C
//   A "K-major" ([M,K] row-major) or "MN-major" ([K,M] row-major); same for B: forward (x W^T), dgrad (dy W) and
//   wgrad (dy^T x, accumulated into an fp32 buffer) of a linear layer.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer (only in the pair's first CTA), warps 2-5
// epilogue (each CTA reads its own 128 accumulator rows from its own tensor memory).
//
// Protocol between the two CTAs (rank 0 = leader).  All loads are ordinary single-destination TMA loads from this
// GPU's memory; nothing is broadcast.
//   full[s]   lives in the leader: armed by the leader's producer with the bytes of BOTH CTAs' stage; the second
//             CTA's loads complete their bytes on the leader's barrier (`cp.async.bulk.tensor...cta_group::2` with
//             the barrier address mapped to rank 0).
//   empty[s]  one per CTA: the leader's MMA thread commits to its own and, with a second commit, to the peer's
//             (address mapped to rank 1).
//   tfull[a]  one per CTA, committed the same way after a tile's last k-block.
//   tempty[a] lives in the leader, expects the 256 epilogue threads of both CTAs; the second CTA's threads arrive
//             through the cluster address.
// Every wait is bounded (ptx.cuh: mbar_wait); on expiry all roles of both CTAs leave their loops, meet at the final
// cluster barrier, free tensor memory and return; the host reads the error word.
#include "ptx.cuh"
#include "host_utils.h"

namespace gk2 {
using namespace gk;

constexpr int BMH = 128;        // rows of A per CTA
constexpr int BNH = 128;        // rows of B (columns of C) staged per CTA
constexpr int TM = 256, TN = 256;
constexpr int BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BMH * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int MAX_STAGES = 7;
constexpr int SMEM_BYTES = MAX_STAGES * STAGE_BYTES + 1024 + 256;
inline int& stages_setting() {
  static int n = 6;
  return n;
}
constexpr int TMEM_COLS = 512;  // two 256-column accumulators

struct P2 {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32, accumulate;
  const void* bias;
  int bias_fp32;
  float alpha;
  int* err;
  int stages;
  int group_m;
};

__device__ __forceinline__ uint32_t cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// Single-destination TMA load issued by either CTA of the pair; the bytes are counted on `bar_cluster_addr`, which
// may be the other CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// Arrives on the barrier at `bar_cluster_addr` (this CTA's or the peer's) once the pair's MMAs issued so far retire.
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void store32(const P2& p, const float (&v)[32], int row, int col0) {
  if (row >= p.M) return;
  int n = p.N - col0;
  if (n <= 0) return;
  if (n > 32) n = 32;
  float o[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) o[j] = v[j] * p.alpha;
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < n)
        o[j] += p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[col0 + j]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + j]);
    }
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (n == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 w = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        if (p.accumulate) {
          const float4 c = *reinterpret_cast<const float4*>(dst + j);
          w.x += c.x; w.y += c.y; w.z += c.z; w.w += c.w;
        }
        *reinterpret_cast<float4*>(dst + j) = w;
      }
    } else {
      for (int j = 0; j < n; ++j) dst[j] = p.accumulate ? dst[j] + o[j] : o[j];
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (n == 32 && !p.accumulate && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 w;
        w.x = pack_bf16x2(o[j], o[j + 1]);
        w.y = pack_bf16x2(o[j + 2], o[j + 3]);
        w.z = pack_bf16x2(o[j + 4], o[j + 5]);
        w.w = pack_bf16x2(o[j + 6], o[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = w;
      }
    } else {
      for (int j = 0; j < n; ++j)
        dst[j] = __float2bfloat16(p.accumulate ? __bfloat162float(dst[j]) + o[j] : o[j]);
    }
  }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, P2 p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int STAGES = p.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tfull = empty + MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int mt = (p.M + TM - 1) / TM, nt = (p.N + TN - 1) / TN;
  const int ntiles = mt * nt;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 256);
    }
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) {
    tmem_alloc2(tmem_holder, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist and both halves of tensor memory are allocated
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < ntiles && ok; tile += n_clusters) {
      int mi, ni;
      raster_tile(tile, mt, nt, p.group_m, mi, ni);
      const int m0 = mi * TM + static_cast<int>(rank) * BMH;
      const int n0 = ni * TN + static_cast<int>(rank) * BNH;
      for (int kb = 0; kb < kblocks; ++kb) {
        ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const int k = kb * BK;
          const uint32_t bar = map_to_rank(smem_u32(&full[s]), 0);
          if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BMH / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tmA, bar, m0 + i * 64, k);
          } else {
            tma_load_2d_pair(sa, &tmA, bar, k, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BNH / 64; ++i) tma_load_2d_pair(sb + i * 8192, &tmB, bar, n0 + i * 64, k);
          } else {
            tma_load_2d_pair(sb, &tmB, bar, k, n0);
          }
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      constexpr uint32_t idesc = make_idesc(TM, TN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int s = 0, acc = 0;
      uint32_t ph = 0, pacc = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < ntiles && ok; tile += n_clusters) {
        ok = mbar_wait(&tempty[acc], pacc ^ 1, p.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_base = smem_u32(smem + s * STAGE_BYTES);
            const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
              const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_base + k4 * (UMMA_K * 128), 8192, 1024)
                                          : make_smem_desc_sw128(a_base + k4 * (UMMA_K * 2), 16, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k4 * (UMMA_K * 128), 8192, 1024)
                                          : make_smem_desc_sw128(b_base + k4 * (UMMA_K * 2), 16, 1024);
              umma2_f16(d_tmem, adesc, bdesc, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
            }
            umma2_commit(smem_u32(&empty[s]));
            umma2_commit(map_to_rank(smem_u32(&empty[s]), 1));
            if (kb == kblocks - 1) {
              umma2_commit(smem_u32(&tfull[acc]));
              umma2_commit(map_to_rank(smem_u32(&tfull[acc]), 1));
            }
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        acc ^= 1;
        if (acc == 0) pacc ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const int row_in_half = quad * 32 + lane;
    const uint32_t tempty_leader0 = map_to_rank(smem_u32(&tempty[0]), 0);
    const uint32_t tempty_leader1 = map_to_rank(smem_u32(&tempty[1]), 0);
    int acc = 0;
    uint32_t pacc = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < ntiles && ok; tile += n_clusters) {
      ok = mbar_wait(&tfull[acc], pacc, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      int mi, ni;
      raster_tile(tile, mt, nt, p.group_m, mi, ni);
      const int row = mi * TM + static_cast<int>(rank) * BMH + row_in_half;
      const int col0 = ni * TN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * TN;
#pragma unroll 1
      for (int c = 0; c < TN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        store32(p, v, row, col0 + c * 32);
      }
      tc_fence_before();
      mbar_arrive_cluster(acc == 0 ? tempty_leader0 : tempty_leader1);
      acc ^= 1;
      if (acc == 0) pacc ^= 1;
    }
  }

  // nobody leaves while the peer may still signal into this CTA's shared memory or read its operand tiles
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const P2& p, cudaStream_t st) {
  static int max_clusters = -1;
  auto* fn = gemm_2cta_kernel<A_MN, B_MN>;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS, 1, 1);
  P2 q = p;
  q.group_m = gk::raster_group_m();
  q.stages = stages_setting() < 2 ? 2 : (stages_setting() > MAX_STAGES ? MAX_STAGES : stages_setting());
  cfg.dynamicSmemBytes = q.stages * STAGE_BYTES + 1024 + 256;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters < 0) {
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return static_cast<int>(cudaGetLastError());
    cfg.gridDim = dim3(2 * (gk::sm_count() / 2), 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = gk::sm_count() / 2 - 2;
    }
    max_clusters = n;
    cfg.dynamicSmemBytes = q.stages * STAGE_BYTES + 1024 + 256;
  }
  const long long tiles = static_cast<long long>((p.M + TM - 1) / TM) * ((p.N + TN - 1) / TN);
  const int clusters = static_cast<int>(tiles < max_clusters ? tiles : max_clusters);
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  if (cudaLaunchKernelEx(&cfg, fn, tmA, tmB, q) != cudaSuccess) {
    const int e = gk::launch_status();
    return e ? e : -7;
  }
  return gk::launch_status();
}

}  // namespace gk2

// Shared-memory ring depth of the pair kernel (2..7 stages of 32 KB per CTA).
GK_EXPORT void gk_gemm_2cta_set_stages(int n) { gk2::stages_setting() = n; }

// C[M,N] (ldc) = alpha * A . B^T (+ bias[N]) (+ C when accumulate); see the header comment.  a_rows / b_rows are the
// outer extents of the operand tensors as stored.  Returns 0, a negative argument error or a positive cudaError_t.
GK_EXPORT int gk_gemm_2cta(const void* A, long long lda, long long a_rows, int a_mn,  //
                           const void* B, long long ldb, long long b_rows, int b_mn,  //
                           void* C, long long ldc, int out_fp32, int accumulate, const void* bias, int bias_fp32,
                           float alpha, int M, int N, int K, int* err, void* stream) {
  using namespace gk2;
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if (a_mn && !b_mn) return -11;  // not a linear-layer layout; the one-CTA kernel serves it
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -15;
  CUtensorMap tmA, tmB;
  int rc = a_mn ? gk::make_tmap_2d(&tmA, A, 2, a_rows, M, lda, 64, 64, true)
                : gk::make_tmap_2d(&tmA, A, 2, a_rows, K, lda, BMH, 64, true);
  if (rc) return -20 + rc;
  rc = b_mn ? gk::make_tmap_2d(&tmB, B, 2, b_rows, N, ldb, 64, 64, true)
            : gk::make_tmap_2d(&tmB, B, 2, b_rows, K, ldb, BNH, 64, true);
  if (rc) return -30 + rc;
  P2 p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = bias; p.bias_fp32 = bias_fp32; p.alpha = alpha; p.err = err;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch2<false, false>(tmA, tmB, p, st);
  if (!a_mn && b_mn) return launch2<false, true>(tmA, tmB, p, st);
  return launch2<true, true>(tmA, tmB, p, st);
}
