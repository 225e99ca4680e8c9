// Decode-shaped GEMM: y[T, N] = x[T, K] . W[N, K]^T (+ bias) for T <= 128 tokens, where the weight is the only
// operand of any size and the kernel's job is to stream it from HBM once with every SM busy and little fixed cost.
//
//   * swap-AB: the 128-row tcgen05 tile runs over output features (rows of W), the token count is the MMA N
//     (16..128), so no tensor-core work is wasted on padding tokens.
//   * split-K over a thread-block cluster: the KS CTAs of a cluster each contract one K slice of the same 128
//     output features, so tiles x KS CTAs fill the GPU even when N / 128 is small (projections of one TP shard).
//   * the partial sums never touch global memory: they are reduce-scattered through distributed shared memory
//     (each CTA owns a slice of the token columns, receives the KS partials of that slice in its own shared memory,
//     adds them and stores its slice), ordered by one cluster barrier.
//
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue (thread = TMEM lane = output feature).
#include "ptx.cuh"
#include "host_utils.h"

namespace gks {
using namespace gk;

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr int A_BYTES = BM * BK * 2;

struct SkParams {
  int T, Tp, N, K, ks, stages;
  void* Y;
  long long ldy;
  int out_fp32;
  const void* bias;
  int bias_fp32;
  int* err;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, SkParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = A_BYTES + p.Tp * 128;
  uint8_t* red_buf = smem + p.stages * stage_bytes;                  // [ks slots][cols per slice][128 rows] fp32
  const int red_bytes = p.ks > 1 ? p.Tp * BM * 4 : 0;
  uint64_t* full = reinterpret_cast<uint64_t*>(red_buf + red_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tfull = empty + MAX_STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tfull + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = p.ks > 1 ? cluster_ctarank() : 0;
  const int tile = blockIdx.x / p.ks;
  const int n0 = tile * BM;
  const int kb_total = (p.K + BK - 1) / BK;
  const int per = (kb_total + p.ks - 1) / p.ks;
  const int kb0 = rank * per;
  const int kblocks = (kb0 + per <= kb_total ? per : (kb_total > kb0 ? kb_total - kb0 : 0));
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.Tp)) tmem_cols <<= 1;

  // Lane 0 of the producer warp initialises the barriers and puts the first loads in flight before anything else
  // happens in the CTA: the tensor-memory allocation, the CTA barrier and the cluster hand-shake all overlap them.
  int pre = 0;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(tfull, 1);
    fence_barrier_init();
    pre = kblocks < p.stages ? kblocks : p.stages;
    // the weight tiles do not depend on the previous kernel: they start streaming while it drains
    for (int kb = 0; kb < pre; ++kb) {
      mbar_expect_tx(&full[kb], stage_bytes);
      tma_load_2d(smem + kb * stage_bytes, &tmW, &full[kb], (kb0 + kb) * BK, n0);
    }
    pdl_wait();  // the activations do
    for (int kb = 0; kb < pre; ++kb)
      tma_load_2d(smem + kb * stage_bytes + A_BYTES, &tmX, &full[kb], (kb0 + kb) * BK, 0);
  }
  if (warp == 2) { tmem_alloc(tmem_holder, tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  // first half of "every CTA of the cluster is running"; the matching wait sits right before the first remote store
  if (p.ks > 1) cluster_arrive();
  pdl_wait();

  bool ok = true;
  if (warp == 0) {
    pre = __shfl_sync(0xffffffff, pre, 0);
    int s = pre == p.stages ? 0 : pre;
    uint32_t ph = pre == p.stages ? 1 : 0;
    for (int kb = pre; kb < kblocks && ok; ++kb) {
      ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
      if (!ok) break;
      if (lane == 0) {
        uint8_t* sa = smem + s * stage_bytes;
        mbar_expect_tx(&full[s], stage_bytes);
        tma_load_2d(sa, &tmW, &full[s], (kb0 + kb) * BK, n0);
        tma_load_2d(sa + A_BYTES, &tmX, &full[s], (kb0 + kb) * BK, 0);
      }
      __syncwarp();
      if (++s == p.stages) { s = 0; ph ^= 1; }
    }
    if (p.ks > 1) cluster_wait();
  } else if (warp == 1) {
    const uint32_t idesc = make_idesc(BM, p.Tp, 1, 1, 0, 0);
    int s = 0;
    uint32_t ph = 0;
    for (int kb = 0; kb < kblocks && ok; ++kb) {
      ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_base = smem_u32(smem + s * stage_bytes), b_base = a_base + A_BYTES;
#pragma unroll
        for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
          umma_f16(tmem_base, make_smem_desc_sw128(a_base + k4 * (UMMA_K * 2), 16, 1024),
                   make_smem_desc_sw128(b_base + k4 * (UMMA_K * 2), 16, 1024), idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        if (kb == kblocks - 1) umma_commit(tfull);
      }
      __syncwarp();
      if (++s == p.stages) { s = 0; ph ^= 1; }
    }
    if (p.ks > 1) cluster_wait();
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // output feature inside the tile = TMEM lane
    if (kblocks > 0) {
      ok = mbar_wait(tfull, 0, p.err, ERR_WAIT_TMEM_FULL);
      tc_fence_after();
    }
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int feat = n0 + row;
    float bias = 0.f;
    if (p.bias && feat < p.N) {
      bias = p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[feat]
                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[feat]);
    }
    if (p.ks == 1) {
      for (int c = 0; c < p.Tp / 16; ++c) {
        uint32_t r[16];
        if (kblocks > 0 && ok) { tmem_ld16(taddr + c * 16, r); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0;
        }
        if (feat < p.N && ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = c * 16 + j;
            if (tok < p.T) {
              const float v = __uint_as_float(r[j]) + bias;
              if (p.out_fp32) reinterpret_cast<float*>(p.Y)[tok * p.ldy + feat] = v;
              else reinterpret_cast<__nv_bfloat16*>(p.Y)[tok * p.ldy + feat] = __float2bfloat16(v);
            }
          }
        }
      }
    } else {
      // reduce-scatter over the cluster: token column `tok` belongs to CTA tok / cs, slot = my rank
      const int cs = p.Tp / p.ks;
      const uint32_t red_local = smem_u32(red_buf);
      cluster_wait();  // every CTA of the cluster has started: its shared memory may be written
      for (int c = 0; c < p.Tp / 16; ++c) {
        uint32_t r[16];
        if (kblocks > 0 && ok) { tmem_ld16(taddr + c * 16, r); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = c * 16 + j;
          const uint32_t owner = tok / cs;
          const int cj = tok - owner * cs;
          const uint32_t off = ((rank * cs + cj) * BM + row) * 4;
          st_cluster_f32(map_to_cta(red_local + off, owner), __uint_as_float(r[j]));
        }
      }
    }
    tc_fence_before();
  }
  if (p.ks > 1) {
    cluster_sync_all();  // all partials have landed in their owners' shared memory
    if (warp >= 2) {
      const int quad = warp & 3;
      const int row = quad * 32 + lane;
      const int feat = n0 + row;
      const int cs = p.Tp / p.ks;
      const float* red = reinterpret_cast<const float*>(red_buf);
      float bias = 0.f;
      if (p.bias && feat < p.N) {
        bias = p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[feat]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[feat]);
      }
      const bool healthy = *reinterpret_cast<volatile int*>(p.err) == 0;
      for (int cj = 0; cj < cs; ++cj) {
        const int tok = rank * cs + cj;
        if (tok >= p.T || feat >= p.N || !healthy) continue;
        float v = bias;
        for (int r = 0; r < p.ks; ++r) v += red[(r * cs + cj) * BM + row];
        if (p.out_fp32) reinterpret_cast<float*>(p.Y)[tok * p.ldy + feat] = v;
        else reinterpret_cast<__nv_bfloat16*>(p.Y)[tok * p.ldy + feat] = __float2bfloat16(v);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
}

}  // namespace gks

using namespace gks;

static int skinny_smem_bytes(int Tp, int ks, int K, int* stages_out) {
  const int stage_bytes = A_BYTES + Tp * 128;
  const int red_bytes = ks > 1 ? Tp * BM * 4 : 0;
  const int budget = gk::decode_smem_cap() > 0 ? gk::decode_smem_cap() : 200 * 1024;
  int stages = (budget - red_bytes - 1024 - 256) / stage_bytes;
  if (stages < 3) stages = 3;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  const int kb_per = ((K + BK - 1) / BK + ks - 1) / ks;
  if (stages > kb_per) stages = kb_per < 2 ? 2 : kb_per;
  if (stages_out) *stages_out = stages;
  return stages * stage_bytes + red_bytes + 1024 + 256;
}

static int skinny_configure() {
  static bool done = false;
  if (!done) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return -6;
    done = true;
  }
  return 0;
}

// How many clusters of `ks` CTAs of this kernel the GPU can hold at once (one wave).
GK_EXPORT int gk_gemm_skinny_max_clusters(int Tp, int ks, int K) {
  if (skinny_configure()) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ks * 148, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = skinny_smem_bytes(Tp, ks, K, nullptr);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_skinny_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

// W [N, K] and X [T, K] bf16 row-major (K contiguous, leading dimensions multiples of 8), T <= 128;
// ks in 1..8 CTAs per cluster; Tp >= T is the padded token count (multiple of 16 and of ks, at most 256).
GK_EXPORT int gk_gemm_skinny(const void* W, long long ldw, const void* X, long long ldx, void* Y, long long ldy,
                             int out_fp32, const void* bias, int bias_fp32, int T, int Tp, int N, int K, int ks,
                             int* err, void* stream) {
  if (T < 1 || T > 128 || ks < 1 || ks > 8 || Tp < T || Tp > 256 || Tp % 16 || Tp % ks) return -1;
  if ((ldw & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(X) & 15)) return -3;
  CUtensorMap tmW, tmX;
  if (gk::make_tmap_2d(&tmW, W, 2, N, K, ldw, BM, BK, true)) return -4;
  if (gk::make_tmap_2d(&tmX, X, 2, T, K, ldx, Tp, BK, true)) return -5;
  SkParams p;
  p.T = T; p.Tp = Tp; p.N = N; p.K = K; p.ks = ks;
  p.Y = Y; p.ldy = ldy; p.out_fp32 = out_fp32; p.bias = bias; p.bias_fp32 = bias_fp32; p.err = err;
  int stages = 0;
  const int smem = skinny_smem_bytes(Tp, ks, K, &stages);
  p.stages = stages;
  if (skinny_configure()) return -6;
  const int tiles = (N + BM - 1) / BM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * ks, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = gk::pdl_flag() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, tmW, tmX, p) != cudaSuccess) return gk::launch_status() ? gk::launch_status() : -7;
  return gk::launch_status();
}
