// ZeRO-1 optimizer step over NVLink peer memory: gradient reduce-scatter, unscale / clip, sharded AdamW and the
// parameter all-gather as peer loads and stores issued by the optimizer kernel itself.
//
// Every rank of the data-parallel group keeps its flat fp32 gradient buffer and its flat bf16 parameter buffer in
// symmetric memory.  The owner of a shard
//   (1) pulls that shard of every peer's gradient buffer (16-byte peer loads), sums in fixed rank order, scales,
//   (2) applies AdamW to its fp32 master / moment shard,
//   (3) pushes the rounded bf16 parameters into every rank's parameter buffer (16-byte peer stores).
// mode 3 does all of it in one pass (no clipping: nothing depends on the global norm); with clipping the global
// norm sits between (1) and (2): mode 1 writes the reduced shard into the local gradient buffer, the norm is reduced,
// mode 2 finishes.  No library collective moves gradient or parameter bytes.  Ranks are ordered by gk_peer_barrier
// (epoch flags in symmetric memory, bounded waits): once before the first pull (every rank's backward is complete)
// and once after the last push (parameters have landed everywhere, gradients may be overwritten).
//
// Replaces the reference's mcore DistributedDataParallel reduce-scatter + DistributedOptimizer step + param
// all-gather (configured in gpatch_v4/training_backend/megatron_backend/mixin.py:311-348, optimizer.py:53-111).
#include "host_utils.h"
#include <cuda_bf16.h>
#include <stdint.h>

namespace gkz {

constexpr int MAX_RANKS = 8;
constexpr int THREADS = 256;
constexpr long long WAIT_CYCLES = 40000000000LL;  // ~20 s: data-parallel ranks may arrive far apart

struct Z1Params {
  const float* grads[MAX_RANKS];     // base of every rank's fp32 gradient buffer
  __nv_bfloat16* params[MAX_RANKS];  // base of every rank's bf16 parameter buffer
  long long shard_start;             // first element of this rank's shard inside the buffers
  long long n;                       // shard elements (multiple of 8)
  int rank, nranks, mode;
  float* reduced;                    // mode 1 out / mode 2 in: fp32 [n] (may alias the own gradient shard)
  float* master; float* m; float* v; // fp32 [n]
  float grad_scale;                  // 1 / dp x loss scale, applied after the sum
  const float* clip;                 // optional device scalar multiplied into the gradient (modes 2, 3)
  float* sumsq;                      // optional: += sum of squares of the scaled, reduced gradient (modes 1, 3)
  float lr, b1, b2, eps, wd, bc1, bc2;
};

__device__ __forceinline__ float4 ld_peer(const float* p) {
  float4 v;
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

constexpr int MAX_GRID = 4096;
// per-CTA partial sums of squares and the ticket that elects the CTA which adds them up (launches that ask for the
// norm are ordered on one stream per device)
__device__ float g_ss_part[MAX_GRID];
__device__ unsigned int g_ss_ticket;

__global__ void __launch_bounds__(THREADS) zero1_kernel(Z1Params p) {
  __shared__ float red[THREADS / 32];
  const long long nvec = p.n >> 3;
  const float clip = (p.clip ? *p.clip : 1.f);
  float ss = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(THREADS) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * THREADS) {
    float g[8];
    if (p.mode == 2) {
      const float4 a = reinterpret_cast<const float4*>(p.reduced)[2 * i], b = reinterpret_cast<const float4*>(p.reduced)[2 * i + 1];
      g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.f;
      // issue every rank's loads before the first add: NVLink latency overlaps across ranks
      float4 a[MAX_RANKS], b[MAX_RANKS];
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        if (r < p.nranks) {
          const float* src = p.grads[r] + p.shard_start + 8 * i;
          a[r] = ld_peer(src);
          b[r] = ld_peer(src + 4);
        }
      }
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        if (r < p.nranks) {
          g[0] += a[r].x; g[1] += a[r].y; g[2] += a[r].z; g[3] += a[r].w;
          g[4] += b[r].x; g[5] += b[r].y; g[6] += b[r].z; g[7] += b[r].w;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        g[j] *= p.grad_scale;
        ss += g[j] * g[j];
      }
    }
    if (p.mode == 1) {
      reinterpret_cast<float4*>(p.reduced)[2 * i] = make_float4(g[0], g[1], g[2], g[3]);
      reinterpret_cast<float4*>(p.reduced)[2 * i + 1] = make_float4(g[4], g[5], g[6], g[7]);
      continue;
    }
    float w[8], mm[8], vv[8];
    {
      const float4 a = reinterpret_cast<const float4*>(p.master)[2 * i], b = reinterpret_cast<const float4*>(p.master)[2 * i + 1];
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
      const float4 c = reinterpret_cast<const float4*>(p.m)[2 * i], d = reinterpret_cast<const float4*>(p.m)[2 * i + 1];
      mm[0] = c.x; mm[1] = c.y; mm[2] = c.z; mm[3] = c.w; mm[4] = d.x; mm[5] = d.y; mm[6] = d.z; mm[7] = d.w;
      const float4 e = reinterpret_cast<const float4*>(p.v)[2 * i], f = reinterpret_cast<const float4*>(p.v)[2 * i + 1];
      vv[0] = e.x; vv[1] = e.y; vv[2] = e.z; vv[3] = e.w; vv[4] = f.x; vv[5] = f.y; vv[6] = f.z; vv[7] = f.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * clip;
      mm[j] = p.b1 * mm[j] + (1.f - p.b1) * gj;
      vv[j] = p.b2 * vv[j] + (1.f - p.b2) * gj * gj;
      const float upd = (mm[j] / p.bc1) / (sqrtf(vv[j] / p.bc2) + p.eps) + p.wd * w[j];
      w[j] -= p.lr * upd;
    }
    reinterpret_cast<float4*>(p.master)[2 * i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(p.master)[2 * i + 1] = make_float4(w[4], w[5], w[6], w[7]);
    reinterpret_cast<float4*>(p.m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(p.m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    reinterpret_cast<float4*>(p.v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(p.v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 o;
    __nv_bfloat162 t2;
    t2 = __floats2bfloat162_rn(w[0], w[1]); o.x = *reinterpret_cast<uint32_t*>(&t2);
    t2 = __floats2bfloat162_rn(w[2], w[3]); o.y = *reinterpret_cast<uint32_t*>(&t2);
    t2 = __floats2bfloat162_rn(w[4], w[5]); o.z = *reinterpret_cast<uint32_t*>(&t2);
    t2 = __floats2bfloat162_rn(w[6], w[7]); o.w = *reinterpret_cast<uint32_t*>(&t2);
    // all-gather: the owner writes its shard into every rank's parameter buffer (own copy first)
#pragma unroll
    for (int pr = 0; pr < MAX_RANKS; ++pr) {
      if (pr < p.nranks) {
        const int dst = (p.rank + pr) % p.nranks;
        reinterpret_cast<uint4*>(p.params[dst] + p.shard_start)[i] = o;
      }
    }
  }
  if (p.sumsq && p.mode != 2) {
    // fixed-order reduction: shuffle tree inside a warp, warps in index order, CTAs in index order by whichever
    // CTA finishes last; the result does not depend on scheduling, so every run of the same grid gives the same norm
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffff, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < THREADS / 32; ++w) t += red[w];
      g_ss_part[blockIdx.x] = t;
      __threadfence();
      const unsigned int ticket = atomicAdd(&g_ss_ticket, 1u);
      if (ticket == gridDim.x - 1) {
        __threadfence();
        float tot = 0.f;
        for (unsigned int b = 0; b < gridDim.x; ++b) tot += __ldcg(&g_ss_part[b]);
        *p.sumsq += tot;
        g_ss_ticket = 0;
      }
    }
  }
}

// Barrier across the ranks of a group: publish `epoch` into slot [slot][rank] of every peer's flag array, then wait
// until every peer's epoch shows up in the own array.  One CTA, one thread per peer; waits are bounded.
__global__ void peer_barrier_kernel(uint32_t* const* flags_by_rank, int rank, int nranks, int slot, uint32_t epoch,
                                    int* err, long long budget, unsigned int* epoch_dev) {
  __threadfence_system();
  const int t = threadIdx.x;
  if (epoch_dev) {
    // the epoch lives on the device (the launch can be replayed from a CUDA graph with frozen arguments): every
    // thread reads the count of barriers done so far, the last statement of the kernel advances it
    epoch = *reinterpret_cast<volatile unsigned int*>(epoch_dev) + 1;
    __syncwarp();
  }
  if (t < nranks && t != rank) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags_by_rank[t] + slot * MAX_RANKS + rank), "r"(epoch)
                 : "memory");
    const uint32_t* f = flags_by_rank[rank] + slot * MAX_RANKS + t;
    const long long t0 = clock64();
    int spins = 0;
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if ((++spins & 63) == 0 && (clock64() - t0 > budget || *reinterpret_cast<volatile int*>(err) != 0)) {
        atomicCAS(err, 0, 6);
        break;
      }
    }
  }
  if (epoch_dev) {
    __syncwarp();
    if (t == 0) *epoch_dev = epoch;
  }
}

static long long g_barrier_budget = WAIT_CYCLES;

}  // namespace gkz

using namespace gkz;

// ptrs: [0..n) gradient buffer base of every rank, [n..2n) parameter buffer base of every rank.
GK_EXPORT int gk_zero1_step(int mode, const unsigned long long* ptrs, int rank, int nranks, long long shard_start,
                            long long n, float* reduced, float* master, float* m, float* v, float grad_scale,
                            const float* clip, float* sumsq, float lr, float b1, float b2, float eps, float wd, int step,
                            int ctas, void* stream) {
  if (n % 8 || shard_start % 8 || nranks < 1 || nranks > MAX_RANKS || mode < 1 || mode > 3) return -1;
  if (n == 0) return 0;
  Z1Params p;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.grads[r] = r < nranks ? reinterpret_cast<const float*>(ptrs[r]) : nullptr;
    p.params[r] = r < nranks ? reinterpret_cast<__nv_bfloat16*>(ptrs[nranks + r]) : nullptr;
  }
  p.shard_start = shard_start; p.n = n; p.rank = rank; p.nranks = nranks; p.mode = mode;
  p.reduced = reduced; p.master = master; p.m = m; p.v = v; p.grad_scale = grad_scale; p.clip = clip; p.sumsq = sumsq;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd;
  p.bc1 = 1.f - powf(b1, static_cast<float>(step));
  p.bc2 = 1.f - powf(b2, static_cast<float>(step));
  long long want = (n / 8 + THREADS - 1) / THREADS;
  int cap = ctas > 0 ? ctas : 4 * gk::sm_count();
  if (cap > MAX_GRID) cap = MAX_GRID;
  const int grid = static_cast<int>(want < cap ? want : cap);
  zero1_kernel<<<grid, THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return gk::launch_status();
}

// flags_dev: device array of nranks pointers (every rank's flag array, [slots][8] uint32, zero-initialised).
GK_EXPORT int gk_peer_barrier(const void* flags_dev, int rank, int nranks, int slot, unsigned int epoch, int* err,
                              void* stream) {
  if (nranks < 1 || nranks > MAX_RANKS) return -1;
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint32_t* const*>(flags_dev), rank, nranks, slot, epoch, err, gkz::g_barrier_budget, nullptr);
  return gk::launch_status();
}

// The same barrier with the epoch kept in device memory (`epoch_dev`: barriers completed so far on this slot, advanced
// by the kernel), so that the launch can be captured in a CUDA graph and replayed.
GK_EXPORT int gk_peer_barrier_dev(const void* flags_dev, int rank, int nranks, int slot, unsigned int* epoch_dev,
                                  int* err, void* stream) {
  if (nranks < 1 || nranks > MAX_RANKS || !epoch_dev) return -1;
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint32_t* const*>(flags_dev), rank, nranks, slot, 0u, err, gkz::g_barrier_budget, epoch_dev);
  return gk::launch_status();
}

// Clock cycles a rank waits for its peers in gk_peer_barrier before it gives up, writes error code 6 and returns
// (0 restores the default of ~20 s).  Failure-detection tests shorten it so that a missing peer shows up quickly.
GK_EXPORT void gk_set_peer_wait_budget(long long cycles) { gkz::g_barrier_budget = cycles > 0 ? cycles : gkz::WAIT_CYCLES; }
