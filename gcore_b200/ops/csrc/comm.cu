// Latency-oriented collectives over NVLink peer memory for the rollout decoder (small tensors, CUDA-graph friendly).
//
// One-shot all-reduce: every rank pushes its vector into slot [rank] of every peer's inbox (posted stores), publishes
// one flag per (source rank, CTA) in the peer's memory, then sums its own vector with the peers' slots as soon as the
// matching flags show the current epoch.  One kernel, one NVLink traversal, no ring steps: for the [batch, hidden]
// partial sums of a tensor-parallel decode step this costs a few microseconds where a library all-reduce costs tens.
//
// The call epoch lives in device memory (state[0]) and is advanced by the last CTA to finish, so the kernel can be
// replayed from a CUDA graph with frozen arguments.  Inboxes are double-buffered by epoch parity (a rank cannot
// complete call n+1 before every peer has started it, so slot parity n is no longer read when call n+2 overwrites it).
// Waits are bounded and report through the error word.
#include "host_utils.h"
#include <cuda_bf16.h>
#include <stdint.h>

namespace gkx {

constexpr int AR_CTAS = 32;
constexpr int AR_THREADS = 256;
constexpr int MAX_RANKS = 8;
constexpr long long WAIT_CYCLES = 1000000000LL;

struct ArParams {
  const __nv_bfloat16* in;
  __nv_bfloat16* out;
  long long n;                       // elements, multiple of 8
  int rank, nranks;
  long long slot_elems;              // capacity of one inbox slot (elements)
  __nv_bfloat16* inbox[MAX_RANKS];   // every rank's inbox base: [2 parity][nranks][slot_elems]
  uint32_t* flags[MAX_RANKS];        // every rank's flags: [2 parity][nranks][AR_CTAS]
  unsigned int* state;               // [0] calls completed, [1] CTA ticket
  int* err;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& w) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    acc[2 * q] += __uint_as_float((ww[q] & 0xFFFFu) << 16);
    acc[2 * q + 1] += __uint_as_float(ww[q] & 0xFFFF0000u);
  }
}

__global__ void __launch_bounds__(AR_THREADS) allreduce_oneshot_kernel(ArParams p) {
  __shared__ int s_ok;
  gk::pdl_launch_dependents();
  gk::pdl_wait();
  const unsigned int calls = *reinterpret_cast<volatile unsigned int*>(p.state);
  const int parity = calls & 1;
  const uint32_t epoch = (calls >> 1) + 1;
  const long long nvec = p.n >> 3;
  const long long per = (nvec + gridDim.x - 1) / gridDim.x;
  const long long v0 = static_cast<long long>(blockIdx.x) * per;
  long long v1 = v0 + per;
  if (v1 > nvec) v1 = nvec;
  const uint4* in = reinterpret_cast<const uint4*>(p.in);
  const long long slot_vec = p.slot_elems >> 3;
  // ---- push my slice to every peer
  for (int pr = 1; pr < p.nranks; ++pr) {
    const int peer = (p.rank + pr) % p.nranks;
    uint4* dst = reinterpret_cast<uint4*>(p.inbox[peer]) + (static_cast<long long>(parity) * p.nranks + p.rank) * slot_vec;
    for (long long i = v0 + threadIdx.x; i < v1; i += AR_THREADS) dst[i] = in[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int pr = 1; pr < p.nranks; ++pr) {
      const int peer = (p.rank + pr) % p.nranks;
      st_release_sys(p.flags[peer] + (parity * p.nranks + p.rank) * AR_CTAS + blockIdx.x, epoch);
    }
    // ---- wait for the same slice from every peer (bounded)
    int ok = 1;
    const long long t0 = clock64();
    for (int pr = 1; pr < p.nranks && ok; ++pr) {
      const int src = (p.rank + pr) % p.nranks;
      const uint32_t* f = p.flags[p.rank] + (parity * p.nranks + src) * AR_CTAS + blockIdx.x;
      int spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
        if ((++spins & 63) == 0 && (clock64() - t0 > WAIT_CYCLES || *reinterpret_cast<volatile int*>(p.err) != 0)) {
          atomicCAS(p.err, 0, 5);
          ok = 0;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const uint4* mine = reinterpret_cast<const uint4*>(p.inbox[p.rank]) + static_cast<long long>(parity) * p.nranks * slot_vec;
    uint4* out = reinterpret_cast<uint4*>(p.out);
    for (long long i = v0 + threadIdx.x; i < v1; i += AR_THREADS) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8(acc, in[i]);
      // fixed summation order (rank 0, 1, ...) so that every rank produces bit-identical results
      float tot[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.nranks; ++r) {
        if (r == p.rank) {
#pragma unroll
          for (int j = 0; j < 8; ++j) tot[j] += acc[j];
        } else {
          add8(tot, __ldcg(mine + static_cast<long long>(r) * slot_vec + i));
        }
      }
      uint4 o;
      __nv_bfloat162 t2;
      t2 = __floats2bfloat162_rn(tot[0], tot[1]); o.x = *reinterpret_cast<uint32_t*>(&t2);
      t2 = __floats2bfloat162_rn(tot[2], tot[3]); o.y = *reinterpret_cast<uint32_t*>(&t2);
      t2 = __floats2bfloat162_rn(tot[4], tot[5]); o.z = *reinterpret_cast<uint32_t*>(&t2);
      t2 = __floats2bfloat162_rn(tot[6], tot[7]); o.w = *reinterpret_cast<uint32_t*>(&t2);
      out[i] = o;
    }
  }
  // ---- the last CTA to finish advances the call counter
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int ticket = atomicAdd(p.state + 1, 1u);
    if (ticket == gridDim.x - 1) {
      p.state[1] = 0;
      __threadfence();
      p.state[0] = calls + 1;
    }
  }
}

// ---- all-reduce + residual add + RMSNorm in one kernel (tensor-parallel decode: the partial sums of a row-parallel
// projection go straight into the next norm).  Same exchange as above, but a CTA owns whole rows: it pushes its rows'
// partials to every peer, waits for the peers' partials of the same rows, and then per row
//   a   = bf16(sum over ranks, fixed order)            (what the separate all-reduce would have stored)
//   res = bf16(a + residual)                           -> res_out      (a alone when there is no residual)
//   y   = bf16(res * rsqrt(mean(res^2) + eps) * gamma) -> y
// The new residual is bit-identical to all-reduce followed by the RMSNorm kernel of elementwise.cu; the normalised
// output agrees to rounding (the sum of squares is added up in another order) and is identical on every rank.
struct ArNormParams {
  ArParams ar;                  // in = partial [rows, H]; out unused; n = rows * H
  const __nv_bfloat16* res_in;  // may be null
  const __nv_bfloat16* gamma;   // [H]
  __nv_bfloat16* res_out;       // [rows, H]
  __nv_bfloat16* y;             // [rows, H]
  int rows, H;
  float eps;
};

__device__ __forceinline__ void unpack_bf16x8(const uint4& w, float (&f)[8]) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    f[2 * q] = __uint_as_float((ww[q] & 0xFFFFu) << 16);
    f[2 * q + 1] = __uint_as_float(ww[q] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 o;
  __nv_bfloat162 t2;
  t2 = __floats2bfloat162_rn(f[0], f[1]); o.x = *reinterpret_cast<uint32_t*>(&t2);
  t2 = __floats2bfloat162_rn(f[2], f[3]); o.y = *reinterpret_cast<uint32_t*>(&t2);
  t2 = __floats2bfloat162_rn(f[4], f[5]); o.z = *reinterpret_cast<uint32_t*>(&t2);
  t2 = __floats2bfloat162_rn(f[6], f[7]); o.w = *reinterpret_cast<uint32_t*>(&t2);
  return o;
}


__global__ void __launch_bounds__(AR_THREADS) allreduce_rmsnorm_kernel(ArNormParams q) {
  __shared__ int s_ok;
  const ArParams& p = q.ar;
  gk::pdl_launch_dependents();
  gk::pdl_wait();
  const unsigned int calls = *reinterpret_cast<volatile unsigned int*>(p.state);
  const int parity = calls & 1;
  const uint32_t epoch = (calls >> 1) + 1;
  const int hv = q.H >> 3;
  const int rpc = (q.rows + gridDim.x - 1) / gridDim.x;
  int r0 = blockIdx.x * rpc, r1 = r0 + rpc;
  if (r0 > q.rows) r0 = q.rows;
  if (r1 > q.rows) r1 = q.rows;
  const long long v0 = static_cast<long long>(r0) * hv, v1 = static_cast<long long>(r1) * hv;
  const uint4* in = reinterpret_cast<const uint4*>(p.in);
  const long long slot_vec = p.slot_elems >> 3;
  for (int pr = 1; pr < p.nranks; ++pr) {
    const int peer = (p.rank + pr) % p.nranks;
    uint4* dst = reinterpret_cast<uint4*>(p.inbox[peer]) + (static_cast<long long>(parity) * p.nranks + p.rank) * slot_vec;
    for (long long i = v0 + threadIdx.x; i < v1; i += AR_THREADS) dst[i] = in[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int pr = 1; pr < p.nranks; ++pr) {
      const int peer = (p.rank + pr) % p.nranks;
      st_release_sys(p.flags[peer] + (parity * p.nranks + p.rank) * AR_CTAS + blockIdx.x, epoch);
    }
    int ok = 1;
    const long long t0 = clock64();
    for (int pr = 1; pr < p.nranks && ok; ++pr) {
      const int src = (p.rank + pr) % p.nranks;
      const uint32_t* f = p.flags[p.rank] + (parity * p.nranks + src) * AR_CTAS + blockIdx.x;
      int spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
        if ((++spins & 63) == 0 && (clock64() - t0 > WAIT_CYCLES || *reinterpret_cast<volatile int*>(p.err) != 0)) {
          atomicCAS(p.err, 0, 5);
          ok = 0;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    // one warp per row (the rows of a CTA run side by side, no block-wide barrier): pass 1 sums the ranks' partials in
    // rank order, adds the residual, stores the new residual and accumulates the sum of squares; pass 2 re-reads the
    // row it just wrote (L1 / L2) and writes the normalised output
    const uint4* mine = reinterpret_cast<const uint4*>(p.inbox[p.rank]) + static_cast<long long>(parity) * p.nranks * slot_vec;
    const uint4* gv = reinterpret_cast<const uint4*>(q.gamma);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int row = r0 + warp; row < r1; row += AR_THREADS / 32) {
      const long long rb = static_cast<long long>(row) * hv;
      float ss = 0.f;
      for (int c = lane; c < hv; c += 32) {
        float tot[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < p.nranks; ++r) {
          const uint4 w = r == p.rank ? in[rb + c] : __ldcg(mine + static_cast<long long>(r) * slot_vec + rb + c);
          add8(tot, w);
        }
        float f[8];
        unpack_bf16x8(pack_bf16x8(tot), f);  // the value a stand-alone all-reduce would have stored
        if (q.res_in) {
          float g[8];
          unpack_bf16x8(reinterpret_cast<const uint4*>(q.res_in)[rb + c], g);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] += g[j];
        }
        const uint4 stored = pack_bf16x8(f);
        reinterpret_cast<uint4*>(q.res_out)[rb + c] = stored;
        unpack_bf16x8(stored, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / q.H + q.eps);
      for (int c = lane; c < hv; c += 32) {
        float f[8], g[8], o[8];
        unpack_bf16x8(reinterpret_cast<const uint4*>(q.res_out)[rb + c], f);   // this lane's own store
        unpack_bf16x8(gv[c], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = f[j] * rstd * g[j];
        reinterpret_cast<uint4*>(q.y)[rb + c] = pack_bf16x8(o);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int ticket = atomicAdd(p.state + 1, 1u);
    if (ticket == gridDim.x - 1) {
      p.state[1] = 0;
      __threadfence();
      p.state[0] = calls + 1;
    }
  }
}

// Segment gather / reduce over peer memory for context parallelism: out[i] = sum over the segments that cover i of
// seg.src[i - seg.start], in segment order (fp32 accumulation, bf16 in and out).  With disjoint segments this is the
// pull of the K/V rows a rank needs from the ranks that own them; with overlapping segments it is the return of the
// partial dK/dV rows to their owner (a reduce-scatter whose summation order is fixed, hence deterministic).
constexpr int MAX_SEGS = 16;
struct RowsSeg { const __nv_bfloat16* src; long long start, end; };
struct RowsParams { __nv_bfloat16* dst; long long n; int nseg; RowsSeg seg[MAX_SEGS]; };

__global__ void __launch_bounds__(256) peer_rows_kernel(RowsParams p) {
  const long long nvec = p.n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i << 3;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 only = make_uint4(0, 0, 0, 0);
    int hits = 0;
    for (int s = 0; s < p.nseg; ++s) {
      if (e >= p.seg[s].start && e < p.seg[s].end) {
        uint4 v;
        asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p.seg[s].src + (e - p.seg[s].start)) : "memory");
        add8(acc, v);
        only = v;
        ++hits;
      }
    }
    uint4 o = only;  // a single source is copied bit-exactly
    if (hits != 1) {
      __nv_bfloat162 t2;
      t2 = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&t2);
      t2 = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&t2);
      t2 = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&t2);
      t2 = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&t2);
    }
    reinterpret_cast<uint4*>(p.dst)[i] = o;
  }
}

// dst[i, 0:cols] = src[i, 0:cols] for i < rows; src may be a peer GPU's memory (weight resync pulls the pieces of a
// rollout tensor straight out of the trainer ranks' staged shards).  16-byte vectors; cols, leading dimensions and
// both base addresses are multiples of 8 elements.
__global__ void __launch_bounds__(256) peer_copy_2d_kernel(__nv_bfloat16* __restrict__ dst, long long dst_ld,
                                                           const __nv_bfloat16* __restrict__ src, long long src_ld,
                                                           long long rows, int cols) {
  const int cv = cols >> 3;
  const long long n = rows * cv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cv;
    const int c = static_cast<int>(i - r * cv);
    uint4 v;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + r * src_ld + c * 8) : "memory");
    *reinterpret_cast<uint4*>(dst + r * dst_ld + c * 8) = v;
  }
}

}  // namespace gkx

using namespace gkx;

GK_EXPORT int gk_peer_copy_2d(void* dst, long long dst_ld, const void* src, long long src_ld, long long rows, int cols,
                              void* stream) {
  if ((cols & 7) || (dst_ld & 7) || (src_ld & 7) || (reinterpret_cast<uintptr_t>(dst) & 15) ||
      (reinterpret_cast<uintptr_t>(src) & 15))
    return -1;
  if (rows == 0 || cols == 0) return 0;
  const long long n = rows * (cols >> 3);
  long long want = (n + 255) / 256;
  const long long cap = 8LL * gk::sm_count();
  peer_copy_2d_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(dst), dst_ld, reinterpret_cast<const __nv_bfloat16*>(src), src_ld, rows, cols);
  return gk::launch_status();
}

// segs: nseg triples (source address, first element, end element) in destination element coordinates; all multiples
// of 8 elements.  Elements covered by no segment become zero.
GK_EXPORT int gk_peer_rows(void* dst, long long n, int nseg, const unsigned long long* segs, void* stream) {
  if (n % 8 || nseg < 0 || nseg > MAX_SEGS) return -1;
  if (n == 0) return 0;
  RowsParams p;
  p.dst = reinterpret_cast<__nv_bfloat16*>(dst);
  p.n = n;
  p.nseg = nseg;
  for (int s = 0; s < nseg; ++s) {
    p.seg[s].src = reinterpret_cast<const __nv_bfloat16*>(segs[3 * s]);
    p.seg[s].start = static_cast<long long>(segs[3 * s + 1]);
    p.seg[s].end = static_cast<long long>(segs[3 * s + 2]);
    if ((p.seg[s].start | p.seg[s].end) & 7) return -2;
  }
  long long want = (n / 8 + 255) / 256;
  const long long cap = 8LL * gk::sm_count();
  peer_rows_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return gk::launch_status();
}

// 1: kernels of the decode chain are launched with programmatic stream serialization (see host_utils.h)
GK_EXPORT void gk_set_pdl(int on) { gk::pdl_flag() = on; }

GK_EXPORT int gk_allreduce_ctas() { return AR_CTAS; }

// ptrs: [0..n) inbox base of every rank, [n..2n) flag base of every rank (device pointers as integers).
// in / out may alias.  n must be a multiple of 8 and at most slot_elems.
GK_EXPORT int gk_allreduce_oneshot(const void* in, void* out, long long n, int rank, int nranks, long long slot_elems,
                                   const unsigned long long* ptrs, unsigned int* state, int* err, void* stream) {
  if (n % 8 || n > slot_elems || nranks < 1 || nranks > MAX_RANKS) return -1;
  if (n == 0) return 0;
  ArParams p;
  p.in = reinterpret_cast<const __nv_bfloat16*>(in);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.n = n; p.rank = rank; p.nranks = nranks; p.slot_elems = slot_elems;
  for (int r = 0; r < nranks; ++r) {
    p.inbox[r] = reinterpret_cast<__nv_bfloat16*>(ptrs[r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(ptrs[nranks + r]);
  }
  p.state = state;
  p.err = err;
  gk::launch_k(allreduce_oneshot_kernel, dim3(AR_CTAS), dim3(AR_THREADS), 0, reinterpret_cast<cudaStream_t>(stream), p);
  return gk::launch_status();
}

// partial [rows, H] bf16 (this rank's partial sums) -> res_out = all-reduce(partial) + res_in, y = RMSNorm(res_out) * gamma.
// Shares inboxes, flags and the call counter with gk_allreduce_oneshot (same ptrs / state).  H % 8 == 0, H <= 8192,
// rows * H <= slot_elems.  res_in may be null and may alias res_out.
GK_EXPORT int gk_allreduce_rmsnorm(const void* partial, const void* res_in, const void* gamma, void* res_out, void* y,
                                   int rows, int H, float eps, int rank, int nranks, long long slot_elems,
                                   const unsigned long long* ptrs, unsigned int* state, int* err, void* stream) {
  const long long n = static_cast<long long>(rows) * H;
  if (H % 8 || n > slot_elems || nranks < 1 || nranks > MAX_RANKS) return -1;
  if (rows == 0) return 0;
  ArNormParams q;
  q.ar.in = reinterpret_cast<const __nv_bfloat16*>(partial);
  q.ar.out = nullptr;
  q.ar.n = n; q.ar.rank = rank; q.ar.nranks = nranks; q.ar.slot_elems = slot_elems;
  for (int r = 0; r < nranks; ++r) {
    q.ar.inbox[r] = reinterpret_cast<__nv_bfloat16*>(ptrs[r]);
    q.ar.flags[r] = reinterpret_cast<uint32_t*>(ptrs[nranks + r]);
  }
  q.ar.state = state;
  q.ar.err = err;
  q.res_in = reinterpret_cast<const __nv_bfloat16*>(res_in);
  q.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  q.res_out = reinterpret_cast<__nv_bfloat16*>(res_out);
  q.y = reinterpret_cast<__nv_bfloat16*>(y);
  q.rows = rows; q.H = H; q.eps = eps;
  gk::launch_k(allreduce_rmsnorm_kernel, dim3(AR_CTAS), dim3(AR_THREADS), 0, reinterpret_cast<cudaStream_t>(stream), q);
  return gk::launch_status();
}
