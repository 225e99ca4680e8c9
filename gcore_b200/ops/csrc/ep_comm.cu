// Expert-parallel dispatch / combine over NVLink peer memory.
//
// The reference moves MoE tokens with one count all-to-all, three uneven all-to-alls (rows, expert ids, weights), a
// host-synchronised split computation, a local sort into expert order and a reverse all-to-all
// (gpatch_v4/models/deepseek_v4/modeling_deepseek_v4.py:1221-1289, a2a.py:23-134; DeepEP variant deepep_a2a.py:77-281).
// Here the exchange is three kernels that address the peers' symmetric buffers directly:
//
//   ep_plan   every rank publishes its per-expert counts into every peer's table (peer stores + epoch flags), waits
//             (bounded) for the peers' counts and derives, without the host: the padded expert-sorted layout of its
//             own receive buffer (offsets for the grouped GEMM) and, for every expert anywhere, the row at which its
//             own tokens start inside the owner's buffer.
//   ep_push   permute + all-to-all in one pass: each (token, k) row is written straight to its final expert-sorted
//             row in the owner's buffer (optionally scaled: the backward of the weighted combine), and the padding
//             rows of the own buffer are zeroed.
//   ep_pull   all-to-all + un-permute + weighted top-k sum in one pass: each token reads its k expert-output rows
//             from the owners' buffers and accumulates them in fp32.
//
// Ranks meet at ep_plan and at gk_peer_barrier (zero1.cu) between push -> grouped GEMM -> pull.
#include "host_utils.h"
#include <cuda_bf16.h>
#include <stdint.h>

namespace gke {

constexpr int MAX_RANKS = 8;
constexpr int MAX_EXPERTS = 512;
constexpr long long WAIT_CYCLES = 40000000000LL;

struct PlanParams {
  const int* cnt;               // [E] rows this rank sends to each global expert
  int* cnt_all[MAX_RANKS];      // every rank's table [2 parity][ep][E]
  uint32_t* flags[MAX_RANKS];   // every rank's flags [2 parity][ep]
  int rank, ep, E, E_local, seg, R_max, parity;
  uint32_t epoch;
  unsigned int* calls_dev;      // optional: calls so far, kept on the device (parity / epoch derive from it)
  int* send_base;               // [E]   first row of my tokens for expert g inside its owner's buffer
  int* offsets;                 // [E_local + 1] padded segment starts of my own buffer
  int* tot_local;               // [E_local] real rows per local expert
  int* err;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) ep_plan_kernel(PlanParams p) {
  __shared__ int s_tot[MAX_EXPERTS], s_before[MAX_EXPERTS], s_pad[MAX_EXPERTS];
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  if (p.calls_dev) {   // replayable form: the call number comes from device memory and is advanced at the end
    const unsigned int calls = *reinterpret_cast<volatile unsigned int*>(p.calls_dev);
    p.parity = calls & 1;
    p.epoch = (calls >> 1) + 1;
    __syncthreads();
    if (tid == 0) *p.calls_dev = calls + 1;
  }
  for (int g = tid; g < p.E; g += blockDim.x) {
    const int c = p.cnt[g];
    for (int r = 0; r < p.ep; ++r) p.cnt_all[r][(p.parity * p.ep + p.rank) * p.E + g] = c;
  }
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < p.ep && tid != p.rank) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[tid] + p.parity * p.ep + p.rank), "r"(p.epoch)
                 : "memory");
    const uint32_t* f = p.flags[p.rank] + p.parity * p.ep + tid;
    const long long t0 = clock64();
    int spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - p.epoch) < 0) {
      if ((++spins & 63) == 0 && (clock64() - t0 > WAIT_CYCLES || *reinterpret_cast<volatile int*>(p.err) != 0)) {
        atomicCAS(p.err, 0, 8);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int* table = p.cnt_all[p.rank] + p.parity * p.ep * p.E;
  for (int g = tid; g < p.E; g += blockDim.x) {
    int tot = 0, before = 0;
    for (int r = 0; r < p.ep; ++r) {
      const int c = __ldcg(table + r * p.E + g);
      tot += c;
      if (r < p.rank) before += c;
    }
    s_tot[g] = tot;
    s_before[g] = before;
    s_pad[g] = (tot + p.seg - 1) / p.seg * p.seg;
  }
  __syncthreads();
  for (int g = tid; g < p.E; g += blockDim.x) {
    const int d = g / p.E_local, e = g - d * p.E_local;
    int off = 0;
    for (int j = 0; j < e; ++j) off += s_pad[d * p.E_local + j];
    p.send_base[g] = off + s_before[g];
    if (off + s_pad[g] > p.R_max) atomicCAS(p.err, 0, 7);  // a receive buffer would overflow
    if (d == p.rank) {
      p.offsets[e] = off;
      p.tot_local[e] = s_tot[g];
      if (e == p.E_local - 1) p.offsets[p.E_local] = off + s_pad[g];
    }
  }
}

struct PushParams {
  const __nv_bfloat16* x;       // [T, H]
  const float* scale;           // optional [T*K]
  const int* idx;               // [T*K] global expert of every (token, k)
  const int* pos;               // [T*K] position among this rank's rows for that expert
  const int* send_base;         // [E]
  const int* offsets;           // [E_local + 1]
  const int* tot_local;         // [E_local]
  __nv_bfloat16* recv[MAX_RANKS];
  int* dst_row;                 // [T*K] out: owner * R_max + row
  int rank, ep, E_local, seg, R_max, K, H;
  long long npairs;
};

__global__ void __launch_bounds__(256) ep_push_kernel(PushParams p) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int hv = p.H >> 3;
  if (warp < p.npairs) {
    const int g = p.idx[warp];
    const int d = g / p.E_local;
    const int row = p.send_base[g] + p.pos[warp];
    if (lane == 0) p.dst_row[warp] = d * p.R_max + row;
    if (row >= p.R_max) return;
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (warp / p.K) * p.H);
    uint4* dst = reinterpret_cast<uint4*>(p.recv[d] + static_cast<long long>(row) * p.H);
    if (p.scale) {
      const float s = p.scale[warp];
      for (int i = lane; i < hv; i += 32) {
        uint4 v = src[i];
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float lo = __uint_as_float((w[q] & 0xFFFFu) << 16) * s, hi = __uint_as_float(w[q] & 0xFFFF0000u) * s;
          __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi);
          w[q] = *reinterpret_cast<uint32_t*>(&t2);
        }
        dst[i] = v;
      }
    } else {
      for (int i = lane; i < hv; i += 32) dst[i] = src[i];
    }
  } else {
    // zero the padding rows of the own buffer (disjoint from every row a peer writes)
    const long long j = warp - p.npairs;
    if (j >= static_cast<long long>(p.E_local) * p.seg) return;
    const int e = static_cast<int>(j / p.seg), r = static_cast<int>(j - static_cast<long long>(e) * p.seg);
    const int row = p.offsets[e] + p.tot_local[e] + r;
    if (row >= p.offsets[e + 1] || row >= p.R_max) return;
    uint4* dst = reinterpret_cast<uint4*>(p.recv[p.rank] + static_cast<long long>(row) * p.H);
    for (int i = lane; i < hv; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
  }
}

struct PullParams {
  const __nv_bfloat16* src[MAX_RANKS];  // every rank's expert-output buffer [R_max, H]
  const int* dst_row;                   // [T*K]
  const float* weight;                  // optional [T*K] (absent: plain sum)
  __nv_bfloat16* y;                     // [T, H]
  __nv_bfloat16* gathered;              // optional [T*K, H]: the raw rows, kept for the weight gradient
  int K, H, R_max;
  long long T;
};

__global__ void __launch_bounds__(256) ep_pull_kernel(PullParams p) {
  const long long t = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= p.T) return;
  const int hv = p.H >> 3;
  for (int c = lane; c < hv; c += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < p.K; k0 += 8) {
      uint4 v[8];
      float w[8];
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        if (k0 + kk < p.K) {
          const int pr = p.dst_row[t * p.K + k0 + kk];
          const int d = pr / p.R_max, row = pr - d * p.R_max;
          v[kk] = ld_peer16(reinterpret_cast<const uint4*>(p.src[d] + static_cast<long long>(row) * p.H) + c);
          w[kk] = p.weight ? p.weight[t * p.K + k0 + kk] : 1.f;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        if (k0 + kk < p.K) {
          if (p.gathered) reinterpret_cast<uint4*>(p.gathered + (t * p.K + k0 + kk) * p.H)[c] = v[kk];
          const uint32_t* ww = reinterpret_cast<const uint32_t*>(&v[kk]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            acc[2 * q] += w[kk] * __uint_as_float((ww[q] & 0xFFFFu) << 16);
            acc[2 * q + 1] += w[kk] * __uint_as_float(ww[q] & 0xFFFF0000u);
          }
        }
      }
    }
    uint4 o;
    __nv_bfloat162 t2;
    t2 = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&t2);
    t2 = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&t2);
    t2 = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&t2);
    t2 = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&t2);
    reinterpret_cast<uint4*>(p.y + t * p.H)[c] = o;
  }
}

// dst[0 : *n_rows) = src[0 : *n_rows): the row count is only known on the device (last padded offset)
__global__ void __launch_bounds__(256) copy_rows_bounded_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                const int* __restrict__ n_rows, int row_vec) {
  const long long n = static_cast<long long>(*n_rows) * row_vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

// Routing bookkeeping of one rank for a small batch (decode steps): per expert the number of (token, k) pairs that
// chose it, and for every pair its rank among the pairs of the same expert in (token, k) order - what a stable sort
// by expert plus a histogram would give, in one launch instead of a dozen.  One CTA; thread e walks the n choices in
// shared memory for expert e (n <= LOCAL_PLAN_MAX: a few hundred pairs in a decode step), so every position is
// written by exactly one thread and the order is the input order.  Also clears the per-call outputs of the
// cross-rank plan (offsets, tot_local) so that the caller needs no memset.
constexpr int LOCAL_PLAN_MAX = 8192;
__global__ void ep_local_plan_kernel(const long long* __restrict__ idx, int n, int E, int* __restrict__ idx32,
                                     int* __restrict__ pos, int* __restrict__ cnt, int* __restrict__ offsets,
                                     int* __restrict__ tot_local, int E_local) {
  __shared__ short s_e[LOCAL_PLAN_MAX];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = static_cast<int>(idx[i]);
    s_e[i] = static_cast<short>(e);
    idx32[i] = e;
  }
  for (int i = threadIdx.x; i <= E_local; i += blockDim.x) {
    offsets[i] = 0;
    if (i < E_local) tot_local[i] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int i = 0; i < n; ++i) {
      if (s_e[i] == e) pos[i] = c++;
    }
    cnt[e] = c;
  }
}

}  // namespace gke

using namespace gke;

// idx: int64 [n] expert of every (token, k) pair.  Outputs: idx32 [n], pos [n], cnt [E] (int32), and zeroed
// offsets [E_local + 1] / tot_local [E_local].  n <= 8192, E <= 1024.
GK_EXPORT int gk_ep_local_plan(const long long* idx, int n, int E, int E_local, int* idx32, int* pos, int* cnt,
                               int* offsets, int* tot_local, void* stream) {
  if (n > LOCAL_PLAN_MAX || E > 32767 || n < 0) return -1;
  int threads = 32;
  while (threads < E && threads < 1024) threads <<= 1;
  ep_local_plan_kernel<<<1, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(idx, n, E, idx32, pos, cnt, offsets,
                                                                                  tot_local, E_local);
  return gk::launch_status();
}

GK_EXPORT int gk_ep_copy_rows(const void* src, void* dst, const int* n_rows, int H, void* stream) {
  if (H % 8) return -1;
  copy_rows_bounded_kernel<<<gk::sm_count() * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), n_rows, H / 8);
  return gk::launch_status();
}

// ptrs: [0..ep) count tables, [ep..2ep) flag arrays of every rank.
static int ep_plan_launch(const int* cnt, const unsigned long long* ptrs, int rank, int ep, int E, int seg, int R_max,
                          unsigned int calls, unsigned int* calls_dev, int* send_base, int* offsets, int* tot_local,
                          int* err, void* stream) {
  if (ep < 1 || ep > MAX_RANKS || E > MAX_EXPERTS || E % ep) return -1;
  PlanParams p;
  p.calls_dev = calls_dev;
  p.cnt = cnt;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.cnt_all[r] = r < ep ? reinterpret_cast<int*>(ptrs[r]) : nullptr;
    p.flags[r] = r < ep ? reinterpret_cast<uint32_t*>(ptrs[ep + r]) : nullptr;
  }
  p.rank = rank; p.ep = ep; p.E = E; p.E_local = E / ep; p.seg = seg; p.R_max = R_max;
  p.parity = calls & 1; p.epoch = (calls >> 1) + 1;
  p.send_base = send_base; p.offsets = offsets; p.tot_local = tot_local; p.err = err;
  ep_plan_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return gk::launch_status();
}

GK_EXPORT int gk_ep_plan(const int* cnt, const unsigned long long* ptrs, int rank, int ep, int E, int seg, int R_max,
                         unsigned int calls, int* send_base, int* offsets, int* tot_local, int* err, void* stream) {
  return ep_plan_launch(cnt, ptrs, rank, ep, E, seg, R_max, calls, nullptr, send_base, offsets, tot_local, err, stream);
}

// The call number (which selects the table parity and the flag epoch) is read from `calls_dev` and advanced by the
// kernel: the launch can be captured in a CUDA graph.
GK_EXPORT int gk_ep_plan_dev(const int* cnt, const unsigned long long* ptrs, int rank, int ep, int E, int seg, int R_max,
                             unsigned int* calls_dev, int* send_base, int* offsets, int* tot_local, int* err,
                             void* stream) {
  if (!calls_dev) return -1;
  return ep_plan_launch(cnt, ptrs, rank, ep, E, seg, R_max, 0u, calls_dev, send_base, offsets, tot_local, err, stream);
}

// recv_ptrs: receive buffer [R_max, H] of every rank.
GK_EXPORT int gk_ep_push(const void* x, const float* scale, const int* idx, const int* pos, const int* send_base,
                         const int* offsets, const int* tot_local, const unsigned long long* recv_ptrs, int* dst_row,
                         int rank, int ep, int E_local, int seg, int R_max, int K, int H, long long T, void* stream) {
  if (ep < 1 || ep > MAX_RANKS || H % 8) return -1;
  PushParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.scale = scale; p.idx = idx; p.pos = pos; p.send_base = send_base; p.offsets = offsets; p.tot_local = tot_local;
  for (int r = 0; r < MAX_RANKS; ++r) p.recv[r] = r < ep ? reinterpret_cast<__nv_bfloat16*>(recv_ptrs[r]) : nullptr;
  p.dst_row = dst_row; p.rank = rank; p.ep = ep; p.E_local = E_local; p.seg = seg; p.R_max = R_max; p.K = K; p.H = H;
  p.npairs = T * K;
  const long long warps = p.npairs + static_cast<long long>(E_local) * seg;
  const long long blocks = (warps + 7) / 8;
  ep_push_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return gk::launch_status();
}

// src_ptrs: expert-output buffer [R_max, H] of every rank.
GK_EXPORT int gk_ep_pull(const unsigned long long* src_ptrs, const int* dst_row, const float* weight, void* y,
                         void* gathered, int ep, int K, int H, int R_max, long long T, void* stream) {
  if (ep < 1 || ep > MAX_RANKS || H % 8) return -1;
  if (T == 0) return 0;
  PullParams p;
  for (int r = 0; r < MAX_RANKS; ++r) p.src[r] = r < ep ? reinterpret_cast<const __nv_bfloat16*>(src_ptrs[r]) : nullptr;
  p.dst_row = dst_row; p.weight = weight; p.y = reinterpret_cast<__nv_bfloat16*>(y);
  p.gathered = reinterpret_cast<__nv_bfloat16*>(gathered); p.K = K; p.H = H; p.R_max = R_max; p.T = T;
  const long long blocks = (T + 7) / 8;
  ep_pull_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return gk::launch_status();
}
