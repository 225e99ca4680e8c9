// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (one kernel does both):
//
//   mode AG : all-gather -> GEMM.  C[tp*Tl, N] = gather(x)[tp*Tl, K] * B^T.  Every rank owns Tl rows of x inside a
//             symmetric buffer that has room for all tp*Tl rows.  A few "communication CTAs" push this rank's rows
//             into every peer's buffer, 128-row chunk by chunk, and publish a per-chunk flag in the peer's memory;
//             the compute CTAs start on the local rows and only wait (bounded) for a remote chunk's flag right
//             before the TMA loads that read it, so the transfer hides behind the math tile by tile.
//   mode RS : GEMM -> reduce-scatter.  y_local[Tl, N] = sum_r (a_r * B_r^T)[rows of this rank].  Tiles whose rows
//             belong to a peer are computed first and their bf16 partials are stored straight into that peer's inbox
//             (posted NVLink writes) followed by a per-tile flag; tiles owned by this rank are computed last and
//             their epilogue adds the peers' partials as soon as each flag is seen.
//
// Replaces the separate NCCL all-gather / reduce-scatter around Megatron's Column / RowParallelLinear with sequence
// parallelism (the call sites the reference configures at gpatch_v4/training_backend/megatron_backend/mixin.py:
// 404-410).  Remote data moves with plain peer stores and TMA loads WITHOUT cluster multicast.  Flags carry a call
// epoch (never reset); buffers are double-buffered by call parity, which is enough because a rank cannot finish call
// n+1 before every peer has started it.  All waits are bounded and report through the error word.
#include "ptx.cuh"
#include "host_utils.h"

namespace gkc {
using namespace gk;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int MAX_RANKS = 8;

struct CommParams {
  int M, N, K;           // M = tp * rows_per_rank for both modes (global rows)
  int mode;              // 1 = AG, 2 = RS
  int rank, nranks;
  int rows_per_rank;     // multiple of 128
  int ncomm;             // communication CTAs (mode AG)
  uint32_t epoch;
  // output
  __nv_bfloat16* C;      // AG: [M, N];  RS: y_local [rows_per_rank, N]
  long long ldc;
  const void* bias;      // AG only, bf16 [N]
  // AG: this rank's rows inside its own gathered buffer, the peers' gathered buffers and flag arrays
  const __nv_bfloat16* ag_local;        // base of the local gathered buffer [M, K]
  __nv_bfloat16* ag_peer[MAX_RANKS];    // base of every rank's gathered buffer (peer pointers)
  uint32_t* ag_peer_flags[MAX_RANKS];   // flags[src_rank * chunks + chunk] in every rank's memory
  const uint32_t* ag_my_flags;
  long long ag_ld;
  // RS: inboxes [src_rank][rows_per_rank, N] in every rank's memory, flags[src_rank * tiles + tile]
  __nv_bfloat16* rs_peer_inbox[MAX_RANKS];
  const __nv_bfloat16* rs_my_inbox;
  uint32_t* rs_peer_flags[MAX_RANKS];
  const uint32_t* rs_my_flags;
  long long rs_ld;
  int* err;
};

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (192 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int EPI_BYTES = 128 * 256;  // epilogue staging: 128 rows x 128 bf16 columns
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *flag >= epoch (epochs only grow; wrap-around after 2^31 calls is not handled).
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, int* err) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 63) == 0) {
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) {
        atomicCAS(err, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
  return true;
}

struct Tile {
  int m0, n0;
  int owner;      // rank owning the rows
  int chunk;      // 128-row chunk index inside the owner's rows
  int tile_id;    // RS: (chunk * n_tiles + n_tile) inside the owner's rows
};

// Tile order.  AG: row chunks rotated so that the local rows come first, then peers in ring order.
// RS: peers' rows first (ring order starting at rank+1), own rows last.
__device__ __forceinline__ Tile decode(const CommParams& p, int BN, int tile) {
  const int nt = (p.N + BN - 1) / BN;
  const int chunks = p.rows_per_rank / BM;
  const int per_rank = chunks * nt;
  const int slot = tile / per_rank;  // which rank's rows, in visiting order
  const int r = tile - slot * per_rank;
  Tile t;
  t.owner = p.mode == 1 ? (p.rank + slot) % p.nranks : (p.rank + 1 + slot) % p.nranks;
  // groups of up to 8 row chunks; inside a group the N tiles sweep slowest, so a wave of CTAs shares few B tiles
  // (the weight streams from HBM once per group) while the group's A rows stay hot in L2
  constexpr int GROUP = 8;
  const int g = r / (GROUP * nt);
  const int in_g = r - g * GROUP * nt;
  const int g_chunks = chunks - g * GROUP < GROUP ? chunks - g * GROUP : GROUP;
  const int n_idx = in_g / g_chunks;
  t.chunk = g * GROUP + (in_g - n_idx * g_chunks);
  t.m0 = t.owner * p.rows_per_rank + t.chunk * BM;
  t.n0 = n_idx * BN;
  t.tile_id = t.chunk * nt + n_idx;
  return t;
}

template <int BN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, CommParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage = smem + STAGES * C::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(stage + C::EPI_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* epi_bar = tempty + 2;  // 128 arrivals: "all rows of the tile are stored"
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(epi_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = p.rows_per_rank / BM;

  if (p.mode == 1 && static_cast<int>(blockIdx.x) < p.ncomm) {
    // ------------------------------------------------------------------ communication CTA (AG): push my rows
    const long long row_bytes = p.K * 2LL;
    const int vec_per_row = static_cast<int>(row_bytes / 16);
    for (int c = blockIdx.x; c < chunks; c += p.ncomm) {
      const long long row0 = static_cast<long long>(p.rank) * p.rows_per_rank + static_cast<long long>(c) * BM;
      const uint4* src = reinterpret_cast<const uint4*>(p.ag_local + row0 * p.ag_ld);
      for (int pr = 1; pr < p.nranks; ++pr) {
        const int peer = (p.rank + pr) % p.nranks;
        uint4* dst = reinterpret_cast<uint4*>(p.ag_peer[peer] + row0 * p.ag_ld);
        if (p.ag_ld == p.K) {
          const int total = BM * vec_per_row;
          for (int i = threadIdx.x; i < total; i += THREADS * 4) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) if (i + u * THREADS < total) v[u] = src[i + u * THREADS];
#pragma unroll
            for (int u = 0; u < 4; ++u) if (i + u * THREADS < total) dst[i + u * THREADS] = v[u];
          }
        } else {
          for (int r = 0; r < BM; ++r) {
            const uint4* s = reinterpret_cast<const uint4*>(p.ag_local + (row0 + r) * p.ag_ld);
            uint4* d = reinterpret_cast<uint4*>(p.ag_peer[peer] + (row0 + r) * p.ag_ld);
            for (int i = threadIdx.x; i < vec_per_row; i += THREADS) d[i] = s[i];
          }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
          __threadfence_system();
          st_release_sys(p.ag_peer_flags[peer] + p.rank * chunks + c, p.epoch);
        }
      }
    }
    return;
  }

  const int ncomm = p.mode == 1 ? p.ncomm : 0;
  const int cta = blockIdx.x - ncomm;
  const int ncta = gridDim.x - ncomm;
  const int nt = (p.N + BN - 1) / BN;
  const int ntiles = p.nranks * chunks * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 128);
    }
    mbar_init(epi_bar, 128);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 2) {
    tmem_alloc(tmem_holder, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const int kblocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    int ready_owner = -1, ready_chunk = -1;
    for (int tile = cta; tile < ntiles && ok; tile += ncta) {
      const Tile t = decode(p, BN, tile);
      if (p.mode == 1 && t.owner != p.rank && (t.owner != ready_owner || t.chunk != ready_chunk)) {
        // the rows of this tile come from a peer: wait until its chunk has landed in the local gathered buffer
        ok = wait_flag(p.ag_my_flags + t.owner * chunks + t.chunk, p.epoch, p.err);
        if (!ok) break;
        fence_proxy_async();  // peer stores (generic proxy) must be visible to the TMA reads that follow
        asm volatile("fence.proxy.async.global;" ::: "memory");
        ready_owner = t.owner;
        ready_chunk = t.chunk;
      }
      for (int kb = 0; kb < kblocks; ++kb) {
        ok = mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          uint8_t* sa = smem + s * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          const int k = kb * BK;
          mbar_expect_tx(&full[s], C::STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full[s], k, t.m0);
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, &full[s], t.n0 + i * 64, k);
          } else {
            tma_load_2d(sb, &tmB, &full[s], k, t.n0);
          }
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, 0, B_MN ? 1 : 0);
    int s = 0, acc = 0;
    uint32_t ph = 0, pacc = 0;
    bool ok = true;
    for (int tile = cta; tile < ntiles && ok; tile += ncta) {
      ok = mbar_wait(&tempty[acc], pacc ^ 1, p.err, ERR_WAIT_TMEM_EMPTY);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < kblocks; ++kb) {
        ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_base = a_base + C::A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
            const uint64_t adesc = make_smem_desc_sw128(a_base + k4 * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k4 * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(b_base + k4 * (UMMA_K * 2), 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
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
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t pacc = 0, epi_ph = 0;
    bool ok = true;
    const int rs_tiles = chunks * nt;
    for (int tile = cta; tile < ntiles && ok; tile += ncta) {
      const Tile t = decode(p, BN, tile);
      ok = mbar_wait(&tfull[acc], pacc, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const int row = t.m0 + row_in_tile;  // global row
      const int lrow = t.chunk * BM + row_in_tile;  // row inside the owner's block
      const bool mine = t.owner == p.rank;
      if (p.mode == 2 && mine) {
        // the peers' partials for this tile must have landed in my inbox
        for (int pr = 1; pr < p.nranks && ok; ++pr) {
          const int src = (p.rank + pr) % p.nranks;
          ok = wait_flag(p.rs_my_flags + src * rs_tiles + t.tile_id, p.epoch, p.err);
        }
        if (!ok) break;
      }
      // Destination of this tile's rows (row 0 of the tile, column n0) and its leading dimension.
      __nv_bfloat16* dst_base;
      long long dst_ld;
      if (p.mode == 1) {
        dst_base = p.C + static_cast<long long>(t.m0) * p.ldc + t.n0;
        dst_ld = p.ldc;
      } else if (mine) {
        dst_base = p.C + static_cast<long long>(t.chunk * BM) * p.ldc + t.n0;
        dst_ld = p.ldc;
      } else {
        dst_base = p.rs_peer_inbox[t.owner] +
                   (static_cast<long long>(p.rank) * p.rows_per_rank + t.chunk * BM) * p.rs_ld + t.n0;
        dst_ld = p.rs_ld;
      }
      (void)row;
      // The tile leaves through a shared-memory staging area, 128 columns at a time, so that every warp-wide store
      // covers whole 256-byte row segments (NVLink and HBM both dislike 64-byte fragments).
#pragma unroll 1
      for (int half = 0; half < BN / 128; ++half) {
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          const int c = half * 4 + c4;
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          const int col0 = t.n0 + c * 32;
          const int ncols = p.N - col0 < 32 ? p.N - col0 : 32;
          if (p.mode == 1 && p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ncols) v[j] += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + j]);
          }
          if (p.mode == 2 && mine && ncols > 0) {
            for (int pr = 1; pr < p.nranks; ++pr) {
              const int src = (p.rank + pr) % p.nranks;
              const __nv_bfloat16* in =
                  p.rs_my_inbox + (static_cast<long long>(src) * p.rows_per_rank + lrow) * p.rs_ld + col0;
              if (ncols == 32) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 w = __ldcg(reinterpret_cast<const uint4*>(in) + j);
                  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    v[8 * j + 2 * q] += bf16_bits_to_float(static_cast<uint16_t>(ww[q] & 0xFFFF));
                    v[8 * j + 2 * q + 1] += bf16_bits_to_float(static_cast<uint16_t>(ww[q] >> 16));
                  }
                }
              } else {
                for (int j = 0; j < ncols; ++j) v[j] += __bfloat162float(in[j]);
              }
            }
          }
          // 4 x 16-byte units of this row; unit u of row r is stored at unit u ^ (r & 15) (bank-conflict free)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
            o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
            o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
            const int unit = c4 * 4 + j;
            *reinterpret_cast<uint4*>(stage + row_in_tile * 256 + ((unit ^ (row_in_tile & 15)) << 4)) = o;
          }
        }
        // each warp stages and drains only the 32 rows of its own TMEM quadrant: a warp-level sync is enough
        __syncwarp();
        {
          const int unit = lane & 15;
          const int colu = t.n0 + half * 128 + unit * 8;  // first column of this 16-byte unit
          const bool vec_ok = (dst_ld & 7) == 0 && (t.n0 & 7) == 0 && (reinterpret_cast<uintptr_t>(dst_base) & 15) == 0;
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int rr = quad * 32 + 2 * i + (lane >> 4);
            const uint4 w = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((unit ^ (rr & 15)) << 4));
            __nv_bfloat16* drow = dst_base + static_cast<long long>(rr) * dst_ld + half * 128 + unit * 8;
            if (vec_ok && colu + 8 <= p.N) {
              *reinterpret_cast<uint4*>(drow) = w;
            } else {
              const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&w);
              for (int j = 0; j < 8; ++j)
                if (colu + j < p.N) drow[j] = e[j];
            }
          }
        }
        __syncwarp();  // the staging rows are free again
      }
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) pacc ^= 1;
      if (p.mode == 2 && !mine) {
        // publish the tile to its owner once all 128 rows are stored (bounded wait: no thread can block for ever)
        mbar_arrive(epi_bar);
        if (threadIdx.x == 64) {
          ok = mbar_wait(epi_bar, epi_ph, p.err, ERR_WAIT_MISC);
          if (ok) {
            __threadfence_system();
            st_release_sys(p.rs_peer_flags[t.owner] + p.rank * rs_tiles + t.tile_id, p.epoch);
          }
        }
        epi_ph ^= 1;
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

template <int BN, bool B_MN>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CommParams& p, int grid, cudaStream_t st) {
  using C = Cfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_comm_kernel<BN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  gemm_comm_kernel<BN, B_MN><<<grid, THREADS, C::SMEM_BYTES, st>>>(tmA, tmB, p);
  return launch_status();
}

}  // namespace gkc

using namespace gkc;

// ptrs layout (device pointers as 64-bit integers, host array):
//   AG: [0..n)  gathered buffer of every rank,  [n..2n) flag array of every rank
//   RS: [0..n)  inbox of every rank,            [n..2n) flag array of every rank
// A: AG -> the local gathered buffer [tp*Tl, K];  RS -> this rank's activations [tp*Tl, K_local].
// B: [N, K] (b_mn = 0) or [K, N] (b_mn = 1).  C: AG -> [tp*Tl, N];  RS -> [Tl, N].
GK_EXPORT int gk_gemm_comm(int mode, const void* A, long long lda, const void* B, long long ldb, long long b_rows,
                           int b_mn, void* C, long long ldc, const void* bias, int M, int N, int K, int rank,
                           int nranks, int rows_per_rank, int ncomm, unsigned epoch, const unsigned long long* ptrs,
                           long long comm_ld, int* err, void* stream) {
  if (mode != 1 && mode != 2) return -1;
  if (nranks < 1 || nranks > MAX_RANKS || rank < 0 || rank >= nranks) return -2;
  if (rows_per_rank % BM || M != rows_per_rank * nranks) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return -4;
  const int bn = N >= 192 ? 256 : 128;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, 2, M, K, lda, BM, 64, true)) return -5;
  if (b_mn) {
    if (make_tmap_2d(&tmB, B, 2, b_rows, N, ldb, 64, 64, true)) return -6;
  } else {
    if (make_tmap_2d(&tmB, B, 2, b_rows, K, ldb, bn, 64, true)) return -6;
  }
  CommParams p;
  p.M = M; p.N = N; p.K = K; p.mode = mode; p.rank = rank; p.nranks = nranks; p.rows_per_rank = rows_per_rank;
  p.epoch = epoch;
  p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc; p.bias = bias;
  p.err = err;
  const int chunks = rows_per_rank / BM;
  if (mode == 1) {
    if (ncomm < 1) ncomm = 1;
    if (ncomm > chunks) ncomm = chunks;
    if (nranks == 1) ncomm = 0;
    p.ncomm = ncomm;
    p.ag_local = reinterpret_cast<const __nv_bfloat16*>(A);
    p.ag_ld = comm_ld;
    for (int r = 0; r < nranks; ++r) {
      p.ag_peer[r] = reinterpret_cast<__nv_bfloat16*>(ptrs[r]);
      p.ag_peer_flags[r] = reinterpret_cast<uint32_t*>(ptrs[nranks + r]);
    }
    p.ag_my_flags = p.ag_peer_flags[rank];
  } else {
    p.ncomm = 0;
    p.rs_ld = comm_ld;
    for (int r = 0; r < nranks; ++r) {
      p.rs_peer_inbox[r] = reinterpret_cast<__nv_bfloat16*>(ptrs[r]);
      p.rs_peer_flags[r] = reinterpret_cast<uint32_t*>(ptrs[nranks + r]);
    }
    p.rs_my_inbox = p.rs_peer_inbox[rank];
    p.rs_my_flags = p.rs_peer_flags[rank];
  }
  const long long tiles = static_cast<long long>(nranks) * chunks * ((N + bn - 1) / bn);
  const int sms = sm_count();
  int compute = static_cast<int>(tiles < sms - p.ncomm ? tiles : sms - p.ncomm);
  if (compute < 1) compute = 1;
  const int grid = compute + p.ncomm;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 256) return b_mn ? launch<256, true>(tmA, tmB, p, grid, st) : launch<256, false>(tmA, tmB, p, grid, st);
  return b_mn ? launch<128, true>(tmA, tmB, p, grid, st) : launch<128, false>(tmA, tmB, p, grid, st);
}
