// Host-side helpers shared by the kernel translation units: TMA descriptor encoding through the driver entry
// point (no link-time dependency on libcuda), launch checking, and per-device attribute caching.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define GK_EXPORT extern "C" __attribute__((visibility("default")))

namespace gk {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Makes the device's primary context current on the calling thread (the driver entry points need one).
inline void bind_primary_context() { cudaFree(nullptr); }

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements with leading dimension `ld` (elements).
// Box = [box_rows, box_cols]; 128-byte swizzle (box_cols * elem_bytes must be <= 128 when swizzled).
inline int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT) break;
    bind_primary_context();  // a thread that has made no runtime call yet (e.g. an autograd worker)
  }
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[gcore_b200] cuTensorMapEncodeTiled(2d) failed: CUresult=%d base=%p elem=%d rows=%llu cols=%llu ld=%llu "
            "box=[%u,%u]\n",
            static_cast<int>(r), base, elem_bytes, (unsigned long long)rows, (unsigned long long)cols,
            (unsigned long long)ld, box_rows, box_cols);
  }
  return r == CUDA_SUCCESS ? 0 : -2;
}

inline int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d2, uint64_t d1, uint64_t d0,
                        uint64_t stride2_elems, uint64_t stride1_elems, uint32_t box2, uint32_t box1,
                        uint32_t box0, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * static_cast<uint64_t>(elem_bytes),
                           stride2_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT) break;
    bind_primary_context();
  }
  return r == CUDA_SUCCESS ? 0 : -2;
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Shared-memory budget of one CTA of a decode-shaped (swap-AB) GEMM launch, in bytes; 0 = as much as the kernel can
// use (the default).  With a budget of about half an SM the CTA of the next GEMM of a decode chain can become resident
// beside the running one and stream its first weight tiles while the running kernel finishes; measured on B200 the
// shallower ring costs each GEMM more (3-7 %) than that overlap returns, so the budget is an experiment switch.
inline int& decode_smem_cap() {
  static int cap = 0;
  return cap;
}

// ---- output-tile order of the persistent dense GEMMs.  Tiles are handed out in bands of `raster_group_m()` tile rows:
// inside a band the row index runs fastest, so the CTAs that run at the same time cover a patch of about group_m
// tile rows x (CTAs / group_m) tile columns.  Every operand tile is then wanted by a handful of CTAs at a time (and
// is re-read from L2 while it is still hot) instead of one B tile by every CTA of the wave at once, which
// concentrates the requests on the few L2 slices that hold it.  0 or 1 = plain row-fastest order.
inline int& raster_group_m() {
  static int g = 16;
  return g;
}
inline int& wide_tail_split() {
  static int on = 1;
  return on;
}
inline int& wide_staged_epilogue() {
  static int on = 1;
  return on;
}
#ifdef __CUDACC__
__device__ __forceinline__ void raster_tile(int tile, int mt, int nt, int group_m, int& mi, int& ni) {
  if (group_m <= 1) {
    mi = tile % mt;
    ni = tile / mt;
    return;
  }
  const int per_band = group_m * nt;
  const int band = tile / per_band;
  const int first = band * group_m;
  const int rows = mt - first < group_m ? mt - first : group_m;
  const int r = tile - band * per_band;
  mi = first + r % rows;
  ni = r / rows;
}
#endif

// ---- programmatic dependent launch: a kernel launched through launch_k may start its prologue while the previous
// kernel of the stream is still draining; it must call pdl_wait() before it touches global memory, and it calls
// pdl_launch_dependents() first so that its own successor may be scheduled early.  Both instructions are no-ops in a
// kernel that was launched the ordinary way.  Off unless gk_set_pdl(1) (the rollout engine switches it on around the
// decode chain, where ~300 short kernels per step make the launch gaps a measurable share of the step).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
inline int& pdl_flag() {
  static int flag = 0;
  return flag;
}
template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  if (!pdl_flag()) {
    kernel<<<grid, block, smem, st>>>(args...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[gcore_b200] kernel launch failed: %s\n", cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return 0;
}

}  // namespace gk
