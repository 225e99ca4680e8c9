// Entry points that allocate nothing.
//
// This header has no counterpart in the reference (Tencent/G-Core-GH ships no native code at all); it exists for
// callers of this library that are not allowed to allocate device memory while they run: code executing while a
// CUDA memory pool is frozen, host threads inside a latency-critical serving loop where a cudaMalloc would
// synchronise the device, or embedders that hand this library a fixed memory budget up front.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size and largest number of row groups the built-in scratch array can serve.
#define GK_NOALLOC_RMSNORM_MAX_H 8192
#define GK_NOALLOC_RMSNORM_MAX_PARTS 296

// RMSNorm backward (same math as gk_rmsnorm_bwd) whose per-CTA partial sums of the weight gradient live in a
// file-scope device array of GK_NOALLOC_RMSNORM_MAX_PARTS * GK_NOALLOC_RMSNORM_MAX_H floats (about 9.3 MiB) instead
// of a caller-provided scratch buffer.  Every GPU that loads the library holds that array until the process exits.
//
//   g, x   [T, H] bf16   upstream gradient and the tensor that was normalised
//   w      [H]    bf16   gain;  rstd [T] fp32 from the forward pass;  dres [T, H] bf16 or NULL (added to dx)
//   dx     [T, H] bf16   output;  dw [H] fp32 output (overwritten, or accumulated into when dw_accumulate != 0)
//
// Returns 0 on success, -1 when H is not a multiple of 8, -2 when H exceeds GK_NOALLOC_RMSNORM_MAX_H (an error line
// is printed to stderr), -3 when the device address of the scratch array cannot be obtained, or a positive
// cudaError_t from the launch.  It calls no cudaMalloc / cudaFree and no allocating library routine.
//
// The first call on each device looks the array's device address up (cudaGetSymbolAddress, with that device
// current); make that first call before any stream capture begins.  All calls on a device share the one array: it
// keeps whatever the previous call left (nothing has to start at zero - every slot that is read is written first by
// the same call), and two calls whose kernels overlap on the GPU (different streams) race on it.
int gk_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                           float* dw, int dw_accumulate, int T, int H, void* stream);

#ifdef __cplusplus
}
#endif
