// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference framework. It exists for users of this
// library whose code runs where a device allocation is not possible or not allowed: inside a
// memory pool that is already fully handed out, in a real-time or driver-owned thread that may not
// call the CUDA allocator (cudaMalloc takes a device-wide lock and can synchronise the device), or
// from a plain C host program that links the shared object without PyTorch's caching allocator.
//
// The regular backward (lf::rmsnorm_bwd, reached through the torch binding) needs a fp32 scratch
// matrix of per-CTA partial weight gradients which the binding allocates per call. Here that scratch
// lives in a file-scope `static __device__` array inside the library image, so every GPU that loads
// the library holds LF_RMSNORM_NOALLOC_SCRATCH_BYTES (about 4.6 MiB) until the process exits.
//
// Contract
//   * dy, x, dx: bf16 [T, H] contiguous; w: bf16 [H]; rstd: fp32 [T] (from the forward); dw: fp32 [H],
//     overwritten. All pointers are device pointers on the CURRENT device, 16-byte aligned.
//   * H must be a multiple of 8 and at most LF_RMSNORM_NOALLOC_MAX_H; 0 <= T <= LF_RMSNORM_NOALLOC_MAX_T
//     (the kernels index rows with a 32-bit int). Larger sizes are rejected with
//     LF_NOALLOC_ERR_TOO_LARGE and nothing is launched.
//   * If the device already carries an error from earlier work, LF_NOALLOC_ERR_CUDA is returned and nothing
//     is launched (the pending error is left in place for its owner to read).
//   * The first call on each device looks up the device address of the scratch array (a host-side
//     symbol is not a device address). That first call should therefore be made before any stream
//     capture is started on that device.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any call.
//   * All calls on one device share the one scratch array. It keeps the previous call's contents;
//     nothing in it has to start at zero because every element that is read is written first by the
//     same call. Two calls whose kernels overlap on the GPU (different streams) race on it: callers
//     must serialise them.
#pragma once
#include <cuda_runtime.h>

#define LF_RMSNORM_NOALLOC_MAX_H 8192
#define LF_RMSNORM_NOALLOC_MAX_CTAS 148
#define LF_RMSNORM_NOALLOC_MAX_T 2147483647LL
#define LF_RMSNORM_NOALLOC_SCRATCH_BYTES (LF_RMSNORM_NOALLOC_MAX_CTAS * LF_RMSNORM_NOALLOC_MAX_H * 4)

#define LF_NOALLOC_OK 0
#define LF_NOALLOC_ERR_TOO_LARGE 1   // H or T above the maximum, or H not a multiple of 8
#define LF_NOALLOC_ERR_BAD_POINTER 2 // null or misaligned pointer
#define LF_NOALLOC_ERR_CUDA 3        // a CUDA runtime call failed (symbol lookup or launch)

#ifdef __cplusplus
extern "C" {
#endif

// Returns LF_NOALLOC_OK or one of the error codes above. `stream` may be 0 (default stream).
int lf_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                           long long T, int H, float w_offset, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
