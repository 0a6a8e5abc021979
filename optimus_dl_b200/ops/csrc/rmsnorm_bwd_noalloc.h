// RMSNorm backward without any allocation.
//
// This entry point has no counterpart in the reference framework. It exists for hosts that
// embed this library where device allocation is off the table while they run: a serving or
// training loop that has handed all device memory to its own pool, code running inside a
// CUDA-graph-managed region of an application, or a plugin that is only given input and output
// buffers. ob_rmsnorm_bwd needs a caller-provided scratch buffer for the per-CTA partial sums of
// the weight gradient; here that scratch is a fixed array compiled into the library
// (OB_RMSNORM_NOALLOC_MAX_FLOATS floats = 4 MiB, resident on every GPU that loads the library
// until the process exits). The function calls no cudaMalloc / cudaFree and no allocating
// library routine.
//
//   dx = rmsnorm_backward(dy, x, w, rstd)          (bf16, [rows, D])
//   dw = sum over rows of dy * x * rstd            (bf16, [D])
//
// Limits: D % 8 == 0, D <= 8192, and min(rows, OB_RMSNORM_NOALLOC_MAX_CTAS) * D must fit the
// array, which holds for every D the kernel supports. Larger requests are refused with
// OB_RMSNORM_NOALLOC_ERR_TOO_LARGE (and a message on stderr); nothing is launched.
//
// First call on a device: looks up the device address of the built-in array (once per device,
// with that device current). Make that first call outside of any stream capture.
//
// Sharing: all calls on one GPU use the same array and it keeps the previous call's contents.
// Each launch overwrites every slot it later reads, so no clearing is needed, but two calls
// whose kernels overlap on the GPU (different streams, no ordering between them) race on it.
// Calls on one stream, or ordered by events, are safe.
//
// Returns 0 on success, one of the negative codes below, or a positive cudaError_t value.
#pragma once
#include <cuda_runtime.h>

#define OB_RMSNORM_NOALLOC_MAX_CTAS 128
#define OB_RMSNORM_NOALLOC_MAX_FLOATS (128 * 8192)
#define OB_RMSNORM_NOALLOC_ERR_SHAPE (-1)
#define OB_RMSNORM_NOALLOC_ERR_TOO_LARGE (-2)
#define OB_RMSNORM_NOALLOC_ERR_DEVICE (-3)

#ifdef __cplusplus
extern "C" {
#endif

int ob_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const void* rstd, void* dx, void* dw_bf16,
                           int rows, int D, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
