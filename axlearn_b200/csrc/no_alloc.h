// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (apple/axlearn); it exists for hosts of
// this library that cannot call cudaMalloc at the point where they need the op: code running
// inside a memory pool whose budget is fixed up front, latency-critical serving loops in which
// an allocation (and the implicit synchronisation it can cause) is forbidden, and embedders
// that own every byte of device memory themselves.  The regular entry point,
// axb_rmsnorm_bwd(), needs a caller-provided fp32 workspace of [ctas, D] partial sums; the
// variant below keeps that workspace inside the library instead.
//
// Contract
//   * Inputs and outputs are the caller's, exactly as for axb_rmsnorm_bwd():
//       x, dy, dx      [rows, D] bf16        scale  [D] bf16        rstd  [rows] fp32
//       dres           optional [rows, D] bf16 added to dx (may be null)
//       dscale_bf16 / dscale_f32   [D], either may be null
//   * D must be a multiple of 8 and at most AXB_NOALLOC_RMSNORM_MAX_D; larger D is rejected
//     with return code -20 and a message on stderr (nothing is launched).
//   * The workspace is one file-scope device array of AXB_NOALLOC_RMSNORM_MAX_CTAS x
//     AXB_NOALLOC_RMSNORM_MAX_D floats (about 9.3 MiB) that every GPU which loads the library
//     holds until the process exits.
//   * The first call on a device looks up the array's device address (once per device, with
//     that device current).  Make this first call before starting any stream capture.
//   * On EVERY call the device that `stream` belongs to must be the current device: the
//     workspace is chosen from the current device, not from the stream.
//   * rows == 0 is allowed: dx is untouched and the scale gradients that were passed are set
//     to zero.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
//   * All calls share the one workspace and it keeps the previous call's contents.  Every
//     element that a call reads is written by that same call first, so nothing has to be
//     cleared; but two calls that overlap on the GPU (different streams, or one device used
//     from two threads) race on it.  Serialise them.
//
// Returns 0 on success, -10 for a bad D, -20 for D above the maximum, -21 if the workspace
// address cannot be resolved, -4 if the launch failed.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define AXB_NOALLOC_RMSNORM_MAX_D 8192
#define AXB_NOALLOC_RMSNORM_MAX_CTAS 296

#ifdef __cplusplus
extern "C" {
#endif

int axb_rmsnorm_bwd_noalloc(const void* x, const void* scale, const float* rstd, const void* dy,
                            const void* dres, void* dx, void* dscale_bf16, float* dscale_f32,
                            int64_t rows, int D, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
