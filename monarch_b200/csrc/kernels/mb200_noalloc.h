// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference; it exists for embedders of this kernel
// library.  Some of them cannot call cudaMalloc where the kernel is needed: code running
// inside a CUDA-graph capture or a real-time loop where allocation is forbidden, a plugin
// hosted by a runtime that owns all device memory and hands out none, or a process that
// has handed its whole memory budget to another allocator.  The regular RMSNorm backward
// (mb200_rmsnorm_bwd) asks its caller for an fp32 scratch buffer of [blocks, d] partial
// weight-gradient sums; this variant keeps that scratch inside the library instead.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest feature dimension accepted, and the size of the built-in scratch.  The scratch
// is a file-scope device array of MB200_NOALLOC_SCRATCH_FLOATS floats (16 MiB); every GPU
// that loads the library holds it until the process exits.
#define MB200_NOALLOC_MAX_D 8192
#define MB200_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// Error codes specific to this entry point (0 = launched; other small values are
// cudaError_t of the failing runtime call).
#define MB200_NOALLOC_ERR_BAD_D 1101       // d is not a multiple of 8 or exceeds MAX_D
#define MB200_NOALLOC_ERR_BAD_ROWS 1102    // rows < 0
#define MB200_NOALLOC_ERR_SYMBOL 1103      // the scratch address could not be resolved

// RMSNorm backward, same arithmetic and arguments as mb200_rmsnorm_bwd minus the scratch
// pointer: dx = d(loss)/dx (+ dres when given); dw ([d], bf16) receives the weight
// gradient, or has it added when dw_accumulate != 0.
//
// * Allocates nothing: no cudaMalloc/cudaFree, no allocating library call.  Inputs and
//   outputs are the caller's.
// * The first call on each device resolves the device address of the built-in scratch
//   (cudaGetSymbolAddress) with that device current and remembers it; make that first
//   call before starting any stream capture.
// * All calls on a device share the one scratch array.  Its contents carry over from the
//   previous call; the kernel overwrites every element it later reads, so nothing needs
//   clearing.  Two calls whose kernels overlap on the GPU (different streams without an
//   ordering between them) race on it: order such calls yourself.
// * d > MB200_NOALLOC_MAX_D (or d % 8 != 0) is refused with MB200_NOALLOC_ERR_BAD_D and a
//   message on stderr; nothing is launched.
int mb200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                              const void* dres, void* dx, void* dw, int dw_accumulate, int rows,
                              int d, void* stream);

#ifdef __cplusplus
}
#endif
