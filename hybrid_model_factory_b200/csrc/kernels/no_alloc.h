// Entry point for callers that are not allowed to allocate device memory.
//
// This declaration has no counterpart in the reference project: it exists for hosts of this
// library that run inside somebody else's memory plan -- an inference server with a frozen
// arena, a plugin called from a framework whose allocator must not be re-entered, code that
// runs while a CUDA graph is being captured elsewhere in the process -- where a cudaMalloc
// (or a PyTorch tensor allocation) at call time is either forbidden or would serialise the
// device.  Such callers own their inputs and outputs but have nowhere to put a kernel's
// temporary workspace.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Upper limits of hmf_rms_norm_bwd_noalloc (the built-in workspace is MAX_SLABS x MAX_D floats = 8 MiB
// per GPU that loads the library, held until the process exits).
#define HMF_NOALLOC_RMSNORM_MAX_D 8192
#define HMF_NOALLOC_RMSNORM_MAX_SLABS 256

// RMSNorm backward: dx [N, D] (bf16) and dw [D] (bf16 when dw_is_bf16, else fp32) from x, w, dy (bf16)
// and the saved rstd [N] (fp32).  Same mathematics and outputs as hmf_rms_norm_bwd, but the partial
// weight-gradient sums live in a workspace compiled into the library instead of a caller buffer:
// the function calls no cudaMalloc / cudaFree and no allocating library routine.
//
//  * D must be a multiple of 8 and at most HMF_NOALLOC_RMSNORM_MAX_D; anything larger is rejected
//    with HMF_ERR_TOO_LARGE (-4) and a message in hmf_last_error().
//  * The first call on each device looks up the workspace address (cudaGetSymbolAddress) with that
//    device current; make that first call before any stream capture starts.
//  * All calls on one GPU share the one workspace.  It keeps whatever the previous call left; this
//    kernel overwrites every word it later reads, so nothing needs clearing, but two calls that
//    overlap on the GPU (different streams, no dependency) race on it.  Serialise them.
int hmf_rms_norm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                             void* dw_out, int dw_is_bf16, long long N, int D, int zero_centered,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
