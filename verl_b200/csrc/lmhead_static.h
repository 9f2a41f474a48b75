// Fused lm_head forward that allocates nothing: its split scratch is a fixed array in device memory.
//
// This entry point has no counterpart in the reference framework. It exists for callers that must not
// touch an allocator on the call path (no cudaMalloc / cudaFree, no allocating library call is made here).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the static scratch array, in floats (4 MiB). A call needs
// T * vb_lmhead_num_splits(T, V) * 4 floats and is refused (-4, with a message on stderr) beyond that.
#define VB_LMHEAD_STATIC_SCRATCH_FLOATS (1 << 20)

int vb_lmhead_static_scratch_floats(void);

// Same contract and results as vb_lmhead_logprob_fwd, without the scratch argument.
//   hidden [T,H] bf16, weight [V,H] bf16, labels [T] int64; outputs fp32 [T], any may be null.
// Set-up: the first call on a device resolves the array's address with cudaGetSymbolAddress; make that first
//   call before any stream capture begins.
// Sharing: all calls on a device use the same array, so calls that overlap in time (different streams or
//   threads) race on it; order them on one stream.
// Initial contents: nothing in the array has to start at zero, every slot that the merge step reads is
//   written earlier in the same call.
// Returns 0, a CUDA error code (> 0), -3 for a bad shape, -4 when the scratch would not fit, -5 when the
//   array's address could not be resolved.
int vb_lmhead_logprob_fwd_static(const void* hidden, const void* weight, const long long* labels, int T, int H, int V,
                                 float inv_temperature, float* logprob, float* entropy, float* lse, float* mean,
                                 int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
