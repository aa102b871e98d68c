// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: nanoPLM reaches attention only through
// PyTorch / flash-attn, which allocate whatever workspace they need on the fly.
//
// Who needs it: code that runs where cudaMalloc is unavailable or forbidden -- a caller holding a
// fixed memory budget that was sized up front, a host thread that may not take the allocator's
// lock or trigger the implicit device synchronisation of cudaMalloc/cudaFree in the middle of a
// latency-critical section, or a plain C program that links the library without PyTorch's caching
// allocator. The regular entry point `nplm_fa_bwd` expects the caller to bring two scratch buffers
// (an fp32 dq accumulator of T*H*D floats and T*H floats of per-row statistics); here that scratch
// lives inside the library, in a file-scope `static __device__` array that every GPU loading the
// library holds until the process exits. The caller passes only inputs and outputs.
//
// Limits (a request beyond them is rejected with NPLM_NOALLOC_TOO_LARGE, nothing is launched):
//     T * H * D <= NPLM_NOALLOC_MAX_DQ_FLOATS     (4 Mi floats = 16 MiB, e.g. 4096 tokens x 16 heads)
//     T * H     <= NPLM_NOALLOC_MAX_STAT_FLOATS   (64 Ki floats = 256 KiB)
//
// The first call on a device looks up the device address of the array (cudaGetSymbolAddress) for
// that device; make that first call before starting any stream capture. The call itself performs
// no cudaMalloc / cudaFree and uses no allocating library routine. The device is taken from
// cudaGetDevice(), not from the stream: the current device must be the one that owns `stream` and
// the tensors. The per-device address cache is filled without a lock; two host threads that make the
// first call on one device at the same time both store the same value, which is harmless.
//
// All calls on a device share the one array and it keeps whatever the previous call left in it.
// The function clears the part that must start at zero on the caller's stream before using it.
// Two calls that overlap on the GPU (different streams, no ordering between them) race on the
// scratch and produce garbage: serialise them.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NPLM_NOALLOC_MAX_DQ_FLOATS ((size_t)4 << 20)
#define NPLM_NOALLOC_MAX_STAT_FLOATS ((size_t)64 << 10)
#define NPLM_NOALLOC_TOO_LARGE (-20)
#define NPLM_NOALLOC_SYMBOL_LOOKUP_FAILED (-21)

// Same arguments and results as nplm_fa_bwd minus the two scratch pointers. Returns 0, a
// cudaError_t (> 0) or one of the negative codes above / of nplm_fa_bwd.
int nplm_fa_bwd_noalloc(const void* qkv, const void* out, const void* dout, const float* lse,
                        void* dqkv, const int* seq_start, const int* seq_end, int T, int H, int D,
                        int window, float scale, int* status, cudaStream_t stream);

// Human-readable text for the codes this entry point can return.
const char* nplm_fa_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
