// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference; it exists for callers of this library that are not in a
// position to allocate device memory themselves.  Typical cases: a serving process whose HBM has been handed out
// completely to a KV-cache page pool and a weight arena at start-up, so that a later cudaMalloc can fail or force
// the owner of the pool to give memory back; a plug-in or custom call that runs inside another runtime which owns
// the device allocator and accounts for every byte; a latency-critical loop in which the implicit device-wide
// synchronisation of cudaMalloc/cudaFree is not acceptable.
//
// b200_rmsnorm_bwd_noalloc computes the same result as b200_norm_bwd(..., is_layernorm = 0): the RMSNorm input
// gradient dx and the weight gradient dw.  The per-CTA partial weight gradients, which b200_norm_bwd keeps in a
// caller-provided scratch buffer, live here in a file-scope device array inside the library:
//
//   size     B200_NOALLOC_CTAS * B200_NOALLOC_MAX_H floats = 148 * 8192 * 4 bytes = 4.6 MiB,
//            resident on every GPU that loads the library, until the process exits;
//   limit    H <= B200_NOALLOC_MAX_H (and H % 8 == 0); larger H is rejected with B200_NOALLOC_ERR_TOO_LARGE
//            and nothing is launched;
//   set-up   the first call on each device looks up the array's device address (no allocation) and caches it;
//            make that first call from ordinary stream code, before any stream capture is begun;
//   sharing  every call on a device uses the same array.  Each call overwrites the part it reads, so nothing has
//            to be cleared between calls, but two calls that overlap in time on one GPU (different streams,
//            different threads) race on it: serialise them on one stream or with events;
//   it calls no cudaMalloc, cudaFree or any allocating library routine; inputs and outputs are the caller's.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_NOALLOC_CTAS 148
#define B200_NOALLOC_MAX_H 8192
#define B200_NOALLOC_ERR_TOO_LARGE (-20)
#define B200_NOALLOC_ERR_SYMBOL (-21)

// dy, x, dx: [rows, H] bf16 (dx written); w: [H] bf16; rstd: [rows] fp32 as saved by b200_norm_fwd;
// dres: optional [rows, H] bf16 added to dx (gradient arriving on the residual branch), may be NULL;
// dw_f32 / dw_bf16: weight gradient outputs, either may be NULL; accumulate != 0 adds to them instead of overwriting.
// Returns 0 on success, B200_NOALLOC_ERR_TOO_LARGE if H exceeds the limit, another negative code on failure.
int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                             float* dw_f32, void* dw_bf16, int accumulate, int rows, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
