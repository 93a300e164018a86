// Allocation-free scoring entry point (this has no counterpart in the reference).
//
// Some embedders of this library may not allocate device memory at the moment they need a
// score: a host application that handed the GPU's memory to its own pool and forbids
// cudaMalloc from plug-ins, a latency-critical scorer whose budget cannot absorb the implicit
// device synchronisation of cudaMalloc / cudaFree, or a callback that runs while another
// component owns the allocator.  The regular path (dz_gemm_bf16_tn_lse + dz_lse_combine)
// needs caller-provided scratch for the per-column-tile log-sum-exp partials; this entry point
// keeps that scratch in a fixed device array inside the library instead.
//
//   log p(target_r | row r) = logit[r, target_r] - logsumexp_n( scale * <A[r, :], W[n, :]> )
//
// Limits (fixed by the size of the built-in scratch, 1 MiB + 2 KiB per GPU that loads the
// library, held until the process exits):  M <= DZ_NOALLOC_MAX_ROWS rows,
// N <= DZ_NOALLOC_MAX_VOCAB columns.  Larger problems are rejected with DZ_ERR_TOO_LARGE (4).
//
// Behaviour to know about:
//  * The first call on each device looks up the device address of the scratch array
//    (cudaGetSymbolAddress) with that device current; make that first call outside any stream
//    capture.  Later calls only launch kernels and one cudaMemsetAsync on `stream`.  Two host
//    threads that both make the first call on one device may both do this lookup; each stores the
//    same address into the per-device slot, so the outcome is the same (the stores are plain, not
//    atomic: if that matters to a race detector, make the first call from one thread).  The
//    kernel launch attributes and the SM count are cached per device as well, so one process may
//    use the entry point on several GPUs.
//  * It never calls cudaMalloc, cudaFree or any allocating library routine.
//  * Every call on a device shares the one scratch array, which still holds the previous
//    call's partials; the part that must start clean is cleared on `stream` by the call itself.
//    Two calls that overlap on the GPU (different streams, no ordering) race on it: serialise
//    them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define DZ_NOALLOC_MAX_ROWS 512
#define DZ_NOALLOC_MAX_VOCAB 65536

#ifdef __cplusplus
extern "C" {
#endif

// A [M, lda] bf16 (K used columns), W [N, ldw] bf16, targets [M] int32 device pointer,
// out_logprob [M] fp32 device pointer, err: device word for wait time-outs (may be null).
// Returns 0 on success, a small positive code for argument errors, 1000 + cudaError_t otherwise.
int dz_token_logprobs_noalloc(const void* A, long long lda, const void* W, long long ldw,
                              const int* targets, float* out_logprob, int M, int N, int K,
                              float scale, uint32_t* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
