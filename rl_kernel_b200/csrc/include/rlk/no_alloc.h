// Entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (RL-Kernel's operators always receive
// their workspaces from PyTorch's allocator).
//
// Who needs it: code that runs where a device allocation is forbidden or unwanted -- a serving
// loop that has handed every free byte of the GPU to its KV-cache pool, a plugin called while
// the host framework has frozen its memory plan, a process whose allocator may not be re-entered
// from the calling thread.  Such callers can pass inputs and outputs they already own, but they
// cannot provide (or let the library create) the temporary buffer the chunked small-M GEMM needs
// between its two kernels.
//
// rlk_det_gemm_split_static computes exactly what rlk_det_gemm_split computes (bitwise the same
// result: C[M,N] = A[M,K] * B[N,K]^T with `nchunks` canonical K chunks combined by the balanced
// bf16 tree) but takes no scratch pointer.  The per-chunk partial results live in a buffer that is
// part of the library image: a file-scope `static __device__` array of RLK_STATIC_SCRATCH_BYTES
// (8 MiB).  Consequences the caller has to know:
//   * every GPU that loads the library carries those 8 MiB until the process exits;
//   * the request must fit: nchunks * M * ldc * 2 bytes <= RLK_STATIC_SCRATCH_BYTES, otherwise the
//     call fails with RLK_ERR_BAD_ARG and launches nothing (for example 8 chunks x 64 rows x
//     ldc 4096 needs 4 MiB);
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and sets a kernel attribute; make that first call before you start
//     capturing a stream;
//   * all calls on a device share the one array, which keeps whatever the previous call left in
//     it.  Nothing in it has to start at zero -- every partial that is read has been written by
//     the same call -- but two calls that overlap on the GPU (different streams, or concurrent
//     host threads) would overwrite each other's partials: serialise them on one stream;
//   * no cudaMalloc, cudaFree or allocating library routine is called, on the first call or later;
//   * a device-side wait that gives up (the bounded-wait safety net) still ends the kernel, but
//     this variant has no status word to record it in; callers that need that report use
//     rlk_det_gemm_split.
// Arguments are those of rlk_det_gemm_split without `scratch`, with two differences: C must not be
// null (rlk_det_gemm_split's leaves-only mode, C == nullptr, has no meaning here because the
// partials never leave the library), and ldc >= N is required so that the last chunk's partials
// stay inside the checked size.  A null A, B or C, or ldc < N, fails with RLK_ERR_BAD_ARG before
// anything is launched.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RLK_STATIC_SCRATCH_BYTES (8ll << 20)

int rlk_det_gemm_split_static(const void* A, const void* B, void* C, int M, int N, int K,
                              long long lda, long long ldb, long long ldc, int nchunks, int tile_n,
                              void* stream);

#ifdef __cplusplus
}
#endif
