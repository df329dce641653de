/* ember_gemm_tc_noalloc: a matrix product for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference engine; it exists only in this library.
 *
 * Who needs it: code that runs where cudaMalloc is off the table.  Examples are a host program
 * that hands its whole device-memory budget out at start-up and forbids later allocations, a
 * latency-critical loop in which the implicit device synchronisation of cudaMalloc/cudaFree is
 * unacceptable, and plug-ins that are only given buffers by their host application and have no
 * allocator of their own.  The regular entry point (ember_gemm_tc) asks its caller for a zeroed
 * scratch buffer for split-K partial sums, which such callers cannot provide; this variant keeps
 * that scratch inside the library instead.
 *
 * What it computes: out = epilogue(A[M,K] . W[N,K]^T) with bf16 operands and fp32 accumulation,
 * for the small-M ("decode") orientation of the tcgen05 kernel, M <= 128.  Epilogues: 0 store
 * bf16, 1 store fp32, 2 add into fp32 `out`, 3 silu(gate) * up over interleaved rows -> bf16.
 * `ldc` is the row stride of `out` in elements (at least N, or N / 2 for epilogue 3; a shorter one
 * is refused, as are null pointers).  Inputs and outputs are the caller's; `err` may be null or
 * point to one device int that collects error bits.
 *
 * Limits: M <= 128, K a multiple of 8, and M * N <= EMBER_NOALLOC_SCRATCH_FLOATS (1,048,576
 * floats = 4 MiB of fp32 scratch).  Larger sizes are refused with an error; nothing is truncated.
 *
 * Cost: the scratch is a file-scope __device__ array, so every GPU that loads this library holds
 * those 4 MiB until the process exits.
 *
 * Set-up: the first call on a device looks the array's device address up
 * (cudaGetSymbolAddress) with that device current.  Make that first call outside any stream
 * capture.  No call allocates or frees device memory, and none calls an allocating library
 * routine.
 *
 * Sharing: every call uses the same array, which keeps whatever the last call left in it.  Each
 * call clears the part it needs on its stream before the kernel runs.  Two calls whose work
 * overlaps on the GPU (different streams without ordering between them) race on the array and
 * give wrong sums; order them.
 *
 * Returns 0, or non-zero with a message from ember_last_error() of this library.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define EMBER_NOALLOC_SCRATCH_FLOATS (1 << 20)

int ember_gemm_tc_noalloc(const void* A, const void* W, void* out, int ldc, int M, int N, int K, int epilogue,
                          int* err, void* stream);

const char* ember_last_error(void);

#ifdef __cplusplus
}
#endif
