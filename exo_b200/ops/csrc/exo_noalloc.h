// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference project: it exists for callers of this
// library that are not in a position to allocate device memory when they need attention results.
// Three kinds of caller are meant:
//   * a serving process that has already handed every free byte of HBM to its paged KV pool, so a
//     later cudaMalloc for attention scratch can fail (or succeed only by fragmenting the pool);
//   * a latency-critical host thread that must not run into the device-wide synchronisation that
//     cudaMalloc / cudaFree imply while other streams are busy;
//   * a plain C / C++ embedder that links this library without PyTorch and therefore has no
//     caching allocator to borrow scratch from.
// They still pass their own inputs and outputs; only the scratch is provided by the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch (one set per GPU that loads the library, held until exit):
//   partial results : EXO_NOALLOC_MAX_FLOATS floats (8 MiB)  >= B * Hq * n_splits * (D + 2)
//   tickets         : EXO_NOALLOC_MAX_TICKETS ints           >= B * Hq
#define EXO_NOALLOC_MAX_FLOATS (2u << 20)
#define EXO_NOALLOC_MAX_TICKETS (16u << 10)

// Paged-KV decode attention, same arithmetic and argument meaning as exo_paged_decode(), but the
// split-KV partials and tickets live in a file-scope __device__ array inside the library instead of
// a caller-supplied workspace.  Calls no cudaMalloc / cudaFree and no allocating library routine.
//
// Returns 0 on success; -7 when the problem needs more scratch than the limits above (nothing is
// launched); -2 for an unsupported shape; a positive cudaError_t value if a CUDA call failed.
//
// The first call on each device looks up the device address of the scratch (cudaGetSymbolAddress,
// with that device current); make that first call before any stream capture.  All calls on a
// device share the one scratch array and it keeps the previous call's contents: the entry point
// clears the ticket words on `stream` before every launch, and two calls whose kernels overlap on
// the GPU (different streams, no dependency) race on it — serialise them.
int exo_paged_decode_noalloc(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                             const int* seq_lens, void* out, float scale, int B, int Hq, int Hkv, int D,
                             int max_blocks, int block_size, int n_splits, int window, const float* sinks, int dtype,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
