// Allocation-free decode attention: the split-KV scratch of exo_paged_decode() kept inside the
// library (declared and documented in exo_noalloc.h; no counterpart in the reference project).
#include "common.cuh"

// regular entry points of attention_decode.cu
extern "C" long exo_paged_decode_workspace(int B, int Hq, int D, int n_splits);
extern "C" int exo_paged_decode(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                                const int* seq_lens, void* out, float* workspace, int* tickets, float scale, int B,
                                int Hq, int Hkv, int D, int max_blocks, int block_size, int n_splits, int window,
                                const float* sinks, int dtype, cudaStream_t st);

// ------------------------------------------------------------------------------------------------
// The scratch is a file-scope device array.  In host code its NAME is only a host-side stand-in
// for the symbol, not a device address, so the address is fetched once per device with
// cudaGetSymbolAddress and that pointer is what the kernel receives.
// ------------------------------------------------------------------------------------------------
#include "exo_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[EXO_NOALLOC_MAX_FLOATS];
static __device__ __align__(256) int g_noalloc_tickets[EXO_NOALLOC_MAX_TICKETS];

namespace {
float* g_noalloc_scratch_addr[16] = {nullptr};
int* g_noalloc_tickets_addr[16] = {nullptr};
}  // namespace

EXO_API int exo_paged_decode_noalloc(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                                     const int* seq_lens, void* out, float scale, int B, int Hq, int Hkv, int D,
                                     int max_blocks, int block_size, int n_splits, int window, const float* sinks,
                                     int dtype, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (n_splits < 1 || n_splits > 64) return -2;
  const long need = exo_paged_decode_workspace(B, Hq, D, n_splits);
  if (need > (long)EXO_NOALLOC_MAX_FLOATS || (long)B * Hq > (long)EXO_NOALLOC_MAX_TICKETS) return -7;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 16) return -1;
  if (!g_noalloc_scratch_addr[dev]) {  // once per device, with that device current
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    void* t = nullptr;
    e = cudaGetSymbolAddress(&t, g_noalloc_tickets);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_tickets_addr[dev] = static_cast<int*>(t);
    g_noalloc_scratch_addr[dev] = static_cast<float*>(p);
  }
  // tickets must start at zero; the scratch is shared and keeps whatever the last call left
  e = cudaMemsetAsync(g_noalloc_tickets_addr[dev], 0, sizeof(int) * (size_t)B * Hq, stream);
  if (e != cudaSuccess) return (int)e;
  return exo_paged_decode(q, kcache, vcache, block_tables, seq_lens, out, g_noalloc_scratch_addr[dev],
                          g_noalloc_tickets_addr[dev], scale, B, Hq, Hkv, D, max_blocks, block_size, n_splits, window,
                          sinks, dtype, stream);
}
