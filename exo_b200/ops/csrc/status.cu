// Per-device status block of the kernel library, in mapped pinned host memory.
//
// Every device-side wait in this library is bounded; a wait that runs out records a code and the
// kernel unwinds normally.  The words those codes go to live in host memory that the GPU can write
// (cudaHostAlloc, mapped), so the serving loop reads them after every step with a plain load: no
// copy, no stream synchronisation of its own, nothing to capture in a CUDA graph.  A kernel's write
// is visible to the host once the kernel has completed, which is when the host looks (the step's
// sampled ids have just been read back).
//
//   word 0  tensor-core kernels (GEMM, attention, MoE): tc::ERR_* of the first wait that expired
//   word 1  streaming GEMV
//   word 2  peer-memory collectives / hand-overs: 4 = a peer never signalled
//   word 3  wait budget of the collectives in microseconds (host-written, read by the launchers)
//
// The reference has no device code; its counterpart of this path is the runner supervisor turning a
// dead or stuck runner into RunnerFailed (src/exo/worker/runner/supervisor.py:364-440).
#include "status.h"

#include <mutex>

namespace {
int* g_block[16] = {nullptr};
std::mutex g_mu;
unsigned long long g_wait_ns = 2000000000ull;   // collectives: 2 s unless the host sets another budget
}  // namespace

int* exo_status_block() {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_block[dev]) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return nullptr;
    memset(p, 0, 64);
    g_block[dev] = static_cast<int*>(p);   // unified addressing: the host pointer is the device pointer
  }
  return g_block[dev];
}

int* exo_status_word(int which) {
  int* b = exo_status_block();
  return b ? b + which : nullptr;
}

unsigned long long exo_wait_budget_ns() { return g_wait_ns; }

// Host address of the current device's status block (4 int32 words used); 0 on failure.
EXO_API void* exo_status_host_ptr() { return exo_status_block(); }

// Sets the wait budget of the peer-memory collectives and hand-overs (microseconds, >= 100).
EXO_API int exo_set_collective_timeout_us(long us) {
  if (us < 100) us = 100;
  g_wait_ns = (unsigned long long)us * 1000ull;
  return 0;
}

// Reads (and optionally clears) word `which` without touching the device.  Call it when the kernels
// of interest have completed.
EXO_API int exo_status_take(int which, int clear) {
  int* b = exo_status_block();
  if (!b || which < 0 || which > 2) return 0;
  volatile int* w = b + which;
  const int v = *w;
  if (v && clear) *w = 0;
  return v;
}
