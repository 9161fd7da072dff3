// Link probes for the placement planner: what THIS machine's HBM and NVLink paths deliver.
//
// The reference's node telemetry probes Thunderbolt / RDMA links and socket reachability
// (src/exo/utils/info_gatherer/info_gatherer.py:444-462, net_profile.py:82-127) and its planner ranks
// cycles by what it finds.  Here the links are NVLink paths through NVSwitch and the planner's cost model
// wants three numbers per GPU: the streaming bandwidth of its own HBM, the one-direction copy bandwidth to
// each peer, and the latency of a small peer copy.  They are measured with plain copies timed by CUDA events
// (a copy kernel of the driver, no library kernel is given peer memory as an operand).
#include <cstdio>
#include "common.cuh"

namespace {
double elapsed_ms(cudaEvent_t a, cudaEvent_t b) {
  float ms = 0.f;
  cudaEventElapsedTime(&ms, a, b);
  return (double)ms;
}
}  // namespace

// Device-to-device copy on the current GPU: bytes read + bytes written over the time, best of `iters`.
// Returns GB/s (0 on failure).  `bytes` should exceed the L2 (>= 256 MiB).
EXO_API double exo_probe_hbm_copy(size_t bytes, int iters) {
  void *a = nullptr, *b = nullptr;
  if (cudaMalloc(&a, bytes) != cudaSuccess) return 0.0;
  if (cudaMalloc(&b, bytes) != cudaSuccess) { cudaFree(a); return 0.0; }
  cudaMemset(a, 1, bytes);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  double best = 1e30;
  for (int i = 0; i < iters + 2; i++) {           // two warm-up rounds
    cudaEventRecord(e0);
    cudaMemcpyAsync(b, a, bytes, cudaMemcpyDeviceToDevice);
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) { best = 1e30; break; }
    if (i >= 2) { const double ms = elapsed_ms(e0, e1); if (ms < best) best = ms; }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(a);
  cudaFree(b);
  return best > 1e29 ? 0.0 : 2.0 * (double)bytes / (best * 1e-3) / 1e9;
}

// One-direction copy from the current GPU to `peer`: bandwidth of `bytes`-sized copies (best of `iters`) and the
// latency of a 4-byte copy (median-free mean over 64 back-to-back copies).  Returns 0 on success, <0 when the
// pair has no peer access.
EXO_API int exo_probe_peer_copy(int peer, size_t bytes, int iters, double* gbps, double* latency_us) {
  int me = -1, can = 0;
  if (cudaGetDevice(&me) != cudaSuccess || peer == me) return -1;
  if (cudaDeviceCanAccessPeer(&can, me, peer) != cudaSuccess || !can) return -2;
  cudaError_t pe = cudaDeviceEnablePeerAccess(peer, 0);
  if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) return -2;
  cudaGetLastError();
  void *src = nullptr, *dst = nullptr;
  if (cudaMalloc(&src, bytes) != cudaSuccess) return -3;
  cudaSetDevice(peer);
  cudaError_t de = cudaMalloc(&dst, bytes);
  cudaSetDevice(me);
  if (de != cudaSuccess) { cudaFree(src); return -3; }
  cudaMemset(src, 1, bytes);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  double best = 1e30;
  int rc = 0;
  for (int i = 0; i < iters + 2 && rc == 0; i++) {
    cudaEventRecord(e0);
    cudaMemcpyPeerAsync(dst, peer, src, me, bytes);
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = -4;
    else if (i >= 2) { const double ms = elapsed_ms(e0, e1); if (ms < best) best = ms; }
  }
  if (rc == 0) {
    cudaEventRecord(e0);
    for (int i = 0; i < 64; i++) cudaMemcpyPeerAsync(dst, peer, src, me, 4);
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = -4;
    else *latency_us = elapsed_ms(e0, e1) * 1e3 / 64.0;
    *gbps = (double)bytes / (best * 1e-3) / 1e9;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(src);
  cudaSetDevice(peer);
  cudaFree(dst);
  cudaSetDevice(me);
  return rc;
}
