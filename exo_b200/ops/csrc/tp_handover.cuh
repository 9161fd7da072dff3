// Tensor-parallel hand-over between a row-parallel projection and the kernel that consumes its
// all-reduced output, without a collective kernel in between.
//
// Producer (row-parallel GEMV): every output element is stored straight into the staging slot
// `[parity][my rank]` of EVERY rank's arena (peer stores over NVSwitch) as the row groups finish;
// the last CTA of the grid then bumps one flag per rank with a release-scoped remote atomic.
// Consumer (the next RMSNorm + GEMV, or the stand-alone finish kernel): waits — bounded — until all
// ranks' flags for `parity` are up, forms  x = residual + sum_r slot[parity][r]  in rank order
// (every rank gets the same bits), and its last CTA clears the flags for the parity's next use.
// Two hand-overs in flight are kept apart by the parity bit; a rank cannot run two ahead of a
// peer because consuming hand-over k needs that peer's push k.
#pragma once
#include <cuda_bf16.h>

constexpr int TP_MAX_RANKS = 8;

struct TpHandover {
  // producer side (n_push > 0)
  __nv_bfloat16* push_dst[TP_MAX_RANKS];    // rank r's staging slot for my partial
  int* push_flag[TP_MAX_RANKS];             // rank r's flag word for (parity, me)
  int* push_ticket;                         // local: CTAs that finished pushing
  int n_push;
  // consumer side (n_part > 0)
  const __nv_bfloat16* part[TP_MAX_RANKS];  // my staging slots, one per source rank
  int* part_flag[TP_MAX_RANKS];             // my flag words for (parity, src)
  int* part_ticket;                         // local: CTAs that finished reading
  int n_part;
  const __nv_bfloat16* x_res;               // residual stream before the reduction (may be null)
  __nv_bfloat16* x_out;                     // reduced residual stream (written by CTA 0; may be null)
  int* status;                              // device-writable status word of the collectives
  unsigned long long wait_ns;               // budget of a wait on a peer
};

__device__ __forceinline__ int tp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 16-byte load that bypasses L1: the staging slots are written by other GPUs while this kernel runs
__device__ __forceinline__ uint4 tp_ld_cg16(const void* p) {
  uint4 r;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
__device__ __forceinline__ unsigned long long tp_gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// One thread per source rank polls; returns false when the budget runs out (and records code 4 in the status word).
__device__ __forceinline__ bool tp_wait_flag(int* flag, int* status, unsigned long long wait_ns) {
  const unsigned long long t0 = tp_gtime();
  while (tp_ld_acquire_sys(flag) < 1) {
    if (tp_gtime() - t0 > wait_ns) {
      atomicExch(status, 4);
      return false;
    }
    __nanosleep(32);
  }
  return true;
}

// Host: fills `out` for the current device from the communicator set up by exo_comm_init.
// mode 1 = producer fields, 2 = consumer fields.  Returns 0, or <0 without a communicator / slot too small.
extern "C" int exo_tp_handover_fill(TpHandover* out, int mode, int parity, long n_elems);
