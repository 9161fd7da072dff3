// Tensor-parallel hand-over between a row-parallel projection and the kernel that consumes its all-reduced
// output, without a collective kernel in between (decode batches).
//
// Producer (row-parallel GEMV, or the GEMM's epilogue): every pair of adjacent outputs is stored straight into
// the slot `[parity][my rank]` of EVERY rank's arena as one 8-byte word that also carries the hand-over's
// sequence number.  Consumer (the next RMSNorm + GEMV, or the reduce + RMSNorm kernel): polls — bounded — the
// words it needs until they carry that number, and forms  x = residual + sum_r slot[parity][r]  in rank order
// (every rank gets the same bits).  Two hand-overs in flight are kept apart by the parity bit; a rank cannot run
// two ahead of a peer because consuming hand-over k needs that peer's push k.
#pragma once
#include <cuda_bf16.h>

constexpr int TP_MAX_RANKS = 8;

struct TpHandover {
  const __nv_bfloat16* x_res;               // residual stream before the reduction (may be null)
  __nv_bfloat16* x_out;                     // reduced residual stream (written by CTA 0; may be null)
  int* status;                              // device-writable status word of the collectives
  unsigned long long wait_ns;               // budget of a wait on a peer
  uint2* ll_mc;                             // multicast address of slot[parity][my rank] (null: store to ll_dst[r])
  uint2* ll_dst[TP_MAX_RANKS];              // rank r's slot[parity][my rank]
  const uint2* ll_part[TP_MAX_RANKS];       // my slots [parity][source rank]
  int* ll_epoch;                            // local: completed hand-overs of this parity
  int* ll_ticket;                           // local: consumer CTAs that have read the slots
  int n_ll;                                 // ranks (0: not a flag-in-data hand-over)
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
// Flag-in-data hand-over.  Every 8-byte word carries two bf16 outputs and the hand-over's sequence number
// (epoch + 1), written with ONE 8-byte store, which arrives whole: the consumer polls the words it needs until
// their sequence number matches, so there is no separate flag, no system-scope fence and no "last CTA" step on
// the producer's side — a row is on its way to every rank the moment it is computed.  With the multicast mapping
// one `multimem.st` reaches all ranks.  The local epoch word of a parity is advanced by the consumer's last CTA;
// all ranks perform the same sequence of hand-overs, so their epochs agree.
__device__ __forceinline__ void tp_ll_store(const TpHandover& h, size_t word, uint32_t data, uint32_t seq) {
  if (h.ll_mc) {
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(h.ll_mc + word), "r"(data), "r"(seq) : "memory");
  } else {
    for (int r = 0; r < h.n_ll; r++)
      asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(h.ll_dst[r] + word), "r"(data), "r"(seq) : "memory");
  }
}
// 16 bytes = two words {data0, seq0, data1, seq1}
__device__ __forceinline__ uint4 tp_ll_load2(const uint2* p) {
  uint4 r;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
// Polls until the four words at `p` (eight bf16 values) carry `seq`; returns false when the budget runs out.
__device__ __forceinline__ bool tp_ll_wait8(const uint2* p, uint32_t seq, unsigned long long wait_ns, uint32_t* data4) {
  unsigned long long t0 = 0;
  for (unsigned it = 0;; it++) {
    const uint4 a = tp_ll_load2(p), b = tp_ll_load2(p + 2);
    if (a.y == seq && a.w == seq && b.y == seq && b.w == seq) {
      data4[0] = a.x; data4[1] = a.z; data4[2] = b.x; data4[3] = b.z;
      return true;
    }
    if ((it & 63) == 63) {
      const unsigned long long now = tp_gtime();
      if (!t0) t0 = now;
      else if (now - t0 > wait_ns) return false;
    }
  }
}

// The same for all source ranks at once: the loads of every rank are in flight together (one L2 round trip per
// poll instead of one per rank), then the eight values are added to `acc` in rank order, so every rank forms the
// same bits.  Returns false when the budget runs out (acc is then left partly summed).
__device__ __forceinline__ bool tp_ll_gather8(const TpHandover& h, size_t word, uint32_t seq, float* acc) {
  uint4 a[TP_MAX_RANKS], b[TP_MAX_RANKS];
  unsigned pending = (1u << h.n_ll) - 1u;
  unsigned long long t0 = 0;
  for (unsigned it = 0; pending; it++) {
#pragma unroll
    for (int r = 0; r < TP_MAX_RANKS; r++)
      if ((pending >> r) & 1u) {
        a[r] = tp_ll_load2(h.ll_part[r] + word);
        b[r] = tp_ll_load2(h.ll_part[r] + word + 2);
      }
#pragma unroll
    for (int r = 0; r < TP_MAX_RANKS; r++)
      if (((pending >> r) & 1u) && a[r].y == seq && a[r].w == seq && b[r].y == seq && b[r].w == seq) pending &= ~(1u << r);
    if (pending && (it & 63) == 63) {
      const unsigned long long now = tp_gtime();
      if (!t0) t0 = now;
      else if (now - t0 > h.wait_ns) return false;
    }
  }
#pragma unroll
  for (int r = 0; r < TP_MAX_RANKS; r++)
    if (r < h.n_ll) {
      const uint4 d = make_uint4(a[r].x, a[r].z, b[r].x, b[r].z);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(p2[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
  return true;
}

// Host: fills `out` for the current device from the communicator set up by exo_comm_init.
// mode 3 / 4 = producer / consumer of a flag-in-data hand-over.  Returns 0, or <0 without a communicator / slot too small.
extern "C" int exo_tp_handover_fill(TpHandover* out, int mode, int parity, long n_elems);
