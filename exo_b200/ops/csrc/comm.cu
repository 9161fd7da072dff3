// Tensor-parallel collectives over NVLink peer memory (no NCCL on this path).
//
// Every rank owns one "arena" allocated with cudaMalloc and exported through CUDA IPC; all ranks
// map all arenas, so a kernel can store straight into a peer's HBM through NVSwitch.  Layout of an
// arena (identical on every rank):
//
//   [0, 4 KB)        flags   int32 [2 parities][8 source ranks]   signals received, reset by reader
//                    tickets int32 [2 parities] at +256          local CTA tickets
//                    status  int32 at +512                       device-side error word (timeouts)
//   [4 KB, ...)      staging [2 parities][n_ranks][slot_bytes]   partials pushed by each source rank
//   [... , end)      gather  [gather_bytes]                      all-gather target (vocab logits)
//   then             the regions of the in-switch reduction (see "reduce + norm" below):
//                    partial [2 parities][x_bytes]  this rank's not-yet-reduced projection output
//                    hbuf / nbuf [2][x_bytes]       residual stream / normalised rows written by the two-shot form
//   header +2048     barrier flags int32 [2 parities][8] "partial ready", +2112 [2][8] "rows broadcast", +2176 tickets [2]
//
// One-shot all-reduce (small / decode-sized tensors): every rank pushes its partial into every
// rank's staging[parity][src], signals with a release-scoped remote atomic, waits (bounded) until
// all sources have signalled, and sums the partials in rank order — every rank computes the same
// bits.  Two calls in flight are separated by the parity bit; a rank cannot run two collectives
// ahead of a peer because each reduction needs that peer's next partial.
//
// Waits are bounded by a globaltimer budget: on expiry the kernel records an error code in the
// status word and returns normally, so the context stays usable and the host raises.
#include "common.cuh"
#include "status.h"
#include "tp_handover.cuh"

namespace {

constexpr int MAX_RANKS = 8;
constexpr size_t HDR_BYTES = 4096;
constexpr size_t BAR_IN = 2048, BAR_OUT = 2112, BAR_TICKET = 2176, BAR_GATHER = 2240;   // tickets: int32 [3]; gather flags [8]
constexpr size_t LL_EPOCH = 2304, LL_TICKET = 2368;   // flag-in-data hand-over: int32 [2 parities] each
constexpr size_t RN_EPOCH = 2432;                     // two-shot reductions completed per parity: int32 [2]

struct CommCtx {
  uint8_t* arena[MAX_RANKS];  // arena[r] = base of rank r's arena as mapped in this process
  int n, rank;
  size_t slot_bytes;          // bytes of one staging slot
  size_t gather_off;          // byte offset of the gather region
  uint8_t* mc;                // multicast address of the arena (nullptr: plain peer loads / stores)
  size_t x_off, x_bytes;      // partial buffers [2 parities][x_bytes] (0 = none)
  size_t h_off, n_off;        // two-shot outputs [2][x_bytes]: residual stream, normalised rows
  size_t ll_off, ll_slot;     // flag-in-data hand-over slots [2 parities][n_ranks][ll_slot] (ll_slot = 0: none)
  int* status;                // device-writable status word (host-mapped)
  unsigned long long wait_ns; // budget of every wait on a peer
};

__device__ __forceinline__ int* flag_ptr(uint8_t* arena, int parity, int src) {
  return reinterpret_cast<int*>(arena) + parity * MAX_RANKS + src;
}
__device__ __forceinline__ uint8_t* slot_ptr(const CommCtx& c, uint8_t* arena, int parity, int src) {
  return arena + HDR_BYTES + ((size_t)parity * c.n + src) * c.slot_bytes;
}
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
  uint4 r;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// Bounded wait until all n sources have signalled `need` times on (parity).  Returns false on timeout.
__device__ bool wait_all(const CommCtx& c, int parity, int need) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.n) {
    const int* f = flag_ptr(c.arena[c.rank], parity, threadIdx.x);
    unsigned long long t0 = gtime();
    while (ld_acquire_sys(f) < need) {
      if (gtime() - t0 > c.wait_ns) {
        ok_s = 0;
        atomicExch(c.status, 4 /* peer timeout */);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return ok_s != 0;
}

// Signal every rank (including self): this CTA's share of (parity) is complete.
__device__ void signal_all(const CommCtx& c, int parity) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.n) red_release_sys_add(flag_ptr(c.arena[threadIdx.x], parity, c.rank), 1);
}

// Last CTA of the grid (local ticket) resets the flags of (parity) for their next use.
__device__ void finish_and_reset(const CommCtx& c, int parity) {
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = reinterpret_cast<int*>(c.arena[c.rank] + 256) + parity;
    __threadfence();
    if (atomicAdd(tk, 1) == (int)gridDim.x - 1) {
      *tk = 0;
      for (int r = 0; r < c.n; r++) *flag_ptr(c.arena[c.rank], parity, r) = 0;
      __threadfence_system();
    }
  }
}

// out = residual + sum_r partial_r     (bf16, fp32 accumulation in rank order), n_vec 16-byte vectors
__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(const CommCtx c, const uint4* __restrict__ in, const uint4* residual, uint4* out, int n_vec,
                         int parity) {
  pdl_trigger();
  pdl_wait();
  const int per = (n_vec + gridDim.x - 1) / gridDim.x;
  const int v0 = blockIdx.x * per, v1 = min(n_vec, v0 + per);
  // push my slice of the partial into every rank's staging[parity][me]
  for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    uint4 x = in[v];
    for (int r = 0; r < c.n; r++) reinterpret_cast<uint4*>(slot_ptr(c, c.arena[r], parity, c.rank))[v] = x;
  }
  signal_all(c, parity);
  const bool ok = wait_all(c, parity, gridDim.x);
  if (ok) {
    for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      float acc[8];
      if (residual) unpack8(residual[v], acc);
      else {
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.f;
      }
      for (int r = 0; r < c.n; r++) {
        float f[8];
        unpack8(ld_cg16(reinterpret_cast<const uint4*>(slot_ptr(c, c.arena[c.rank], parity, r)) + v), f);
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] += f[e];
      }
      out[v] = pack8(acc);
    }
  }
  finish_and_reset(c, parity);
}

// Two-shot all-reduce for large tensors: reduce-scatter (each rank pushes slice j to rank j),
// rank j sums its slice, then broadcasts the reduced slice to everyone's `out` through a second
// staging round.  Bytes on the wire per rank: 2 (n-1)/n of the tensor instead of (n-1) x.
__global__ void __launch_bounds__(256)
allreduce_twoshot_kernel(const CommCtx c, const uint4* __restrict__ in, const uint4* residual, uint4* out, int n_vec,
                         int parity) {
  pdl_trigger();
  pdl_wait();
  const int n = c.n;
  const int per_rank = (n_vec + n - 1) / n;  // slice owned by each rank
  // phase 1: scatter — my contribution to slice j goes to rank j's staging[parity][me] (slice-local index)
  for (int j = 0; j < n; j++) {
    const int s0 = j * per_rank, s1 = min(n_vec, s0 + per_rank);
    uint4* dst = reinterpret_cast<uint4*>(slot_ptr(c, c.arena[j], parity, c.rank));
    for (int v = s0 + blockIdx.x * blockDim.x + threadIdx.x; v < s1; v += gridDim.x * blockDim.x) dst[v - s0] = in[v];
  }
  signal_all(c, parity);
  bool ok = wait_all(c, parity, gridDim.x);
  // phase 2: reduce my slice and push the result into every rank's second half of the slot
  const int m0 = c.rank * per_rank, m1 = min(n_vec, m0 + per_rank);
  const size_t half = c.slot_bytes / 2 / sizeof(uint4);
  if (ok) {
    for (int v = m0 + blockIdx.x * blockDim.x + threadIdx.x; v < m1; v += gridDim.x * blockDim.x) {
      float acc[8];
      if (residual) unpack8(residual[v], acc);
      else {
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.f;
      }
      for (int r = 0; r < n; r++) {
        float f[8];
        unpack8(ld_cg16(reinterpret_cast<const uint4*>(slot_ptr(c, c.arena[c.rank], parity, r)) + (v - m0)), f);
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] += f[e];
      }
      uint4 y = pack8(acc);
      for (int r = 0; r < n; r++)
        (reinterpret_cast<uint4*>(slot_ptr(c, c.arena[r], parity, c.rank)) + half)[v - m0] = y;
    }
  }
  signal_all(c, parity);
  ok = wait_all(c, parity, 2 * gridDim.x) && ok;
  // phase 3: gather the reduced slices from my staging into out
  if (ok) {
    for (int j = 0; j < n; j++) {
      const int s0 = j * per_rank, s1 = min(n_vec, s0 + per_rank);
      const uint4* src = reinterpret_cast<const uint4*>(slot_ptr(c, c.arena[c.rank], parity, j)) + half;
      for (int v = s0 + blockIdx.x * blockDim.x + threadIdx.x; v < s1; v += gridDim.x * blockDim.x)
        out[v] = ld_cg16(src + (v - s0));
    }
  }
  finish_and_reset(c, parity);
}

// All-gather of column shards: in [rows, cols] local shard → every rank's gather region
// [rows, n * cols] at column offset rank * cols.  cols * 2 bytes must be a multiple of 16.
__global__ void __launch_bounds__(256)
allgather_cols_kernel(const CommCtx c, const uint4* __restrict__ in, int rows, int cols_vec, int parity) {
  pdl_trigger();
  pdl_wait();
  const int total = rows * cols_vec;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int r = i / cols_vec, cv = i - r * cols_vec;
    uint4 x = in[i];
    const size_t dst = (size_t)r * c.n * cols_vec + (size_t)c.rank * cols_vec + cv;
    for (int p = 0; p < c.n; p++) reinterpret_cast<uint4*>(c.arena[p] + c.gather_off)[dst] = x;
  }
  signal_all(c, parity);
  wait_all(c, parity, gridDim.x);
  finish_and_reset(c, parity);
}


// ---- reduce + norm: the all-reduce after a row-parallel projection, fused with the residual add and the RMSNorm ----
//
// The projection (our GEMM) writes this rank's partial  y_r [rows, cols]  into partial[parity] of its OWN arena: no
// peer stores.  One kernel then forms   h = residual + sum_r y_r   and   x = RMSNorm(h) * w:
//   * one-shot (decode batches): every rank reduces every row.  With the multicast mapping one
//     `multimem.ld_reduce` per 16 bytes returns the sum over all ranks, formed inside NVSwitch; without it the rows
//     are read from each peer's arena with plain loads and summed in rank order.
//   * two-shot (prefill chunks): rank j reduces rows [j R, (j+1) R) only, and writes its h and x rows into every
//     rank's hbuf / nbuf (`multimem.st`, or peer stores): (n-1)/n + 2/n of the tensor per direction instead of n-1.
// Synchronisation: CTA 0 raises "partial ready" on every rank once (one remote atomic per peer and collective, not
// per CTA); every CTA waits for all ranks' flags (bounded).  The last CTA of the grid (local ticket) clears the
// flags of the parity; in the two-shot form it first raises "rows broadcast" on every rank and waits for everyone
// else's, so that when the kernel completes all rows have landed.  Parities alternate per collective, and a rank
// cannot get two collectives ahead of a peer (it needs that peer's next partial), which is what makes reuse safe.

__device__ __forceinline__ int* bar_ptr(uint8_t* arena, size_t base, int parity, int src) {
  return reinterpret_cast<int*>(arena + base) + parity * MAX_RANKS + src;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait of the whole CTA until every rank's flag (base, parity) has reached `need` (wrap-safe comparison).
__device__ bool wait_ranks_ge(const CommCtx& c, size_t base, int parity, int need) {
  __shared__ int ok_g;
  if (threadIdx.x == 0) ok_g = 1;
  __syncthreads();
  if (threadIdx.x < c.n) {
    const int* f = bar_ptr(c.arena[c.rank], base, parity, threadIdx.x);
    const unsigned long long t0 = gtime();
    while (ld_acquire_sys(f) - need < 0) {
      if (gtime() - t0 > c.wait_ns) {
        ok_g = 0;
        atomicExch(c.status, 4 /* peer timeout */);
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  return ok_g != 0;
}

// Bounded wait of the whole CTA until every rank has raised flag (base, parity) at least once.
__device__ bool wait_ranks(const CommCtx& c, size_t base, int parity) {
  __shared__ int ok_w;
  if (threadIdx.x == 0) ok_w = 1;
  __syncthreads();
  if (threadIdx.x < c.n) {
    const int* f = bar_ptr(c.arena[c.rank], base, parity, threadIdx.x);
    const unsigned long long t0 = gtime();
    while (ld_acquire_sys(f) < 1) {
      if (gtime() - t0 > c.wait_ns) {
        ok_w = 0;
        atomicExch(c.status, 4 /* peer timeout */);
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  return ok_w != 0;
}

constexpr int RN_THREADS = 256, RN_WARPS = RN_THREADS / 32;

// One warp per row: all of the row's 16-byte vectors are requested before the first is used (VPL of them per
// lane), the row stays in registers as packed bf16 between the sum of squares and the scaling, and warps never
// wait for one another inside the row loop.
//   TWO = false: h_out / x_out are this rank's private [rows, cols] tensors and every rank computes all rows.
//   TWO = true:  this rank computes rows [rank R, (rank + 1) R) only.  Its normalised rows go into nbuf[parity] of
//                EVERY rank; its residual-stream rows go into hbuf[parity] of every rank when `bcast_h`, else into
//                the same rows of the private h_out (the stream then stays sharded by rows: the next reduction of
//                the same shape needs exactly these rows as its residual).
template <bool MC, bool TWO, int VPL>
__global__ void __launch_bounds__(RN_THREADS)
reduce_norm_kernel(const CommCtx c, const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ norm_w,
                   float eps, __nv_bfloat16* h_out, __nv_bfloat16* x_out, int rows, int cols, int parity, int mode) {
  pdl_trigger();
  pdl_wait();
  __shared__ int last_s;
  const bool bcast_h = mode & 1, defer_wait = mode & 2;
  if (blockIdx.x == 0 && threadIdx.x < c.n) {
    __threadfence_system();   // the partial was written by earlier kernels of this stream: publish it system-wide
    red_release_sys_add(bar_ptr(c.arena[threadIdx.x], BAR_IN, parity, c.rank), 1);
  }
  const bool ok = wait_ranks(c, BAR_IN, parity);
  const int n_vec = cols / 8, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int row0 = 0, row1 = rows;
  if (TWO) {
    const int per = (rows + c.n - 1) / c.n;
    row0 = min(rows, c.rank * per);
    row1 = min(rows, row0 + per);
  }
  const size_t part_off = c.x_off + (size_t)parity * c.x_bytes;
  if (ok) {
    for (int row = row0 + blockIdx.x * RN_WARPS + warp; row < row1; row += gridDim.x * RN_WARPS) {
      const size_t base = (size_t)row * cols;
      uint4 hp[VPL];
      if (MC) {
#pragma unroll
        for (int j = 0; j < VPL; j++) {
          const int iv = lane + 32 * j;
          if (iv < n_vec) hp[j] = multimem_ld_reduce_bf16x8(c.mc + part_off + (base + (size_t)iv * 8) * 2);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VPL; j++) {
        const int iv = lane + 32 * j;
        if (iv < n_vec) {
          const size_t off = base + (size_t)iv * 8;
          float v[8];
          if (MC) unpack8(hp[j], v);
          else {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = 0.f;
            for (int r = 0; r < c.n; r++) {
              float f[8];
              unpack8(ld_cg16(c.arena[r] + part_off + off * 2), f);
#pragma unroll
              for (int e = 0; e < 8; e++) v[e] += f[e];
            }
          }
          if (residual) {
            float r8[8];
            unpack8(*reinterpret_cast<const uint4*>(residual + off), r8);
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] += r8[e];
          }
          hp[j] = pack8(v);                            // the residual stream is kept in bf16: normalise what is stored
          if (TWO && bcast_h) {
            const size_t boff = c.h_off + (size_t)parity * c.x_bytes + off * 2;
            if (MC) multimem_st16(c.mc + boff, hp[j]);
            else
              for (int r = 0; r < c.n; r++) *reinterpret_cast<uint4*>(c.arena[r] + boff) = hp[j];
          } else {
            *reinterpret_cast<uint4*>(h_out + off) = hp[j];
          }
          unpack8(hp[j], v);
#pragma unroll
          for (int e = 0; e < 8; e++) ss += v[e] * v[e];
        }
      }
      if (norm_w) {
        const float rstd = rsqrtf(warp_sum(ss) / cols + eps);
#pragma unroll
        for (int j = 0; j < VPL; j++) {
          const int iv = lane + 32 * j;
          if (iv < n_vec) {
            const size_t off = base + (size_t)iv * 8;
            float v[8], w8[8];
            unpack8(hp[j], v);
            unpack8(*reinterpret_cast<const uint4*>(norm_w + (size_t)iv * 8), w8);
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = v[e] * rstd * w8[e];
            const uint4 packed = pack8(v);
            if (TWO) {
              const size_t boff = c.n_off + (size_t)parity * c.x_bytes + off * 2;
              if (MC) multimem_st16(c.mc + boff, packed);
              else
                for (int r = 0; r < c.n; r++) *reinterpret_cast<uint4*>(c.arena[r] + boff) = packed;
            } else {
              *reinterpret_cast<uint4*>(x_out + off) = packed;
            }
          }
        }
      }
    }
  }
  // ---- last CTA of the grid: (two-shot) tell everyone my rows are out and wait for theirs, then clear the flags ----
  if (TWO) __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = reinterpret_cast<int*>(c.arena[c.rank] + BAR_TICKET) + parity;
    __threadfence();
    const int last = atomicAdd(tk, 1) == (int)gridDim.x - 1;
    if (last) *tk = 0;
    last_s = last;
  }
  __syncthreads();
  if (!last_s) return;
  if (TWO) {
    // "rows broadcast" flags carry the number of the two-shot reduction on this parity (never reset): rank j's rows of
    // reduction e are complete once flag[j] >= e.  Every rank performs the same sequence, so the numbers agree.
    int* ep = reinterpret_cast<int*>(c.arena[c.rank] + RN_EPOCH) + parity;
    const int epoch = *reinterpret_cast<volatile int*>(ep) + 1;
    __threadfence_system();
    if (threadIdx.x < c.n) st_release_sys(bar_ptr(c.arena[threadIdx.x], BAR_OUT, parity, c.rank), epoch);
    // deferred: the consumer (a GEMM that waits for each owner's flag before it loads that owner's rows) does the
    // waiting, tile by tile, so its first tiles run while the last rows are still on their way
    if (!defer_wait) wait_ranks_ge(c, BAR_OUT, parity, epoch);
    __syncthreads();
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(ep) = epoch;
      __threadfence();
    }
  }
  if (threadIdx.x < c.n) {
    *bar_ptr(c.arena[c.rank], BAR_IN, parity, threadIdx.x) = 0;
    __threadfence_system();
  }
}

// All-gather of residual-stream rows that a two-shot reduction left sharded: this rank's rows [rank R, (rank + 1) R)
// of `src` go into hbuf[parity] of every rank; when the kernel completes every rank's rows have landed.
template <bool MC>
__global__ void __launch_bounds__(RN_THREADS)
gather_rows_kernel(const CommCtx c, const __nv_bfloat16* __restrict__ src, int rows, int cols, int parity) {
  pdl_trigger();
  pdl_wait();
  __shared__ int last_s;
  const int per = (rows + c.n - 1) / c.n;
  const int row0 = min(rows, c.rank * per), row1 = min(rows, row0 + per);
  const size_t v0 = (size_t)row0 * cols / 8, v1 = (size_t)row1 * cols / 8;
  const size_t hb = c.h_off + (size_t)parity * c.x_bytes;
  for (size_t v = v0 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < v1; v += (size_t)gridDim.x * blockDim.x) {
    const uint4 x = reinterpret_cast<const uint4*>(src)[v];
    if (MC) multimem_st16(c.mc + hb + v * 16, x);
    else
      for (int r = 0; r < c.n; r++) *reinterpret_cast<uint4*>(c.arena[r] + hb + v * 16) = x;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = reinterpret_cast<int*>(c.arena[c.rank] + BAR_TICKET) + 2;      // third ticket word: the gathers' own
    __threadfence();
    const int last = atomicAdd(tk, 1) == (int)gridDim.x - 1;
    if (last) *tk = 0;
    last_s = last;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence_system();
  if (threadIdx.x < c.n) red_release_sys_add(bar_ptr(c.arena[threadIdx.x], BAR_GATHER, 0, c.rank), 1);
  wait_ranks(c, BAR_GATHER, 0);
  if (threadIdx.x < c.n) {
    *bar_ptr(c.arena[c.rank], BAR_GATHER, 0, threadIdx.x) = 0;
    __threadfence_system();
  }
}

CommCtx g_ctx[16];
bool g_ctx_set[16] = {false};

}  // namespace

// ---- arena management (host) ------------------------------------------------------------------
EXO_API void* exo_symm_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, bytes);
  cudaDeviceSynchronize();
  return p;
}
EXO_API int exo_symm_free(void* p) { return (int)cudaFree(p); }
EXO_API int exo_symm_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
EXO_API void* exo_symm_open(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}
EXO_API int exo_symm_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
EXO_API size_t exo_comm_header_bytes() { return HDR_BYTES; }

// arenas: n pointers (index = rank; own arena at [rank]).
// `mc` = multicast address of the arena or null; x_off / x_bytes / h_off / n_off describe the regions of the
// reduce + norm kernels (x_bytes = 0: not present), ll_off / ll_slot those of the flag-in-data hand-over.
EXO_API int exo_comm_init(void** arenas, void* mc, int n, int rank, size_t slot_bytes, size_t gather_off, size_t x_off, size_t x_bytes, size_t h_off, size_t n_off, size_t ll_off,
                          size_t ll_slot) {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || n > MAX_RANKS || n < 1 || rank < 0 || rank >= n) return -1;
  int* status = exo_status_word(EXO_STATUS_COMM);
  if (!status) return -1;
  CommCtx c;
  for (int i = 0; i < MAX_RANKS; i++) c.arena[i] = i < n ? (uint8_t*)arenas[i] : nullptr;
  c.n = n; c.rank = rank; c.slot_bytes = slot_bytes; c.gather_off = gather_off;
  c.mc = (uint8_t*)mc; c.x_off = x_off; c.x_bytes = x_bytes; c.h_off = h_off; c.n_off = n_off;
  c.ll_off = ll_off; c.ll_slot = ll_slot;
  c.status = status;
  c.wait_ns = exo_wait_budget_ns();
  g_ctx[dev] = c;
  g_ctx_set[dev] = true;
  return 0;
}

// Forget the communicator of the current device (after its arenas have been unmapped).
EXO_API int exo_comm_reset() {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16) return -1;
  g_ctx_set[dev] = false;
  return 0;
}

EXO_API int exo_comm_status() {  // reads and clears the status word of the collectives; does not touch the device
  return exo_status_take(EXO_STATUS_COMM, 1);
}

static int grid_for(int n_vec) {
  int g = (n_vec + 255) / 256;
  if (g > 64) g = 64;  // few CTAs: every CTA costs n remote atomics and the tensors are small
  return g < 1 ? 1 : g;
}

// out = residual + all-reduce(in) over bf16 tensors of n_elems (multiple of 8) elements.
EXO_API int exo_allreduce_bf16(const void* in, const void* residual, void* out, long n_elems, int parity,
                               cudaStream_t st) {
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_ctx_set[dev]) return -4;
  CommCtx c = g_ctx[dev];
  c.wait_ns = exo_wait_budget_ns();
  if (n_elems % 8) return -2;
  const int n_vec = (int)(n_elems / 8);
  const size_t bytes = (size_t)n_elems * 2;
  cudaError_t e;
  if (bytes <= c.slot_bytes && bytes <= (512u << 10)) {
    e = launch_pdl(allreduce_oneshot_kernel, dim3(grid_for(n_vec)), dim3(256), 0, st, c, (const uint4*)in,
                   (const uint4*)residual, (uint4*)out, n_vec, parity);
  } else {
    const int per_rank = (n_vec + c.n - 1) / c.n;
    if ((size_t)per_rank * 16 > c.slot_bytes / 2) return -6;  // slot too small
    e = launch_pdl(allreduce_twoshot_kernel, dim3(148), dim3(256), 0, st, c, (const uint4*)in, (const uint4*)residual,
                   (uint4*)out, n_vec, parity);
  }
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// gather region of every rank ← [rows, n*cols] with this rank's [rows, cols] shard in place.
EXO_API int exo_allgather_cols_bf16(const void* in, int rows, int cols, int parity, cudaStream_t st) {
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_ctx_set[dev]) return -4;
  CommCtx c = g_ctx[dev];
  c.wait_ns = exo_wait_budget_ns();
  if (cols % 8) return -2;
  int total = rows * (cols / 8);
  cudaError_t e = launch_pdl(allgather_cols_kernel, dim3(grid_for(total)), dim3(256), 0, st, c, (const uint4*)in, rows,
                             cols / 8, parity);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}


// h = residual + sum over ranks of partial[parity];  x = RMSNorm(h) * norm_w  (norm_w null: h only).
// The partial must have been written into this rank's partial[parity] region (exo_comm_region(0, parity)) by
// earlier work of the same stream.
//   two_shot = 0: h_out / x_out are private [rows, cols] tensors of the caller; every rank computes every row.
//   two_shot = 1: x lands in exo_comm_region(2, parity) on every rank (x_out ignored).  mode bit 0 set: so does h, in
//                 exo_comm_region(1, parity) (h_out ignored); clear: only this rank's rows [rank R, (rank+1) R),
//                 R = ceil(rows / n), of the private h_out are written.  mode bit 1 set: the kernel does not wait for
//                 the other ranks' rows; the consumer must (exo_comm_gate + a gated GEMM).
// rows * cols * 2 must fit the region; cols % 8 == 0 and cols <= 8192.
EXO_API int exo_reduce_norm_bf16(const void* residual, const void* norm_w, float eps, void* h_out, void* x_out, int rows,
                                 int cols, int parity, int two_shot, int mode, cudaStream_t st) {
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_ctx_set[dev]) return -4;
  CommCtx c = g_ctx[dev];
  c.wait_ns = exo_wait_budget_ns();
  if (rows <= 0 || cols % 8 || cols > 8192) return -2;
  if (!c.x_bytes || (size_t)rows * cols * 2 > c.x_bytes) return -6;
  EXO_REQUIRE_ALIGNED16(residual); EXO_REQUIRE_ALIGNED16(norm_w); EXO_REQUIRE_ALIGNED16(h_out); EXO_REQUIRE_ALIGNED16(x_out);
  const int bcast_h = mode & 1;
  if ((!two_shot || !bcast_h) && !h_out) return -2;
  if (!two_shot) mode &= 1;
  if (!two_shot && norm_w && !x_out) return -2;
  const auto* res = (const __nv_bfloat16*)residual;
  const auto* nw = (const __nv_bfloat16*)norm_w;
  auto* ho = (__nv_bfloat16*)h_out;
  auto* xo = (__nv_bfloat16*)x_out;
  const int my_rows = two_shot ? (rows + c.n - 1) / c.n : rows;
  int grid = (my_rows + RN_WARPS - 1) / RN_WARPS;
  if (grid > 296) grid = 296;
  const bool wide = cols > 4096;      // vectors per lane: 16 up to 4096 columns, 32 up to 8192
  cudaError_t e;
#define RN_LAUNCH(MCV, TWOV)                                                                                                  \
  e = wide ? launch_pdl(reduce_norm_kernel<MCV, TWOV, 32>, dim3(grid), dim3(RN_THREADS), 0, st, c, res, nw, eps, ho, xo, rows, \
                        cols, parity, mode)                                                                                    \
           : launch_pdl(reduce_norm_kernel<MCV, TWOV, 16>, dim3(grid), dim3(RN_THREADS), 0, st, c, res, nw, eps, ho, xo, rows, \
                        cols, parity, mode)
  if (two_shot) {
    if (c.mc) { RN_LAUNCH(true, true); } else { RN_LAUNCH(false, true); }
  } else {
    if (c.mc) { RN_LAUNCH(true, false); } else { RN_LAUNCH(false, false); }
  }
#undef RN_LAUNCH
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// What a GEMM needs to consume the rows of a deferred-wait two-shot reduction as they arrive: rank j's rows
// [j R, (j+1) R), R = ceil(rows / n), are complete once flags[j] >= *epoch (the reduction kernel, which precedes the
// GEMM in the stream, has advanced the epoch word by then).  Returns 0, or <0 without a communicator.
int exo_comm_gate(int parity, int rows, const int** flags, const int** epoch, int* rows_per_flag, int* rank,
                  unsigned long long* wait_ns, int** status) {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || !g_ctx_set[dev]) return -4;
  const CommCtx& c = g_ctx[dev];
  *flags = reinterpret_cast<const int*>(c.arena[c.rank] + BAR_OUT) + (parity & 1) * MAX_RANKS;
  *epoch = reinterpret_cast<const int*>(c.arena[c.rank] + RN_EPOCH) + (parity & 1);
  *rows_per_flag = (rows + c.n - 1) / c.n;
  *rank = c.rank;
  *wait_ns = exo_wait_budget_ns();
  *status = c.status;
  return 0;
}

// Completes a residual stream that a two-shot reduction left sharded by rows: every rank's rows of `src`
// ([rows, cols], this rank's rows valid) are gathered into exo_comm_region(1, parity) of every rank.
EXO_API int exo_gather_rows_bf16(const void* src, int rows, int cols, int parity, cudaStream_t st) {
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_ctx_set[dev]) return -4;
  CommCtx c = g_ctx[dev];
  c.wait_ns = exo_wait_budget_ns();
  if (rows <= 0 || cols % 8) return -2;
  if (!c.x_bytes || (size_t)rows * cols * 2 > c.x_bytes) return -6;
  EXO_REQUIRE_ALIGNED16(src);
  const size_t vecs = (size_t)((rows + c.n - 1) / c.n) * cols / 8;
  int grid = (int)((vecs + RN_THREADS - 1) / RN_THREADS);
  if (grid > 148) grid = 148;
  if (grid < 1) grid = 1;
  cudaError_t e = c.mc ? launch_pdl(gather_rows_kernel<true>, dim3(grid), dim3(RN_THREADS), 0, st, c, (const __nv_bfloat16*)src, rows, cols, parity)
                       : launch_pdl(gather_rows_kernel<false>, dim3(grid), dim3(RN_THREADS), 0, st, c, (const __nv_bfloat16*)src, rows, cols, parity);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// Local address of a region of the reduce + norm kernels: which = 0 partial, 1 hbuf, 2 nbuf.
EXO_API void* exo_comm_region(int which, int parity) {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || !g_ctx_set[dev]) return nullptr;
  const CommCtx& c = g_ctx[dev];
  if (!c.x_bytes) return nullptr;
  const size_t off = which == 0 ? c.x_off : which == 1 ? c.h_off : c.n_off;
  return c.arena[c.rank] + off + (size_t)(parity & 1) * c.x_bytes;
}

// 1 when the communicator of the current device reduces through the NVLink multicast mapping.
EXO_API int exo_comm_has_multicast() {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || !g_ctx_set[dev]) return 0;
  return g_ctx[dev].mc ? 1 : 0;
}

// ---- hand-over (row-parallel projection -> consumer, no collective kernel) -----------------------
namespace {

// Stand-alone consumer of a flag-in-data hand-over (nobody took it in a projection's prologue):
// out = residual + sum_r slot[r].  The last CTA advances the parity's epoch.
__global__ void __launch_bounds__(256) ll_finish_kernel(const TpHandover h, __nv_bfloat16* out, int n_vec) {
  pdl_trigger();
  pdl_wait();
  const uint32_t seq = (uint32_t)(*reinterpret_cast<volatile const int*>(h.ll_epoch) + 1);
  bool ok = true;
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += gridDim.x * blockDim.x) {
    float acc[8];
    if (h.x_res) unpack8(reinterpret_cast<const uint4*>(h.x_res)[v], acc);
    else {
#pragma unroll
      for (int e = 0; e < 8; e++) acc[e] = 0.f;
    }
    if (ok && !tp_ll_gather8(h, (size_t)v * 4, seq, acc)) {
      ok = false;
      atomicExch(h.status, 4);
    }
    reinterpret_cast<uint4*>(out)[v] = pack8(acc);
  }
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(h.ll_ticket, 1) == (int)gridDim.x - 1) {
    *h.ll_ticket = 0;
    *reinterpret_cast<volatile int*>(h.ll_epoch) = (int)seq;
    __threadfence();
  }
}


// Consumer of a flag-in-data hand-over for decode batches (the producer is the GEMM's epilogue): one CTA per row
// forms h = residual + sum_r slot[r] (rank order, rounded to bf16), leaves it in h_out and writes RMSNorm(h) * w
// into x_out (norm_w null: h only).  The whole collective is ONE one-way trip of the producers' stores; nothing
// is signalled back.  The last CTA advances the parity's epoch.
template <int V>
__global__ void __launch_bounds__(256)
ll_reduce_norm_kernel(const TpHandover h, const __nv_bfloat16* __restrict__ norm_w, float eps, __nv_bfloat16* h_out,
                      __nv_bfloat16* x_out, int rows, int cols) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const uint32_t seq = (uint32_t)(*reinterpret_cast<volatile const int*>(h.ll_epoch) + 1);
  const int n_vec = cols / 8;
  bool ok = true;      // after the first wait that ran out, the rest of this thread's words are not polled again
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = (size_t)row * cols;
    float v[V][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V; j++) {
      const int iv = threadIdx.x + j * 256;
      if (iv < n_vec) {
        const size_t off = base + (size_t)iv * 8;
        if (h.x_res) unpack8(*reinterpret_cast<const uint4*>(h.x_res + off), v[j]);
        else {
#pragma unroll
          for (int e = 0; e < 8; e++) v[j][e] = 0.f;
        }
        if (ok && !tp_ll_gather8(h, off / 2, seq, v[j])) { ok = false; atomicExch(h.status, 4); }
        const uint4 packed = pack8(v[j]);
        *reinterpret_cast<uint4*>(h_out + off) = packed;
        unpack8(packed, v[j]);
#pragma unroll
        for (int e = 0; e < 8; e++) ss += v[j][e] * v[j][e];
      }
    }
    if (norm_w) {
      ss = warp_sum(ss);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; w++) tot += red[w];
      const float rstd = rsqrtf(tot / cols + eps);
#pragma unroll
      for (int j = 0; j < V; j++) {
        const int iv = threadIdx.x + j * 256;
        if (iv < n_vec) {
          float w8[8];
          unpack8(*reinterpret_cast<const uint4*>(norm_w + (size_t)iv * 8), w8);
#pragma unroll
          for (int e = 0; e < 8; e++) v[j][e] = v[j][e] * rstd * w8[e];
          *reinterpret_cast<uint4*>(x_out + base + (size_t)iv * 8) = pack8(v[j]);
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(h.ll_ticket, 1) == (int)gridDim.x - 1) {
    *h.ll_ticket = 0;
    *reinterpret_cast<volatile int*>(h.ll_epoch) = (int)seq;
    __threadfence();
  }
}


// Producer of a flag-in-data hand-over for a tensor that some other kernel computed (the combined expert outputs of
// a MoE layer): reads y [rows, cols] bf16 and sends it to every rank's slot as (two values, sequence number) words.
__global__ void __launch_bounds__(256) ll_push_kernel(const TpHandover h, const __nv_bfloat16* __restrict__ y, size_t n_words) {
  pdl_trigger();
  pdl_wait();
  const uint32_t seq = (uint32_t)(*reinterpret_cast<volatile const int*>(h.ll_epoch) + 1);
  const uint32_t* src = reinterpret_cast<const uint32_t*>(y);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x)
    tp_ll_store(h, i, src[i], seq);
}

}  // namespace

int exo_tp_handover_fill(TpHandover* out, int mode, int parity, long n_elems) {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || !g_ctx_set[dev]) return -4;
  const CommCtx& c = g_ctx[dev];
  memset(out, 0, sizeof(*out));
  uint8_t* mine = c.arena[c.rank];
  out->status = c.status;
  out->wait_ns = exo_wait_budget_ns();
  if (mode == 3 || mode == 4) {
    // two bf16 per 8-byte word: n_elems values take 4 * n_elems bytes of a slot
    if (!c.ll_slot || (size_t)n_elems * 4 > c.ll_slot || (n_elems & 1)) return -6;
    out->n_ll = c.n;
    out->ll_epoch = reinterpret_cast<int*>(mine + LL_EPOCH) + parity;
    const size_t my_slot = c.ll_off + ((size_t)parity * c.n + c.rank) * c.ll_slot;
    if (mode == 3) {
      out->ll_mc = c.mc ? reinterpret_cast<uint2*>(c.mc + my_slot) : nullptr;
      for (int r = 0; r < c.n; r++) out->ll_dst[r] = reinterpret_cast<uint2*>(c.arena[r] + my_slot);
    } else {
      for (int r = 0; r < c.n; r++)
        out->ll_part[r] = reinterpret_cast<const uint2*>(mine + c.ll_off + ((size_t)parity * c.n + r) * c.ll_slot);
      out->ll_ticket = reinterpret_cast<int*>(mine + LL_TICKET) + parity;
    }
    return 0;
  }
  return -2;
}



// Sends y [rows, cols] bf16 (rows * cols even) to every rank as the hand-over of `parity`; consumed like a
// projection's own hand-over (exo_tp_ll_reduce_norm / exo_tp_ll_finish / the streaming GEMV's prologue).
EXO_API int exo_tp_ll_push(const void* y, int rows, int cols, int parity, cudaStream_t st) {
  const long n = (long)rows * cols;
  if (n <= 0 || (n & 1)) return -2;
  TpHandover h;
  int rc = exo_tp_handover_fill(&h, 3, parity, n);
  if (rc) return rc;
  const size_t n_words = (size_t)n / 2;
  int grid = (int)((n_words + 255) / 256);
  if (grid > 148) grid = 148;
  cudaError_t e = launch_pdl(ll_push_kernel, dim3(grid), dim3(256), 0, st, h, (const __nv_bfloat16*)y, n_words);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// h_out = residual + sum over ranks of the flag-in-data hand-over on `parity`; x_out = RMSNorm(h_out) * norm_w
// (norm_w null: h_out only).  [rows, cols] bf16, cols % 8 == 0, cols <= 8192.
EXO_API int exo_tp_ll_reduce_norm(const void* residual, const void* norm_w, float eps, void* h_out, void* x_out, int rows,
                                  int cols, int parity, cudaStream_t st) {
  if (cols % 8 || cols > 8192 || rows <= 0 || !h_out || (norm_w && !x_out)) return -2;
  EXO_REQUIRE_ALIGNED16(residual); EXO_REQUIRE_ALIGNED16(norm_w); EXO_REQUIRE_ALIGNED16(h_out); EXO_REQUIRE_ALIGNED16(x_out);
  TpHandover h;
  int rc = exo_tp_handover_fill(&h, 4, parity, (long)((rows + 1) & ~1) * cols);
  if (rc) return rc;
  h.x_res = (const __nv_bfloat16*)residual;
  const int per_thread = (cols / 8 + 255) / 256;
  cudaError_t e;
  if (per_thread <= 2)
    e = launch_pdl(ll_reduce_norm_kernel<2>, dim3(rows), dim3(256), 0, st, h, (const __nv_bfloat16*)norm_w, eps,
                   (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out, rows, cols);
  else
    e = launch_pdl(ll_reduce_norm_kernel<4>, dim3(rows), dim3(256), 0, st, h, (const __nv_bfloat16*)norm_w, eps,
                   (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out, rows, cols);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// out = residual + sum over ranks of the flag-in-data hand-over on `parity` (n_elems multiple of 8).
EXO_API int exo_tp_ll_finish(const void* residual, void* out, long n_elems, int parity, cudaStream_t st) {
  if (n_elems % 8) return -2;
  EXO_REQUIRE_ALIGNED16(residual); EXO_REQUIRE_ALIGNED16(out);
  TpHandover h;
  int rc = exo_tp_handover_fill(&h, 4, parity, n_elems);
  if (rc) return rc;
  h.x_res = (const __nv_bfloat16*)residual;
  const int n_vec = (int)(n_elems / 8);
  int grid = (n_vec + 255) / 256;
  if (grid > 32) grid = 32;
  cudaError_t e = launch_pdl(ll_finish_kernel, dim3(grid), dim3(256), 0, st, h, (__nv_bfloat16*)out, n_vec);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}
