// Batch-1/2 linear layer as a persistent, bulk-async-copy pipelined weight stream.
//
//   y[m, n] = sum_k f(x)[m, k] * W[n, k]          (bf16 in, fp32 accumulate, M = 1 or 2)
//
// Decode at batch 1 reads every weight byte once and does two flops with it: the only thing that
// matters is keeping HBM busy.  One CTA per SM stays resident for the whole call.  A producer warp
// walks the CTA's row groups and keeps a ring of STAGES shared-memory buffers full with
// `cp.async.bulk` copies (a group of RS consecutive weight rows is one contiguous run of bytes), so
// ~150 KB per SM are always in flight no matter what the eight consumer warps are doing, and — the
// weights being constants — it starts BEFORE the programmatic-dependent-launch wait, i.e. while the
// previous kernel of the decode step is still draining.  Each consumer warp owns one eighth of the
// K range, holds its slice of the (normalised) activation in registers for the whole kernel, and
// dots it with every row of every stage; per-row partials meet in shared memory.
//
// Fused: RMSNorm prologue (sum of squares + norm weight), bias, residual add, SwiGLU epilogue
// (a stage then carries RS/2 gate rows and the matching RS/2 up rows as two copies).
#include <cstdlib>
#include <cstring>
#include "status.h"
#include "tc_common.cuh"
#include "tp_handover.cuh"

namespace {

#ifndef EXO_GEMV_WARPS
#define EXO_GEMV_WARPS 8
#endif
constexpr int CONSUMER_WARPS = EXO_GEMV_WARPS;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int RS_MAX = 32;

struct StreamParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* W;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  const __nv_bfloat16* norm_w;
  float eps;
  int N, K, RS, n_groups, ldo, stages, stage_bytes;
  int* err;
  TpHandover ho;   // tensor-parallel hand-over (all zero when the projection is not part of one)
};

__device__ __forceinline__ void bulk_g2s(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(tc::smem_u32(smem)), "l"(gmem), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

// HO: 0 = plain projection, 1 = its output is handed over to every rank (flag-in-data words, see tp_handover.cuh),
// 2 = its input is such a hand-over
template <int M, int JV, int RB, bool NORM, bool SWIGLU, int HO>
__global__ void __launch_bounds__(THREADS, 1) gemv_stream_kernel(const StreamParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  uint64_t* full = reinterpret_cast<uint64_t*>(base);
  uint64_t* empty = full + 8;
  float* part = reinterpret_cast<float*>(base + 128);                     // [2][RS_MAX][CONSUMER_WARPS][M]
  float* red = part + 2 * RS_MAX * CONSUMER_WARPS * M;                    // [CONSUMER_WARPS][M]
  uint8_t* ring = base + 128 + ((2 * RS_MAX * CONSUMER_WARPS * M + CONSUMER_WARPS * M) * 4 + 127) / 128 * 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K, RS = p.RS, F = p.N / 2;
  const int row_bytes = K * 2;
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; i++) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], CONSUMER_WARPS); }
    tc::fence_barrier_init();
  }
  __syncthreads();
  const int my_groups = (p.n_groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (warp == CONSUMER_WARPS) {
    // ------------------------------ producer ------------------------------
    if (tc::elect_one()) {
      for (int i = 0; i < my_groups; i++) {
        const int st = i % p.stages, g = blockIdx.x + i * gridDim.x;
        if (i >= p.stages && !tc::mbar_wait(&empty[st], ((i / p.stages) - 1) & 1)) {
          atomicExch(p.err, tc::ERR_EMPTY_TIMEOUT);
          break;
        }
        uint8_t* dst = ring + (size_t)st * p.stage_bytes;
        if (SWIGLU) {
          const int half = RS / 2, r0 = g * half, rows = min(half, F - r0);
          const uint32_t bytes = (uint32_t)rows * row_bytes;
          tc::mbar_expect_tx(&full[st], 2 * bytes);
          bulk_g2s(dst, p.W + (size_t)r0 * K, bytes, &full[st]);
          bulk_g2s(dst + (size_t)half * row_bytes, p.W + (size_t)(F + r0) * K, bytes, &full[st]);
        } else {
          const int r0 = g * RS, rows = min(RS, p.N - r0);
          const uint32_t bytes = (uint32_t)rows * row_bytes;
          tc::mbar_expect_tx(&full[st], bytes);
          bulk_g2s(dst, p.W + (size_t)r0 * K, bytes, &full[st]);
        }
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  const int KS = K / CONSUMER_WARPS;          // this warp's K slice
  const int k_lo = warp * KS, nvec = KS / 8;  // in 16-byte vectors
  pdl_wait();                                 // x comes from the previous kernel
  uint32_t ll_seq = 0;
  bool ll_ok = true;
  if constexpr (HO != 0) ll_seq = (uint32_t)(*reinterpret_cast<volatile const int*>(p.ho.ll_epoch) + 1);
  float xr[M][JV][8];
  float ss[M];
#pragma unroll
  for (int m = 0; m < M; m++) {
    ss[m] = 0.f;
#pragma unroll
    for (int j = 0; j < JV; j++) {
      const int v = lane + 32 * j;
      if (v < nvec) {
        if constexpr (HO == 2) {
          // x is handed over by the row-parallel projection of every rank: residual + partials in rank order,
          // rounded to bf16 (the same bits on every rank, and the value a separate all-reduce would have left in
          // memory).  Each lane polls exactly the words it needs until they carry this hand-over's sequence number.
          const size_t off = (size_t)m * K + k_lo + v * 8;
          float acc[8];
          if (p.ho.x_res) unpack8(*reinterpret_cast<const uint4*>(p.ho.x_res + off), acc);
          else {
#pragma unroll
            for (int e = 0; e < 8; e++) acc[e] = 0.f;
          }
          if (ll_ok && !tp_ll_gather8(p.ho, off / 2, ll_seq, acc)) {
            ll_ok = false;
            atomicExch(p.ho.status, 4 /* peer timeout */);
          }
          const uint4 packed = pack8(acc);
          if (blockIdx.x == 0 && p.ho.x_out) *reinterpret_cast<uint4*>(p.ho.x_out + off) = packed;
          unpack8(packed, xr[m][j]);
        } else {
          unpack8(*reinterpret_cast<const uint4*>(p.x + (size_t)m * K + k_lo + v * 8), xr[m][j]);
        }
        if (NORM) {
          float nw[8];
          unpack8(*reinterpret_cast<const uint4*>(p.norm_w + k_lo + v * 8), nw);
#pragma unroll
          for (int e = 0; e < 8; e++) { ss[m] += xr[m][j][e] * xr[m][j][e]; xr[m][j][e] *= nw[e]; }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; e++) xr[m][j][e] = 0.f;
      }
    }
  }
  float rstd[M];
#pragma unroll
  for (int m = 0; m < M; m++) rstd[m] = 1.f;
  if (NORM) {
#pragma unroll
    for (int m = 0; m < M; m++) {
      float v = warp_sum(ss[m]);
      if (lane == 0) red[warp * M + m] = v;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
#pragma unroll
    for (int m = 0; m < M; m++) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < CONSUMER_WARPS; w++) t += red[w * M + m];
      rstd[m] = rsqrtf(t / K + p.eps);
    }
  }

  bool ok = true;
  for (int i = 0; i < my_groups; i++) {
    const int st = i % p.stages, g = blockIdx.x + i * gridDim.x;
    if (ok && !tc::mbar_wait(&full[st], (i / p.stages) & 1)) {
      atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
      ok = false;
    }
    const uint8_t* src = ring + (size_t)st * p.stage_bytes + (size_t)k_lo * 2;
    float* pb = part + (size_t)(i & 1) * RS_MAX * CONSUMER_WARPS * M;
    // RB rows at a time: RB independent load / FMA / shuffle chains per lane hide each other's latency
    for (int rb = 0; rb < RS; rb += RB) {
      float acc[RB][M][2];
#pragma unroll
      for (int rr = 0; rr < RB; rr++)
#pragma unroll
        for (int m = 0; m < M; m++) { acc[rr][m][0] = 0.f; acc[rr][m][1] = 0.f; }
#pragma unroll
      for (int j = 0; j < JV; j++) {
        const int v = lane + 32 * j;
        if (v < nvec) {
          uint4 wv[RB];
#pragma unroll
          for (int rr = 0; rr < RB; rr++)
            wv[rr] = *reinterpret_cast<const uint4*>(src + (size_t)(rb + rr) * row_bytes + v * 16);
#pragma unroll
          for (int rr = 0; rr < RB; rr++) {
            float wf[8];
            unpack8(wv[rr], wf);
#pragma unroll
            for (int m = 0; m < M; m++)
#pragma unroll
              for (int e = 0; e < 8; e++) acc[rr][m][e & 1] += wf[e] * xr[m][j][e];
          }
        }
      }
      float tot[RB][M];
#pragma unroll
      for (int rr = 0; rr < RB; rr++)
#pragma unroll
        for (int m = 0; m < M; m++) tot[rr][m] = acc[rr][m][0] + acc[rr][m][1];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int rr = 0; rr < RB; rr++)
#pragma unroll
          for (int m = 0; m < M; m++) tot[rr][m] += __shfl_xor_sync(0xffffffffu, tot[rr][m], o);
      if (lane == 0) {
#pragma unroll
        for (int rr = 0; rr < RB; rr++)
#pragma unroll
          for (int m = 0; m < M; m++) pb[((rb + rr) * CONSUMER_WARPS + warp) * M + m] = tot[rr][m];
      }
    }
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&empty[st]);  // this warp is done reading the stage
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
    // finalise: thread t handles (row slot, m)
    const int t = threadIdx.x;
    if (ok) {
      if (SWIGLU) {
        const int half = RS / 2;
        if (t < half * M) {
          const int r = t / M, m = t % M, n = g * half + r;
          if (n < F) {
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; w++) {
              gsum += pb[(r * CONSUMER_WARPS + w) * M + m];
              usum += pb[((r + half) * CONSUMER_WARPS + w) * M + m];
            }
            gsum *= rstd[m];
            usum *= rstd[m];
            if (p.bias) { gsum += __bfloat162float(p.bias[n]); usum += __bfloat162float(p.bias[F + n]); }
            p.out[(size_t)m * p.ldo + n] = __float2bfloat16_rn(silu_f(gsum) * usum);   // column-parallel: never handed over
          }
        }
      } else if (HO == 1) {
        // row-parallel projection under tensor parallelism: two adjacent outputs + the sequence number leave for
        // every rank's slot as one 8-byte store, straight from the registers that hold them
        if (t < (RS / 2) * M) {
          const int pr = t / M, m = t % M, n = g * RS + 2 * pr;
          if (n < p.N) {
            float y0 = 0.f, y1 = 0.f;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; w++) {
              y0 += pb[((2 * pr) * CONSUMER_WARPS + w) * M + m];
              y1 += pb[((2 * pr + 1) * CONSUMER_WARPS + w) * M + m];
            }
            y0 *= rstd[m];
            y1 *= rstd[m];
            if (p.bias) { y0 += __bfloat162float(p.bias[n]); y1 += __bfloat162float(p.bias[n + 1]); }
            const __nv_bfloat162 pk = __floats2bfloat162_rn(y0, y1);
            tp_ll_store(p.ho, ((size_t)m * p.ldo + n) / 2, *reinterpret_cast<const uint32_t*>(&pk), ll_seq);
          }
        }
      } else if (t < RS * M) {
        const int r = t / M, m = t % M, n = g * RS + r;
        if (n < p.N) {
          float y = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMER_WARPS; w++) y += pb[(r * CONSUMER_WARPS + w) * M + m];
          y *= rstd[m];
          if (p.bias) y += __bfloat162float(p.bias[n]);
          if (p.residual) y += __bfloat162float(p.residual[(size_t)m * p.ldo + n]);
          p.out[(size_t)m * p.ldo + n] = __float2bfloat16_rn(y);
        }
      }
    }
  }
  if constexpr (HO == 2) {
    // every CTA has read the slots once it is here: the last one advances the parity's epoch, which is what the
    // next hand-over on this parity (two hand-overs from now) will stamp its words with
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
    if (threadIdx.x == 0 && atomicAdd(p.ho.ll_ticket, 1) == (int)gridDim.x - 1) {
      *p.ho.ll_ticket = 0;
      *reinterpret_cast<volatile int*>(p.ho.ll_epoch) = (int)ll_seq;
      __threadfence();
    }
  }
}

int* g_err_stream[16] = {nullptr};

template <int M, int JV, int RB>
int launch_stream_rb(const StreamParams& p, bool norm, bool swiglu, int grid, size_t smem, cudaStream_t st) {
  cudaError_t e;
#define L(NORM, SW, HO)                                                                                          \
  {                                                                                                              \
    static bool attr = false;                                                                                    \
    if (!attr) {                                                                                                 \
      if (cudaFuncSetAttribute(gemv_stream_kernel<M, JV, RB, NORM, SW, HO>,                                      \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)          \
        return -3;                                                                                               \
      attr = true;                                                                                               \
    }                                                                                                            \
    e = launch_pdl(gemv_stream_kernel<M, JV, RB, NORM, SW, HO>, dim3(grid), dim3(THREADS), smem, st, p);          \
  }
  // The hand-over roles are separate instantiations: a row-parallel projection that pushes its output has
  // neither norm nor SwiGLU, and a projection that consumes a hand-over always normalises it first.
  if (p.ho.n_ll > 0 && p.ho.ll_epoch && !p.ho.ll_ticket) {
    if (norm || swiglu) return -2;
    L(false, false, 1)
  } else if (p.ho.n_ll > 0) {
    if (!norm) return -2;
    if (swiglu) L(true, true, 2) else L(true, false, 2)
  } else if (norm) { if (swiglu) L(true, true, 0) else L(true, false, 0) }
  else { if (swiglu) L(false, true, 0) else L(false, false, 0) }
#undef L
  return (int)e;
}

// long rows (JV >= 4) come one or two per stage; short rows in blocks of four
template <int M, int JV>
int launch_stream(const StreamParams& p, bool norm, bool swiglu, int grid, size_t smem, cudaStream_t st) {
  if constexpr (JV >= 4) {
    if (p.RS % 2 == 0) return launch_stream_rb<M, JV, 2>(p, norm, swiglu, grid, smem, st);
    return launch_stream_rb<M, JV, 1>(p, norm, swiglu, grid, smem, st);
  } else {
    if (p.RS % 4 == 0) return launch_stream_rb<M, JV, 4>(p, norm, swiglu, grid, smem, st);
    if (p.RS % 2 == 0) return launch_stream_rb<M, JV, 2>(p, norm, swiglu, grid, smem, st);
    return launch_stream_rb<M, JV, 1>(p, norm, swiglu, grid, smem, st);
  }
}

}  // namespace

EXO_API int exo_gemv_stream_init() {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16) return -1;
  if (!g_err_stream[dev]) g_err_stream[dev] = exo_status_word(EXO_STATUS_GEMV);    // host-mapped: read without a copy
  return g_err_stream[dev] ? 0 : -1;
}

// Reads and clears the streaming kernels' status word (no device access; call once the kernels have completed).
EXO_API int exo_gemv_stream_last_error() { return exo_status_take(EXO_STATUS_GEMV, 1); }

// CTAs co-resident per SM (EXO_GEMV_CTAS_PER_SM, 1 or 2).  With 2, each CTA's ring is half as deep
// and the grid twice as wide: the same bytes are in flight per SM, and a CTA of the NEXT kernel in
// the stream can become resident (programmatic dependent launch) and start its weight stream while
// this kernel's last CTAs drain.
static int ctas_per_sm() {
  static int v = 0;
  if (!v) {
    const char* e = getenv("EXO_GEMV_CTAS_PER_SM");
    v = (e && e[0] == '2') ? 2 : 1;
  }
  return v;
}

// Stage geometry for a (M, K, swiglu) problem; false when the ring would not hold two stages.
static bool stream_config(int M, int K, int swiglu, int* RS_out, int* stages_out, size_t* fixed_out) {
  const int row_bytes = K * 2;
  int RS = (32 * 1024) / row_bytes;  // ~32 KB stages
  if (RS < 1) RS = 1;
  if (RS > RS_MAX) RS = RS_MAX;
  if (RS >= 4) RS &= ~3;  // whole row blocks
  if (swiglu) { RS &= ~1; if (RS < 2) RS = 2; }
  const size_t fixed = 128 + ((2 * RS_MAX * CONSUMER_WARPS * M + CONSUMER_WARPS * M) * 4 + 127) / 128 * 128 + 128;
  // The whole shared memory of the SM is the ring: ~190 KB in flight per SM is what it takes to
  // cover HBM latency at full bandwidth (a 104 KB ring, tried so that the next kernel's CTA could
  // co-reside and prefetch, lost 25 % of the bandwidth).
  static const size_t big = getenv("EXO_GEMV_RING_KB") ? (size_t)atoi(getenv("EXO_GEMV_RING_KB")) * 1024 : (size_t)196 * 1024;   // A/B switch, read once (227 KB measured 1-3 % slower)
  size_t budget = ctas_per_sm() == 2 ? 104 * 1024 : big;
  if (ctas_per_sm() == 2 && (size_t)RS * row_bytes > 16 * 1024) {   // smaller stages so that the ring still has depth
    RS = (16 * 1024) / row_bytes;
    if (RS < 1) RS = 1;
    if (RS >= 4) RS &= ~3;
    if (swiglu) { RS &= ~1; if (RS < 2) RS = 2; }
  }
  int stages = (int)((budget - fixed) / ((size_t)RS * row_bytes));
  if (stages > 8) stages = 8;
  *RS_out = RS; *stages_out = stages; *fixed_out = fixed;
  return stages >= 2;
}

// Returns 1 when (M, N, K) is served by the streaming kernel.
EXO_API int exo_gemv_stream_supported(int M, int N, int K, int swiglu) {
  if (M < 1 || M > 2) return 0;
  if (K % (8 * CONSUMER_WARPS) != 0 || K < 256) return 0;
  int jv = (K / 8 / CONSUMER_WARPS + 31) / 32;
  if (jv > 16 || (M == 2 && jv > 8)) return 0;
  if (swiglu && (N % 2)) return 0;
  if ((long)N * K < (1 << 20)) return 0;  // tiny matrices: the plain kernel has less set-up
  int RS, stages; size_t fixed;
  return stream_config(M, K, swiglu, &RS, &stages, &fixed) ? 1 : 0;
}

static int gemv_stream_launch(const void* x, const void* W, const void* bias, const void* residual, void* out,
                              const void* norm_w, float eps, int M, int N, int K, int swiglu, const TpHandover* ho,
                              cudaStream_t st);

EXO_API int exo_gemv_stream(const void* x, const void* W, const void* bias, const void* residual, void* out,
                            const void* norm_w, float eps, int M, int N, int K, int swiglu, cudaStream_t st) {
  return gemv_stream_launch(x, W, bias, residual, out, norm_w, eps, M, N, K, swiglu, nullptr, st);
}

// Row-parallel projection whose output is handed to every rank (mode 1: `out` is not written; N must be even), or a
// projection whose input is the hand-over of the previous one (mode 2: x = x_res + partials, and
// the reduced residual stream is left in x_out).  `parity` alternates per hand-over.
EXO_API int exo_gemv_stream_tp(const void* x, const void* W, const void* bias, void* out, const void* norm_w, float eps,
                               int M, int N, int K, int swiglu, int mode, int parity, const void* x_res, void* x_out,
                               cudaStream_t st) {
  TpHandover ho;
  int rc = exo_tp_handover_fill(&ho, mode == 1 ? 3 : 4, parity, mode == 1 ? (long)M * N : (long)M * K);
  if (rc) return rc;
  if (mode == 2) {
    ho.x_res = (const __nv_bfloat16*)x_res;
    ho.x_out = (__nv_bfloat16*)x_out;
  }
  return gemv_stream_launch(x, W, bias, nullptr, out, norm_w, eps, M, N, K, swiglu, &ho, st);
}

static int gemv_stream_launch(const void* x, const void* W, const void* bias, const void* residual, void* out,
                              const void* norm_w, float eps, int M, int N, int K, int swiglu, const TpHandover* ho,
                              cudaStream_t st) {
  if (!exo_gemv_stream_supported(M, N, K, swiglu)) return -2;
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_err_stream[dev]) return -4;
  StreamParams p;
  p.x = (const __nv_bfloat16*)x; p.W = (const __nv_bfloat16*)W; p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual; p.out = (__nv_bfloat16*)out; p.norm_w = (const __nv_bfloat16*)norm_w;
  p.eps = eps; p.N = N; p.K = K; p.ldo = swiglu ? N / 2 : N; p.err = g_err_stream[dev];
  if (ho) p.ho = *ho; else memset(&p.ho, 0, sizeof(p.ho));
  const int row_bytes = K * 2;
  int RS, stages; size_t fixed;
  const bool push = ho && ho->n_ll > 0 && !ho->ll_ticket;       // outputs leave in pairs: an even number of rows per stage
  if (push && (N & 1)) return -2;
  if (!stream_config(M, K, swiglu || push, &RS, &stages, &fixed)) return -2;
  const int rows_total = swiglu ? N / 2 : N;
  const int rows_per_group = swiglu ? RS / 2 : RS;
  p.RS = RS;
  p.n_groups = (rows_total + rows_per_group - 1) / rows_per_group;
  p.stage_bytes = RS * row_bytes;
  const int max_grid = 148 * ctas_per_sm();
  int grid = p.n_groups < max_grid ? p.n_groups : max_grid;
  // A CTA that has only one or two row groups to stream (a tensor-parallel shard, a small projection) needs no deeper
  // ring than that: the shared memory it leaves free lets the next kernel's CTAs become resident while this one still
  // runs, and their weight stream starts before the programmatic-dependent-launch wait.
  const int per_cta = (p.n_groups + grid - 1) / grid;
  static const bool full_ring = getenv("EXO_GEMV_FULL_RING") != nullptr;   // A/B switch, read once
  if (!full_ring && stages > per_cta) stages = per_cta < 2 ? 2 : per_cta;
  p.stages = stages;
  const size_t smem = fixed + (size_t)stages * p.stage_bytes;
  const int jv = (K / 8 / CONSUMER_WARPS + 31) / 32;
  int rc;
#define BY_JV(MM)                                                                              \
  if (jv <= 1) rc = launch_stream<MM, 1>(p, norm_w != nullptr, swiglu != 0, grid, smem, st);      \
  else if (jv <= 2) rc = launch_stream<MM, 2>(p, norm_w != nullptr, swiglu != 0, grid, smem, st); \
  else if (jv <= 4) rc = launch_stream<MM, 4>(p, norm_w != nullptr, swiglu != 0, grid, smem, st); \
  else if (jv <= 8) rc = launch_stream<MM, 8>(p, norm_w != nullptr, swiglu != 0, grid, smem, st); \
  else rc = launch_stream<1, 16>(p, norm_w != nullptr, swiglu != 0, grid, smem, st)
  if (M == 1) { BY_JV(1); } else { BY_JV(2); }
#undef BY_JV
  if (rc) return rc;
  EXO_CHECK_LAUNCH();
  return 0;
}
