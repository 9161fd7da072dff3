// Shared by the tcgen05 GEMM kernels (bf16 weights, fp8 weights): problem description and the
// epilogue run by warps 2..5 — accumulator read-back, bias / residual, split-K reduction in split
// order by the last CTA of a tile, and the tensor-parallel hand-over of a row-parallel output.
#pragma once
#include "tc_common.cuh"
#include "tp_handover.cuh"

namespace gemm {

constexpr int BM = 128;  // output features per CTA (TMEM lanes)
constexpr int BK = 64;   // K elements per pipeline step (one 128-byte swizzle atom of bf16)

struct GemmParams {
  int M, N, K;            // x rows, W rows (output features), reduction length
  int kb_per_split;       // K blocks handled by one split
  int bn_rows;            // activation rows per CTA when fewer than the kernel's BN (0: BN); a multiple of 16
  int rows_fastest;       // 1: blockIdx.x walks the row tiles and blockIdx.y the feature tiles (prefill launches)
  int splits;
  const __nv_bfloat16* bias;       // [N] or null
  const __nv_bfloat16* residual;   // [M, ldo] or null (may alias out)
  __nv_bfloat16* out;              // [M, ldo]
  int ldo;
  float* partial;         // [splits, M, N] fp32 (split-K only)
  int* counters;          // [tiles] zero-initialised, self-resetting
  int* err;               // device error word
  TpHandover ho;          // row-parallel output handed to every rank (n_ll > 0): `out` is then not written
  // all-gather -> GEMM: the activation rows arrive from the other ranks while the kernel runs (null: plain GEMM)
  const int* row_flags;   // row_flags[j] >= *row_epoch once rows [j * rows_per_flag, (j + 1) * rows_per_flag) have landed
  const int* row_epoch;   // number of the reduction that produced these rows (device word, read when the kernel runs)
  int rows_per_flag;
  int m_tile_shift;       // row tiles are walked starting at this rank's own rows, which are there first
  unsigned long long gate_wait_ns;
  int* gate_status;       // status word of the collectives (a peer that never delivers: code 4)
};

// Called by the four epilogue warps (threads 64..191) once the MMA warp has committed `acc_full`.
// HO: the output goes to every rank's hand-over slot as flag-in-data words instead of `out` (a separate
// instantiation, so that the plain kernel's store loop carries none of it); N must be even.
template <int BN, bool HO = false>
__device__ __forceinline__ void epilogue(const GemmParams& p, uint32_t tmem, uint64_t* acc_full, int* abort_flag,
                                         int* is_last_s, int n0, int m0, int split, int nkb, int warp, int lane, int bn = BN) {
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int n = n0 + quad * 32 + lane;       // output feature owned by this thread
    uint32_t ll_seq = 0;                       // sequence number of this hand-over's words (see tp_handover.cuh)
    if constexpr (HO) ll_seq = (uint32_t)(*reinterpret_cast<volatile const int*>(p.ho.ll_epoch) + 1);
    bool ok = tc::mbar_wait_backoff(acc_full, 0, 400);
    if (!ok) { atomicExch(p.err, tc::ERR_ACC_TIMEOUT); *abort_flag = 1; }
    tc::tc_fence_after();
    ok = ok && !*(volatile int*)abort_flag && nkb > 0;
    const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
    if (p.splits == 1) {
      float bias = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll 1
      for (int c = 0; c < bn; c += 16) {
        float v[16];
        tc::tmem_ld16(taddr + c, v);   // warp-collective: executed by all lanes regardless of bounds
        tc::tmem_ld_wait();
        if constexpr (HO) {
          // Hand-over: adjacent lanes own adjacent features.  Lanes pair up, the even lane keeps the even rows and
          // the odd lane the odd rows of the pair's two features, and each word (two bf16 + sequence number)
          // leaves for every rank as one 8-byte store.  Warp-collective: no lane may skip the shuffles.
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float mine0 = v[j] + bias, mine1 = v[j + 1] + bias;
            const float other = __shfl_xor_sync(0xffffffffu, (lane & 1) ? mine0 : mine1, 1);
            const int m = m0 + c + j + (lane & 1);
            const int ne = n & ~1;
            if (ok && m < p.M && ne < p.N) {
              const __nv_bfloat162 pk = (lane & 1) ? __floats2bfloat162_rn(other, mine1) : __floats2bfloat162_rn(mine0, other);
              tp_ll_store(p.ho, ((size_t)m * p.ldo + ne) / 2, *reinterpret_cast<const uint32_t*>(&pk), ll_seq);
            }
          }
        } else if (ok && n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; j++) {
            int m = m0 + c + j;
            if (m < p.M) {
              float y = v[j] + bias;
              size_t o = (size_t)m * p.ldo + n;
              if (p.residual) y += __bfloat162float(p.residual[o]);
              p.out[o] = __float2bfloat16_rn(y);
            }
          }
        }
      }
    } else {
      // split-K: publish the fp32 partial tile
      float* part = p.partial + (size_t)split * p.M * p.N;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        tc::tmem_ld16(taddr + c, v);
        tc::tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; j++) {
            int m = m0 + c + j;
            if (m < p.M) part[(size_t)m * p.N + n] = ok ? v[j] : 0.f;
          }
        }
      }
      __threadfence();
      // named barrier over the 4 epilogue warps (128 threads), then one thread takes a ticket
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        int tile = blockIdx.y * gridDim.x + blockIdx.x;
        int ticket = atomicAdd(&p.counters[tile], 1);
        *is_last_s = (ticket == p.splits - 1);
        if (*is_last_s) p.counters[tile] = 0;  // self-reset for the next launch / graph replay
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*is_last_s) {
        // The last split of this tile to arrive sums the partial planes.  All 128 epilogue threads take
        // part: a thread owns four consecutive features and every fourth row, and keeps eight 16-byte
        // loads in flight per row (the planes are a split apart in memory), so the reduce costs a few
        // L2 round trips instead of one per (split, row).  Splits are added in index order: the sum
        // does not depend on which CTA came last.
        __threadfence();
        const int et = threadIdx.x - 64;          // 0..127 among the epilogue warps
        const int nq = n0 + (et & 31) * 4;
        const int mcount = min(BN, p.M - m0);
        const size_t plane = (size_t)p.M * p.N;
        const bool vec = (p.N & 3) == 0 && nq + 3 < p.N;
        for (int mm = et >> 5; mm < mcount; mm += 8) {      // two rows per pass: up to 16 loads in flight per thread
          const bool two = mm + 4 < mcount;
          const float* base0 = p.partial + (size_t)(m0 + mm) * p.N + nq;
          const float* base1 = base0 + (size_t)4 * p.N;
          float y[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
          if (vec) {
            int sp = 0;
            for (; sp + 8 <= p.splits; sp += 8) {
              float4 v[2][8];
#pragma unroll
              for (int u = 0; u < 8; u++) {
                v[0][u] = __ldcg(reinterpret_cast<const float4*>(base0 + (size_t)(sp + u) * plane));
                v[1][u] = two ? __ldcg(reinterpret_cast<const float4*>(base1 + (size_t)(sp + u) * plane)) : make_float4(0, 0, 0, 0);
              }
#pragma unroll
              for (int r = 0; r < 2; r++)
#pragma unroll
                for (int u = 0; u < 8; u++) { y[r][0] += v[r][u].x; y[r][1] += v[r][u].y; y[r][2] += v[r][u].z; y[r][3] += v[r][u].w; }
            }
            float4 t[2][7];
            const int rem = p.splits - sp;
#pragma unroll
            for (int u = 0; u < 7; u++) {
              t[0][u] = u < rem ? __ldcg(reinterpret_cast<const float4*>(base0 + (size_t)(sp + u) * plane)) : make_float4(0, 0, 0, 0);
              t[1][u] = (two && u < rem) ? __ldcg(reinterpret_cast<const float4*>(base1 + (size_t)(sp + u) * plane)) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
              for (int u = 0; u < 7; u++) { y[r][0] += t[r][u].x; y[r][1] += t[r][u].y; y[r][2] += t[r][u].z; y[r][3] += t[r][u].w; }
          } else {
            for (int sp = 0; sp < p.splits; sp++)
#pragma unroll
              for (int j = 0; j < 4; j++)
                if (nq + j < p.N) {
                  y[0][j] += __ldcg(base0 + (size_t)sp * plane + j);
                  if (two) y[1][j] += __ldcg(base1 + (size_t)sp * plane + j);
                }
          }
#pragma unroll
          for (int r = 0; r < 2; r++) {
            if (r == 1 && !two) break;
            if constexpr (HO) {
              // a thread holds four consecutive features of one row: two words (N is even under a hand-over)
#pragma unroll
              for (int j = 0; j < 4; j += 2) {
                if (nq + j < p.N) {
                  const float a = y[r][j] + (p.bias ? __bfloat162float(p.bias[nq + j]) : 0.f);
                  const float b2 = y[r][j + 1] + (p.bias ? __bfloat162float(p.bias[nq + j + 1]) : 0.f);
                  const __nv_bfloat162 pk = __floats2bfloat162_rn(a, b2);
                  tp_ll_store(p.ho, ((size_t)(m0 + mm + 4 * r) * p.ldo + nq + j) / 2, *reinterpret_cast<const uint32_t*>(&pk), ll_seq);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                if (nq + j < p.N) {
                  size_t o = (size_t)(m0 + mm + 4 * r) * p.ldo + nq + j;
                  float v = y[r][j] + (p.bias ? __bfloat162float(p.bias[nq + j]) : 0.f);
                  if (p.residual) v += __bfloat162float(p.residual[o]);
                  p.out[o] = __float2bfloat16_rn(v);
                }
              }
            }
          }
        }
      }
    }
}

// Gate/up pair: accumulator 0 holds the gate rows [n0, n0+128), accumulator 1 (BN columns further on) the up rows of
// the same features; writes silu(gate) * up to out[M, F] (ldo = F).  Each projection is rounded to bf16 before
// the activation, as the unfused form (GEMM, then the SwiGLU kernel) does.
template <int BN>
__device__ __forceinline__ void epilogue_swiglu(const GemmParams& p, uint32_t tmem, uint64_t* acc_full, int* abort_flag, int n0,
                                                int m0, int nkb, int warp, int lane, int bn = BN) {
  const int quad = warp & 3;
  const int n = n0 + quad * 32 + lane, F = p.N / 2;
  bool ok = tc::mbar_wait_backoff(acc_full, 0, 400);
  if (!ok) { atomicExch(p.err, tc::ERR_ACC_TIMEOUT); *abort_flag = 1; }
  tc::tc_fence_after();
  ok = ok && !*(volatile int*)abort_flag && nkb > 0;
  const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
  for (int c = 0; c < bn; c += 16) {
    float g[16], u[16];
    tc::tmem_ld16(taddr + c, g);
    tc::tmem_ld16(taddr + BN + c, u);
    tc::tmem_ld_wait();
    if (ok && n < F) {
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int m = m0 + c + j;
        if (m < p.M) {
          const float gb = __bfloat162float(__float2bfloat16_rn(g[j])), ub = __bfloat162float(__float2bfloat16_rn(u[j]));
          p.out[(size_t)m * p.ldo + n] = __float2bfloat16_rn(silu_f(gb) * ub);
        }
      }
    }
  }
}

}  // namespace gemm
