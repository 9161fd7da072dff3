// Decode attention (one query token per sequence) with the KV stream feeding the tensor cores
// directly: split-KV flash decoding for grouped-query attention, head_dim 128, 16-key pages, bf16.
//
// One CTA = (sequence, KV head, split).  The sequence's keys are walked in blocks of 128, each
// block gathered page by page by TMA into 128-byte-swizzled shared memory through a 3-stage ring
// (up to 192 KB of K/V in flight per SM, which is what keeps HBM busy at small batch).  The
// tiles are consumed where they land, by tcgen05.mma, in "swapped" form so that the 128 keys (or
// the 128 head dims) fill the MMA's M and the few query heads of the group are the N:
//   S^T[key, head] = K[key, :] . Q[head, :]      A = K tile (K-major),  B = Q (16 rows: G heads + padding)
//   O^T[dim, head] += V[:, dim]^T . P[head, :]   A = V tile (MN-major), B = P (16 x 128, written by the threads)
// Thread t owns TMEM lane t: key t of the block for the softmax, head dim t for the output.  Only
// the block maximum needs a cross-thread reduction per block; row sums are kept per thread and
// reduced once.  Splits write (O, m, l) partials; the last CTA of a (sequence, KV head) to finish
// merges them (ticket counter, reset by that CTA so the buffer is reusable without a memset).
// Every wait is bounded: on a timeout the kernel records a code, drains and returns.
#include <cstdlib>
#include <cuda_bf16.h>
#include "tc_common.cuh"

namespace {

constexpr int BN = 128, HD = 128, PAGE = 16, NQ = 16, STAGES = 3;
constexpr uint32_t HALF = 128 * 128, TILE = 2 * HALF;       // [128 x 64] / [128 x 128] bf16
constexpr uint32_t QHALF = NQ * 128, QTILE = 2 * QHALF;     // [16 x 64] / [16 x 128] bf16
constexpr uint32_t TMEM_COLS = 64, S_COL = 0, O_COL = 32;   // S^T double buffered at 0 / 16, O^T at 32

struct __align__(1024) Smem {
  uint8_t k[STAGES][TILE];
  uint8_t v[STAGES][TILE];
  uint8_t q[QTILE];
  uint8_t p[QTILE];
  uint64_t q_full, k_full[STAGES], v_full[STAGES], s_done[2], pv_done;
  float wred[4][NQ];
  uint32_t tmem_base;
  int is_last;
};

struct Params {
  const int* block_tables;
  const int* seq_lens;
  __nv_bfloat16* out;      // [B, Hq, 128]
  float* part_o;           // [B, Hq, ns, 128]
  float* part_ml;          // [B, Hq, ns, 2]
  int* tickets;            // [B, Hkv]
  int* err;
  float scale_log2;
  int Hq, Hkv, max_blocks, window, ns;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand over a [128 keys x 128 dims] tile (two 64-dim halves): 8-key groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(HALF >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void load_kv_block(uint8_t* dst, const CUtensorMap* map, const int* table, int n_pages,
                                              int first_page, int kv_head, uint64_t* bar) {
  tc::mbar_expect_tx(bar, TILE);
#pragma unroll
  for (int pg = 0; pg < BN / PAGE; pg++) {
    int idx = first_page + pg;
    if (idx >= n_pages) idx = n_pages - 1;        // past the end: finite data, masked below
    int page = table[idx];
    tc::tma_load_2d(dst + pg * (PAGE * 128), map, kv_head * HD, page * PAGE, bar);
    tc::tma_load_2d(dst + HALF + pg * (PAGE * 128), map, kv_head * HD + 64, page * PAGE, bar);
  }
}

template <int G>
__global__ void __launch_bounds__(128, 1)
decode_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  pdl_trigger();
  if (tid == 0) {
    tc::prefetch_tmap(&tmap_q);
    tc::prefetch_tmap(&tmap_k);
    tc::prefetch_tmap(&tmap_v);
    tc::mbar_init(&s.q_full, 1);
    for (int i = 0; i < STAGES; i++) {
      tc::mbar_init(&s.k_full[i], 1);
      tc::mbar_init(&s.v_full[i], 1);
    }
    tc::mbar_init(&s.s_done[0], 1);
    tc::mbar_init(&s.s_done[1], 1);
    tc::mbar_init(&s.pv_done, 1);
    tc::fence_barrier_init();
  }
  reinterpret_cast<uint4*>(s.p)[tid] = make_uint4(0, 0, 0, 0);           // rows G..15 of P stay zero
  reinterpret_cast<uint4*>(s.p)[tid + 128] = make_uint4(0, 0, 0, 0);
  if (warp == 0) {
    tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  pdl_wait();      // q, the appended K/V row and the step's plan come from the preceding kernels

  const int n = p.seq_lens[b];
  const int lo_key = p.window > 0 ? max(0, n - p.window) : 0;
  const int first_blk = lo_key / BN, last_blk = (n + BN - 1) / BN;
  const int per = (last_blk - first_blk + p.ns - 1) / p.ns;
  const int blk_a = first_blk + split * per, blk_b = min(last_blk, blk_a + per);
  const int nblk = max(0, blk_b - blk_a);
  const int n_pages = (n + PAGE - 1) / PAGE;
  const int* table = p.block_tables + (size_t)b * p.max_blocks;

  constexpr uint32_t IDESC_S = tc::umma_idesc_bf16(BN, NQ);
  constexpr uint32_t IDESC_PV = tc::umma_idesc_bf16(HD, NQ) | (1u << 15);     // A operand (V) MN-major
  bool failed = false;
  int pending_k[STAGES] = {0, 0, 0}, pending_v[STAGES] = {0, 0, 0};

  auto issue_s = [&](int j) {     // S^T(j) = K(j) Q^T into S buffer j & 1
    const int st = j % STAGES;
    if (!tc::mbar_wait(&s.k_full[st], (j / STAGES) & 1)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
    pending_k[st] = 0;
    if (failed) return;
    tc::tc_fence_after();
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
      tc::umma_bf16(tmem + S_COL + (j & 1) * NQ,
                    tc::umma_desc_sw128(tc::smem_u32(s.k[st]) + (ks >> 2) * HALF + (ks & 3) * 32),
                    tc::umma_desc_sw128(tc::smem_u32(s.q) + (ks >> 2) * QHALF + (ks & 3) * 32), IDESC_S, ks > 0);
    }
    tc::umma_commit(&s.s_done[j & 1]);
  };

  if (tid == 0 && nblk > 0) {
    tc::mbar_expect_tx(&s.q_full, QTILE);
    tc::tma_load_2d(s.q, &tmap_q, 0, b * p.Hq + kvh * G, &s.q_full);
    tc::tma_load_2d(s.q + QHALF, &tmap_q, 64, b * p.Hq + kvh * G, &s.q_full);
    for (int j = 0; j < STAGES && j < nblk; j++) {
      load_kv_block(s.k[j], &tmap_k, table, n_pages, (blk_a + j) * (BN / PAGE), kvh, &s.k_full[j]);
      load_kv_block(s.v[j], &tmap_v, table, n_pages, (blk_a + j) * (BN / PAGE), kvh, &s.v_full[j]);
      pending_k[j] = pending_v[j] = 1;
    }
    if (!tc::mbar_wait(&s.q_full, 0)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
    if (!failed) issue_s(0);
  }

  float m_run[G], l_thr[G];
#pragma unroll
  for (int g = 0; g < G; g++) { m_run[g] = -INFINITY; l_thr[g] = 0.f; }

  for (int j = 0; j < nblk; j++) {
    if (!tc::mbar_wait(&s.s_done[j & 1], (j >> 1) & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
      break;
    }
    tc::tc_fence_after();
    if (tid == 0 && !failed && j + 1 < nblk) issue_s(j + 1);    // overlaps this block's softmax
    // ---- this thread's key: scores of the G heads ----
    float sv[NQ];
    tc::tmem_ld16(lane_addr + S_COL + (j & 1) * NQ, sv);
    tc::tmem_ld_wait();
    const int key = (blk_a + j) * BN + tid;
    const bool vis = key >= lo_key && key < n;
    float sc[G], mx[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      sc[g] = vis ? sv[g] * p.scale_log2 : -INFINITY;
      mx[g] = sc[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xffffffffu, mx[g], o));
    }
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; g++) s.wred[warp][g] = mx[g];
    }
    __syncthreads();
    float alpha[G];
    bool moved = false;
    uint16_t pb[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      float m_blk = fmaxf(fmaxf(s.wred[0][g], s.wred[1][g]), fmaxf(s.wred[2][g], s.wred[3][g]));
      float m_new = fmaxf(m_run[g], m_blk);
      float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[g] = m_run[g] == -INFINITY ? (m_new == -INFINITY ? 1.f : 0.f) : ex2(m_run[g] - m_use);
      moved |= alpha[g] != 1.f;
      __nv_bfloat16 pv = __float2bfloat16_rn(vis ? ex2(sc[g] - m_use) : 0.f);
      l_thr[g] = l_thr[g] * alpha[g] + __bfloat162float(pv);
      pb[g] = *reinterpret_cast<uint16_t*>(&pv);
      m_run[g] = m_new;
    }
    if (j > 0) {     // P and O^T are still being read by the previous block's MMA until this fires
      if (!tc::mbar_wait(&s.pv_done, (j - 1) & 1)) {
        if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
        failed = true;
        break;
      }
      tc::tc_fence_after();
      if (tid == 0 && j - 1 + STAGES < nblk) {     // stage of block j-1 is free: refill it
        const int st = (j - 1) % STAGES, nb = j - 1 + STAGES;
        load_kv_block(s.k[st], &tmap_k, table, n_pages, (blk_a + nb) * (BN / PAGE), kvh, &s.k_full[st]);
        load_kv_block(s.v[st], &tmap_v, table, n_pages, (blk_a + nb) * (BN / PAGE), kvh, &s.v_full[st]);
        pending_k[st] = pending_v[st] = 1;
      }
    }
    // P[head g][key tid], K-major with the 128-byte swizzle
    {
      const int col = tid & 63;
      uint8_t* base = s.p + (tid >> 6) * QHALF + (col & 7) * 2;
#pragma unroll
      for (int g = 0; g < G; g++)
        *reinterpret_cast<uint16_t*>(base + g * 128 + (((col >> 3) ^ (g & 7)) << 4)) = pb[g];
    }
    if (j > 0 && moved) {       // same decision in every thread: alpha is a CTA-wide quantity
      float ov[NQ];
      tc::tmem_ld16(lane_addr + O_COL, ov);
      tc::tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < G; g++) ov[g] *= alpha[g];
      tmem_st16(lane_addr + O_COL, ov);
      tmem_st_wait();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    if (tid == 0 && !failed) {
      tc::tc_fence_after();
      const int st = j % STAGES;
      if (!tc::mbar_wait(&s.v_full[st], (j / STAGES) & 1)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
      pending_v[st] = 0;
      if (!failed) {
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ks++) {
          tc::umma_bf16(tmem + O_COL, umma_desc_mn(tc::smem_u32(s.v[st]) + ks * 2048),
                        tc::umma_desc_sw128(tc::smem_u32(s.p) + (ks >> 2) * QHALF + (ks & 3) * 32), IDESC_PV,
                        j > 0 || ks > 0);
        }
        tc::umma_commit(&s.pv_done);
      }
    }
  }
  if (nblk > 0 && !failed) {
    if (!tc::mbar_wait(&s.pv_done, (nblk - 1) & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
    }
  }
  tc::tc_fence_after();

  // ---- partial result of this split: O^T column g for head dim `tid`, plus (m, l) ----
  float ov[NQ];
#pragma unroll
  for (int i = 0; i < NQ; i++) ov[i] = 0.f;
  if (nblk > 0 && !failed) {
    tc::tmem_ld16(lane_addr + O_COL, ov);
    tc::tmem_ld_wait();
  }
  float l_tot[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    float v = l_thr[g];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    l_tot[g] = v;
  }
  __syncthreads();      // wred: last read in the loop
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < G; g++) s.wred[warp][g] = l_tot[g];
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; g++) l_tot[g] = s.wred[0][g] + s.wred[1][g] + s.wred[2][g] + s.wred[3][g];

  if (!failed) {
    if (p.ns == 1) {
#pragma unroll
      for (int g = 0; g < G; g++) {
        float inv = l_tot[g] > 0.f ? 1.f / l_tot[g] : 0.f;
        p.out[((size_t)b * p.Hq + kvh * G + g) * HD + tid] = __float2bfloat16_rn(ov[g] * inv);
      }
    } else {
#pragma unroll
      for (int g = 0; g < G; g++) {
        size_t row = ((size_t)b * p.Hq + kvh * G + g) * p.ns + split;
        p.part_o[row * HD + tid] = ov[g];
        if (tid == 0) {
          p.part_ml[row * 2] = m_run[g];
          p.part_ml[row * 2 + 1] = l_tot[g];
        }
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        int* tk = p.tickets + b * p.Hkv + kvh;
        int old = atomicAdd(tk, 1);
        s.is_last = old == p.ns - 1;
        if (s.is_last) *tk = 0;
      }
      __syncthreads();
      if (s.is_last) {
        __threadfence();
#pragma unroll
        for (int g = 0; g < G; g++) {
          size_t row0 = ((size_t)b * p.Hq + kvh * G + g) * p.ns;
          float M = -INFINITY;
          for (int sp = 0; sp < p.ns; sp++) M = fmaxf(M, __ldcg(p.part_ml + (row0 + sp) * 2));
          float L = 0.f, o = 0.f;
          for (int sp = 0; sp < p.ns; sp++) {
            float m_s = __ldcg(p.part_ml + (row0 + sp) * 2);
            float w = m_s == -INFINITY ? 0.f : ex2(m_s - M);
            L += __ldcg(p.part_ml + (row0 + sp) * 2 + 1) * w;
            o += __ldcg(p.part_o + (row0 + sp) * HD + tid) * w;
          }
          p.out[((size_t)b * p.Hq + kvh * G + g) * HD + tid] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        }
      }
    }
  }
  // ---- unwind ----
  if (tid == 0 && failed) {
    for (int i = 0; i < STAGES; i++) {
      if (pending_k[i]) tc::mbar_wait(&s.k_full[i], 0, 1u << 16) || tc::mbar_wait(&s.k_full[i], 1, 1u << 16);
      if (pending_v[i]) tc::mbar_wait(&s.v_full[i], 0, 1u << 16) || tc::mbar_wait(&s.v_full[i], 1, 1u << 16);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
}


// ---- two warpgroups per CTA -------------------------------------------------------------------
// Same data path, but the CTA's key blocks alternate between two warpgroups, each with its own
// S^T / O^T accumulators, P tile, running max and barriers, over the shared K/V ring: one
// warpgroup's max-reduction / exp / P store runs while the other's MMAs and TMA refills proceed,
// so the per-block dependency chain of a warpgroup no longer bounds the stream.  The two partial
// results are merged through shared memory before the split's partial is published.
struct __align__(1024) Smem2 {
  uint8_t k[STAGES][TILE];
  uint8_t v[STAGES][TILE];
  uint8_t q[QTILE];
  uint8_t p[2][QTILE];
  uint64_t q_full, k_full[STAGES], v_full[STAGES], s_done[2], pv_done[2];
  float wred[2][4][NQ];
  float xo[NQ][HD];        // warpgroup 1's O^T for the merge
  float xml[2][NQ];        // warpgroup 1's (m, l)
  uint32_t tmem_base;
  int is_last;
};

template <int G>
__global__ void __launch_bounds__(256, 1)
decode_attn2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem2& s = *reinterpret_cast<Smem2*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int wg = threadIdx.x >> 7, tid = threadIdx.x & 127, warp = tid >> 5, lane = tid & 31;

  pdl_trigger();
  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmap_q);
    tc::prefetch_tmap(&tmap_k);
    tc::prefetch_tmap(&tmap_v);
    tc::mbar_init(&s.q_full, 1);
    for (int i = 0; i < STAGES; i++) {
      tc::mbar_init(&s.k_full[i], 1);
      tc::mbar_init(&s.v_full[i], 1);
    }
    for (int i = 0; i < 2; i++) {
      tc::mbar_init(&s.s_done[i], 1);
      tc::mbar_init(&s.pv_done[i], 1);
    }
    tc::fence_barrier_init();
  }
  reinterpret_cast<uint4*>(s.p[wg])[tid] = make_uint4(0, 0, 0, 0);
  reinterpret_cast<uint4*>(s.p[wg])[tid + 128] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x < 32) {
    tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t s_col = S_COL + wg * NQ, o_col = O_COL + wg * NQ;
  pdl_wait();

  const int n = p.seq_lens[b];
  const int lo_key = p.window > 0 ? max(0, n - p.window) : 0;
  const int first_blk = lo_key / BN, last_blk = (n + BN - 1) / BN;
  const int per = (last_blk - first_blk + p.ns - 1) / p.ns;
  const int blk_a = first_blk + split * per, blk_b = min(last_blk, blk_a + per);
  const int nblk = max(0, blk_b - blk_a);
  const int n_pages = (n + PAGE - 1) / PAGE;
  const int* table = p.block_tables + (size_t)b * p.max_blocks;

  constexpr uint32_t IDESC_S = tc::umma_idesc_bf16(BN, NQ);
  constexpr uint32_t IDESC_PV = tc::umma_idesc_bf16(HD, NQ) | (1u << 15);
  bool failed = false;

  auto load_block = [&](int j) {
    const int st = j % STAGES;
    load_kv_block(s.k[st], &tmap_k, table, n_pages, (blk_a + j) * (BN / PAGE), kvh, &s.k_full[st]);
    load_kv_block(s.v[st], &tmap_v, table, n_pages, (blk_a + j) * (BN / PAGE), kvh, &s.v_full[st]);
  };
  if (threadIdx.x == 0 && nblk > 0) {
    tc::mbar_expect_tx(&s.q_full, QTILE);
    tc::tma_load_2d(s.q, &tmap_q, 0, b * p.Hq + kvh * G, &s.q_full);
    tc::tma_load_2d(s.q + QHALF, &tmap_q, 64, b * p.Hq + kvh * G, &s.q_full);
    for (int j = 0; j < STAGES && j < nblk; j++) load_block(j);
  }

  float m_run[G], l_thr[G];
#pragma unroll
  for (int g = 0; g < G; g++) { m_run[g] = -INFINITY; l_thr[g] = 0.f; }
  int n_mine = 0;

  for (int j = wg; j < nblk; j += 2, n_mine++) {
    const int st = j % STAGES;
    if (tid == 0) {        // S^T(j) = K(j) Q^T
      if (n_mine == 0 && !tc::mbar_wait(&s.q_full, 0)) failed = true;
      if (!failed && !tc::mbar_wait(&s.k_full[st], (j / STAGES) & 1)) failed = true;
      if (failed) atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
      else {
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
          tc::umma_bf16(tmem + s_col, tc::umma_desc_sw128(tc::smem_u32(s.k[st]) + (ks >> 2) * HALF + (ks & 3) * 32),
                        tc::umma_desc_sw128(tc::smem_u32(s.q) + (ks >> 2) * QHALF + (ks & 3) * 32), IDESC_S, ks > 0);
        }
        tc::umma_commit(&s.s_done[wg]);
      }
    }
    if (!tc::mbar_wait(&s.s_done[wg], n_mine & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
      break;
    }
    tc::tc_fence_after();
    float sv[NQ];
    tc::tmem_ld16(lane_addr + s_col, sv);
    tc::tmem_ld_wait();
    const int key = (blk_a + j) * BN + tid;
    const bool vis = key >= lo_key && key < n;
    float sc[G], mx[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      sc[g] = vis ? sv[g] * p.scale_log2 : -INFINITY;
      mx[g] = sc[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xffffffffu, mx[g], o));
    }
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; g++) s.wred[wg][warp][g] = mx[g];
    }
    asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");
    float alpha[G];
    bool moved = false;
    uint16_t pb[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      float m_blk = fmaxf(fmaxf(s.wred[wg][0][g], s.wred[wg][1][g]), fmaxf(s.wred[wg][2][g], s.wred[wg][3][g]));
      float m_new = fmaxf(m_run[g], m_blk);
      float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[g] = m_run[g] == -INFINITY ? (m_new == -INFINITY ? 1.f : 0.f) : ex2(m_run[g] - m_use);
      moved |= alpha[g] != 1.f;
      __nv_bfloat16 pv = __float2bfloat16_rn(vis ? ex2(sc[g] - m_use) : 0.f);
      l_thr[g] = l_thr[g] * alpha[g] + __bfloat162float(pv);
      pb[g] = *reinterpret_cast<uint16_t*>(&pv);
      m_run[g] = m_new;
    }
    if (n_mine > 0) {     // this warpgroup's previous O^T MMA still reads P and O^T until this fires
      if (!tc::mbar_wait(&s.pv_done[wg], (n_mine - 1) & 1)) {
        if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
        failed = true;
        break;
      }
      tc::tc_fence_after();
    }
    {
      const int col = tid & 63;
      uint8_t* base = s.p[wg] + (tid >> 6) * QHALF + (col & 7) * 2;
#pragma unroll
      for (int g = 0; g < G; g++)
        *reinterpret_cast<uint16_t*>(base + g * 128 + (((col >> 3) ^ (g & 7)) << 4)) = pb[g];
    }
    if (n_mine > 0 && moved) {
      float ov[NQ];
      tc::tmem_ld16(lane_addr + o_col, ov);
      tc::tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < G; g++) ov[g] *= alpha[g];
      tmem_st16(lane_addr + o_col, ov);
      tmem_st_wait();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");
    if (tid == 0 && !failed) {
      tc::tc_fence_after();
      if (!tc::mbar_wait(&s.v_full[st], (j / STAGES) & 1)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
      if (!failed) {
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ks++) {
          tc::umma_bf16(tmem + o_col, umma_desc_mn(tc::smem_u32(s.v[st]) + ks * 2048),
                        tc::umma_desc_sw128(tc::smem_u32(s.p[wg]) + (ks >> 2) * QHALF + (ks & 3) * 32), IDESC_PV,
                        n_mine > 0 || ks > 0);
        }
        tc::umma_commit(&s.pv_done[wg]);
        // the stage is free as soon as these MMAs have read it: refill it with the block three ahead
        if (j + STAGES < nblk) {
          if (tc::mbar_wait(&s.pv_done[wg], n_mine & 1)) load_block(j + STAGES);
          else { failed = true; atomicExch(p.err, tc::ERR_ACC_TIMEOUT); }
        }
      }
    }
  }
  if (n_mine > 0 && !failed) {
    if (!tc::mbar_wait(&s.pv_done[wg], (n_mine - 1) & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
    }
  }
  tc::tc_fence_after();

  float ov[NQ];
#pragma unroll
  for (int i = 0; i < NQ; i++) ov[i] = 0.f;
  if (n_mine > 0 && !failed) {
    tc::tmem_ld16(lane_addr + o_col, ov);
    tc::tmem_ld_wait();
  }
  float l_tot[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    float v = l_thr[g];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    l_tot[g] = v;
  }
  asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < G; g++) s.wred[wg][warp][g] = l_tot[g];
  }
  asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");
#pragma unroll
  for (int g = 0; g < G; g++) l_tot[g] = s.wred[wg][0][g] + s.wred[wg][1][g] + s.wred[wg][2][g] + s.wred[wg][3][g];
  // ---- merge warpgroup 1 into warpgroup 0 ----
  if (wg == 1) {
#pragma unroll
    for (int g = 0; g < G; g++) {
      s.xo[g][tid] = ov[g];
      if (tid == 0) { s.xml[0][g] = m_run[g]; s.xml[1][g] = failed ? -1.f : l_tot[g]; }
    }
  }
  __syncthreads();
  if (wg == 0) {
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float m1 = s.xml[0][g], l1 = s.xml[1][g];
      if (l1 < 0.f) failed = true;
      const float M = fmaxf(m_run[g], m1);
      const float w0 = m_run[g] == -INFINITY ? 0.f : ex2(m_run[g] - M), w1 = m1 == -INFINITY ? 0.f : ex2(m1 - M);
      ov[g] = ov[g] * w0 + s.xo[g][tid] * w1;
      l_tot[g] = l_tot[g] * w0 + fmaxf(l1, 0.f) * w1;
      m_run[g] = M;
    }
    if (!failed) {
      if (p.ns == 1) {
#pragma unroll
        for (int g = 0; g < G; g++) {
          float inv = l_tot[g] > 0.f ? 1.f / l_tot[g] : 0.f;
          p.out[((size_t)b * p.Hq + kvh * G + g) * HD + tid] = __float2bfloat16_rn(ov[g] * inv);
        }
      } else {
#pragma unroll
        for (int g = 0; g < G; g++) {
          size_t row = ((size_t)b * p.Hq + kvh * G + g) * p.ns + split;
          p.part_o[row * HD + tid] = ov[g];
          if (tid == 0) {
            p.part_ml[row * 2] = m_run[g];
            p.part_ml[row * 2 + 1] = l_tot[g];
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid == 0) {
          int* tk = p.tickets + b * p.Hkv + kvh;
          int old = atomicAdd(tk, 1);
          s.is_last = old == p.ns - 1;
          if (s.is_last) *tk = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s.is_last) {
          __threadfence();
#pragma unroll
          for (int g = 0; g < G; g++) {
            size_t row0 = ((size_t)b * p.Hq + kvh * G + g) * p.ns;
            float M = -INFINITY;
            for (int sp = 0; sp < p.ns; sp++) M = fmaxf(M, __ldcg(p.part_ml + (row0 + sp) * 2));
            float L = 0.f, o = 0.f;
            for (int sp = 0; sp < p.ns; sp++) {
              float m_s = __ldcg(p.part_ml + (row0 + sp) * 2);
              float w = m_s == -INFINITY ? 0.f : ex2(m_s - M);
              L += __ldcg(p.part_ml + (row0 + sp) * 2 + 1) * w;
              o += __ldcg(p.part_o + (row0 + sp) * HD + tid) * w;
            }
            p.out[((size_t)b * p.Hq + kvh * G + g) * HD + tid] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
          }
        }
      }
    }
  }
  // ---- unwind: give copies that may still be in flight a bounded time to land, free the TMEM ----
  if (failed && tid == 0) {
    for (int i = 0; i < STAGES; i++) {
      tc::mbar_wait(&s.k_full[i], 0, 1u << 14) || tc::mbar_wait(&s.k_full[i], 1, 1u << 14);
      tc::mbar_wait(&s.v_full[i], 0, 1u << 14) || tc::mbar_wait(&s.v_full[i], 1, 1u << 14);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tc::tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace

int* exo_tc_err_ptr();

// Splits per (sequence, KV head): enough CTAs for a few waves over the 148 SMs, never more than
// the 128-key blocks of the longest possible context.
EXO_API int exo_decode_attn_tc_splits(int B, int Hkv, int max_len) {
  long pairs = (long)B * Hkv;
  int nb = (max_len + BN - 1) / BN;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 32 && s <= nb; s++) {
    long ctas = pairs * s;
    double rounds = (double)((ctas + 147) / 148);
    double cost = rounds * ((nb + s - 1) / s + 1.5);      // 1.5 block-times of fixed cost per CTA
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  return best;
}

EXO_API long exo_decode_attn_tc_workspace(int B, int Hq, int ns) { return (long)B * Hq * ns * (HD + 2) + 64; }

// q [B, Hq, 128] bf16 (one row per sequence); `tickets` [B*Hkv] zero before the first launch.
// Returns <0 for shapes this kernel does not take (-2) or when set-up is missing.
EXO_API int exo_decode_attn_tc(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                               const int* seq_lens, void* out, float* workspace, int* tickets, float scale, int B, int Hq,
                               int Hkv, int D, int n_blocks, int max_blocks, int block_size, int ns, int window,
                               cudaStream_t st) {
  if (B <= 0) return 0;
  int G = Hkv > 0 ? Hq / Hkv : 0;
  if (D != HD || block_size != PAGE || G * Hkv != Hq || (G != 1 && G != 2 && G != 4 && G != 8) || ns < 1 || ns > 32)
    return -2;
  int* err = exo_tc_err_ptr();
  if (!err) return -4;
  const CUtensorMap* tq = exo_tmap_2d_bf16(q, (uint64_t)B * Hq, (uint64_t)HD, NQ);
  const CUtensorMap* tk = exo_tmap_2d_bf16(kcache, (uint64_t)n_blocks * PAGE, (uint64_t)Hkv * HD, PAGE);
  const CUtensorMap* tv = exo_tmap_2d_bf16(vcache, (uint64_t)n_blocks * PAGE, (uint64_t)Hkv * HD, PAGE);
  if (!tq || !tk || !tv) return -5;
  size_t smem = sizeof(Smem) + 1024;
  Params p;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.out = (__nv_bfloat16*)out;
  p.part_o = workspace; p.part_ml = workspace + (size_t)B * Hq * ns * HD;
  p.tickets = tickets; p.err = err; p.scale_log2 = scale * 1.4426950408889634f;
  p.Hq = Hq; p.Hkv = Hkv; p.max_blocks = max_blocks; p.window = window; p.ns = ns;
  dim3 grid(ns, Hkv, B);
  cudaError_t e = cudaSuccess;
  static int two_wg = -1;
  if (two_wg < 0) {
    const char* ev = getenv("EXO_DECODE_ATTN_WARPGROUPS");
    two_wg = (ev && ev[0] == '1') ? 0 : 1;      // two warpgroups unless EXO_DECODE_ATTN_WARPGROUPS=1
  }
  if (two_wg) {
    size_t smem2 = sizeof(Smem2) + 1024;
#define LAUNCH2(GG)                                                                                                  \
  do {                                                                                                               \
    static bool attr_set = false;                                                                                    \
    if (!attr_set) {                                                                                                 \
      if (cudaFuncSetAttribute(decode_attn2_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2) !=  \
          cudaSuccess)                                                                                               \
        return -3;                                                                                                   \
      attr_set = true;                                                                                               \
    }                                                                                                                \
    e = launch_pdl(decode_attn2_kernel<GG>, grid, dim3(256), smem2, st, *tq, *tk, *tv, p);                           \
  } while (0)
    switch (G) {
      case 1: LAUNCH2(1); break;
      case 2: LAUNCH2(2); break;
      case 4: LAUNCH2(4); break;
      default: LAUNCH2(8); break;
    }
#undef LAUNCH2
    if (e != cudaSuccess) return (int)e;
    EXO_CHECK_LAUNCH();
    return 0;
  }
#define LAUNCH(GG)                                                                                                  \
  do {                                                                                                              \
    static bool attr_set = false;                                                                                   \
    if (!attr_set) {                                                                                                \
      if (cudaFuncSetAttribute(decode_attn_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=   \
          cudaSuccess)                                                                                              \
        return -3;                                                                                                  \
      attr_set = true;                                                                                              \
    }                                                                                                               \
    e = launch_pdl(decode_attn_kernel<GG>, grid, dim3(128), smem, st, *tq, *tk, *tv, p);                            \
  } while (0)
  switch (G) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    default: LAUNCH(8); break;
  }
#undef LAUNCH
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}
