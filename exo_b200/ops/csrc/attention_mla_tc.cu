// Multi-head latent attention (DeepSeek-V2/V3, Kimi) over the paged latent cache, weight-absorbed form,
// on the 5th-generation tensor cores.  bf16, 16-token pages, kv_lora_rank 512, rope sub-vector 64.
//
// Every token's cache row is [c (512 latent dims) | k_rope (64 dims)], shared by all heads: the cache is at
// once the K and the V of ONE multi-query group whose "heads" are the query heads.  With the up-projections
// folded into the query (q_lat = q_nope . W_UK) and the output (o = o_lat . W_UV), attention is
//   S^T[key, head]  = C[key, 0:576] . Q[head, 0:576]         A = cache tile (K-major),  B = Q  (16 heads)
//   O^T[dim, head] += C[key, dim]^T . P[head, key]           A = the SAME tile read MN-major, B = P
// so a block of 128 keys is fetched once (TMA page gather, 144 KB) and feeds both products from shared memory:
// four [128 keys x 128 dims] tiles of the latent part plus one [128 x 64] rope tile.  Shared memory holds five
// latent tiles and two rope tiles, i.e. one block plus the first tile and the rope tile of the next.
//
// One CTA = (split of the keys, group of up to 16 heads, query token); 128 threads, thread t owns TMEM lane t:
// key t of the block for the softmax, output dims t, 128 + t, 256 + t, 384 + t for the result.  The same kernel
// serves decode (one token per sequence, split-KV merged by a second small kernel) and prefill chunks (the token's causal
// limit is its key count).  The reference computes this attention with mlx-lm's DeepSeek model and slices the
// absorbed projections per rank (src/exo/worker/engines/mlx/auto_parallel.py:688-721).
// Every wait is bounded: on a timeout the kernel records a code, drains and returns.
#include <cuda_bf16.h>
#include "tc_common.cuh"

namespace {

constexpr int BN = 128, PAGE = 16, NQ = 16, LAT = 512, ROPE = 64, DQK = LAT + ROPE;
constexpr int NT = LAT / 128;                 // latent tiles per key block
constexpr int SLOTS = 5;                      // latent-tile slots in shared memory
constexpr uint32_t HALF = 128 * 128;          // [128 keys x 64 dims] bf16
constexpr uint32_t TILE = 2 * HALF;           // [128 keys x 128 dims]
constexpr uint32_t QCHUNK = NQ * 128;         // [16 heads x 64 dims]
constexpr int QCHUNKS = DQK / 64;             // 9
constexpr uint32_t QBYTES = QCHUNKS * QCHUNK;
constexpr uint32_t PTILE = 2 * QCHUNK;        // P [16 heads x 128 keys]
constexpr uint32_t TMEM_COLS = 128, S_COL = 0, O_COL = 32;   // S^T: 16 columns; O^T: four 16-column tiles from 32

struct __align__(1024) Smem {
  uint8_t tile[SLOTS][TILE];
  uint8_t rope[2][HALF];
  uint8_t q[QBYTES];
  uint8_t p[PTILE];
  uint64_t q_full, tile_full[SLOTS], rope_full[2], s_done, pv_done;
  float wred[4][NQ];
  uint32_t tmem_base;
  int is_last;
  int abort;           // set by thread 0 when one of ITS waits ran out: every thread leaves the loop at the next barrier
};

struct Params {
  const int* block_tables;   // [B, max_blocks]
  const int* seq_lens;       // [B] keys of each sequence including this step's tokens
  const int* cu_q;           // [B + 1] or null (decode: token t is sequence t)
  const int* tok_seq;        // [T] sequence of each token, or null (decode)
  __nv_bfloat16* out;        // [T, H, 512]
  float* part_o;             // [T * H, ns, 512]
  float* part_ml;            // [T * H, ns, 2]
  int* err;
  float scale_log2;
  int H, groups, max_blocks, ns;
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

// MN-major A operand over a [128 keys x 128 dims] tile stored as two 64-dim halves: 8-key groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(HALF >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int G>
__global__ void __launch_bounds__(128, 1)
mla_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int split = blockIdx.x, grp = blockIdx.y, t = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  pdl_trigger();
  if (tid == 0) {
    tc::prefetch_tmap(&tmap_q);
    tc::prefetch_tmap(&tmap_c);
    tc::mbar_init(&s.q_full, 1);
    for (int i = 0; i < SLOTS; i++) tc::mbar_init(&s.tile_full[i], 1);
    tc::mbar_init(&s.rope_full[0], 1);
    tc::mbar_init(&s.rope_full[1], 1);
    tc::mbar_init(&s.s_done, 1);
    tc::mbar_init(&s.pv_done, 1);
    s.abort = 0;
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
  pdl_wait();      // q, the appended cache row and the step's plan come from the preceding kernels

  const int b = p.tok_seq ? p.tok_seq[t] : t;
  int n = p.seq_lens[b];
  if (p.cu_q) n -= p.cu_q[b + 1] - 1 - t;          // causal: a prompt token sees the keys up to its own position
  n = max(n, 0);
  const int last_blk = (n + BN - 1) / BN;
  const int per = (last_blk + p.ns - 1) / p.ns;
  const int blk_a = split * per, blk_b = min(last_blk, blk_a + per);
  const int nblk = max(0, blk_b - blk_a);
  const int n_pages = (n + PAGE - 1) / PAGE;
  const int* table = p.block_tables + (size_t)b * p.max_blocks;
  const int q_row = t * p.H + grp * G;

  constexpr uint32_t IDESC_S = tc::umma_idesc_bf16(BN, NQ);
  constexpr uint32_t IDESC_PV = tc::umma_idesc_bf16(128, NQ) | (1u << 15);     // A operand (the cache tile) MN-major
  bool failed = false;

  auto load_tile = [&](int j, int dt) {          // latent dims [128 dt, 128 dt + 128) of key block j
    const int slot = (NT * j + dt) % SLOTS;
    uint64_t* bar = &s.tile_full[slot];
    tc::mbar_expect_tx(bar, TILE);
#pragma unroll
    for (int pg = 0; pg < BN / PAGE; pg++) {
      int idx = (blk_a + j) * (BN / PAGE) + pg;
      if (idx >= n_pages) idx = n_pages - 1;     // past the end: finite data, masked below
      const int page = table[idx];
      tc::tma_load_2d(s.tile[slot] + pg * (PAGE * 128), &tmap_c, dt * 128, page * PAGE, bar);
      tc::tma_load_2d(s.tile[slot] + HALF + pg * (PAGE * 128), &tmap_c, dt * 128 + 64, page * PAGE, bar);
    }
  };
  auto load_rope = [&](int j) {
    uint64_t* bar = &s.rope_full[j & 1];
    tc::mbar_expect_tx(bar, HALF);
#pragma unroll
    for (int pg = 0; pg < BN / PAGE; pg++) {
      int idx = (blk_a + j) * (BN / PAGE) + pg;
      if (idx >= n_pages) idx = n_pages - 1;
      tc::tma_load_2d(s.rope[j & 1] + pg * (PAGE * 128), &tmap_c, LAT, table[idx] * PAGE, bar);
    }
  };

  if (tid == 0 && nblk > 0) {
    tc::mbar_expect_tx(&s.q_full, QBYTES);
#pragma unroll
    for (int c = 0; c < QCHUNKS; c++) tc::tma_load_2d(s.q + c * QCHUNK, &tmap_q, c * 64, q_row, &s.q_full);
    for (int dt = 0; dt < NT; dt++) load_tile(0, dt);
    load_rope(0);
    if (nblk > 1) { load_tile(1, 0); load_rope(1); }
    if (!tc::mbar_wait(&s.q_full, 0)) { failed = true; s.abort = 1; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
  }

  float m_run[G], l_thr[G];
#pragma unroll
  for (int g = 0; g < G; g++) { m_run[g] = -INFINITY; l_thr[g] = 0.f; }

  for (int j = 0; j < nblk; j++) {
    if (tid == 0) {                  // S^T(j) = C(j) Q^T over the 576 dims, tile by tile as the copies land
      for (int dt = 0; dt < NT && !failed; dt++) {
        const int seq = NT * j + dt, slot = seq % SLOTS;
        if (!tc::mbar_wait(&s.tile_full[slot], (seq / SLOTS) & 1)) { failed = true; break; }
        tc::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          tc::umma_bf16(tmem + S_COL, tc::umma_desc_sw128(tc::smem_u32(s.tile[slot]) + (kk >> 2) * HALF + (kk & 3) * 32),
                        tc::umma_desc_sw128(tc::smem_u32(s.q) + (2 * dt + (kk >> 2)) * QCHUNK + (kk & 3) * 32), IDESC_S,
                        (dt | kk) != 0);
        }
      }
      if (!failed && !tc::mbar_wait(&s.rope_full[j & 1], (j >> 1) & 1)) failed = true;
      if (failed) { s.abort = 1; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
      else {
        tc::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
          tc::umma_bf16(tmem + S_COL, tc::umma_desc_sw128(tc::smem_u32(s.rope[j & 1]) + kk * 32),
                        tc::umma_desc_sw128(tc::smem_u32(s.q) + (QCHUNKS - 1) * QCHUNK + kk * 32), IDESC_S, true);
        }
      }
      tc::umma_commit(&s.s_done);     // also when nothing was issued: the waiters below must not depend on `failed`
    }
    if (!tc::mbar_wait(&s.s_done, j & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
      break;
    }
    tc::tc_fence_after();
    if (tid == 0 && !failed && j + 2 < nblk) load_rope(j + 2);     // this block's rope tile has been read
    // ---- this thread's key: scores of the G heads ----
    float sv[NQ];
    tc::tmem_ld16(lane_addr + S_COL, sv);
    tc::tmem_ld_wait();
    const int key = (blk_a + j) * BN + tid;
    const bool vis = key < n;
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
    if (s.abort) { failed = true; break; }      // thread 0 could not get its tiles: same decision in every thread
    float alpha[G];
    bool moved = false;
    uint16_t pb[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float m_blk = fmaxf(fmaxf(s.wred[0][g], s.wred[1][g]), fmaxf(s.wred[2][g], s.wred[3][g]));
      const float m_new = fmaxf(m_run[g], m_blk);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[g] = m_run[g] == -INFINITY ? (m_new == -INFINITY ? 1.f : 0.f) : ex2(m_run[g] - m_use);
      moved |= alpha[g] != 1.f;
      const __nv_bfloat16 pv = __float2bfloat16_rn(vis ? ex2(sc[g] - m_use) : 0.f);
      l_thr[g] = l_thr[g] * alpha[g] + __bfloat162float(pv);
      pb[g] = *reinterpret_cast<const uint16_t*>(&pv);
      m_run[g] = m_new;
    }
    // P[head g][key tid], K-major with the 128-byte swizzle (the previous block's P . C product has completed:
    // its barrier is waited at the end of every iteration)
    {
      const int col = tid & 63;
      uint8_t* base = s.p + (tid >> 6) * QCHUNK + (col & 7) * 2;
#pragma unroll
      for (int g = 0; g < G; g++)
        *reinterpret_cast<uint16_t*>(base + g * 128 + (((col >> 3) ^ (g & 7)) << 4)) = pb[g];
    }
    if (j > 0 && moved) {       // same decision in every thread: alpha is a CTA-wide quantity
#pragma unroll
      for (int dt = 0; dt < NT; dt++) {
        float ov[NQ];
        tc::tmem_ld16(lane_addr + O_COL + dt * NQ, ov);
        tc::tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < G; g++) ov[g] *= alpha[g];
        tmem_st16(lane_addr + O_COL + dt * NQ, ov);
      }
      tmem_st_wait();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc::tc_fence_after();
      if (!failed) {
#pragma unroll
        for (int dt = 0; dt < NT; dt++) {
          const int slot = (NT * j + dt) % SLOTS;
#pragma unroll
          for (int ks = 0; ks < BN / 16; ks++) {
            tc::umma_bf16(tmem + O_COL + dt * NQ, umma_desc_mn(tc::smem_u32(s.tile[slot]) + ks * 2048),
                          tc::umma_desc_sw128(tc::smem_u32(s.p) + (ks >> 2) * QCHUNK + (ks & 3) * 32), IDESC_PV,
                          j > 0 || ks > 0);
          }
        }
      }
      tc::umma_commit(&s.pv_done);
    }
    if (!tc::mbar_wait(&s.pv_done, j & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
      break;
    }
    tc::tc_fence_after();
    if (tid == 0 && !failed) {     // the block's four latent tiles are free: bring in the rest of the next block
      if (j + 1 < nblk)
        for (int dt = 1; dt < NT; dt++) load_tile(j + 1, dt);
      if (j + 2 < nblk) load_tile(j + 2, 0);
    }
  }
  __syncthreads();
  failed = failed || s.abort != 0;
  tc::tc_fence_after();

  // ---- partial result of this split: O^T column g for dims tid + 128 dt, plus (m, l) ----
  float ov[NT][NQ];
#pragma unroll
  for (int dt = 0; dt < NT; dt++)
#pragma unroll
    for (int i = 0; i < NQ; i++) ov[dt][i] = 0.f;
  if (nblk > 0 && !failed) {
#pragma unroll
    for (int dt = 0; dt < NT; dt++) tc::tmem_ld16(lane_addr + O_COL + dt * NQ, ov[dt]);
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
        const float inv = l_tot[g] > 0.f ? 1.f / l_tot[g] : 0.f;
#pragma unroll
        for (int dt = 0; dt < NT; dt++)
          p.out[((size_t)q_row + g) * LAT + dt * 128 + tid] = __float2bfloat16_rn(ov[dt][g] * inv);
      }
    } else {
#pragma unroll
      for (int g = 0; g < G; g++) {
        const size_t row = ((size_t)q_row + g) * p.ns + split;
#pragma unroll
        for (int dt = 0; dt < NT; dt++) p.part_o[row * LAT + dt * 128 + tid] = ov[dt][g];
        if (tid == 0) {
          p.part_ml[row * 2] = m_run[g];
          p.part_ml[row * 2 + 1] = l_tot[g];
        }
      }
    }
  }
  // ---- unwind: give copies that may still be in flight a bounded time to land, free the TMEM ----
  if (failed && tid == 0) {
    for (int i = 0; i < SLOTS; i++) tc::mbar_wait(&s.tile_full[i], 0, 1u << 14) || tc::mbar_wait(&s.tile_full[i], 1, 1u << 14);
    for (int i = 0; i < 2; i++) tc::mbar_wait(&s.rope_full[i], 0, 1u << 14) || tc::mbar_wait(&s.rope_full[i], 1, 1u << 14);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
}

// Merge of the key splits: one CTA per (token, head) column, 128 threads x 4 output dims.  A kernel of its own so
// that the 16 .. 128 columns of a token are merged by as many SMs at once (merged by the last split's CTA alone, the
// partials of all heads were one CTA's serial chain of L2 round trips, longer than the attention itself).
__global__ void __launch_bounds__(128)
mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* out, int ns) {
  pdl_trigger();
  pdl_wait();
  __shared__ float w_s[32];
  __shared__ float inv_s;
  const size_t col = blockIdx.x;
  const int tid = threadIdx.x;
  if (tid < 32) {
    const float m_s = tid < ns ? __ldcg(part_ml + (col * ns + tid) * 2) : -INFINITY;
    const float l_s = tid < ns ? __ldcg(part_ml + (col * ns + tid) * 2 + 1) : 0.f;
    float M = m_s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float w = m_s == -INFINITY ? 0.f : ex2(m_s - M);
    float L = l_s * w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    w_s[tid] = w;
    if (tid == 0) inv_s = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  const float* po = part_o + col * ns * LAT + tid;
  float o[NT] = {0.f, 0.f, 0.f, 0.f};
  int sp = 0;
  for (; sp + 4 <= ns; sp += 4) {
    float v[4][NT];
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
      for (int dt = 0; dt < NT; dt++) v[u][dt] = __ldcg(po + (size_t)(sp + u) * LAT + dt * 128);
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
      for (int dt = 0; dt < NT; dt++) o[dt] += v[u][dt] * w_s[sp + u];
  }
  for (; sp < ns; sp++)
#pragma unroll
    for (int dt = 0; dt < NT; dt++) o[dt] += __ldcg(po + (size_t)sp * LAT + dt * 128) * w_s[sp];
#pragma unroll
  for (int dt = 0; dt < NT; dt++) out[col * LAT + dt * 128 + tid] = __float2bfloat16_rn(o[dt] * inv_s);
}

// ---- small CUDA-core kernels around the attention: cache append, query absorption, output absorption ----------

// Cache row of each new token: [RMSNorm(kv_a[0:512]) * w | RoPE(kv_a[512:576])], rope on adjacent pairs.
__global__ void __launch_bounds__(128)
mla_kv_append_kernel(const __nv_bfloat16* __restrict__ kva, const __nv_bfloat16* __restrict__ norm_w, float eps,
                     const int* __restrict__ positions, const float* __restrict__ inv_freq, float mscale,
                     __nv_bfloat16* cache, const int* __restrict__ slots, int T) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[4];
  const int t = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* row = kva + (size_t)t * DQK;
  __nv_bfloat16* dst = cache + (size_t)slots[t] * DQK;
  float v[4];
  {
    const uint2 u = *reinterpret_cast<const uint2*>(row + tid * 4);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h2[0]), c = __bfloat1622float2(h2[1]);
    v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
  }
  float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float rstd = rsqrtf((red[0] + red[1] + red[2] + red[3]) / LAT + eps);
  {
    const uint2 wu = *reinterpret_cast<const uint2*>(norm_w + tid * 4);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wu);
    const float2 wa = __bfloat1622float2(w2[0]), wc = __bfloat1622float2(w2[1]);
    uint2 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
    o2[0] = __floats2bfloat162_rn(v[0] * rstd * wa.x, v[1] * rstd * wa.y);
    o2[1] = __floats2bfloat162_rn(v[2] * rstd * wc.x, v[3] * rstd * wc.y);
    *reinterpret_cast<uint2*>(dst + tid * 4) = o;
  }
  if (tid < ROPE / 2) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + LAT + 2 * tid));
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[tid], &sn, &cs);
    sn *= mscale; cs *= mscale;
    *reinterpret_cast<__nv_bfloat162*>(dst + LAT + 2 * tid) = __floats2bfloat162_rn(x.x * cs - x.y * sn, x.y * cs + x.x * sn);
  }
}

// Query in cache space: out[t, h, 0:512] = q_nope[t, h, :] . W_UK[h] ([128 x 512]), out[t, h, 512:576] = RoPE(q_rope).
// grid (H, 9): blocks 0..7 of y own 64 latent columns each and keep their [128 x 64] slice of W_UK[h] in shared
// memory across the tokens; block 8 rotates the rope sub-vector.  For decode batches (the weights are read once).
__global__ void __launch_bounds__(256)
mla_q_absorb_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ w_uk,
                    const int* __restrict__ positions, const float* __restrict__ inv_freq, float mscale,
                    __nv_bfloat16* out, int T, int H, int rope_only) {
  pdl_trigger();
  constexpr int NOPE = 128, QD = NOPE + ROPE;
  __shared__ float wsm[NOPE][64 + 1];
  __shared__ float qs[NOPE];
  __shared__ float part[4][64];
  const int h = blockIdx.x, tid = threadIdx.x;
  if (blockIdx.y == 8 || rope_only) {
    pdl_wait();
    for (int i = tid; i < T * (ROPE / 2); i += 256) {
      const int t = i / (ROPE / 2), pr = i % (ROPE / 2);
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q + ((size_t)t * H + h) * QD + NOPE + 2 * pr));
      float sn, cs;
      sincosf((float)positions[t] * inv_freq[pr], &sn, &cs);
      sn *= mscale; cs *= mscale;
      *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * H + h) * DQK + LAT + 2 * pr) =
          __floats2bfloat162_rn(x.x * cs - x.y * sn, x.y * cs + x.x * sn);
    }
    return;
  }
  const int c0 = blockIdx.y * 64;
  for (int i = tid; i < NOPE * 64; i += 256) {          // weights are constants: loaded before the dependency wait
    const int nn = i >> 6, c = i & 63;
    wsm[nn][c] = __bfloat162float(w_uk[((size_t)h * NOPE + nn) * LAT + c0 + c]);
  }
  pdl_wait();
  const int c = tid & 63, pt = tid >> 6;
  for (int t = 0; t < T; t++) {
    __syncthreads();
    if (tid < NOPE) qs[tid] = __bfloat162float(q[((size_t)t * H + h) * QD + tid]);
    __syncthreads();
    float acc = 0.f;
#pragma unroll 8
    for (int nn = pt * 32; nn < pt * 32 + 32; nn++) acc += qs[nn] * wsm[nn][c];
    part[pt][c] = acc;
    __syncthreads();
    if (tid < 64) out[((size_t)t * H + h) * DQK + c0 + tid] = __float2bfloat16_rn(part[0][tid] + part[1][tid] + part[2][tid] + part[3][tid]);
  }
}

// Attention output back to head space: out[t, h, v] = o_lat[t, h, :] . W_UV[h, v, :]  (v < 128, 512 latent dims).
// grid (H, 16): a warp owns one v and keeps its W_UV row in registers across the tokens.  For decode batches.
__global__ void __launch_bounds__(256)
mla_o_absorb_kernel(const __nv_bfloat16* __restrict__ o_lat, const __nv_bfloat16* __restrict__ w_uv, __nv_bfloat16* out,
                    int T, int H) {
  pdl_trigger();
  constexpr int VD = 128;
  const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int v = blockIdx.y * 8 + warp;
  float w[16];
  {
    const __nv_bfloat16* wr = w_uv + ((size_t)h * VD + v) * LAT + lane * 16;
    unpack8(*reinterpret_cast<const uint4*>(wr), w);
    unpack8(*reinterpret_cast<const uint4*>(wr + 8), w + 8);
  }
  pdl_wait();
  for (int t = 0; t < T; t++) {
    const __nv_bfloat16* xr = o_lat + ((size_t)t * H + h) * LAT + lane * 16;
    float x[16];
    unpack8(*reinterpret_cast<const uint4*>(xr), x);
    unpack8(*reinterpret_cast<const uint4*>(xr + 8), x + 8);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) acc += x[i] * w[i];
    acc = warp_sum(acc);
    if (lane == 0) out[((size_t)t * H + h) * VD + v] = __float2bfloat16_rn(acc);
  }
}

}  // namespace

int* exo_tc_err_ptr();

// Splits per (token, head group): enough CTAs for a few waves over the 148 SMs.
EXO_API int exo_mla_attn_splits(int n_ctas_unsplit, int max_len) {
  const int nb = (max_len + BN - 1) / BN;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 32 && s <= nb; s++) {
    const long ctas = (long)n_ctas_unsplit * s;
    const double rounds = (double)((ctas + 147) / 148);
    const double cost = rounds * ((nb + s - 1) / s + 1.0);      // one block-time of fixed cost per CTA
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  return best;
}

EXO_API long exo_mla_attn_workspace(int T, int H, int ns) { return (long)T * H * ns * (LAT + 2) + 64; }

// q [T, H, 576] bf16 in cache space (see exo_mla_q_absorb), cache [n_blocks, 16, 576] bf16, out [T, H, 512].
// cu_q / tok_seq null: decode (token t is sequence t).  ns > 1 needs `workspace` (exo_mla_attn_workspace floats).
// Returns -2 for shapes this kernel does not take.
EXO_API int exo_mla_attn_tc(const void* q, const void* cache, const int* block_tables, const int* seq_lens, const int* cu_q,
                            const int* tok_seq, void* out, float* workspace, float scale, int T, int H,
                            int kv_lora, int rope_dim, int n_blocks, int max_blocks, int block_size, int ns,
                            cudaStream_t st) {
  if (T <= 0) return 0;
  if (kv_lora != LAT || rope_dim != ROPE || block_size != PAGE || ns < 1 || ns > 32) return -2;
  int G = H;
  if (H >= NQ) {
    if (H % NQ) return -2;
    G = NQ;
  } else if (H != 1 && H != 2 && H != 4 && H != 8) {
    return -2;
  }
  const int groups = H / G;
  int* err = exo_tc_err_ptr();
  if (!err) return -4;
  const CUtensorMap* tq = exo_tmap_2d_bf16(q, (uint64_t)T * H, (uint64_t)DQK, NQ);
  const CUtensorMap* tcm = exo_tmap_2d_bf16(cache, (uint64_t)n_blocks * PAGE, (uint64_t)DQK, PAGE);
  if (!tq || !tcm) return -5;
  const size_t smem = sizeof(Smem) + 1024;
  Params p;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = cu_q; p.tok_seq = tok_seq;
  p.out = (__nv_bfloat16*)out;
  p.part_o = workspace; p.part_ml = workspace ? workspace + (size_t)T * H * ns * LAT : nullptr;
  p.err = err; p.scale_log2 = scale * 1.4426950408889634f;
  p.H = H; p.groups = groups; p.max_blocks = max_blocks; p.ns = ns;
  if (ns > 1 && !workspace) return -2;
  dim3 grid(ns, groups, T);
  cudaError_t e = cudaSuccess;
#define LAUNCH(GG)                                                                                                \
  do {                                                                                                            \
    static bool attr_set = false;                                                                                 \
    if (!attr_set) {                                                                                              \
      if (cudaFuncSetAttribute(mla_attn_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=    \
          cudaSuccess)                                                                                            \
        return -3;                                                                                                \
      attr_set = true;                                                                                            \
    }                                                                                                             \
    e = launch_pdl(mla_attn_kernel<GG>, grid, dim3(128), smem, st, *tq, *tcm, p);                                 \
  } while (0)
  switch (G) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    case 8: LAUNCH(8); break;
    default: LAUNCH(16); break;
  }
#undef LAUNCH
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  if (ns > 1) {
    e = launch_pdl(mla_merge_kernel, dim3(T * H), dim3(128), 0, st, (const float*)p.part_o, (const float*)p.part_ml,
                   (__nv_bfloat16*)out, ns);
    if (e != cudaSuccess) return (int)e;
    EXO_CHECK_LAUNCH();
  }
  return 0;
}

// kv_a [T, 576] -> cache rows at `slots` (RMSNorm of the latent part, RoPE of the rope part).
EXO_API int exo_mla_kv_append(const void* kva, const void* norm_w, float eps, const int* positions, const float* inv_freq,
                              float mscale, void* cache, const int* slots, int T, int kv_lora, int rope_dim,
                              cudaStream_t st) {
  if (T <= 0) return 0;
  if (kv_lora != LAT || rope_dim != ROPE) return -2;
  EXO_REQUIRE_ALIGNED16(kva); EXO_REQUIRE_ALIGNED16(norm_w); EXO_REQUIRE_ALIGNED16(cache);
  cudaError_t e = launch_pdl(mla_kv_append_kernel, dim3(T), dim3(128), 0, st, (const __nv_bfloat16*)kva,
                             (const __nv_bfloat16*)norm_w, eps, positions, inv_freq, mscale, (__nv_bfloat16*)cache, slots, T);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// q [T, H, 192] (128 nope + 64 rope) and W_UK [H, 128, 512] -> out [T, H, 576].  Meant for decode batches
// (every block walks all T tokens).  rope_only: just out[..., 512:576] = RoPE(q[..., 128:192]); the latent part is
// then the caller's (prefill chunks run it as tensor-core GEMMs per head).
EXO_API int exo_mla_q_absorb(const void* q, const void* w_uk, const int* positions, const float* inv_freq, float mscale,
                             void* out, int T, int H, int nope, int kv_lora, int rope_dim, int rope_only, cudaStream_t st) {
  if (T <= 0) return 0;
  if (nope != 128 || kv_lora != LAT || rope_dim != ROPE) return -2;
  cudaError_t e = launch_pdl(mla_q_absorb_kernel, dim3(H, rope_only ? 1 : 9), dim3(256), 0, st, (const __nv_bfloat16*)q,
                             (const __nv_bfloat16*)w_uk, positions, inv_freq, mscale, (__nv_bfloat16*)out, T, H, rope_only);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// o_lat [T, H, 512] and W_UV [H, 128, 512] -> out [T, H, 128].  Decode batches (T <= 64).
EXO_API int exo_mla_o_absorb(const void* o_lat, const void* w_uv, void* out, int T, int H, int v_dim, int kv_lora,
                             cudaStream_t st) {
  if (T <= 0) return 0;
  if (v_dim != 128 || kv_lora != LAT) return -2;
  EXO_REQUIRE_ALIGNED16(o_lat); EXO_REQUIRE_ALIGNED16(w_uv);
  cudaError_t e = launch_pdl(mla_o_absorb_kernel, dim3(H, 16), dim3(256), 0, st, (const __nv_bfloat16*)o_lat,
                             (const __nv_bfloat16*)w_uv, (__nv_bfloat16*)out, T, H);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}
