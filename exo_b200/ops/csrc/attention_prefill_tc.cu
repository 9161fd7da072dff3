// Prefill attention on the 5th-generation tensor cores: ragged causal flash attention over the
// paged KV cache.
//
// One CTA = 128 query rows of one sequence x one query head.  Q (128 x 128 bf16) is brought in
// once by TMA; the keys and values of the sequence are walked in blocks of 128 keys, each block
// gathered page by page (16 keys per page) with TMA tile loads straight out of the KV pool into
// 128-byte-swizzled shared memory, double buffered.  Per block:
//   S = Q K^T        tcgen05.mma, both operands K-major, accumulator in TMEM columns [0,128)
//   softmax          every thread owns one query row (= one TMEM lane): tcgen05.ld, running
//                    max / sum in the exp2 domain, causal + length (+ sliding window) mask,
//                    P written as bf16 into swizzled shared memory
//   O += P V         tcgen05.mma with V as an MN-major B operand (the pool keeps V as
//                    [key][dim], which is exactly the MN-major 128B-swizzle atom),
//                    accumulator in TMEM columns [128,256), rescaled in place (tcgen05.ld/st)
//                    only by warps in which some row's maximum moved
// Every mbarrier wait is bounded; on a timeout the kernel records a code, drains, frees its TMEM
// and returns.
#include <cuda_bf16.h>
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;         // query rows per CTA
constexpr int BN = 128;         // keys per block
constexpr int HD = 128;         // head dimension
constexpr int PAGE = 16;        // keys per KV page
constexpr uint32_t HALF = 128 * 128;      // bytes of a [128 rows x 64 bf16] half tile
constexpr uint32_t TILE = 2 * HALF;       // [128 x 128] bf16
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t S_COL = 0, O_COL = 128;

struct __align__(1024) Smem {
  uint8_t q[TILE];
  uint8_t k[2][TILE];
  uint8_t v[2][TILE];
  uint8_t p[TILE];
  uint64_t q_full, k_full[2], v_full[2], s_done, o_done;
  uint32_t tmem_base;
};

struct Params {
  const int* block_tables;   // [B, max_blocks]
  const int* seq_lens;       // [B] keys per sequence (after this step's append)
  const int* cu_q;           // [B+1] query row offsets
  __nv_bfloat16* out;        // [T, Hq, 128]
  int* err;
  float scale_log2;          // softmax scale * log2(e)
  int B, Hq, Hkv, max_blocks, window;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// V block as an MN-major B operand: rows = keys (K of the MMA) 128 B apart, 8-key groups 1024 B
// apart (SBO), the second 64 head-dims one half tile further (LBO).
__device__ __forceinline__ uint64_t umma_desc_v(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(HALF >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// 128 keys of one sequence -> one [128 x 128] tile: 8 pages x 2 column halves.  Pages past the
// sequence's last page re-read the last page (finite values; those keys are masked anyway).
__device__ __forceinline__ void load_kv_block(uint8_t* dst, const CUtensorMap* map, const int* table, int n_pages,
                                              int first_page, int kv_head, uint64_t* bar) {
  tc::mbar_expect_tx(bar, TILE);
#pragma unroll
  for (int pg = 0; pg < BN / PAGE; pg++) {
    int idx = first_page + pg;
    if (idx >= n_pages) idx = n_pages - 1;
    int page = table[idx];
    tc::tma_load_2d(dst + pg * (PAGE * 128), map, kv_head * HD, page * PAGE, bar);
    tc::tma_load_2d(dst + HALF + pg * (PAGE * 128), map, kv_head * HD + 64, page * PAGE, bar);
  }
}

__global__ void __launch_bounds__(128, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  // ---- which (sequence, 128-row tile) is this CTA? (uniform across the CTA) ----
  int t = blockIdx.x, seq = -1;
  for (int s = 0; s < p.B; s++) {
    int nt = (p.cu_q[s + 1] - p.cu_q[s] + BM - 1) / BM;
    if (t < nt) { seq = s; break; }
    t -= nt;
  }
  if (seq < 0) return;
  const int head = blockIdx.y, kv_head = head / (p.Hq / p.Hkv);
  const int q0 = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q0, kv_len = p.seq_lens[seq];
  const int row0 = t * BM;                                   // first row of the tile inside the sequence
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = row0 + tid;
  const bool row_valid = row < q_len;
  const int qpos = kv_len - q_len + row;                     // absolute position of this thread's query
  const int last_row = min(row0 + BM, q_len) - 1;
  const int k_end = min(kv_len, kv_len - q_len + last_row + 1);            // keys any row of the tile may see
  int k_begin = 0;
  if (p.window > 0) k_begin = max(0, (kv_len - q_len + row0) - p.window + 1);
  const int blk_lo = k_begin / BN, blk_hi = (k_end + BN - 1) / BN;        // key blocks [blk_lo, blk_hi)
  const int n_iter = blk_hi - blk_lo;
  const int n_pages = (kv_len + PAGE - 1) / PAGE;
  const int* table = p.block_tables + (size_t)seq * p.max_blocks;

  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  if (tid == 0) {
    tc::prefetch_tmap(&tmap_q);
    tc::prefetch_tmap(&tmap_k);
    tc::prefetch_tmap(&tmap_v);
    tc::mbar_init(&s.q_full, 1);
    tc::mbar_init(&s.k_full[0], 1);
    tc::mbar_init(&s.k_full[1], 1);
    tc::mbar_init(&s.v_full[0], 1);
    tc::mbar_init(&s.v_full[1], 1);
    tc::mbar_init(&s.s_done, 1);
    tc::mbar_init(&s.o_done, 1);
    tc::fence_barrier_init();
  }
  if (warp == 0) {
    tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 TMEM lanes

  constexpr uint32_t IDESC_S = tc::umma_idesc_bf16(BM, BN);
  constexpr uint32_t IDESC_PV = tc::umma_idesc_bf16(BM, HD) | (1u << 16);      // B operand MN-major
  bool failed = false;
  int pending_k[2] = {0, 0}, pending_v[2] = {0, 0};      // thread 0: loads issued and not yet waited for

  if (tid == 0 && n_iter > 0) {
    tc::mbar_expect_tx(&s.q_full, TILE);
    tc::tma_load_2d(s.q, &tmap_q, head * HD, q0 + row0, &s.q_full);
    tc::tma_load_2d(s.q + HALF, &tmap_q, head * HD + 64, q0 + row0, &s.q_full);
    load_kv_block(s.k[0], &tmap_k, table, n_pages, blk_lo * (BN / PAGE), kv_head, &s.k_full[0]);
    load_kv_block(s.v[0], &tmap_v, table, n_pages, blk_lo * (BN / PAGE), kv_head, &s.v_full[0]);
    pending_k[0] = pending_v[0] = 1;
    if (n_iter > 1) {
      load_kv_block(s.k[1], &tmap_k, table, n_pages, (blk_lo + 1) * (BN / PAGE), kv_head, &s.k_full[1]);
      pending_k[1] = 1;
    }
    if (!tc::mbar_wait(&s.q_full, 0)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
    // S(0) = Q K(0)^T
    if (!failed && !tc::mbar_wait(&s.k_full[0], 0)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
    pending_k[0] = 0;
    if (!failed) {
      tc::tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < HD / 16; ks++) {
        uint32_t off = (ks >> 2) * HALF + (ks & 3) * 32;
        tc::umma_bf16(tmem + S_COL, tc::umma_desc_sw128(tc::smem_u32(s.q) + off),
                      tc::umma_desc_sw128(tc::smem_u32(s.k[0]) + off), IDESC_S, ks > 0);
      }
      tc::umma_commit(&s.s_done);
    }
  }

  float m_run = -INFINITY, l_run = 0.f;
  for (int it = 0; it < n_iter; it++) {
    const int buf = it & 1;
    // ---- S(it) ready (this also means O += P V of the previous block has finished) ----
    if (!tc::mbar_wait(&s.s_done, it & 1)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
      break;
    }
    tc::tc_fence_after();
    if (tid == 0) {
      // K buffer `buf` and V buffer `buf^1` are free now: prefetch K(it+2) and V(it+1)
      if (it + 2 < n_iter) {
        load_kv_block(s.k[buf], &tmap_k, table, n_pages, (blk_lo + it + 2) * (BN / PAGE), kv_head, &s.k_full[buf]);
        pending_k[buf] = 1;
      }
      if (it + 1 < n_iter) {
        load_kv_block(s.v[buf ^ 1], &tmap_v, table, n_pages, (blk_lo + it + 1) * (BN / PAGE), kv_head, &s.v_full[buf ^ 1]);
        pending_v[buf ^ 1] = 1;
      }
    }
    // ---- softmax of this thread's row ----
    const int key0 = (blk_lo + it) * BN;
    int hi = min(qpos + 1, kv_len) - key0;                 // keys [lo, hi) of this block are visible to the row
    int lo = p.window > 0 ? max(0, qpos - p.window + 1 - key0) : 0;
    if (!row_valid) hi = 0;
    float m_blk = -INFINITY;
#pragma unroll
    for (int c = 0; c < BN / 32; c++) {
      float sv[32];
      tc::tmem_ld32(lane_addr + S_COL + c * 32, sv);
      tc::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i++) {
        int kk = c * 32 + i;
        if (kk >= lo && kk < hi) m_blk = fmaxf(m_blk, sv[i]);
      }
    }
    const float m_new = fmaxf(m_run, m_blk * p.scale_log2);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;      // a row with nothing visible yet
    const float alpha = m_run == -INFINITY ? (m_new == -INFINITY ? 1.f : 0.f) : ex2(m_run - m_use);
    float l_blk = 0.f;
#pragma unroll
    for (int c = 0; c < BN / 32; c++) {
      float sv[32];
      tc::tmem_ld32(lane_addr + S_COL + c * 32, sv);
      tc::tmem_ld_wait();
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        int kk = c * 32 + i;
        float p0 = (kk >= lo && kk < hi) ? ex2(sv[i] * p.scale_log2 - m_use) : 0.f;
        float p1 = (kk + 1 >= lo && kk + 1 < hi) ? ex2(sv[i + 1] * p.scale_log2 - m_use) : 0.f;
        __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
        l_blk += __low2float(b) + __high2float(b);           // sum what the MMA will actually see
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&b);
      }
      // P row: 32 keys = four 16-byte chunks, 128-byte swizzle (chunk index ^ (row & 7))
      uint8_t* prow = s.p + (c >> 1) * HALF + tid * 128;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        int chunk = ((c & 1) * 4 + q) ^ (tid & 7);
        *reinterpret_cast<uint4*>(prow + chunk * 16) =
            make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
      }
    }
    l_run = l_run * alpha + l_blk;
    m_run = m_new;
    // ---- rescale O where a maximum moved (warp-uniform decision) ----
    if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int c = 0; c < HD / 32; c++) {
        float ov[32];
        tc::tmem_ld32(lane_addr + O_COL + c * 32, ov);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) ov[i] *= alpha;
        tmem_st32(lane_addr + O_COL + c * 32, ov);
      }
      tmem_st_wait();
    }
    tc::fence_proxy_async();          // P (generic-proxy stores) -> visible to the MMA's async proxy
    tc::tc_fence_before();
    __syncthreads();
    if (tid == 0 && !failed) {
      tc::tc_fence_after();
      if (!tc::mbar_wait(&s.v_full[buf], (it >> 1) & 1)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
      pending_v[buf] = 0;
      if (!failed) {
        tc::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ks++) {       // 16 keys per MMA
          uint32_t aoff = (ks >> 2) * HALF + (ks & 3) * 32;
          tc::umma_bf16(tmem + O_COL, tc::umma_desc_sw128(tc::smem_u32(s.p) + aoff),
                        umma_desc_v(tc::smem_u32(s.v[buf]) + ks * 2048), IDESC_PV, it > 0 || ks > 0);
        }
        if (it + 1 < n_iter) {
          // S(it+1) = Q K(it+1)^T; every thread has finished reading S(it)
          if (!tc::mbar_wait(&s.k_full[buf ^ 1], ((it + 1) >> 1) & 1)) { failed = true; atomicExch(p.err, tc::ERR_FULL_TIMEOUT); }
          pending_k[buf ^ 1] = 0;
          if (!failed) {
            tc::tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) {
              uint32_t off = (ks >> 2) * HALF + (ks & 3) * 32;
              tc::umma_bf16(tmem + S_COL, tc::umma_desc_sw128(tc::smem_u32(s.q) + off),
                            tc::umma_desc_sw128(tc::smem_u32(s.k[buf ^ 1]) + off), IDESC_S, ks > 0);
            }
            tc::umma_commit(&s.s_done);
          }
        } else {
          tc::umma_commit(&s.o_done);
        }
      }
    }
  }

  // ---- epilogue: O / l -> out ----
  if (n_iter > 0 && !failed) {
    if (!tc::mbar_wait(&s.o_done, 0)) {
      if (tid == 0) atomicExch(p.err, tc::ERR_ACC_TIMEOUT);
      failed = true;
    }
  }
  tc::tc_fence_after();
  if (!failed) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* orow = p.out + ((size_t)(q0 + row) * p.Hq + head) * HD;
#pragma unroll
    for (int c = 0; c < HD / 32; c++) {
      float ov[32];
      if (n_iter > 0) {
        tc::tmem_ld32(lane_addr + O_COL + c * 32, ov);
        tc::tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; i++) ov[i] = 0.f;
      }
      if (row_valid) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 w;
          __nv_bfloat162 b0 = __floats2bfloat162_rn(ov[i] * inv, ov[i + 1] * inv);
          __nv_bfloat162 b1 = __floats2bfloat162_rn(ov[i + 2] * inv, ov[i + 3] * inv);
          __nv_bfloat162 b2 = __floats2bfloat162_rn(ov[i + 4] * inv, ov[i + 5] * inv);
          __nv_bfloat162 b3 = __floats2bfloat162_rn(ov[i + 6] * inv, ov[i + 7] * inv);
          w.x = *reinterpret_cast<uint32_t*>(&b0);
          w.y = *reinterpret_cast<uint32_t*>(&b1);
          w.z = *reinterpret_cast<uint32_t*>(&b2);
          w.w = *reinterpret_cast<uint32_t*>(&b3);
          *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
        }
      }
    }
  }
  // ---- unwind: let copies still in flight land, then give the TMEM back ----
  if (tid == 0 && failed) {
    for (int b = 0; b < 2; b++) {
      if (pending_k[b]) tc::mbar_wait(&s.k_full[b], 0, 1u << 16) || tc::mbar_wait(&s.k_full[b], 1, 1u << 16);
      if (pending_v[b]) tc::mbar_wait(&s.v_full[b], 0, 1u << 16) || tc::mbar_wait(&s.v_full[b], 1, 1u << 16);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace

int* exo_tc_err_ptr();   // the tensor-core kernels' shared device error word (set up by exo_gemm_init)

// q [T, Hq, 128] bf16; kcache / vcache [n_blocks, 16, Hkv, 128] bf16; out [T, Hq, 128] bf16.
// Returns 0, or <0 when this shape is not handled here (the caller then uses the generic kernel).
EXO_API int exo_prefill_attn_tc(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                                const int* seq_lens, const int* cu_q, void* out, float scale, int T, int B, int Hq, int Hkv,
                                int D, int n_blocks, int max_blocks, int block_size, int window, cudaStream_t st) {
  if (D != HD || block_size != PAGE || Hq % Hkv != 0 || T <= 0 || B <= 0) return -2;
  int* err = exo_tc_err_ptr();
  if (!err) return -4;
  // box rows: 128 query rows, 16 keys per page; 64 columns (128 bytes) wide
  const CUtensorMap* tq = exo_tmap_2d_bf16(q, (uint64_t)T, (uint64_t)Hq * HD, BM);
  const CUtensorMap* tk = exo_tmap_2d_bf16(kcache, (uint64_t)n_blocks * PAGE, (uint64_t)Hkv * HD, PAGE);
  const CUtensorMap* tv = exo_tmap_2d_bf16(vcache, (uint64_t)n_blocks * PAGE, (uint64_t)Hkv * HD, PAGE);
  if (!tq || !tk || !tv) return -5;
  size_t smem = sizeof(Smem) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  Params p;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = cu_q;
  p.out = (__nv_bfloat16*)out; p.err = err;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.max_blocks = max_blocks; p.window = window;
  dim3 grid((T + BM - 1) / BM + B, Hq);     // upper bound on the number of 128-row tiles; surplus CTAs exit at once
  prefill_attn_kernel<<<grid, 128, smem, st>>>(*tq, *tk, *tv, p);
  EXO_CHECK_LAUNCH();
  return 0;
}
