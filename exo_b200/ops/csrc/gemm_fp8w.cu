// Linear layer with block-scaled fp8 (e4m3) weights and bf16 activations on the tcgen05 tensor cores:
//   out[M, N] = x[M, K] . bf16(Wq[N, K] * scale)^T  (+bias)(+residual)
//
// The weight bytes are what decode is bound by, so they cross HBM once, as fp8.  The CTA has the
// roles of the bf16 GEMM (warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = epilogue) plus four
// more warps; warps 2..9 work during the main loop as converters (two threads per weight row): the weights are stored tiled (each 128x64 block
// contiguous, its scales behind it), so one bulk copy per stage brings a raw tile and its scales as
// 8448 consecutive DRAM bytes, next to the TMA load of the activation tile; thread r of the four warps turns row r of a raw tile into 64 bf16
// values — the e4m3 bit pattern is re-based into a bf16 pattern with two logic ops per pair and one
// packed bf16 multiply applies the block scale together with the exponent re-bias — and stores them
// in the 128-byte-swizzled layout the MMA reads.  A second, shorter ring holds the converted tiles.
// Scales: one e8m0 byte per 32 weights of a row ("mxfp8"), or one fp32 per 128x128 block ("dsfp8").
//
// The accumulator read-back, split-K and hand-over epilogue is the bf16 kernel's.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

#include "fp8_convert.cuh"
#include "gemm_common.cuh"

int exo_gemm_scratch(int** err, int** counters, float** partial, size_t* partial_floats);

namespace {

using gemm::BK;
using gemm::BM;
using gemm::GemmParams;
using namespace fp8cvt;

struct ScaleParams {
  const uint8_t* tiles;   // [ceil(N/128), kt, TILE_BYTES]
  int kind;               // 1 = e8m0 per 1x32, 2 = fp32 per tile
  int kt;                 // tiles along K
};

template <int BN, int RS, int AS>
struct SmemF {
  alignas(1024) __nv_bfloat16 a[AS][BM * BK];
  alignas(1024) __nv_bfloat16 b[RS][BN * BK];
  alignas(128) uint8_t raw[RS][TILE_BYTES];
  uint64_t raw_full[RS], raw_empty[RS], a_full[AS], a_empty[AS], acc_full;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

template <int BN, int RS, int AS>
__global__ void __launch_bounds__(320, (BN <= 64 ? 2 : 1))
gemm_fp8w_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p, const ScaleParams sp) {
  extern __shared__ uint8_t smem_raw[];
  using S = SmemF<BN, RS, AS>;
  S& s = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t STAGE_BYTES = TILE_BYTES + BN * BK * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN, split = blockIdx.z;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb0 = split * p.kb_per_split;
  const int nkb = min(p.kb_per_split, kb_total - kb0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < RS; i++) { tc::mbar_init(&s.raw_full[i], 1); tc::mbar_init(&s.raw_empty[i], 1); }
    for (int i = 0; i < AS; i++) { tc::mbar_init(&s.a_full[i], 256); tc::mbar_init(&s.a_empty[i], 1); }
    tc::mbar_init(&s.acc_full, 1);
    s.abort_flag = 0;
    s.is_last = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = s.tmem_base;

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::prefetch_tmap(&tmap_x);
      const uint8_t* wt = sp.tiles + ((size_t)blockIdx.x * sp.kt + kb0) * TILE_BYTES;
      for (int i = 0; i < nkb; i++) {
        const int rs = i % RS;
        if (i >= RS && !tc::mbar_wait(&s.raw_empty[rs], ((i / RS) - 1) & 1)) {
          atomicExch(p.err, tc::ERR_EMPTY_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&s.raw_full[rs], STAGE_BYTES);
        const int k = (kb0 + i) * BK;
        bulk_g2s(tc::smem_u32(s.raw[rs]), wt + (size_t)i * TILE_BYTES, TILE_BYTES, tc::smem_u32(&s.raw_full[rs]));
        tc::tma_load_2d(s.b[rs], &tmap_x, k, m0, &s.raw_full[rs]);
      }
    }
  } else if (warp == 1) {
    if (tc::elect_one()) {
      constexpr uint32_t idesc = tc::umma_idesc_bf16(BM, BN);
      for (int i = 0; i < nkb; i++) {
        const int rs = i % RS, as = i % AS;
        if (!tc::mbar_wait(&s.a_full[as], (i / AS) & 1) || !tc::mbar_wait(&s.raw_full[rs], (i / RS) & 1)) {
          atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::tc_fence_after();
        const uint64_t ad = tc::umma_desc_sw128(tc::smem_u32(s.a[as]));
        const uint64_t bd = tc::umma_desc_sw128(tc::smem_u32(s.b[rs]));
#pragma unroll
        for (int k = 0; k < BK / 16; k++) tc::umma_bf16(tmem, ad + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
        tc::umma_commit(&s.a_empty[as]);
        tc::umma_commit(&s.raw_empty[rs]);
      }
      tc::umma_commit(&s.acc_full);
    }
  } else {
    // ---- converters: thread c of 256 takes half h = c / 128 of row r = c % 128 of every raw tile ----
    const int c = threadIdx.x - 64, r = c & 127, h = c >> 7;
    for (int i = 0; i < nkb; i++) {
      const int rs = i % RS, as = i % AS;
      if (!tc::mbar_wait_backoff(&s.raw_full[rs], (i / RS) & 1, 32, 1u << 24) ||
          (i >= AS && !tc::mbar_wait_backoff(&s.a_empty[as], ((i / AS) - 1) & 1, 32, 1u << 24))) {
        atomicExch(p.err, tc::ERR_TILE_TIMEOUT);
        s.abort_flag = 1;
        break;
      }
      tc::tc_fence_after();
      uint32_t c_lo, c_hi;
      tile_scales(tc::smem_u32(s.raw[rs]), sp.kind, r, c_lo, c_hi);
      convert_half_row(tc::smem_u32(s.raw[rs]), tc::smem_u32(s.a[as]), r, h, h ? c_hi : c_lo);
      tc::fence_proxy_async();       // the MMA reads these stores through the async proxy
      tc::mbar_arrive(&s.a_full[as]);
    }
    if (warp < 6)     // warps 2..5 own the four TMEM lane quadrants
    gemm::epilogue<BN>(p, tmem, &s.acc_full, &s.abort_flag, &s.is_last, n0, m0, split, nkb, warp, lane);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---- A operand in tensor memory -----------------------------------------------------------------
// The widened weights need not go back through shared memory: the MMA can take its A operand from
// tensor memory (row i of the [128 x 16] operand on lane i, two bf16 per 32-bit column), which is
// exactly how the converter threads hold them — thread (quadrant, lane) owns weight row
// 32*quadrant + lane.  So a converter loads its half row from the raw tile, widens it in registers
// and writes 16 columns with one tcgen05.st; no swizzled store, no proxy fence, and the MMA reads
// only the activation tile from shared memory.  Per K block the shared-memory traffic drops from
// ~57 KB to ~24 KB (BN = 32), which is what bounded the shared-memory form.
template <int BN, int RS>
struct SmemFT {
  alignas(1024) __nv_bfloat16 b[RS][BN * BK];
  alignas(128) uint8_t raw[RS][TILE_BYTES];
  uint64_t raw_full[RS], raw_empty[RS], a_full[4], a_empty[4], acc_full;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ void tmem_st16u(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"((uint32_t)acc)
      : "memory");
}

// F16: both MMA operands are f16 (the activations arrive converted, the weights are widened with the hardware
// e4m3 -> f16 converter): half the widening instructions of the bf16 form.
// HO: the output leaves for every rank's hand-over slot as flag-in-data words (row-parallel projection of a decode
// step under tensor parallelism, see tp_handover.cuh) instead of being stored to `out`.
template <int BN, int RS, bool F16, bool HO = false>
__global__ void __launch_bounds__(320, (BN <= 64 ? 2 : 1))
gemm_fp8w_ta_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p, const ScaleParams sp) {
  extern __shared__ uint8_t smem_raw[];
  using S = SmemFT<BN, RS>;
  S& s = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int AS = 4;                                    // A stages in tensor memory, 32 columns each
  constexpr uint32_t A_COL = BN < 32 ? 32 : BN;            // accumulator first, then the A ring
  constexpr uint32_t NEED = A_COL + AS * 32;
  constexpr uint32_t TMEM_COLS = NEED <= 64 ? 64 : NEED <= 128 ? 128 : NEED <= 256 ? 256 : 512;
  constexpr uint32_t STAGE_BYTES = TILE_BYTES + BN * BK * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN, split = blockIdx.z;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb0 = split * p.kb_per_split;
  const int nkb = min(p.kb_per_split, kb_total - kb0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < RS; i++) {
      tc::mbar_init(&s.raw_full[i], 1);
      tc::mbar_init(&s.raw_empty[i], 1);
    }
    for (int i = 0; i < AS; i++) { tc::mbar_init(&s.a_full[i], 256); tc::mbar_init(&s.a_empty[i], 1); }
    tc::mbar_init(&s.acc_full, 1);
    s.abort_flag = 0;
    s.is_last = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = s.tmem_base;

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::prefetch_tmap(&tmap_x);
      const uint8_t* wt = sp.tiles + ((size_t)blockIdx.x * sp.kt + kb0) * TILE_BYTES;
      for (int i = 0; i < nkb; i++) {
        const int rs = i % RS;
        if (i >= RS && !tc::mbar_wait(&s.raw_empty[rs], ((i / RS) - 1) & 1)) {
          atomicExch(p.err, tc::ERR_EMPTY_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&s.raw_full[rs], STAGE_BYTES);
        bulk_g2s(tc::smem_u32(s.raw[rs]), wt + (size_t)i * TILE_BYTES, TILE_BYTES, tc::smem_u32(&s.raw_full[rs]));
        tc::tma_load_2d(s.b[rs], &tmap_x, (kb0 + i) * BK, m0, &s.raw_full[rs]);
      }
    }
  } else if (warp == 1) {
    if (tc::elect_one()) {
      // kind::f16 descriptor: operand formats 1 = bf16, 0 = f16 (bits 7..9 and 10..12); fp32 accumulation either way
      constexpr uint32_t idesc = F16 ? (tc::umma_idesc_bf16(BM, BN) & ~((1u << 7) | (1u << 10))) : tc::umma_idesc_bf16(BM, BN);
      for (int i = 0; i < nkb; i++) {
        const int rs = i % RS, as = i % AS;
        if (!tc::mbar_wait(&s.a_full[as], (i / AS) & 1) || !tc::mbar_wait(&s.raw_full[rs], (i / RS) & 1)) {
          atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::tc_fence_after();
        const uint64_t bd = tc::umma_desc_sw128(tc::smem_u32(s.b[rs]));
        const uint32_t a_t = tmem + A_COL + as * 32;
#pragma unroll
        for (int k = 0; k < BK / 16; k++) umma_bf16_ts(tmem, a_t + 8 * k, bd + 2 * k, idesc, (i | k) != 0);
        tc::umma_commit(&s.a_empty[as]);
        tc::umma_commit(&s.raw_empty[rs]);   // the raw bytes were consumed before a_full; the activation tile only now
      }
      tc::umma_commit(&s.acc_full);
    }
  } else {
    // converters: warp w works on lane quadrant w % 4 (the only TMEM lanes it may touch); warps 2..5 take the first
    // 32 weights of their rows' K block, warps 6..9 the second 32
    const int quad = warp & 3, h = (warp - 2) >> 2, r = quad * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + A_COL + 16 * h;
    for (int i = 0; i < nkb; i++) {
      const int rs = i % RS, as = i % AS;
      if (!tc::mbar_wait_backoff(&s.raw_full[rs], (i / RS) & 1, 32, 1u << 24) ||
          (i >= AS && !tc::mbar_wait_backoff(&s.a_empty[as], ((i / AS) - 1) & 1, 32, 1u << 24))) {
        atomicExch(p.err, tc::ERR_TILE_TIMEOUT);
        s.abort_flag = 1;
        break;
      }
      tc::tc_fence_after();
      const uint32_t raw = tc::smem_u32(s.raw[rs]);
      uint32_t c_lo, c_hi;
      if constexpr (F16) tile_scales_f16(raw, sp.kind, r, c_lo, c_hi);
      else tile_scales(raw, sp.kind, r, c_lo, c_hi);
      const uint32_t c2 = h ? c_hi : c_lo;
      const uint4 w0 = lds16(raw + r * 64 + h * 32 + ((r >> 1) & 1) * 16);
      const uint4 w1 = lds16(raw + r * 64 + h * 32 + (((r >> 1) & 1) ^ 1) * 16);
      const uint4 lo = ((r >> 1) & 1) ? w1 : w0, hi = ((r >> 1) & 1) ? w0 : w1;     // bytes 0..15 / 16..31 of the half row
      uint32_t o[16];
      if constexpr (F16) {
        cvt4_f16(lo.x, c2, o[0], o[1]); cvt4_f16(lo.y, c2, o[2], o[3]); cvt4_f16(lo.z, c2, o[4], o[5]); cvt4_f16(lo.w, c2, o[6], o[7]);
        cvt4_f16(hi.x, c2, o[8], o[9]); cvt4_f16(hi.y, c2, o[10], o[11]); cvt4_f16(hi.z, c2, o[12], o[13]); cvt4_f16(hi.w, c2, o[14], o[15]);
      } else {
        const uint4 o0 = cvt8(lo.x, lo.y, c2), o1 = cvt8(lo.z, lo.w, c2), o2 = cvt8(hi.x, hi.y, c2), o3 = cvt8(hi.z, hi.w, c2);
        o[0] = o0.x; o[1] = o0.y; o[2] = o0.z; o[3] = o0.w; o[4] = o1.x; o[5] = o1.y; o[6] = o1.z; o[7] = o1.w;
        o[8] = o2.x; o[9] = o2.y; o[10] = o2.z; o[11] = o2.w; o[12] = o3.x; o[13] = o3.y; o[14] = o3.z; o[15] = o3.w;
      }
      tmem_st16u(lane_base + as * 32, o);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc::tc_fence_before();
      tc::mbar_arrive(&s.a_full[as]);
    }
    if (warp < 6)     // warps 2..5 own the four TMEM lane quadrants of the accumulator
      gemm::epilogue<BN, HO>(p, tmem, &s.acc_full, &s.abort_flag, &s.is_last, n0, m0, split, nkb, warp, lane);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int BN, int RS, bool F16, bool HO = false>
int launch_fp8w_ta_t(const CUtensorMap* tx, const GemmParams& p, const ScaleParams& sp, cudaStream_t st) {
  using S = SmemFT<BN, RS>;
  const size_t smem = sizeof(S) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8w_ta_kernel<BN, RS, F16, HO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  dim3 grid((p.N + BM - 1) / BM, (p.M + BN - 1) / BN, p.splits);
  gemm_fp8w_ta_kernel<BN, RS, F16, HO><<<grid, 320, smem, st>>>(*tx, p, sp);
  EXO_CHECK_LAUNCH();
  return 0;
}
template <int BN, int RS>
int launch_fp8w_ta(const CUtensorMap* tx, const GemmParams& p, const ScaleParams& sp, bool f16, cudaStream_t st) {
  if (p.ho.n_ll > 0) {
    if constexpr (BN <= 64)       // hand-overs are decode batches
      return f16 ? launch_fp8w_ta_t<BN, RS, true, true>(tx, p, sp, st) : launch_fp8w_ta_t<BN, RS, false, true>(tx, p, sp, st);
    else
      return -2;
  }
  return f16 ? launch_fp8w_ta_t<BN, RS, true>(tx, p, sp, st) : launch_fp8w_ta_t<BN, RS, false>(tx, p, sp, st);
}

// x bf16 -> f16 (saturating), for the f16-operand form of the GEMM
__global__ void bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ y, long n8) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float f[8];
  unpack8(reinterpret_cast<const uint4*>(x)[i], f);
  uint4 o;
  __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int j = 0; j < 4; j++)
    h[j] = __floats2half2_rn(fminf(fmaxf(f[2 * j], -65504.f), 65504.f), fminf(fmaxf(f[2 * j + 1], -65504.f), 65504.f));
  reinterpret_cast<uint4*>(y)[i] = o;
}

template <int BN, int RS, int AS>
int launch_fp8w(const CUtensorMap* tx, const GemmParams& p, const ScaleParams& sp, cudaStream_t st) {
  using S = SmemF<BN, RS, AS>;
  const size_t smem = sizeof(S) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8w_kernel<BN, RS, AS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  dim3 grid((p.N + BM - 1) / BM, (p.M + BN - 1) / BN, p.splits);
  gemm_fp8w_kernel<BN, RS, AS><<<grid, 320, smem, st>>>(*tx, p, sp);
  EXO_CHECK_LAUNCH();
  return 0;
}

}  // namespace

// `tiles`: the weight in the tiled form [ceil(N/128), ceil(K/64), 8448]; scale_kind 1 = e8m0 per 1x32, 2 = fp32 per tile.
EXO_API int exo_bf16_to_f16(const void* x, void* y, long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  bf16_to_f16_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__half*)y, n / 8);
  EXO_CHECK_LAUNCH();
  return 0;
}

static int gemm_fp8w_impl(const void* x, const void* tiles, int scale_kind, const void* bias, const void* residual, void* out,
                          int M, int N, int K, int ldo, int splits, bool x_f16, cudaStream_t st, const TpHandover* ho = nullptr);

EXO_API int exo_gemm_fp8w(const void* x, const void* tiles, int scale_kind, const void* bias,
                          const void* residual, void* out, int M, int N, int K, int ldo, int splits, cudaStream_t st) {
  return gemm_fp8w_impl(x, tiles, scale_kind, bias, residual, out, M, N, K, ldo, splits, false, st);
}
// Row-parallel projection of a decode batch (M <= 64) under tensor parallelism: the [M, N] output goes to every rank's
// hand-over slot as flag-in-data words (see tp_handover.cuh); N even.  x_f16: the activations are f16 (as below).
EXO_API int exo_gemm_fp8w_tp(const void* x, const void* tiles, int scale_kind, const void* bias, int M, int N, int K,
                             int splits, int parity, int x_f16, cudaStream_t st) {
  if ((N & 1) || M > 64) return -2;
  TpHandover ho;
  int rc = exo_tp_handover_fill(&ho, 3, parity, (long)((M + 1) & ~1) * N);
  if (rc) return rc;
  return gemm_fp8w_impl(x, tiles, scale_kind, bias, nullptr, nullptr, M, N, K, N, splits, x_f16 != 0, st, &ho);
}
// The same with f16 activations `x16` (see exo_bf16_to_f16): both MMA operands f16.
EXO_API int exo_gemm_fp8w_f16(const void* x16, const void* tiles, int scale_kind, const void* bias,
                              const void* residual, void* out, int M, int N, int K, int ldo, int splits, cudaStream_t st) {
  return gemm_fp8w_impl(x16, tiles, scale_kind, bias, residual, out, M, N, K, ldo, splits, true, st);
}

static int gemm_fp8w_impl(const void* x, const void* tiles, int scale_kind, const void* bias, const void* residual, void* out,
                          int M, int N, int K, int ldo, int splits, bool x_f16, cudaStream_t st, const TpHandover* ho) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || K < BK || (scale_kind != 1 && scale_kind != 2) || ((uintptr_t)tiles & 15)) return -2;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  size_t partial_floats = 0;
  if (exo_gemm_scratch(&p.err, &p.counters, &p.partial, &partial_floats)) return -4;
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const CUtensorMap* tx = exo_tmap_2d_bf16(x, M, K, bn);
  if (!tx) return -5;
  p.M = M; p.N = N; p.K = K;
  const int kb_total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  p.kb_per_split = (kb_total + splits - 1) / splits;
  splits = (kb_total + p.kb_per_split - 1) / p.kb_per_split;
  p.splits = splits;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.out = (__nv_bfloat16*)out;
  p.ldo = ldo;
  if (ho) p.ho = *ho; else memset(&p.ho, 0, sizeof(p.ho));
  p.row_flags = nullptr; p.row_epoch = nullptr; p.rows_per_flag = 1; p.m_tile_shift = 0; p.gate_wait_ns = 0; p.gate_status = nullptr;
  if (splits > 1) {
    const long tiles = (long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    if ((size_t)splits * M * N > partial_floats || tiles > (1 << 16)) return -6;
  }
  ScaleParams sp;
  sp.tiles = (const uint8_t*)tiles;
  sp.kind = scale_kind;
  sp.kt = kb_total;
  static int smem_a = -1;
  if (smem_a < 0) { const char* e = getenv("EXO_FP8_SMEM_A"); smem_a = (e && e[0] == '1') ? 1 : 0; }
  if (!smem_a || x_f16 || ho) {      // A operand from tensor memory (default); EXO_FP8_SMEM_A=1 selects the shared-memory form below
    switch (bn) {
      case 16: return launch_fp8w_ta<16, 8>(tx, p, sp, x_f16, st);     // 8 x (8.25 + 2) KB
      case 32: return launch_fp8w_ta<32, 8>(tx, p, sp, x_f16, st);     // 8 x (8.25 + 4) KB
      case 64: return launch_fp8w_ta<64, 6>(tx, p, sp, x_f16, st);     // 6 x (8.25 + 8) KB
      case 128: return launch_fp8w_ta<128, 6>(tx, p, sp, x_f16, st);   // 6 x (8.25 + 16) KB
      default: return launch_fp8w_ta<256, 4>(tx, p, sp, x_f16, st);    // 4 x (8.25 + 32) KB
    }
  }
  switch (bn) {
    // decode shapes: two CTAs per SM (eight converter warps hide each other's latencies)
    case 16: return launch_fp8w<16, 6, 2>(tx, p, sp, st);     // 32 + 12 + 48 KB
    case 32: return launch_fp8w<32, 6, 2>(tx, p, sp, st);     // 32 + 24 + 48 KB
    case 64: return launch_fp8w<64, 4, 2>(tx, p, sp, st);     // 32 + 32 + 32 KB
    case 128: return launch_fp8w<128, 4, 3>(tx, p, sp, st);   // 48 + 64 + 32 KB
    default: return launch_fp8w<256, 4, 2>(tx, p, sp, st);    // 32 + 128 + 32 KB
  }
}
