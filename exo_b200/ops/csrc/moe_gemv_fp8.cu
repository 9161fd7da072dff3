// Routed experts with block-scaled fp8 weights for a handful of tokens (decode at batch 1..4): two grouped GEMV kernels
// that stream the chosen experts' weight tiles straight from HBM on CUDA cores.
//
// At these sizes the grouped tensor-core GEMM has one 128-feature CTA per (expert, feature tile): a token that routes to
// one or two local experts keeps 16..32 CTAs busy, each with ~50 KB in flight, and the GPU idles at a few percent of its
// bandwidth.  Here a CTA takes 8 (gate/up) or 16 (down) features, its 8 warps split those rows and the reduction
// dimension between them and keep 16 weight tiles per warp in flight, two CTAs per SM, so that one local pair already
// covers the SMs.
//
//   gate/up   hs[pair, f] = silu(Wg[e][f] . x[t]) * (Wu[e][f] . x[t])          grid (F/8, pairs)
//   down      out[t, n]   = sum_s w[t, s] * (Wd[e_s][n] . hs[t*k + s])          grid (H/16, tokens)
//
// Weights are in the tiled storage of the fp8 GEMMs: [E, rows/128, K/64, 8448] bytes, a tile being 128 rows x 64 e4m3
// values (row-major) followed by its scales (mxfp8: one e8m0 byte per row and 32 values; dsfp8: one fp32 per tile).
// Pairs whose expert lives on another rank are skipped (their CTAs return; the down kernel leaves them out of the sum).
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int TILE_BYTES = 8448, TILE_BODY = 8192, TILE_ROWS = 128, TILE_K = 64;
constexpr int Q_ROWS = 16;          // output features per CTA of the down projection
constexpr int G_ROWS = 8;           // features per CTA of the gate/up projection (8 gate rows + 8 up rows)
constexpr int Q_THREADS = 256;
constexpr int Q_UNROLL = 16;        // weight tiles in flight per warp

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Activations wait in shared memory as f16, scaled by 1/64: a run of 16 products is then summed in packed f16 (the
// conversion e4m3 -> f16 is exact, and f16 -> f32 conversions, a quarter-rate instruction, would otherwise outnumber the
// multiply-adds), and 448 (the largest e4m3) times an activation outlier of a few hundred, eight times over, still
// stays far below the f16 maximum.  The runs themselves are added up in fp32.
constexpr float X_SCALE = 1.f / 64.f, X_UNSCALE = 64.f;

// sum over 16 e4m3 weights (one 16-byte piece of a tile row) times 16 activations
__device__ __forceinline__ float dot16(const uint4& w, const __half* __restrict__ x) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  const uint4 xa = *reinterpret_cast<const uint4*>(x), xb = *reinterpret_cast<const uint4*>(x + 8);
  const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
  __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(words[i] & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(words[i] >> 16), __NV_E4M3);
    a0 = __hfma2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&xw[2 * i]), a0);
    a1 = __hfma2(*reinterpret_cast<const __half2*>(&hi), *reinterpret_cast<const __half2*>(&xw[2 * i + 1]), a1);
  }
  const float2 f = __half22float2(__hadd2(a0, a1));
  return f.x + f.y;
}

// One weight tile's worth of work for a lane: 16 bytes of one of 8 neighbouring tile rows and the row's scale.
template <int KIND>
struct TilePiece {
  uint4 w;
  float s;
  __device__ __forceinline__ void load(const uint8_t* __restrict__ body, const uint8_t* __restrict__ tail, size_t off, bool on) {
    w = on ? ldg_stream16(body + off) : make_uint4(0, 0, 0, 0);
    if (KIND == 1) s = on ? __uint_as_float((uint32_t)__ldg(tail + off) << 23) : 0.f;       // e8m0: 2^(e - 127)
    else s = on ? __ldg(reinterpret_cast<const float*>(tail + off)) : 0.f;
  }
};

// Lane l of a warp works on row l / 4 of 8 neighbouring rows of a 128-row weight tile and on bytes [16 * (l % 4), +16)
// of every tile row; the caller adds the four lanes of a row.

// hs[pair, f] = silu(Wg[e][f] . x[t]) * (Wu[e][f] . x[t]).  A CTA takes 8 features of one pair: warp = (gate | up,
// quarter of the reduction dimension), 16 tiles in flight per warp.
template <int KIND>
__global__ void __launch_bounds__(Q_THREADS, 2)
moe_gemv8_gate_up_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w_gu, const int* __restrict__ ids,
                         int k, int H, int F, int expert_offset, int E, __nv_bfloat16* __restrict__ hs) {
  extern __shared__ __align__(16) __half q_smem[];
  __half* xs = q_smem;                             // [KT * 64] (zero beyond H), scaled by X_SCALE
  __shared__ float part[4][2][8];                  // [K quarter][gate | up][row]
  const int pair = blockIdx.y;
  const int e = ids[pair] - expert_offset;
  if (e < 0 || e >= E) return;
  const int KT = (H + TILE_K - 1) / TILE_K, NT = 2 * F / TILE_ROWS;
  const __nv_bfloat16* xr = x + (size_t)(pair / k) * H;
  for (int i = threadIdx.x; i < KT * TILE_K; i += Q_THREADS) xs[i] = __float2half_rn(i < H ? __bfloat162float(xr[i]) * X_SCALE : 0.f);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int up = warp & 1, kq = warp >> 1;
  const int f0 = blockIdx.x * G_ROWS;
  const int row0 = up ? F + f0 : f0;                                    // first of this warp's 8 rows of [2F]
  const int row = row0 % TILE_ROWS + (lane >> 2), c = lane & 3;
  const uint8_t* tiles = w_gu + ((size_t)e * NT + row0 / TILE_ROWS) * KT * TILE_BYTES;
  const uint8_t* body = tiles + row * TILE_K + c * 16;
  const uint8_t* tail = tiles + TILE_BODY + (KIND == 1 ? row * 2 + (c >> 1) : 0);
  const int q = (KT + 3) / 4, kt0 = min(KT, kq * q), kt1 = min(KT, kt0 + q);
  float acc = 0.f;
  for (int kt = kt0; kt < kt1; kt += Q_UNROLL) {
    TilePiece<KIND> p[Q_UNROLL];
#pragma unroll
    for (int u = 0; u < Q_UNROLL; u++) p[u].load(body, tail, (size_t)(kt + u) * TILE_BYTES, kt + u < kt1);
#pragma unroll
    for (int u = 0; u < Q_UNROLL; u++)
      if (kt + u < kt1) acc += p[u].s * dot16(p[u].w, xs + (kt + u) * TILE_K + c * 16);     // (the activations end at kt1 too)
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if ((lane & 3) == 0) part[kq][up][lane >> 2] = acc;
  __syncthreads();
  if (threadIdx.x < G_ROWS) {
    const int r = threadIdx.x, f = f0 + r;
    if (f < F) {
      const float g = (part[0][0][r] + part[1][0][r] + part[2][0][r] + part[3][0][r]) * X_UNSCALE;
      const float u = (part[0][1][r] + part[1][1][r] + part[2][1][r] + part[3][1][r]) * X_UNSCALE;
      hs[(size_t)pair * F + f] = __float2bfloat16_rn(silu_f(g) * u);
    }
  }
}

// out[t, n] = sum_s w[t, s] * (Wd[e_s][n] . hs[t*k + s]).  A CTA takes 16 output features of one token: warp = (8 rows,
// quarter of the reduction dimension) and walks the token's LOCAL pairs and its tiles of each as one sequence, 16 tiles
// in flight whatever the number of pairs.
constexpr int MAX_K = 32;

template <int KIND>
__global__ void __launch_bounds__(Q_THREADS, 2)
moe_gemv8_down_kernel(const __nv_bfloat16* __restrict__ hs, const uint8_t* __restrict__ w_down, const int* __restrict__ ids,
                      const float* __restrict__ weights, int k, int H, int F, int expert_offset, int E,
                      __nv_bfloat16* __restrict__ out) {
  extern __shared__ __align__(16) __half q_smem[];
  __half* hsm = q_smem;                            // [local pairs][KT * 64], scaled by X_SCALE
  __shared__ float part[4][2][8];                  // [K quarter][rows 0-7, 8-15][row]
  __shared__ int loc_e[MAX_K];
  __shared__ float loc_w[MAX_K];
  __shared__ int n_loc;
  const int t = blockIdx.y;
  const int KT = (F + TILE_K - 1) / TILE_K, NT = (H + TILE_ROWS - 1) / TILE_ROWS, KP = KT * TILE_K;
  if (threadIdx.x == 0) {
    int n = 0;
    for (int s = 0; s < k; s++) {
      const int e = ids[t * k + s] - expert_offset;
      if (e >= 0 && e < E) { loc_e[n] = e | (s << 16); loc_w[n] = weights[t * k + s]; n++; }
    }
    n_loc = n;
  }
  __syncthreads();
  const int n = n_loc;
  for (int j = 0; j < n; j++) {
    const __nv_bfloat16* src = hs + (size_t)(t * k + (loc_e[j] >> 16)) * F;
    for (int i = threadIdx.x; i < KP; i += Q_THREADS) hsm[j * KP + i] = __float2half_rn(i < F ? __bfloat162float(src[i]) * X_SCALE : 0.f);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = warp & 1, kq = warp >> 1;
  const int n0 = blockIdx.x * Q_ROWS + half * 8;                        // first of this warp's 8 output rows
  const int q = (KT + 3) / 4, kt0 = min(KT, kq * q), kt1 = min(KT, kt0 + q), tpw = kt1 - kt0;
  float acc = 0.f;
  if (n0 < H && tpw > 0) {
    const int row = n0 % TILE_ROWS + (lane >> 2), c = lane & 3;
    const size_t row_tile = (size_t)(n0 / TILE_ROWS) * KT * TILE_BYTES, per_expert = (size_t)NT * KT * TILE_BYTES;
    const uint8_t* body0 = w_down + row_tile + row * TILE_K + c * 16;
    const uint8_t* tail0 = w_down + row_tile + TILE_BODY + (KIND == 1 ? row * 2 + (c >> 1) : 0);
    const int total = n * tpw;
    int lj = 0, lk = 0;                                                 // (local pair, tile within this warp's quarter) of item j0
    for (int j0 = 0; j0 < total; j0 += Q_UNROLL) {
      TilePiece<KIND> p[Q_UNROLL];
      int pj[Q_UNROLL], pk[Q_UNROLL];
#pragma unroll
      for (int u = 0; u < Q_UNROLL; u++) {
        const bool on = j0 + u < total;
        pj[u] = lj;
        pk[u] = kt0 + lk;
        const size_t off = on ? (size_t)(loc_e[lj] & 0xffff) * per_expert + (size_t)(kt0 + lk) * TILE_BYTES : 0;
        p[u].load(body0, tail0, off, on);
        if (++lk == tpw) { lk = 0; lj++; }
      }
#pragma unroll
      for (int u = 0; u < Q_UNROLL; u++)
        if (j0 + u < total) acc += loc_w[pj[u]] * p[u].s * dot16(p[u].w, hsm + pj[u] * KP + pk[u] * TILE_K + c * 16);
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if ((lane & 3) == 0) part[kq][half][lane >> 2] = acc;
  __syncthreads();
  if (threadIdx.x < Q_ROWS) {
    const int r = threadIdx.x, nn = blockIdx.x * Q_ROWS + r;
    if (nn < H)
      out[(size_t)t * H + nn] = __float2bfloat16_rn((part[0][r >> 3][r & 7] + part[1][r >> 3][r & 7] + part[2][r >> 3][r & 7] +
                                                     part[3][r >> 3][r & 7]) * X_UNSCALE);
  }
}

}  // namespace

// x [T, H] bf16, ids [T, k] (global expert ids), weights [T, k] fp32, hs [T*k, F] bf16 scratch, out [T, H] bf16 (every
// row written: zeros where no expert of the token is local).  w_gate_up / w_down: tiled fp8 storage of E local experts;
// scale_kind 1 (e8m0 per row and 32 values) or 2 (fp32 per tile).  F must be a multiple of 128 (gate rows and up rows
// start on tile boundaries), H of 8.
EXO_API int exo_moe_experts_gemv_fp8(const void* x, const void* w_gate_up, const void* w_down, const void* weights, const void* ids,
                                     void* out, void* hs, int T, int k, int H, int F, int E, int expert_offset, int scale_kind,
                                     cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % TILE_ROWS || H % 8 || k > MAX_K || E > 65535 || (scale_kind != 1 && scale_kind != 2)) return -2;
  const size_t sm1 = (size_t)((H + TILE_K - 1) / TILE_K) * TILE_K * sizeof(__half);
  const size_t sm2 = (size_t)k * ((F + TILE_K - 1) / TILE_K) * TILE_K * sizeof(__half);
  if (sm1 > 200 * 1024 || sm2 > 200 * 1024) return -2;
  static bool opted = false;
  if (!opted) {
    if (cudaFuncSetAttribute(moe_gemv8_gate_up_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(moe_gemv8_gate_up_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(moe_gemv8_down_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(moe_gemv8_down_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return -3;
    opted = true;
  }
  const dim3 g1((F + G_ROWS - 1) / G_ROWS, T * k), g2((H + Q_ROWS - 1) / Q_ROWS, T);
  if (scale_kind == 1) {
    moe_gemv8_gate_up_kernel<1><<<g1, Q_THREADS, sm1, st>>>((const __nv_bfloat16*)x, (const uint8_t*)w_gate_up, (const int*)ids, k, H,
                                                            F, expert_offset, E, (__nv_bfloat16*)hs);
    moe_gemv8_down_kernel<1><<<g2, Q_THREADS, sm2, st>>>((const __nv_bfloat16*)hs, (const uint8_t*)w_down, (const int*)ids,
                                                         (const float*)weights, k, H, F, expert_offset, E, (__nv_bfloat16*)out);
  } else {
    moe_gemv8_gate_up_kernel<2><<<g1, Q_THREADS, sm1, st>>>((const __nv_bfloat16*)x, (const uint8_t*)w_gate_up, (const int*)ids, k, H,
                                                            F, expert_offset, E, (__nv_bfloat16*)hs);
    moe_gemv8_down_kernel<2><<<g2, Q_THREADS, sm2, st>>>((const __nv_bfloat16*)hs, (const uint8_t*)w_down, (const int*)ids,
                                                         (const float*)weights, k, H, F, expert_offset, E, (__nv_bfloat16*)out);
  }
  EXO_CHECK_LAUNCH();
  return 0;
}
