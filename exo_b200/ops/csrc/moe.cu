// Mixture-of-experts kernels for sm_100a: top-k routing, the token→expert plan, and the expert
// SwiGLU FFNs as grouped tcgen05 GEMMs (or grouped GEMVs for a handful of tokens).
//
// Reference roles: the `SwitchGLU` / `gather_mm` path of mlx-lm's MoE blocks that the reference's
// auto-parallel wraps (src/exo/worker/engines/mlx/auto_parallel.py, the `*MoE*ShardingStrategy`
// classes), and the routers of Qwen3-MoE (softmax top-k) and DeepSeek-V3 (sigmoid, bias, groups).
//
// Data path for T tokens with k experts each (P = T*k pairs), E local experts starting at
// `expert_offset` of the global numbering:
//   route     logits [T, E_all]                     -> weights [T, k] fp32, ids [T, k] int32
//   count     ids                                   -> counts [E]
//   plan      counts                                -> offsets [E], tiles [(expert, row0, rows)], n_tiles
//   scatter   x [T, H], ids                         -> xs [P, H] rows grouped by expert, pos [P]
//   gemm gu   xs, W_gate_up [E, 2F, H]              -> hs [P, F] = silu(gate) * up   (two accumulators)
//   gemm down hs, W_down [E, H, F]                  -> ys [P, H]
//   combine   ys, pos, weights                      -> out [T, H] = sum_s w[t, s] * ys[pos[t, s]]
// Nothing is read back by the host: the GEMM grid is sized for the worst case and a CTA whose
// tile index is past `n_tiles` returns at once.  A GEMM CTA owns 128 output features (the TMEM
// lanes) of one expert and up to BN pair rows (MMA N) of that expert's segment; rows that belong
// to the next segment are computed and not stored.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "fp8_convert.cuh"
#include "tc_common.cuh"

int* exo_tc_err_ptr();

namespace {

// ------------------------------------------------------------------------------------------
// routing: one warp per token
// ------------------------------------------------------------------------------------------
constexpr int ROUTE_MAX_PER_LANE = 16;      // E <= 512
constexpr int ROUTE_MAX_K = 16;

struct RouteParams {
  const void* logits;     // [T, E]
  const void* bias;       // [E] or null (sigmoid only)
  float* weights;         // [T, k]
  int* ids;               // [T, k]
  int T, E, k, n_group, topk_group;
  int logits_dt, bias_dt, sigmoid, norm;
  float scaling;
};

__device__ __forceinline__ float ld_as_f(const void* p, int dt, size_t i) {
  return dt == EXO_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}

// (value, index) arg-max over the warp; ties go to the lower index.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(128) moe_route_kernel(const RouteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= p.T) return;
  const int per = (p.E + 31) / 32;
  // lane l owns experts l, l+32, ...: score = probability / sigmoid, sel = what the top-k runs on
  float score[ROUTE_MAX_PER_LANE], sel[ROUTE_MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < ROUTE_MAX_PER_LANE; j++) {
    const int e = lane + 32 * j;
    score[j] = (j < per && e < p.E) ? ld_as_f(p.logits, p.logits_dt, (size_t)t * p.E + e) : -INFINITY;
    mx = fmaxf(mx, score[j]);
  }
  if (!p.sigmoid) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; j++) {
      score[j] = score[j] == -INFINITY ? 0.f : __expf(score[j] - mx);
      sum += score[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; j++) {
      const int e = lane + 32 * j;
      score[j] *= inv;
      sel[j] = (j < per && e < p.E) ? score[j] : -INFINITY;
    }
  } else {
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; j++) {
      const int e = lane + 32 * j;
      const bool in = j < per && e < p.E;
      score[j] = in ? 1.f / (1.f + __expf(-score[j])) : 0.f;
      sel[j] = in ? score[j] + (p.bias ? ld_as_f(p.bias, p.bias_dt, e) : 0.f) : -INFINITY;
    }
    if (p.n_group > 1) {
      // group score = sum of the group's two best `sel`; keep the best `topk_group` groups.
      // Lane g scans group g through shared memory (n_group <= 32).
      __shared__ float sh[4][32 * ROUTE_MAX_PER_LANE];
#pragma unroll
      for (int j = 0; j < ROUTE_MAX_PER_LANE; j++)
        if (j < per && lane + 32 * j < p.E) sh[warp][lane + 32 * j] = sel[j];
      __syncwarp();
      const int eg = p.E / p.n_group;
      float gs = -INFINITY;
      if (lane < p.n_group) {
        float a = -INFINITY, b = -INFINITY;
        for (int i = 0; i < eg; i++) {
          float v = sh[warp][lane * eg + i];
          if (v > a) { b = a; a = v; } else if (v > b) b = v;
        }
        gs = a + b;
      }
      uint32_t keep = 0;
      for (int r = 0; r < p.topk_group; r++) {
        float v = gs;
        int i = lane;
        warp_argmax(v, i);
        keep |= 1u << i;
        if (lane == i) gs = -INFINITY;
      }
#pragma unroll
      for (int j = 0; j < ROUTE_MAX_PER_LANE; j++) {
        const int e = lane + 32 * j;
        if (j < per && e < p.E && !((keep >> (e / eg)) & 1u)) sel[j] = -INFINITY;
      }
    }
  }
  // k rounds of arg-max; the winner's lane removes it from the running
  float w_mine = 0.f;      // lane r keeps the r-th weight / id
  int id_mine = 0;
  float wsum = 0.f;
  for (int r = 0; r < p.k; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; j++) {
      const int e = lane + 32 * j;
      if (j < per && e < p.E && (sel[j] > bv)) { bv = sel[j]; bi = e; }
    }
    warp_argmax(bv, bi);
    if (bi == 0x7fffffff) bi = 0;           // fewer selectable experts than k: degenerate input
    float sc = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; j++)
      if (lane + 32 * j == bi) { sc = score[j]; sel[j] = -INFINITY; }
    sc = __shfl_sync(0xffffffffu, sc, bi & 31);
    wsum += sc;
    if (lane == r) { w_mine = sc; id_mine = bi; }
  }
  if (lane < p.k) {
    float w = w_mine;
    if (p.norm) w = p.sigmoid ? w / (wsum + 1e-20f) : w / wsum;
    p.weights[(size_t)t * p.k + lane] = w * p.scaling;
    p.ids[(size_t)t * p.k + lane] = id_mine;
  }
}

// eight bf16 -> eight f16 (saturating): token rows for the f16-operand form of the fp8 expert GEMMs
__device__ __forceinline__ uint4 bf16x8_to_f16x8(const uint4& v) {
  float f[8];
  unpack8(v, f);
  uint4 o;
  __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int j = 0; j < 4; j++)
    h[j] = __floats2half2_rn(fminf(fmaxf(f[2 * j], -65504.f), 65504.f), fminf(fmaxf(f[2 * j + 1], -65504.f), 65504.f));
  return o;
}

// ------------------------------------------------------------------------------------------
// plan: counts -> offsets and the tile list
// ------------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ ids, int P, int expert_offset, int E, int* __restrict__ counts) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  int e = ids[i] - expert_offset;
  if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
}

// One block of 1024 threads, E <= 1024.  plan[0] = n_tiles, plan[1 + 4*i ..] = (expert, row0, rows, 0).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ counts, int E, int bn, int max_tiles,
                                                        int* __restrict__ offsets, int* __restrict__ cursor,
                                                        int* __restrict__ plan) {
  __shared__ int s_rows[1024], s_tiles[1024];
  const int e = threadIdx.x;
  const int cnt = e < E ? counts[e] : 0;
  const int nt = (cnt + bn - 1) / bn;
  s_rows[e] = cnt;
  s_tiles[e] = nt;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {       // inclusive Hillis-Steele scans of both
    int a = e >= d ? s_rows[e - d] : 0, b = e >= d ? s_tiles[e - d] : 0;
    __syncthreads();
    s_rows[e] += a;
    s_tiles[e] += b;
    __syncthreads();
  }
  const int row0 = s_rows[e] - cnt, tile0 = s_tiles[e] - nt;
  if (e < E) {
    offsets[e] = row0;
    cursor[e] = 0;
    for (int i = 0; i < nt && tile0 + i < max_tiles; i++) {
      int* q = plan + 1 + 4 * (tile0 + i);
      q[0] = e;
      q[1] = row0 + i * bn;
      q[2] = min(bn, cnt - i * bn);
      q[3] = 0;
    }
  }
  if (e == 1023) plan[0] = min(s_tiles[1023], max_tiles);
}

// Up to 4096 pairs (decode batches): count, offsets, tile list and every pair's row in ONE block, so that the plan
// costs one launch instead of memset + count + plan, and the row copy needs no atomics.
__global__ void __launch_bounds__(1024) moe_plan_small_kernel(const int* __restrict__ ids, int P, int expert_offset, int E, int bn,
                                                              int max_tiles, int* __restrict__ plan, int* __restrict__ pos) {
  __shared__ int s_cnt[1024], s_rows[1024], s_tiles[1024];
  const int t = threadIdx.x;
  s_cnt[t] = 0;
  __syncthreads();
  int slot[4], ex[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = t + j * 1024;
    slot[j] = -1;
    ex[j] = 0;
    if (i < P) {
      const int e = ids[i] - expert_offset;
      if (e >= 0 && e < E) { ex[j] = e; slot[j] = atomicAdd(&s_cnt[e], 1); }
    }
  }
  __syncthreads();
  const int cnt = t < E ? s_cnt[t] : 0, nt = (cnt + bn - 1) / bn;
  s_rows[t] = cnt;
  s_tiles[t] = nt;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const int a = t >= d ? s_rows[t - d] : 0, b = t >= d ? s_tiles[t - d] : 0;
    __syncthreads();
    s_rows[t] += a;
    s_tiles[t] += b;
    __syncthreads();
  }
  const int row0 = s_rows[t] - cnt, tile0 = s_tiles[t] - nt;
  if (t == 1023) plan[0] = min(s_tiles[1023], max_tiles);
  __syncthreads();
  s_cnt[t] = row0;                      // reuse: first row of expert t
  if (t < E) {
    for (int i = 0; i < nt && tile0 + i < max_tiles; i++) {
      int* q = plan + 1 + 4 * (tile0 + i);
      q[0] = t;
      q[1] = row0 + i * bn;
      q[2] = min(bn, cnt - i * bn);
      q[3] = 0;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = t + j * 1024;
    if (i < P) pos[i] = slot[j] >= 0 ? s_cnt[ex[j]] + slot[j] : -1;
  }
}

// One warp per pair: copy the token's row to the place the plan gave it.
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ pos, int P,
                                                              int k, int H, __nv_bfloat16* __restrict__ xs, int to_f16) {
  const int pair = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= P) return;
  const int dst = pos[pair];
  if (dst < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / k) * H);
  uint4* d = reinterpret_cast<uint4*>(xs + (size_t)dst * H);
  for (int i = lane; i < H / 8; i += 32) d[i] = to_f16 ? bf16x8_to_f16x8(src[i]) : src[i];
}

// One warp per pair: take a slot in the expert's segment and copy the token's row there.
__global__ void __launch_bounds__(256) moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                                                          int P, int k, int H, int expert_offset, int E,
                                                          const int* __restrict__ offsets, int* __restrict__ cursor,
                                                          int* __restrict__ pos, __nv_bfloat16* __restrict__ xs, int to_f16) {
  const int pair = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= P) return;
  const int e = ids[pair] - expert_offset;
  int dst = -1;
  if (e >= 0 && e < E) {
    if (lane == 0) dst = offsets[e] + atomicAdd(&cursor[e], 1);
    dst = __shfl_sync(0xffffffffu, dst, 0);
  }
  if (lane == 0) pos[pair] = dst;
  if (dst < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / k) * H);
  uint4* d = reinterpret_cast<uint4*>(xs + (size_t)dst * H);
  for (int i = lane; i < H / 8; i += 32) d[i] = to_f16 ? bf16x8_to_f16x8(src[i]) : src[i];
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ pos,
                                                          const float* __restrict__ weights, int k, int H,
                                                          __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < k; s++) {
      const int r = pos[t * k + s];
      if (r < 0) continue;
      const float w = weights[t * k + s];
      float v[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(ys + (size_t)r * H) + c), v);
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] += w * v[j];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = pack8(acc);
  }
}

// ------------------------------------------------------------------------------------------
// grouped GEMM on tcgen05
// ------------------------------------------------------------------------------------------
constexpr int BM = 128, BK = 64;

// expert activations: 0 silu(gate) * up, 1 gelu_tanh(gate) * up, 2 relu(up)^2 (no gate: one projection of F rows)
enum { ACT_SWIGLU = 0, ACT_GEGLU = 1, ACT_RELU2 = 2 };
__device__ __forceinline__ float gelu_tanh_f(float g) {
  return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

struct GroupedParams {
  const int* plan;        // [1 + 4 * max_tiles]
  int rows_w;             // weight rows per expert in the 2-D view (2F for gate_up, H for down)
  int n_out;              // output features per pair row (F for gate_up, H for down)
  int K;
  __nv_bfloat16* out;     // [P, n_out]
  int* err;
  // block-scaled fp8 expert weights (FP8 kernels only): tiled storage [E, nt, kt, TILE_BYTES] (see fp8_convert.cuh)
  const uint8_t* tiles;
  int scale_kind, nt, kt;
  int f16;                // fp8 kernels: both MMA operands f16 (token rows arrive as f16)
  int out_f16;            // write `out` as f16 (the gate/up result that feeds an f16 down projection)
  int act;                // DUAL kernels: ACT_SWIGLU / ACT_GEGLU; single kernels: ACT_RELU2 squares the rectified output
  float limit;            // > 0: SwiGLU with the activated gate capped at +limit and the up projection clamped to +-limit (Step-3.5)
};

// FP8: the weight tiles arrive as bytes in `raw`; eight converter warps widen them into tensor memory, from where
// the MMA takes its A operand (see gemm_fp8w.cu), before the MMA warp may use the stage.
template <int BN, int STAGES, bool DUAL, bool FP8>
struct GSmem {
  alignas(1024) __nv_bfloat16 a[FP8 ? 1 : STAGES][FP8 ? 64 : (DUAL ? 2 : 1) * BM * BK];     // unused with fp8 weights
  alignas(1024) __nv_bfloat16 b[STAGES][BN * BK];
  alignas(128) uint8_t raw[FP8 ? STAGES : 1][FP8 ? (DUAL ? 2 : 1) * fp8cvt::TILE_BYTES : 128];
  uint64_t full[STAGES], empty[STAGES], conv[STAGES], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, int STAGES, bool DUAL, bool FP8>
__global__ void __launch_bounds__(FP8 ? 320 : 192, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const GroupedParams p) {
  if ((int)blockIdx.y >= __ldg(p.plan)) return;     // past the last tile of this step: uniform exit, nothing held
  extern __shared__ uint8_t smem_raw[];
  using S = GSmem<BN, STAGES, DUAL, FP8>;
  S& s = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * BN;
  constexpr uint32_t A_COLS = (DUAL ? 64 : 32);                   // fp8: one stage of widened weights in tensor memory
  constexpr uint32_t A_COL0 = ACC_COLS < 32 ? 32 : ACC_COLS;
  constexpr uint32_t NEED = A_COL0 + (FP8 ? STAGES * A_COLS : 0);
  constexpr uint32_t TMEM_COLS = NEED <= 32 ? 32 : NEED <= 64 ? 64 : NEED <= 128 ? 128 : NEED <= 256 ? 256 : 512;
  static_assert(NEED <= 512, "accumulators and the A ring must fit the 512 tensor-memory columns");
  constexpr uint32_t STAGE_BYTES = (DUAL ? 2 : 1) * (FP8 ? fp8cvt::TILE_BYTES : BM * BK * 2) + BN * BK * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* tile = p.plan + 1 + 4 * blockIdx.y;
  const int expert = __ldg(tile), row0 = __ldg(tile + 1), rows = __ldg(tile + 2);
  const int n0 = blockIdx.x * BM;
  const int nkb = (p.K + BK - 1) / BK;
  const int half = p.rows_w / 2;                     // DUAL: gate rows [0, F), up rows [F, 2F)

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) {
      tc::mbar_init(&s.full[i], 1);
      tc::mbar_init(&s.empty[i], 1);
      tc::mbar_init(&s.conv[i], 256);
    }
    tc::mbar_init(&s.acc_full, 1);
    s.abort_flag = 0;
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
  const int wrow = expert * p.rows_w + n0;

  if (warp == 0) {
    if (tc::elect_one()) {
      tc::prefetch_tmap(&tmap_w);
      tc::prefetch_tmap(&tmap_x);
      for (int i = 0; i < nkb; i++) {
        const int st = i % STAGES;
        if (i >= STAGES && !tc::mbar_wait(&s.empty[st], ((i / STAGES) - 1) & 1)) {
          atomicExch(p.err, tc::ERR_EMPTY_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&s.full[st], STAGE_BYTES);
        if constexpr (FP8) {
          // tile (expert, feature tile j, K block i); the up half of a gate/up pair is nt/2 feature tiles further on
          const uint8_t* t0 = p.tiles + (((size_t)expert * p.nt + blockIdx.x) * p.kt + i) * fp8cvt::TILE_BYTES;
          fp8cvt::bulk_g2s(tc::smem_u32(s.raw[st]), t0, fp8cvt::TILE_BYTES, tc::smem_u32(&s.full[st]));
          if (DUAL)
            fp8cvt::bulk_g2s(tc::smem_u32(s.raw[st]) + fp8cvt::TILE_BYTES, t0 + (size_t)(p.nt / 2) * p.kt * fp8cvt::TILE_BYTES,
                             fp8cvt::TILE_BYTES, tc::smem_u32(&s.full[st]));
        } else {
          tc::tma_load_2d(s.a[st], &tmap_w, i * BK, wrow, &s.full[st]);
          if (DUAL) tc::tma_load_2d(s.a[st] + BM * BK, &tmap_w, i * BK, wrow + half, &s.full[st]);
        }
        tc::tma_load_2d(s.b[st], &tmap_x, i * BK, row0, &s.full[st]);
      }
    }
  } else if (warp == 1) {
    if (tc::elect_one()) {
      constexpr uint32_t idesc_bf = tc::umma_idesc_bf16(BM, BN), idesc_h = idesc_bf & ~((1u << 7) | (1u << 10));     // operand formats: 1 = bf16, 0 = f16
      const uint32_t idesc = (FP8 && p.f16) ? idesc_h : idesc_bf;
      for (int i = 0; i < nkb; i++) {
        const int st = i % STAGES;
        if ((FP8 && !tc::mbar_wait(&s.conv[st], (i / STAGES) & 1)) || !tc::mbar_wait(&s.full[st], (i / STAGES) & 1)) {
          atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::tc_fence_after();
        const uint64_t bd = tc::umma_desc_sw128(tc::smem_u32(s.b[st]));
        if constexpr (FP8) {
          const uint32_t a_t = tmem + A_COL0 + st * A_COLS;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            fp8cvt::umma_bf16_ts(tmem, a_t + 8 * k, bd + 2 * k, idesc, (i | k) != 0);
            if (DUAL) fp8cvt::umma_bf16_ts(tmem + BN, a_t + 32 + 8 * k, bd + 2 * k, idesc, (i | k) != 0);
          }
        } else {
          const uint64_t ad = tc::umma_desc_sw128(tc::smem_u32(s.a[st]));
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            tc::umma_bf16(tmem, ad + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
            if (DUAL) {
              const uint64_t ud = tc::umma_desc_sw128(tc::smem_u32(s.a[st] + BM * BK));
              tc::umma_bf16(tmem + BN, ud + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
            }
          }
        }
        tc::umma_commit(&s.empty[st]);
      }
      tc::umma_commit(&s.acc_full);
    }
  } else {
    if constexpr (FP8) {
      // 256 converter threads (warps 2..9).  Warp w may touch the tensor-memory lanes of quadrant w % 4 only, so it
      // widens the rows of that quadrant: warps 2..5 take the first 32 weights of every row's K block (of both tiles of
      // a gate/up stage), warps 6..9 the second 32.  The stage's columns are free: the producer only refilled the
      // stage after the MMAs that read them had completed.
      const int quad = warp & 3, h = (warp - 2) >> 2, r = quad * 32 + lane;
      const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + A_COL0 + 16 * h;
      for (int i = 0; i < nkb; i++) {
        const int st = i % STAGES;
        if (!tc::mbar_wait_backoff(&s.full[st], (i / STAGES) & 1, 32, 1u << 24)) {
          atomicExch(p.err, tc::ERR_TILE_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::tc_fence_after();
        const uint32_t raw0 = tc::smem_u32(s.raw[st]);
        uint32_t c0, c1;
        if (p.f16) {
          fp8cvt::tile_scales_f16(raw0, p.scale_kind, r, c0, c1);
          fp8cvt::convert_half_row_tmem_f16(raw0, lane_base + st * A_COLS, r, h, h ? c1 : c0);
          if (DUAL) {
            fp8cvt::tile_scales_f16(raw0 + fp8cvt::TILE_BYTES, p.scale_kind, r, c0, c1);
            fp8cvt::convert_half_row_tmem_f16(raw0 + fp8cvt::TILE_BYTES, lane_base + st * A_COLS + 32, r, h, h ? c1 : c0);
          }
        } else {
          fp8cvt::tile_scales(raw0, p.scale_kind, r, c0, c1);
          fp8cvt::convert_half_row_tmem(raw0, lane_base + st * A_COLS, r, h, h ? c1 : c0);
          if (DUAL) {
            fp8cvt::tile_scales(raw0 + fp8cvt::TILE_BYTES, p.scale_kind, r, c0, c1);
            fp8cvt::convert_half_row_tmem(raw0 + fp8cvt::TILE_BYTES, lane_base + st * A_COLS + 32, r, h, h ? c1 : c0);
          }
        }
        fp8cvt::tmem_st_fence();
        tc::mbar_arrive(&s.conv[st]);
      }
    }
    if (!FP8 || warp < 6) {       // warps 2..5 own the four TMEM lane quadrants
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    bool ok = tc::mbar_wait_backoff(&s.acc_full, 0, 400);
    if (!ok) { atomicExch(p.err, tc::ERR_ACC_TIMEOUT); s.abort_flag = 1; }
    tc::tc_fence_after();
    ok = ok && !*(volatile int*)&s.abort_flag;
    const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
    const bool n_ok = n < p.n_out;
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
      float g[16], u[16];
      tc::tmem_ld16(taddr + c, g);
      if (DUAL) tc::tmem_ld16(taddr + BN + c, u);
      tc::tmem_ld_wait();
      if (ok && n_ok) {
#pragma unroll
        for (int j = 0; j < 16; j++) {
          if (c + j < rows) {
            float y;
            if (DUAL) {   // the projection is rounded to bf16 before the activation, as the unfused form does
              const float gb = __bfloat162float(__float2bfloat16_rn(g[j])), ub = __bfloat162float(__float2bfloat16_rn(u[j]));
              float a = p.act == ACT_GEGLU ? gelu_tanh_f(gb) : silu_f(gb), ul = ub;
              if (p.limit > 0.f) { a = fminf(a, p.limit); ul = fminf(fmaxf(ub, -p.limit), p.limit); }
              y = a * ul;
            } else {
              y = g[j];
              if (p.act == ACT_RELU2) {
                const float rb = fmaxf(__bfloat162float(__float2bfloat16_rn(y)), 0.f);
                y = rb * rb;
              }
            }
            const size_t o = (size_t)(row0 + c + j) * p.n_out + n;
            if (FP8 && p.out_f16) reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(fminf(fmaxf(y, -65504.f), 65504.f));
            else p.out[o] = __float2bfloat16_rn(y);
          }
        }
      }
    }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool DUAL, bool FP8>
int launch_grouped(const CUtensorMap* tw, const CUtensorMap* tx, const GroupedParams& p, int n_tiles_w, int max_tiles,
                   cudaStream_t st) {
  using S = GSmem<BN, STAGES, DUAL, FP8>;
  const size_t smem = sizeof(S) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(moe_grouped_gemm_kernel<BN, STAGES, DUAL, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  moe_grouped_gemm_kernel<BN, STAGES, DUAL, FP8><<<dim3(n_tiles_w, max_tiles), FP8 ? 320 : 192, smem, st>>>(*tw, *tx, p);
  EXO_CHECK_LAUNCH();
  return 0;
}

template <bool DUAL>
int grouped_dispatch(int bn, const CUtensorMap* tw, const CUtensorMap* tx, const GroupedParams& p, int n_tiles_w,
                     int max_tiles, cudaStream_t st) {
  if (p.tiles) {      // fp8 weights: a stage also holds the raw byte tiles
    switch (bn) {
      // stages: shared memory holds raw tiles and token tiles only; the widened weights take 32 (64 for a gate/up
      // pair) tensor-memory columns per stage next to the accumulators
      case 16: return launch_grouped<16, 6, DUAL, true>(tw, tx, p, n_tiles_w, max_tiles, st);
      case 32: return launch_grouped<32, 6, DUAL, true>(tw, tx, p, n_tiles_w, max_tiles, st);
      case 64: return launch_grouped<64, 5, DUAL, true>(tw, tx, p, n_tiles_w, max_tiles, st);
      default: return launch_grouped<128, 4, DUAL, true>(tw, tx, p, n_tiles_w, max_tiles, st);
    }
  }
  switch (bn) {
    case 16: return launch_grouped<16, 5, DUAL, false>(tw, tx, p, n_tiles_w, max_tiles, st);
    case 32: return launch_grouped<32, 5, DUAL, false>(tw, tx, p, n_tiles_w, max_tiles, st);
    case 64: return launch_grouped<64, 4, DUAL, false>(tw, tx, p, n_tiles_w, max_tiles, st);
    default: return launch_grouped<128, 4, DUAL, false>(tw, tx, p, n_tiles_w, max_tiles, st);
  }
}

// ------------------------------------------------------------------------------------------
// grouped GEMV for a handful of pairs: every (pair, 16-feature chunk) is one CTA
// ------------------------------------------------------------------------------------------
constexpr int GV_ROWS = 16, GV_THREADS = 256;

// dot of two bf16 rows of length K (K % 8 == 0): the weight row streams from global, x sits in shared
__device__ __forceinline__ float dot_row(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* xs, int K, int lane) {
  float acc = 0.f;
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  const uint4* xp = reinterpret_cast<const uint4*>(xs);
  int i = lane;
  for (; i + 96 < K / 8; i += 128) {        // four 16-byte loads in flight per lane
    uint4 a0 = ld_stream16(wp + i), a1 = ld_stream16(wp + i + 32), a2 = ld_stream16(wp + i + 64), a3 = ld_stream16(wp + i + 96);
    float f[8], g[8];
    unpack8(a0, f); unpack8(xp[i], g);
#pragma unroll
    for (int j = 0; j < 8; j++) acc += f[j] * g[j];
    unpack8(a1, f); unpack8(xp[i + 32], g);
#pragma unroll
    for (int j = 0; j < 8; j++) acc += f[j] * g[j];
    unpack8(a2, f); unpack8(xp[i + 64], g);
#pragma unroll
    for (int j = 0; j < 8; j++) acc += f[j] * g[j];
    unpack8(a3, f); unpack8(xp[i + 96], g);
#pragma unroll
    for (int j = 0; j < 8; j++) acc += f[j] * g[j];
  }
  for (; i < K / 8; i += 32) {
    float f[8], g[8];
    unpack8(ld_stream16(wp + i), f); unpack8(xp[i], g);
#pragma unroll
    for (int j = 0; j < 8; j++) acc += f[j] * g[j];
  }
  return warp_sum(acc);
}

// hs[pair, f] = silu(Wg[e][f] . x[t]) * (Wu[e][f] . x[t])
__global__ void __launch_bounds__(GV_THREADS)
moe_gemv_gate_up_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_gu, const int* __restrict__ ids,
                        int k, int H, int F, int expert_offset, int E, int act, float limit, __nv_bfloat16* __restrict__ hs) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gv_smem);
  const int pair = blockIdx.y;
  const int e = ids[pair] - expert_offset;
  if (e < 0 || e >= E) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / k) * H);
  for (int i = threadIdx.x; i < H / 8; i += GV_THREADS) reinterpret_cast<uint4*>(xs)[i] = src[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* wg = w_gu + (size_t)e * (act == ACT_RELU2 ? 1 : 2) * F * H;
  for (int r = warp; r < GV_ROWS; r += GV_THREADS / 32) {
    const int f = blockIdx.x * GV_ROWS + r;
    if (f >= F) break;
    float g = dot_row(wg + (size_t)f * H, xs, H, lane);
    float u = act == ACT_RELU2 ? 0.f : dot_row(wg + (size_t)(F + f) * H, xs, H, lane);
    if (lane == 0) {
      g = __bfloat162float(__float2bfloat16_rn(g));
      u = __bfloat162float(__float2bfloat16_rn(u));
      float a = act == ACT_GEGLU ? gelu_tanh_f(g) : silu_f(g);
      if (limit > 0.f) { a = fminf(a, limit); u = fminf(fmaxf(u, -limit), limit); }
      const float y = act == ACT_RELU2 ? fmaxf(g, 0.f) * fmaxf(g, 0.f) : a * u;
      hs[(size_t)pair * F + f] = __float2bfloat16_rn(y);
    }
  }
}

// out[t, n] = sum_s w[t, s] * bf16(Wd[e_s][n] . hs[t*k + s])
__global__ void __launch_bounds__(GV_THREADS)
moe_gemv_down_kernel(const __nv_bfloat16* __restrict__ hs, const __nv_bfloat16* __restrict__ w_down, const int* __restrict__ ids,
                     const float* __restrict__ weights, int k, int H, int F, int expert_offset, int E,
                     __nv_bfloat16* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  __nv_bfloat16* hsm = reinterpret_cast<__nv_bfloat16*>(gv_smem);     // [k, F]
  const int t = blockIdx.y;
  for (int s = 0; s < k; s++) {
    const int e = ids[t * k + s] - expert_offset;
    if (e < 0 || e >= E) continue;
    const uint4* src = reinterpret_cast<const uint4*>(hs + (size_t)(t * k + s) * F);
    for (int i = threadIdx.x; i < F / 8; i += GV_THREADS) reinterpret_cast<uint4*>(hsm + (size_t)s * F)[i] = src[i];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < GV_ROWS; r += GV_THREADS / 32) {
    const int n = blockIdx.x * GV_ROWS + r;
    if (n >= H) break;
    float acc = 0.f;
    for (int s = 0; s < k; s++) {
      const int e = ids[t * k + s] - expert_offset;
      if (e < 0 || e >= E) continue;
      float y = dot_row(w_down + ((size_t)e * H + n) * F, hsm + (size_t)s * F, F, lane);
      acc += weights[t * k + s] * __bfloat162float(__float2bfloat16_rn(y));
    }
    if (lane == 0) out[(size_t)t * H + n] = __float2bfloat16_rn(acc);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// entry points
// ------------------------------------------------------------------------------------------
EXO_API int exo_moe_route(const void* logits, const void* bias, void* weights, void* ids, int T, int E, int k, int n_group,
                          int topk_group, int logits_dt, int bias_dt, int sigmoid, int norm, float scaling, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 32 * ROUTE_MAX_PER_LANE || k > ROUTE_MAX_K || k > E || n_group > 32 || (n_group > 1 && E % n_group)) return -2;
  RouteParams p;
  p.logits = logits; p.bias = bias; p.weights = (float*)weights; p.ids = (int*)ids;
  p.T = T; p.E = E; p.k = k; p.n_group = n_group; p.topk_group = topk_group;
  p.logits_dt = logits_dt; p.bias_dt = bias_dt; p.sigmoid = sigmoid; p.norm = norm; p.scaling = scaling;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, st>>>(p);
  EXO_CHECK_LAUNCH();
  return 0;
}

// Tile height of the grouped GEMMs for P pairs over E local experts (shape-based, no device read).
EXO_API int exo_moe_tile_rows(int P, int E) {
  int avg = (P + E - 1) / E;
  return avg <= 16 ? 16 : avg <= 32 ? 32 : avg <= 64 ? 64 : 128;
}
// Worst-case number of row tiles: every expert may end in a partial tile.
EXO_API int exo_moe_max_tiles(int P, int E, int bn) { return (P < E ? P : E) + P / bn; }

// ints of scratch: counts[E] offsets[E] cursor[E] plan[1 + 4*max_tiles]
EXO_API long exo_moe_plan_ints(int E, int max_tiles) { return 3L * E + 1 + 4L * max_tiles; }

// The whole expert block for T tokens (grouped tcgen05 GEMMs).  `scratch` holds exo_moe_plan_ints
// ints, `pos` P ints, `xs`/`ys` [P, H] and `hs` [P, F] bf16.
// Block-scaled fp8 experts: `scale_kind` 1 (e8m0 per 1x32) or 2 (fp32 per tile) and `w_gate_up` / `w_down` in the tiled
// form [E, 2F/128, H/64, 8448] / [E, ceil(H/128), F/64, 8448]; 0 = bf16 weights.
EXO_API int exo_moe_experts_grouped(const void* x, const void* w_gate_up, const void* w_down, const void* weights,
                                    const void* ids, void* out, void* scratch, void* pos, void* xs, void* hs, void* ys, int T,
                                    int k, int H, int F, int E, int expert_offset, int scale_kind, int tile_rows, int f16_operands,
                                    int act, float limit, cudaStream_t st) {
  const int f16 = (scale_kind && f16_operands) ? 1 : 0;
  if (T <= 0) return 0;
  if (act < 0 || act > ACT_RELU2 || (act == ACT_RELU2 && scale_kind)) return -2;     // non-gated experts: bf16 weights only
  if (E > 1024 || H % 8 || F % 8 || H < BK || F < BK) return -2;
  if (scale_kind && (H % 64 || F % 128)) return -2;      // whole K tiles; gate and up halves on tile boundaries
  int* err = exo_tc_err_ptr();
  if (!err) return -4;
  const int P = T * k;
  // tile_rows: 16/32/64/128 chosen by the caller from the pairs it EXPECTS to be local (0 = from all pairs)
  const int bn = (tile_rows == 16 || tile_rows == 32 || tile_rows == 64 || tile_rows == 128) ? tile_rows : exo_moe_tile_rows(P, E);
  const int max_tiles = exo_moe_max_tiles(P, E, bn);
  int* counts = (int*)scratch;
  int* offsets = counts + E;
  int* cursor = offsets + E;
  int* plan = cursor + E;
  if (P <= 4096) {      // decode batches: the whole plan in one block, then a plain row gather
    moe_plan_small_kernel<<<1, 1024, 0, st>>>((const int*)ids, P, expert_offset, E, bn, max_tiles, plan, (int*)pos);
    moe_gather_rows_kernel<<<(P + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, (const int*)pos, P, k, H, (__nv_bfloat16*)xs, f16);
  } else {
    if (cudaMemsetAsync(counts, 0, sizeof(int) * E, st) != cudaSuccess) return -7;
    moe_count_kernel<<<(P + 255) / 256, 256, 0, st>>>((const int*)ids, P, expert_offset, E, counts);
    moe_plan_kernel<<<1, 1024, 0, st>>>(counts, E, bn, max_tiles, offsets, cursor, plan);
    moe_scatter_kernel<<<(P + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, (const int*)ids, P, k, H, expert_offset, E, offsets,
                                                    cursor, (int*)pos, (__nv_bfloat16*)xs, f16);
  }
  EXO_CHECK_LAUNCH();
  const CUtensorMap* t_xs = exo_tmap_2d_bf16(xs, P, H, bn);
  // fp8: the weights are not read through a tensor map (the activations' map stands in for the unused argument)
  const int up_rows = act == ACT_RELU2 ? F : 2 * F;          // rows of the first projection per expert
  const CUtensorMap* t_wgu = scale_kind ? t_xs : exo_tmap_2d_bf16(w_gate_up, (uint64_t)E * up_rows, H, BM);
  const CUtensorMap* t_wd = scale_kind ? t_xs : exo_tmap_2d_bf16(w_down, (uint64_t)E * H, F, BM);
  const CUtensorMap* t_hs = exo_tmap_2d_bf16(hs, P, F, bn);
  if (!t_wgu || !t_xs || !t_wd || !t_hs) return -5;
  GroupedParams g;
  g.plan = plan; g.err = err;
  g.rows_w = up_rows; g.n_out = F; g.K = H; g.out = (__nv_bfloat16*)hs;
  g.scale_kind = scale_kind;
  g.f16 = f16; g.out_f16 = f16;
  g.act = act;
  g.limit = act == ACT_SWIGLU ? limit : 0.f;
  g.tiles = scale_kind ? (const uint8_t*)w_gate_up : nullptr;
  g.nt = up_rows / BM; g.kt = H / BK;
  int rc = act == ACT_RELU2 ? grouped_dispatch<false>(bn, t_wgu, t_xs, g, (F + BM - 1) / BM, max_tiles, st)
                            : grouped_dispatch<true>(bn, t_wgu, t_xs, g, (F + BM - 1) / BM, max_tiles, st);
  if (rc) return rc;
  g.rows_w = H; g.n_out = H; g.K = F; g.out = (__nv_bfloat16*)ys;
  g.out_f16 = 0;
  g.act = ACT_SWIGLU;
  g.limit = 0.f;
  g.tiles = scale_kind ? (const uint8_t*)w_down : nullptr;
  g.nt = (H + BM - 1) / BM; g.kt = F / BK;
  rc = grouped_dispatch<false>(bn, t_wd, t_hs, g, (H + BM - 1) / BM, max_tiles, st);
  if (rc) return rc;
  moe_combine_kernel<<<T, 256, 0, st>>>((const __nv_bfloat16*)ys, (const int*)pos, (const float*)weights, k, H,
                                       (__nv_bfloat16*)out);
  EXO_CHECK_LAUNCH();
  return 0;
}

// The same block for a handful of tokens: two grouped GEMV kernels, no plan.  `hs` is [T*k, F].
EXO_API int exo_moe_experts_gemv(const void* x, const void* w_gate_up, const void* w_down, const void* weights, const void* ids,
                                 void* out, void* hs, int T, int k, int H, int F, int E, int expert_offset, int act, float limit,
                                 cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || F % 8 || act < 0 || act > ACT_RELU2) return -2;
  const size_t sm1 = (size_t)H * 2, sm2 = (size_t)k * F * 2;
  if (sm1 > 200 * 1024 || sm2 > 200 * 1024) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(moe_gemv_gate_up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(moe_gemv_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  moe_gemv_gate_up_kernel<<<dim3((F + GV_ROWS - 1) / GV_ROWS, T * k), GV_THREADS, sm1, st>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate_up, (const int*)ids, k, H, F, expert_offset, E, act,
      act == ACT_SWIGLU ? limit : 0.f, (__nv_bfloat16*)hs);
  moe_gemv_down_kernel<<<dim3((H + GV_ROWS - 1) / GV_ROWS, T), GV_THREADS, sm2, st>>>(
      (const __nv_bfloat16*)hs, (const __nv_bfloat16*)w_down, (const int*)ids, (const float*)weights, k, H, F, expert_offset, E,
      (__nv_bfloat16*)out);
  EXO_CHECK_LAUNCH();
  return 0;
}
