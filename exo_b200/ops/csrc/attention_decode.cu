// Paged-KV decode attention (one query token per sequence), split over the KV length.
//
// Grid (n_splits, Hkv * (g / GT), B).  A CTA streams its slice of one KV head once and scores
// it against GT query heads that share that KV head (GQA), so K/V bytes are read once per group.
// Inside a warp, LW lanes cooperate on one key (8 lanes with D/8 dims each; 16 lanes at D = 256 and 32 at D = 512, which keeps
// the per-lane state at 16 dims), 32/LW lane-groups x 2 keys are in
// flight per iteration; every (lane-group, head) keeps its own online-softmax state, merged at the
// end through shuffles and shared memory.  Each split publishes (m, l, o) partials to a workspace
// and takes a ticket; the CTA that draws the last ticket of its (sequence, head group) merges the
// splits and writes the output, so there is no second launch.
#include "common.cuh"

template <typename T, int D, int GT>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const T* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ block_tables, const int* __restrict__ seq_lens,
                    float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ tickets,
                    T* __restrict__ out, float scale, int Hq, int Hkv, int max_blocks, int block_size, int window,
                    const float* __restrict__ sinks) {
  constexpr int LW = D > 256 ? 32 : D > 128 ? 16 : 8;  // lanes per key (16 dims per lane from 128 up)
  constexpr int NLG = 32 / LW;          // lane groups (keys side by side) per warp
  constexpr int DPL = D / LW;           // dims per lane
  constexpr int U = 2;                  // keys per lane-group per iteration
  const int split = blockIdx.x, n_splits = gridDim.x, b = blockIdx.z;
  const int g = Hq / Hkv, tiles_per_kv = g / GT;
  const int kvh = blockIdx.y / tiles_per_kv, h0 = kvh * g + (blockIdx.y % tiles_per_kv) * GT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lg = lane / LW, ls = lane % LW;
  pdl_trigger();
  pdl_wait();  // q, the appended K/V row and the step inputs come from the preceding kernels
  const int n = seq_lens[b];
  const int lo_lim = (window > 0 && n > window) ? n - window : 0;
  // chunk of keys for this split, in whole blocks
  const int start = lo_lim / block_size * block_size;
  const int per = ((n - start + n_splits - 1) / n_splits + block_size - 1) / block_size * block_size;
  const int t0 = start + split * per, t1 = min(n, t0 + per);

  float qr[GT][DPL], acc[GT][DPL], m[GT], l[GT];
#pragma unroll
  for (int i = 0; i < GT; i++) {
    const T* qp = q + ((size_t)b * Hq + h0 + i) * D + ls * DPL;
#pragma unroll
    for (int d = 0; d < DPL; d++) { qr[i][d] = Cvt<T>::to_f(qp[d]) * scale; acc[i][d] = 0.f; }
    m[i] = -INFINITY;
    l[i] = 0.f;
  }
  const int* bt = block_tables + (size_t)b * max_blocks;
  for (int base = t0 + warp * (NLG * U); base < t1; base += 4 * NLG * U) {  // warp-uniform trip count
    float kf[U][DPL], vf[U][DPL];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      int t = base + u * NLG + lg;
      valid[u] = t < t1 && t >= lo_lim;
      if (valid[u]) {
        int blk = bt[t / block_size];
        size_t off = (((size_t)blk * block_size + t % block_size) * Hkv + kvh) * D + ls * DPL;
        if constexpr (sizeof(T) == 2) {
#pragma unroll
          for (int d = 0; d < DPL; d += 8) {
            unpack8(*reinterpret_cast<const uint4*>(kcache + off + d), kf[u] + d);
            unpack8(*reinterpret_cast<const uint4*>(vcache + off + d), vf[u] + d);
          }
        } else {
#pragma unroll
          for (int d = 0; d < DPL; d++) { kf[u][d] = Cvt<T>::to_f(kcache[off + d]); vf[u][d] = Cvt<T>::to_f(vcache[off + d]); }
        }
      } else {
#pragma unroll
        for (int d = 0; d < DPL; d++) { kf[u][d] = 0.f; vf[u][d] = 0.f; }
      }
    }
#pragma unroll
    for (int i = 0; i < GT; i++) {
      float s[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        float a = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; d++) a += qr[i][d] * kf[u][d];
#pragma unroll
        for (int o = 1; o < LW; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        s[u] = valid[u] ? a : -INFINITY;
      }
      float mn = fmaxf(m[i], fmaxf(s[0], s[1]));
      if (mn > -INFINITY) {
        float corr = __expf(m[i] - mn);
        float p0 = __expf(s[0] - mn), p1 = __expf(s[1] - mn);
        l[i] = l[i] * corr + p0 + p1;
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[i][d] = acc[i][d] * corr + p0 * vf[0][d] + p1 * vf[1][d];
        m[i] = mn;
      }
    }
  }
  // merge the lane-groups of the warp
#pragma unroll
  for (int i = 0; i < GT; i++) {
#pragma unroll
    for (int o = LW; o <= 16; o <<= 1) {
      float mo = __shfl_xor_sync(0xffffffffu, m[i], o), lo2 = __shfl_xor_sync(0xffffffffu, l[i], o);
      float mn = fmaxf(m[i], mo);
      float c0 = (m[i] == -INFINITY) ? 0.f : __expf(m[i] - mn), c1 = (mo == -INFINITY) ? 0.f : __expf(mo - mn);
      l[i] = l[i] * c0 + lo2 * c1;
#pragma unroll
      for (int d = 0; d < DPL; d++) {
        float ao = __shfl_xor_sync(0xffffffffu, acc[i][d], o);
        acc[i][d] = acc[i][d] * c0 + ao * c1;
      }
      m[i] = mn;
    }
  }
  // merge the 4 warps through shared memory
  __shared__ float sm_m[4][GT], sm_l[4][GT];
  __shared__ float sm_o[4][GT][D];
  __shared__ int is_last;
  if (lg == 0) {
#pragma unroll
    for (int i = 0; i < GT; i++) {
      if (ls == 0) { sm_m[warp][i] = m[i]; sm_l[warp][i] = l[i]; }
#pragma unroll
      for (int d = 0; d < DPL; d++) sm_o[warp][i][ls * DPL + d] = acc[i][d];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GT * D; idx += blockDim.x) {
    int i = idx / D, d = idx % D;
    float mn = fmaxf(fmaxf(sm_m[0][i], sm_m[1][i]), fmaxf(sm_m[2][i], sm_m[3][i]));
    float o = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      float c = (sm_m[w][i] == -INFINITY) ? 0.f : __expf(sm_m[w][i] - mn);
      o += sm_o[w][i][d] * c;
      lt += sm_l[w][i] * c;
    }
    if (n_splits == 1) {  // nothing to merge across CTAs: finish here
      float sink = 0.f;
      if (sinks) { float sk = sinks[h0 + i], m2 = fmaxf(mn, sk); o *= __expf(mn - m2); lt = lt * __expf(mn - m2) + __expf(sk - m2); }
      (void)sink;
      out[((size_t)b * Hq + h0 + i) * D + d] = Cvt<T>::from_f(lt > 0.f ? o / lt : 0.f);
    } else {
      size_t pi = ((size_t)b * Hq + h0 + i) * n_splits + split;
      part_o[pi * D + d] = o;
      if (d == 0) { part_ml[pi * 2] = mn; part_ml[pi * 2 + 1] = lt; }
    }
  }
  if (n_splits == 1) return;
  // ticket: the last split of this (sequence, head group) to finish merges all of them
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = tickets + (size_t)b * gridDim.y + blockIdx.y;
    int t = atomicAdd(tk, 1);
    is_last = (t == n_splits - 1);
    if (is_last) *tk = 0;  // self-reset for the next launch / graph replay
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // parallel merge: one thread per (head, split) turns its (m, l) into a normalised weight, then
  // every thread accumulates its output dims with the split loads unrolled (independent loads)
  __shared__ float wgt[GT][64];
  __shared__ float hm[GT], hl[GT];
  for (int idx = threadIdx.x; idx < GT * 64; idx += blockDim.x) {
    int i = idx / 64, s2 = idx % 64;
    size_t bh = (size_t)b * Hq + h0 + i;
    wgt[i][s2] = s2 < n_splits ? __ldcg(part_ml + (bh * n_splits + s2) * 2) : -INFINITY;
  }
  __syncthreads();
  if (threadIdx.x < GT) {
    int i = threadIdx.x;
    float mn = -INFINITY;
    for (int s2 = 0; s2 < n_splits; s2++) mn = fmaxf(mn, wgt[i][s2]);
    if (sinks) mn = fmaxf(mn, sinks[h0 + i]);
    hm[i] = mn;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GT * 64; idx += blockDim.x) {
    int i = idx / 64, s2 = idx % 64;
    size_t bh = (size_t)b * Hq + h0 + i;
    float ms = wgt[i][s2];
    float c = (ms == -INFINITY) ? 0.f : __expf(ms - hm[i]);
    float lpart = s2 < n_splits ? __ldcg(part_ml + (bh * n_splits + s2) * 2 + 1) * c : 0.f;
    // sum of l * c over the 64 slots of this head: two warps per head → shuffle + smem
    lpart = warp_sum(lpart);
    __syncwarp();
    wgt[i][s2] = c;
    if ((s2 & 31) == 0) sm_l[s2 >> 5][i] = lpart;
  }
  __syncthreads();
  if (threadIdx.x < GT) {
    int i = threadIdx.x;
    float lsum = sm_l[0][i] + sm_l[1][i];
    if (sinks) lsum += __expf(sinks[h0 + i] - hm[i]);
    hl[i] = lsum > 0.f ? 1.f / lsum : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GT * D; idx += blockDim.x) {
    int i = idx / D, d = idx % D;
    size_t bh = (size_t)b * Hq + h0 + i;
    const float* po = part_o + bh * n_splits * D + d;
    float o = 0.f;
    int s2 = 0;
    for (; s2 + 8 <= n_splits; s2 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; u++) v[u] = __ldcg(po + (size_t)(s2 + u) * D);
#pragma unroll
      for (int u = 0; u < 8; u++) o += v[u] * wgt[i][s2 + u];
    }
    for (; s2 < n_splits; s2++) o += __ldcg(po + (size_t)s2 * D) * wgt[i][s2];
    out[bh * D + d] = Cvt<T>::from_f(o * hl[i]);
  }
}

// workspace floats needed: partial outputs + (m, l) pairs + one ticket word per (sequence, head group)
EXO_API long exo_paged_decode_workspace(int B, int Hq, int D, int n_splits) {
  return (long)B * Hq * n_splits * (D + 2) + (long)B * Hq + 64;
}

EXO_API int exo_paged_decode_splits(int B, int Hkv, int max_len) {
  int want = (3 * 148 + B * Hkv - 1) / (B * Hkv);
  int cap = (max_len + 63) / 64;
  int s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

// `tickets` must be zero before the first launch (the kernel leaves it zero afterwards).
EXO_API int exo_paged_decode(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                             const int* seq_lens, void* out, float* workspace, int* tickets, float scale, int B, int Hq,
                             int Hkv, int D, int max_blocks, int block_size, int n_splits, int window,
                             const float* sinks, int dtype, cudaStream_t st) {
  if (B == 0) return 0;
  int g = Hq / Hkv;
  if (g * Hkv != Hq) return -2;
  float* part_o = workspace;
  float* part_ml = workspace + (size_t)B * Hq * n_splits * D;
  int GT = (g % 4 == 0) ? 4 : (g % 2 == 0 ? 2 : 1);
  dim3 grid(n_splits, Hkv * (g / GT), B);
  if (D == 512 && (size_t)4 * GT * D * sizeof(float) > 40 * 1024) return -2;
  cudaError_t e = cudaSuccess;
#define LAUNCH(TT, DD, GG)                                                                                        \
  e = launch_pdl(paged_decode_kernel<TT, DD, GG>, grid, dim3(128), 0, st, (const TT*)q, (const TT*)kcache,         \
                 (const TT*)vcache, block_tables, seq_lens, part_o, part_ml, tickets, (TT*)out, scale, Hq, Hkv,    \
                 max_blocks, block_size, window, sinks)
#define BY_G(TT, DD)                       \
  if (GT == 4) LAUNCH(TT, DD, 4);          \
  else if (GT == 2) LAUNCH(TT, DD, 2);     \
  else LAUNCH(TT, DD, 1)
  if (dtype == EXO_BF16) {
    if (D == 128) { BY_G(__nv_bfloat16, 128); }
    else if (D == 64) { BY_G(__nv_bfloat16, 64); }
    else if (D == 256) { BY_G(__nv_bfloat16, 256); }
    else if (D == 512) { BY_G(__nv_bfloat16, 512); }
    else return -2;
  } else {
    if (D == 128) { BY_G(float, 128); }
    else if (D == 64) { BY_G(float, 64); }
    else if (D == 256) { BY_G(float, 256); }
    else if (D == 512) { BY_G(float, 512); }
    else return -2;
  }
#undef BY_G
#undef LAUNCH
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}
