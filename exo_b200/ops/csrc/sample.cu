// Filtered sampling (temperature, top-k, top-p, min-p) in three multi-CTA passes over the logits.
//
//   p_i = softmax(l / T);  keep i  iff  #{p > p_i} < top_k  and  mass{p > p_i} < top_p  and  p_i >= min_p * p_max
//   (the arg-max is always kept); then inverse CDF over the kept tokens in vocabulary order with the caller's uniform.
//
// Work is in q_i = exp((l_i - l_max) / T) in (0, 1] and in u_i = -ln q_i.  Every sum of q is kept in 2^-32 fixed point
// (64-bit integer adds are associative), so the result does not depend on the order in which CTAs or atomics land:
// ranks of a tensor-parallel group that sample the same logits pick the same token.
//
//   pass 1  (chunks x rows CTAs)  per-chunk max / arg-max; clears the row's histogram
//   pass 2  (chunks x rows CTAs)  histogram of u in NB bins of width 1/32 (count and mass per bin); the last CTA of a
//           row scans the bins and finds the one bin b* in which the top-k / top-p predicate flips: every token of a
//           lower bin (larger q) is kept, every token of a higher bin is dropped
//   pass 3  (chunks x rows CTAs)  per-chunk kept mass of the bins below b* and a list of the q values inside b*; the
//           last CTA of the row resolves the exact threshold inside b* from the list (all pairs, <= CAP entries), adds
//           the list's kept entries to their chunks, picks the chunk that holds uniform * total and walks it
//
// A row whose boundary bin holds more than CAP tokens (a nearly flat distribution) goes through one more pass between 2
// and 3: the boundary bin alone is histogrammed again in NB sub-bins (width 2^-15 in u), which finds the boundary
// sub-bin; pass 3 then lists that sub-bin.  Rows without such a bin return from the extra pass at once.  Only a row
// whose boundary SUB-bin still holds more than CAP tokens (many equal logits) is flagged and re-done by the single-CTA
// bisection kernel in basic.cu, which the launcher always enqueues behind pass 3 (it returns at once for rows that are
// not flagged).
#include "common.cuh"

namespace {

constexpr int NB = 1024;            // histogram bins over u in [0, 32); the last bin also takes u >= 32
constexpr float BINS_PER_U = 32.f;
constexpr int CAP = 1024;           // boundary-bin entries resolved exactly
constexpr int NT = 512;
constexpr int MAX_CHUNKS = 64;
constexpr float FX_ONE = 4294967296.f;   // 2^32
typedef unsigned long long u64;

struct RowWs {                      // per-row scratch, zero-initialised once; the kernels leave tickets and n_list at zero
  float pv[MAX_CHUNKS];
  int pi[MAX_CHUNKS];
  int cnt[NB];
  u64 mass[NB];
  u64 chunk_mass[MAX_CHUNKS];
  u64 list[CAP];
  int list_chunk[CAP];
  int cnt2[NB];                     // second level: the boundary bin alone, in NB sub-bins
  u64 mass2[NB];
  u64 c_mass;                       // mass of the bins below b*
  u64 pmass;                        // top_p * total mass (fixed point); ~0 when top-p is off
  int c_cnt;                        // tokens in the bins below b*
  int b_star;                       // NB when nothing is cut by top-k / top-p
  int resolve;                      // 1: the threshold inside b* comes from the list; 0: b* is dropped entirely
  int n_list;
  int ticket2, ticket3;
  int fallback;
  int refine;                       // 1: the boundary bin is too full for the list and gets a second histogram
  int s_star;                       // boundary sub-bin (NB: none, the whole bin is on one side)
  int ticket_r;
};

template <typename T>
__device__ __forceinline__ float ldf(const T* p) { return Cvt<T>::to_f(*p); }

// f(index, value) for every token of [c0, c1), each thread taking 16-byte groups when the row allows it
template <typename T, typename F>
__device__ __forceinline__ void for_tokens(const T* __restrict__ x, int c0, int c1, F f) {
  constexpr int VEC = 16 / (int)sizeof(T);
  int tid = threadIdx.x;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    int a0 = (c0 + VEC - 1) / VEC * VEC, a1 = c1 / VEC * VEC;
    if (a0 >= a1) { a0 = c1; a1 = c1; }
    for (int i = c0 + tid; i < a0; i += NT) f(i, ldf(x + i));
    for (int i = a0 + tid * VEC; i < a1; i += NT * VEC) {
      uint4 v = *reinterpret_cast<const uint4*>(x + i);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < VEC; j++) f(i + j, Cvt<T>::to_f(e[j]));
    }
    for (int i = a1 + tid; i < c1; i += NT) f(i, ldf(x + i));
  } else {
    for (int i = c0 + tid; i < c1; i += NT) f(i, ldf(x + i));
  }
}

__device__ __forceinline__ void merge_max(const RowWs* ws, int chunks, float& lmax, int& bi) {
  // every thread of warp 0 ends with the row's max and arg-max (lowest index among equals)
  int l = threadIdx.x & 31;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int c = l; c < chunks; c += 32) {
    float v = __ldcg(&ws->pv[c]);
    int i = __ldcg(&ws->pi[c]);
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  lmax = best;
  bi = idx == 0x7fffffff ? 0 : idx;
}

__device__ __forceinline__ u64 to_fx(float q) { return __float2ull_rn(q * FX_ONE); }
__device__ __forceinline__ int bin_of(float u) {
  int b = (int)(u * BINS_PER_U);
  return b < 0 ? 0 : (b > NB - 1 ? NB - 1 : b);
}
// sub-bin of a token that lies in bin b
__device__ __forceinline__ int sub_bin_of(float u, int b) {
  int s = (int)((u * BINS_PER_U - (float)b) * (float)NB);
  return s < 0 ? 0 : (s > NB - 1 ? NB - 1 : s);
}
// the tokens of a row fall into three classes against the boundary (b*, s*): kept whole, listed, dropped
__device__ __forceinline__ bool above_boundary(int b, float u, int b_star, int refined, int s_star) {
  return b < b_star || (refined && b == b_star && sub_bin_of(u, b) < s_star);
}
__device__ __forceinline__ bool on_boundary(int b, float u, int b_star, int refined, int s_star) {
  return b == b_star && (!refined || sub_bin_of(u, b) == s_star);
}

template <typename T>
__global__ void __launch_bounds__(NT) sample_max_kernel(const T* __restrict__ logits, RowWs* __restrict__ wsa, int V,
                                                        size_t stride, int chunk, int chunks) {
  __shared__ float sv[NT / 32];
  __shared__ int si[NT / 32];
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
  RowWs* ws = wsa + row;
  for (int i = c * NT + tid; i < NB; i += chunks * NT) { ws->cnt[i] = 0; ws->mass[i] = 0; ws->cnt2[i] = 0; ws->mass2[i] = 0; }
  const T* x = logits + (size_t)row * stride;
  int c0 = c * chunk, c1 = min(V, c0 + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for_tokens(x, c0, c1, [&](int i, float v) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    best = tid < NT / 32 ? sv[tid] : -INFINITY;
    bi = tid < NT / 32 ? si[tid] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (tid == 0) { ws->pv[c] = best; ws->pi[c] = bi; }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) sample_hist_kernel(const T* __restrict__ logits,
                                                         const float* __restrict__ temperature,
                                                         const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                         const float* __restrict__ min_p, RowWs* __restrict__ wsa,
                                                         int V, size_t stride, int chunk, int chunks) {
  // the mass of a bin is summed as two 16-bit halves of the 2^-32 fixed-point value: 32-bit shared-memory adds, and no
  // half can overflow within one chunk (at most 65536 tokens)
  __shared__ unsigned h_cnt[NB], h_hi[NB], h_lo[NB];
  __shared__ float s_lmax;
  __shared__ int s_last;
  __shared__ int s_wc[NT / 32];
  __shared__ u64 s_wm[NT / 32];
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
  float temp = temperature[row];
  if (temp <= 0.f) return;          // greedy rows: pass 3 writes the arg-max
  RowWs* ws = wsa + row;
  for (int i = tid; i < NB; i += NT) { h_cnt[i] = 0; h_hi[i] = 0; h_lo[i] = 0; }
  if (tid < 32) {
    float lm; int bi;
    merge_max(ws, chunks, lm, bi);
    if (tid == 0) s_lmax = lm;
  }
  __syncthreads();
  float lmax = s_lmax, inv_t = 1.f / fmaxf(temp, 1e-6f);
  const T* x = logits + (size_t)row * stride;
  int c0 = c * chunk, c1 = min(V, c0 + chunk);
  int far_cnt = 0;                  // u beyond the histogram: one shared bin, summed in registers first
  u64 far_mass = 0;
  for_tokens(x, c0, c1, [&](int i, float l) {
    float u = (lmax - l) * inv_t;
    u64 fx = to_fx(__expf(-u));
    int b = bin_of(u);
    if (b == NB - 1) { far_cnt++; far_mass += fx; }
    else {
      atomicAdd(&h_cnt[b], 1u);
      atomicAdd(&h_hi[b], (unsigned)(fx >> 16));
      atomicAdd(&h_lo[b], (unsigned)(fx & 0xffffu));
    }
  });
  if (__any_sync(0xffffffffu, far_cnt)) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      far_cnt += __shfl_xor_sync(0xffffffffu, far_cnt, o);
      far_mass += __shfl_xor_sync(0xffffffffu, far_mass, o);
    }
    if ((tid & 31) == 0 && far_cnt) { atomicAdd(&ws->cnt[NB - 1], far_cnt); atomicAdd(&ws->mass[NB - 1], far_mass); }
  }
  __syncthreads();
  for (int i = tid; i < NB; i += NT)
    if (h_cnt[i]) { atomicAdd(&ws->cnt[i], (int)h_cnt[i]); atomicAdd(&ws->mass[i], ((u64)h_hi[i] << 16) + h_lo[i]); }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&ws->ticket2, 1) == chunks - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- the row's last CTA: find the boundary bin.  Thread t owns bins [2t, 2t+2). ----
  int k = top_k[row];
  if (k <= 0 || k > V) k = V;
  float tp = top_p[row];
  int n0 = __ldcg(&ws->cnt[2 * tid]), n1 = __ldcg(&ws->cnt[2 * tid + 1]);
  u64 m0 = __ldcg(&ws->mass[2 * tid]), m1 = __ldcg(&ws->mass[2 * tid + 1]);
  int cs = n0 + n1;
  u64 ms = m0 + m1;
  // inclusive scan over threads (warp shuffles, then over the 16 warp totals)
  int lane = tid & 31, w = tid >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int oc = __shfl_up_sync(0xffffffffu, cs, o);
    u64 om = __shfl_up_sync(0xffffffffu, ms, o);
    if (lane >= o) { cs += oc; ms += om; }
  }
  if (lane == 31) { s_wc[w] = cs; s_wm[w] = ms; }
  __syncthreads();
  int pc = 0;
  u64 pm = 0, total = 0;
  for (int j = 0; j < NT / 32; j++) {
    if (j < w) { pc += s_wc[j]; pm += s_wm[j]; }
    total += s_wm[j];
  }
  int c_excl = pc + cs - (n0 + n1);       // tokens in bins below 2t
  u64 m_excl = pm + ms - (m0 + m1);
  u64 pmass = tp >= 1.f ? ~0ull : (u64)((double)tp * (double)total);
  if (tid == 0) {
    ws->pmass = pmass;
    ws->b_star = NB; ws->resolve = 0; ws->c_cnt = 0; ws->c_mass = 0; ws->fallback = 0; ws->refine = 0; ws->s_star = NB;
    ws->ticket2 = 0;
  }
  __syncthreads();
  // bin b is kept whole iff  C(b+1) <= k  and  M(b+1) <= pmass;  it is dropped whole iff  C(b) >= k  or  M(b) >= pmass;
  // the predicate is monotone in b, so exactly one bin (or none) is neither
  float mp = min_p[row];
#pragma unroll
  for (int j = 0; j < 2; j++) {
    int b = 2 * tid + j;
    int cb = j ? c_excl + n0 : c_excl, cb1 = cb + (j ? n1 : n0);
    u64 mb = j ? m_excl + m0 : m_excl, mb1 = mb + (j ? m1 : m0);
    bool whole = cb1 <= k && mb1 <= pmass;
    bool prev_whole = b == 0 ? true : (cb <= k && mb <= pmass);
    if (!whole && prev_whole) {           // first bin that is not kept whole
      bool dropped = cb >= k || mb >= pmass;
      int n = j ? n1 : n0;
      // a bin entirely under the min-p floor needs no threshold: min-p drops its tokens anyway
      bool under_floor = __expf(-(float)b / BINS_PER_U) * 1.001f < mp;
      ws->b_star = b;
      ws->c_cnt = cb;
      ws->c_mass = mb;
      if (!dropped && !under_floor) {
        if (n <= CAP) ws->resolve = 1; else ws->refine = 1;
      }
    }
  }
}

// Second level, for rows whose boundary bin is too full: the same histogram over that bin alone (CTAs of other rows
// return at once), and the same scan, continued from the count and mass of the bins below it.
template <typename T>
__global__ void __launch_bounds__(NT) sample_refine_kernel(const T* __restrict__ logits,
                                                           const float* __restrict__ temperature,
                                                           const int* __restrict__ top_k, RowWs* __restrict__ wsa, int V,
                                                           size_t stride, int chunk, int chunks) {
  __shared__ unsigned h_cnt[NB], h_hi[NB], h_lo[NB];
  __shared__ float s_lmax;
  __shared__ int s_last;
  __shared__ int s_wc[NT / 32];
  __shared__ u64 s_wm[NT / 32];
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
  RowWs* ws = wsa + row;
  float temp = temperature[row];
  if (temp <= 0.f || !__ldcg(&ws->refine)) return;
  for (int i = tid; i < NB; i += NT) { h_cnt[i] = 0; h_hi[i] = 0; h_lo[i] = 0; }
  if (tid < 32) {
    float lm; int bi;
    merge_max(ws, chunks, lm, bi);
    if (tid == 0) s_lmax = lm;
  }
  __syncthreads();
  float lmax = s_lmax, inv_t = 1.f / fmaxf(temp, 1e-6f);
  const int b_star = __ldcg(&ws->b_star);
  const T* x = logits + (size_t)row * stride;
  int c0 = c * chunk, c1 = min(V, c0 + chunk);
  for_tokens(x, c0, c1, [&](int i, float l) {
    float u = (lmax - l) * inv_t;
    if (bin_of(u) != b_star) return;
    u64 fx = to_fx(__expf(-u));
    int sb = sub_bin_of(u, b_star);
    atomicAdd(&h_cnt[sb], 1u);
    atomicAdd(&h_hi[sb], (unsigned)(fx >> 16));
    atomicAdd(&h_lo[sb], (unsigned)(fx & 0xffffu));
  });
  __syncthreads();
  for (int i = tid; i < NB; i += NT)
    if (h_cnt[i]) { atomicAdd(&ws->cnt2[i], (int)h_cnt[i]); atomicAdd(&ws->mass2[i], ((u64)h_hi[i] << 16) + h_lo[i]); }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&ws->ticket_r, 1) == chunks - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- the row's last CTA: the boundary sub-bin.  Thread t owns sub-bins [2t, 2t+2). ----
  int k = top_k[row];
  if (k <= 0 || k > V) k = V;
  int n0 = __ldcg(&ws->cnt2[2 * tid]), n1 = __ldcg(&ws->cnt2[2 * tid + 1]);
  u64 m0 = __ldcg(&ws->mass2[2 * tid]), m1 = __ldcg(&ws->mass2[2 * tid + 1]);
  int cs = n0 + n1;
  u64 ms = m0 + m1;
  int lane = tid & 31, w = tid >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int oc = __shfl_up_sync(0xffffffffu, cs, o);
    u64 om = __shfl_up_sync(0xffffffffu, ms, o);
    if (lane >= o) { cs += oc; ms += om; }
  }
  if (lane == 31) { s_wc[w] = cs; s_wm[w] = ms; }
  __syncthreads();
  const int base_c = __ldcg(&ws->c_cnt);
  const u64 base_m = __ldcg(&ws->c_mass), pmass = __ldcg(&ws->pmass);
  int pc = base_c;
  u64 pm = base_m;
  for (int j = 0; j < w; j++) { pc += s_wc[j]; pm += s_wm[j]; }
  int c_excl = pc + cs - (n0 + n1);       // tokens above sub-bin 2t (the lower bins included)
  u64 m_excl = pm + ms - (m0 + m1);
  __syncthreads();
  if (tid == 0) { ws->ticket_r = 0; ws->s_star = NB; }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 2; j++) {
    int sb = 2 * tid + j;
    int cb = j ? c_excl + n0 : c_excl, cb1 = cb + (j ? n1 : n0);
    u64 mb = j ? m_excl + m0 : m_excl, mb1 = mb + (j ? m1 : m0);
    bool whole = cb1 <= k && mb1 <= pmass;
    bool prev_whole = cb <= k && mb <= pmass;       // true for sub-bin 0: the bin was not dropped whole
    if (!whole && prev_whole) {
      bool dropped = cb >= k || mb >= pmass;
      int n = j ? n1 : n0;
      ws->s_star = sb;
      ws->c_cnt = cb;
      ws->c_mass = mb;
      if (!dropped) {
        if (n <= CAP) ws->resolve = 1; else ws->fallback = 1;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) sample_draw_kernel(const T* __restrict__ logits,
                                                         const float* __restrict__ temperature,
                                                         const int* __restrict__ top_k, const float* __restrict__ min_p,
                                                         const float* __restrict__ uniform, RowWs* __restrict__ wsa,
                                                         int* __restrict__ out, int* __restrict__ need, int V,
                                                         size_t stride, int chunk, int chunks) {
  __shared__ float s_lmax;
  __shared__ int s_bi, s_last, s_pick, s_chunk;
  __shared__ u64 s_red[NT / 32];
  __shared__ u64 s_tau, s_target, s_before;
  __shared__ u64 s_cm[MAX_CHUNKS];
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.y, c = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  RowWs* ws = wsa + row;
  float temp = temperature[row];
  if (tid < 32) {
    float lm; int bi;
    merge_max(ws, chunks, lm, bi);
    if (tid == 0) { s_lmax = lm; s_bi = bi; }
  }
  __syncthreads();
  int bi = s_bi;
  if (temp <= 0.f) {
    if (c == 0 && tid == 0) { out[row] = bi; need[row] = 0; }
    return;
  }
  if (__ldcg(&ws->fallback)) {
    if (c == 0 && tid == 0) need[row] = 1;
    return;
  }
  float lmax = s_lmax, inv_t = 1.f / fmaxf(temp, 1e-6f), mp = min_p[row];
  int b_star = __ldcg(&ws->b_star), resolve = __ldcg(&ws->resolve);
  const int refined = __ldcg(&ws->refine), s_star = __ldcg(&ws->s_star);
  const T* x = logits + (size_t)row * stride;
  int c0 = c * chunk, c1 = min(V, c0 + chunk);
  u64 loc = 0;
  for_tokens(x, c0, c1, [&](int i, float l) {
    float u = (lmax - l) * inv_t;
    float q = __expf(-u);
    int b = bin_of(u);
    if (resolve && on_boundary(b, u, b_star, refined, s_star)) {
      int slot = atomicAdd(&ws->n_list, 1);
      if (slot < CAP) { ws->list[slot] = to_fx(q); ws->list_chunk[slot] = i == bi ? -1 : c; }  // the arg-max is counted below
    }
    bool keep = (above_boundary(b, u, b_star, refined, s_star) && q >= mp) || i == bi;
    if (keep) loc += to_fx(q);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) loc += __shfl_xor_sync(0xffffffffu, loc, o);
  if (lane == 0) s_red[w] = loc;
  __syncthreads();
  if (tid == 0) {
    u64 t = 0;
    for (int j = 0; j < NT / 32; j++) t += s_red[j];
    ws->chunk_mass[c] = t;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&ws->ticket3, 1) == chunks - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- the row's last CTA ----
  for (int j = tid; j < chunks; j += NT) s_cm[j] = __ldcg(&ws->chunk_mass[j]);
  if (tid == 0) s_tau = ~0ull;
  __syncthreads();
  if (resolve) {
    // exact threshold inside the boundary bin: entry i is kept iff the tokens strictly above it (the lower bins plus
    // the larger entries of this bin) number fewer than k and weigh less than top_p * total
    int n = min(__ldcg(&ws->n_list), CAP);
    int k = top_k[row];
    if (k <= 0 || k > V) k = V;
    u64 pmass = __ldcg(&ws->pmass), cm = __ldcg(&ws->c_mass);
    int cc = __ldcg(&ws->c_cnt);
    u64 fmin = to_fx(mp);
    u64 lowest = ~0ull;
    for (int i = tid; i < n; i += NT) {
      u64 me = __ldcg(&ws->list[i]);
      int gt = 0;
      u64 mgt = 0;
      for (int j = 0; j < n; j++) {
        u64 o = __ldcg(&ws->list[j]);
        if (o > me) { gt++; mgt += o; }
      }
      if (cc + gt < k && cm + mgt < pmass && me < lowest) lowest = me;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      u64 ov = __shfl_xor_sync(0xffffffffu, lowest, o);
      lowest = ov < lowest ? ov : lowest;
    }
    if (lane == 0 && lowest != ~0ull) atomicMin(&s_tau, lowest);
    __syncthreads();
    u64 tau = s_tau;
    // the kept entries join their chunks (min-p applies to them like to everyone else)
    for (int i = tid; i < n; i += NT) {
      u64 me = __ldcg(&ws->list[i]);
      int ch = __ldcg(&ws->list_chunk[i]);
      if (me >= tau && me >= fmin && ch >= 0) atomicAdd(&s_cm[ch], me);
    }
    __syncthreads();
  }
  if (tid == 0) {
    u64 total = 0;
    for (int j = 0; j < chunks; j++) total += s_cm[j];
    double tgt = (double)uniform[row] * (double)total;
    u64 target = (u64)tgt;
    if (target >= total) target = total ? total - 1 : 0;
    u64 run = 0;
    int cs = chunks - 1;
    for (int j = 0; j < chunks; j++) {
      if (run + s_cm[j] > target) { cs = j; break; }
      run += s_cm[j];
    }
    s_chunk = cs;
    s_target = target;
    s_before = run;
    s_pick = -1;
    ws->ticket3 = 0;
    ws->n_list = 0;
  }
  __syncthreads();
  // walk the chosen chunk: contiguous span per thread, scan of the span sums, the owning thread finds the token
  u64 tau = s_tau, fmin = to_fx(mp);
  int cs = s_chunk;
  int d0 = cs * chunk, d1 = min(V, d0 + chunk);
  int span = (d1 - d0 + NT - 1) / NT;
  int e0 = d0 + tid * span, e1 = min(d1, e0 + span);
  u64 mine = 0;
  for (int i = e0; i < e1; i++) {
    float u = (lmax - ldf(x + i)) * inv_t;
    float q = __expf(-u);
    int b = bin_of(u);
    u64 fx = to_fx(q);
    bool keep = (above_boundary(b, u, b_star, refined, s_star) && q >= mp) ||
                (resolve && on_boundary(b, u, b_star, refined, s_star) && fx >= tau && fx >= fmin) || i == bi;
    if (keep) mine += fx;
  }
  u64 incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u64 ov = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += ov;
  }
  if (lane == 31) s_red[w] = incl;
  __syncthreads();
  u64 before = s_before;
  for (int j = 0; j < w; j++) before += s_red[j];
  before += incl - mine;
  u64 target = s_target;
  if (mine && target >= before && target < before + mine) {
    u64 run = before;
    for (int i = e0; i < e1; i++) {
      float u = (lmax - ldf(x + i)) * inv_t;
      float q = __expf(-u);
      int b = bin_of(u);
      u64 fx = to_fx(q);
      bool keep = (above_boundary(b, u, b_star, refined, s_star) && q >= mp) ||
                  (resolve && on_boundary(b, u, b_star, refined, s_star) && fx >= tau && fx >= fmin) || i == bi;
      if (!keep) continue;
      run += fx;
      if (run > target) { s_pick = i; break; }
    }
  }
  __syncthreads();
  if (tid == 0) {
    out[row] = s_pick >= 0 ? s_pick : bi;
    need[row] = 0;
  }
}

}  // namespace

static inline size_t need_bytes(int cap_rows) { return ((size_t)cap_rows * 4 + 255) & ~(size_t)255; }

// bytes for up to cap_rows rows: the per-row switches of the bisection kernel, then one RowWs per row
EXO_API long exo_sample_workspace(int cap_rows) { return (long)(need_bytes(cap_rows) + (size_t)cap_rows * sizeof(RowWs)); }

EXO_API int exo_sample_chunks(int rows, int V) {
  int c = (3 * 148 + rows - 1) / rows;
  int cap = (V + 2047) / 2048;
  c = c < cap ? c : cap;
  return c < 1 ? 1 : (c > MAX_CHUNKS ? MAX_CHUNKS : c);
}

// the single-CTA bisection sampler (basic.cu) with a per-row switch
int exo_sample_rows(const void* logits, const float* temperature, const int* top_k, const float* top_p,
                    const float* min_p, const float* uniform, int* out, const int* need, int rows, int V, long stride,
                    int dtype, cudaStream_t st);

// workspace: exo_sample_workspace(cap_rows) bytes with cap_rows >= rows, zeroed once by the caller and then only ever
// touched by these kernels
EXO_API int exo_sample_fast(const void* logits, const float* temperature, const int* top_k, const float* top_p,
                            const float* min_p, const float* uniform, int* out, void* workspace, int cap_rows, int rows,
                            int V, long stride, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (rows > cap_rows) return (int)cudaErrorInvalidValue;
  int* need = (int*)workspace;
  RowWs* ws = (RowWs*)((char*)workspace + need_bytes(cap_rows));
  int chunks = exo_sample_chunks(rows, V);
  int chunk = (V + chunks - 1) / chunks;
  dim3 grid(chunks, rows);
  cudaError_t e;
#define LAUNCH3(T)                                                                                                    \
  e = launch_pdl(sample_max_kernel<T>, grid, dim3(NT), 0, st, (const T*)logits, ws, V, (size_t)stride, chunk, chunks); \
  if (e != cudaSuccess) return (int)e;                                                                                \
  e = launch_pdl(sample_hist_kernel<T>, grid, dim3(NT), 0, st, (const T*)logits, temperature, top_k, top_p, min_p, ws, \
                 V, (size_t)stride, chunk, chunks);                                                                   \
  if (e != cudaSuccess) return (int)e;                                                                                \
  e = launch_pdl(sample_refine_kernel<T>, grid, dim3(NT), 0, st, (const T*)logits, temperature, top_k, ws, V,          \
                 (size_t)stride, chunk, chunks);                                                                      \
  if (e != cudaSuccess) return (int)e;                                                                                \
  e = launch_pdl(sample_draw_kernel<T>, grid, dim3(NT), 0, st, (const T*)logits, temperature, top_k, min_p, uniform,   \
                 ws, out, need, V, (size_t)stride, chunk, chunks);                                                    \
  if (e != cudaSuccess) return (int)e;
  if (dtype == EXO_BF16) { LAUNCH3(__nv_bfloat16) } else { LAUNCH3(float) }
#undef LAUNCH3
  EXO_CHECK_LAUNCH();
  return exo_sample_rows(logits, temperature, top_k, top_p, min_p, uniform, out, need, rows, V, stride, dtype, st);
}
