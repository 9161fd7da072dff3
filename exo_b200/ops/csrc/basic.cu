// Row-wise and element-wise hot ops: fused residual-add + RMSNorm, SwiGLU, embedding gather,
// fused per-head norm + RoPE + paged-KV append, argmax and filtered sampling.
// All are HBM/latency-bound; they exist to keep each decode step to a handful of launches.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// h = x (+ residual); out = h * rsqrt(mean(h^2) + eps) * w.   One CTA per row.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                               T* __restrict__ out, T* __restrict__ h_out, int cols, float eps) {
  __shared__ float red[32];
  size_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const T* rr = res ? res + row * cols : nullptr;
  pdl_trigger();
  pdl_wait();
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float h = Cvt<T>::to_f(xr[c]);
    if (rr) {
      h += Cvt<T>::to_f(rr[c]);
      T hq = Cvt<T>::from_f(h);
      h_out[row * cols + c] = hq;
      h = Cvt<T>::to_f(hq);  // normalise the value the residual stream actually keeps
    }
    ss += h * h;
  }
  float tot = block_sum(ss, red);
  float rstd = rsqrtf(tot / cols + eps);
  // second pass re-reads the row (each thread reads back exactly what it wrote: L1/L2 resident)
  const T* hr = rr ? h_out + row * cols : xr;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[row * cols + c] = Cvt<T>::from_f(Cvt<T>::to_f(hr[c]) * rstd * Cvt<T>::to_f(w[c]));
}

// bf16 rows of up to 512 * VPT * 8 values: every thread keeps its 16-byte vectors in registers, so the row is read
// once (x and the residual), summed, and written once (the new residual stream and the normalised row).
template <int VPT>
__global__ void __launch_bounds__(512) rmsnorm_vec_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res,
                                                          const uint4* __restrict__ w, uint4* __restrict__ out,
                                                          uint4* __restrict__ h_out, int nvec, float eps) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * nvec;
  pdl_trigger();
  pdl_wait();
  float h[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int v = threadIdx.x + j * 512;
    if (v < nvec) {
      unpack8(x[base + v], h[j]);
      if (res) {
        float r[8];
        unpack8(res[base + v], r);
#pragma unroll
        for (int e = 0; e < 8; e++) h[j][e] += r[e];
        const uint4 hq = pack8(h[j]);
        h_out[base + v] = hq;
        unpack8(hq, h[j]);      // normalise the value the residual stream actually keeps
      }
#pragma unroll
      for (int e = 0; e < 8; e++) ss += h[j][e] * h[j][e];
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (nvec * 8) + eps);
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int v = threadIdx.x + j * 512;
    if (v < nvec) {
      float wf[8];
      unpack8(w[v], wf);
#pragma unroll
      for (int e = 0; e < 8; e++) h[j][e] = h[j][e] * rstd * wf[e];
      out[base + v] = pack8(h[j]);
    }
  }
}

EXO_API int exo_rmsnorm(const void* x, const void* res, const void* w, void* out, void* h_out, int rows, int cols,
                        float eps, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (res && !h_out) return -2;
  int threads = cols >= 2048 ? 512 : 256;
  cudaError_t e;
  const bool aligned = !(((uintptr_t)x | (uintptr_t)res | (uintptr_t)w | (uintptr_t)out | (uintptr_t)h_out) & 15);
  if (dtype == EXO_BF16 && cols % 8 == 0 && cols >= 1024 && cols <= 512 * 4 * 8 && aligned) {
    const int nvec = cols / 8;
#define RV(V)                                                                                                        \
  e = launch_pdl(rmsnorm_vec_kernel<V>, dim3(rows), dim3(512), 0, st, (const uint4*)x, (const uint4*)res, (const uint4*)w, \
                 (uint4*)out, (uint4*)h_out, nvec, eps)
    if (nvec <= 512) RV(1);
    else if (nvec <= 1024) RV(2);
    else RV(4);
#undef RV
    if (e != cudaSuccess) return (int)e;
    EXO_CHECK_LAUNCH();
    return 0;
  }
  if (dtype == EXO_BF16)
    e = launch_pdl(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, st, (const __nv_bfloat16*)x,
                   (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (__nv_bfloat16*)h_out, cols,
                   eps);
  else
    e = launch_pdl(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, st, (const float*)x, (const float*)res,
                   (const float*)w, (float*)out, (float*)h_out, cols, eps);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// out[r, c] = silu(gu[r, c]) * gu[r, F + c]
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t rows, int F) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t n = rows * (size_t)F;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / F;
    int c = (int)(i - r * F);
    float g = Cvt<T>::to_f(gu[r * 2 * F + c]), u = Cvt<T>::to_f(gu[r * 2 * F + F + c]);
    out[i] = Cvt<T>::from_f(silu_f(g) * u);
  }
}

// out[r, c] = min(silu(gu[r, c]), limit) * clamp(gu[r, F + c], -limit, limit)      (Step-3.5's clamped SwiGLU)
template <typename T>
__global__ void swiglu_clamp_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t rows, int F, float limit) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t n = rows * (size_t)F;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / F;
    int c = (int)(i - r * F);
    float g = Cvt<T>::to_f(gu[r * 2 * F + c]), u = Cvt<T>::to_f(gu[r * 2 * F + F + c]);
    out[i] = Cvt<T>::from_f(fminf(silu_f(g), limit) * fminf(fmaxf(u, -limit), limit));
  }
}

EXO_API int exo_swiglu_clamp(const void* gu, void* out, int rows, int F, float limit, int dtype, cudaStream_t st) {
  size_t n = (size_t)rows * F;
  if (n == 0) return 0;
  if (!(limit > 0.f)) return -2;
  int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == EXO_BF16)
    swiglu_clamp_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F, limit);
  else
    swiglu_clamp_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, (float*)out, rows, F, limit);
  EXO_CHECK_LAUNCH();
  return 0;
}

// out[r, c] = gelu_tanh(gu[r, c]) * gu[r, F + c]
template <typename T>
__global__ void geglu_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t rows, int F) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t n = rows * (size_t)F;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / F;
    int c = (int)(i - r * F);
    float g = Cvt<T>::to_f(gu[r * 2 * F + c]), u = Cvt<T>::to_f(gu[r * 2 * F + F + c]);
    float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    out[i] = Cvt<T>::from_f(0.5f * g * (1.f + t) * u);
  }
}

EXO_API int exo_geglu(const void* gu, void* out, int rows, int F, int dtype, cudaStream_t st) {
  size_t n = (size_t)rows * F;
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == EXO_BF16)
    geglu_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F);
  else
    geglu_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, (float*)out, rows, F);
  EXO_CHECK_LAUNCH();
  return 0;
}

EXO_API int exo_swiglu(const void* gu, void* out, int rows, int F, int dtype, cudaStream_t st) {
  size_t n = (size_t)rows * F;
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == EXO_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F);
  else
    swiglu_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, (float*)out, rows, F);
  EXO_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// out[t, :] = table[ids[t], :]
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                 int cols, int vocab) {
  int id = ids[blockIdx.x];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* src = table + (size_t)id * cols;
  T* dst = out + (size_t)blockIdx.x * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = src[c];
}

EXO_API int exo_embedding(const void* table, const int* ids, void* out, int T_, int cols, int vocab, int dtype,
                          cudaStream_t st) {
  if (T_ == 0) return 0;
  if (dtype == EXO_BF16)
    embedding_kernel<__nv_bfloat16><<<T_, 256, 0, st>>>((const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, cols, vocab);
  else
    embedding_kernel<float><<<T_, 256, 0, st>>>((const float*)table, ids, (float*)out, cols, vocab);
  EXO_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// Fused: split qkv, optional per-head RMSNorm on q/k, RoPE (half-rotation, first rot dims) on q/k,
// write q to q_out [T, n_q, D], k/v into the paged caches at slot[t].  One warp per (token, head).
// Lane l owns elements j*32+l; the RoPE partner i+rot/2 stays in the same lane because rot % 64 == 0.
// ------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void qk_rope_append_kernel(const T* __restrict__ qkv, const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, float mscale, int n_q, int n_kv, int rot,
                                      T* __restrict__ q_out, T* __restrict__ kcache, T* __restrict__ vcache,
                                      const int* __restrict__ slots, const T* __restrict__ q_norm,
                                      const T* __restrict__ k_norm, float eps, int T_, int v_unit_norm) {
  constexpr int E = D / 32;
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int heads = n_q + 2 * n_kv;
  if (warp >= T_ * heads) return;
  int t = warp / heads, hd = warp - t * heads;
  const T* src = qkv + (size_t)t * heads * D + (size_t)hd * D;
  float v[E];
#pragma unroll
  for (int j = 0; j < E; j++) v[j] = Cvt<T>::to_f(src[j * 32 + lane]);
  bool is_q = hd < n_q, is_k = !is_q && hd < n_q + n_kv;
  if (!is_q && !is_k && v_unit_norm) {      // v heads normalised without a weight (Gemma-4)
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < E; j++) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
    for (int j = 0; j < E; j++) v[j] *= rstd;
  }
  if (is_q || is_k) {
    const T* nw = is_q ? q_norm : k_norm;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < E; j++) ss += v[j] * v[j];
      ss = warp_sum(ss);
      float rstd = rsqrtf(ss / D + eps);
#pragma unroll
      for (int j = 0; j < E; j++) {
        // round as the unfused op would (norm output is stored in T before RoPE)
        v[j] = Cvt<T>::to_f(Cvt<T>::from_f(v[j] * rstd * Cvt<T>::to_f(nw[j * 32 + lane])));
      }
    }
    float pos = (float)positions[t];
    int half = rot / 2;
    int EH = half / 32;  // elements per lane in each rotated half
    for (int j = 0; j < EH; j++) {
      int i = j * 32 + lane;
      float s, c;
      sincosf(pos * inv_freq[i], &s, &c);
      s *= mscale;
      c *= mscale;
      float a = v[j], b = v[j + EH];
      v[j] = a * c - b * s;
      v[j + EH] = b * c + a * s;
    }
  }
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * n_q + hd) * D;
  } else {
    size_t slot = (size_t)slots[t];
    int kvh = is_k ? hd - n_q : hd - n_q - n_kv;
    dst = (is_k ? kcache : vcache) + (slot * n_kv + kvh) * D;
  }
#pragma unroll
  for (int j = 0; j < E; j++) dst[j * 32 + lane] = Cvt<T>::from_f(v[j]);
}

EXO_API int exo_qk_rope_append(const void* qkv, const int* positions, const float* inv_freq, float mscale, int n_q,
                               int n_kv, int head_dim, int rot, void* q_out, void* kcache, void* vcache,
                               const int* slots, const void* q_norm, const void* k_norm, float eps, int T_, int dtype,
                               int v_unit_norm, cudaStream_t st) {
  if (T_ == 0) return 0;
  if (rot % 64 != 0 || rot > head_dim) return -2;
  long warps = (long)T_ * (n_q + 2 * n_kv);
  int blocks = (int)((warps * 32 + 255) / 256);
#define LAUNCH(TT, DD)                                                                                              \
  qk_rope_append_kernel<TT, DD><<<blocks, 256, 0, st>>>((const TT*)qkv, positions, inv_freq, mscale, n_q, n_kv, rot, \
                                                        (TT*)q_out, (TT*)kcache, (TT*)vcache, slots,                 \
                                                        (const TT*)q_norm, (const TT*)k_norm, eps, T_, v_unit_norm)
  if (dtype == EXO_BF16) {
    if (head_dim == 128) LAUNCH(__nv_bfloat16, 128);
    else if (head_dim == 64) LAUNCH(__nv_bfloat16, 64);
    else if (head_dim == 256) LAUNCH(__nv_bfloat16, 256);
    else if (head_dim == 512) LAUNCH(__nv_bfloat16, 512);
    else return -2;
  } else {
    if (head_dim == 128) LAUNCH(float, 128);
    else if (head_dim == 64) LAUNCH(float, 64);
    else if (head_dim == 256) LAUNCH(float, 256);
    else if (head_dim == 512) LAUNCH(float, 512);
    else return -2;
  }
#undef LAUNCH
  EXO_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// argmax over the last dim, two stages: grid (chunks, rows) finds per-chunk maxima, one warp per row
// merges them.  Ties resolve to the lowest index.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void argmax_combine(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}

template <typename T>
__global__ void argmax_partial_kernel(const T* __restrict__ logits, float* __restrict__ pv, int* __restrict__ pi,
                                      int V, size_t stride, int chunk) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_trigger();
  pdl_wait();
  const T* row = logits + (size_t)blockIdx.y * stride;
  int c0 = blockIdx.x * chunk, c1 = min(V, c0 + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
    float v = Cvt<T>::to_f(row[c]);
    if (v > best) { best = v; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    int nw = blockDim.x >> 5;
    best = l < nw ? sv[l] : -INFINITY;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (l == 0) { pv[blockIdx.y * gridDim.x + blockIdx.x] = best; pi[blockIdx.y * gridDim.x + blockIdx.x] = bi; }
  }
}

__global__ void argmax_merge_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int* __restrict__ out,
                                    int chunks) {
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.x, l = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = l; c < chunks; c += 32) argmax_combine(best, bi, pv[row * chunks + c], pi[row * chunks + c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (l == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

EXO_API int exo_argmax_chunks(int rows, int V) {
  int c = (4 * 148 + rows - 1) / rows;
  int cap = (V + 1023) / 1024;
  c = c < cap ? c : cap;
  return c < 1 ? 1 : (c > 256 ? 256 : c);
}

// scratch: chunks*rows floats (pv) and chunks*rows ints (pi)
EXO_API int exo_argmax(const void* logits, int* out, float* pv, int* pi, int chunks, int rows, int V, long stride,
                       int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  int chunk = (V + chunks - 1) / chunks;
  dim3 grid(chunks, rows);
  cudaError_t e;
  if (dtype == EXO_BF16)
    e = launch_pdl(argmax_partial_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (const __nv_bfloat16*)logits, pv, pi,
                   V, (size_t)stride, chunk);
  else
    e = launch_pdl(argmax_partial_kernel<float>, grid, dim3(256), 0, st, (const float*)logits, pv, pi, V,
                   (size_t)stride, chunk);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(argmax_merge_kernel, dim3(rows), dim3(32), 0, st, (const float*)pv, (const int*)pi, out, chunks);
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// Filtered sampling.  One CTA (1024 threads) per row.
//   p_i = softmax(l / T);  keep i  iff  #{p > p_i} < top_k  and  mass{p > p_i} < top_p  and  p_i >= min_p * p_max
//   then inverse CDF over the kept tokens in vocabulary order with the caller's uniform number.
// The keep set is {p >= tau}; tau is found by bisection on the (monotone) predicate.  T <= 0 → argmax.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void sample_kernel(const T* __restrict__ logits, const float* __restrict__ temperature,
                              const int* __restrict__ top_k, const float* __restrict__ top_p,
                              const float* __restrict__ min_p, const float* __restrict__ uniform,
                              int* __restrict__ out, const int* __restrict__ need, int V, size_t stride) {
  if (need && !need[blockIdx.x]) return;  // rows the multi-CTA sampler already finished
  __shared__ float red[32];
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float part[1024];
  const T* row = logits + (size_t)blockIdx.x * stride;
  int tid = threadIdx.x, nt = blockDim.x;
  float temp = temperature[blockIdx.x];
  // max (and argmax for greedy rows)
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = tid; c < V; c += nt) {
    float v = Cvt<T>::to_f(row[c]);
    if (v > best) { best = v; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = bi; }
  __syncthreads();
  {
    int l = tid & 31, nw = nt >> 5;
    best = l < nw ? sv[l] : -INFINITY;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
  }
  if (temp <= 0.f) {
    if (tid == 0) out[blockIdx.x] = bi;
    return;
  }
  float inv_t = 1.f / fmaxf(temp, 1e-6f);
  float lmax = best;
  float s = 0.f;
  for (int c = tid; c < V; c += nt) s += __expf((Cvt<T>::to_f(row[c]) - lmax) * inv_t);
  float Z = block_sum(s, red);
  // work with unnormalised q_i = exp((l_i - lmax)/T) in (0, 1]; q_max = 1
  int k = top_k[blockIdx.x];
  if (k <= 0 || k > V) k = V;
  float pmass = top_p[blockIdx.x] * Z;
  float qmin = min_p[blockIdx.x];  // relative to q_max = 1
  // bisection for the smallest tau with  count{q > tau} < k  and  mass{q > tau} < pmass
  float lo = 0.f, hi = 1.f;  // predicate false at lo (unless trivially true), true at hi (count = 0)
  bool trivial = (k >= V) && (top_p[blockIdx.x] >= 1.f);
  if (!trivial) {
    for (int it = 0; it < 26; it++) {
      float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int c = tid; c < V; c += nt) {
        float q = __expf((Cvt<T>::to_f(row[c]) - lmax) * inv_t);
        if (q > mid) { cnt += 1.f; mass += q; }
      }
      cnt = block_sum(cnt, red);
      mass = block_sum(mass, red);
      bool ok = (cnt < (float)k) && (mass < pmass);
      if (ok) hi = mid; else lo = mid;
    }
  } else {
    hi = 0.f;
  }
  // keep {q >= tau}: tau is the largest q value <= hi that is still kept, i.e. keep q > lo when searched
  float tau = trivial ? 0.f : lo;
  float thr = fmaxf(tau, 0.f);
  // contiguous chunk per thread for an index-ordered CDF
  int chunk = (V + nt - 1) / nt;
  int c0 = tid * chunk, c1 = min(V, c0 + chunk);
  float loc = 0.f;
  for (int c = c0; c < c1; c++) {
    float q = __expf((Cvt<T>::to_f(row[c]) - lmax) * inv_t);
    bool keep = (trivial || q > thr) && q >= qmin;
    if (c == bi) keep = true;
    loc += keep ? q : 0.f;
  }
  part[tid] = loc;
  __syncthreads();
  // inclusive scan of part[] (Hillis-Steele, 1024 entries)
  for (int o = 1; o < nt; o <<= 1) {
    float add = tid >= o ? part[tid - o] : 0.f;
    __syncthreads();
    part[tid] += add;
    __syncthreads();
  }
  float total = part[nt - 1];
  float target = uniform[blockIdx.x] * total;
  float before = tid ? part[tid - 1] : 0.f;
  bool mine = (target >= before && target < part[tid]) || (tid == nt - 1 && target >= total);
  if (tid == 0) out[blockIdx.x] = bi;  // fallback, overwritten below by the owning thread
  __syncthreads();
  if (mine && loc > 0.f) {
    float run = before;
    int pick = -1, last_kept = -1;
    for (int c = c0; c < c1; c++) {
      float q = __expf((Cvt<T>::to_f(row[c]) - lmax) * inv_t);
      bool keep = (trivial || q > thr) && q >= qmin;
      if (c == bi) keep = true;
      if (!keep) continue;
      last_kept = c;
      run += q;
      if (run > target) { pick = c; break; }
    }
    if (pick < 0) pick = last_kept;
    if (pick >= 0) out[blockIdx.x] = pick;
  }
}

// need: per-row switch (nullptr = every row); rows whose entry is 0 return at once
int exo_sample_rows(const void* logits, const float* temperature, const int* top_k, const float* top_p,
                    const float* min_p, const float* uniform, int* out, const int* need, int rows, int V, long stride,
                    int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (dtype == EXO_BF16)
    sample_kernel<__nv_bfloat16><<<rows, 1024, 0, st>>>((const __nv_bfloat16*)logits, temperature, top_k, top_p, min_p,
                                                        uniform, out, need, V, (size_t)stride);
  else
    sample_kernel<float><<<rows, 1024, 0, st>>>((const float*)logits, temperature, top_k, top_p, min_p, uniform, out,
                                                need, V, (size_t)stride);
  EXO_CHECK_LAUNCH();
  return 0;
}

EXO_API int exo_sample(const void* logits, const float* temperature, const int* top_k, const float* top_p,
                       const float* min_p, const float* uniform, int* out, int rows, int V, long stride, int dtype,
                       cudaStream_t st) {
  return exo_sample_rows(logits, temperature, top_k, top_p, min_p, uniform, out, nullptr, rows, V, stride, dtype, st);
}
