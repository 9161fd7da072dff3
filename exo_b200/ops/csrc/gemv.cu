// Small-batch linear layers (M <= 8 rows): y = x W^T, weight-bandwidth bound.
//
// Every weight byte is read exactly once with 16-byte streaming loads; each warp produces two
// output rows so that two independent load streams are in flight per lane.  Three fusions remove
// whole launches and activation round trips from the decode step:
//   * prologue RMSNorm: the warp's lanes cover all of K anyway, so sum(x^2) is accumulated in the
//     same loop and y = rstd * (W . (x * norm_w));
//   * epilogue SwiGLU: the warp's two rows are gate row n and up row n + F, it writes silu(g) * u;
//   * epilogue bias / residual add (out may alias residual).
#include "common.cuh"

template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load_stream(const __nv_bfloat16* p, float* f) { unpack8(ld_stream16(p), f); }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    unpack8(*reinterpret_cast<const uint4*>(p), f);
  }
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) { unpack8(u, f); }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load_stream(const float* p, float* f) {
    uint4 u = ld_stream16(p);
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ void load(const float* p, float* f) {
    float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
};

// CTA = 128 threads cooperating on R output rows: the K range is dealt out in 16-byte vectors,
// vector (it * 128 + tid) to thread tid, U vectors per row issued back to back, so a thread has
// U * R independent 16-byte loads in flight and the grid has N / R CTAs — enough outstanding
// bytes to cover HBM latency even for a 4096 x 4096 projection (the whole matrix is in flight).
template <typename T, int M, int R, bool NORM, bool SWIGLU>
__global__ void __launch_bounds__(128)
linear_small_kernel(const T* __restrict__ x, const T* __restrict__ W, const T* __restrict__ bias,
                    const T* residual, T* out, const T* __restrict__ norm_w, float eps, int N, int K, int ldo) {
  constexpr int V = Vec16<T>::N;
  constexpr int U = 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_trigger();  // the next kernel in the stream may begin launching (it waits before reading our output)
  // output rows of this CTA: R consecutive rows, or R/2 (gate, up) pairs when SWIGLU
  int rows[R];
  const int F = N / 2;
#pragma unroll
  for (int i = 0; i < R; i++) {
    if (SWIGLU) rows[i] = min((int)blockIdx.x * (R / 2) + i / 2, F - 1) + (i & 1) * F;
    else rows[i] = min((int)blockIdx.x * R + i, N - 1);
  }
  const T* wp[R];
#pragma unroll
  for (int i = 0; i < R; i++) wp[i] = W + (size_t)rows[i] * K;
  float acc[R][M], ss[M];
#pragma unroll
  for (int m = 0; m < M; m++) {
    ss[m] = 0.f;
#pragma unroll
    for (int i = 0; i < R; i++) acc[i][m] = 0.f;
  }
  const int stride = 128 * V;  // elements covered by the CTA per vector step
  uint4 wv[U][R];
  // first batch of weights is requested BEFORE waiting on the producer of x (weights never change)
#pragma unroll
  for (int u = 0; u < U; u++) {
    int k = (u * 128 + tid) * V;
#pragma unroll
    for (int i = 0; i < R; i++) wv[u][i] = k < K ? ld_stream16(wp[i] + k) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  for (int k0 = 0; k0 < K; k0 += U * stride) {
    uint4 nx[U][R];
    const int kn0 = k0 + U * stride;
    if (kn0 < K) {
#pragma unroll
      for (int u = 0; u < U; u++) {
        int k = kn0 + (u * 128 + tid) * V;
#pragma unroll
        for (int i = 0; i < R; i++) nx[u][i] = k < K ? ld_stream16(wp[i] + k) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      int k = k0 + (u * 128 + tid) * V;
      if (k < K) {
        float nw[V];
        if (NORM) Vec16<T>::load(norm_w + k, nw);
        float wf[R][V];
#pragma unroll
        for (int i = 0; i < R; i++) Vec16<T>::unpack(wv[u][i], wf[i]);
#pragma unroll
        for (int m = 0; m < M; m++) {
          float xf[V];
          Vec16<T>::load(x + (size_t)m * K + k, xf);
#pragma unroll
          for (int j = 0; j < V; j++) {
            float xv = xf[j];
            if (NORM) { ss[m] += xv * xv; xv *= nw[j]; }
#pragma unroll
            for (int i = 0; i < R; i++) acc[i][m] += wf[i][j] * xv;
          }
        }
      }
    }
    if (kn0 < K) {
#pragma unroll
      for (int u = 0; u < U; u++)
#pragma unroll
        for (int i = 0; i < R; i++) wv[u][i] = nx[u][i];
    }
  }
  // reduce: lanes by shuffle, warps through shared memory
  __shared__ float red[4][R * M + M];
#pragma unroll
  for (int m = 0; m < M; m++) {
#pragma unroll
    for (int i = 0; i < R; i++) {
      float v = warp_sum(acc[i][m]);
      if (lane == 0) red[warp][i * M + m] = v;
    }
    if (NORM) {
      float v = warp_sum(ss[m]);
      if (lane == 0) red[warp][R * M + m] = v;
    }
  }
  __syncthreads();
  if (tid < M) {
    const int m = tid;
    float rstd = 1.f;
    if (NORM) rstd = rsqrtf((red[0][R * M + m] + red[1][R * M + m] + red[2][R * M + m] + red[3][R * M + m]) / K + eps);
    float y[R];
#pragma unroll
    for (int i = 0; i < R; i++) {
      y[i] = (red[0][i * M + m] + red[1][i * M + m] + red[2][i * M + m] + red[3][i * M + m]) * rstd;
      if (bias) y[i] += Cvt<T>::to_f(bias[rows[i]]);
    }
    if (SWIGLU) {
#pragma unroll
      for (int i = 0; i < R; i += 2)
        if ((int)blockIdx.x * (R / 2) + i / 2 < F) out[(size_t)m * ldo + rows[i]] = Cvt<T>::from_f(silu_f(y[i]) * y[i + 1]);
    } else {
#pragma unroll
      for (int i = 0; i < R; i++) {
        if ((int)blockIdx.x * R + i < N) {
          float v = y[i];
          if (residual) v += Cvt<T>::to_f(residual[(size_t)m * ldo + rows[i]]);
          out[(size_t)m * ldo + rows[i]] = Cvt<T>::from_f(v);
        }
      }
    }
  }
}

template <typename T, int M>
static int launch_small(const void* x, const void* W, const void* bias, const void* residual, void* out,
                        const void* norm_w, float eps, int N, int K, int swiglu, cudaStream_t st) {
  constexpr int R = M <= 2 ? 4 : 2;
  int blocks = swiglu ? (N / 2 + R / 2 - 1) / (R / 2) : (N + R - 1) / R;
  int ldo = swiglu ? N / 2 : N;
  cudaError_t e;
#define L(NORM, SW)                                                                                             \
  e = launch_pdl(linear_small_kernel<T, M, R, NORM, SW>, dim3(blocks), dim3(128), 0, st, (const T*)x, (const T*)W, \
                 (const T*)bias, (const T*)residual, (T*)out, (const T*)norm_w, eps, N, K, ldo)
  if (norm_w) { if (swiglu) L(true, true); else L(true, false); }
  else { if (swiglu) L(false, true); else L(false, false); }
#undef L
  return (int)e;
}

// y[M,N] = f(x[M,K]) W[N,K]^T ; M in 1..8.  norm_w != null → RMSNorm prologue.  swiglu != 0 → out is [M, N/2].
EXO_API int exo_linear_small(const void* x, const void* W, const void* bias, const void* residual, void* out,
                             const void* norm_w, float eps, int M, int N, int K, int swiglu, int dtype,
                             cudaStream_t st) {
  if (M <= 0 || M > 8) return -2;
  int vec = dtype == EXO_BF16 ? 8 : 4;
  if (K % vec != 0) return -2;
  if (swiglu && (N % 2)) return -2;
  int rc = 0;
#define BY_M(T)                                                                                        \
  switch (M) {                                                                                         \
    case 1: rc = launch_small<T, 1>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    case 2: rc = launch_small<T, 2>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    case 3: rc = launch_small<T, 3>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    case 4: rc = launch_small<T, 4>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    case 5: rc = launch_small<T, 5>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    case 6: rc = launch_small<T, 6>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    case 7: rc = launch_small<T, 7>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break;  \
    default: rc = launch_small<T, 8>(x, W, bias, residual, out, norm_w, eps, N, K, swiglu, st); break; \
  }
  if (dtype == EXO_BF16) { BY_M(__nv_bfloat16) } else { BY_M(float) }
#undef BY_M
  if (rc) return rc;
  EXO_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// Generic fp32/bf16 tiled GEMM on CUDA cores: y[M,N] = x[M,K] W[N,K]^T (+bias)(+residual).
// Only used for fp32 models (the CPU-oracle configs run on a GPU) — bf16 models go to tcgen05.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
linear_tiled_kernel(const T* __restrict__ x, const T* __restrict__ W, const T* __restrict__ bias, const T* residual,
                    T* out, int M, int N, int K) {
  __shared__ float xs[32][33], ws[32][33];
  int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int r = ty + i * 8;
      int m = m0 + r, n = n0 + r, k = k0 + tx;
      xs[r][tx] = (m < M && k < K) ? Cvt<T>::to_f(x[(size_t)m * K + k]) : 0.f;
      ws[r][tx] = (n < N && k < K) ? Cvt<T>::to_f(W[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; kk++) {
      float wv = ws[tx][kk];
#pragma unroll
      for (int i = 0; i < 4; i++) acc[i] += xs[ty + i * 8][kk] * wv;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int m = m0 + ty + i * 8, n = n0 + tx;
    if (m < M && n < N) {
      float y = acc[i];
      if (bias) y += Cvt<T>::to_f(bias[n]);
      if (residual) y += Cvt<T>::to_f(residual[(size_t)m * N + n]);
      out[(size_t)m * N + n] = Cvt<T>::from_f(y);
    }
  }
}

EXO_API int exo_linear_tiled(const void* x, const void* W, const void* bias, const void* residual, void* out, int M,
                             int N, int K, int dtype, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + 31) / 32, (M + 31) / 32);
  if (dtype == EXO_BF16)
    linear_tiled_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)W,
                                                             (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                                                             (__nv_bfloat16*)out, M, N, K);
  else
    linear_tiled_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (const float*)W, (const float*)bias,
                                                     (const float*)residual, (float*)out, M, N, K);
  EXO_CHECK_LAUNCH();
  return 0;
}
