// Gated delta rule (the linear-attention layers of Qwen3-Next / Qwen3.5) over a ragged batch, between the layer's input
// projection and its output projection.  Three launches, all sized from device-side sequence descriptors so that a decode
// step can be captured in a CUDA graph:
//
//   gdn_conv_kernel        causal depthwise convolution + SiLU of the q | k | v columns, every token in parallel; a
//                          sequence's first taps-1 tokens take their history from its state seat
//   gdn_conv_state_kernel  the seat's new history (the sequence's last taps-1 inputs), after the convolution has read the old
//   gdn_delta_kernel       one CTA per (value head, sequence): the [DK, DV] state lives in registers (DK/32 lanes share
//                          column j, 32 rows each) from the first token of the sequence's chunk to the last, so HBM sees the state
//                          once in and once out per step and otherwise only each token's q, k, v, z, b, a.  Per token:
//                          L2-normalise q and k, S *= exp(g), delta = (v - k.S) * beta, S += k (x) delta, o = q.S, then
//                          RMSNorm over the head, * weight * silu(z).
//
// The next token's operands are fetched into registers while the current one is computed (the recurrence is a serial
// chain; without the prefetch every step would wait a full memory round trip).
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

struct SeqInfo {
  int t0, t1, seat, fresh;
};

__device__ __forceinline__ SeqInfo seq_info(int s, const int* cu_q, const int* seats, const int* positions) {
  SeqInfo i;
  i.t0 = cu_q[s];
  i.t1 = cu_q[s + 1];
  i.seat = seats[s];
  i.fresh = (i.t1 > i.t0) ? (positions[i.t0] == 0) : 1;
  return i;
}

// ---------------------------------------------------------------------------------------------------------------
// grid (ceil(C / 256), T): token t, channels c.  y[t, c] = silu(sum_j w[c, j] * x[t - (taps-1) + j, c])
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gdn_conv_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ w, const T* __restrict__ conv_state,
                                const int* __restrict__ cu_q, const int* __restrict__ seats, const int* __restrict__ positions,
                                int B, int C, int taps, T* __restrict__ y) {
  __shared__ int s_seq;
  const int t = blockIdx.y;
  if (threadIdx.x == 0) {
    // the sequence that holds token t: the last s with cu_q[s] <= t (B is small; empty sequences repeat a boundary)
    int lo = 0, hi = B;            // invariant: cu_q[lo] <= t, answer in [lo, hi)
    if (t >= cu_q[B]) lo = -1;
    else
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (cu_q[mid] <= t) lo = mid; else hi = mid;
      }
    s_seq = lo;
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = s_seq;
  if (s < 0) {                      // a padding token that belongs to no sequence
    y[(size_t)t * C + c] = Cvt<T>::from_f(0.f);
    return;
  }
  const SeqInfo q = seq_info(s, cu_q, seats, positions);
  const int hist = taps - 1;
  float acc = 0.f;
  for (int j = 0; j < taps; j++) {
    const int src = t - hist + j;
    float x;
    if (src >= q.t0) x = Cvt<T>::to_f(proj[(size_t)src * ld + c]);
    else if (q.fresh) x = 0.f;
    else x = Cvt<T>::to_f(conv_state[((size_t)q.seat * C + c) * hist + (hist + src - q.t0)]);
    acc += x * w[(size_t)c * taps + j];
  }
  y[(size_t)t * C + c] = Cvt<T>::from_f(silu_f(acc));
}

// grid (ceil(C / 256), B): the last taps-1 inputs of sequence s become its seat's history
template <typename T>
__global__ void gdn_conv_state_kernel(const T* __restrict__ proj, int ld, T* __restrict__ conv_state, const int* __restrict__ cu_q,
                                      const int* __restrict__ seats, const int* __restrict__ positions, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const SeqInfo q = seq_info(blockIdx.y, cu_q, seats, positions);
  const int L = q.t1 - q.t0, hist = taps - 1;
  if (L <= 0) return;
  T* st = conv_state + ((size_t)q.seat * C + c) * hist;
  T keep[MAX_TAPS];
  for (int j = 0; j < hist; j++) {
    const int src = q.t1 - hist + j;
    if (src >= q.t0) keep[j] = proj[(size_t)src * ld + c];
    else keep[j] = q.fresh ? Cvt<T>::from_f(0.f) : st[j + L];          // older inputs shift towards the front
  }
  for (int j = 0; j < hist; j++) st[j] = keep[j];
}

// ---------------------------------------------------------------------------------------------------------------
// grid (hv, B), DV * DK/32 threads: column j of the head's state is held by DK/32 neighbouring lanes, 32 rows each, so
// the per-token chain is 32 fused multiply-adds long whatever DK is, and k.S / q.S are finished with lane shuffles.
// y: convolved q | k | v [T, 2*hk*DK + hv*DV]; proj supplies z, b, a at column offsets.
// ---------------------------------------------------------------------------------------------------------------
template <typename T, int DK>
__global__ void __launch_bounds__(DK >= 64 ? 512 : 256) gdn_delta_kernel(
    const T* __restrict__ y, const T* __restrict__ proj, int ld, int z_off, int b_off, int a_off,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, const T* __restrict__ norm_w, float eps,
    float* __restrict__ rec_state, const int* __restrict__ cu_q, const int* __restrict__ seats,
    const int* __restrict__ positions, int hk, int hv, int DV, T* __restrict__ out) {
  constexpr int P = DK / 32;           // lanes per column
  constexpr int SEG = 36;              // floats between the parts' q / k segments in shared memory: 16-byte aligned, and
                                       // the P lanes of a column hit different banks
  const int h = blockIdx.x, tid = threadIdx.x;
  const int j = tid / P, part = tid % P;
  const SeqInfo sq = seq_info(blockIdx.y, cu_q, seats, positions);
  if (sq.t1 <= sq.t0) return;
  const int kh = h / (hv / hk);
  const int C = 2 * hk * DK + hv * DV;
  const int q_col = kh * DK, k_col = hk * DK + kh * DK, v_col = 2 * hk * DK + h * DV + j;
  __shared__ __align__(16) float s_q[2][P * SEG], s_k[2][P * SEG];
  __shared__ float s_red[2][32];
  float S[32];
  float* st = rec_state + (((size_t)sq.seat * hv + h) * DK + part * 32) * DV + j;
  if (sq.fresh) {
#pragma unroll
    for (int i = 0; i < 32; i++) S[i] = 0.f;
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++) S[i] = st[(size_t)i * DV];
  }
  const float neg_a = -__expf(a_log[h]), dtb = dt_bias[h], nw = Cvt<T>::to_f(norm_w[j]);
  const float q_scale = rsqrtf((float)DK);
  const int lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;

  // operands of the token about to be processed, fetched one token ahead
  float nq[P], nk[P], nv, nz, nb, na;
  auto fetch = [&](int t) {
    const T* row = y + (size_t)t * C;
#pragma unroll
    for (int r = 0; r < P; r++) {
      // every warp holds the whole q and k of the head (lane l: elements l, l+32, ...): the norms need no block barrier
      nq[r] = Cvt<T>::to_f(row[q_col + r * 32 + lane]);
      nk[r] = Cvt<T>::to_f(row[k_col + r * 32 + lane]);
    }
    nv = Cvt<T>::to_f(row[v_col]);
    const T* pr = proj + (size_t)t * ld;
    nz = Cvt<T>::to_f(pr[z_off + h * DV + j]);
    nb = Cvt<T>::to_f(pr[b_off + h]);
    na = Cvt<T>::to_f(pr[a_off + h]);
  };
  fetch(sq.t0);
#pragma unroll 1
  for (int t = sq.t0; t < sq.t1; t++) {
    const int buf = (t - sq.t0) & 1;
    float qs = 0.f, ks = 0.f, qk = 0.f;
#pragma unroll
    for (int r = 0; r < P; r++) { qs += nq[r] * nq[r]; ks += nk[r] * nk[r]; qk += nq[r] * nk[r]; }
    qs = warp_sum(qs);
    ks = warp_sum(ks);
    qk = warp_sum(qk);
    const float qn = rsqrtf(qs + 1e-6f) * q_scale, kn = rsqrtf(ks + 1e-6f);
    qk *= qn * kn;                         // q . k of the normalised vectors
    if (warp == 0) {
#pragma unroll
      for (int r = 0; r < P; r++) { s_q[buf][r * SEG + lane] = nq[r] * qn; s_k[buf][r * SEG + lane] = nk[r] * kn; }
    }
    const float v = nv, z = nz;
    const float beta = 1.f / (1.f + __expf(-nb));
    const float xa = na + dtb;
    const float decay = __expf(neg_a * (xa > 20.f ? xa : log1pf(__expf(xa))));
    __syncthreads();                       // q, k of this token visible; the other buffer is free again
    if (t + 1 < sq.t1) fetch(t + 1);
    // o = q.(S' + k (x) delta) = q.S' + (q.k) delta with S' the decayed state: one pass gives k.S' and q.S' ...
    const float* kk = &s_k[buf][part * SEG];
    const float* qq = &s_q[buf][part * SEG];
    float mem = 0.f, o = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
      const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
      S[i] *= decay; S[i + 1] *= decay; S[i + 2] *= decay; S[i + 3] *= decay;
      mem += S[i] * k4.x + S[i + 1] * k4.y + S[i + 2] * k4.z + S[i + 3] * k4.w;
      o += S[i] * q4.x + S[i + 1] * q4.y + S[i + 2] * q4.z + S[i + 3] * q4.w;
    }
#pragma unroll
    for (int m = 1; m < P; m <<= 1) {
      mem += __shfl_xor_sync(0xffffffffu, mem, m);
      o += __shfl_xor_sync(0xffffffffu, o, m);
    }
    const float delta = (v - mem) * beta;
    o += qk * delta;
    // ... and the second pass adds k (x) delta
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
      S[i] += k4.x * delta; S[i + 1] += k4.y * delta; S[i + 2] += k4.z * delta; S[i + 3] += k4.w * delta;
    }
    // RMSNorm over the head's DV outputs (every column counted once)
    float ss = warp_sum(part == 0 ? o * o : 0.f);
    if (lane == 0) s_red[buf][warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w2 = 0; w2 < n_warps; w2++) tot += s_red[buf][w2];
    const float r = rsqrtf(tot / (float)DV + eps);
    if (part == 0) out[(size_t)t * hv * DV + h * DV + j] = Cvt<T>::from_f(o * r * nw * silu_f(z));
  }
#pragma unroll
  for (int i = 0; i < 32; i++) st[(size_t)i * DV] = S[i];
}

template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ x, const T* __restrict__ gate, int ldg, T* __restrict__ out, size_t rows,
                                    int n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = rows * (size_t)n;
  for (; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n;
    const int c = (int)(i - r * n);
    const float g = Cvt<T>::to_f(gate[r * ldg + c]);
    out[i] = Cvt<T>::from_f(Cvt<T>::to_f(x[i]) / (1.f + __expf(-g)));
  }
}

template <typename T>
__global__ void scaled_add_kernel(const T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ logit, T* __restrict__ out,
                                  size_t rows, int n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = rows * (size_t)n;
  for (; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n;
    const float s = 1.f / (1.f + __expf(-Cvt<T>::to_f(logit[r])));
    out[i] = Cvt<T>::from_f(Cvt<T>::to_f(y[i]) + Cvt<T>::to_f(x[i]) * s);
  }
}

template <typename T>
int launch_gated_delta(const void* proj, int ld, const float* conv_w, const float* a_log, const float* dt_bias, const void* norm_w,
                       float eps, void* conv_state, float* rec_state, const int* seats, const int* cu_q, const int* positions,
                       int T_, int B, int hk, int hv, int dk, int dv, int taps, void* y, void* out, cudaStream_t st) {
  const int C = 2 * hk * dk + hv * dv;
  if (taps < 2 || taps > MAX_TAPS || dv % 32 || dv * (dk / 32) > (dk >= 64 ? 512 : 256) || hv % hk) return -2;
  if (T_ == 0 || B == 0) return 0;
  dim3 gc((C + 255) / 256, T_);
  gdn_conv_kernel<T><<<gc, 256, 0, st>>>((const T*)proj, ld, conv_w, (const T*)conv_state, cu_q, seats, positions, B, C, taps, (T*)y);
  dim3 gs((C + 255) / 256, B);
  gdn_conv_state_kernel<T><<<gs, 256, 0, st>>>((const T*)proj, ld, (T*)conv_state, cu_q, seats, positions, C, taps);
  dim3 gd(hv, B);
  const int z_off = C, b_off = C + hv * dv, a_off = C + hv * dv + hv;
#define EXO_GDN(DK)                                                                                                          \
  gdn_delta_kernel<T, DK><<<gd, dv * (DK / 32), 0, st>>>((const T*)y, (const T*)proj, ld, z_off, b_off, a_off, a_log, dt_bias,           \
                                              (const T*)norm_w, eps, rec_state, cu_q, seats, positions, hk, hv, dv, (T*)out)
  if (dk == 128) EXO_GDN(128);
  else if (dk == 64) EXO_GDN(64);
  else if (dk == 32) EXO_GDN(32);
  else return -2;
#undef EXO_GDN
  return 0;
}

}  // namespace

// proj [T, ld]: q | k | v | z | b | a of this rank's heads; y [T, 2*hk*dk + hv*dv] scratch; out [T, hv*dv].
// Returns -2 for head sizes the kernels are not built for (dk in {32, 64, 128}; dv a multiple of 32 with
// dv * dk / 32 threads fitting a CTA: dv <= 128 at dk = 128, else dv <= 256).
EXO_API int exo_gated_delta(const void* proj, int ld, const float* conv_w, const float* a_log, const float* dt_bias,
                            const void* norm_w, float eps, void* conv_state, float* rec_state, const int* seats, const int* cu_q,
                            const int* positions, int T, int B, int hk, int hv, int dk, int dv, int taps, void* y, void* out,
                            int dtype, cudaStream_t st) {
  int rc = dtype == EXO_BF16
               ? launch_gated_delta<__nv_bfloat16>(proj, ld, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q,
                                                   positions, T, B, hk, hv, dk, dv, taps, y, out, st)
               : launch_gated_delta<float>(proj, ld, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q,
                                           positions, T, B, hk, hv, dk, dv, taps, y, out, st);
  if (rc) return rc;
  EXO_CHECK_LAUNCH();
  return 0;
}

EXO_API int exo_sigmoid_gate(const void* x, const void* gate, int ldg, void* out, int rows, int n, int dtype, cudaStream_t st) {
  const size_t total = (size_t)rows * n;
  if (!total) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == EXO_BF16)
    sigmoid_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, ldg,
                                                               (__nv_bfloat16*)out, rows, n);
  else
    sigmoid_gate_kernel<float><<<blocks, 256, 0, st>>>((const float*)x, (const float*)gate, ldg, (float*)out, rows, n);
  EXO_CHECK_LAUNCH();
  return 0;
}

EXO_API int exo_scaled_add(const void* y, const void* x, const void* logit, void* out, int rows, int n, int dtype, cudaStream_t st) {
  const size_t total = (size_t)rows * n;
  if (!total) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == EXO_BF16)
    scaled_add_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)x,
                                                             (const __nv_bfloat16*)logit, (__nv_bfloat16*)out, rows, n);
  else
    scaled_add_kernel<float><<<blocks, 256, 0, st>>>((const float*)y, (const float*)x, (const float*)logit, (float*)out, rows, n);
  EXO_CHECK_LAUNCH();
  return 0;
}
