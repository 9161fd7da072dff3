// Gated delta rule (the linear-attention layers of Qwen3-Next / Qwen3.5) over a ragged batch, between the layer's input
// projection and its output projection.  Three launches, all sized from device-side sequence descriptors so that a decode
// step can be captured in a CUDA graph:
//
//   gdn_conv_kernel        causal depthwise convolution + SiLU of the q | k | v columns, tokens in parallel; a
//                          sequence's first taps-1 tokens take their history from its state seat
//   gdn_conv_state_kernel  the seat's new history (the sequence's last taps-1 inputs), after the convolution has read the old
//   gdn_delta_kernel       one CTA per (value head, sequence): the [DK, DV] state lives in registers (a 16 x 2 patch
//                          per thread) from the first token of the sequence's chunk to the last, so HBM sees
//                          the state once in and once out per step and otherwise only each token's q, k, v, z, b, a.
//                          Per token: L2-normalise q and k, S *= exp(g), delta = (v - k.S) * beta, S += k (x) delta,
//                          o = q.S, then RMSNorm over the head, * weight * silu(z).
//
// The recurrence is a serial chain over the tokens of a sequence; everything around it (operand loads, the q / k norms,
// the output norm and gate) is done for 16 tokens at a time by all warps in parallel, so that the serial part runs from
// shared memory without a block barrier per token.
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
// grid (ceil(C / 256), ceil(T / n_tok)): n_tok tokens per CTA (16 for prompts, 1 for decode-sized steps, where the
// tokens are the only parallelism there is), one channel per thread.
// y[t, c] = silu(sum_j w[c, j] * x[t - (taps-1) + j, c])
// ---------------------------------------------------------------------------------------------------------------
constexpr int GDN_CONV_TOK = 16;

template <typename T>
__global__ void gdn_conv_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ w, const T* __restrict__ conv_state,
                                const int* __restrict__ cu_q, const int* __restrict__ seats, const int* __restrict__ positions,
                                int T_, int B, int C, int taps, int n_tok, const float* __restrict__ bias, T* __restrict__ y) {
  __shared__ int s_seq[GDN_CONV_TOK];
  const int base = blockIdx.y * n_tok;
  if (threadIdx.x < n_tok) {
    // the sequence that holds token t: the last s with cu_q[s] <= t (B is small; empty sequences repeat a boundary)
    const int t = base + threadIdx.x;
    int lo = 0, hi = B;            // invariant: cu_q[lo] <= t, answer in [lo, hi)
    if (t >= cu_q[B]) lo = -1;
    else
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (cu_q[mid] <= t) lo = mid; else hi = mid;
      }
    s_seq[threadIdx.x] = lo;
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int hist = taps - 1;
  float wc[MAX_TAPS];
  for (int j = 0; j < taps; j++) wc[j] = w[(size_t)c * taps + j];
  for (int i = 0; i < n_tok; i++) {
    const int t = base + i;
    if (t >= T_) break;
    const int s = s_seq[i];
    if (s < 0) {                    // a padding token that belongs to no sequence
      y[(size_t)t * C + c] = Cvt<T>::from_f(0.f);
      continue;
    }
    const SeqInfo q = seq_info(s, cu_q, seats, positions);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; j++) {
      const int src = t - hist + j;
      float x;
      if (src >= q.t0) x = Cvt<T>::to_f(proj[(size_t)src * ld + c]);
      else if (q.fresh) x = 0.f;
      else x = Cvt<T>::to_f(conv_state[((size_t)q.seat * C + c) * hist + (hist + src - q.t0)]);
      acc += x * wc[j];
    }
    y[(size_t)t * C + c] = Cvt<T>::from_f(silu_f(acc));
  }
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
// grid (hv, B), (DV / 2) * (DK / 16) threads: a thread holds a 16-row x 2-column patch of the head's [DK, DV] state, so
// DK/16 neighbouring lanes share a column pair and k.S / q.S are finished with lane shuffles.  (The patch shape is a
// balance: every k and q value read from shared memory feeds two columns, which halves the shared-memory traffic that
// bounds a 32 x 1 patch, and the shuffle tree stays three levels deep at DK = 128.)
// Tokens are taken TB at a time: (A) all threads bring the block's q, k, v, z and gates into shared memory and the
// warps normalise q and k, one token per warp; (B) the serial part walks the TB tokens with no block barrier; (C) the
// warps normalise and gate the TB outputs, one token per warp, and store them.
// y: convolved q | k | v [T, 2*hk*DK + hv*DV]; proj supplies z, b, a at column offsets.
// ---------------------------------------------------------------------------------------------------------------
constexpr int GDN_TB = 16;
constexpr int GDN_SEG = 20;            // floats between 16-row segments of q / k in shared memory: 16-byte aligned, and the
                                       // lanes of a column pair (one segment each) hit different banks

__device__ __forceinline__ int gdn_at(int i) { return (i >> 4) * GDN_SEG + (i & 15); }

__device__ __forceinline__ void gdn_cp16(void* smem, const void* g) {
  const unsigned s_addr = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s_addr), "l"(g) : "memory");
}

// bytes of dynamic shared memory the kernel below needs
static size_t gdn_smem_bytes(int dk, int dv, size_t elem) {
  return 2 * GDN_TB * (2 * dk + 2 * dv) * elem + (2 * GDN_TB * (dk / 16) * GDN_SEG + GDN_TB * dv + 3 * GDN_TB) * sizeof(float);
}

// MODE 0: gated delta rule as described above.  MODE 1: the Mamba-2 state-space recurrence on the same machinery, with
// q := C, k := B (one pair per group of heads, not normalised), v := x, the `a` column holding dt:
//   dt = softplus(a + dt_bias);  S *= exp(-exp(a_log) dt);  S += B (x) (dt x);  y = C.S + skip[h] * x
// and the raw y stored (the grouped gated norm over several heads is mamba_norm_kernel's).
template <typename T, int DK, int MODE>
__global__ void __launch_bounds__(DK >= 64 ? 512 : 256) gdn_delta_kernel(
    const T* __restrict__ y, const T* __restrict__ proj, int ld, int z_off, int b_off, int a_off,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, const T* __restrict__ norm_w, float eps,
    float* __restrict__ rec_state, const int* __restrict__ cu_q, const int* __restrict__ seats,
    const int* __restrict__ positions, int hk, int hv, int DV, int nsplit, int aligned, const float* __restrict__ skip,
    T* __restrict__ out) {
  constexpr int PL = DK / 16;          // lanes per column pair
  constexpr int QK = PL * GDN_SEG;     // floats per token of q (or k) in shared memory
  constexpr int TB = GDN_TB;
  constexpr int EPC = 16 / (int)sizeof(T);   // elements per 16-byte copy
  // nsplit CTAs share a head, DVs = DV / nsplit columns each (columns never interact inside the recurrence); with
  // nsplit > 1 the CTA stores the raw outputs and gdn_norm_gate_kernel finishes them
  const int h = blockIdx.x / nsplit, DVs = DV / nsplit, c0 = (blockIdx.x % nsplit) * DVs;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int j0 = (tid / PL) * 2, part = tid % PL;          // column pair within the CTA's slice
  const SeqInfo sq = seq_info(blockIdx.y, cu_q, seats, positions);
  if (sq.t1 <= sq.t0) return;
  const int kh = h / (hv / hk);
  const int C = 2 * hk * DK + hv * DV;
  const int q_col = kh * DK, k_col = hk * DK + kh * DK, v_base = 2 * hk * DK + h * DV + c0;
  extern __shared__ __align__(16) unsigned char gdn_smem[];
  // two stages of the block's operands as they lie in memory (filled by asynchronous copies one block ahead) ...
  T* raw = reinterpret_cast<T*>(gdn_smem);
  const int stage_elems = TB * (2 * DK + 2 * DVs);
  auto raw_q = [&](int stage) { return raw + stage * stage_elems; };
  auto raw_k = [&](int stage) { return raw + stage * stage_elems + TB * DK; };
  auto raw_v = [&](int stage) { return raw + stage * stage_elems + 2 * TB * DK; };
  auto raw_z = [&](int stage) { return raw + stage * stage_elems + 2 * TB * DK + TB * DVs; };
  // ... and what the serial part reads and writes, in fp32
  float* s_q = reinterpret_cast<float*>(raw + 2 * stage_elems);   // [TB][QK]
  float* s_k = s_q + TB * QK;                // [TB][QK]
  float* s_o = s_k + TB * QK;                // [TB][DV]
  float* s_decay = s_o + TB * DVs;            // [TB]
  float* s_beta = s_decay + TB;              // [TB]
  float* s_qk = s_beta + TB;                 // [TB]
  float S0[16], S1[16];                      // rows part*16 .. +16 of columns j0 and j0 + 1
  float* st = rec_state + (((size_t)sq.seat * hv + h) * DK + part * 16) * DV + c0 + j0;
  if (sq.fresh) {
#pragma unroll
    for (int i = 0; i < 16; i++) { S0[i] = 0.f; S1[i] = 0.f; }
  } else {
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const float2 t2 = *reinterpret_cast<const float2*>(st + (size_t)i * DV);
      S0[i] = t2.x;
      S1[i] = t2.y;
    }
  }
  const float neg_a = -__expf(a_log[h]), dtb = dt_bias[h];
  const float q_scale = rsqrtf((float)DK);
  const int lane = tid & 31, warp = tid >> 5, n_warps = nthreads >> 5;

  float pre_a = 0.f, pre_b = 0.f;            // gate inputs of token tid of the block in flight
  auto issue = [&](int tb0, int stage) {
    const int nb = min(TB, sq.t1 - tb0);
    T *dq = raw_q(stage), *dk_ = raw_k(stage), *dv_ = raw_v(stage), *dz = raw_z(stage);
    if (aligned) {
      for (int c = tid; c < nb * (DK / EPC); c += nthreads) {
        const int tok = c / (DK / EPC), e = (c % (DK / EPC)) * EPC;
        const T* row = y + (size_t)(tb0 + tok) * C;
        gdn_cp16(dq + tok * DK + e, row + q_col + e);
        gdn_cp16(dk_ + tok * DK + e, row + k_col + e);
      }
      const int vc = DVs / EPC;
      for (int c = tid; c < nb * vc; c += nthreads) {
        const int tok = c / vc, e = (c % vc) * EPC;
        gdn_cp16(dv_ + tok * DVs + e, y + (size_t)(tb0 + tok) * C + v_base + e);
        gdn_cp16(dz + tok * DVs + e, proj + (size_t)(tb0 + tok) * ld + z_off + h * DV + c0 + e);
      }
    } else {                                 // rows that do not start on 16-byte boundaries: element by element
      for (int idx = tid; idx < nb * DK; idx += nthreads) {
        const int tok = idx / DK, i = idx % DK;
        const T* row = y + (size_t)(tb0 + tok) * C;
        dq[tok * DK + i] = row[q_col + i];
        dk_[tok * DK + i] = row[k_col + i];
      }
      for (int idx = tid; idx < nb * DVs; idx += nthreads) {
        const int tok = idx / DVs, jj = idx % DVs;
        dv_[tok * DVs + jj] = y[(size_t)(tb0 + tok) * C + v_base + jj];
        dz[tok * DVs + jj] = proj[(size_t)(tb0 + tok) * ld + z_off + h * DV + c0 + jj];
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (tid < nb) {
      const T* pr = proj + (size_t)(tb0 + tid) * ld;
      pre_a = Cvt<T>::to_f(pr[a_off + h]);
      pre_b = Cvt<T>::to_f(pr[b_off + h]);
    }
  };

  issue(sq.t0, 0);
  int stage = 0;
#pragma unroll 1
  for (int tb0 = sq.t0; tb0 < sq.t1; tb0 += TB, stage ^= 1) {
    const int nb = min(TB, sq.t1 - tb0);
    // ---- A: gates of this block, then start the next block's copies and wait for this block's
    if (tid < nb) {
      const float xa = pre_a + dtb;
      const float sp = xa > 20.f ? xa : log1pf(__expf(xa));
      s_decay[tid] = __expf(neg_a * sp);                                          // exp(-exp(a_log) * softplus(a + dt_bias))
      s_beta[tid] = MODE == 0 ? 1.f / (1.f + __expf(-pre_b)) : sp;                // sigmoid(b), or the time step itself
    }
    if (tb0 + TB < sq.t1) {
      issue(tb0 + TB, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const T *rq = raw_q(stage), *rk = raw_k(stage), *rv = raw_v(stage), *rz = raw_z(stage);
    for (int tok = warp; tok < nb; tok += n_warps) {          // L2-normalise q (and scale it) and k; keep q . k
      float qv[DK / 32], kv[DK / 32], qs = 0.f, ks = 0.f, qk = 0.f;
#pragma unroll
      for (int r = 0; r < DK / 32; r++) {
        qv[r] = Cvt<T>::to_f(rq[tok * DK + r * 32 + lane]);
        kv[r] = Cvt<T>::to_f(rk[tok * DK + r * 32 + lane]);
        qs += qv[r] * qv[r]; ks += kv[r] * kv[r]; qk += qv[r] * kv[r];
      }
      qs = warp_sum(qs);
      ks = warp_sum(ks);
      qk = warp_sum(qk);
      const float qn = MODE == 0 ? rsqrtf(qs + 1e-6f) * q_scale : 1.f, kn = MODE == 0 ? rsqrtf(ks + 1e-6f) : 1.f;
#pragma unroll
      for (int r = 0; r < DK / 32; r++) {
        s_q[tok * QK + gdn_at(r * 32 + lane)] = qv[r] * qn;
        s_k[tok * QK + gdn_at(r * 32 + lane)] = kv[r] * kn;
      }
      if (lane == 0) s_qk[tok] = qk * qn * kn;
    }
    __syncthreads();
    // ---- B: the recurrence.  o = q.(S' + k (x) delta) = q.S' + (q.k) delta with S' the decayed state: one pass
    // gives k.S' and q.S', a second one adds k (x) delta
#pragma unroll 1
    for (int tok = 0; tok < nb; tok++) {
      const float* kk = s_k + tok * QK + part * GDN_SEG;
      const float* qq = s_q + tok * QK + part * GDN_SEG;
      const float decay = s_decay[tok];
      const float v0 = Cvt<T>::to_f(rv[tok * DVs + j0]), v1 = Cvt<T>::to_f(rv[tok * DVs + j0 + 1]);
      float kr[16];
      float mem0 = 0.f, mem1 = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
        kr[i] = k4.x; kr[i + 1] = k4.y; kr[i + 2] = k4.z; kr[i + 3] = k4.w;
        const float qr[4] = {q4.x, q4.y, q4.z, q4.w};
        float m0 = 0.f, m1 = 0.f, p0 = 0.f, p1 = 0.f;     // a short chain per group of four rows, summed afterwards
#pragma unroll
        for (int e = 0; e < 4; e++) {
          S0[i + e] *= decay;
          S1[i + e] *= decay;
          m0 += S0[i + e] * kr[i + e];
          m1 += S1[i + e] * kr[i + e];
          p0 += S0[i + e] * qr[e];
          p1 += S1[i + e] * qr[e];
        }
        mem0 += m0; mem1 += m1; o0 += p0; o1 += p1;
      }
#pragma unroll
      for (int m = 1; m < PL; m <<= 1) {
        mem0 += __shfl_xor_sync(0xffffffffu, mem0, m);
        mem1 += __shfl_xor_sync(0xffffffffu, mem1, m);
        o0 += __shfl_xor_sync(0xffffffffu, o0, m);
        o1 += __shfl_xor_sync(0xffffffffu, o1, m);
      }
      const float beta = s_beta[tok], qk = s_qk[tok];
      const float d0 = (MODE == 0 ? v0 - mem0 : v0) * beta, d1 = (MODE == 0 ? v1 - mem1 : v1) * beta;
      o0 += qk * d0;
      o1 += qk * d1;
      if (MODE == 1) { o0 += skip[h] * v0; o1 += skip[h] * v1; }
#pragma unroll
      for (int i = 0; i < 16; i++) { S0[i] += kr[i] * d0; S1[i] += kr[i] * d1; }
      if (part == 0) *reinterpret_cast<float2*>(s_o + tok * DVs + j0) = make_float2(o0, o1);
    }
    __syncthreads();
    // ---- C: RMSNorm over each head output, * weight * silu(z)
    for (int tok = warp; tok < nb; tok += n_warps) {
      T* dst = out + (size_t)(tb0 + tok) * hv * DV + h * DV + c0;
      if (nsplit > 1 || MODE == 1) {      // a slice of the head (or the state-space form): raw outputs, normalised by the next kernel
        for (int jj = lane; jj < DVs; jj += 32) dst[jj] = Cvt<T>::from_f(s_o[tok * DVs + jj]);
        continue;
      }
      float ss = 0.f;
      for (int jj = lane; jj < DV; jj += 32) { const float o = s_o[tok * DV + jj]; ss += o * o; }
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)DV + eps);
      for (int jj = lane; jj < DV; jj += 32)
        dst[jj] = Cvt<T>::from_f(s_o[tok * DV + jj] * r * Cvt<T>::to_f(norm_w[jj]) * silu_f(Cvt<T>::to_f(rz[tok * DV + jj])));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 16; i++) *reinterpret_cast<float2*>(st + (size_t)i * DV) = make_float2(S0[i], S1[i]);
}

// one warp per (token, value head): out = rmsnorm(out) * w * silu(z), in place over the raw outputs of a split launch
template <typename T>
__global__ void gdn_norm_gate_kernel(T* __restrict__ out, const T* __restrict__ proj, int ld, int z_off, const T* __restrict__ norm_w,
                                     float eps, int rows, int hv, int DV) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * hv) return;
  const int t = w / hv, h = w % hv;
  T* o = out + (size_t)t * hv * DV + h * DV;
  const T* z = proj + (size_t)t * ld + z_off + h * DV;
  float v[8], ss = 0.f;                 // DV <= 256
#pragma unroll
  for (int r = 0; r < 8; r++) {
    const int jj = r * 32 + lane;
    v[r] = jj < DV ? Cvt<T>::to_f(o[jj]) : 0.f;
    ss += v[r] * v[r];
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)DV + eps);
#pragma unroll
  for (int r = 0; r < 8; r++) {
    const int jj = r * 32 + lane;
    if (jj < DV) o[jj] = Cvt<T>::from_f(v[r] * rs * Cvt<T>::to_f(norm_w[jj]) * silu_f(Cvt<T>::to_f(z[jj])));
  }
}

// Mamba-2 output: y * silu(z), RMS-normalised over groups of `gsize` neighbouring channels, times the weight.  One warp
// per (token, group); in place over the raw outputs.
template <typename T>
__global__ void mamba_norm_kernel(T* __restrict__ out, const T* __restrict__ proj, int ld, int z_off, const T* __restrict__ norm_w,
                                  float eps, int rows, int width, int gsize) {
  const int groups = width / gsize;
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * groups) return;
  const int t = w / groups, g = w % groups;
  T* o = out + (size_t)t * width + g * gsize;
  const T* z = proj + (size_t)t * ld + z_off + g * gsize;
  float ss = 0.f;
  for (int j = lane; j < gsize; j += 32) {
    const float v = Cvt<T>::to_f(o[j]) * silu_f(Cvt<T>::to_f(z[j]));
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)gsize + eps);
  for (int j = lane; j < gsize; j += 32) {
    const float v = Cvt<T>::to_f(o[j]) * silu_f(Cvt<T>::to_f(z[j]));
    o[j] = Cvt<T>::from_f(v * rs * Cvt<T>::to_f(norm_w[g * gsize + j]));
  }
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
                       int T_, int B, int hk, int hv, int dk, int dv, int taps, void* y, void* out, int mode,
                       const float* conv_bias, const float* skip, int norm_group, cudaStream_t st) {
  const int C = 2 * hk * dk + hv * dv;
  if (taps < 2 || taps > MAX_TAPS || dv % 32 || dv * (dk / 32) > (dk >= 64 ? 512 : 256) || hv % hk) return -2;
  if (T_ == 0 || B == 0) return 0;
  const int n_tok = T_ >= 1024 ? GDN_CONV_TOK : 1;
  dim3 gc((C + 255) / 256, (T_ + n_tok - 1) / n_tok);
  gdn_conv_kernel<T><<<gc, 256, 0, st>>>((const T*)proj, ld, conv_w, (const T*)conv_state, cu_q, seats, positions, T_, B, C, taps,
                                         n_tok, conv_bias, (T*)y);
  dim3 gs((C + 255) / 256, B);
  gdn_conv_state_kernel<T><<<gs, 256, 0, st>>>((const T*)proj, ld, (T*)conv_state, cu_q, seats, positions, C, taps);
  // heads x sequences fill the GPU by themselves in a batched decode; a single prompt gets its heads split by columns
  int nsplit = 1;
  while (nsplit < 4 && (long)hv * B * nsplit < 148 && (dv / (nsplit * 2)) % 32 == 0) nsplit *= 2;
  const int dvs = dv / nsplit;
  dim3 gd(hv * nsplit, B);
  const int z_off = C, b_off = C + hv * dv, a_off = C + hv * dv + hv;
  // asynchronous 16-byte copies need every row segment to start on a 16-byte boundary
  const size_t el = sizeof(T);
  const int aligned = ((uintptr_t)y % 16 == 0 && (uintptr_t)proj % 16 == 0 && (C * el) % 16 == 0 && ((size_t)ld * el) % 16 == 0 &&
                       (dk * el) % 16 == 0 && (dvs * el) % 16 == 0 && (z_off * el) % 16 == 0) ? 1 : 0;
  const size_t smem = gdn_smem_bytes(dk, dvs, el);
#define EXO_GDN_M(DK, MM)                                                                                                    \
  do {                                                                                                                       \
    static bool opted = false;                                                                                               \
    if (!opted) {                                                                                                            \
      if (cudaFuncSetAttribute(gdn_delta_kernel<T, DK, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) \
        return -3;                                                                                                           \
      opted = true;                                                                                                          \
    }                                                                                                                        \
    gdn_delta_kernel<T, DK, MM><<<gd, (dvs / 2) * (DK / 16), smem, st>>>((const T*)y, (const T*)proj, ld, z_off, b_off, a_off, a_log, \
                                                                         dt_bias, (const T*)norm_w, eps, rec_state, cu_q, seats, \
                                                                         positions, hk, hv, dv, nsplit, aligned, skip, (T*)out); \
  } while (0)
#define EXO_GDN(DK) do { if (mode == 1) EXO_GDN_M(DK, 1); else EXO_GDN_M(DK, 0); } while (0)
  if (dk == 128) EXO_GDN(128);
  else if (dk == 64) EXO_GDN(64);
  else if (dk == 32) EXO_GDN(32);
  else return -2;
#undef EXO_GDN
#undef EXO_GDN_M
  if (mode == 1) {
    const int width = hv * dv;
    const long warps = (long)T_ * (width / norm_group);
    mamba_norm_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>((T*)out, (const T*)proj, ld, z_off, (const T*)norm_w, eps,
                                                                                T_, width, norm_group);
  } else if (nsplit > 1) {
    const long warps = (long)T_ * hv;
    gdn_norm_gate_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>((T*)out, (const T*)proj, ld, z_off, (const T*)norm_w,
                                                                                  eps, T_, hv, dv);
  }
  return 0;
}

}  // namespace

// proj [T, ld]: q | k | v | z | b | a of this rank's heads; y [T, 2*hk*dk + hv*dv] scratch; out [T, hv*dv].
// Returns -2 for head sizes the kernels are not built for (dk in {32, 64, 128}; dv a multiple of 32 with
// dv * dk / 32 threads fitting a CTA: dv <= 128 at dk = 128, else dv <= 256).
// mode 0: gated delta rule (norm_w [dv]).  mode 1: Mamba-2 (proj columns C | B | x | z | dt | dt; conv_bias [channels], skip
// [hv] = the D of the skip connection, norm_w [hv*dv] applied over groups of norm_group channels).
EXO_API int exo_gated_delta(const void* proj, int ld, const float* conv_w, const float* a_log, const float* dt_bias,
                            const void* norm_w, float eps, void* conv_state, float* rec_state, const int* seats, const int* cu_q,
                            const int* positions, int T, int B, int hk, int hv, int dk, int dv, int taps, void* y, void* out,
                            int dtype, int mode, const float* conv_bias, const float* skip, int norm_group, cudaStream_t st) {
  if (mode == 1 && (!skip || norm_group <= 0 || (hv * dv) % norm_group)) return -2;
  int rc = dtype == EXO_BF16
               ? launch_gated_delta<__nv_bfloat16>(proj, ld, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q,
                                                   positions, T, B, hk, hv, dk, dv, taps, y, out, mode, conv_bias, skip, norm_group, st)
               : launch_gated_delta<float>(proj, ld, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q,
                                           positions, T, B, hk, hv, dk, dv, taps, y, out, mode, conv_bias, skip, norm_group, st);
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
