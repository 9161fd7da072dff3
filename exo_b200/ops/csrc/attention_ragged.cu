// General ragged causal attention over the paged KV cache (any query length per sequence, any
// dtype): the reference-quality kernel used for fp32 models, odd shapes and as the numerical
// cross-check of the tensor-core prefill kernel.  One warp owns one query token and the GT query
// heads that share a KV head; lanes split the head dim; keys are visited in order with an online
// softmax, so K/V rows are read once per group of heads.
#include "common.cuh"

template <typename T, int D, int GT>
__global__ void __launch_bounds__(128)
paged_ragged_kernel(const T* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ block_tables, const int* __restrict__ seq_lens,
                    const int* __restrict__ cu_q, const int* __restrict__ tok_seq, T* __restrict__ out, float scale,
                    int Hq, int Hkv, int max_blocks, int block_size, int window, const float* __restrict__ sinks,
                    int T_) {
  constexpr int E = D / 32;
  const int g = Hq / Hkv, tiles_per_kv = g / GT;
  int warp_global = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  int t = warp_global / (Hkv * tiles_per_kv);
  if (t >= T_) return;
  int rem = warp_global % (Hkv * tiles_per_kv);
  int kvh = rem / tiles_per_kv, h0 = kvh * g + (rem % tiles_per_kv) * GT;
  int b = tok_seq[t];
  int n = seq_lens[b], qlen = cu_q[b + 1] - cu_q[b];
  int pos = n - qlen + (t - cu_q[b]);  // absolute position of this query; attends to keys <= pos
  int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  float qr[GT][E], acc[GT][E], m[GT], l[GT];
#pragma unroll
  for (int i = 0; i < GT; i++) {
    const T* qp = q + ((size_t)t * Hq + h0 + i) * D;
#pragma unroll
    for (int j = 0; j < E; j++) { qr[i][j] = Cvt<T>::to_f(qp[j * 32 + lane]) * scale; acc[i][j] = 0.f; }
    m[i] = -INFINITY;
    l[i] = 0.f;
  }
  const int* bt = block_tables + (size_t)b * max_blocks;
  for (int k = lo; k <= pos; k++) {
    int blk = bt[k / block_size];
    size_t off = (((size_t)blk * block_size + k % block_size) * Hkv + kvh) * D;
    float kf[E], vf[E];
#pragma unroll
    for (int j = 0; j < E; j++) {
      kf[j] = Cvt<T>::to_f(kcache[off + j * 32 + lane]);
      vf[j] = Cvt<T>::to_f(vcache[off + j * 32 + lane]);
    }
#pragma unroll
    for (int i = 0; i < GT; i++) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < E; j++) s += qr[i][j] * kf[j];
      s = warp_sum(s);
      float mn = fmaxf(m[i], s);
      float corr = __expf(m[i] - mn), p = __expf(s - mn);
      l[i] = l[i] * corr + p;
#pragma unroll
      for (int j = 0; j < E; j++) acc[i][j] = acc[i][j] * corr + p * vf[j];
      m[i] = mn;
    }
  }
#pragma unroll
  for (int i = 0; i < GT; i++) {
    float lt = l[i], sc = 1.f;
    if (sinks) {
      float sk = sinks[h0 + i], mn = fmaxf(m[i], sk);
      sc = __expf(m[i] - mn);
      lt = l[i] * sc + __expf(sk - mn);
    }
    float inv = lt > 0.f ? sc / lt : 0.f;
    T* op = out + ((size_t)t * Hq + h0 + i) * D;
#pragma unroll
    for (int j = 0; j < E; j++) op[j * 32 + lane] = Cvt<T>::from_f(acc[i][j] * inv);
  }
}

// tok_seq[t] = index of the sequence token t belongs to (built on device from cu_q)
__global__ void token_seq_kernel(const int* __restrict__ cu_q, int* __restrict__ tok_seq, int B) {
  int b = blockIdx.x;
  for (int t = cu_q[b] + threadIdx.x; t < cu_q[b + 1]; t += blockDim.x) tok_seq[t] = b;
}

EXO_API int exo_token_seq(const int* cu_q, int* tok_seq, int B, cudaStream_t st) {
  if (B == 0) return 0;
  token_seq_kernel<<<B, 256, 0, st>>>(cu_q, tok_seq, B);
  EXO_CHECK_LAUNCH();
  return 0;
}

EXO_API int exo_paged_ragged(const void* q, const void* kcache, const void* vcache, const int* block_tables,
                             const int* seq_lens, const int* cu_q, const int* tok_seq, void* out, float scale, int T_,
                             int Hq, int Hkv, int D, int max_blocks, int block_size, int window, const float* sinks,
                             int dtype, cudaStream_t st) {
  if (T_ == 0) return 0;
  int g = Hq / Hkv;
  if (g * Hkv != Hq) return -2;
  int GT = (g % 4 == 0) ? 4 : (g % 2 == 0 ? 2 : 1);
  if (D == 512 && GT > 2) GT = 2;      // 16 values per lane and head: two heads' state is what the registers hold
  long warps = (long)T_ * Hkv * (g / GT);
  int blocks = (int)((warps + 3) / 4);
#define LAUNCH(TT, DD, GG)                                                                                          \
  paged_ragged_kernel<TT, DD, GG><<<blocks, 128, 0, st>>>((const TT*)q, (const TT*)kcache, (const TT*)vcache,        \
                                                          block_tables, seq_lens, cu_q, tok_seq, (TT*)out, scale, Hq, \
                                                          Hkv, max_blocks, block_size, window, sinks, T_)
#define BY_G(TT, DD)                   \
  if (GT == 4) LAUNCH(TT, DD, 4);      \
  else if (GT == 2) LAUNCH(TT, DD, 2); \
  else LAUNCH(TT, DD, 1)
  if (dtype == EXO_BF16) {
    if (D == 128) { BY_G(__nv_bfloat16, 128); }
    else if (D == 64) { BY_G(__nv_bfloat16, 64); }
    else if (D == 256) { BY_G(__nv_bfloat16, 256); }
    else if (D == 512) { if (GT == 2) LAUNCH(__nv_bfloat16, 512, 2); else LAUNCH(__nv_bfloat16, 512, 1); }
    else return -2;
  } else {
    if (D == 128) { BY_G(float, 128); }
    else if (D == 64) { BY_G(float, 64); }
    else if (D == 256) { BY_G(float, 256); }
    else if (D == 512) { if (GT == 2) LAUNCH(float, 512, 2); else LAUNCH(float, 512, 1); }
    else return -2;
  }
#undef BY_G
#undef LAUNCH
  EXO_CHECK_LAUNCH();
  return 0;
}
