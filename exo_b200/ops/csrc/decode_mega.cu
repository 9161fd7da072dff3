// One decode step of a dense transformer at batch 1 as ONE persistent kernel.
//
// At batch 1 a decode step reads every weight byte once; the only thing that matters is that HBM never idles.  As
// separate kernels (norm+QKV, RoPE/append, attention, O, gate/up, down: six launches per layer) every kernel pays a
// ring fill and a drain, and the small projections spend as long starting and stopping as streaming.  Here one CTA per
// SM stays resident for the whole step.  The CTA's share of the step's weight matrices — every layer's QKV, O, gate/up
// and down, then the vocabulary projection — is one long schedule of row groups; a ring of shared-memory stages is
// kept full along that schedule with `cp.async.bulk` copies (thread 0 refills a stage the moment all eight warps have
// left it), so the weight stream runs on through the phase boundaries: while the warps wait for the inputs of a phase,
// its first stages are already landing.  The eight warps run the phases:
//
//   A  qkv  = W_qkv . rmsnorm(h)                      (+bias)
//   B  attention of the new token: CTA (kv head, key split) applies q/k norm and RoPE, scores its key range of the
//      paged cache (the new token's k, v come straight from qkv) and publishes a partial (m, l, o); CTA (kv head, g)
//      combines the partials of query head g
//   C  h'  = h + W_o . attn
//   D  act = silu(W_gate . rmsnorm(h')) * (W_up . rmsnorm(h'))
//   E  h   = h' + W_down . act
//   ...next layer...; finally  logits = W_head . rmsnorm(h).
//
// There is no grid barrier, no atomic and no fence between the phases.  A vector that one phase hands to the next
// (qkv, attn, h', act, h) lives in global memory as 4-byte words {bf16 value, 16-bit tag}; an attention partial as
// 8-byte words {fp32 value, 32-bit tag}.  A word is written with one store, which arrives whole, and the tag names the
// (step, layer, phase) that wrote it: a consumer polls exactly the words it needs (L2 loads, with a time limit) until
// they carry the tag it expects.  Measured on B200, a counter- or flag-based grid barrier with its fences cost ~8 us
// under the weight stream's memory traffic, five times per layer; a tagged word costs one L2 round trip after its
// producer's store.  Buffer reuse is safe without further synchronisation because every phase needs the complete
// output of the one before it: by the time any CTA can write a buffer again, every CTA has finished reading its
// previous contents (the dependency chain is written out beside each buffer below).
//
// On an expired wait the CTA records an error in the host-mapped status word and stops waiting (its output is then
// meaningless, the host raises after the step), so the kernel always ends.  All CTAs are co-resident by construction:
// the grid is at most one CTA per SM and a CTA takes the SM's whole shared memory.
#include <cstdlib>
#include <cstring>
#include "status.h"
#include "tc_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;
typedef unsigned int u32;
constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS;          // 256 threads: the register file allows 255 per thread, and the phases need them
constexpr int RS_MAX = 32;
constexpr int G_MAX = 8;          // query heads per KV head
constexpr int HD = 128;           // head dim
constexpr int PW = HD + 2;        // words of one attention partial: m, l, o[HD]
constexpr int TRACE_SLOTS = 1024;
constexpr int FEED_THREAD = CONSUMERS - 32;   // lane 0 of the last warp walks the weight schedule

struct MegaLayer {
  const bf16* w_qkv; const bf16* b_qkv; const bf16* w_o; const bf16* w_gu; const bf16* w_down;
  const bf16* norm_attn; const bf16* norm_ffn; const bf16* q_norm; const bf16* k_norm;
  bf16* kcache; bf16* vcache;
};

struct MegaParams {
  const MegaLayer* layers;
  int n_layers;
  const bf16* embed; const int* tokens;
  const bf16* final_norm; const bf16* lm_head; bf16* logits; int vocab;
  // tagged vectors (u32 words).  Who may still be reading when a buffer is written again:
  u32* qkv;      // written A(l), read B(l).  A(l+1) needs E(l) <- D(l) <- C(l) <- every partial of B(l): all readers done.
  u32* attn;     // written B(l), read C(l).  B(l+1) needs A(l+1) on every CTA, and a CTA runs C(l) before that.
  u32* h_mid;    // written C(l), read D(l), E(l).  C(l+1) needs A(l+1) on every CTA, after its E(l).
  u32* act;      // written D(l), read E(l).  D(l+1) needs C(l+1) on every CTA, after its E(l).
  u32* h_out;    // written E(l), read A(l+1), C(l+1).  E(l+1) needs D(l+1) on every CTA, after its C(l+1).
  uint2* part;   // [n_kv][splits][G][PW] written B(l), read by the combiners of B(l); B(l+1) needs attn(l) complete.
  int* epoch;    // tag base of this launch; CTA 0 advances it when it is done
  unsigned long long* trace;      // optional [148][TRACE_SLOTS]: CTA c stamps the global timer at the end of each phase
                                  // (first half) and its thread 0's cumulative time spent waiting for weights (second half)
  const int* positions; const int* slots; const int* block_table; const int* seq_lens;
  const float* inv_freq; float mscale, eps, scale; int rot;
  int H, F, nq, nkv, block_size;
  int rs_h, rs_gu, rs_f;          // weight rows per ring stage for K = H (qkv, o, head), gate/up, K = F (down)
  int stages, slot_bytes;
  int* err;
  unsigned long long wait_ns;
};

__device__ __forceinline__ void bulk_g2s(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(tc::smem_u32(smem)), "l"(gmem), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void consumer_sync() { __syncthreads(); }

// ---- tagged words ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ u32 ld_word(const u32* p) {
  u32 v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_word4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_word(u32* p, u32 v) { asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_pair(uint2* p, float v, u32 tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ u32 pack_word(float v, u32 tag) {
  return (u32)__bfloat16_as_ushort(__float2bfloat16_rn(v)) | (tag << 16);
}
__device__ __forceinline__ float word_value(u32 w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ bool word_is(u32 w, u32 tag) { return (w >> 16) == (tag & 0xffffu); }

// Bounded spin bookkeeping: `it` counts polls, the clock is read every 64th.
struct Deadline {
  unsigned it = 0;
  unsigned long long t0 = 0;
  __device__ __forceinline__ bool expired(unsigned long long budget) {
    if ((++it & 63u) != 0) return false;
    const unsigned long long now = gtime();
    if (!t0) { t0 = now; return false; }
    return now - t0 > budget;
  }
};

struct Shared {
  uint64_t* full;
  float* part;      // [2][RS_MAX][CONSUMER_WARPS]
  float* red;       // [CONSUMER_WARPS]
  float* qs;        // [G_MAX][HD]   scaled, rotated queries
  float* kv_new;    // [2][HD]       the new token's rotated k, and v
  float* acc;       // [G_MAX][PW]   cross-warp merge of the attention state
  int* flag;
  uint8_t* ring;
};

// One value of a tagged vector (a residual element): polls until the tag is there.
__device__ __forceinline__ float wait_word(const MegaParams& p, const u32* w, u32 tag, bool ok) {
  u32 v = ld_word(w);
  if (ok && !word_is(v, tag)) {
    Deadline d;
    while (!word_is(v = ld_word(w), tag)) {
      if (d.expired(p.wait_ns)) { atomicExch(p.err, tc::ERR_TILE_TIMEOUT); break; }
    }
  }
  return word_value(v);
}

// ---- the weight schedule ---------------------------------------------------------------------------------------------
// Matrix `mat` of layer `li` (0 QKV, 1 O, 2 gate/up, 3 down; li == n_layers: the vocabulary projection).
struct MatDesc { const bf16* W; int rows_total, per, K; bool swiglu; };
__device__ __forceinline__ MatDesc mat_desc(const MegaParams& p, int li, int mat) {
  MatDesc d;
  if (li >= p.n_layers) { d.W = p.lm_head; d.rows_total = p.vocab; d.per = p.rs_h; d.K = p.H; d.swiglu = false; return d; }
  const MegaLayer& L = p.layers[li];
  if (mat == 0) { d.W = L.w_qkv; d.rows_total = (p.nq + 2 * p.nkv) * HD; d.per = p.rs_h; d.K = p.H; d.swiglu = false; }
  else if (mat == 1) { d.W = L.w_o; d.rows_total = p.H; d.per = p.rs_h; d.K = p.H; d.swiglu = false; }
  else if (mat == 2) { d.W = L.w_gu; d.rows_total = p.F; d.per = p.rs_gu / 2; d.K = p.H; d.swiglu = true; }
  else { d.W = L.w_down; d.rows_total = p.H; d.per = p.rs_f; d.K = p.F; d.swiglu = false; }
  return d;
}

// Thread 0's cursor along the CTA's schedule: the next row group to bring in.
struct Feeder {
  int li, mat, g;
  uint32_t seq;
  bool done;
  MatDesc d;
  __device__ __forceinline__ void settle(const MegaParams& p) {       // move on to the next matrix that has a group for this CTA
    while (!done) {
      d = mat_desc(p, li, mat);
      if (g * d.per < d.rows_total) return;
      g = blockIdx.x;
      if (li >= p.n_layers) { done = true; return; }
      if (++mat == 4) { mat = 0; li++; }
      if (li >= p.n_layers && !p.lm_head) { done = true; return; }
    }
  }
  __device__ __forceinline__ void init(const MegaParams& p) {
    li = 0; mat = 0; g = blockIdx.x; seq = 0; done = p.n_layers == 0 && !p.lm_head;
    settle(p);
  }
  // Bring the next group into stage seq % stages (the caller knows that stage is free).
  __device__ __forceinline__ void issue(const MegaParams& p, const Shared& s) {
    if (done) return;
    const int st = seq % p.stages;
    uint8_t* dst = s.ring + (size_t)st * p.slot_bytes;
    const int row_bytes = d.K * 2;
    const int r0 = g * d.per, rows = min(d.per, d.rows_total - r0);
    const uint32_t bytes = (uint32_t)rows * row_bytes;
    if (d.swiglu) {
      tc::mbar_expect_tx(&s.full[st], 2 * bytes);
      bulk_g2s(dst, d.W + (size_t)r0 * d.K, bytes, &s.full[st]);
      bulk_g2s(dst + (size_t)d.per * row_bytes, d.W + (size_t)(d.rows_total + r0) * d.K, bytes, &s.full[st]);
    } else {
      tc::mbar_expect_tx(&s.full[st], bytes);
      bulk_g2s(dst, d.W + (size_t)r0 * d.K, bytes, &s.full[st]);
    }
    seq++;
    g += gridDim.x;
    if (g * d.per >= d.rows_total) settle(p);       // the common case stays inside the matrix: no descriptor rebuild
  }
};

// ---- consumers: one streamed projection ----------------------------------------------------------------------------
// x: the input vector, either tagged words (x_ll, tag_in) or plain bf16 (x_plain: an embedding row).
// EPI 0: out = y (+bias);  1: out = residual + y;  2: out = silu(gate) * up.
// The result goes out as tagged words (out_ll, tag_out), or as plain bf16 (out_plain: the logits).
template <int JV, int RB, bool NORM, int EPI>
__device__ __forceinline__ bool gemv_phase(const MegaParams& p, const Shared& s, const u32* x_ll, const bf16* x_plain,
                                           u32 tag_in, const bf16* norm_w, const bf16* bias, const u32* res_ll,
                                           const bf16* res_plain, u32 tag_res, u32* out_ll, bf16* out_plain, u32 tag_out,
                                           int N, int K, int RS, uint32_t& seq, Feeder& feed, unsigned long long* starve, bool ok) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KS = K / CONSUMER_WARPS, k_lo = warp * KS, nvec = KS / 8;
  const int row_bytes = K * 2;
  float xr[JV][8];
  if (x_plain) {
#pragma unroll
    for (int j = 0; j < JV; j++) {
      const int v = lane + 32 * j;
      if (v < nvec) unpack8(*reinterpret_cast<const uint4*>(x_plain + k_lo + v * 8), xr[j]);
    }
  } else {
    // poll this lane's words until all of them carry the tag: every round has all loads in flight together
    Deadline d;
    for (;;) {
      bool all = true;
#pragma unroll
      for (int j = 0; j < JV; j++) {
        const int v = lane + 32 * j;
        if (v < nvec) {
          const uint4 a = ld_word4(x_ll + k_lo + v * 8), b = ld_word4(x_ll + k_lo + v * 8 + 4);
          all = all && word_is(a.x, tag_in) && word_is(a.y, tag_in) && word_is(a.z, tag_in) && word_is(a.w, tag_in) &&
                word_is(b.x, tag_in) && word_is(b.y, tag_in) && word_is(b.z, tag_in) && word_is(b.w, tag_in);
          xr[j][0] = word_value(a.x); xr[j][1] = word_value(a.y); xr[j][2] = word_value(a.z); xr[j][3] = word_value(a.w);
          xr[j][4] = word_value(b.x); xr[j][5] = word_value(b.y); xr[j][6] = word_value(b.z); xr[j][7] = word_value(b.w);
        }
      }
      if (all || !ok) break;
      if (d.expired(p.wait_ns)) { atomicExch(p.err, tc::ERR_TILE_TIMEOUT); ok = false; break; }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < JV; j++) {
    const int v = lane + 32 * j;
    if (v < nvec) {
      if (NORM) {
        float nw[8];
        unpack8(*reinterpret_cast<const uint4*>(norm_w + k_lo + v * 8), nw);
#pragma unroll
        for (int e = 0; e < 8; e++) { ss += xr[j][e] * xr[j][e]; xr[j][e] *= nw[e]; }
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) xr[j][e] = 0.f;
    }
  }
  float rstd = 1.f;
  consumer_sync();                             // red[] and flag are free again; all warps hold their slice of x
  if (NORM) {
    ss = warp_sum(ss);
    if (lane == 0) s.red[warp] = ss;
  }
  if (!ok) *s.flag = 0;
  consumer_sync();
  ok = ok && *s.flag != 0;                     // one warp's expired wait stops every warp's waiting
  if (NORM) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < CONSUMER_WARPS; w++) t += s.red[w];
    rstd = rsqrtf(t / K + p.eps);
  }
  const int rows_total = EPI == 2 ? N / 2 : N, per = EPI == 2 ? RS / 2 : RS;
  const int n_groups = (rows_total + per - 1) / per;
  for (int g = blockIdx.x; g < n_groups; g += gridDim.x, seq++) {
    const int st = seq % p.stages;
    // the residual element this thread will add: complete since the phase that consumed the whole vector, so a plain
    // L2 load issued now, a whole group's work before it is needed
    float resv = 0.f;
    if (EPI == 1 && threadIdx.x < RS && g * RS + (int)threadIdx.x < N)
      resv = res_plain ? __bfloat162float(res_plain[g * RS + threadIdx.x]) : word_value(ld_word(res_ll + g * RS + threadIdx.x));
    const long long c0 = starve ? clock64() : 0;
    if (ok && !tc::mbar_wait(&s.full[st], (seq / p.stages) & 1)) {
      atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
      ok = false;
    }
    const long long c1 = starve ? clock64() : 0;
    const uint8_t* src = s.ring + (size_t)st * p.slot_bytes + (size_t)k_lo * 2;
    float* pb = s.part + (size_t)(seq & 1) * RS_MAX * CONSUMER_WARPS;
    for (int rb = 0; rb < RS; rb += RB) {
      float acc[RB][2];
#pragma unroll
      for (int rr = 0; rr < RB; rr++) { acc[rr][0] = 0.f; acc[rr][1] = 0.f; }
#pragma unroll
      for (int j = 0; j < JV; j++) {
        const int v = lane + 32 * j;
        if (v < nvec) {
          uint4 wv[RB];
#pragma unroll
          for (int rr = 0; rr < RB; rr++)
            wv[rr] = *reinterpret_cast<const uint4*>(src + (size_t)(rb + rr) * row_bytes + v * 16);
#pragma unroll
          for (int rr = 0; rr < RB; rr++) {
            float wf[8];
            unpack8(wv[rr], wf);
#pragma unroll
            for (int e = 0; e < 8; e++) acc[rr][e & 1] += wf[e] * xr[j][e];
          }
        }
      }
      float tot[RB];
#pragma unroll
      for (int rr = 0; rr < RB; rr++) tot[rr] = acc[rr][0] + acc[rr][1];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int rr = 0; rr < RB; rr++) tot[rr] += __shfl_xor_sync(0xffffffffu, tot[rr], o);
      if (lane == 0) {
#pragma unroll
        for (int rr = 0; rr < RB; rr++) pb[(rb + rr) * CONSUMER_WARPS + warp] = tot[rr];
      }
    }
    const long long c2 = starve ? clock64() : 0;
    consumer_sync();                           // every warp has left the stage: it can take the next group of the schedule
    if (starve) { const long long c3 = clock64(); starve[0] += c1 - c0; starve[1] += c2 - c1; starve[2] += c3 - c2; }
    if (threadIdx.x == FEED_THREAD) feed.issue(p, s);   // a warp that has no rows to finalise
    const int t = threadIdx.x;
    if (EPI == 2) {
      const int half = RS / 2;
      if (t < half) {
        const int n = g * half + t;
        if (n < rows_total) {
          float gs = 0.f, us = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMER_WARPS; w++) { gs += pb[t * CONSUMER_WARPS + w]; us += pb[(t + half) * CONSUMER_WARPS + w]; }
          gs *= rstd; us *= rstd;
          if (bias) { gs += __bfloat162float(bias[n]); us += __bfloat162float(bias[rows_total + n]); }
          st_word(out_ll + n, pack_word(silu_f(gs) * us, tag_out));
        }
      }
    } else if (t < RS) {
      const int n = g * RS + t;
      if (n < N) {
        float y = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; w++) y += pb[t * CONSUMER_WARPS + w];
        y *= rstd;
        if (bias) y += __bfloat162float(bias[n]);
        if (EPI == 1) y += resv;
        if (out_plain) out_plain[n] = __float2bfloat16_rn(y);
        else st_word(out_ll + n, pack_word(y, tag_out));
      }
    }
  }
  return ok;
}

// ---- consumers: attention of the new token ---------------------------------------------------------------------------
// lane owns elements j*32 + lane of a head (the RoPE partner of an element is then in the same lane)
__device__ __forceinline__ bool load_head_ll(const MegaParams& p, const u32* src, u32 tag, int lane, float* v, bool ok) {
  Deadline d;
  for (;;) {
    bool all = true;
#pragma unroll
    for (int j = 0; j < HD / 32; j++) {
      const u32 w = ld_word(src + j * 32 + lane);
      all = all && word_is(w, tag);
      v[j] = word_value(w);
    }
    if (__all_sync(0xffffffffu, all) || !ok) break;
    if (d.expired(p.wait_ns)) { atomicExch(p.err, tc::ERR_TILE_TIMEOUT); ok = false; }
    ok = __all_sync(0xffffffffu, ok);
  }
  return ok;
}

__device__ __forceinline__ void norm_rope(const MegaParams& p, float* v, const bf16* nw, float pos, int lane) {
  constexpr int E = HD / 32;
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < E; j++) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / HD + p.eps);
#pragma unroll
    for (int j = 0; j < E; j++) v[j] = __bfloat162float(__float2bfloat16_rn(v[j] * rstd * __bfloat162float(nw[j * 32 + lane])));
  }
  const int EH = p.rot / 64;                 // elements per lane in each rotated half (rot is a multiple of 64)
  for (int j = 0; j < EH; j++) {
    float sn, cs;
    sincosf(pos * p.inv_freq[j * 32 + lane], &sn, &cs);
    sn *= p.mscale; cs *= p.mscale;
    const float a = v[j], b = v[j + EH];
    v[j] = a * cs - b * sn;
    v[j + EH] = b * cs + a * sn;
  }
}

// merge (m2, l2, o2) into (m1, l1, o1)
template <int N>
__device__ __forceinline__ void merge_state(float& m1, float& l1, float* o1, float m2, float l2, const float* o2) {
  const float mn = fmaxf(m1, m2);
  const float c1 = m1 == -INFINITY ? 0.f : __expf(m1 - mn), c2 = m2 == -INFINITY ? 0.f : __expf(m2 - mn);
#pragma unroll
  for (int j = 0; j < N; j++) o1[j] = o1[j] * c1 + o2[j] * c2;
  l1 = l1 * c1 + l2 * c2;
  m1 = mn;
}

template <int GT>
__device__ __forceinline__ bool attention_phase(const MegaParams& p, const Shared& s, const MegaLayer& L, u32 tag_qkv,
                                              u32 tag_out, bool ok) {
  constexpr int E = HD / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.nq / p.nkv, splits = (int)gridDim.x / p.nkv;
  const int kvh = (int)blockIdx.x / splits, split = (int)blockIdx.x - kvh * splits;
  if (kvh >= p.nkv) return ok;               // the CTAs past n_kv * splits sit this phase out
  const int pos = p.positions[0], seq_len = p.seq_lens[0];
  const float fpos = (float)pos;
  // the group's queries and the new token's k, v: rounded to bf16 as the unfused kernels store them
  for (int u = warp; u < G + 2; u += CONSUMER_WARPS) {
    float v[E];
    if (u < G) {
      ok = load_head_ll(p, p.qkv + (size_t)(kvh * G + u) * HD, tag_qkv, lane, v, ok);
      norm_rope(p, v, L.q_norm, fpos, lane);
#pragma unroll
      for (int j = 0; j < E; j++) s.qs[u * HD + j * 32 + lane] = __bfloat162float(__float2bfloat16_rn(v[j])) * p.scale;
    } else {
      const bool is_k = u == G;
      ok = load_head_ll(p, p.qkv + (size_t)(p.nq + (is_k ? 0 : p.nkv) + kvh) * HD, tag_qkv, lane, v, ok);
      if (is_k) norm_rope(p, v, L.k_norm, fpos, lane);
      bf16* dst = (is_k ? L.kcache : L.vcache) + ((size_t)p.slots[0] * p.nkv + kvh) * HD;
#pragma unroll
      for (int j = 0; j < E; j++) {
        const bf16 r = __float2bfloat16_rn(v[j]);
        s.kv_new[(is_k ? 0 : HD) + j * 32 + lane] = __bfloat162float(r);
        if (split == 0) dst[j * 32 + lane] = r;          // one CTA of the head appends to the cache
      }
    }
  }
  if (!ok) *s.flag = 0;
  consumer_sync();
  ok = *s.flag != 0;
  // this warp's share of the split's keys
  const int per = (seq_len + splits - 1) / splits;
  const int k0 = split * per, k1 = min(seq_len, k0 + per);
  float q[GT][E];
#pragma unroll
  for (int g = 0; g < GT; g++)
#pragma unroll
    for (int j = 0; j < E; j++) q[g][j] = g < G ? s.qs[g * HD + lane * E + j] : 0.f;
  float m[GT], l[GT], o[GT][E];
#pragma unroll
  for (int g = 0; g < GT; g++) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < E; j++) o[g][j] = 0.f;
  }
  // KU consecutive keys per warp and round: all their K and V loads are in flight before the first score is formed
  constexpr int KU = GT <= 4 ? 8 : 4;
  for (int kb = k0 + warp * KU; kb < k1; kb += CONSUMER_WARPS * KU) {
    uint2 kr[KU], vr[KU];
#pragma unroll
    for (int u = 0; u < KU; u++) {
      const int key = kb + u;
      if (key < k1 && key != pos) {
        const size_t slot = (size_t)p.block_table[key / p.block_size] * p.block_size + key % p.block_size;
        kr[u] = *reinterpret_cast<const uint2*>(L.kcache + (slot * p.nkv + kvh) * HD + lane * E);
        vr[u] = *reinterpret_cast<const uint2*>(L.vcache + (slot * p.nkv + kvh) * HD + lane * E);
      }
    }
#pragma unroll
    for (int u = 0; u < KU; u++) {
      const int key = kb + u;
      if (key >= k1) break;
      float kf[E], vf[E];
      if (key == pos) {
#pragma unroll
        for (int j = 0; j < E; j++) { kf[j] = s.kv_new[lane * E + j]; vf[j] = s.kv_new[HD + lane * E + j]; }
      } else {
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kr[u]);
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vr[u]);
        kf[0] = __low2float(k2[0]); kf[1] = __high2float(k2[0]); kf[2] = __low2float(k2[1]); kf[3] = __high2float(k2[1]);
        vf[0] = __low2float(v2[0]); vf[1] = __high2float(v2[0]); vf[2] = __low2float(v2[1]); vf[3] = __high2float(v2[1]);
      }
      float sc[GT];
#pragma unroll
      for (int g = 0; g < GT; g++) {
        sc[g] = 0.f;
        if (g < G) {
#pragma unroll
          for (int j = 0; j < E; j++) sc[g] += q[g][j] * kf[j];
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int g = 0; g < GT; g++)
          if (g < G) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], off);
#pragma unroll
      for (int g = 0; g < GT; g++) {
        if (g < G) {
          const float mn = fmaxf(m[g], sc[g]);
          const float corr = __expf(m[g] - mn), pr = __expf(sc[g] - mn);
          l[g] = l[g] * corr + pr;
#pragma unroll
          for (int j = 0; j < E; j++) o[g][j] = o[g][j] * corr + pr * vf[j];
          m[g] = mn;
        }
      }
    }
  }
  // merge the eight warps' states, one warp at a time, into acc[g] = (m, l, o[HD])
  for (int w = 0; w < CONSUMER_WARPS; w++) {
    if (warp == w) {
#pragma unroll
      for (int g = 0; g < GT; g++) {
        if (g < G) {
          float* a = s.acc + g * PW;
          if (w == 0) {
            if (lane == 0) { a[0] = m[g]; a[1] = l[g]; }
#pragma unroll
            for (int j = 0; j < E; j++) a[2 + lane * E + j] = o[g][j];
          } else {
            float am = a[0], al = a[1], ao[E];
#pragma unroll
            for (int j = 0; j < E; j++) ao[j] = a[2 + lane * E + j];
            __syncwarp();
            merge_state<E>(am, al, ao, m[g], l[g], o[g]);
#pragma unroll
            for (int j = 0; j < E; j++) a[2 + lane * E + j] = ao[j];
            if (lane == 0) { a[0] = am; a[1] = al; }
          }
        }
      }
    }
    consumer_sync();
  }
  // publish this split's partial as tagged pairs
  uint2* mine = p.part + ((size_t)(kvh * splits + split) * G) * PW;
  for (int i = threadIdx.x; i < G * PW; i += CONSUMERS) st_pair(mine + i, s.acc[i], tag_out);
  // CTA (kvh, g) combines query head g of the group (g + splits, ... too when there are fewer splits than heads)
  for (int g = split; g < G; g += splits) {
    consumer_sync();                           // acc is free again
    float M = -INFINITY, den = 0.f, out[E];
#pragma unroll
    for (int j = 0; j < E; j++) out[j] = 0.f;
    for (int sp = warp; sp < splits; sp += CONSUMER_WARPS) {
      const uint2* a = p.part + ((size_t)(kvh * splits + sp) * G + g) * PW;
      uint4 h0, o01, o23;
      Deadline d;
      for (;;) {
        h0 = ld_word4(a);                                          // (m, tag), (l, tag)
        o01 = ld_word4(a + 2 + lane * E);                           // (o[4 lane], tag), (o[4 lane + 1], tag)
        o23 = ld_word4(a + 2 + lane * E + 2);
        const bool all = h0.y == tag_out && h0.w == tag_out && o01.y == tag_out && o01.w == tag_out &&
                         o23.y == tag_out && o23.w == tag_out;
        if (__all_sync(0xffffffffu, all) || !ok) break;
        if (d.expired(p.wait_ns)) { atomicExch(p.err, tc::ERR_TILE_TIMEOUT); ok = false; }
        ok = __all_sync(0xffffffffu, ok);
      }
      const float o2[E] = {__uint_as_float(o01.x), __uint_as_float(o01.z), __uint_as_float(o23.x), __uint_as_float(o23.z)};
      merge_state<E>(M, den, out, __uint_as_float(h0.x), __uint_as_float(h0.z), o2);
    }
    float* a = s.acc + warp * PW;              // one slot per warp (the buffer has CONSUMER_WARPS == G_MAX slots)
    if (lane == 0) { a[0] = M; a[1] = den; }
#pragma unroll
    for (int j = 0; j < E; j++) a[2 + lane * E + j] = out[j];
    consumer_sync();
    if (warp == 0) {
      for (int w = 1; w < CONSUMER_WARPS; w++) {
        const float* b = s.acc + w * PW;
        float o2[E];
#pragma unroll
        for (int j = 0; j < E; j++) o2[j] = b[2 + lane * E + j];
        merge_state<E>(M, den, out, b[0], b[1], o2);
      }
      const float inv = den > 0.f ? 1.f / den : 0.f;
      u32* dst = p.attn + (size_t)(kvh * G + g) * HD + lane * E;
#pragma unroll
      for (int j = 0; j < E; j++) st_word(dst + j, pack_word(out[j] * inv, tag_out));
    }
  }
  return ok;
}

template <int JV_H, int RB_H, int JV_F, int RB_F>
__global__ void __launch_bounds__(THREADS, 1) decode_mega_kernel(const MegaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  Shared s;
  s.full = reinterpret_cast<uint64_t*>(base);
  s.part = reinterpret_cast<float*>(base + 128);
  s.red = s.part + 2 * RS_MAX * CONSUMER_WARPS;
  s.qs = s.red + CONSUMER_WARPS;
  s.kv_new = s.qs + G_MAX * HD;
  s.acc = s.kv_new + 2 * HD;
  s.flag = reinterpret_cast<int*>(s.acc + G_MAX * PW);
  s.ring = base + 128 + ((2 * RS_MAX * CONSUMER_WARPS + CONSUMER_WARPS + G_MAX * HD + 2 * HD + G_MAX * PW + 4) * 4 + 127) / 128 * 128;
  pdl_trigger();
  Feeder feed;
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; i++) tc::mbar_init(&s.full[i], 1);
    tc::fence_barrier_init();
    *s.flag = 1;
  }
  __syncthreads();
  if (threadIdx.x == FEED_THREAD) {
    // the weights are constants: the ring starts filling before the previous kernel of the stream has finished
    feed.init(p);
    for (int i = 0; i < p.stages; i++) feed.issue(p, s);
  }
  const int qkv_rows = (p.nq + 2 * p.nkv) * HD;
  uint32_t seq = 0;

  // ------------------------------ consumers ------------------------------
  pdl_wait();                                   // the step's inputs and the tag base come from earlier kernels
  bool ok = true;
  const u32 base_tag = (u32)*reinterpret_cast<volatile const int*>(p.epoch);
  const bf16* h0 = p.embed + (size_t)p.tokens[0] * p.H;             // the token's embedding row: layer 0's residual stream
  unsigned long long* tr = p.trace ? p.trace + (size_t)blockIdx.x * TRACE_SLOTS : nullptr;
  int n_stamp = 0;
  // trace only: cycles thread 32 (a warp that finalises no rows) spent waiting for weights, computing, and at the
  // block barrier, cumulative
  unsigned long long cyc[3] = {0, 0, 0};
  unsigned long long* starve = tr && threadIdx.x == 32 ? cyc : nullptr;
#define STAMP()                                                              \
  if (tr && n_stamp < TRACE_SLOTS / 4) {                                     \
    if (threadIdx.x == 32) {                                                 \
      tr[TRACE_SLOTS / 4 + n_stamp] = cyc[0];                                \
      tr[TRACE_SLOTS / 2 + n_stamp] = cyc[1];                                \
      tr[3 * TRACE_SLOTS / 4 + n_stamp] = cyc[2];                            \
    }                                                                        \
    if (threadIdx.x == 0) tr[n_stamp] = gtime();                             \
    n_stamp++;                                                               \
  }
  STAMP();
  for (int li = 0; li < p.n_layers; li++) {
    const MegaLayer& L = p.layers[li];
    const u32 t = base_tag + 1 + (u32)li * 5;   // tags of this layer's phases A .. E: t .. t + 4; E of the layer before: t - 1
    const bool first = li == 0;
    ok = gemv_phase<JV_H, RB_H, true, 0>(p, s, p.h_out, first ? h0 : nullptr, t - 1, L.norm_attn, L.b_qkv, nullptr, nullptr, 0,
                                         p.qkv, nullptr, t, qkv_rows, p.H, p.rs_h, seq, feed, starve, ok);
    STAMP();
    ok = p.nq <= 4 * p.nkv ? attention_phase<4>(p, s, L, t, t + 1, ok) : attention_phase<8>(p, s, L, t, t + 1, ok);
    STAMP();
    ok = gemv_phase<JV_H, RB_H, false, 1>(p, s, p.attn, nullptr, t + 1, nullptr, nullptr, p.h_out, first ? h0 : nullptr, t - 1,
                                          p.h_mid, nullptr, t + 2, p.H, p.H, p.rs_h, seq, feed, starve, ok);
    STAMP();
    ok = gemv_phase<JV_H, RB_H, true, 2>(p, s, p.h_mid, nullptr, t + 2, L.norm_ffn, nullptr, nullptr, nullptr, 0,
                                         p.act, nullptr, t + 3, 2 * p.F, p.H, p.rs_gu, seq, feed, starve, ok);
    STAMP();
    ok = gemv_phase<JV_F, RB_F, false, 1>(p, s, p.act, nullptr, t + 3, nullptr, nullptr, p.h_mid, nullptr, t + 2,
                                          p.h_out, nullptr, t + 4, p.H, p.F, p.rs_f, seq, feed, starve, ok);
    STAMP();
  }
  const u32 t_last = base_tag + (u32)p.n_layers * 5;
  if (p.lm_head)
    ok = gemv_phase<JV_H, RB_H, true, 0>(p, s, p.h_out, p.n_layers ? nullptr : h0, t_last, p.final_norm, nullptr, nullptr, nullptr, 0,
                                         nullptr, p.logits, 0, p.vocab, p.H, p.rs_h, seq, feed, starve, ok);
  STAMP();
#undef STAMP
  // CTA 0 cannot be here before every CTA has produced its share of every phase: the next launch starts from new tags
  if (blockIdx.x == 0 && threadIdx.x == 0) *reinterpret_cast<volatile int*>(p.epoch) = (int)t_last;
}

size_t fixed_smem() {
  return 128 + ((2 * RS_MAX * CONSUMER_WARPS + CONSUMER_WARPS + G_MAX * HD + 2 * HD + G_MAX * PW + 4) * 4 + 127) / 128 * 128 + 128;
}

int rows_per_stage(int K, bool pairs) {
  int rs = (32 * 1024) / (K * 2);
  if (rs < 1) rs = 1;
  if (rs > RS_MAX) rs = RS_MAX;
  if (rs >= 4) rs &= ~3;
  if (pairs) { rs &= ~1; if (rs < 2) rs = 2; }
  return rs;
}

int jv_of(int K) { return (K / 8 / CONSUMER_WARPS + 31) / 32; }

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

// Which (hidden, ffn) shapes the kernel is built for: 0 = none, else the variant number.
EXO_API int exo_decode_mega_variant(int H, int F, int nq, int nkv, int head_dim, int rot) {
  if (head_dim != HD || nq * head_dim != H || nkv < 1 || nq % nkv || nq / nkv > G_MAX || rot % 64 || rot > HD) return 0;
  if (H % 64 || F % 64 || nkv > 148) return 0;
  const int jh = jv_of(H), jf = jv_of(F);
  const int rh = rows_per_stage(H, false), rgu = rows_per_stage(H, true), rf = rows_per_stage(F, false);
  if (rgu != rh) return 0;
  if (jh <= 2 && rh % 4 == 0) {
    if (jf <= 4 && rf % 2 == 0) return 2;
    if (jf <= 8) return 1;
    if (jf <= 16) return 3;
  }
  if (jh <= 4 && rh % 2 == 0 && jf <= 16) return 4;
  return 0;
}

// Scratch: the tagged vectors, the attention partials and the tag base.  Zeroed once by the caller.
EXO_API long exo_decode_mega_workspace(int H, int F, int nq, int nkv) {
  const size_t qkv = align256((size_t)(nq + 2 * nkv) * HD * 4), hv = align256((size_t)H * 4), act = align256((size_t)F * 4);
  const size_t part = align256((size_t)148 * (nq / nkv) * PW * 8);
  return (long)(qkv + 3 * hv + act + part + 256);
}

// layers: device array of n_layers MegaLayer records (11 pointers each, in the order of the struct above).
// workspace: exo_decode_mega_workspace bytes.  trace: nullptr, or 148 * 1024 64-bit words.
EXO_API int exo_decode_mega(const void* layers, int n_layers, const void* embed, const int* tokens, const void* final_norm,
                            const void* lm_head, void* logits, int vocab, void* workspace, const int* positions,
                            const int* slots, const int* block_table, const int* seq_lens, const float* inv_freq,
                            float mscale, float eps, float scale, int rot, int H, int F, int nq, int nkv, int head_dim,
                            int block_size, int n_sm, void* trace, cudaStream_t st) {
  const int variant = exo_decode_mega_variant(H, F, nq, nkv, head_dim, rot);
  if (!variant) return -2;
  int* err = exo_status_word(EXO_STATUS_GEMV);
  if (!err) return -4;
  MegaParams p;
  memset(&p, 0, sizeof(p));
  p.layers = (const MegaLayer*)layers; p.n_layers = n_layers;
  p.embed = (const bf16*)embed; p.tokens = tokens;
  p.final_norm = (const bf16*)final_norm; p.lm_head = (const bf16*)lm_head; p.logits = (bf16*)logits; p.vocab = vocab;
  const size_t qkv = align256((size_t)(nq + 2 * nkv) * HD * 4), hv = align256((size_t)H * 4), act = align256((size_t)F * 4);
  const size_t part = align256((size_t)148 * (nq / nkv) * PW * 8);
  char* w = (char*)workspace;
  p.qkv = (u32*)w; w += qkv;
  p.attn = (u32*)w; w += hv;
  p.h_mid = (u32*)w; w += hv;
  p.h_out = (u32*)w; w += hv;
  p.act = (u32*)w; w += act;
  p.part = (uint2*)w; w += part;
  p.epoch = (int*)w;
  p.trace = (unsigned long long*)trace;
  p.positions = positions; p.slots = slots; p.block_table = block_table; p.seq_lens = seq_lens;
  p.inv_freq = inv_freq; p.mscale = mscale; p.eps = eps; p.scale = scale; p.rot = rot;
  p.H = H; p.F = F; p.nq = nq; p.nkv = nkv; p.block_size = block_size;
  p.rs_h = rows_per_stage(H, false); p.rs_gu = rows_per_stage(H, true); p.rs_f = rows_per_stage(F, false);
  size_t slot = (size_t)p.rs_h * H * 2;
  if ((size_t)p.rs_f * F * 2 > slot) slot = (size_t)p.rs_f * F * 2;
  slot = (slot + 127) / 128 * 128;
  const size_t fixed = fixed_smem();
  int stages = (int)((224 * 1024 - fixed) / slot);      // all but a few KB of the SM's shared memory is the ring
  if (stages > 8) stages = 8;
  if (stages < 2) return -2;
  p.stages = stages; p.slot_bytes = (int)slot;
  p.err = err;
  p.wait_ns = (unsigned long long)exo_wait_budget_ns();
  const size_t smem = fixed + (size_t)stages * slot;
  int grid = n_sm > 0 && n_sm < 148 ? n_sm : 148;
  if (grid < nkv) return -2;
  cudaError_t e = cudaErrorInvalidValue;
#define LAUNCH(A, B, C, D)                                                                                             \
  {                                                                                                                    \
    static bool attr = false;                                                                                          \
    if (!attr) {                                                                                                       \
      if (cudaFuncSetAttribute(decode_mega_kernel<A, B, C, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                               227 * 1024) != cudaSuccess) return -3;                                                  \
      attr = true;                                                                                                     \
    }                                                                                                                  \
    e = launch_pdl(decode_mega_kernel<A, B, C, D>, dim3(grid), dim3(THREADS), smem, st, p);                             \
  }
  if (variant == 1) LAUNCH(2, 4, 8, 1)
  else if (variant == 2) LAUNCH(2, 4, 4, 2)
  else if (variant == 3) LAUNCH(2, 4, 16, 1)
  else LAUNCH(4, 2, 16, 1)
#undef LAUNCH
  if (e != cudaSuccess) return (int)e;
  EXO_CHECK_LAUNCH();
  return 0;
}
