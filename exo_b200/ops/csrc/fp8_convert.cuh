// Widening block-scaled e4m3 weights to bf16 inside a kernel (shared by the fp8-weight GEMMs).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace fp8cvt {

// x holds two e4m3 bytes at bits [15:8] and [31:24].  Moving exponent and mantissa down by four
// bits gives bf16 patterns worth value * 2^-120 (subnormals included); c2 = two copies of the
// bf16 2^120 * scale.
__device__ __forceinline__ uint32_t cvt_pair(uint32_t x, uint32_t c2) {
  uint32_t y = (x & 0x80008000u) | ((x >> 4) & 0x07F007F0u);
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&y), *reinterpret_cast<__nv_bfloat162*>(&c2));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint4 cvt8(uint32_t w0, uint32_t w1, uint32_t c2) {
  uint4 o;
  o.x = cvt_pair(__byte_perm(w0, 0, 0x1404), c2);
  o.y = cvt_pair(__byte_perm(w0, 0, 0x3424), c2);
  o.z = cvt_pair(__byte_perm(w1, 0, 0x1404), c2);
  o.w = cvt_pair(__byte_perm(w1, 0, 0x3424), c2);
  return o;
}
// bf16 x2 of 2^120 * 2^(e - 127) for an e8m0 byte (exponent field e + 120, kept finite)
__device__ __forceinline__ uint32_t c2_from_e8m0(uint32_t e) {
  uint32_t f = min(e + 120u, 254u) << 7;
  return f | (f << 16);
}
__device__ __forceinline__ uint32_t c2_from_f32(float s) {
  __nv_bfloat16 b = __float2bfloat16_rn(fminf(s * 1.329227995784916e36f, 3.0e38f));     // * 2^120
  uint32_t f = *reinterpret_cast<uint16_t*>(&b);
  return f | (f << 16);
}

__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts16(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Row `r` (0..127) of a raw [128 x 64] byte tile -> row r of a 128-byte-swizzled bf16 [128 x 64] tile.
// c_lo / c_hi: the multipliers of the row's two 32-weight blocks.  `raw_tile` / `a_tile` are
// shared-memory addresses (cvta'd).  The rows of the raw tile are 64 bytes apart, so the threads of
// a warp start at different 16-byte pieces of their rows ((q + r/2) mod 4): eight neighbouring
// threads then touch eight different bank groups.
__device__ __forceinline__ void convert_row(uint32_t raw_tile, uint32_t a_tile, int r, uint32_t c_lo, uint32_t c_hi) {
  const uint32_t src = raw_tile + r * 64, dst = a_tile + r * 128;
  const int rot = (r >> 1) & 3;
  // all loads first, all stores last: the 32 independent pair conversions in between can then be interleaved by
  // the compiler (one warp per scheduler converts, so its own instruction-level parallelism is what hides latency)
  uint4 w[4], o[8];
#pragma unroll
  for (int q = 0; q < 4; q++) w[q] = lds16(src + ((q + rot) & 3) * 16);
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const uint32_t c2 = ((q + rot) & 3) < 2 ? c_lo : c_hi;
    o[2 * q] = cvt8(w[q].x, w[q].y, c2);
    o[2 * q + 1] = cvt8(w[q].z, w[q].w, c2);
  }
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int qq = (q + rot) & 3;
    sts16(dst + (((2 * qq) ^ (r & 7)) << 4), o[2 * q]);
    sts16(dst + (((2 * qq + 1) ^ (r & 7)) << 4), o[2 * q + 1]);
  }
}

// Half a row: bytes [32h, 32h + 32) of row r -> chunks 4h .. 4h+3 of the swizzled bf16 row, all under
// one multiplier.  Two threads per row (256 converter threads per tile) halve the per-thread chain.
__device__ __forceinline__ void convert_half_row(uint32_t raw_tile, uint32_t a_tile, int r, int h, uint32_t c2) {
  const uint32_t src = raw_tile + r * 64 + h * 32, dst = a_tile + r * 128;
  const int rot = (r >> 1) & 1;
  uint4 w[2], o[4];
#pragma unroll
  for (int q = 0; q < 2; q++) w[q] = lds16(src + ((q + rot) & 1) * 16);
#pragma unroll
  for (int q = 0; q < 2; q++) {
    o[2 * q] = cvt8(w[q].x, w[q].y, c2);
    o[2 * q + 1] = cvt8(w[q].z, w[q].w, c2);
  }
#pragma unroll
  for (int q = 0; q < 2; q++) {
    const int qq = 2 * h + ((q + rot) & 1);
    sts16(dst + (((2 * qq) ^ (r & 7)) << 4), o[2 * q]);
    sts16(dst + (((2 * qq + 1) ^ (r & 7)) << 4), o[2 * q + 1]);
  }
}

// Tiled weight storage (see ops/quant.py): every 128x64 block of the matrix is TILE_BYTES
// consecutive bytes — 8192 e4m3 values row-major, then 256 bytes of scales: 128 rows x 2 e8m0 bytes
// (kind 1) or one fp32 (kind 2).  A pipeline stage is one bulk copy of a tile.
constexpr uint32_t TILE_BODY = 128 * 64, TILE_BYTES = TILE_BODY + 256;

__device__ __forceinline__ void bulk_g2s(uint32_t smem, const void* gmem, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem), "l"(gmem), "r"(bytes), "r"(bar)
               : "memory");
}
// multipliers of row r of the tile at shared address `tile`
__device__ __forceinline__ void tile_scales(uint32_t tile, int kind, int r, uint32_t& c_lo, uint32_t& c_hi) {
  if (kind == 1) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(tile + TILE_BODY + 2 * r));
    c_lo = c2_from_e8m0(v & 0xffu);
    c_hi = c2_from_e8m0((v >> 8) & 0xffu);
  } else {
    float f;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(tile + TILE_BODY));
    c_lo = c_hi = c2_from_f32(f);
  }
}

// ---- e4m3 -> f16 with the hardware converter ------------------------------------------------------
// With f16 operands on both sides of the MMA the widening is two instructions per pair: the packed
// e4m3x2 -> f16x2 conversion (exact) and one packed multiply by the block scale (a power of two for
// e8m0 scales: exact too while the product stays in f16's range, which block-scaled weights do).
__device__ __forceinline__ void cvt4_f16(uint32_t w, uint32_t s2, uint32_t& p0, uint32_t& p1) {
  uint32_t a, b;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
      : "=r"(a), "=r"(b)
      : "r"(w));
  __half2 x = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&s2));
  __half2 y = __hmul2(*reinterpret_cast<__half2*>(&b), *reinterpret_cast<__half2*>(&s2));
  p0 = *reinterpret_cast<uint32_t*>(&x);
  p1 = *reinterpret_cast<uint32_t*>(&y);
}
// f16 x2 of 2^(e - 127); scales below f16's subnormal range become 0, above its range the largest power of two
__device__ __forceinline__ uint32_t s2_f16_from_e8m0(uint32_t e) {
  const int ex = (int)e - 127;                 // value 2^ex
  uint32_t h;
  if (ex >= -14) h = (uint32_t)min(ex + 15, 30) << 10;          // normal
  else if (ex >= -24) h = 1u << (ex + 24);                      // subnormal: 2^ex = 2^-24 * 2^(ex+24)
  else h = 0;
  return h | (h << 16);
}
__device__ __forceinline__ uint32_t s2_f16_from_f32(float s) {
  __half b = __float2half_rn(fminf(s, 65504.f));
  uint32_t h = *reinterpret_cast<uint16_t*>(&b);
  return h | (h << 16);
}
// f16 multipliers of row r of the tile at shared address `tile`
__device__ __forceinline__ void tile_scales_f16(uint32_t tile, int kind, int r, uint32_t& s_lo, uint32_t& s_hi) {
  if (kind == 1) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(tile + 128 * 64 + 2 * r));
    s_lo = s2_f16_from_e8m0(v & 0xffu);
    s_hi = s2_f16_from_e8m0((v >> 8) & 0xffu);
  } else {
    float f;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(tile + 128 * 64));
    s_lo = s_hi = s2_f16_from_f32(f);
  }
}

// ---- widened weights straight into tensor memory (the MMA's A operand) ----------------------------
// A [128 x 16] bf16 A operand in tensor memory has row i on lane i and two values per 32-bit column, which is how a
// converter thread holds its row: `n_words` consecutive columns are written with one tcgen05.st.
__device__ __forceinline__ void tmem_st16w(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_fence() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
// bytes [32h, 32h+32) of row r of the raw tile -> 16 columns at `taddr` (the caller adds lane quadrant, stage and 16*h)
__device__ __forceinline__ void convert_half_row_tmem(uint32_t raw_tile, uint32_t taddr, int r, int h, uint32_t c2) {
  const int rot = (r >> 1) & 1;
  const uint4 w0 = lds16(raw_tile + r * 64 + h * 32 + rot * 16);
  const uint4 w1 = lds16(raw_tile + r * 64 + h * 32 + (rot ^ 1) * 16);
  const uint4 lo = rot ? w1 : w0, hi = rot ? w0 : w1;
  const uint4 o0 = cvt8(lo.x, lo.y, c2), o1 = cvt8(lo.z, lo.w, c2), o2 = cvt8(hi.x, hi.y, c2), o3 = cvt8(hi.z, hi.w, c2);
  uint32_t o[16] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w, o2.x, o2.y, o2.z, o2.w, o3.x, o3.y, o3.z, o3.w};
  tmem_st16w(taddr, o);
}
// the same with f16 results (hardware e4m3 -> f16 converter and one packed multiply by the f16 scale `s2`)
__device__ __forceinline__ void convert_half_row_tmem_f16(uint32_t raw_tile, uint32_t taddr, int r, int h, uint32_t s2) {
  const int rot = (r >> 1) & 1;
  const uint4 w0 = lds16(raw_tile + r * 64 + h * 32 + rot * 16);
  const uint4 w1 = lds16(raw_tile + r * 64 + h * 32 + (rot ^ 1) * 16);
  const uint4 lo = rot ? w1 : w0, hi = rot ? w0 : w1;
  uint32_t o[16];
  cvt4_f16(lo.x, s2, o[0], o[1]); cvt4_f16(lo.y, s2, o[2], o[3]); cvt4_f16(lo.z, s2, o[4], o[5]); cvt4_f16(lo.w, s2, o[6], o[7]);
  cvt4_f16(hi.x, s2, o[8], o[9]); cvt4_f16(hi.y, s2, o[10], o[11]); cvt4_f16(hi.z, s2, o[12], o[13]); cvt4_f16(hi.w, s2, o[14], o[15]);
  tmem_st16w(taddr, o);
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], kind::f16
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"((uint32_t)acc)
      : "memory");
}

}  // namespace fp8cvt
