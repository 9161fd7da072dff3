// Widening block-scaled e4m3 weights to bf16 inside a kernel (shared by the fp8-weight GEMMs).
#pragma once
#include <cuda_bf16.h>
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
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int qq = (q + (r >> 1)) & 3;
    const uint4 w = lds16(src + qq * 16);
    const uint32_t c2 = qq < 2 ? c_lo : c_hi;
    sts16(dst + (((2 * qq) ^ (r & 7)) << 4), cvt8(w.x, w.y, c2));
    sts16(dst + (((2 * qq + 1) ^ (r & 7)) << 4), cvt8(w.z, w.w, c2));
  }
}

// The multipliers of ONE weight row, handed out K block by K block (64 weights = two 1x32 blocks).
// The loads run ahead of their use: with e8m0 scales and a 16-byte aligned start, one 16-byte load
// covers eight K blocks and the next one is issued eight blocks early; otherwise the scales of
// block i+1 are requested while block i is being converted.  kind 1: e8m0 bytes [rows, ld = K/32];
// kind 2: fp32 [rows/128, ld = ceil(K/128)].
struct ScaleStream {
  const uint8_t* row8;
  const float* rowf;
  int kind, kb0, nkb, k32;
  bool valid, vec;
  uint4 cur, nxt;
  uint32_t n_lo, n_hi;

  __device__ __forceinline__ void fetch(int kb, uint32_t& lo, uint32_t& hi) const {
    if (kind == 1) {
      lo = 2 * kb < k32 ? c2_from_e8m0(__ldg(row8 + 2 * kb)) : 0u;
      hi = 2 * kb + 1 < k32 ? c2_from_e8m0(__ldg(row8 + 2 * kb + 1)) : 0u;
    } else {
      lo = hi = c2_from_f32(__ldg(rowf + (kb >> 1)));
    }
  }
  __device__ __forceinline__ void init(const void* scale, int kind_, int ld, long n, int kb0_, int nkb_, int K, bool valid_) {
    kind = kind_; kb0 = kb0_; nkb = nkb_; k32 = K / 32; valid = valid_ && nkb_ > 0;
    row8 = reinterpret_cast<const uint8_t*>(scale) + (size_t)n * ld;
    rowf = reinterpret_cast<const float*>(scale) + (size_t)(n >> 7) * ld;
    vec = kind == 1 && (ld & 15) == 0 && (kb0 & 7) == 0 && (K & 63) == 0 && ((reinterpret_cast<uintptr_t>(scale) & 15) == 0);
    cur = nxt = make_uint4(0, 0, 0, 0);
    n_lo = n_hi = 0;
    if (!valid) return;
    if (vec) cur = __ldg(reinterpret_cast<const uint4*>(row8 + 2 * kb0));
    else fetch(kb0, n_lo, n_hi);
  }
  // multipliers of K block kb0 + i; call with i = 0, 1, 2, ... in order
  __device__ __forceinline__ void next(int i, uint32_t& c_lo, uint32_t& c_hi) {
    if (!valid) { c_lo = c_hi = 0; return; }
    if (vec) {
      const int j = i & 7;
      if (j == 0) {
        if (i) cur = nxt;
        if (i + 8 < nkb) nxt = __ldg(reinterpret_cast<const uint4*>(row8 + 2 * (kb0 + i + 8)));
      }
      const int wsel = j >> 1;
      const uint32_t w = wsel == 0 ? cur.x : wsel == 1 ? cur.y : wsel == 2 ? cur.z : cur.w;
      const uint32_t sh = (j & 1) * 16;
      c_lo = c2_from_e8m0((w >> sh) & 0xffu);
      c_hi = c2_from_e8m0((w >> (sh + 8)) & 0xffu);
    } else {
      c_lo = n_lo; c_hi = n_hi;
      if (i + 1 < nkb) fetch(kb0 + i + 1, n_lo, n_hi);
    }
  }
};

}  // namespace fp8cvt
