// Integer arithmetic shared by the grouped-INT4 kernels.
#pragma once
#include <cstdint>

namespace tb {

// ---------------------------------------------------------------------------
// Integer inner product (used by every kernel variant but the fp32 one).  Each 32-element block of x is turned once per
// CTA into a 24-bit block-fixed-point form: sx = 2^(floor(log2 max|x|) - 22) and
// q_i = rint(x_i / sx), |q_i| < 2^23, split into three byte digits
// q = d2 * 65536 + d1 * 256 + d0 (d0, d1 unsigned, d2 signed).  The nibbles stay
// unsigned bytes (two AND/shift per word give eight of them), and
//   sum_i q_i * code4_i = 65536 * dp4a(d2) + 256 * dp4a(d1) + dp4a(d0)
// is exact integer arithmetic; the -8 offset of the codes is applied through
// S = sum_i q_i, which is the same for every row.  Per element that is 0.75
// dp4a + 0.4 ALU instructions instead of ~3 for the fp32 path, which is what
// keeps the kernel on the HBM roofline rather than on the issue slots.  The
// only approximation is the rounding of x_i to a multiple of sx <= 2^-22 max|x|
// of its block, i.e. an absolute error per product no larger than the rounding
// error fp32 accumulation already makes at the block's magnitude.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int dp4a_us(uint32_t a_unsigned, uint32_t b_signed, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t dp4a_uu(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Digits are laid out per 8-element word wd as xq[wd*6 + {E0,E1,E2,O0,O1,O2}] (E = the even
// elements of the word, O = the odd ones, index = digit).  Returns sum_i q_i * code4_i over
// NWORDS words as fp32 (exact integer parts, combined in fp32).
template <int NWORDS>
__device__ __forceinline__ float idot_words(const uint32_t (&w)[NWORDS], const uint32_t (&xq)[NWORDS * 6]) {
  // two independent accumulator sets (even / odd elements) keep the dp4a chains short
  uint32_t d0 = 0, d1 = 0, e0 = 0, e1 = 0;
  int d2 = 0, e2 = 0;
#pragma unroll
  for (int wd = 0; wd < NWORDS; ++wd) {
    const uint32_t t = w[wd] & 0x0F0F0F0Fu;         // elements 0,2,4,6 of the word
    const uint32_t u = (w[wd] >> 4) & 0x0F0F0F0Fu;  // elements 1,3,5,7
    d0 = dp4a_uu(t, xq[wd * 6 + 0], d0);
    d1 = dp4a_uu(t, xq[wd * 6 + 1], d1);
    d2 = dp4a_us(t, xq[wd * 6 + 2], d2);
    e0 = dp4a_uu(u, xq[wd * 6 + 3], e0);
    e1 = dp4a_uu(u, xq[wd * 6 + 4], e1);
    e2 = dp4a_us(u, xq[wd * 6 + 5], e2);
  }
  d0 += e0; d1 += e1; d2 += e2;
  const int i01 = (int)(d0 + (d1 << 8));  // < 2^25, exact
  return fmaf(65536.0f, (float)d2, (float)i01);
}

// The same with the offset of the codes taken in the INTEGER domain: sum(q * (nibble - 8)) =
// sum(q * nibble) - 8 * S with 8 * S = 65536 * s8hi + s8lo (0 <= s8lo < 65536).  Both sums are about
// 2^30 when a block of x has one sign; subtracting them as floats would cost ~2^-15 of the block maximum.
template <int NWORDS>
__device__ __forceinline__ float idot_words_off(const uint32_t (&w)[NWORDS], const uint32_t (&xq)[NWORDS * 6], int s8hi, int s8lo) {
  uint32_t d0 = 0, d1 = 0, e0 = 0, e1 = 0;
  int d2 = 0, e2 = 0;
#pragma unroll
  for (int wd = 0; wd < NWORDS; ++wd) {
    const uint32_t t = w[wd] & 0x0F0F0F0Fu;
    const uint32_t u = (w[wd] >> 4) & 0x0F0F0F0Fu;
    d0 = dp4a_uu(t, xq[wd * 6 + 0], d0);
    d1 = dp4a_uu(t, xq[wd * 6 + 1], d1);
    d2 = dp4a_us(t, xq[wd * 6 + 2], d2);
    e0 = dp4a_uu(u, xq[wd * 6 + 3], e0);
    e1 = dp4a_uu(u, xq[wd * 6 + 4], e1);
    e2 = dp4a_us(u, xq[wd * 6 + 5], e2);
  }
  d0 += e0; d1 += e1; d2 += e2;
  const int i01 = (int)(d0 + (d1 << 8)) - s8lo;  // |.| < 2^25, exact
  return fmaf(65536.0f, (float)(d2 - s8hi), (float)i01);
}
// 8 * S as the two integers idot_words_off takes.
__device__ __forceinline__ void split_offset(int S, int& s8hi, int& s8lo) {
  const int s8 = S * 8;   // |S| <= 32 * 2^23: no overflow
  s8hi = s8 >> 16;        // arithmetic shift: floor
  s8lo = s8 & 0xFFFF;
}

__device__ __forceinline__ float idot32(const uint4 wv, const uint32_t (&xq)[24]) {
  const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
  return idot_words<4>(w, xq);
}

// Quantises NE consecutive elements of a 32-element block whose maximum magnitude is
// `amax` (NE = 32: the whole block; 16: one half, the maximum taken over both halves):
// digits + sx + S = sum(q) of these elements (the -8 offset of the codes contributes -8 * S).
template <int NE>
__device__ __forceinline__ void quantize_part_int(const float (&v)[NE], float amax, uint32_t (&dig)[NE / 8 * 6],
                                                  float& sx, int& S) {
  int e = (__float_as_int(amax) >> 23) & 0xFF;  // biased exponent of the block maximum
  if (e < 24) e = 24;                           // tiny / zero blocks: fixed scale 2^-125
  // Inf or NaN in the block (e == 255): the scale becomes NaN and so does the output.
  sx = (e == 255) ? __int_as_float(0x7FC00000) : __int_as_float((e - 22) << 23);
  const float inv = __int_as_float((276 - (e == 255 ? 254 : e)) << 23);
  S = 0;
  int q[NE];
#pragma unroll
  for (int i = 0; i < NE; ++i) {
    int qi = __float2int_rn(v[i] * inv);
    qi = max(-8388607, min(8388607, qi));
    q[i] = qi;
    S += qi;
  }
  // byte d of four elements -> one word: two byte permutes pick the byte from each pair, a third joins them
#pragma unroll
  for (int wd = 0; wd < NE / 8; ++wd)
#pragma unroll
    for (int par = 0; par < 2; ++par)
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        const uint32_t sel = (uint32_t)d | ((uint32_t)(4 + d) << 4);
        const uint32_t lo = __byte_perm((uint32_t)q[wd * 8 + par], (uint32_t)q[wd * 8 + 2 + par], sel);
        const uint32_t hi = __byte_perm((uint32_t)q[wd * 8 + 4 + par], (uint32_t)q[wd * 8 + 6 + par], sel);
        dig[wd * 6 + par * 3 + d] = __byte_perm(lo, hi, 0x5410);
      }
}

// The same with the offset term of the codes as a float: corr = -8 * sx * sum(q).
template <int NE>
__device__ __forceinline__ void quantize_part(const float (&v)[NE], float amax, uint32_t (&dig)[NE / 8 * 6],
                                              float& sx, float& corr) {
  int S;
  quantize_part_int<NE>(v, amax, dig, sx, S);
  corr = -8.0f * (float)S * sx;
}

template <int NE>
__device__ __forceinline__ float abs_max(const float (&v)[NE]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NE; ++i) amax = fmaxf(amax, fabsf(v[i]));
  return amax;
}

// Quantises one 32-element block (already normalised) into digits + (sx, -8*S*sx).
__device__ __forceinline__ void quantize_block(const float (&v)[32], uint32_t (&dig)[24], float& sx,
                                               float& corr) {
  quantize_part<32>(v, abs_max<32>(v), dig, sx, corr);
}

}  // namespace tb
