// Per-format arithmetic of one 32-wide block of a weight row against 32 activations held in
// registers: shared by the dequant-GEMV kernel and the single-kernel decode step.
#pragma once
#include "common.cuh"

namespace cb {

// ---- per-format block arithmetic -------------------------------------------------------------
// A thread owns one 32-wide column block kb of x and walks down the rows of W.
//
// Q4_0.  A nibble masked in place inside its 32-bit word, `w & (0xF << p)`, reinterpreted as a
// float, is the (sub)normal number nibble * 2^(p-149): the binary32 encoding is linear in its
// integer bit pattern below 2^24.  So with x pre-multiplied by 2^(64-p) (a power of two: exact),
// one AND plus one FMA accumulates x*nibble*2^-85 exactly as an fp32 FMA of x and nibble would,
// with no shift, integer-to-float conversion or subtraction per weight.  The "-8" offset of
// Q4_0 is folded into the accumulator's start value -8*sum(x)*2^-85, and 2^85 into the block
// scale.  Nibbles of the top byte (bits 24..31 overlap the exponent field) are taken from
// w >> 8.  Valid for |x| < 2^62; FMA with subnormal operands runs at full rate.
struct BlkQ4 {
  static constexpr bool HAS_M = false, HAS_QH = false;
  static constexpr int WORDS = 4;
  float xs[32];
  float c0;
  __device__ __forceinline__ void prep(const float *xv) {
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) sum += xv[j];
    c0 = sum * -0x1p-82f;  // -8 * 2^-85
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xs[8 * i + 0] = xv[4 * i + 0] * 0x1p64f;        // byte 0 low  nibble, p = 0
      xs[8 * i + 1] = xv[16 + 4 * i + 0] * 0x1p60f;   // byte 0 high nibble, p = 4
      xs[8 * i + 2] = xv[4 * i + 1] * 0x1p56f;        // byte 1 low,  p = 8
      xs[8 * i + 3] = xv[16 + 4 * i + 1] * 0x1p52f;   // byte 1 high, p = 12
      xs[8 * i + 4] = xv[4 * i + 2] * 0x1p48f;        // byte 2 low,  p = 16
      xs[8 * i + 5] = xv[16 + 4 * i + 2] * 0x1p44f;   // byte 2 high, p = 20
      xs[8 * i + 6] = xv[4 * i + 3] * 0x1p48f;        // byte 3 low  (of w >> 8), p = 16
      xs[8 * i + 7] = xv[16 + 4 * i + 3] * 0x1p44f;   // byte 3 high (of w >> 8), p = 20
    }
  }
  __device__ __forceinline__ float dot(const uint32_t *w, float scale) const {
    float a0 = c0, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t q = w[i], q8 = q >> 8;
      a0 = fmaf(xs[8 * i + 0], __uint_as_float(q & 0x0000000Fu), a0);
      a1 = fmaf(xs[8 * i + 1], __uint_as_float(q & 0x000000F0u), a1);
      a0 = fmaf(xs[8 * i + 2], __uint_as_float(q & 0x00000F00u), a0);
      a1 = fmaf(xs[8 * i + 3], __uint_as_float(q & 0x0000F000u), a1);
      a0 = fmaf(xs[8 * i + 4], __uint_as_float(q & 0x000F0000u), a0);
      a1 = fmaf(xs[8 * i + 5], __uint_as_float(q & 0x00F00000u), a1);
      a0 = fmaf(xs[8 * i + 6], __uint_as_float(q8 & 0x000F0000u), a0);
      a1 = fmaf(xs[8 * i + 7], __uint_as_float(q8 & 0x00F00000u), a1);
    }
    return (a0 + a1) * (scale * 0x1p85f);
  }
  // the block read from (shared) memory
  __device__ __forceinline__ float dotp(const uint4 *src, float scale) const {
    const uint4 v = src[0];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    return dot(w, scale);
  }
};

// Q8_0: sign-extended byte -> float -> FMA; (float)q * scale is exact in fp32 (8 + 11 bits), so
// scaling the 32-term sum once per block only changes where the roundings of the sum fall.
struct BlkQ8 {
  static constexpr bool HAS_M = false, HAS_QH = false;
  static constexpr int WORDS = 8;
  float xs[32];
  __device__ __forceinline__ void prep(const float *xv) {
#pragma unroll
    for (int j = 0; j < 32; ++j) xs[j] = xv[j];
  }
  __device__ __forceinline__ float dot(const uint32_t *w, float scale) const {
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t q = w[i];
      a0 = fmaf(xs[4 * i + 0], (float)(int8_t)(q), a0);
      a1 = fmaf(xs[4 * i + 1], (float)(int8_t)(q >> 8), a1);
      a0 = fmaf(xs[4 * i + 2], (float)(int8_t)(q >> 16), a0);
      a1 = fmaf(xs[4 * i + 3], (float)(int8_t)(q >> 24), a1);
    }
    return (a0 + a1) * scale;
  }
  __device__ __forceinline__ float dotp(const uint4 *src, float scale) const {
    const uint4 u = src[0], v = src[1];
    const uint32_t w[8] = {u.x, u.y, u.z, u.w, v.x, v.y, v.z, v.w};
    return dot(w, scale);
  }
};

// Q4_1: w = q * d + m.  The nibble arithmetic of BlkQ4 without the -8 offset; the minimum enters
// once per block as m * sum(x).
struct BlkQ41 {
  static constexpr bool HAS_M = true, HAS_QH = false;
  static constexpr int WORDS = 4;
  BlkQ4 nib;
  float sumx;
  __device__ __forceinline__ void prep(const float *xv) {
    nib.prep(xv);
    nib.c0 = 0.0f;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) sum += xv[j];
    sumx = sum;
  }
  __device__ __forceinline__ float dotx(const uint32_t *w, float scale, float mn, uint32_t) const {
    return nib.dot(w, scale) + mn * sumx;
  }
};

// Q5_0 (w = (q - 16) * d) and Q5_1 (w = q * d + m): code = nibble | bit e of qh << 4, converted
// with an integer-to-float instruction per weight.
template <bool WITH_MIN>
struct BlkQ5 {
  static constexpr bool HAS_M = WITH_MIN, HAS_QH = true;
  static constexpr int WORDS = 4;
  float xs[32];
  float sumx;
  __device__ __forceinline__ void prep(const float *xv) {
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      xs[j] = xv[j];
      sum += xv[j];
    }
    sumx = sum;
  }
  __device__ __forceinline__ float dotx(const uint32_t *w, float scale, float mn, uint32_t qh) const {
    constexpr int OFF = WITH_MIN ? 0 : 16;
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int j = 4 * i + b;  // byte j: elements j and j + 16
        const int lo = (int)((w[i] >> (8 * b)) & 15u) | (int)(((qh >> j) & 1u) << 4);
        const int hi = (int)((w[i] >> (8 * b + 4)) & 15u) | (int)(((qh >> (j + 16)) & 1u) << 4);
        a0 = fmaf(xs[j], (float)(lo - OFF), a0);
        a1 = fmaf(xs[j + 16], (float)(hi - OFF), a1);
      }
    }
    const float r = (a0 + a1) * scale;
    return WITH_MIN ? r + mn * sumx : r;
  }
};

// fp16 weights: 32 halves = 16 words
struct BlkF16 {
  static constexpr bool HAS_M = false, HAS_QH = false;
  static constexpr int WORDS = 16;
  float xs[32];
  __device__ __forceinline__ void prep(const float *xv) {
#pragma unroll
    for (int j = 0; j < 32; ++j) xs[j] = xv[j];
  }
  __device__ __forceinline__ float dot(const uint32_t *w, float) const {
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      a0 = fmaf(xs[2 * i], f.x, a0);
      a1 = fmaf(xs[2 * i + 1], f.y, a1);
    }
    return a0 + a1;
  }
  __device__ __forceinline__ float dotp(const uint4 *src, float) const {
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {   // one 16-byte piece (8 halves) at a time
      const uint4 v = src[q];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        a0 = fmaf(xs[8 * q + 2 * i], f.x, a0);
        a1 = fmaf(xs[8 * q + 2 * i + 1], f.y, a1);
      }
    }
    return a0 + a1;
  }
};

// fp32 weights: 32 floats = 32 words
struct BlkF32 {
  static constexpr bool HAS_M = false, HAS_QH = false;
  static constexpr int WORDS = 32;
  float xs[32];
  __device__ __forceinline__ void prep(const float *xv) {
#pragma unroll
    for (int j = 0; j < 32; ++j) xs[j] = xv[j];
  }
  __device__ __forceinline__ float dot(const uint32_t *w, float) const {
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      a0 = fmaf(xs[2 * i], __uint_as_float(w[2 * i]), a0);
      a1 = fmaf(xs[2 * i + 1], __uint_as_float(w[2 * i + 1]), a1);
    }
    return a0 + a1;
  }
  __device__ __forceinline__ float dotp(const uint4 *src, float) const {
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {   // one 16-byte piece (4 floats) at a time
      const float4 v = reinterpret_cast<const float4 *>(src)[q];
      a0 = fmaf(xs[4 * q], v.x, a0);
      a1 = fmaf(xs[4 * q + 1], v.y, a1);
      a0 = fmaf(xs[4 * q + 2], v.z, a0);
      a1 = fmaf(xs[4 * q + 3], v.w, a1);
    }
    return a0 + a1;
  }
};

}  // namespace cb
