// The 32-weight GGUF block formats that stay packed in device memory besides Q8_0: the four
// nibble formats (ggml's published layouts; the reference's loader knows their type ids,
// external/gguf/tensor-info.lisp:3-34, and implements Q8_0 only, dequantize.lisp:40-53):
//   Q4_0  d, qs[16]              w = (q - 8) * d          q = 4-bit code
//   Q4_1  d, m, qs[16]           w = q * d + m
//   Q5_0  d, qh[4], qs[16]       w = (q - 16) * d         q = 4-bit code | bit e of qh << 4
//   Q5_1  d, m, qh[4], qs[16]    w = q * d + m
// Byte j of qs holds element j (low nibble) and element j + 16 (high nibble).  On the device the
// fields of a matrix are split into arrays so that every code load is 16-byte aligned:
// codes[blocks][16], d[blocks] fp16, m[blocks] fp16 (the _1 formats), qh[blocks] u32 (the 5-bit
// formats).  Values are formed with separately rounded fp32 operations (the code product, then
// the offset), which is how the Python `gguf` package dequantises.
#pragma once
#include "common.cuh"

namespace cb {

__host__ __device__ constexpr bool type_is_nibble(int t) {
  return t == CATEN_B200_Q4_0 || t == CATEN_B200_Q4_1 || t == CATEN_B200_Q5_0 || t == CATEN_B200_Q5_1;
}
__host__ __device__ constexpr bool type_has_min(int t) { return t == CATEN_B200_Q4_1 || t == CATEN_B200_Q5_1; }
__host__ __device__ constexpr bool type_has_qh(int t) { return t == CATEN_B200_Q5_0 || t == CATEN_B200_Q5_1; }
// formats the kernels read in packed form
__host__ __device__ constexpr bool type_is_packed(int t) { return type_is_nibble(t) || t == CATEN_B200_Q8_0; }
__host__ __device__ constexpr int type_code_bytes(int t) { return t == CATEN_B200_Q8_0 ? 32 : 16; }
// bytes of one block in the file
__host__ __device__ constexpr int type_block_bytes(int t) {
  return 2 + (type_has_min(t) ? 2 : 0) + (type_has_qh(t) ? 4 : 0) + type_code_bytes(t);
}

// weight value of code q (nibble, with bit 4 from qh already merged for the 5-bit formats)
template <int WT>
__device__ __forceinline__ float nibble_value(int q, float d, float m) {
  if (WT == CATEN_B200_Q4_0) return (float)(q - 8) * d;
  if (WT == CATEN_B200_Q5_0) return (float)(q - 16) * d;
  return __fadd_rn(__fmul_rn((float)q, d), m);  // Q4_1, Q5_1
}

__device__ __forceinline__ float nibble_value_rt(int type, int q, float d, float m) {
  switch (type) {
    case CATEN_B200_Q4_0: return nibble_value<CATEN_B200_Q4_0>(q, d, m);
    case CATEN_B200_Q5_0: return nibble_value<CATEN_B200_Q5_0>(q, d, m);
    case CATEN_B200_Q4_1: return nibble_value<CATEN_B200_Q4_1>(q, d, m);
    default: return nibble_value<CATEN_B200_Q5_1>(q, d, m);
  }
}

// Eight consecutive weights of row `row`: elements part*8 .. part*8+7 of its 32-wide column block kb, as fp32
// (zeros beyond the last row).  Dense fp32 / fp16 rows, Q8_0, and the four nibble formats.
template <int WT>
__device__ __forceinline__ void load_w8(const void *qs, const __half *d, const __half *mins, const uint32_t *qh5, int64_t row,
                                        int64_t N, int64_t K, int64_t nkb, int kb, int part, float *o) {
  if (row >= N) {
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = 0.0f;
    return;
  }
  if (WT == CATEN_B200_F32) {
    const float4 *p = reinterpret_cast<const float4 *>((const float *)qs + row * K + (int64_t)kb * 32 + part * 8);
    const float4 a = p[0], b = p[1];
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  } else if (WT == CATEN_B200_F16) {
    const uint4 v = *reinterpret_cast<const uint4 *>((const __half *)qs + row * K + (int64_t)kb * 32 + part * 8);
    const __half *h = reinterpret_cast<const __half *>(&v);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = __half2float(h[e]);
  } else if (WT == CATEN_B200_Q8_0) {
    const int64_t bi = row * nkb + kb;
    const uint2 v = *reinterpret_cast<const uint2 *>((const int8_t *)qs + bi * 32 + part * 8);
    const float sc = __half2float(d[bi]);
    const int8_t *q = reinterpret_cast<const int8_t *>(&v);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = (float)q[e] * sc;
  } else if (type_is_nibble(WT)) {
    // elements part*8 .. part*8+7 of the block: parts 0,1 are the low nibbles of bytes 0-7, 8-15;
    // parts 2,3 the high nibbles of the same bytes; the 5-bit formats take bit 4 from qh
    const int64_t bi = row * nkb + kb;
    const uint2 v = *reinterpret_cast<const uint2 *>((const uint8_t *)qs + bi * 16 + (part & 1) * 8);
    const float sc = __half2float(d[bi]);
    const float mn = type_has_min(WT) ? __half2float(mins[bi]) : 0.0f;
    const uint32_t hb = type_has_qh(WT) ? qh5[bi] >> (part * 8) : 0u;
    const uint8_t *q = reinterpret_cast<const uint8_t *>(&v);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int nib = part < 2 ? (q[e] & 0x0F) : (q[e] >> 4);
      o[e] = nibble_value<WT>(nib | (int)(((hb >> e) & 1u) << 4), sc, mn);
    }
  }
}

}  // namespace cb
