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

}  // namespace cb
