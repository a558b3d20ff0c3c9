// GGUF block formats beyond those the kernels consume packed (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0): the
// 256-element "K" formats Q2_K, Q3_K, Q4_K, Q5_K, Q6_K.  The reference lists these type ids but
// implements none of them (external/gguf/tensor-info.lisp:3-34, 36-41); what it does for the
// types it knows is dequantise to fp32 at load (external/gguf/dequantize.lisp:14-53), and that is
// what happens here for these formats: the raw blocks are expanded once, on the device, into an
// fp32 weight that the fp32 kernels then use.  Formulas are ggml's published block layouts; each
// value is computed with separately rounded fp32 operations (scale products first, then the code
// product, then the offset), which is also how the Python `gguf` package dequantises.
#include "common.cuh"

namespace cb {

__device__ __forceinline__ float h2f(const uint8_t *p) {
  return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// 6-bit scale and minimum of sub-block j (0..7) from the 12 packed bytes of a Q4_K / Q5_K block
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int *sc, int *mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// K formats: 256 weights per block; one thread per weight
__global__ void dequant_block256_kernel(int type, const uint8_t *__restrict__ blocks, float *__restrict__ out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t blk = i >> 8;
  const int e = (int)(i & 255);
  float w;
  if (type == CATEN_B200_Q4_K || type == CATEN_B200_Q5_K) {
    // d, dmin, scales[12], (Q5_K: qh[32],) qs[128]; sub-block = e / 32, pairs of sub-blocks share 32 code bytes
    const uint8_t *b = blocks + blk * (type == CATEN_B200_Q4_K ? 144 : 176);
    const int sub = e >> 5, l = e & 31, g = sub >> 1, upper = sub & 1;
    int sc, mn;
    scale_min_k4(sub, b + 4, &sc, &mn);
    const float d = h2f(b) * (float)sc, m = h2f(b + 2) * (float)mn;
    const uint8_t *qs = b + (type == CATEN_B200_Q4_K ? 16 : 48);
    int q = upper ? qs[32 * g + l] >> 4 : qs[32 * g + l] & 15;
    if (type == CATEN_B200_Q5_K) q += (b[16 + l] >> sub) & 1 ? 16 : 0;
    w = d * (float)q - m;
  } else if (type == CATEN_B200_Q2_K) {
    // scales[16] (low nibble: scale, high nibble: minimum, per 16 weights), qs[64] (2-bit codes), d, dmin;
    // element = 128 half + 32 j + l uses bits [2j, 2j+2) of byte 32 half + l
    const uint8_t *b = blocks + blk * 84;
    const int half = e >> 7, j = (e >> 5) & 3, l = e & 31;
    const int sc = b[e >> 4];
    const float dl = h2f(b + 80) * (float)(sc & 15), ml = h2f(b + 82) * (float)(sc >> 4);
    const int q = (b[16 + 32 * half + l] >> (2 * j)) & 3;
    w = dl * (float)q - ml;
  } else if (type == CATEN_B200_Q3_K) {
    // hmask[32] (bit e/32 of byte e%32: high bit of the code), qs[64] (low 2 bits, laid out as in Q2_K),
    // scales[12] (16 six-bit scales: low nibbles in bytes 0..7, two more bits each in bytes 8..11), d
    const uint8_t *b = blocks + blk * 110;
    const int half = e >> 7, j = (e >> 5) & 3, l = e & 31, i = e >> 4;
    const uint8_t *s = b + 96;
    const int lo4 = (i < 8 ? s[i] : s[i - 8] >> 4) & 15, hi2 = (s[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
    const float dl = h2f(b + 108) * (float)((lo4 | (hi2 << 4)) - 32);
    const int ql = (b[32 + 32 * half + l] >> (2 * j)) & 3;
    const int q = ql - (((b[l] >> (e >> 5)) & 1) ? 0 : 4);
    w = dl * (float)q;
  } else {  // Q6_K: ql[128], qh[64], scales[16] (int8), d
    const uint8_t *b = blocks + blk * 210;
    const int half = e >> 7, r = e & 127, quarter = r >> 5, l = r & 31;  // element = 128 half + 32 quarter + l
    const uint8_t *ql = b + 64 * half, *qh = b + 128 + 32 * half;
    const int8_t *sc = reinterpret_cast<const int8_t *>(b + 192) + 8 * half;
    const int lo = (quarter & 1) ? ql[l + 32] : ql[l];
    const int nib = quarter >= 2 ? lo >> 4 : lo & 15;
    const int q = (nib | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
    const float d = h2f(b + 208) * (float)sc[(l >> 4) + 2 * quarter];
    w = d * (float)q;
  }
  out[i] = w;
}

// bytes of `n` weights in block format `type`, or -1 when the format is not one of this file's
int64_t extra_type_nbytes(int type, int64_t n, int64_t cols) {
  switch (type) {
    case CATEN_B200_Q2_K: return cols % 256 ? -1 : n / 256 * 84;
    case CATEN_B200_Q3_K: return cols % 256 ? -1 : n / 256 * 110;
    case CATEN_B200_Q4_K: return cols % 256 ? -1 : n / 256 * 144;
    case CATEN_B200_Q5_K: return cols % 256 ? -1 : n / 256 * 176;
    case CATEN_B200_Q6_K: return cols % 256 ? -1 : n / 256 * 210;
  }
  return -1;
}

int launch_dequant_extra(caten_b200_ctx *ctx, int type, const uint8_t *d_blocks, int64_t n, float *out) {
  if (n <= 0) return 0;
  const int64_t grid = (n + 255) / 256;
  if (grid > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "dequant: tensor too large");
  dequant_block256_kernel<<<(unsigned)grid, 256, 0, ctx->stream>>>(type, d_blocks, out, n);
  CB_LAUNCH_CHECK(ctx, "dequant_extra");
  return 0;
}

}  // namespace cb
