// fp32 GEMM on the CUDA cores with in-kernel dequantisation:
//   y[m, o] = act(sum_k x[m,k] * W[o,k] + bias[o]) + res[m, o]
// This is the CATEN_B200_PREC_FP32 path for more than a few rows.  Each output is accumulated
// as `acc = acc + x*w` with k ascending, a rounded multiply followed by a rounded add — the same
// order and roundings as the C loop BACKEND=CLANG renders for !matmul (source/byoc/clang.lisp:58-111,
// api/high-level-ops.lisp:85-86) when gcc targets baseline x86-64 (no FMA contraction).
#include "common.cuh"
#include "blocks32.cuh"

namespace cb {


constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 32, SG_LD = 68;

template <int WT>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const void *__restrict__ qs, const __half *__restrict__ d,
                                                        const __half *__restrict__ mins, const uint32_t *__restrict__ qh5,
                                                        const float *__restrict__ x, const float *__restrict__ bias,
                                                        const float *res, float *y, int act, int64_t M, int64_t N,
                                                        int64_t K, int64_t nkb) {
  __shared__ __align__(16) float Xs[SG_BK * SG_LD];  // [k][m]
  __shared__ __align__(16) float Ws[SG_BK * SG_LD];  // [k][n]
  pdl_enter();
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * SG_BM, n0 = (int64_t)blockIdx.x * SG_BN;
  const int lrow = tid & 63, part = tid >> 6;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[a][e] = 0.0f;
  for (int kb = 0; kb < (int)(K / 32); ++kb) {
    float xv[8], wv[8];
    if (m0 + lrow < M) {
      const float4 *p = reinterpret_cast<const float4 *>(x + (m0 + lrow) * K + (int64_t)kb * 32 + part * 8);
      const float4 a = p[0], b = p[1];
      xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w; xv[4] = b.x; xv[5] = b.y; xv[6] = b.z; xv[7] = b.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) xv[e] = 0.0f;
    }
    if (WT == WT_F32_T) {
      // b[k, n]: thread reads 8 consecutive k for its column (coalesced across the 64 columns)
#pragma unroll
      for (int e = 0; e < 8; ++e)
        wv[e] = n0 + lrow < N ? ((const float *)qs)[((int64_t)kb * 32 + part * 8 + e) * N + n0 + lrow] : 0.0f;
    } else {
      load_w8<WT>(qs, d, mins, qh5, n0 + lrow, N, K, nkb, kb, part, wv);
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      Xs[(part * 8 + e) * SG_LD + lrow] = xv[e];
      Ws[(part * 8 + e) * SG_LD + lrow] = wv[e];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_BK; ++k) {
      const float4 xa = *reinterpret_cast<const float4 *>(Xs + k * SG_LD + 4 * ty);
      const float4 wa = *reinterpret_cast<const float4 *>(Ws + k * SG_LD + 4 * tx);
      const float xr[4] = {xa.x, xa.y, xa.z, xa.w}, wr[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[a][e] = acc[a][e] + xr[a] * wr[e];  // rounded mul, rounded add
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int64_t m = m0 + 4 * ty + a;
    if (m >= M) continue;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int64_t o = n0 + 4 * tx + e;
      if (o >= N) continue;
      float v = acc[a][e];
      if (bias) v = v + bias[o];
      v = apply_act(v, act);
      if (res) v = res[m * N + o] + v;
      y[m * N + o] = v;
    }
  }
}

template <int WT>
static int launch_simt(caten_b200_ctx *ctx, const void *qs, const __half *d, const __half *mins, const uint32_t *qh5, const float *x,
                       const float *bias, const float *res, int act, float *y, int64_t M, int64_t N, int64_t K) {
  if (K % 32) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm: inner dimension %lld is not a multiple of 32", (long long)K);
  const int64_t gx = (N + SG_BN - 1) / SG_BN, gy = (M + SG_BM - 1) / SG_BM;
  if (gy > 65535) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm: too many rows for one launch (%lld)", (long long)M);
  launch_k(ctx, gemm_simt_kernel<WT>, dim3((unsigned)gx, (unsigned)gy), dim3(256), 0, qs, d, mins, qh5, x, bias, res, y, act, M, N, K, K / 32);
  CB_LAUNCH_CHECK(ctx, "gemm_simt_kernel");
  return 0;
}

int launch_gemm_simt(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                     const float *res, int act, float *y, int64_t M) {
  if (M <= 0) return 0;
#define SIMT_CASE(T) \
  case T: return launch_simt<T>(ctx, w->qs, w->d, w->m, w->qh, x, bias, res, act, y, M, w->rows, w->cols)
  switch (w->type) {
    SIMT_CASE(CATEN_B200_F32);
    SIMT_CASE(CATEN_B200_F16);
    SIMT_CASE(CATEN_B200_Q8_0);
    SIMT_CASE(CATEN_B200_Q4_0);
    SIMT_CASE(CATEN_B200_Q4_1);
    SIMT_CASE(CATEN_B200_Q5_0);
    SIMT_CASE(CATEN_B200_Q5_1);
  }
#undef SIMT_CASE
  return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm: weight type %d", w->type);
}

int launch_relu_matmul_simt(caten_b200_ctx *ctx, const float *a, const float *b, float *c, int64_t M, int64_t K, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  return launch_simt<WT_F32_T>(ctx, b, nullptr, nullptr, nullptr, a, nullptr, nullptr, CATEN_B200_ACT_RELU, c, M, N, K);
}

}  // namespace cb
