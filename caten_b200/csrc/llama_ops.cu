// The two Llama-style building blocks of source/nn that the GPT-2 path does not use but the same
// Transformer code takes for Llama-family models: RMSNorm (source/nn/normalization.lisp:70-85) and
// rotary positional encoding (source/nn/positional-encoding.lisp:3-56).  Both are HBM-bound
// element-wise kernels: one read and one write of the tensor.
#include "common.cuh"

namespace cb {

// y = x * (1 / sqrt(eps + mean(x * x))) [* weight]: one CTA of 256 threads per row, the row in
// registers (x is read once); d % 4 == 0, d <= 8192.
constexpr int RMS_THREADS = 256, RMS_MAXV = 8;

__global__ void __launch_bounds__(RMS_THREADS) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ y, int d4,
                                                              float invd, float eps) {
  __shared__ float red[RMS_THREADS / 32];
  pdl_enter();
  const int64_t row = blockIdx.x;
  const float4 *xr = reinterpret_cast<const float4 *>(x) + row * d4;
  float4 v[RMS_MAXV];
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < RMS_MAXV; ++i) {
    const int c = threadIdx.x + RMS_THREADS * i;
    if (c < d4) {
      v[i] = xr[c];
      sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int k = 1; k < RMS_THREADS / 32; ++k) t += red[k];
  const float rs = 1.0f / sqrtf(eps + t * invd);   // !recip (!sqrt (!add eps mean))
  float4 *yr = reinterpret_cast<float4 *>(y) + row * d4;
#pragma unroll
  for (int i = 0; i < RMS_MAXV; ++i) {
    const int c = threadIdx.x + RMS_THREADS * i;
    if (c < d4) {
      float4 o = make_float4(v[i].x * rs, v[i].y * rs, v[i].z * rs, v[i].w * rs);
      if (w) {
        const float4 g = reinterpret_cast<const float4 *>(w)[c];
        o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;
      }
      yr[c] = o;
    }
  }
}

int launch_rmsnorm(caten_b200_ctx *ctx, const float *x, const float *w, float *y, int64_t rows, int64_t d, float eps) {
  if (rows <= 0) return 0;
  if (d % 4 || d > 4 * RMS_THREADS * RMS_MAXV) return fail(ctx, CATEN_B200_EUNSUPPORTED, "rmsnorm: d=%lld (need d%%4==0, d<=8192)", (long long)d);
  if (rows > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "rmsnorm: too many rows");
  launch_k(ctx, rmsnorm_kernel, dim3((unsigned)rows), dim3(RMS_THREADS), 0, x, w, y, (int)(d / 4), 1.0f / (float)d, eps);
  CB_LAUNCH_CHECK(ctx, "rmsnorm_kernel");
  return 0;
}

// x [B, S, H, hd]: the pair (x[2i], x[2i+1]) of every head is rotated by the angle (pos0 + s) * theta_i,
//   theta_i = exp(-((2 i) / hd) * log(base)),  i < hd / 2;
// an odd last element is copied.  theta, sine and cosine are evaluated through double and rounded to
// fp32 once, which is what the C the reference renders does (libm functions applied to floats,
// source/codegen/renderer.lisp:362-370); cos(a) is taken as sin(a + pi/2) as the reference composes it
// (api/high-level-ops.lisp:119-122).
__global__ void __launch_bounds__(256) rope_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t total_pairs, int S, int H, int hd,
                                                   float base, int pos0) {
  pdl_enter();
  const int half = hd / 2;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_pairs) return;
  const int i = (int)(idx % half);
  const int64_t head = idx / half;           // (b * S + s) * H + h
  const int s = (int)((head / H) % S);
  const float expo = (float)(2 * i) * (1.0f / (float)hd);
  const float logb = (float)(log2((double)base)) * 0.6931472f;                       // !log = log2 * (log 2)
  const float theta = (float)exp2((double)(-(expo * logb)) * (double)(1.0f / 0.6931472f));  // !exp = exp2(x * 1/ln2)
  const float ang = (float)(pos0 + s) * theta;
  const float sn = (float)sin((double)ang);
  const float cs = (float)sin((double)(ang + 1.5707964f));
  const float *xp = x + head * hd + 2 * i;
  float *yp = y + head * hd + 2 * i;
  const float x0 = xp[0], x1 = xp[1];
  yp[0] = x0 * cs + (-(x1 * sn));
  yp[1] = x0 * sn + x1 * cs;
  if ((hd & 1) && i == half - 1) yp[2] = xp[2];
}

int launch_rope(caten_b200_ctx *ctx, const float *x, float *y, int64_t B, int64_t S, int64_t H, int64_t hd, float base, int64_t pos0) {
  if (B * S * H <= 0) return 0;
  if (hd < 2 || hd > 0x7fffffff || S > 0x7fffffff || H > 0x7fffffff) return fail(ctx, CATEN_B200_EINVAL, "rope: bad shape");
  const int64_t pairs = B * S * H * (hd / 2);
  const int64_t grid = (pairs + 255) / 256;
  if (grid > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "rope: tensor too large");
  launch_k(ctx, rope_kernel, dim3((unsigned)grid), dim3(256), 0, x, y, pairs, (int)S, (int)H, (int)hd, base, (int)pos0);
  CB_LAUNCH_CHECK(ctx, "rope_kernel");
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

int caten_b200_rmsnorm(caten_b200_ctx *ctx, const float *d_x, const float *d_weight, float *d_y, int64_t rows, int64_t d, float eps) {
  if (!ctx) return fail(nullptr, CATEN_B200_EINVAL, "rmsnorm: ctx is NULL");
  cudaSetDevice(ctx->device);
  if (!d_x || !d_y) return fail(ctx, CATEN_B200_EINVAL, "rmsnorm: NULL argument");
  if (rows < 0 || d <= 0) return fail(ctx, CATEN_B200_EINVAL, "rmsnorm: bad shape");
  return launch_rmsnorm(ctx, d_x, d_weight, d_y, rows, d, eps);
}

int caten_b200_rope(caten_b200_ctx *ctx, const float *d_x, float *d_y, int64_t B, int64_t S, int64_t H, int64_t head_dim, float base,
                    int64_t pos0) {
  if (!ctx) return fail(nullptr, CATEN_B200_EINVAL, "rope: ctx is NULL");
  cudaSetDevice(ctx->device);
  if (!d_x || !d_y) return fail(ctx, CATEN_B200_EINVAL, "rope: NULL argument");
  if (B < 0 || S < 0 || H < 0) return fail(ctx, CATEN_B200_EINVAL, "rope: bad shape");
  return launch_rope(ctx, d_x, d_y, B, S, H, head_dim, base, pos0);
}

}  // extern "C"
