// Dequant-GEMV for decode with one sequence: y[o] = act(sum_k x[k] * W[o,k] + bias[o]) + res[o]
// (source/nn/linear.lisp:12-17 with M = 1).  HBM-bound: the packed weights are streamed once
// with 128-bit loads and unpacked in registers; x lives in registers (quantised types) or
// shared memory (fp32/fp16 weights).  fp32 accumulation throughout.
#include "common.cuh"
#include "blocks32.cuh"
#include "gemv_blocks.cuh"

namespace cb {

struct GemvArgs {
  const void *qs;
  const __half *d, *m;   // scales; minima (Q4_1, Q5_1)
  const uint32_t *qh;    // fifth code bits (Q5_0, Q5_1)
  const float *x, *bias, *res;
  float *y;
  int act, N, nkb, G;
};

constexpr int GEMV_MAX_THREADS = 512;

__device__ __forceinline__ uint4 ld_stream(const uint4 *p) { return __ldcs(p); }

// Thread t < G*nkb owns column block kb = t % nkb and row offset ro = t / nkb; a CTA iteration
// covers G*RI consecutive rows (RI independent 16/32-byte loads in flight per thread).  The
// per-(row, block) partial sums go through shared memory and are added in a fixed order (lane
// strided, then a butterfly), so results do not depend on scheduling.
template <class BLK, int RI>
__global__ void __launch_bounds__(GEMV_MAX_THREADS) gemv_blocked_kernel(GemvArgs a) {
  extern __shared__ float red[];
  // The packed weights depend on no other kernel: the first loads of this CTA's rows are issued
  // before waiting for the kernel that produces x, so their HBM latency overlaps its tail.
  pdl_launch_dependents();
  constexpr int W = BLK::WORDS;
  const int tid = threadIdx.x, nkb = a.nkb, G = a.G;
  const bool active = tid < G * nkb;
  const int kb = active ? tid % nkb : 0, ro = active ? tid / nkb : 0;
  const uint4 *qs = reinterpret_cast<const uint4 *>(a.qs);
  const int rows_per_iter = G * RI;
  const int warp = tid >> 5, lane = tid & 31, nwarps = (blockDim.x + 31) >> 5;
  const int64_t stride = (int64_t)gridDim.x * rows_per_iter;

  // The loads of iteration i+1 are issued before iteration i is reduced, and the partial sums
  // alternate between two shared-memory buffers, so there is one barrier per iteration and the
  // packed stream stays in flight across it.
  uint32_t qn[RI][W];
  float scn[RI], mnn[RI];
  uint32_t qhn[RI];
  auto load = [&](int64_t base) {
#pragma unroll
    for (int i = 0; i < RI; ++i) {
      const int64_t row = base + i * G + ro;
      const bool ok = active && row < a.N;
      const int64_t bidx = row * nkb + kb;
#pragma unroll
      for (int j = 0; j < W / 4; ++j) {
        const uint4 v = ok ? ld_stream(qs + bidx * (W / 4) + j) : make_uint4(0, 0, 0, 0);
        qn[i][4 * j] = v.x; qn[i][4 * j + 1] = v.y; qn[i][4 * j + 2] = v.z; qn[i][4 * j + 3] = v.w;
      }
      scn[i] = ok ? __half2float(a.d[bidx]) : 0.0f;
      if (BLK::HAS_M) mnn[i] = ok ? __half2float(a.m[bidx]) : 0.0f;
      if (BLK::HAS_QH) qhn[i] = ok ? a.qh[bidx] : 0u;
    }
  };
  int64_t base = (int64_t)blockIdx.x * rows_per_iter;
  if (base < a.N) load(base);
  pdl_wait();
  BLK blk;
  {
    float xv[32];
    const float4 *xp = reinterpret_cast<const float4 *>(a.x + (int64_t)kb * 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 v = xp[i];
      xv[4 * i] = v.x; xv[4 * i + 1] = v.y; xv[4 * i + 2] = v.z; xv[4 * i + 3] = v.w;
    }
    blk.prep(xv);
  }
  int buf = 0;
  for (; base < a.N; base += stride) {
    uint32_t q[RI][W], qhc[RI];
    float sc[RI], mn[RI];
#pragma unroll
    for (int i = 0; i < RI; ++i) {
      sc[i] = scn[i];
      mn[i] = BLK::HAS_M ? mnn[i] : 0.0f;
      qhc[i] = BLK::HAS_QH ? qhn[i] : 0u;
#pragma unroll
      for (int j = 0; j < W; ++j) q[i][j] = qn[i][j];
    }
    if (base + stride < a.N) load(base + stride);
    float *rb = red + buf * rows_per_iter * nkb;
    if (active) {
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        float r;
        if constexpr (BLK::HAS_M || BLK::HAS_QH) r = blk.dotx(q[i], sc[i], mn[i], qhc[i]);
        else r = blk.dot(q[i], sc[i]);
        rb[(i * G + ro) * nkb + kb] = r;
      }
    }
    __syncthreads();
    for (int r = warp; r < rows_per_iter; r += nwarps) {
      const int64_t row = base + r;
      if (row >= a.N) break;
      float s = 0.0f;
      for (int k = lane; k < nkb; k += 32) s += rb[r * nkb + k];
      s = warp_sum(s);
      if (lane == 0) {
        if (a.bias) s = s + a.bias[row];
        s = apply_act(s, a.act);
        if (a.res) s = a.res[row] + s;
        a.y[row] = s;
      }
    }
    buf ^= 1;
  }
}

// fp32 / fp16 weights: one warp per row, RI rows in flight, x in shared memory.
template <typename T> struct DenseLoad;
template <> struct DenseLoad<float> {
  static constexpr int VEC = 4;
  __device__ static __forceinline__ void load(const float *p, float *o) {
    const float4 v = __ldcs(reinterpret_cast<const float4 *>(p));
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct DenseLoad<__half> {
  static constexpr int VEC = 8;
  __device__ static __forceinline__ void load(const __half *p, float *o) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(p));
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
};

template <typename T, int RI>
__global__ void __launch_bounds__(256) gemv_dense_kernel(const T *__restrict__ W, const float *__restrict__ x,
                                                         const float *__restrict__ bias, const float *__restrict__ res,
                                                         float *__restrict__ y, int act, int N, int K) {
  extern __shared__ float xs[];
  // weights depend on no other kernel: the first tile of this warp's rows is loaded before the
  // wait for the producer of x
  pdl_launch_dependents();
  constexpr int VEC = DenseLoad<T>::VEC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = K / VEC;
  const int64_t first = ((int64_t)blockIdx.x * 8 + warp) * RI;
  float w0[RI][VEC];
#pragma unroll
  for (int i = 0; i < RI; ++i) {
    if (first + i < N && lane < nvec) DenseLoad<T>::load(W + (first + i) * K + (int64_t)lane * VEC, w0[i]);
    else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) w0[i][j] = 0.0f;
    }
  }
  pdl_wait();
  for (int i = threadIdx.x; i < K; i += blockDim.x) xs[i] = x[i];
  __syncthreads();
  for (int64_t base = first; base < N; base += (int64_t)gridDim.x * 8 * RI) {
    float acc[RI];
#pragma unroll
    for (int i = 0; i < RI; ++i) acc[i] = 0.0f;
    int c = lane;
    if (base == first && c < nvec) {  // the tile fetched before the wait
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float xv = xs[c * VEC + j];
#pragma unroll
        for (int i = 0; i < RI; ++i) acc[i] = fmaf(xv, w0[i][j], acc[i]);
      }
      c += 32;
    }
    // four tiles per lane in flight; the products are still added in increasing k
    for (; c < nvec; c += 32 * 4) {
      float wv[4][RI][VEC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int i = 0; i < RI; ++i) {
          if (c + 32 * u < nvec && base + i < N) {
            DenseLoad<T>::load(W + (base + i) * K + (int64_t)(c + 32 * u) * VEC, wv[u][i]);
          } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) wv[u][i][j] = 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (c + 32 * u < nvec) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            const float xv = xs[(c + 32 * u) * VEC + j];
#pragma unroll
            for (int i = 0; i < RI; ++i) acc[i] = fmaf(xv, wv[u][i][j], acc[i]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < RI; ++i) {
      float s = warp_sum(acc[i]);
      const int64_t row = base + i;
      if (lane == 0 && row < N) {
        if (bias) s = s + bias[row];
        s = apply_act(s, act);
        if (res) s = res[row] + s;
        y[row] = s;
      }
    }
  }
}

template <class BLK, int RI>
static int launch_blocked(caten_b200_ctx *ctx, const GemvArgs &a) {
  const int threads = ((a.G * a.nkb + 31) / 32) * 32;
  const size_t smem = 2 * (size_t)a.G * RI * a.nkb * sizeof(float);
  int occ = 1;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, gemv_blocked_kernel<BLK, RI>, threads, smem);
  if (occ < 1) occ = 1;
  const int64_t slabs = ((int64_t)a.N + a.G * RI - 1) / (a.G * RI);
  int64_t grid = (int64_t)ctx->sm_count * occ;
  if (grid > slabs) grid = slabs;
  launch_k(ctx, gemv_blocked_kernel<BLK, RI>, dim3((unsigned)grid), dim3(threads), smem, a);
  CB_LAUNCH_CHECK(ctx, "gemv_blocked_kernel");
  return 0;
}

int launch_gemv(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                const float *res, int act, float *y) {
  if (w->rows > 0x7fffffff || w->cols > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemv: dimension too large");
  const int N = (int)w->rows, K = (int)w->cols;
  if (type_is_packed(w->type)) {
    GemvArgs a;
    a.qs = w->qs; a.d = w->d; a.m = w->m; a.qh = w->qh; a.x = x; a.bias = bias; a.res = res; a.y = y; a.act = act; a.N = N;
    a.nkb = (int)w->nkb;
    if (a.nkb > GEMV_MAX_THREADS) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemv: cols=%d too wide (max %d)", K, GEMV_MAX_THREADS * 32);
    a.G = GEMV_MAX_THREADS / a.nkb;
    // few rows: keep every SM busy with single-row-group iterations; many rows: 4 loads in flight
    const bool deep = (int64_t)N >= (int64_t)a.G * 4 * ctx->sm_count;
    switch (w->type) {
      case CATEN_B200_Q4_0: return deep ? launch_blocked<BlkQ4, 4>(ctx, a) : launch_blocked<BlkQ4, 1>(ctx, a);
      case CATEN_B200_Q4_1: return deep ? launch_blocked<BlkQ41, 4>(ctx, a) : launch_blocked<BlkQ41, 1>(ctx, a);
      case CATEN_B200_Q5_0: return deep ? launch_blocked<BlkQ5<false>, 4>(ctx, a) : launch_blocked<BlkQ5<false>, 1>(ctx, a);
      case CATEN_B200_Q5_1: return deep ? launch_blocked<BlkQ5<true>, 4>(ctx, a) : launch_blocked<BlkQ5<true>, 1>(ctx, a);
      default: return deep ? launch_blocked<BlkQ8, 4>(ctx, a) : launch_blocked<BlkQ8, 1>(ctx, a);
    }
  }
  const size_t smem = (size_t)K * sizeof(float);
  if (smem > 160 * 1024) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemv: cols=%d too wide", K);
  // two rows per warp when that still gives every SM a CTA, else one row per warp (more CTAs)
  const bool two = ((int64_t)N + 15) / 16 >= ctx->sm_count;
  const int64_t groups = two ? ((int64_t)N + 15) / 16 : ((int64_t)N + 7) / 8;
  int64_t grid = (int64_t)ctx->sm_count * 4;
  if (grid > groups) grid = groups;
  if (w->type == CATEN_B200_F32) {
    if (K % 4) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemv f32: cols %% 4 != 0");
    if (smem > 48 * 1024) {
      cudaFuncSetAttribute(gemv_dense_kernel<float, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaFuncSetAttribute(gemv_dense_kernel<float, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (two) launch_k(ctx, gemv_dense_kernel<float, 2>, dim3((unsigned)grid), dim3(256), smem, (const float *)w->qs, x, bias, res, y, act, N, K);
    else launch_k(ctx, gemv_dense_kernel<float, 1>, dim3((unsigned)grid), dim3(256), smem, (const float *)w->qs, x, bias, res, y, act, N, K);
  } else if (w->type == CATEN_B200_F16) {
    if (K % 8) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemv f16: cols %% 8 != 0");
    if (smem > 48 * 1024) {
      cudaFuncSetAttribute(gemv_dense_kernel<__half, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaFuncSetAttribute(gemv_dense_kernel<__half, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (two) launch_k(ctx, gemv_dense_kernel<__half, 2>, dim3((unsigned)grid), dim3(256), smem, (const __half *)w->qs, x, bias, res, y, act, N, K);
    else launch_k(ctx, gemv_dense_kernel<__half, 1>, dim3((unsigned)grid), dim3(256), smem, (const __half *)w->qs, x, bias, res, y, act, N, K);
  } else {
    return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemv: weight type %d", w->type);
  }
  CB_LAUNCH_CHECK(ctx, "gemv_dense_kernel");
  return 0;
}

}  // namespace cb
