// Temperature / top-k sampling of the next token from a row of logits.  The reference's generate
// loop only ever takes the argmax (apps/gpt2/gpt2.lisp:104-107, api/high-level-ops.lisp:314-343), so
// this entry has no counterpart there; it exists so that the loop can stay on the device when a
// caller wants sampled text.  Randomness comes from the caller (one uniform number per row), which
// keeps the kernel a pure function of its inputs.
//
// Per row (one CTA): m = max; keep the logits >= the k-th largest (all when k <= 0 or k >= V; ties
// at the threshold are all kept); w_i = exp2((x_i - m) * log2(e) / T) for kept i, else 0; the
// result is the first index i (in index order) whose running sum of w reaches u * sum(w).
#include <limits.h>

#include "common.cuh"

namespace cb {

constexpr int SAMPLE_THREADS = 1024;

// order-preserving map float -> uint32 (larger float <=> larger key)
__device__ __forceinline__ uint32_t sample_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_max(float v, float *red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = red[0];
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w) m = fmaxf(m, red[w]);
  return m;
}

// inclusive scan of one value per thread over the CTA, in thread order; returns this thread's
// prefix and writes the CTA total to *total
__device__ __forceinline__ float block_scan(float v, float *red, float *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = red[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    red[32 + lane] = s;  // inclusive prefix over the warps
  }
  __syncthreads();
  *total = red[32 + SAMPLE_THREADS / 32 - 1];
  return v + (warp > 0 ? red[32 + warp - 1] : 0.0f);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float *__restrict__ logits, int64_t V, float inv_t_log2e, int top_k,
                                                                const float *__restrict__ uniform, int64_t *__restrict__ out) {
  __shared__ float red[64];
  __shared__ unsigned hist[256];
  __shared__ uint32_t sel_prefix, sel_k;
  __shared__ long long found;
  pdl_enter();
  const float *x = logits + (int64_t)blockIdx.x * V;
  const int tid = threadIdx.x;
  float m = -INFINITY;
  for (int64_t i = tid; i < V; i += SAMPLE_THREADS) m = fmaxf(m, x[i]);
  m = block_max(m, red);

  // key of the k-th largest logit by an 8-bit radix select from the top byte down
  uint32_t thr = 0u;  // keep everything
  if (top_k > 0 && top_k < V) {
    if (tid == 0) { sel_prefix = 0u; sel_k = (uint32_t)top_k; }
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += SAMPLE_THREADS) hist[b] = 0u;
      __syncthreads();
      const uint32_t prefix = sel_prefix, mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (int64_t i = tid; i < V; i += SAMPLE_THREADS) {
        const uint32_t k = sample_key(x[i]);
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {  // walk the bins from the largest byte value down to the one holding the k-th largest
        uint32_t need = sel_k, b = 255;
        for (;; --b) {
          if (hist[b] >= need || b == 0) break;
          need -= hist[b];
        }
        sel_k = need;
        sel_prefix = prefix | (b << shift);
      }
      __syncthreads();
    }
    thr = sel_prefix;
  }

  // pass 1: total weight; pass 2: first index whose running sum reaches u * total
  float total = 0.0f, carry = 0.0f, target = 0.0f;
  if (tid == 0) found = LLONG_MAX;
  for (int pass = 0; pass < 2; ++pass) {
    carry = 0.0f;
    for (int64_t base = 0; base < V; base += SAMPLE_THREADS) {
      const int64_t i = base + tid;
      float w = 0.0f;
      if (i < V && sample_key(x[i]) >= thr) w = exp2f((x[i] - m) * inv_t_log2e);
      float chunk;
      const float pre = carry + block_scan(w, red, &chunk);
      if (pass == 1 && w > 0.0f && pre >= target) atomicMin(&found, (long long)i);
      carry += chunk;
      if (pass == 1) {
        __syncthreads();
        if (found != LLONG_MAX) break;  // uniform: every thread reads the same shared value after the barrier
      }
    }
    if (pass == 0) {
      total = carry;
      target = uniform[blockIdx.x] * total;
      __syncthreads();
    }
  }
  __syncthreads();
  if (tid == 0) {
    long long f = found;
    if (f == LLONG_MAX) {  // rounding left the last kept weight just short of the target: take the last kept index
      for (int64_t i = V - 1; i >= 0; --i)
        if (sample_key(x[i]) >= thr) { f = i; break; }
    }
    out[blockIdx.x] = f;
  }
}

int launch_sample(caten_b200_ctx *ctx, const float *logits, int64_t rows, int64_t V, float temperature, int top_k, const float *uniform,
                  int64_t *out) {
  if (rows <= 0) return 0;
  if (rows > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "sample: too many rows");
  const float inv_t_log2e = 1.4426950408889634f / temperature;
  launch_k(ctx, sample_kernel, dim3((unsigned)rows), dim3(SAMPLE_THREADS), 0, logits, V, inv_t_log2e, top_k, uniform, out);
  CB_LAUNCH_CHECK(ctx, "sample_kernel");
  return 0;
}

}  // namespace cb
