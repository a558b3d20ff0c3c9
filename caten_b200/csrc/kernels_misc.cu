// Small HBM-bound kernels of the GPT-2 graph: weight re-layout and dequantisation, LayerNorm,
// token+position embedding gather, arg-max.
#include "common.cuh"
#include "blocks32.cuh"

namespace cb {

// ---------------------------------------------------------------------------------------------
// GGUF blocks -> separate arrays of codes, scales, minima and fifth bits.  A block in the file is
// [fp16 d][fp16 m (Q4_1, Q5_1)][u32 qh (Q5_0, Q5_1)][codes: 32 int8 (Q8_0) or 16 bytes of nibbles]
// (external/gguf/dequantize.lisp:40-53 reads the Q8_0 fields in the same order).  The bytes are
// copied unchanged; only their placement differs.
// ---------------------------------------------------------------------------------------------
template <int TYPE>
__global__ void repack_kernel(const uint8_t *__restrict__ src, int64_t nblocks, uint8_t *__restrict__ qs,
                              __half *__restrict__ d, __half *__restrict__ m, uint32_t *__restrict__ qh) {
  constexpr int QBYTES = type_code_bytes(TYPE);
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const uint8_t *p = src + b * type_block_bytes(TYPE);
  d[b] = __ushort_as_half((uint16_t)((uint16_t)p[0] | ((uint16_t)p[1] << 8)));
  p += 2;
  if (type_has_min(TYPE)) {
    m[b] = __ushort_as_half((uint16_t)((uint16_t)p[0] | ((uint16_t)p[1] << 8)));
    p += 2;
  }
  if (type_has_qh(TYPE)) {
    qh[b] = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    p += 4;
  }
  uint32_t w[QBYTES / 4];
#pragma unroll
  for (int i = 0; i < QBYTES / 4; ++i)
    w[i] = (uint32_t)p[4 * i] | ((uint32_t)p[4 * i + 1] << 8) | ((uint32_t)p[4 * i + 2] << 16) | ((uint32_t)p[4 * i + 3] << 24);
  uint4 *o = reinterpret_cast<uint4 *>(qs + b * QBYTES);
#pragma unroll
  for (int i = 0; i < QBYTES / 16; ++i) o[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

int launch_repack(caten_b200_ctx *ctx, int type, const uint8_t *d_blocks, int64_t nblocks, void *qs, __half *d, __half *m,
                  uint32_t *qh) {
  const int threads = 256;
  const int64_t grid = (nblocks + threads - 1) / threads;
  if (grid > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "repack: too many blocks");
#define REPACK_CASE(T) \
  case T: repack_kernel<T><<<(unsigned)grid, threads, 0, ctx->stream>>>(d_blocks, nblocks, (uint8_t *)qs, d, m, qh); break
  switch (type) {
    REPACK_CASE(CATEN_B200_Q4_0);
    REPACK_CASE(CATEN_B200_Q4_1);
    REPACK_CASE(CATEN_B200_Q5_0);
    REPACK_CASE(CATEN_B200_Q5_1);
    REPACK_CASE(CATEN_B200_Q8_0);
    default: return fail(ctx, CATEN_B200_EUNSUPPORTED, "repack: type %d", type);
  }
#undef REPACK_CASE
  CB_LAUNCH_CHECK(ctx, "repack_kernel");
  return 0;
}

// Q8_0: w = (float)code * (float)scale, one rounded fp32 multiply (external/gguf/dequantize.lisp:51);
// the nibble formats: the formulas of blocks32.cuh.
__global__ void dequant_kernel(int type, const void *__restrict__ qs, const __half *__restrict__ d,
                               const __half *__restrict__ m, const uint32_t *__restrict__ qh, int64_t n,
                               float *__restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t blk = i >> 5;
  const int j = (int)(i & 31);
  if (type == CATEN_B200_F32) {
    out[i] = ((const float *)qs)[i];
  } else if (type == CATEN_B200_F16) {
    out[i] = __half2float(((const __half *)qs)[i]);
  } else if (type == CATEN_B200_Q8_0) {
    const int q = ((const int8_t *)qs)[blk * 32 + j];
    out[i] = (float)q * __half2float(d[blk]);
  } else {
    const uint8_t byte = ((const uint8_t *)qs)[blk * 16 + (j & 15)];
    int q = j < 16 ? (byte & 0x0F) : (byte >> 4);
    if (type_has_qh(type)) q |= (int)((qh[blk] >> j) & 1u) << 4;
    out[i] = nibble_value_rt(type, q, __half2float(d[blk]), type_has_min(type) ? __half2float(m[blk]) : 0.0f);
  }
}

int launch_dequant(caten_b200_ctx *ctx, const caten_b200_weight *w, float *out) {
  const int64_t n = w->rows * w->cols;
  const int threads = 256;
  const int64_t grid = (n + threads - 1) / threads;
  if (grid > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "dequant: tensor too large");
  dequant_kernel<<<(unsigned)grid, threads, 0, ctx->stream>>>(w->type, w->qs, w->d, w->m, w->qh, n, out);
  CB_LAUNCH_CHECK(ctx, "dequant_kernel");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// LayerNorm (source/nn/normalization.lisp:48-58): u = sum(x)*(1/d); dl = x - u;
// var = sum(dl*dl)*(1/d); y = dl * (1/sqrt(var+eps)) * gamma + beta.  One CTA of 256 threads per
// row, the row held in registers (x is read from HBM once); d % 4 == 0, d <= 2048.
// ---------------------------------------------------------------------------------------------
constexpr int LN_THREADS = 256, LN_MAXV = 2;  // float4 per thread

__device__ __forceinline__ float ln_block_sum(float v, float *red) {
  v = warp_sum(v);
  __syncthreads();  // protects `red` from the previous use
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int w = 1; w < LN_THREADS / 32; ++w) t += red[w];
  return t;
}

// PARTS: the row is residual + a pending split-K linear output (the batched partial-tile loads take ~64 more
// registers, which only the few-row decode launches can afford: without them 8 CTAs share an SM instead of 2).
template <bool PARTS>
__global__ void __launch_bounds__(LN_THREADS, PARTS ? 2 : 8) layernorm_kernel(const float *__restrict__ x, const float *__restrict__ g,
                                                               const float *__restrict__ b, float *__restrict__ y,
                                                               int d4, float invd, float eps, int64_t src_stride,
                                                               uint2 *__restrict__ yhi, uint2 *__restrict__ ylo,
                                                               const PartIn pin, float *__restrict__ xout) {
  __shared__ float red[LN_THREADS / 32];
  // Few-row launches (PARTS: a decode step) are one chain of latencies.  gamma and beta are parameters (written at
  // load), so they are staged in shared memory before the dependency wait and the loads the kernel ends with are not
  // one more L2 round trip behind its two reductions.  The many-row launches are bandwidth-bound and read them in place.
  __shared__ float4 gam[PARTS ? LN_THREADS * LN_MAXV : 1], bet[PARTS ? LN_THREADS * LN_MAXV : 1], pbias[PARTS ? LN_THREADS * LN_MAXV : 1];
  if (PARTS) {
#pragma unroll
    for (int i = 0; i < LN_MAXV; ++i) {
      const int c = threadIdx.x + LN_THREADS * i;
      if (c < d4) {
        gam[c] = reinterpret_cast<const float4 *>(g)[c];
        bet[c] = reinterpret_cast<const float4 *>(b)[c];
        if (pin.bias) pbias[c] = *reinterpret_cast<const float4 *>(pin.bias + 4 * c);  // the pending linear's bias: a parameter too
      }
    }
  }
  pdl_enter();
  const int64_t row = blockIdx.x;
  const int64_t src_row = src_stride > 1 ? (row + 1) * src_stride - 1 : row;
  const float4 *xr = reinterpret_cast<const float4 *>(x) + src_row * d4;
  float4 v[LN_MAXV];
  float sum = 0.0f;
  if (PARTS && pin.splits > 0) {
    // x is the residual input; the row normalised is residual + the pending linear output, which
    // also becomes the new residual stream.  The partial tiles of all the thread's columns are
    // fetched together, eight splits at a time (the kernel is latency-bound: 256 CTAs, a few
    // loads each), and added in split order.
    const float *src[LN_MAXV];
    float4 t[LN_MAXV];
    bool on[LN_MAXV];
#pragma unroll
    for (int i = 0; i < LN_MAXV; ++i) {
      const int c = threadIdx.x + LN_THREADS * i, o = 4 * c;
      on[i] = c < d4;
      const long long tile = (src_row / pin.bnx) * pin.tiles_x + (o >> 7);
      src[i] = pin.part + (tile * pin.bnx + (src_row % pin.bnx)) * 128 + (o & 127);
      t[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (on[i]) v[i] = xr[c];
    }
    for (int z0 = 0; z0 < pin.splits; z0 += 8) {
      float4 a[LN_MAXV][8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < LN_MAXV; ++i)
          if (on[i] && z0 + u < pin.splits) a[i][u] = __ldcs(reinterpret_cast<const float4 *>(src[i] + (long long)(z0 + u) * pin.zstride));
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < LN_MAXV; ++i)
          if (on[i] && z0 + u < pin.splits) { t[i].x += a[i][u].x; t[i].y += a[i][u].y; t[i].z += a[i][u].z; t[i].w += a[i][u].w; }
    }
#pragma unroll
    for (int i = 0; i < LN_MAXV; ++i) {
      const int c = threadIdx.x + LN_THREADS * i;
      if (on[i]) {
        if (pin.bias) {
          const float4 bb = pbias[c];
          t[i].x = t[i].x + bb.x; t[i].y = t[i].y + bb.y; t[i].z = t[i].z + bb.z; t[i].w = t[i].w + bb.w;
        }
        v[i].x = v[i].x + t[i].x; v[i].y = v[i].y + t[i].y; v[i].z = v[i].z + t[i].z; v[i].w = v[i].w + t[i].w;
        reinterpret_cast<float4 *>(xout)[src_row * d4 + c] = v[i];
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < LN_MAXV; ++i) {
      const int c = threadIdx.x + LN_THREADS * i;
      if (c < d4) {
        v[i] = xr[c];
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
  }
  const float u = ln_block_sum(sum, red) * invd;
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    const int c = threadIdx.x + LN_THREADS * i;
    if (c < d4) {
      v[i].x -= u; v[i].y -= u; v[i].z -= u; v[i].w -= u;
      sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  const float var = ln_block_sum(sq, red) * invd;
  const float rs = 1.0f / sqrtf(var + eps);
  float4 *yr = reinterpret_cast<float4 *>(y) + row * d4;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    const int c = threadIdx.x + LN_THREADS * i;
    if (c < d4) {
      const float4 gg = PARTS ? gam[c] : reinterpret_cast<const float4 *>(g)[c];  // (staged by this same thread)
      const float4 bb = PARTS ? bet[c] : reinterpret_cast<const float4 *>(b)[c];
      float4 o;
      o.x = (v[i].x * rs) * gg.x + bb.x;
      o.y = (v[i].y * rs) * gg.y + bb.y;
      o.z = (v[i].z * rs) * gg.z + bb.z;
      o.w = (v[i].w * rs) * gg.w + bb.w;
      if (yhi) {  // split bf16 operand of the GEMM that consumes this row
        yhi[row * d4 + c] = make_uint2(pack_bf16(o.x, o.y), pack_bf16(o.z, o.w));
        if (ylo) ylo[row * d4 + c] = make_uint2(pack_bf16(bf16_lo(o.x), bf16_lo(o.y)), pack_bf16(bf16_lo(o.z), bf16_lo(o.w)));
      } else {
        yr[c] = o;
      }
    }
  }
}

int launch_layernorm_strided(caten_b200_ctx *ctx, const float *x, const float *g, const float *b, float *y,
                             int64_t rows, int64_t d, float eps, int64_t src_stride, BfOut bf) {
  if (rows <= 0) return 0;
  if (d % 4 || d > 4 * LN_THREADS * LN_MAXV) return fail(ctx, CATEN_B200_EUNSUPPORTED, "layernorm: d=%lld (need d%%4==0, d<=2048)", (long long)d);
  if (rows > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "layernorm: too many rows");
  launch_k(ctx, layernorm_kernel<false>, dim3((unsigned)rows), dim3(LN_THREADS), 0, x, g, b, y, (int)(d / 4), 1.0f / (float)d, eps, src_stride,
                                                                   (uint2 *)bf.hi, (uint2 *)bf.lo, PartIn(), (float *)nullptr);
  CB_LAUNCH_CHECK(ctx, "layernorm_kernel");
  return 0;
}

int launch_layernorm_pending(caten_b200_ctx *ctx, const PartIn &pin, const float *res, float *xout, const float *g, const float *b,
                             float *y, int64_t rows, int64_t d, float eps, int64_t src_stride, BfOut bf) {
  if (rows <= 0) return 0;
  if (pin.splits <= 0 || !res || !xout) return fail(ctx, CATEN_B200_EINVAL, "layernorm: no pending linear output");
  if (d % 4 || d > 4 * LN_THREADS * LN_MAXV) return fail(ctx, CATEN_B200_EUNSUPPORTED, "layernorm: d=%lld (need d%%4==0, d<=2048)", (long long)d);
  if (rows > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "layernorm: too many rows");
  launch_k(ctx, layernorm_kernel<true>, dim3((unsigned)rows), dim3(LN_THREADS), 0, res, g, b, y, (int)(d / 4), 1.0f / (float)d, eps, src_stride,
                                                                   (uint2 *)bf.hi, (uint2 *)bf.lo, pin, xout);
  CB_LAUNCH_CHECK(ctx, "layernorm_kernel");
  return 0;
}

int launch_layernorm(caten_b200_ctx *ctx, const float *x, const float *g, const float *b, float *y, int64_t rows,
                     int64_t d, float eps) {
  return launch_layernorm_strided(ctx, x, g, b, y, rows, d, eps, 1, BfOut());
}

// ---------------------------------------------------------------------------------------------
// h[b,i,:] = wte[tok[b,i]] + wpe[n+i] (external/llm/layers.lisp:83-85).  The reference builds the
// token embedding as sum_v where(v == tok, W[v,:], 0) (source/nn/embedding.lisp:17-25): an id that
// matches no v contributes a zero row, which is kept here.
// ---------------------------------------------------------------------------------------------
__global__ void embed_kernel(const float *__restrict__ ids_f32, const int64_t *__restrict__ ids_i64,
                             const float *__restrict__ wte, const float *__restrict__ wpe, float *__restrict__ out,
                             int64_t s, int64_t n, const int *__restrict__ d_n, int d4, int64_t V, int64_t T) {
  pdl_enter();
  if (d_n) n = *d_n;  // position kept on the device (decode replayed from a CUDA graph)
  const int64_t r = blockIdx.x;
  int64_t tok = -1;
  if (ids_i64) {
    tok = ids_i64[r];
  } else {
    const float t = ids_f32[r];
    if (t >= 0.0f && t < (float)V && truncf(t) == t) tok = (int64_t)t;
  }
  const bool has_tok = tok >= 0 && tok < V;
  const int64_t pos = n + (r % s);
  const bool has_pos = pos >= 0 && pos < T;
  const float4 *te = reinterpret_cast<const float4 *>(wte) + (has_tok ? tok : 0) * d4;
  const float4 *pe = reinterpret_cast<const float4 *>(wpe) + (has_pos ? pos : 0) * d4;
  float4 *o = reinterpret_cast<float4 *>(out) + r * d4;
  for (int c = threadIdx.x; c < d4; c += blockDim.x) {
    float4 a = has_tok ? te[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 p = has_pos ? pe[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
    o[c] = a;
  }
}

int launch_embed(caten_b200_ctx *ctx, const float *ids_f32, const int64_t *ids_i64, const float *wte,
                 const float *wpe, float *out, int64_t B, int64_t s, int64_t n, int64_t d, int64_t V, int64_t T, const int *d_n) {
  if (B * s <= 0) return 0;
  if (d % 4) return fail(ctx, CATEN_B200_EUNSUPPORTED, "embed: d %% 4 != 0");
  if ((ids_f32 == nullptr) == (ids_i64 == nullptr)) return fail(ctx, CATEN_B200_EINVAL, "embed: pass exactly one id array");
  launch_k(ctx, embed_kernel, dim3((unsigned)(B * s)), dim3(128), 0, ids_f32, ids_i64, wte, wpe, out, s, n, d_n, (int)(d / 4), V, T);
  CB_LAUNCH_CHECK(ctx, "embed_kernel");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// arg-max with the reference's tie rule: the lowest index among the maxima
// (source/api/high-level-ops.lisp:321-325).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ x, int64_t V, int64_t *__restrict__ out) {
  pdl_enter();
  const float *xr = x + (int64_t)blockIdx.x * V;
  float best = -INFINITY;
  int64_t bi = V;  // V = "nothing seen"
  for (int64_t v = threadIdx.x; v < V; v += blockDim.x) {
    const float f = xr[v];
    if (f > best || bi == V) {
      if (f > best || bi == V) { best = f; bi = v; }
    }
  }
  __shared__ float sv[256];
  __shared__ int64_t si[256];
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      const float ov = sv[threadIdx.x + o];
      const int64_t oi = si[threadIdx.x + o];
      const float mv = sv[threadIdx.x];
      const int64_t mi = si[threadIdx.x];
      if (oi < V && (mi == V || ov > mv || (ov == mv && oi < mi))) {
        sv[threadIdx.x] = ov;
        si[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[blockIdx.x] = si[0] == V ? 0 : si[0];
}

// End of a graph-replayed decode step: the new ids become the next step's input, are recorded in
// the per-position history, and the device-side position advances.
__global__ void finish_step_kernel(const int64_t *__restrict__ out_ids, int64_t *__restrict__ ids_io,
                                   int64_t *__restrict__ hist, int *__restrict__ d_pos, int B) {
  pdl_enter();
  const int pos = *d_pos;
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int64_t v = out_ids[b];
    ids_io[b] = v;
    hist[(int64_t)pos * B + b] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) *d_pos = pos + 1;
}

// Start of a run of graph-replayed steps: loads the input ids (int64, or float32 as the reference's
// caller passes them; an id that is not an integer selects no embedding row, kept as -1) and the
// start position into the device-side state.
__global__ void begin_steps_kernel(const float *__restrict__ ids_f32, const int64_t *__restrict__ ids_i64,
                                   int64_t *__restrict__ ids_io, int *__restrict__ d_pos, int n, int B) {
  pdl_enter();
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    if (ids_i64) {
      ids_io[b] = ids_i64[b];
    } else {
      const float t = ids_f32[b];
      ids_io[b] = (t >= 0.0f && t < 9.0e15f && truncf(t) == t) ? (int64_t)t : -1;
    }
  }
  if (threadIdx.x == 0) *d_pos = n;
}

int launch_begin_steps(caten_b200_ctx *ctx, const float *ids_f32, const int64_t *ids_i64, int64_t *ids_io, int *d_pos,
                       int64_t n, int64_t B) {
  launch_k(ctx, begin_steps_kernel, dim3(1), dim3(256), 0, ids_f32, ids_i64, ids_io, d_pos, (int)n, (int)B);
  CB_LAUNCH_CHECK(ctx, "begin_steps_kernel");
  return 0;
}

int launch_finish_step(caten_b200_ctx *ctx, const int64_t *out_ids, int64_t *ids_io, int64_t *hist, int *d_pos, int64_t B) {
  launch_k(ctx, finish_step_kernel, dim3(1), dim3(256), 0, out_ids, ids_io, hist, d_pos, (int)B);
  CB_LAUNCH_CHECK(ctx, "finish_step_kernel");
  return 0;
}

int launch_argmax(caten_b200_ctx *ctx, const float *x, int64_t rows, int64_t V, int64_t *out) {
  if (rows <= 0) return 0;
  if (V <= 0) return fail(ctx, CATEN_B200_EINVAL, "argmax: V <= 0");
  launch_k(ctx, argmax_kernel, dim3((unsigned)rows), dim3(256), 0, x, V, out);
  CB_LAUNCH_CHECK(ctx, "argmax_kernel");
  return 0;
}

}  // namespace cb
