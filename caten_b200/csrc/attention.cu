// Causal softmax attention over the fp32 KV cache, head dim 64 (every GPT-2 size,
// apps/gpt2/gpt2.lisp:38-41).  Cache layout [B, H, T, 64]: one head's history is one contiguous
// stream of 256-byte rows.
//
// Reference semantics (external/llm/layers.lisp:3-5,19-51): cache[:, n:n+s] = k, v;
// S = (q.K^T) * 0.125 + mask; P = softmax(S) with exp(x) = exp2(x * 1/ln2); O = P.V.
#include "common.cuh"

namespace cb {

constexpr float kInvLn2 = 1.0f / 0.6931472f;  // (/ (log 2)) in single float, api/function.lisp:437-440

// ---------------------------------------------------------------------------------------------
// Decode (s = 1): one CTA per (head, sequence).  HBM-bound: K and V rows of this head are each
// read once, 16 lanes x 16 bytes per row, 4 rows in flight per half-warp.  The CTA first stores
// this step's k and v rows at position n, so no separate append kernel runs in decode.
// Scores are kept in shared memory (t <= T floats) and the softmax is the reference's two-pass
// form (max, then exp and sum), not an online rescaling.
// ---------------------------------------------------------------------------------------------
#ifndef ATT_U
#define ATT_U 4  // rows in flight per half-warp
#endif
__global__ void __launch_bounds__(256, 6) attn_decode_kernel(const float *__restrict__ qkv, float *__restrict__ kc,
                                                          float *__restrict__ vc, float *__restrict__ out, int H,
                                                          int T, int n, const int *__restrict__ d_n,
                                                          __nv_bfloat16 *__restrict__ ohi, __nv_bfloat16 *__restrict__ olo,
                                                          const PartIn pin, long long prefetch_bytes) {
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  float *kb = kc + ((int64_t)b * H + h) * T * 64;
  float *vb = vc + ((int64_t)b * H + h) * T * 64;
  // Under programmatic dependent launch the first CTAs of this grid become resident while the kernels before it
  // (LayerNorm, the qkv linear) still run, and would idle in the wait below.  The history of this head, rows [0, n)
  // of K and V, was written by earlier steps and depends on nothing in flight, so those CTAs ask for it to be
  // brought into L2 meanwhile (HBM is nearly idle during the linears): one bulk L2 prefetch of up to 32 KB per
  // participating thread.  Only a hint: L2 is coherent, nothing reads through it, and a stale position only changes
  // how much is asked for.  Limited to the streams that together fit `prefetch_bytes` of the 126 MB L2 (measured:
  // 2-5 % of a step; asking for more than ~100 MB, or asking a layer ahead from the LayerNorm kernels, which
  // delays the linears' own weight loads behind the prefetch, made steps slower).
  {
    constexpr long long PIECE = 32 << 10;
    int np = d_n ? *d_n : n;
    np = np < 0 ? 0 : (np > T - 1 ? T - 1 : np);
    const long long stream_bytes = 256ll * np;
    const int pieces = (int)((stream_bytes + PIECE - 1) / PIECE);
    if (tid < 2 * pieces && ((long long)b * H + h + 1) * 2 * stream_bytes <= prefetch_bytes) {
      const int which = tid >= pieces ? 1 : 0, i = tid - which * pieces;
      const char *src = reinterpret_cast<const char *>(which ? vb : kb) + (long long)i * PIECE;
      const long long left = stream_bytes - (long long)i * PIECE;
      const unsigned bytes = (unsigned)(left < PIECE ? left : PIECE);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
    }
  }
  pdl_enter();
  if (d_n) n = *d_n;  // position kept on the device (decode replayed from a CUDA graph)
  extern __shared__ float smem[];
  float *q = smem;            // 64
  float *part = smem + 64;    // 16 x 64
  float *red = part + 1024;   // 32
  float *sc = red + 32;       // t
  const int d = H * 64, t = n + 1;
  const float *row = qkv + (int64_t)b * 3 * d;
  if (pin.splits > 0) {
    // the qkv linear left split-K partial tiles: sum this head's q, k, v entries here
    if (tid < 192) {
      const int which = tid >> 6, e = tid & 63;
      const float val = partin_load1(pin, b, which * d + h * 64 + e);
      if (which == 0) q[e] = val;
      else if (which == 1) kb[(int64_t)n * 64 + e] = val;
      else vb[(int64_t)n * 64 + e] = val;
    }
  } else if (tid < 64) {
    q[tid] = row[h * 64 + tid];
    kb[(int64_t)n * 64 + tid] = row[d + h * 64 + tid];
    vb[(int64_t)n * 64 + tid] = row[2 * d + h * 64 + tid];
  }
  __syncthreads();
  const int hw = tid >> 4, l16 = tid & 15;
  const float4 q4 = reinterpret_cast<const float4 *>(q)[l16];
  for (int j0 = 0; j0 < t; j0 += 16 * ATT_U) {
    float4 k4[ATT_U];
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      const int j = j0 + u * 16 + hw;
      k4[u] = j < t ? __ldcs(reinterpret_cast<const float4 *>(kb + (int64_t)j * 64) + l16) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      float p = fmaf(q4.x, k4[u].x, fmaf(q4.y, k4[u].y, fmaf(q4.z, k4[u].z, q4.w * k4[u].w)));
      p += __shfl_xor_sync(0xffffffffu, p, 8);
      p += __shfl_xor_sync(0xffffffffu, p, 4);
      p += __shfl_xor_sync(0xffffffffu, p, 2);
      p += __shfl_xor_sync(0xffffffffu, p, 1);
      const int j = j0 + u * 16 + hw;
      if (l16 == 0 && j < t) sc[j] = p * 0.125f;
    }
  }
  __syncthreads();
  // row max
  float m = -INFINITY;
  for (int j = tid; j < t; j += 256) m = fmaxf(m, sc[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  float ss = 0.0f;
  for (int j = tid; j < t; j += 256) {
    const float e = exp2f((sc[j] - m) * kInvLn2);
    sc[j] = e;
    ss += e;
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  ss = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) ss += red[w];
  const float inv = 1.0f / ss;
  // O = P.V
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < t; j0 += 16 * ATT_U) {
    float4 v4[ATT_U];
    float p[ATT_U];
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      const int j = j0 + u * 16 + hw;
      const bool ok = j < t;
      v4[u] = ok ? __ldcs(reinterpret_cast<const float4 *>(vb + (int64_t)j * 64) + l16) : make_float4(0.f, 0.f, 0.f, 0.f);
      p[u] = ok ? sc[j] * inv : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      acc.x = fmaf(p[u], v4[u].x, acc.x);
      acc.y = fmaf(p[u], v4[u].y, acc.y);
      acc.z = fmaf(p[u], v4[u].z, acc.z);
      acc.w = fmaf(p[u], v4[u].w, acc.w);
    }
  }
  reinterpret_cast<float4 *>(part + hw * 64)[l16] = acc;
  __syncthreads();
  if (tid < 64) {
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < 16; ++w) o += part[w * 64 + tid];
    const int64_t at = (int64_t)b * d + h * 64 + tid;
    if (ohi) {  // split bf16 operand of the projection GEMM
      const __nv_bfloat16 hh = __float2bfloat16_rn(o);
      ohi[at] = hh;
      if (olo) olo[at] = __float2bfloat16_rn(o - __bfloat162float(hh));
    } else {
      out[at] = o;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill (s > 1): append kernel + tiled causal attention with running max / sum.
// ---------------------------------------------------------------------------------------------
__global__ void kv_append_kernel(const float *__restrict__ qkv, float *__restrict__ kc, float *__restrict__ vc,
                                 int s, int n, int H, int T) {
  pdl_enter();
  const int64_t r = blockIdx.x;  // row of qkv = b*s + i
  const int64_t b = r / s;
  const int i = (int)(r % s);
  const int d4 = H * 16;
  const float4 *row = reinterpret_cast<const float4 *>(qkv) + r * 3 * d4;
  for (int c = threadIdx.x; c < d4; c += blockDim.x) {
    const int h = c >> 4, l = c & 15;
    const int64_t dst = (((b * H + h) * T) + n + i) * 16 + l;
    reinterpret_cast<float4 *>(kc)[dst] = row[d4 + c];
    reinterpret_cast<float4 *>(vc)[dst] = row[2 * d4 + c];
  }
}

constexpr int PF_LD = 68;  // padded leading dimension of the 64x64 tiles (floats)

// One CTA = 64 queries of one (sequence, head); 256 threads as a 16x16 grid, each owning a 4x4
// block of the 64x64 score tile and of the 64x64 output tile.  Q and K tiles are stored
// transposed ([c][row]) so the inner products read float4s without bank conflicts.
__global__ void __launch_bounds__(256) attn_prefill_kernel(const float *__restrict__ qkv, const float *__restrict__ kc,
                                                           const float *__restrict__ vc, float *__restrict__ out,
                                                           int s, int n, int H, int T, __nv_bfloat16 *__restrict__ ohi,
                                                           __nv_bfloat16 *__restrict__ olo) {
  extern __shared__ float smem[];
  pdl_enter();
  float *Qt = smem;                 // [64 c][PF_LD i]
  float *Kt = Qt + 64 * PF_LD;      // [64 c][PF_LD j]
  float *Vs = Kt + 64 * PF_LD;      // [64 j][PF_LD c]
  float *Pt = Vs + 64 * PF_LD;      // [64 j][PF_LD i]
  const int q0 = blockIdx.x * 64, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  const int d = H * 64, t = n + s;
  const int tx = tid & 15, ty = tid >> 4;
  const int lane = tid & 31, warp = tid >> 5;
  const float *kb = kc + ((int64_t)b * H + h) * T * 64;
  const float *vb = vc + ((int64_t)b * H + h) * T * 64;
  // Q tile, transposed; lane <-> query row, so the shared-memory stores are conflict-free
  for (int it = 0; it < 2; ++it) {
    const int i = lane + 32 * it;
    const bool ok = q0 + i < s;
    const float4 *src = reinterpret_cast<const float4 *>(qkv + ((int64_t)b * s + q0 + i) * 3 * d + h * 64);
    for (int c4 = warp; c4 < 16; c4 += 8) {
      const float4 v = ok ? src[c4] : make_float4(0.f, 0.f, 0.f, 0.f);
      Qt[(4 * c4 + 0) * PF_LD + i] = v.x;
      Qt[(4 * c4 + 1) * PF_LD + i] = v.y;
      Qt[(4 * c4 + 2) * PF_LD + i] = v.z;
      Qt[(4 * c4 + 3) * PF_LD + i] = v.w;
    }
  }
  float m_run[4], l_run[4], o[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    m_run[a] = -INFINITY;
    l_run[a] = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) o[a][c] = 0.0f;
  }
  const int kend = min(t, n + q0 + 64);  // keys beyond the last query of this tile are masked
  for (int j0 = 0; j0 < kend; j0 += 64) {
    __syncthreads();  // previous tile fully consumed (also orders the Q stores before first use)
    for (int it = 0; it < 2; ++it) {
      const int j = lane + 32 * it;
      const bool ok = j0 + j < t;
      const float4 *src = reinterpret_cast<const float4 *>(kb + (int64_t)(j0 + j) * 64);
      for (int c4 = warp; c4 < 16; c4 += 8) {
        const float4 v = ok ? src[c4] : make_float4(0.f, 0.f, 0.f, 0.f);
        Kt[(4 * c4 + 0) * PF_LD + j] = v.x;
        Kt[(4 * c4 + 1) * PF_LD + j] = v.y;
        Kt[(4 * c4 + 2) * PF_LD + j] = v.z;
        Kt[(4 * c4 + 3) * PF_LD + j] = v.w;
      }
    }
    for (int e = tid; e < 64 * 16; e += 256) {
      const int j = e >> 4, c4 = e & 15;
      const float4 v = j0 + j < t ? reinterpret_cast<const float4 *>(vb + (int64_t)(j0 + j) * 64)[c4]
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4 *>(Vs + j * PF_LD + 4 * c4) = v;
    }
    __syncthreads();
    float sacc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) sacc[a][c] = 0.0f;
#pragma unroll 8
    for (int c = 0; c < 64; ++c) {
      const float4 qv = *reinterpret_cast<const float4 *>(Qt + c * PF_LD + 4 * ty);
      const float4 kv = *reinterpret_cast<const float4 *>(Kt + c * PF_LD + 4 * tx);
      const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[a][e] = fmaf(qa[a], ka[e], sacc[a][e]);
    }
    // scale, mask, running softmax (rows = 4*ty + a, shared by the 16 lanes with equal ty)
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int qi = q0 + 4 * ty + a;  // query index within this step
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + 4 * tx + e;
        float v = sacc[a][e] * 0.125f;
        if (j >= qi + n + 1 || j >= t) v = -INFINITY;
        sacc[a][e] = v;
        mx = fmaxf(mx, v);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      const float m_new = fmaxf(m_run[a], mx);
      // a row past the end of the sequence, or one whose keys in this tile are all masked while
      // nothing has been seen yet, keeps m_new = -inf: guard the subtraction
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = exp2f((m_run[a] - m_use) * kInvLn2);
      float rs = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f((sacc[a][e] - m_use) * kInvLn2);
        sacc[a][e] = p;
        rs += p;
      }
      rs += __shfl_xor_sync(0xffffffffu, rs, 8);
      rs += __shfl_xor_sync(0xffffffffu, rs, 4);
      rs += __shfl_xor_sync(0xffffffffu, rs, 2);
      rs += __shfl_xor_sync(0xffffffffu, rs, 1);
      l_run[a] = l_run[a] * corr + rs;
      m_run[a] = m_new;
#pragma unroll
      for (int c = 0; c < 4; ++c) o[a][c] *= corr;
    }
    // P tile, transposed: Pt[j][i]
#pragma unroll
    for (int e = 0; e < 4; ++e)
      *reinterpret_cast<float4 *>(Pt + (4 * tx + e) * PF_LD + 4 * ty) =
          make_float4(sacc[0][e], sacc[1][e], sacc[2][e], sacc[3][e]);
    __syncthreads();
#pragma unroll 8
    for (int j = 0; j < 64; ++j) {
      const float4 pv = *reinterpret_cast<const float4 *>(Pt + j * PF_LD + 4 * ty);
      const float4 vv = *reinterpret_cast<const float4 *>(Vs + j * PF_LD + 4 * tx);
      const float pa[4] = {pv.x, pv.y, pv.z, pv.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[a][c] = fmaf(pa[a], va[c], o[a][c]);
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int qi = q0 + 4 * ty + a;
    if (qi < s) {
      const float inv = 1.0f / l_run[a];
      float4 r = make_float4(o[a][0] * inv, o[a][1] * inv, o[a][2] * inv, o[a][3] * inv);
      const int64_t at = ((int64_t)b * s + qi) * d + h * 64 + 4 * tx;
      if (ohi) {
        *reinterpret_cast<uint2 *>(ohi + at) = make_uint2(pack_bf16(r.x, r.y), pack_bf16(r.z, r.w));
        if (olo)
          *reinterpret_cast<uint2 *>(olo + at) = make_uint2(pack_bf16(bf16_lo(r.x), bf16_lo(r.y)), pack_bf16(bf16_lo(r.z), bf16_lo(r.w)));
      } else {
        *reinterpret_cast<float4 *>(out + at) = r;
      }
    }
  }
}

int launch_attention(caten_b200_ctx *ctx, const float *qkv, float *kc, float *vc, float *out, int64_t B, int64_t s,
                     int64_t n, int64_t H, int64_t T, const int *d_n, BfOut bf, const PartIn *pending_qkv, int tensor_cores) {
  if (B <= 0 || s <= 0) return 0;
  if (pending_qkv && pending_qkv->splits > 0 && s != 1) return fail(ctx, CATEN_B200_EINVAL, "attention: a pending qkv is only supported for single-token steps");
  if (n < 0 || n + s > T) return fail(ctx, CATEN_B200_EINVAL, "attention: positions [%lld,%lld) outside the cache (T=%lld)", (long long)n, (long long)(n + s), (long long)T);
  if (H > 65535 || B > 65535) return fail(ctx, CATEN_B200_EUNSUPPORTED, "attention: B or H > 65535");
  if (s == 1) {
    // with a device-side position the launch is sized for the longest context the cache allows
    const size_t smem = (64 + 1024 + 32 + (size_t)(d_n ? T : n + 1)) * sizeof(float);
    if (smem > 200 * 1024) return fail(ctx, CATEN_B200_EUNSUPPORTED, "attention: context too long for the decode kernel");
    if (smem > 48 * 1024)
      CB_CUDA(ctx, cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    launch_k(ctx, attn_decode_kernel, dim3((unsigned)H, (unsigned)B), dim3(256), smem, qkv, kc, vc, out, (int)H, (int)T, (int)n, d_n, bf.hi, bf.lo,
             pending_qkv ? *pending_qkv : PartIn(), ctx->attn_prefetch_bytes);
    CB_LAUNCH_CHECK(ctx, "attn_decode_kernel");
    return 0;
  }
  if (d_n) return fail(ctx, CATEN_B200_EINVAL, "attention: a device-side position is only supported for single-token steps");
  launch_k(ctx, kv_append_kernel, dim3((unsigned)(B * s)), dim3(128), 0, qkv, kc, vc, (int)s, (int)n, (int)H, (int)T);
  CB_LAUNCH_CHECK(ctx, "kv_append_kernel");
  if (tensor_cores) return launch_attention_tc(ctx, qkv, kc, vc, out, B, s, n, H, T, bf);
  const size_t smem = 4 * 64 * PF_LD * sizeof(float);
  CB_CUDA(ctx, cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  launch_k(ctx, attn_prefill_kernel, dim3((unsigned)((s + 63) / 64), (unsigned)H, (unsigned)B), dim3(256), smem, 
      qkv, kc, vc, out, (int)s, (int)n, (int)H, (int)T, bf.hi, bf.lo);
  CB_LAUNCH_CHECK(ctx, "attn_prefill_kernel");
  return 0;
}

}  // namespace cb
