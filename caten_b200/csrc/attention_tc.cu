// Prefill attention (s > 1) on the 5th-generation tensor cores, head dim 64, fp32 KV cache
// [B, H, T, 64].  Same semantics as the SIMT kernels in attention.cu
// (external/llm/layers.lisp:3-5,19-51: S = (q.K^T) * 0.125 + causal mask; P = softmax(S) with
// exp(x) = exp2(x * 1/ln2), two passes: row maximum first, then exp and sum; O = P.V), with both
// contractions as bf16 hi/lo split products accumulated in fp32 (every operand x = x_hi + x_lo;
// q.K^T keeps all four products, P.V drops only lo*lo), so the result stays within about 2^-16
// of the fp32 one.
//
// One CTA = 128 queries of one (sequence, head) = the 128 lanes of tensor memory; keys go in
// steps of 64.  A CTA uses 256 of the 512 TMEM columns and under half of the shared memory, so
// two CTAs share an SM and one's MMAs overlap the other's softmax.  Per step:
//   all 8 warps  copy the NEXT step's K (and V) rows from the cache into a staging buffer in shared
//                memory (cp.async, 16 bytes per thread, coalesced; in flight during this step's
//                MMAs and softmax), and split the current step's staged rows into bf16 hi/lo,
//                stored as 128-byte-swizzled K-major tiles in shared memory:
//                K tiles  = 64 keys x 64 dims, hi and lo             (K-major B operands of S = Q.K^T)
//                V tiles  = 64 keys x 64 dims, hi and lo             (MN-major B operands of O += P.V)
//   one thread   issues S[128 x 64] = (Q_hi + Q_lo) . (K_hi + K_lo)^T as four MMAs per 16 dims into
//                the same 64 columns (Q tile in shared memory)
//   all 8 warps  read their query's scores from tensor memory (warps w and w+4 share lanes and
//                take 32 keys each), mask, and
//                p = exp2((s - max)/ln2), accumulate the row sum, split p into bf16 hi/lo and
//                write it back to tensor memory as the A operand of the second product
//   one thread   issues O[128 x 64] += P_hi.V_hi + P_lo.V_hi + P_hi.V_lo, accumulating over the
//                key steps in tensor memory
// The softmax is single-pass with a lazily moved reference maximum: each step exchanges the
// maximum of its visible scores between the row's two threads; the reference only moves (and O and
// the row sum are rescaled, O by a TMEM load / multiply / store) when a step exceeds it by more
// than AT_TAU, which in causal attention happens in the first steps and then rarely.  Softmax is
// invariant to the reference, so this equals the reference's two-pass form up to rounding.  The
// phases of a step are sequential within the CTA (block-wide barriers + one mbarrier the MMAs
// commit to).
// TMEM columns: [0,64) S, [128,192) P (hi 32, lo 32), [192,256) O.
//
// The mbarrier waits are bounded; when one runs out the CTA records it in the context's status
// word, skips the remaining work and its output, frees its tensor memory and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace cb {

namespace {

constexpr float kAtInvLn2 = 1.0f / 0.6931472f;  // (/ (log 2)) in single float, api/function.lisp:437-440
constexpr int AT_Q = 128;                        // queries per CTA (MMA M)
constexpr int AT_K = 64;                         // keys per step
constexpr float AT_TAU = 8.0f;                   // slack of the running maximum, in units of the score
constexpr uint32_t AT_COLS = 256;                // TMEM columns per CTA
constexpr uint32_t AT_COL_S = 0, AT_COL_P = 128, AT_COL_O = 192;
constexpr uint32_t AT_OFF_Q = 0, AT_OFF_K = 32768, AT_OFF_V = 49152;
// staging of the raw fp32 rows: 256 bytes per row padded to 272, so that threads reading one row
// each (16 bytes at a time) spread over all banks
constexpr uint32_t AT_STAGE_LD = 272;
constexpr uint32_t AT_OFF_SK = 65536, AT_OFF_SV = AT_OFF_SK + AT_K * AT_STAGE_LD, AT_OFF_MISC = AT_OFF_SV + AT_K * AT_STAGE_LD;
// tiles + staging + exchange buffer + barrier / TMEM slot / abort flag + alignment slack; two CTAs fit one SM
constexpr size_t AT_SMEM = AT_OFF_MISC + 1024 + 64 + 1024;
static_assert(2 * (AT_SMEM + 1024) <= 227 * 1024, "two CTAs per SM");

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {  // src_bytes 0: zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a K-major tile with 128-byte rows
// and the 128-byte swizzle (8-row groups of 1024 bytes)
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint4 pack8(const float4 a, const float4 b) {
  return make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
}
__device__ __forceinline__ uint4 pack8_lo(const float4 a, const float4 b) {
  return make_uint4(pack_bf16(bf16_lo(a.x), bf16_lo(a.y)), pack_bf16(bf16_lo(a.z), bf16_lo(a.w)),
                    pack_bf16(bf16_lo(b.x), bf16_lo(b.y)), pack_bf16(bf16_lo(b.z), bf16_lo(b.w)));
}
// 8 consecutive fp32 of one row -> one chunk of the hi row and one of the lo row
__device__ __forceinline__ void st_split8(unsigned char *tile, int row_hi, int row_lo, int chunk, const float4 a, const float4 b) {
  *reinterpret_cast<uint4 *>(tile + sw128(row_hi, chunk)) = pack8(a, b);
  *reinterpret_cast<uint4 *>(tile + sw128(row_lo, chunk)) = pack8_lo(a, b);
}

// 2^x by the special-function unit alone (what exp2f uses inside, without its scaling of results
// below 2^-126, which flush to zero here: such probabilities do not register in a row sum >= 1/e^8)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float4 scale4(float4 v, float c) { return make_float4(v.x * c, v.y * c, v.z * c, v.w * c); }

}  // namespace

__global__ void __launch_bounds__(256, 2) attn_prefill_tc_kernel(const float *__restrict__ qkv, const float *__restrict__ kc,
                                                                  const float *__restrict__ vc, float *__restrict__ out,
                                                                  int s, int n, int H, int T, __nv_bfloat16 *__restrict__ ohi,
                                                                  __nv_bfloat16 *__restrict__ olo, int *status,
                                                                  uint32_t idesc_n64) {
  extern __shared__ unsigned char at_raw[];
  unsigned char *sm = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(at_raw) + 1023) & ~(uintptr_t)1023);
  float *red = reinterpret_cast<float *>(sm + AT_OFF_MISC);
  const uint32_t bar = smem_u32(sm + AT_OFF_MISC + 1024);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + AT_OFF_MISC + 1024 + 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + AT_OFF_MISC + 1024 + 12);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3;  // 32-lane quadrant of tensor memory this warp may access
  const int hf = warp >> 2;   // which half (of a step's keys / of the head dims) this thread takes
  const int r = quad * 32 + lane;  // query row within the tile = TMEM lane
  const int ck = tid & 63, cq = tid >> 6;  // conversion: key row of the step, and which 16 of its 64 dims
  const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * AT_Q;  // tiles with the longest history first
  const int h = blockIdx.y, b = blockIdx.z;
  const int d = H * 64, t = n + s;

  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(AT_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  pdl_enter();

  const float *kb = kc + ((int64_t)b * H + h) * T * 64;
  const float *vb = vc + ((int64_t)b * H + h) * T * 64;
  const int kend = min(t, n + q0 + AT_Q);  // keys beyond the last query of this tile are masked
  const int nblk = (kend + AT_K - 1) / AT_K;
  const int qi = min(q0 + r, s - 1);  // rows past the end of the step mask like the last row (their output is dropped)
  const int jmax = n + qi;            // last visible key of this query (< t)

  const uint64_t dq_hi = umma_desc(smem_u32(sm + AT_OFF_Q)), dq_lo = umma_desc(smem_u32(sm + AT_OFF_Q + 16384));
  const uint64_t dk = umma_desc(smem_u32(sm + AT_OFF_K)), dk_lo = umma_desc(smem_u32(sm + AT_OFF_K + 8192));
  const uint64_t dv_hi = umma_desc(smem_u32(sm + AT_OFF_V)), dv_lo = umma_desc(smem_u32(sm + AT_OFF_V + 8192));
  const uint32_t idesc_pv = idesc_n64 | (1u << 16);  // B operand MN-major: V rows (keys) with the dims contiguous
  uint32_t ph = 0;
  int ok = 1;

  // copy the 64 rows [j0, j0+64) of one head's K or V history into a staging buffer; rows past
  // the end of the context are zero-filled
  auto prefetch = [&](const float *base, int j0, uint32_t stage_off) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int piece = tid + 256 * i, row = piece >> 4, c16 = piece & 15;
      const bool okk = j0 + row < t;
      cp_async16(smem_u32(sm + stage_off + row * AT_STAGE_LD + c16 * 16), base + (int64_t)(okk ? j0 + row : 0) * 64 + c16 * 4, okk ? 16u : 0u);
    }
  };
  auto staged_row = [&](uint32_t stage_off, float4 *v) {  // this thread's 16 dims of its key row
    const float4 *src = reinterpret_cast<const float4 *>(sm + stage_off + ck * AT_STAGE_LD + 64 * cq);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = src[i];
  };
  // one warp polls the mbarrier; the others park at the block barrier instead of spinning (their
  // issue slots go to the other CTA of the SM)
  auto wait_mma = [&]() {
    if (warp == 0 && !mbar_wait(bar, ph, abort_flag)) {
      ok = 0;
      *abort_flag = 1;
    }
    ph ^= 1u;
    ok = __syncthreads_and(ok);
  };

  prefetch(kb, 0, AT_OFF_SK);
  prefetch(vb, 0, AT_OFF_SV);
  cp_async_commit();
  // Q tile: rows [0,128) hi, [128,256) lo; the 1/8 score scale is folded in (a power of two: exact)
  {
    const bool okq = q0 + r < s;
    const float4 *src = reinterpret_cast<const float4 *>(qkv + ((int64_t)b * s + (okq ? q0 + r : 0)) * 3 * d + h * 64 + 32 * hf);
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = okq ? scale4(src[i], 0.125f) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) st_split8(sm + AT_OFF_Q, r, 128 + r, 4 * hf + c, v[2 * c], v[2 * c + 1]);
  }
  cp_async_wait_all();
  __syncthreads();  // step 0 of K and V is staged (and the Q tile is written)

  // ---- key steps: scores, running maximum, probabilities, row sums, O ---------------------------------
  float m = -INFINITY;  // the row's reference maximum: the same value in both threads of a row
  float lsum = 0.0f;    // this thread's part of the row sum, relative to m
  for (int blk = 0; blk < nblk && ok; ++blk) {
    const int j0 = blk * AT_K;
    {
      // split this thread's part of the staged rows in registers, then (once the previous step's
      // P.V has read the V^T tile and P) store it into the tiles
      float4 kv[4], vv[4];
      staged_row(AT_OFF_SK, kv);
      staged_row(AT_OFF_SV, vv);
      uint4 khi[2], klo[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        khi[c] = pack8(kv[2 * c], kv[2 * c + 1]);
        klo[c] = pack8_lo(kv[2 * c], kv[2 * c + 1]);
      }
      uint4 vhi[2], vlo[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        vhi[c] = pack8(vv[2 * c], vv[2 * c + 1]);
        vlo[c] = pack8_lo(vv[2 * c], vv[2 * c + 1]);
      }
      if (blk > 0) wait_mma();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        *reinterpret_cast<uint4 *>(sm + AT_OFF_K + sw128(ck, 2 * cq + c)) = khi[c];
        *reinterpret_cast<uint4 *>(sm + AT_OFF_K + sw128(64 + ck, 2 * cq + c)) = klo[c];
      }
      // V tiles (hi, then lo): rows = keys, the 64 dims contiguous: the MMA reads them as an MN-major B operand
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        *reinterpret_cast<uint4 *>(sm + AT_OFF_V + sw128(ck, 2 * cq + c)) = vhi[c];
        *reinterpret_cast<uint4 *>(sm + AT_OFF_V + 8192 + sw128(ck, 2 * cq + c)) = vlo[c];
      }
    }
    fence_proxy_async();
    tc_fence_before();
    ok = __syncthreads_and(ok);  // tiles complete, staging buffers free
    if (!ok) break;
    if (warp == 0) {  // converged warp, one elected lane: the descriptors stay in uniform registers
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint64_t adv = (uint64_t)(2 * k4);  // 16 bf16 = 32 bytes = 2 descriptor units
          umma_bf16(tmem_base + AT_COL_S, dq_hi + adv, dk + adv, idesc_n64, k4 > 0 ? 1u : 0u);
          umma_bf16(tmem_base + AT_COL_S, dq_lo + adv, dk + adv, idesc_n64, 1u);
          umma_bf16(tmem_base + AT_COL_S, dq_hi + adv, dk_lo + adv, idesc_n64, 1u);
          umma_bf16(tmem_base + AT_COL_S, dq_lo + adv, dk_lo + adv, idesc_n64, 1u);
        }
        umma_commit(bar);
      }
      __syncwarp();
    }
    // the next step's rows start to arrive while the MMAs run (issued after them: the MMAs are the critical path)
    if (blk + 1 < nblk) {
      prefetch(kb, j0 + AT_K, AT_OFF_SK);
      prefetch(vb, j0 + AT_K, AT_OFF_SV);
      cp_async_commit();
    }
    wait_mma();
    tc_fence_after();
    {
      // this thread's 32 keys in one round trip to tensor memory
      uint32_t a[32];
      tmem_ld16(tlane + AT_COL_S + 32 * hf, a);
      tmem_ld16(tlane + AT_COL_S + 32 * hf + 16, a + 16);
      tmem_ld_wait();
      // maximum of the visible scores of this step: over this thread's 32 keys, then over the row's two threads
      const int lim = jmax - j0 - 32 * hf;  // key e of this thread is visible iff e <= lim
      float mloc = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (e <= lim) mloc = fmaxf(mloc, __uint_as_float(a[e]));
      red[hf * 128 + r] = mloc;
      __syncthreads();
      const float mstep = fmaxf(red[r], red[128 + r]);
      // The reference maximum only moves when the step's maximum exceeds it by more than AT_TAU
      // (probabilities then stay below e^AT_TAU, harmless in fp32 / split bf16); when it moves, O and
      // the row sum accumulated so far are rescaled.  Softmax is invariant to the shift, so this is
      // the two-pass result up to rounding.  Step 0 always sees key 0, so m is finite from then on.
      const bool move = mstep > m + AT_TAU;  // also true at step 0 (m = -inf)
      const float m_new = move ? mstep : m;
      if (blk > 0 && __any_sync(0xffffffffu, move)) {
        const float scale = move ? exp2f((m - m_new) * kAtInvLn2) : 1.0f;
        lsum *= scale;
        uint32_t o[32];
        tmem_ld16(tlane + AT_COL_O + 32 * hf, o);
        tmem_ld16(tlane + AT_COL_O + 32 * hf + 16, o + 16);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * scale);
        tmem_st16(tlane + AT_COL_O + 32 * hf, o);
        tmem_st16(tlane + AT_COL_O + 32 * hf + 16, o + 16);
      }
      m = m_new;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float p[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float val = __uint_as_float(a[16 * c + e]);
          p[e] = (16 * c + e <= lim) ? ex2_approx((val - m) * kAtInvLn2) : 0.0f;
          lsum += p[e];
        }
        uint32_t phi[8], plo[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          phi[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
          plo[e] = pack_bf16(bf16_lo(p[2 * e]), bf16_lo(p[2 * e + 1]));
        }
        // 16 keys = 8 columns; key k of the step sits in column k / 2
        tmem_st8(tlane + AT_COL_P + 16 * hf + 8 * c, phi);
        tmem_st8(tlane + AT_COL_P + 32 + 16 * hf + 8 * c, plo);
      }
    }
    tmem_st_wait();
    tc_fence_before();
    cp_async_wait_all();
    ok = __syncthreads_and(ok);  // P is written; the next step's rows are staged
    if (!ok) break;
    if (warp == 0) {  // converged warp, one elected lane: the descriptors stay in uniform registers
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint64_t adv = (uint64_t)(128 * k4);  // 16 keys = 16 rows of 128 bytes = 128 descriptor units
          const uint32_t p_hi = tmem_base + AT_COL_P + 8 * k4, p_lo = p_hi + 32;
          umma_bf16_ts(tmem_base + AT_COL_O, p_hi, dv_hi + adv, idesc_pv, (blk > 0 || k4 > 0) ? 1u : 0u);
          umma_bf16_ts(tmem_base + AT_COL_O, p_lo, dv_hi + adv, idesc_pv, 1u);
          umma_bf16_ts(tmem_base + AT_COL_O, p_hi, dv_lo + adv, idesc_pv, 1u);
        }
        umma_commit(bar);
      }
      __syncwarp();
    }
  }
  if (ok && nblk > 0) wait_mma();
  tc_fence_after();
  red[hf * 128 + r] = lsum;
  ok = __syncthreads_and(ok);
  if (ok) {
    const float inv = 1.0f / (red[r] + red[128 + r]);
    uint32_t a[32];
    tmem_ld16(tlane + AT_COL_O + 32 * hf, a);
    tmem_ld16(tlane + AT_COL_O + 32 * hf + 16, a + 16);
    tmem_ld_wait();
    float o[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) o[e] = __uint_as_float(a[e]) * inv;
    if (q0 + r < s) {
      const int64_t at = ((int64_t)b * s + q0 + r) * d + h * 64 + 32 * hf;
      if (ohi) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float *p = o + 8 * i;
          *reinterpret_cast<uint4 *>(ohi + at + 8 * i) =
              make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
          if (olo)
            *reinterpret_cast<uint4 *>(olo + at + 8 * i) =
                make_uint4(pack_bf16(bf16_lo(p[0]), bf16_lo(p[1])), pack_bf16(bf16_lo(p[2]), bf16_lo(p[3])),
                           pack_bf16(bf16_lo(p[4]), bf16_lo(p[5])), pack_bf16(bf16_lo(p[6]), bf16_lo(p[7])));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<float4 *>(out + at + 4 * i) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    }
  } else if (tid == 0) {
    atomicCAS(status, 0, DEV_WAIT_TIMEOUT);
    status[1] = 10;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(AT_COLS) : "memory");
  }
}

int launch_attention_tc(caten_b200_ctx *ctx, const float *qkv, const float *kc, const float *vc, float *out, int64_t B, int64_t s,
                        int64_t n, int64_t H, int64_t T, BfOut bf) {
  const uint32_t base = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_Q >> 4) << 24);  // fp32 accumulate, bf16 x bf16, M = 128
  const uint32_t idesc_n64 = base | ((uint32_t)(64 >> 3) << 17);
  CB_CUDA(ctx, cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM));
  launch_k(ctx, attn_prefill_tc_kernel, dim3((unsigned)((s + AT_Q - 1) / AT_Q), (unsigned)H, (unsigned)B), dim3(256), AT_SMEM, qkv, kc, vc,
           out, (int)s, (int)n, (int)H, (int)T, bf.hi, bf.lo, ctx->d_status, idesc_n64);
  CB_LAUNCH_CHECK(ctx, "attn_prefill_tc_kernel");
  return 0;
}

}  // namespace cb
