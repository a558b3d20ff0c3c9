// Tensor-core GEMM for many activation rows (prefill, relu(matmul)):
//   y[m, o] = act(sum_k x[m,k] * W[o,k] + bias[o]) + res[m, o]          (source/nn/linear.lisp:12-17)
// With thousands of rows a weight tile is reused by many activation tiles, so the weights are
// expanded ONCE per call into a bf16 (hi[, lo]) copy in device memory and both operands of the MMA
// then come from shared memory through TMA; nothing is converted inside the GEMM loop.  The kernel
// is persistent (one CTA per SM walks over output tiles) and specialised by warp:
//   warp 0      one lane issues the TMA loads of the W and x tiles into a ring of stages
//   warp 1      issues tcgen05.mma (A = W tile, B = x tile, both K-major with 128-byte swizzle)
//               into one of TWO accumulators in tensor memory (2 x 256 columns)
//   warps 2..9  epilogue: read the other accumulator with tcgen05.ld, add bias, apply the
//               activation and the residual, store — while the next tile's MMAs run
// Tile = 128 output features (TMEM lanes) x 256 rows (TMEM columns); a stage holds 64 k (bf16) or 32 k (split bf16).
// Split-bf16 (NSPLIT = 3) issues W_hi.x_hi + W_lo.x_hi + W_hi.x_lo per k-step, as the decode GEMM.
// Every mbarrier wait is bounded: when one runs out the role records it in the status word,
// every role leaves its loop, copies in flight are awaited, tensor memory is freed.
#include "blocks32.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

namespace cb {

constexpr int GD_BM = 128;   // output features per tile (MMA M, TMEM lanes)
constexpr int GD_BN = 256;   // activation rows per tile (MMA N, TMEM columns)
constexpr int GD_BK = 64;    // k granularity of the operands (K % 64 == 0)
// k per stage: 64 (128-byte rows, 128-byte swizzle) in bf16; 32 (64-byte rows, 64-byte swizzle) in split bf16, where a
// 64-k stage of hi and lo tiles is 96 KB and only two would fit: four 48 KB stages keep three loads in flight
template <int NSPLIT> struct GdStage { static constexpr int BK = NSPLIT == 3 ? 32 : 64; };
constexpr int GD_EPI_WARPS = 8;
constexpr int GD_THREADS = (2 + GD_EPI_WARPS) * 32;

struct GdArgs {
  const float *bias, *res;
  float *y;
  __nv_bfloat16 *yhi, *ylo;   // when yhi is set the result is written as split bf16 instead of y
  int *status;
  int act, M, N, K;
  int tiles_f, tiles;         // feature tiles per row tile; all tiles
  int stages;
  uint32_t idesc;
};

// ---- pre-pass: operands -> bf16 hi (and lo), K-major --------------------------------------------

__device__ __forceinline__ void store_split8(const float *w, __nv_bfloat16 *hi, __nv_bfloat16 *lo, int64_t at) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(w[2 * e]), h1 = __float2bfloat16_rn(w[2 * e + 1]);
    h[e] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(w[2 * e] - __bfloat162float(h0));
    const __nv_bfloat16 l1 = __float2bfloat16_rn(w[2 * e + 1] - __bfloat162float(h1));
    l[e] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
  }
  *reinterpret_cast<uint4 *>(hi + at) = make_uint4(h[0], h[1], h[2], h[3]);
  if (lo) *reinterpret_cast<uint4 *>(lo + at) = make_uint4(l[0], l[1], l[2], l[3]);
}

// one thread = 8 consecutive weights of a row (a quarter of a 32-wide block)
template <int WT>
__global__ void __launch_bounds__(256) wsplit_kernel(const void *__restrict__ qs, const __half *__restrict__ d,
                                                     const __half *__restrict__ mins, const uint32_t *__restrict__ qh5, int64_t N,
                                                     int64_t K, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo) {
  pdl_enter();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t per_row = K / 8;
  if (idx >= N * per_row) return;
  const int64_t row = idx / per_row;
  const int o8 = (int)(idx - row * per_row);
  float w[8];
  load_w8<WT>(qs, d, mins, qh5, row, N, K, K / 32, o8 >> 2, o8 & 3, w);
  store_split8(w, hi, lo, row * K + (int64_t)o8 * 8);
}

// b[K, N] fp32 -> hi / lo [N, K] bf16 (transposed through a shared-memory tile)
__global__ void __launch_bounds__(256) bt_split_kernel(const float *__restrict__ b, int64_t K, int64_t N, __nv_bfloat16 *__restrict__ hi,
                                                       __nv_bfloat16 *__restrict__ lo) {
  __shared__ float tile[32][33];
  pdl_enter();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t k0 = (int64_t)blockIdx.y * 32, n0 = (int64_t)blockIdx.x * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t k = k0 + ty + 8 * i, n = n0 + tx;
    tile[ty + 8 * i][tx] = (k < K && n < N) ? b[k * N + n] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t n = n0 + ty + 8 * i, k = k0 + tx;
    if (n < N && k < K) {
      const float v = tile[tx][ty + 8 * i];
      const __nv_bfloat16 h = __float2bfloat16_rn(v);
      hi[n * K + k] = h;
      if (lo) lo[n * K + k] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
  }
}

// x fp32 [M, K] -> bf16 hi (and lo)
__global__ void __launch_bounds__(256) xsplit_kernel(const float *__restrict__ x, int64_t n8, __nv_bfloat16 *__restrict__ hi,
                                                     __nv_bfloat16 *__restrict__ lo) {
  pdl_enter();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4 *>(x)[2 * i], c = reinterpret_cast<const float4 *>(x)[2 * i + 1];
  const float w[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
  store_split8(w, hi, lo, i * 8);
}

// ---- the GEMM -----------------------------------------------------------------------------------

// Epilogue of one 16-row x 32-feature block of a warp.  A thread reads its feature's 16 accumulators (one per
// row) from tensor memory; stored directly that would be 4-byte stores 128 bytes apart per warp instruction,
// which the store path sustains at a fraction of what the MMAs produce.  So the block goes through a 2 KB
// shared-memory tile of the warp and comes back transposed: a lane then owns four consecutive features of
// four rows and moves 16 bytes per instruction (bias, activation, residual and the optional split-bf16
// output are applied on that side).
template <int ACT>
__device__ __forceinline__ void gd_store_block(const GdArgs &a, const float *stg, int lane, float4 bias4, int64_t o0, bool o_ok, int m_first) {
  const int fg = lane & 7, tr = lane >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int t = 4 * j + tr;
    const int64_t m = (int64_t)m_first + t;
    if (!o_ok || m >= a.M) continue;
    const float4 acc = *reinterpret_cast<const float4 *>(stg + t * 32 + 4 * fg);
    float v[4] = {acc.x + bias4.x, acc.y + bias4.y, acc.z + bias4.z, acc.w + bias4.w};
    const int64_t at = m * a.N + o0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (ACT == CATEN_B200_ACT_GELU) v[e] = gelu_ref(v[e]);
      if (ACT == CATEN_B200_ACT_RELU) v[e] = v[e] > 0.0f ? v[e] : 0.0f;
    }
    if (a.res) {
      const float4 r = *reinterpret_cast<const float4 *>(a.res + at);
      v[0] = r.x + v[0]; v[1] = r.y + v[1]; v[2] = r.z + v[2]; v[3] = r.w + v[3];
    }
    if (a.yhi) {
      uint32_t h[2], l[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const __nv_bfloat16 h0 = __float2bfloat16_rn(v[2 * e]), h1 = __float2bfloat16_rn(v[2 * e + 1]);
        h[e] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
        const __nv_bfloat16 l0 = __float2bfloat16_rn(v[2 * e] - __bfloat162float(h0));
        const __nv_bfloat16 l1 = __float2bfloat16_rn(v[2 * e + 1] - __bfloat162float(h1));
        l[e] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
      }
      *reinterpret_cast<uint2 *>(a.yhi + at) = make_uint2(h[0], h[1]);
      if (a.ylo) *reinterpret_cast<uint2 *>(a.ylo + at) = make_uint2(l[0], l[1]);
    } else {
      *reinterpret_cast<float4 *>(a.y + at) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

// K-major operand tile whose rows are BK bf16 wide: 128-byte rows with the 128-byte swizzle (8-row groups 1024 bytes
// apart) or 64-byte rows with the 64-byte swizzle (8-row groups 512 bytes apart)
template <int BK>
__device__ __forceinline__ uint64_t gd_desc(uint32_t saddr) {
  if (BK == 64) return umma_desc(saddr);
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;  // SWIZZLE_64B
  return d;
}

template <int NSPLIT>
__global__ void __launch_bounds__(GD_THREADS, 1)
gemm_dense_kernel(const __grid_constant__ CUtensorMap tw_hi, const __grid_constant__ CUtensorMap tw_lo,
                  const __grid_constant__ CUtensorMap tx_hi, const __grid_constant__ CUtensorMap tx_lo, const GdArgs a) {
  constexpr int BK = GdStage<NSPLIT>::BK;
  constexpr uint32_t ROW_BYTES = BK * 2u;
  constexpr uint32_t W_BYTES = GD_BM * ROW_BYTES, X_BYTES = GD_BN * ROW_BYTES;
  constexpr uint32_t STAGE_BYTES = (W_BYTES + X_BYTES) * (NSPLIT == 3 ? 2u : 1u);
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  smem += 1024;
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (S + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (2 * S + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (2 * S + 2 + b); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4);
  // [0] some role gave up a wait; [1] never set (for waits that must run their full limit)
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // stage layout: W_hi, [W_lo,] x_hi[, x_lo]
  const uint32_t stage0 = smem_u32(smem);
  auto st_whi = [&](int s) { return stage0 + (uint32_t)s * STAGE_BYTES; };
  auto st_wlo = [&](int s) { return stage0 + (uint32_t)s * STAGE_BYTES + W_BYTES; };
  auto st_xhi = [&](int s) { return stage0 + (uint32_t)s * STAGE_BYTES + (NSPLIT == 3 ? 2u : 1u) * W_BYTES; };
  auto st_xlo = [&](int s) { return st_xhi(s) + X_BYTES; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int num_k = a.K / BK;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), GD_EPI_WARPS);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  if (warp == 0 && lane == 0) {
    tma_prefetch_map(&tw_hi);
    tma_prefetch_map(&tx_hi);
    if (NSPLIT == 3) {
      tma_prefetch_map(&tw_lo);
      tma_prefetch_map(&tx_lo);
    }
  }
  // both operands and the residual were written by preceding kernels
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int issued = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x) {
        const int f0 = (tile % a.tiles_f) * GD_BM, m0 = (tile / a.tiles_f) * GD_BN;
        for (int kc = 0; kc < num_k; ++kc) {
          if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 11; a.status[2] = tile; }
            ok = false;
            break;
          }
          mbar_expect_tx(full(s), STAGE_BYTES);
          tma_load_2d(st_whi(s), &tw_hi, full(s), kc * BK, f0);
          if (NSPLIT == 3) tma_load_2d(st_wlo(s), &tw_lo, full(s), kc * BK, f0);
          tma_load_2d(st_xhi(s), &tx_hi, full(s), kc * BK, m0);
          if (NSPLIT == 3) tma_load_2d(st_xlo(s), &tx_lo, full(s), kc * BK, m0);
          ++issued;
          if (++s == S) { s = 0; ph ^= 1u; }
        }
      }
      if (*abort_flag) {
        // let the copies this thread started land before the CTA's shared memory is released
        for (int i = issued > S ? issued - S : 0; i < issued; ++i) mbar_wait(full(i % S), (uint32_t)(i / S) & 1u, abort_flag + 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (uniform control flow, one elected lane issues) ----------------
    int s = 0, it = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++it) {
      const int b = it & 1;
      // the epilogue has drained this accumulator (first use of each passes at once)
      if (!mbar_wait(acc_empty(b), (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag)) {
        if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 12; a.status[2] = tile; }
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + (uint32_t)b * GD_BN;
      for (int kc = 0; kc < num_k; ++kc) {
        if (!mbar_wait(full(s), ph, abort_flag)) {
          if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 13; a.status[2] = tile; }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t dwh = gd_desc<BK>(st_whi(s)), dwl = gd_desc<BK>(st_wlo(s));
        const uint64_t dxh = gd_desc<BK>(st_xhi(s)), dxl = gd_desc<BK>(st_xlo(s));
        if (elect_one()) {
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t adv = (uint64_t)(k4 * 2);  // 16 bf16 = 32 bytes = 2 descriptor units
            umma_bf16(acc, dwh + adv, dxh + adv, a.idesc, (kc > 0 || k4 > 0) ? 1u : 0u);
            if (NSPLIT == 3) {
              umma_bf16(acc, dwl + adv, dxh + adv, a.idesc, 1u);
              umma_bf16(acc, dwh + adv, dxl + adv, a.idesc, 1u);
            }
          }
          umma_commit(empty(s));  // frees the stage when these MMAs have read it
        }
        __syncwarp();
        if (++s == S) { s = 0; ph ^= 1u; }
      }
      if (ok && elect_one()) umma_commit(acc_full(b));
      __syncwarp();
    }
  } else {
    // ---------------- epilogue ----------------
    // a warp reaches the TMEM lanes of quadrant (warp % 4); the two warps of a quadrant split the columns
    const int quad = warp & 3, half = (warp - 2) >> 2;
    float *stg = reinterpret_cast<float *>(smem + (size_t)S * STAGE_BYTES) + (warp - 2) * 512;  // 16 rows x 32 features
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++it) {
      const int b = it & 1;
      const int f0 = (tile % a.tiles_f) * GD_BM, m0 = (tile / a.tiles_f) * GD_BN;
      int got = 0;
      if (lane == 0) {
        got = mbar_wait(acc_full(b), ((uint32_t)it >> 1) & 1u, abort_flag) ? 1 : 0;
        if (!got && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 14; a.status[2] = tile; }
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { ok = false; break; }
      tc_fence_after();
      // after the transpose a lane owns features o0 .. o0 + 3 (N % 4 == 0: all inside or all outside)
      const int64_t o0 = (int64_t)f0 + quad * 32 + 4 * (lane & 7);
      const bool o_ok = o0 < a.N;
      float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a.bias && o_ok) bias4 = *reinterpret_cast<const float4 *>(a.bias + o0);
      const uint32_t trow = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * GD_BN + half * (GD_BN / 2));
      for (int c = 0; c < GD_BN / 2; c += 16) {
        uint32_t r[16];
        tmem_ld16(trow + (uint32_t)c, r);
        tmem_ld_wait();
        __syncwarp();  // the previous block has been read out of the staging tile
#pragma unroll
        for (int i = 0; i < 16; ++i) stg[i * 32 + lane] = __uint_as_float(r[i]);
        __syncwarp();
        const int m_first = m0 + half * (GD_BN / 2) + c;
        if (a.act == CATEN_B200_ACT_GELU) gd_store_block<CATEN_B200_ACT_GELU>(a, stg, lane, bias4, o0, o_ok, m_first);
        else if (a.act == CATEN_B200_ACT_RELU) gd_store_block<CATEN_B200_ACT_RELU>(a, stg, lane, bias4, o0, o_ok, m_first);
        else gd_store_block<CATEN_B200_ACT_NONE>(a, stg, lane, bias4, o0, o_ok, m_first);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(b));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- host ---------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// rows x K bf16, K contiguous; a box is `box_rows` rows of `bk` k (128 bytes with the 128-byte swizzle, or 64 with
// the 64-byte one), zero fill outside
static int make_map(caten_b200_ctx *ctx, CUtensorMap *map, const void *base, int64_t rows, int64_t K, int box_rows, int bk) {
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)bk, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = ((EncodeTiledFn)ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box,
                                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, CATEN_B200_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return 0;
}

template <int WT>
static int launch_wsplit(caten_b200_ctx *ctx, const WSrc &ws, int64_t N, int64_t K, __nv_bfloat16 *hi, __nv_bfloat16 *lo) {
  const int64_t n8 = N * (K / 8);
  launch_k(ctx, wsplit_kernel<WT>, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, ws.qs, ws.d, ws.m, ws.qh, N, K, hi, lo);
  CB_LAUNCH_CHECK(ctx, "wsplit_kernel");
  return 0;
}

bool gemm_dense_applies(const caten_b200_ctx *ctx, int64_t M, int64_t N, int64_t K) {
  // enough rows that expanding the weights once is cheap next to the GEMM and the tiles fill the GPU
  return ctx->dense_gemm && M >= 1024 && N % 4 == 0 && K % GD_BK == 0 && K >= GD_BK && (M + GD_BN - 1) / GD_BN * ((N + GD_BM - 1) / GD_BM) >= ctx->sm_count;
}

// wt: a ggml type or WT_F32_T (then ws.qs is b[K, N] fp32).  x: fp32 [M, K], or its split bf16 copy when xhi is given.
int launch_gemm_dense(caten_b200_ctx *ctx, int wt, const WSrc &ws, const float *x, const __nv_bfloat16 *xhi, const __nv_bfloat16 *xlo,
                      const float *bias, const float *res, int act, float *y, BfOut ybf, int64_t M, int64_t N, int64_t K, int nsplit) {
  if (!ctx->encode_tiled) return fail(ctx, CATEN_B200_ECUDA, "gemm_dense: cuTensorMapEncodeTiled is not available");
  if (K % GD_BK || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_dense: shape %lldx%lldx%lld", (long long)M, (long long)N, (long long)K);
  if (nsplit != 1 && nsplit != 3) return fail(ctx, CATEN_B200_EINVAL, "gemm_dense: nsplit must be 1 or 3");
  const int parts = nsplit == 3 ? 2 : 1;
  // bf16 copy of the weights
  const size_t wb = ((size_t)N * K * 2 + 1023) & ~(size_t)1023;
  if (int rc = scratch_reserve(ctx, &ctx->wbf, wb * parts)) return rc;
  __nv_bfloat16 *whi = (__nv_bfloat16 *)ctx->wbf.ptr, *wlo = parts == 2 ? (__nv_bfloat16 *)((uint8_t *)ctx->wbf.ptr + wb) : nullptr;
  int rc = 0;
  switch (wt) {
    case CATEN_B200_F32: rc = launch_wsplit<CATEN_B200_F32>(ctx, ws, N, K, whi, wlo); break;
    case CATEN_B200_F16: rc = launch_wsplit<CATEN_B200_F16>(ctx, ws, N, K, whi, wlo); break;
    case CATEN_B200_Q4_0: rc = launch_wsplit<CATEN_B200_Q4_0>(ctx, ws, N, K, whi, wlo); break;
    case CATEN_B200_Q4_1: rc = launch_wsplit<CATEN_B200_Q4_1>(ctx, ws, N, K, whi, wlo); break;
    case CATEN_B200_Q5_0: rc = launch_wsplit<CATEN_B200_Q5_0>(ctx, ws, N, K, whi, wlo); break;
    case CATEN_B200_Q5_1: rc = launch_wsplit<CATEN_B200_Q5_1>(ctx, ws, N, K, whi, wlo); break;
    case CATEN_B200_Q8_0: rc = launch_wsplit<CATEN_B200_Q8_0>(ctx, ws, N, K, whi, wlo); break;
    case WT_F32_T:
      launch_k(ctx, bt_split_kernel, dim3((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32)), dim3(256), 0, (const float *)ws.qs, K, N, whi, wlo);
      CB_LAUNCH_CHECK(ctx, "bt_split_kernel");
      break;
    default: return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_dense: weight type %d", wt);
  }
  if (rc) return rc;
  // bf16 copy of the activations, unless their producer already wrote one
  if (!xhi) {
    const size_t xb = ((size_t)M * K * 2 + 1023) & ~(size_t)1023;
    if (int rc2 = scratch_reserve(ctx, &ctx->xbf, xb * parts)) return rc2;
    __nv_bfloat16 *h = (__nv_bfloat16 *)ctx->xbf.ptr, *l = parts == 2 ? (__nv_bfloat16 *)((uint8_t *)ctx->xbf.ptr + xb) : nullptr;
    const int64_t n8 = M * K / 8;
    launch_k(ctx, xsplit_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, x, n8, h, l);
    CB_LAUNCH_CHECK(ctx, "xsplit_kernel");
    xhi = h;
    xlo = l;
  } else if (nsplit == 3 && !xlo) {
    return fail(ctx, CATEN_B200_EINVAL, "gemm_dense: split-bf16 needs the lo part of x");
  }
  if (((uintptr_t)xhi | (uintptr_t)xlo) & 15) return fail(ctx, CATEN_B200_EINVAL, "gemm_dense: bf16 operand must be 16-byte aligned");

  CUtensorMap twh, twl, txh, txl;
  const int bk = nsplit == 3 ? GdStage<3>::BK : GdStage<1>::BK;
  if ((rc = make_map(ctx, &twh, whi, N, K, GD_BM, bk))) return rc;
  if ((rc = make_map(ctx, &twl, wlo ? wlo : whi, N, K, GD_BM, bk))) return rc;
  if ((rc = make_map(ctx, &txh, xhi, M, K, GD_BN, bk))) return rc;
  if ((rc = make_map(ctx, &txl, nsplit == 3 ? xlo : xhi, M, K, GD_BN, bk))) return rc;

  GdArgs a;
  a.bias = bias; a.res = res; a.y = y; a.yhi = ybf.hi; a.ylo = ybf.lo; a.status = ctx->d_status;
  a.act = act; a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.tiles_f = (int)((N + GD_BM - 1) / GD_BM);
  const int64_t tiles = (int64_t)a.tiles_f * ((M + GD_BN - 1) / GD_BN);
  if (tiles > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_dense: too many tiles");
  a.tiles = (int)tiles;
  const size_t stage = (size_t)(GD_BM + GD_BN) * (size_t)bk * 2 * parts;
  int stages = (int)((200 * 1024) / stage);  // 1 KB slack + 1 KB barriers + stages + 16 KB of epilogue staging fit 227 KB
  if (stages > 6) stages = 6;
  a.stages = stages;
  a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(GD_BN >> 3) << 17) | ((uint32_t)(GD_BM >> 4) << 24);
  const size_t smem = 2048 + stage * stages + (size_t)GD_EPI_WARPS * 2048;
  const int grid = tiles < ctx->sm_count ? (int)tiles : ctx->sm_count;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(GD_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = take_pdl(ctx) ? 1 : 0;
  if (nsplit == 3) {
    CB_CUDA(ctx, cudaFuncSetAttribute(gemm_dense_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CB_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_dense_kernel<3>, twh, twl, txh, txl, a));
  } else {
    CB_CUDA(ctx, cudaFuncSetAttribute(gemm_dense_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CB_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_dense_kernel<1>, twh, twl, txh, txl, a));
  }
  CB_LAUNCH_CHECK(ctx, "gemm_dense_kernel");
  return 0;
}

}  // namespace cb
