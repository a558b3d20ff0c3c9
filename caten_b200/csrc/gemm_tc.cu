// Dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only:
//   y[m, o] = act(sum_k x[m,k] * W[o,k] + bias[o]) + res[m, o]
//
// Orientation.  The packed weight tile is the MMA "A" operand (128 rows of W = 128 TMEM lanes)
// and the activations are the "B" operand (BNX rows of x = BNX TMEM columns), i.e. the kernel
// computes y^T tiles.  W is then streamed from HBM exactly once per 256 activation rows, small
// batches (8..256 rows in decode) cost one narrow MMA instead of a padded 128-row one, and in
// the epilogue one thread owns one output feature, so bias is a scalar and stores of a fixed
// activation row are coalesced across the warp.
//
// Pipeline per CTA (320 threads), K in chunks of 64:
//   warps 0-7  load the packed weight chunk (128 rows x 64 k) with vector loads, dequantise in
//              registers to bf16 and write it to shared memory in the 128-byte-swizzled K-major
//              layout tcgen05.mma reads; after the K loop they run the epilogue
//              (tcgen05.ld -> bias/activation/residual -> global)
//   warp 8     one lane issues the TMA loads of the activation chunk (bf16 copy of x made by a
//              small pre-pass; tiled cp.async.bulk.tensor, no multicast)
//   warp 9     allocates TMEM; one lane issues tcgen05.mma and commits to the stage's mbarrier
// NSPLIT = 1: plain bf16 operands.  NSPLIT = 3: x = x_hi + x_lo and w = w_hi + w_lo in bf16 and
// three products (hi*hi + lo*hi + hi*lo) accumulate in the same fp32 TMEM tile.
//
// Every mbarrier wait is bounded; when one runs out the kernel records it in the context's
// status word, stops issuing work, waits (bounded) for its own TMA copies, frees TMEM and returns.
#include "common.cuh"

namespace cb {

constexpr int WT_F32_T = 100;  // fp32 operand given as [K, N] row-major (relu_matmul's b)

constexpr int TC_BM = 128;      // weight rows per CTA (MMA M)
constexpr int TC_BK = 64;       // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int TC_WBYTES = TC_BM * TC_BK * 2;
constexpr int TC_THREADS = 320;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

struct TcArgs {
  const void *qs;
  const __half *d;
  const float *bias, *res;
  float *y;
  int *status;
  int act, M, N, K, nkb, bnx, stages;
  uint32_t idesc, tmem_cols;
};

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
    if (mbar_try(bar, parity)) return true;
    if (i > 1024) {
      if (*abort_flag) return false;
      __nanosleep(64);
    }
  }
  return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;          // leading-dimension byte offset (unused for swizzled K-major): 1
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;          // version
  d |= (uint64_t)2 << 61;          // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- operand split and swizzled stores ----------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);  // .x = a in the low half
  return *reinterpret_cast<const uint32_t *>(&v);
}
// residual of the bf16 rounding, itself rounded to bf16
__device__ __forceinline__ float bf16_lo(float w) { return w - __bfloat162float(__float2bfloat16_rn(w)); }

// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a [rows x 128 B] tile, Swizzle<3,4,3>
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

template <int NSPLIT>
__device__ __forceinline__ void store8(uint8_t *whi, uint8_t *wlo, int r, int c, const float *w) {
  *reinterpret_cast<uint4 *>(whi + swz(r, c)) =
      make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
  if (NSPLIT == 3) {
    float l[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) l[e] = bf16_lo(w[e]);
    *reinterpret_cast<uint4 *>(wlo + swz(r, c)) =
        make_uint4(pack_bf16(l[0], l[1]), pack_bf16(l[2], l[3]), pack_bf16(l[4], l[5]), pack_bf16(l[6], l[7]));
  }
}

// Weight chunk (128 rows x 64 k) -> shared memory, by the 256 producer threads.
template <int WT, int NSPLIT>
__device__ __forceinline__ void produce_w(const TcArgs &a, int n0, int kc, uint8_t *whi, uint8_t *wlo, int tid) {
  if (WT == CATEN_B200_Q4_0 || WT == CATEN_B200_Q8_0) {
    // thread = (row, block of 32): two adjacent threads read 32 (Q4_0) / 64 (Q8_0) contiguous bytes
    const int r = tid >> 1, blk = tid & 1;
    const int64_t row = (int64_t)n0 + r;
    const bool ok = row < a.N;
    const int64_t bi = row * a.nkb + (int64_t)kc * 2 + blk;
    const float sc = ok ? __half2float(a.d[bi]) : 0.0f;
    if (WT == CATEN_B200_Q4_0) {
      const uint4 q = ok ? __ldcs(reinterpret_cast<const uint4 *>(a.qs) + bi) : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
      const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
      // chunk 0: low nibbles of bytes 0-7, 1: low of bytes 8-15, 2: high of 0-7, 3: high of 8-15
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t word = wd[(c & 1) * 2 + (e >> 2)];
          const int nib = (int)((word >> (8 * (e & 3) + (c >> 1) * 4)) & 0xF);
          w[e] = (float)(nib - 8) * sc;
        }
        store8<NSPLIT>(whi, wlo, r, blk * 4 + c, w);
      }
    } else {
      const uint4 *p = reinterpret_cast<const uint4 *>(a.qs) + bi * 2;
      const uint4 q0 = ok ? __ldcs(p) : make_uint4(0, 0, 0, 0), q1 = ok ? __ldcs(p + 1) : make_uint4(0, 0, 0, 0);
      const uint32_t wd[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = (float)(int8_t)(wd[2 * c + (e >> 2)] >> (8 * (e & 3))) * sc;
        store8<NSPLIT>(whi, wlo, r, blk * 4 + c, w);
      }
    }
  } else if (WT == CATEN_B200_F32) {
    // warp w covers rows 16w..16w+15, two rows per load instruction, 16 lanes x 16 B per row
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = 16 * warp + 2 * j + (lane >> 4), c4 = lane & 15;
      const int64_t row = (int64_t)n0 + r;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < a.N) v = __ldcs(reinterpret_cast<const float4 *>((const float *)a.qs + row * a.K + (int64_t)kc * 64) + c4);
      const uint32_t off = swz(r, c4 >> 1) + (c4 & 1) * 8;
      *reinterpret_cast<uint2 *>(whi + off) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
      if (NSPLIT == 3)
        *reinterpret_cast<uint2 *>(wlo + off) = make_uint2(pack_bf16(bf16_lo(v.x), bf16_lo(v.y)), pack_bf16(bf16_lo(v.z), bf16_lo(v.w)));
    }
  } else if (WT == CATEN_B200_F16) {
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = 16 * warp + 4 * j + (lane >> 3), c = lane & 7;
      const int64_t row = (int64_t)n0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < a.N) v = __ldcs(reinterpret_cast<const uint4 *>((const __half *)a.qs + row * a.K + (int64_t)kc * 64) + c);
      const __half *h = reinterpret_cast<const __half *>(&v);
      float w[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = __half2float(h[e]);
      store8<NSPLIT>(whi, wlo, r, c, w);
    }
  } else {  // WT_F32_T: b[k, n]; thread = (n, half of the 64 k); loads coalesced across n
    const int r = tid & 127, kh = tid >> 7;
    const int64_t col = (int64_t)n0 + r;
    const float *b = (const float *)a.qs + ((int64_t)kc * 64 + kh * 32) * a.N + col;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float w[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) w[e] = col < a.N ? __ldcs(b + (int64_t)(c * 8 + e) * a.N) : 0.0f;
      store8<NSPLIT>(whi, wlo, r, kh * 4 + c, w);
    }
  }
}

template <int WT, int NSPLIT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_hi, const __grid_constant__ CUtensorMap tm_lo, const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages, bnx = a.bnx;
  const uint32_t xbytes = (uint32_t)bnx * 128u;
  const uint32_t stage_bytes = (TC_WBYTES + xbytes) * (NSPLIT == 3 ? 2u : 1u);
  // barriers + bookkeeping live after the stage buffers
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)S * stage_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_w = [&](int s) { return bar0 + 8u * s; };
  auto full_x = [&](int s) { return bar0 + 8u * (S + s); };
  auto empty = [&](int s) { return bar0 + 8u * (2 * S + s); };
  const uint32_t accum_bar = bar0 + 8u * (3 * S);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * S + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  auto stage_whi = [&](int s) { return smem + (size_t)s * stage_bytes; };
  auto stage_wlo = [&](int s) { return smem + (size_t)s * stage_bytes + TC_WBYTES; };
  auto stage_xhi = [&](int s) { return smem + (size_t)s * stage_bytes + (NSPLIT == 3 ? 2 : 1) * TC_WBYTES; };
  auto stage_xlo = [&](int s) { return stage_xhi(s) + xbytes; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * TC_BM, m0 = blockIdx.y * bnx;
  const int num_k = a.K / TC_BK;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_w(s), 256);
      mbar_init(full_x(s), 1);
      mbar_init(empty(s), 1);
    }
    mbar_init(accum_bar, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;  // second word: a flag nothing sets, for waits that must not be cut short
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // ---------------- weight producers ----------------
    for (int kc = 0; kc < num_k; ++kc) {
      const int s = kc % S;
      const uint32_t ph = (uint32_t)(kc / S) & 1u;
      if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
        if (!*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 1; a.status[2] = kc; }
        break;
      }
      produce_w<WT, NSPLIT>(a, n0, kc, stage_whi(s), stage_wlo(s), tid);
      fence_proxy_async();
      mbar_arrive(full_w(s));
    }
    // ---------------- epilogue ----------------
    bool ok = !*abort_flag && mbar_wait(accum_bar, 0, abort_flag);
    if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 2; }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int quad = warp & 3;
      const int64_t o = (int64_t)n0 + quad * 32 + lane;  // output feature of this thread
      const bool o_ok = o < a.N;
      const float bias = (a.bias && o_ok) ? a.bias[o] : 0.0f;
      const int half_cols = bnx >= 32 ? bnx / 2 : bnx;
      const int c_begin = (warp >> 2) * half_cols, c_end = bnx >= 32 ? c_begin + half_cols : (warp < 4 ? bnx : 0);
      for (int c = c_begin; c < c_end; c += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int64_t m = (int64_t)m0 + c + i;
          if (o_ok && m < a.M) {
            float v = __uint_as_float(r[i]);
            if (a.bias) v = v + bias;
            v = apply_act(v, a.act);
            if (a.res) v = a.res[m * a.N + o] + v;
            a.y[m * a.N + o] = v;
          }
        }
      }
    }
    tc_fence_before();
  } else if (warp == 8) {
    // ---------------- activation TMA producer ----------------
    if (lane == 0) {
      int issued = 0;
      for (int kc = 0; kc < num_k; ++kc) {
        const int s = kc % S;
        const uint32_t ph = (uint32_t)(kc / S) & 1u;
        if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 3; a.status[2] = kc; }
          break;
        }
        mbar_expect_tx(full_x(s), xbytes * (NSPLIT == 3 ? 2u : 1u));
        tma_load_2d(smem_u32(stage_xhi(s)), &tm_hi, full_x(s), kc * TC_BK, m0);
        if (NSPLIT == 3) tma_load_2d(smem_u32(stage_xlo(s)), &tm_lo, full_x(s), kc * TC_BK, m0);
        issued = kc + 1;
      }
      if (*abort_flag) {
        // let the copies this thread started land before the CTA's shared memory is released
        for (int kc = issued > S ? issued - S : 0; kc < issued; ++kc)
          mbar_wait(full_x(kc % S), (uint32_t)(kc / S) & 1u, abort_flag + 1 /* never set: full wait */);
      }
    }
  } else {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      for (int kc = 0; kc < num_k && ok; ++kc) {
        const int s = kc % S;
        const uint32_t ph = (uint32_t)(kc / S) & 1u;
        ok = mbar_wait(full_w(s), ph, abort_flag) && mbar_wait(full_x(s), ph, abort_flag);
        if (!ok) {
          if (!*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 4; a.status[2] = kc; }
          break;
        }
        tc_fence_after();
        const uint64_t dwh = umma_desc(smem_u32(stage_whi(s))), dxh = umma_desc(smem_u32(stage_xhi(s)));
        const uint64_t dwl = umma_desc(smem_u32(stage_wlo(s))), dxl = umma_desc(smem_u32(stage_xlo(s)));
#pragma unroll
        for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
          const uint64_t adv = (uint64_t)(k4 * 2);  // 16 bf16 = 32 bytes = 2 descriptor units
          umma_bf16(tmem_base, dwh + adv, dxh + adv, a.idesc, (kc > 0 || k4 > 0) ? 1u : 0u);
          if (NSPLIT == 3) {
            umma_bf16(tmem_base, dwl + adv, dxh + adv, a.idesc, 1u);
            umma_bf16(tmem_base, dwh + adv, dxl + adv, a.idesc, 1u);
          }
        }
        umma_commit(empty(s));
      }
      if (ok) umma_commit(accum_bar);
    }
    __syncwarp();
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
  }
}

// x -> bf16 hi (and lo) copies, row-major [M, K]
__global__ void split_bf16_kernel(const float4 *__restrict__ x, uint2 *__restrict__ hi, uint2 *__restrict__ lo, int64_t n4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v = x[i];
  hi[i] = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  if (lo) lo[i] = make_uint2(pack_bf16(bf16_lo(v.x), bf16_lo(v.y)), pack_bf16(bf16_lo(v.z), bf16_lo(v.w)));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_x_map(caten_b200_ctx *ctx, CUtensorMap *map, void *base, int64_t M, int64_t K, int bnx) {
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)bnx};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = ((EncodeTiledFn)ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, CATEN_B200_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return 0;
}

template <int WT, int NSPLIT>
static int launch_tc_t(caten_b200_ctx *ctx, const CUtensorMap &mh, const CUtensorMap &ml, const TcArgs &a, dim3 grid, size_t smem) {
  CB_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<WT, NSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  gemm_tc_kernel<WT, NSPLIT><<<grid, TC_THREADS, smem, ctx->stream>>>(mh, ml, a);
  CB_LAUNCH_CHECK(ctx, "gemm_tc_kernel");
  return 0;
}

static int run_tc(caten_b200_ctx *ctx, int wt, const void *qs, const __half *d, int64_t nkb, const float *x,
                  const float *bias, const float *res, int act, float *y, int64_t M, int64_t N, int64_t K, int nsplit) {
  if (M <= 0 || N <= 0) return 0;
  if (!ctx->encode_tiled) return fail(ctx, CATEN_B200_ECUDA, "gemm_tc: cuTensorMapEncodeTiled is not available");
  if (K % TC_BK) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_tc: inner dimension %lld is not a multiple of 64", (long long)K);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_tc: dimension too large");
  if (nsplit != 1 && nsplit != 3) return fail(ctx, CATEN_B200_EINVAL, "gemm_tc: nsplit must be 1 or 3");
  // activations -> bf16 (hi[, lo]) in the context's scratch buffer
  const size_t xb = (size_t)M * K * 2;
  const size_t xb_al = (xb + 1023) & ~(size_t)1023;
  if (int rc = scratch_reserve(ctx, &ctx->xbf, xb_al * (nsplit == 3 ? 2 : 1))) return rc;
  uint8_t *xhi = (uint8_t *)ctx->xbf.ptr, *xlo = nsplit == 3 ? xhi + xb_al : nullptr;
  const int64_t n4 = M * K / 4;
  split_bf16_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, ctx->stream>>>((const float4 *)x, (uint2 *)xhi, (uint2 *)xlo, n4);
  CB_LAUNCH_CHECK(ctx, "split_bf16_kernel");

  const int max_bnx = nsplit == 3 ? 128 : 256;
  int bnx = 16;
  while (bnx < max_bnx && bnx < M) bnx *= 2;
  CUtensorMap mh, ml;
  if (int rc = make_x_map(ctx, &mh, xhi, M, K, bnx)) return rc;
  if (int rc = make_x_map(ctx, &ml, nsplit == 3 ? xlo : xhi, M, K, bnx)) return rc;

  TcArgs a;
  a.qs = qs; a.d = d; a.bias = bias; a.res = res; a.y = y; a.status = ctx->d_status; a.act = act;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.nkb = (int)nkb; a.bnx = bnx;
  const size_t stage = (size_t)(TC_WBYTES + bnx * 128) * (nsplit == 3 ? 2 : 1);
  int stages = (int)((200 * 1024) / stage);
  if (stages > 8) stages = 8;
  if (stages > K / TC_BK) stages = (int)(K / TC_BK);
  if (stages < 1) stages = 1;
  a.stages = stages;
  a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bnx >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
  a.tmem_cols = bnx < 32 ? 32u : (uint32_t)bnx;
  const size_t smem = 1024 + stage * stages + (3 * stages + 1) * 8 + 16;
  const int64_t gy = (M + bnx - 1) / bnx;
  if (gy > 65535) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_tc: too many rows for one launch (%lld)", (long long)M);
  const dim3 grid((unsigned)((N + TC_BM - 1) / TC_BM), (unsigned)gy);

#define TC_CASE(WT)                                                              \
  case WT:                                                                       \
    return nsplit == 3 ? launch_tc_t<WT, 3>(ctx, mh, ml, a, grid, smem) : launch_tc_t<WT, 1>(ctx, mh, ml, a, grid, smem)
  switch (wt) {
    TC_CASE(CATEN_B200_F32);
    TC_CASE(CATEN_B200_F16);
    TC_CASE(CATEN_B200_Q4_0);
    TC_CASE(CATEN_B200_Q8_0);
    TC_CASE(WT_F32_T);
  }
#undef TC_CASE
  return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_tc: weight type %d", wt);
}

int launch_gemm_tc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                   const float *res, int act, float *y, int64_t M, int nsplit) {
  return run_tc(ctx, w->type, w->qs, w->d, w->nkb, x, bias, res, act, y, M, w->rows, w->cols, nsplit);
}

int launch_relu_matmul_tc(caten_b200_ctx *ctx, const float *a, const float *b, float *c, int64_t M, int64_t K, int64_t N, int nsplit) {
  return run_tc(ctx, WT_F32_T, b, nullptr, 0, a, nullptr, nullptr, CATEN_B200_ACT_RELU, c, M, N, K, nsplit);
}

}  // namespace cb
