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
// Pipeline per CTA, K in chunks of 64:
//   producer warps (16, or 8 for fp32 weights) load one weight row each (64 k of packed
//              weights), dequantise in registers to bf16 and write the result to TENSOR MEMORY
//              (tcgen05.st): the weight tile is the MMA's A operand read from TMEM, so shared
//              memory carries only the activations; after the K loop they run the epilogue
//              (tcgen05.ld -> bias/activation/residual -> global)
//   TMA warp   one lane issues the TMA loads of the activation chunk (bf16 copy of x written by
//              the kernel that produced x; tiled cp.async.bulk.tensor, no multicast) into the
//              128-byte-swizzled K-major layout tcgen05.mma reads as B
//   MMA warp   allocates TMEM; one lane issues tcgen05.mma (A in TMEM, B in shared memory) and
//              commits to the stage's mbarrier
// TMEM: columns [0, 256) accumulator, [256, 512) ring of weight stages (32 columns hi [+ 32 lo]).
// NSPLIT = 1: plain bf16 operands.  NSPLIT = 3: x = x_hi + x_lo and w = w_hi + w_lo in bf16.  With
// 256 activation rows three products (hi*hi + lo*hi + hi*lo) accumulate in one fp32 TMEM tile;
// with at most 128 rows B is the 2*rows-row tile [x_hi; x_lo], so two MMAs per k-step give all
// four products in two column blocks that the epilogue adds.
//
// Every mbarrier wait is bounded; when one runs out the kernel records it in the context's
// status word, stops issuing work, waits (bounded) for its own TMA copies, frees TMEM and returns.
#include <atomic>

#include "common.cuh"
#include "blocks32.cuh"
#include "tcgen05.cuh"

namespace cb {


constexpr int TC_BM = 128;      // weight rows per CTA (MMA M)
constexpr int TC_BK = 64;       // k per stage: 64 bf16 = one 128-byte swizzle row

struct TcArgs {
  const void *qs;
  const __half *d, *m;   // per-block scales; minima (Q4_1, Q5_1)
  const uint32_t *qh;    // per-block fifth code bits (Q5_0, Q5_1)
  const float *bias, *res;
  float *y;
  int *status;
  int act, M, N, K, nkb, bnx, stages;
  uint32_t idesc;
  int concat;  // 1: B operand = [x_hi; x_lo], accumulator columns [bnx, 2 bnx) hold the x_lo products
  // split-K: grid.z CTAs share one output tile, each covering `cps` K-chunks; partial tiles go
  // to `part` and splitk_reduce_kernel adds them in split order and applies the epilogue
  int splits, cps;
  int cluster;  // 1: the `splits` CTAs of a tile form a thread-block cluster and reduce through distributed shared memory
  float *part;
  // when yhi is set the epilogue writes the result as split bf16 (operand of the next GEMM), not y
  __nv_bfloat16 *yhi, *ylo;
};


// Optional timestamps of CTA (0,0,0) (development builds only: -DDS_TIMING), one stream of (tag, SM cycle) pairs per role:
// 0 = first producer warp, 1 = activation TMA lane, 2 = MMA warp; read back with cb_debug_tc_marks().
#ifdef DS_TIMING
__device__ long long g_tc_marks[3][256][2];
__device__ int g_tc_marks_n[3];
#define TC_MARK(role, tag, k) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (k) < 256) { g_tc_marks[role][k][0] = (tag); g_tc_marks[role][k][1] = clock64(); g_tc_marks_n[role] = ++(k); } } while (0)
#else
#define TC_MARK(role, tag, k) do { } while (0)
#endif

// ---- weight rows: global memory -> registers -> bf16 in tensor memory -----------------------------
//
// The weight tile is the MMA's A operand and lives in tensor memory, not in shared memory: TMEM
// lane = weight row (128 per CTA), and a 32-bit TMEM column holds two consecutive k (low half =
// even k), so a 64-k chunk of bf16 is 32 columns.  A producer thread owns one row: it loads the
// row's 64 k of packed weights, converts them in registers and writes them with tcgen05.st.  The
// tensor core then reads A from TMEM and only the activations (B) from shared memory, which keeps
// the shared-memory port for the TMA writes and the B reads.
//
// The producer warps form GROUPS groups of 4 (one warp per 32-lane TMEM quadrant); the groups
// take the chunks in turn.  DEPTH chunks of a group's future loads are in flight.

constexpr int TC_WCOL0 = 256;  // first TMEM column of the weight stages (the accumulator has columns [0, 256))

// 16 consecutive k given as fp32 -> 8 columns of hi (and lo) at column offset `col` of the stage
template <int NSPLIT>
__device__ __forceinline__ void emit16(uint32_t t_hi, int col, const float *w) {
  uint32_t h[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) h[e] = pack_bf16(w[2 * e], w[2 * e + 1]);
  tmem_st8(t_hi + col, h);
  if (NSPLIT == 3) {
    uint32_t l[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) l[e] = pack_bf16(bf16_lo(w[2 * e]), bf16_lo(w[2 * e + 1]));
    tmem_st8(t_hi + 32 + col, l);
  }
}

template <int WT> struct WRow;

// Q4_0, converted with packed bf16 arithmetic (two weights per instruction, no fp32 detour):
//   A  = code - 8                      exact in bf16 (|A| <= 8)
//   d  = dh + dl, dh = bf16(d)         exact: an fp16 scale has 11 significant bits, dl at most 3
//   hi = bf16(A * dh)                  one rounding
//   lo = bf16(A * dl + (A * dh - hi))  the inner difference is exact; hi + lo = A * d to 2^-17
// NSPLIT = 1 stores bf16(A * d) (correctly rounded: A * dl is exact, then one fused rounding).
template <> struct WRow<CATEN_B200_Q4_0> {
  static constexpr int DEPTH = 3, GROUPS = 4;
  uint4 q[2];     // the chunk's two blocks; byte j: low nibble = element j, high nibble = element j + 16
  uint32_t sc2;   // their two fp16 scales
  __device__ __forceinline__ void load(const TcArgs &a, int64_t row, bool ok, int kc) {
    if (ok) {
      const int64_t bi = row * a.nkb + (int64_t)kc * 2;
      q[0] = __ldcs(reinterpret_cast<const uint4 *>(a.qs) + bi);
      q[1] = __ldcs(reinterpret_cast<const uint4 *>(a.qs) + bi + 1);
      sc2 = *reinterpret_cast<const uint32_t *>(a.d + bi);  // bi is even: 4-byte aligned
    } else {
      q[0] = q[1] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
      sc2 = 0u;
    }
  }
  // code bytes FIRST, FIRST + 1 of `word` (shifted so that the wanted nibbles are the low ones)
  // -> bf16x2 (code0 - 8, code1 - 8); 0x4300 | n is the bf16 value 128 + n
  template <int FIRST> static __device__ __forceinline__ __nv_bfloat162 codes2(uint32_t word) {
    const uint32_t two = __byte_perm(word, 0u, FIRST == 0 ? 0x4140u : 0x4342u);
    const uint32_t bits = (two & 0x000F000Fu) | 0x43004300u;
    const uint32_t off = 0x43084308u;  // bf16x2 (136, 136)
    return __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&bits), *reinterpret_cast<const __nv_bfloat162 *>(&off));
  }
  template <int NSPLIT> __device__ __forceinline__ void store(uint32_t t_hi) const {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const float d = __half2float(__ushort_as_half((unsigned short)(b ? sc2 >> 16 : sc2 & 0xFFFFu)));
      const __nv_bfloat16 dh1 = __float2bfloat16_rn(d);
      const __nv_bfloat16 dl1 = __float2bfloat16_rn(d - __bfloat162float(dh1));
      const __nv_bfloat162 dh = __halves2bfloat162(dh1, dh1), dl = __halves2bfloat162(dl1, dl1);
      const uint32_t wd[4] = {q[b].x, q[b].y, q[b].z, q[b].w};
      uint32_t h[16], l[16];
#pragma unroll
      for (int p = 0; p < 16; ++p) {  // pair p = elements 2p, 2p + 1 of the block
        const uint32_t word = wd[(p & 7) >> 1] >> (p >= 8 ? 4 : 0);
        const __nv_bfloat162 A = (p & 1) ? codes2<2>(word) : codes2<0>(word);
        if (NSPLIT == 3) {
          const __nv_bfloat162 hv = __hmul2(A, dh);
          const __nv_bfloat162 lv = __hfma2(A, dl, __hfma2(A, dh, __hneg2(hv)));
          h[p] = *reinterpret_cast<const uint32_t *>(&hv);
          l[p] = *reinterpret_cast<const uint32_t *>(&lv);
        } else {
          const __nv_bfloat162 hv = __hfma2(A, dh, __hmul2(A, dl));
          h[p] = *reinterpret_cast<const uint32_t *>(&hv);
        }
      }
      tmem_st16(t_hi + 16 * b, h);
      if (NSPLIT == 3) tmem_st16(t_hi + 32 + 16 * b, l);
    }
  }
};

// Q4_1, Q5_0, Q5_1: each weight is formed in fp32 exactly as the dequantiser forms it (code
// product, then the minimum), then split into bf16 terms.
template <int WT> struct WRowNibble {
  static constexpr int DEPTH = 2, GROUPS = 4;
  uint4 q[2];       // the chunk's two blocks of nibbles
  uint32_t sc2;     // their fp16 scales
  uint32_t mn2;     // their fp16 minima (the _1 formats)
  uint32_t hb[2];   // their fifth code bits (the 5-bit formats)
  __device__ __forceinline__ void load(const TcArgs &a, int64_t row, bool ok, int kc) {
    if (ok) {
      const int64_t bi = row * a.nkb + (int64_t)kc * 2;  // even: the pairs below are naturally aligned
      q[0] = __ldcs(reinterpret_cast<const uint4 *>(a.qs) + bi);
      q[1] = __ldcs(reinterpret_cast<const uint4 *>(a.qs) + bi + 1);
      sc2 = *reinterpret_cast<const uint32_t *>(a.d + bi);
      mn2 = type_has_min(WT) ? *reinterpret_cast<const uint32_t *>(a.m + bi) : 0u;
      if (type_has_qh(WT)) {
        const uint2 h = *reinterpret_cast<const uint2 *>(a.qh + bi);
        hb[0] = h.x; hb[1] = h.y;
      } else {
        hb[0] = hb[1] = 0u;
      }
    } else {
      // codes that dequantise to zero with scale and minimum zero
      q[0] = q[1] = make_uint4(0u, 0u, 0u, 0u);
      sc2 = mn2 = 0u;
      hb[0] = hb[1] = 0u;
    }
  }
  template <int NSPLIT> __device__ __forceinline__ void store(uint32_t t_hi) const {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const float d = __half2float(__ushort_as_half((unsigned short)(b ? sc2 >> 16 : sc2 & 0xFFFFu)));
      const float mn = __half2float(__ushort_as_half((unsigned short)(b ? mn2 >> 16 : mn2 & 0xFFFFu)));
      const uint32_t wd[4] = {q[b].x, q[b].y, q[b].z, q[b].w};
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // elements 0..15: low nibbles of the 16 bytes; 16..31: high nibbles
        float w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int nib = (int)((wd[e >> 2] >> (8 * (e & 3) + 4 * half)) & 15u);
          const int code = nib | (int)(((hb[b] >> (16 * half + e)) & 1u) << 4);
          w[e] = nibble_value<WT>(code, d, mn);
        }
        emit16<NSPLIT>(t_hi, 16 * b + 8 * half, w);
      }
    }
  }
};
template <> struct WRow<CATEN_B200_Q4_1> : WRowNibble<CATEN_B200_Q4_1> {};
template <> struct WRow<CATEN_B200_Q5_0> : WRowNibble<CATEN_B200_Q5_0> {};
template <> struct WRow<CATEN_B200_Q5_1> : WRowNibble<CATEN_B200_Q5_1> {};

template <> struct WRow<CATEN_B200_Q8_0> {
  static constexpr int DEPTH = 2, GROUPS = 4;
  uint4 q[4];   // 2 blocks x 32 codes
  uint32_t sc2;
  __device__ __forceinline__ void load(const TcArgs &a, int64_t row, bool ok, int kc) {
    if (ok) {
      const int64_t bi = row * a.nkb + (int64_t)kc * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = __ldcs(reinterpret_cast<const uint4 *>(a.qs) + bi * 2 + j);
      sc2 = *reinterpret_cast<const uint32_t *>(a.d + bi);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = make_uint4(0, 0, 0, 0);
      sc2 = 0u;
    }
  }
  template <int NSPLIT> __device__ __forceinline__ void store(uint32_t t_hi) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // 16 codes each
      const float d = __half2float(__ushort_as_half((unsigned short)(j >= 2 ? sc2 >> 16 : sc2 & 0xFFFFu)));
      const uint32_t wd[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
      float w[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) w[e] = (float)(int8_t)(wd[e >> 2] >> (8 * (e & 3))) * d;
      emit16<NSPLIT>(t_hi, 8 * j, w);
    }
  }
};

template <> struct WRow<CATEN_B200_F16> {
  static constexpr int DEPTH = 1, GROUPS = 4;
  uint4 v[8];
  __device__ __forceinline__ void load(const TcArgs &a, int64_t row, bool ok, int kc) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      v[j] = ok ? __ldcs(reinterpret_cast<const uint4 *>((const __half *)a.qs + row * a.K + (int64_t)kc * 64) + j) : make_uint4(0, 0, 0, 0);
  }
  template <int NSPLIT> __device__ __forceinline__ void store(uint32_t t_hi) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half *h = reinterpret_cast<const __half *>(&v[2 * j]);
      float w[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) w[e] = __half2float(h[e]);
      emit16<NSPLIT>(t_hi, 8 * j, w);
    }
  }
};

// fp32 rows: 64 floats per thread and chunk; two groups of four warps so that the registers fit
template <> struct WRow<CATEN_B200_F32> {
  static constexpr int DEPTH = 1, GROUPS = 2;
  float4 v[16];
  __device__ __forceinline__ void load(const TcArgs &a, int64_t row, bool ok, int kc) {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      v[j] = ok ? __ldcs(reinterpret_cast<const float4 *>((const float *)a.qs + row * a.K + (int64_t)kc * 64) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  template <int NSPLIT> __device__ __forceinline__ void store(uint32_t t_hi) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) emit16<NSPLIT>(t_hi, 8 * j, reinterpret_cast<const float *>(&v[4 * j]));
  }
};

// b[k, n] (relu_matmul): the "row" is column n of b; loads are coalesced across the warp's lanes
template <> struct WRow<WT_F32_T> {
  static constexpr int DEPTH = 1, GROUPS = 2;
  float v[64];
  __device__ __forceinline__ void load(const TcArgs &a, int64_t row, bool ok, int kc) {
    const float *b = (const float *)a.qs + (int64_t)kc * 64 * a.N + row;
#pragma unroll
    for (int e = 0; e < 64; ++e) v[e] = ok ? __ldcs(b + (int64_t)e * a.N) : 0.0f;
  }
  template <int NSPLIT> __device__ __forceinline__ void store(uint32_t t_hi) const {
#pragma unroll
    for (int j = 0; j < 4; ++j) emit16<NSPLIT>(t_hi, 8 * j, v + 16 * j);
  }
};

template <int WT> constexpr int tc_threads() { return (WRow<WT>::GROUPS * 4 + 2) * 32; }

// Epilogue of one 16-column group held in registers: y[m, o] = act(acc + bias) + res.
template <int ACT>
__device__ __forceinline__ void epi_store16(const TcArgs &a, const uint32_t *r, float bias, int64_t o, int m_first) {
  float *yp = a.y + (int64_t)m_first * a.N + o;
  const float *rp = a.res ? a.res + (int64_t)m_first * a.N + o : nullptr;
  const int lim = a.M - m_first < 16 ? a.M - m_first : 16;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (i < lim) {
      float v = __uint_as_float(r[i]) + bias;
      if (ACT == CATEN_B200_ACT_GELU) v = gelu_ref(v);
      if (ACT == CATEN_B200_ACT_RELU) v = v > 0.0f ? v : 0.0f;
      if (rp) v = rp[(int64_t)i * a.N] + v;
      if (a.yhi) {
        const int64_t at = ((int64_t)m_first + i) * a.N + o;
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        a.yhi[at] = h;
        if (a.ylo) a.ylo[at] = __float2bfloat16_rn(v - __bfloat162float(h));
      } else {
        yp[(int64_t)i * a.N] = v;
      }
    }
  }
}

template <int WT, int NSPLIT>
__global__ void __launch_bounds__(tc_threads<WT>(), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_hi, const __grid_constant__ CUtensorMap tm_lo, const TcArgs a) {
  constexpr int GROUPS = WRow<WT>::GROUPS, DEPTH = WRow<WT>::DEPTH;
  constexpr int NPROD = GROUPS * 128;           // producer threads
  constexpr int TMA_WARP = GROUPS * 4, MMA_WARP = GROUPS * 4 + 1;
  constexpr uint32_t WCOLS = NSPLIT == 3 ? 64u : 32u;  // TMEM columns of one weight stage (hi [, lo])
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.stages, bnx = a.bnx;
  const uint32_t xbytes = (uint32_t)bnx * 128u;
  const uint32_t stage_bytes = xbytes * (NSPLIT == 3 ? 2u : 1u);
  // first 1 KB: barriers + bookkeeping; then the activation stages (reused as the split-K staging tile)
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  smem += 1024;
  const uint32_t bar0 = smem_u32(bars);
  // full(s): both operands of the stage are in place (one arrival per warp of the producer group that wrote the
  // weight stage, plus the TMA lane's arrive.expect_tx for the activation tile): the MMA warp's loop is a chain of
  // waits and issues in one thread, and a second barrier per chunk cost it a quarter of its time with few rows
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (S + s); };
  const uint32_t accum_bar = bar0 + 8u * (2 * S);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 1);
  // [0] some role gave up a wait; [1] never set (for waits that must not be cut short);
  // [3] thread 0's verdict for the producer warps: accumulator ready
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  auto stage_xhi = [&](int s) { return smem + (size_t)s * stage_bytes; };
  auto stage_xlo = [&](int s) { return smem + (size_t)s * stage_bytes + xbytes; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * TC_BM, m0 = blockIdx.y * bnx;
  const int kc0 = blockIdx.z * a.cps;
  const int num_k = min(a.K / TC_BK - kc0, a.cps);  // chunks of this CTA: [kc0, kc0 + num_k)

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full(s), 5);
      mbar_init(empty(s), 1);
    }
    mbar_init(accum_bar, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    abort_flag[2] = 0;
    abort_flag[3] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The packed weights do not depend on the preceding kernel: the producers start streaming them
  // at once.  Only the activation loads and the epilogue (residual reads, output / partial-tile
  // writes) wait for it.
  pdl_launch_dependents();

  if (warp < GROUPS * 4) {
    // ---------------- weight producers ----------------
    // Warps run independently.  For its chunk a warp's lane 0 polls the stage's `empty` mbarrier,
    // the warp converts its 32 rows and writes them to the stage's TMEM columns, and lane 0
    // arrives on `full`.  A group that is ahead starts on its next stage while the MMAs of
    // earlier chunks run, so conversion, barrier latency and the MMAs overlap.
    const int g = warp >> 2, quad = warp & 3;
    const int64_t row = (int64_t)n0 + quad * 32 + lane;
    const bool row_ok = row < a.N;
    const uint32_t t_quad = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)TC_WCOL0;
    // An mbarrier wait tells two consecutive phases apart and no more, so a group must not skip
    // a phase of a stage's `empty` barrier: with S stages at most S groups take chunks (then a
    // group's previous wait guarantees that its stage is at most one phase behind).
    const int ga = S < GROUPS ? S : GROUPS;
    if (WT == WT_F32_T) pdl_wait();  // this "weight" is an ordinary activation: another kernel may have just written it
    WRow<WT> ring[DEPTH];
#pragma unroll
    for (int j = 0; j < DEPTH; ++j)
      if (g < ga && j * ga + g < num_k) ring[j].load(a, row, row_ok, kc0 + j * ga + g);
    int s = g;
    uint32_t ph = 0;
    bool alive = g < ga;
    // ring[0] is always the chunk being converted: after each chunk the ring shifts down by one
    // (a few register moves) and the new load goes to the last slot, so the conversion code
    // exists once in the kernel instead of once per slot (a launch starts with a cold
    // instruction cache, and this loop is most of the kernel's code).
    int pmk = 0;
    (void)pmk;
    for (int kc = g; kc < num_k && alive; kc += ga) {
      int got = 0;
      if (lane == 0) {
        got = mbar_wait(empty(s), ph ^ 1u, abort_flag) ? 1 : 0;
        if (!got && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 1; a.status[2] = kc; }
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        alive = false;
      } else {
        tc_fence_after();  // the MMAs that read this stage are complete (their commit fired `empty`)
        if (warp == 0 && lane == 0) TC_MARK(0, 10, pmk);
        ring[0].template store<NSPLIT>(t_quad + (uint32_t)s * WCOLS);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (warp == 0 && lane == 0) TC_MARK(0, 11, pmk);
        if (lane == 0) mbar_arrive(full(s));
#pragma unroll
        for (int j = 0; j + 1 < DEPTH; ++j) ring[j] = ring[j + 1];
        if (kc + DEPTH * ga < num_k) ring[DEPTH - 1].load(a, row, row_ok, kc0 + kc + DEPTH * ga);
        s += ga;
        while (s >= S) { s -= S; ph ^= 1u; }
      }
    }
    // ---------------- epilogue ----------------
    pdl_wait();
    if (tid == 0) {
      const bool got = !*abort_flag && mbar_wait(accum_bar, 0, abort_flag);
      if (!got && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 2; }
      abort_flag[3] = got ? 1 : 0;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NPROD) : "memory");
    if (abort_flag[3]) {
      tc_fence_after();
      const int64_t o = row;  // output feature of this thread
      const bool o_ok = row_ok;
      const float bias = (a.bias && o_ok) ? a.bias[o] : 0.0f;
      // the warps of a TMEM lane quadrant share the columns in groups of at least 16
      const int ngroups = bnx / 16 < GROUPS ? bnx / 16 : GROUPS, per_group = bnx / ngroups, cgroup = g;
      const int c_begin = cgroup * per_group, c_end = cgroup < ngroups ? c_begin + per_group : c_begin;
      const uint32_t trow = tmem_base + ((uint32_t)(quad * 32) << 16);
      for (int c = c_begin; c < c_end; c += 16) {
        uint32_t r[16];
        tmem_ld16(trow + (uint32_t)c, r);
        if (a.concat) {
          // columns [bnx, 2 bnx) hold the products with the low part of x
          uint32_t r2[16];
          tmem_ld16(trow + (uint32_t)(bnx + c), r2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
        } else {
          tmem_ld_wait();
        }
        if (a.splits == 1) {
          if (o_ok && m0 + c < a.M) {
            if (a.act == CATEN_B200_ACT_GELU) epi_store16<CATEN_B200_ACT_GELU>(a, r, bias, o, m0 + c);
            else if (a.act == CATEN_B200_ACT_RELU) epi_store16<CATEN_B200_ACT_RELU>(a, r, bias, o, m0 + c);
            else epi_store16<CATEN_B200_ACT_NONE>(a, r, bias, o, m0 + c);
          }
        } else if (a.cluster) {
          // partial tile -> this CTA's shared memory, [column][row]; the stage buffers are free now
          // (the accumulator barrier fired: every MMA has read them and every TMA copy has landed)
          float *stg = reinterpret_cast<float *>(smem) + quad * 32 + lane;
#pragma unroll
          for (int i = 0; i < 16; ++i) stg[(c + i) * TC_BM] = __uint_as_float(r[i]);
        } else {
          // partial tile -> part[split][tile][column][row]: a warp stores 128 contiguous bytes
          const int tiles = gridDim.x * gridDim.y, tile = blockIdx.y * gridDim.x + blockIdx.x;
          float *mine = a.part + ((size_t)blockIdx.z * tiles + tile) * bnx * TC_BM + quad * 32 + lane;
#pragma unroll
          for (int i = 0; i < 16; ++i) mine[(c + i) * TC_BM] = __uint_as_float(r[i]);
        }
      }
    }
    tc_fence_before();
  } else if (warp == TMA_WARP) {
    // ---------------- activation TMA producer ----------------
    if (lane == 0) {
      // the tensor maps are fetched while the preceding kernel still runs, not by the first copy after the wait
      tma_prefetch_map(&tm_hi);
      if (NSPLIT == 3) tma_prefetch_map(&tm_lo);
      pdl_wait();  // x is written by the preceding kernel
      int issued = 0, s = 0;
      uint32_t ph = 0;
      for (int kc = 0; kc < num_k; ++kc) {
        if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 3; a.status[2] = kc; }
          break;
        }
        mbar_expect_tx(full(s), stage_bytes);
        tma_load_2d(smem_u32(stage_xhi(s)), &tm_hi, full(s), (kc0 + kc) * TC_BK, m0);
        if (NSPLIT == 3) tma_load_2d(smem_u32(stage_xlo(s)), &tm_lo, full(s), (kc0 + kc) * TC_BK, m0);
        issued = kc + 1;
        if (++s == S) { s = 0; ph ^= 1u; }
      }
      if (*abort_flag) {
        // let the copies this thread started land before the CTA's shared memory is released
        for (int kc = issued > S ? issued - S : 0; kc < issued; ++kc)
          mbar_wait(full(kc % S), (uint32_t)(kc / S) & 1u, abort_flag + 1);
      }
    }
  } else {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loop (waits, descriptor arithmetic) in uniform control flow, so the
    // operands of tcgen05.mma can be computed once per warp; one elected lane issues the MMAs and
    // the commits.
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    const uint32_t t_w0 = tmem_base + (uint32_t)TC_WCOL0;
    const uint64_t dx0 = umma_desc(smem_u32(smem));  // descriptor of stage 0's x_hi tile
    const uint32_t stage16 = stage_bytes >> 4, xlo16 = xbytes >> 4;  // in descriptor address units
    // With few activation rows an MMA is short and this loop — one thread's chain of a barrier test, eight issues and
    // a commit, ~600 cycles per chunk — sets the pace of the K loop (the producers are 1.5-2 k cycles ahead); with 256
    // rows a chunk's twelve MMAs take 1.54 k cycles on the tensor pipe and hide it.
    int mk = 0;
    (void)mk;
    if (lane == 0) TC_MARK(2, 1, mk);
    for (int kc = 0; kc < num_k; ++kc) {
      ok = mbar_wait(full(s), ph, abort_flag);
      if (!ok) {
        if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT); a.status[1] = 4; a.status[2] = kc; }
        break;
      }
      tc_fence_after();
      const uint32_t a_hi = t_w0 + (uint32_t)s * WCOLS, a_lo = a_hi + 32u;
      const uint64_t dxh = dx0 + (uint64_t)((uint32_t)s * stage16), dxl = dxh + (uint64_t)xlo16;
      if (elect_one()) {
#pragma unroll
        for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
          const uint64_t adv = (uint64_t)(k4 * 2);  // 16 bf16 = 32 bytes = 2 descriptor units
          const uint32_t first = (kc > 0 || k4 > 0) ? 1u : 0u;
          if (NSPLIT == 3 && a.concat) {
            // B = [x_hi; x_lo] (2 bnx rows, adjacent in the stage): one MMA per weight part
            umma_bf16_ts(tmem_base, a_hi + 8u * k4, dxh + adv, a.idesc, first);
            umma_bf16_ts(tmem_base, a_lo + 8u * k4, dxh + adv, a.idesc, 1u);
          } else {
            umma_bf16_ts(tmem_base, a_hi + 8u * k4, dxh + adv, a.idesc, first);
            if (NSPLIT == 3) {
              umma_bf16_ts(tmem_base, a_lo + 8u * k4, dxh + adv, a.idesc, 1u);
              umma_bf16_ts(tmem_base, a_hi + 8u * k4, dxl + adv, a.idesc, 1u);
            }
          }
        }
        umma_commit(empty(s));  // frees the stage when these MMAs have read it
      }
      __syncwarp();
      if (lane == 0) TC_MARK(2, 22, mk);
      if (++s == S) { s = 0; ph ^= 1u; }
    }
    if (ok && elect_one()) umma_commit(accum_bar);
    __syncwarp();
  }
  __syncthreads();
  if (a.cluster) {
    // Split-K reduction inside the cluster.  Both cluster barriers are executed by every thread
    // of every CTA unconditionally (also after a timed-out wait), so no CTA can be left waiting.
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid < NPROD && abort_flag[3]) {
      const int rank = blockIdx.z, nsp = a.splits;
      const uint32_t stg0 = smem_u32(smem);
      const int mine = (bnx - rank + nsp - 1) / nsp;  // columns rank, rank + nsp, ... of the tile
      for (int item = tid; item < mine * 32; item += NPROD) {
        const int col = rank + (item >> 5) * nsp, r4 = (item & 31) * 4;
        const int64_t m = (int64_t)m0 + col;
        if (m >= a.M) continue;
        const uint32_t local = stg0 + (uint32_t)(col * TC_BM + r4) * 4u;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < nsp; ++z) {  // fixed order: the sum does not depend on timing
          uint32_t remote;
          float4 p;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(z));
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(p.x), "=f"(p.y), "=f"(p.z), "=f"(p.w) : "r"(remote) : "memory");
          v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        const float r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int64_t o = (int64_t)n0 + r4 + e;
          if (o < a.N) {
            float t = r[e];
            if (a.bias) t = t + a.bias[o];
            t = apply_act(t, a.act);
            if (a.res) t = a.res[m * a.N + o] + t;
            if (a.yhi) {
              const __nv_bfloat16 h = __float2bfloat16_rn(t);
              a.yhi[m * a.N + o] = h;
              if (a.ylo) a.ylo[m * a.N + o] = __float2bfloat16_rn(t - __bfloat162float(h));
            } else {
              a.y[m * a.N + o] = t;
            }
          }
        }
      }
    }
    // peers may still be reading this CTA's shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Sums the split-K partial tiles part[split][tile][column][row] in split order (so the result is
// the same on every run) and applies bias / activation / residual.  A thread owns four consecutive
// weight rows (one float4 per split, four splits in flight): partial reads and y stores are
// coalesced and the loads of different splits overlap.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ part, int splits, int tiles_x, int tiles,
                                                            int bnx, const float *__restrict__ bias, const float *res, float *y,
                                                            __nv_bfloat16 *yhi, __nv_bfloat16 *ylo, int act, int M, int N) {
  pdl_enter();
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int row = (int)(idx & 31) * 4;
  const int64_t rest = idx >> 5;
  const int col = (int)(rest % bnx), tile = (int)(rest / bnx);
  if (tile >= tiles) return;
  const int64_t o = (int64_t)(tile % tiles_x) * TC_BM + row, m = (int64_t)(tile / tiles_x) * bnx + col;
  if (o >= N || m >= M) return;
  const size_t zstride = (size_t)tiles * bnx * TC_BM;
  const float *p = part + ((size_t)tile * bnx + col) * TC_BM + row;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  int z = 0;
  for (; z + 4 <= splits; z += 4) {
    const float4 a0 = __ldcs(reinterpret_cast<const float4 *>(p + (size_t)z * zstride));
    const float4 a1 = __ldcs(reinterpret_cast<const float4 *>(p + (size_t)(z + 1) * zstride));
    const float4 a2 = __ldcs(reinterpret_cast<const float4 *>(p + (size_t)(z + 2) * zstride));
    const float4 a3 = __ldcs(reinterpret_cast<const float4 *>(p + (size_t)(z + 3) * zstride));
    v.x += a0.x; v.y += a0.y; v.z += a0.z; v.w += a0.w;
    v.x += a1.x; v.y += a1.y; v.z += a1.z; v.w += a1.w;
    v.x += a2.x; v.y += a2.y; v.z += a2.z; v.w += a2.w;
    v.x += a3.x; v.y += a3.y; v.z += a3.z; v.w += a3.w;
  }
  for (; z < splits; ++z) {
    const float4 a0 = __ldcs(reinterpret_cast<const float4 *>(p + (size_t)z * zstride));
    v.x += a0.x; v.y += a0.y; v.z += a0.z; v.w += a0.w;
  }
  float r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (o + e < N) {
      float t = r[e];
      if (bias) t = t + bias[o + e];
      t = apply_act(t, act);
      if (res) t = res[m * N + o + e] + t;
      if (yhi) {
        const __nv_bfloat16 h = __float2bfloat16_rn(t);
        yhi[m * N + o + e] = h;
        if (ylo) ylo[m * N + o + e] = __float2bfloat16_rn(t - __bfloat162float(h));
      } else {
        y[m * N + o + e] = t;
      }
    }
  }
}

// x -> bf16 hi (and lo) copies, row-major [M, K]
__global__ void split_bf16_kernel(const float4 *__restrict__ x, uint2 *__restrict__ hi, uint2 *__restrict__ lo, int64_t n4) {
  pdl_enter();
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
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(tc_threads<WT>());
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute at[2];
  int na = 0;
  if (take_pdl(ctx)) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (a.cluster) {  // the CTAs that share an output tile (same x, y; all z) are one cluster
    at[na].id = cudaLaunchAttributeClusterDimension;
    at[na].val.clusterDim.x = 1;
    at[na].val.clusterDim.y = 1;
    at[na].val.clusterDim.z = grid.z;
    ++na;
  }
  cfg.attrs = at;
  cfg.numAttrs = na;
  CB_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tc_kernel<WT, NSPLIT>, mh, ml, a));
  CB_LAUNCH_CHECK(ctx, "gemm_tc_kernel");
  return 0;
}

static int launch_tc(caten_b200_ctx *ctx, int wt, int nsplit, const CUtensorMap &mh, const CUtensorMap &ml, const TcArgs &a, dim3 grid,
                     size_t smem) {
#define TC_CASE(WT) \
  case WT: return nsplit == 3 ? launch_tc_t<WT, 3>(ctx, mh, ml, a, grid, smem) : launch_tc_t<WT, 1>(ctx, mh, ml, a, grid, smem)
  switch (wt) {
    TC_CASE(CATEN_B200_F32);
    TC_CASE(CATEN_B200_F16);
    TC_CASE(CATEN_B200_Q4_0);
    TC_CASE(CATEN_B200_Q4_1);
    TC_CASE(CATEN_B200_Q5_0);
    TC_CASE(CATEN_B200_Q5_1);
    TC_CASE(CATEN_B200_Q8_0);
    TC_CASE(WT_F32_T);
    default: return fail(ctx, CATEN_B200_EUNSUPPORTED, "gemm_tc: weight type %d", wt);
  }
#undef TC_CASE
}

// Tile shape, pipeline depth and split-K factor of one launch.
struct TcPlan {
  int bnx, stages, splits, cps, concat;
  uint32_t idesc;
  int64_t gx, gy, tiles;
  size_t stage_bytes;
};

static int tc_plan(caten_b200_ctx *ctx, const char *who, int64_t M, int64_t N, int64_t K, int nsplit, int split_cap, TcPlan *p) {
  if (!ctx->encode_tiled) return fail(ctx, CATEN_B200_ECUDA, "%s: cuTensorMapEncodeTiled is not available", who);
  if (K % TC_BK) return fail(ctx, CATEN_B200_EUNSUPPORTED, "%s: inner dimension %lld is not a multiple of 64", who, (long long)K);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "%s: dimension too large", who);
  if (nsplit != 1 && nsplit != 3) return fail(ctx, CATEN_B200_EINVAL, "%s: nsplit must be 1 or 3", who);
  int bnx = 16;
  while (bnx < 256 && bnx < M) bnx *= 2;
  p->bnx = bnx;
  p->concat = (nsplit == 3 && bnx <= 128) ? 1 : 0;
  const int mma_n = p->concat ? 2 * bnx : bnx;
  p->idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
  p->stage_bytes = (size_t)bnx * 128 * (nsplit == 3 ? 2 : 1);
  p->gy = (M + bnx - 1) / bnx;
  if (p->gy > 65535) return fail(ctx, CATEN_B200_EUNSUPPORTED, "%s: too many rows for one launch (%lld)", who, (long long)M);
  p->gx = (N + TC_BM - 1) / TC_BM;
  p->tiles = p->gx * p->gy;
  // split-K when the output tiles alone cannot occupy the GPU (decode: few activation rows)
  const int num_k = (int)(K / TC_BK);
  int splits = 1;
  if (p->tiles < ctx->sm_count) {
    const int by_work = num_k / 4 > 0 ? num_k / 4 : 1;        // at least 4 chunks per CTA (2 or 1 measured no faster)
    const int by_fill = (int)(ctx->sm_count / p->tiles);      // one wave: every CTA resident at once
    splits = by_work < by_fill ? by_work : by_fill;
    if (splits > split_cap) splits = split_cap;
  }
  p->cps = (num_k + splits - 1) / splits;
  p->splits = (num_k + p->cps - 1) / p->cps;
  // ring depth: weight stages in TMEM (256 columns), activation stages in shared memory
  int stages = nsplit == 3 ? 4 : 8;
  if ((size_t)stages * p->stage_bytes > 200 * 1024) stages = (int)((200 * 1024) / p->stage_bytes);
  if (stages > p->cps) stages = p->cps;
  if (stages < 1) stages = 1;
  p->stages = stages;
  return 0;
}

static WSrc wsrc_of(const caten_b200_weight *w) { return WSrc{w->qs, w->d, w->m, w->qh, w->nkb}; }

static int run_tc(caten_b200_ctx *ctx, int wt, const WSrc &ws, const float *x,
                  const float *bias, const float *res, int act, float *y, int64_t M, int64_t N, int64_t K, int nsplit,
                  const __nv_bfloat16 *xhi_pre = nullptr, const __nv_bfloat16 *xlo_pre = nullptr, BfOut ybf = BfOut(),
                  PartIn *defer = nullptr) {
  if (defer) *defer = PartIn();
  if (M <= 0 || N <= 0) return 0;
  // thousands of rows (prefill): expand the weights once, both operands through TMA
  // (its epilogue moves 16 bytes at a time: bias, residual and outputs must be aligned for that)
  const uintptr_t align_bits = (uintptr_t)bias | (uintptr_t)res | (uintptr_t)y | (uintptr_t)ybf.hi | (uintptr_t)ybf.lo;
  if (gemm_dense_applies(ctx, M, N, K) && !(align_bits & 15)) return launch_gemm_dense(ctx, wt, ws, x, xhi_pre, xlo_pre, bias, res, act, y, ybf, M, N, K, nsplit);
  TcPlan p;
  // reduce inside a cluster: always (mode 1) or only when this launch needs its own epilogue (mode 2)
  const bool own_epilogue = !(defer && act == CATEN_B200_ACT_NONE && !ybf.hi && N % 4 == 0);
  const bool want_cluster = ctx->splitk_cluster == 1 || (ctx->splitk_cluster == 2 && own_epilogue);
  if (int rc = tc_plan(ctx, "gemm_tc", M, N, K, nsplit, want_cluster ? 8 : 32, &p)) return rc;  // 8 = portable cluster size
  uint8_t *xhi, *xlo;
  if (xhi_pre) {
    // the producer of x already wrote the split bf16 operand
    if (nsplit == 3 && !xlo_pre) return fail(ctx, CATEN_B200_EINVAL, "gemm_tc: split-bf16 needs the lo part of x");
    if (((uintptr_t)xhi_pre | (uintptr_t)xlo_pre) & 15) return fail(ctx, CATEN_B200_EINVAL, "gemm_tc: bf16 operand must be 16-byte aligned");
    xhi = (uint8_t *)xhi_pre;
    xlo = (uint8_t *)xlo_pre;
  } else {
    // activations -> bf16 (hi[, lo]) in the context's scratch buffer
    const size_t xb = (size_t)M * K * 2;
    const size_t xb_al = (xb + 1023) & ~(size_t)1023;
    if (int rc = scratch_reserve(ctx, &ctx->xbf, xb_al * (nsplit == 3 ? 2 : 1))) return rc;
    xhi = (uint8_t *)ctx->xbf.ptr;
    xlo = nsplit == 3 ? xhi + xb_al : nullptr;
    const int64_t n4 = M * K / 4;
    launch_k(ctx, split_bf16_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, (const float4 *)x, (uint2 *)xhi, (uint2 *)xlo, n4);
    CB_LAUNCH_CHECK(ctx, "split_bf16_kernel");
  }
  CUtensorMap mh, ml;
  if (int rc = make_x_map(ctx, &mh, xhi, M, K, p.bnx)) return rc;
  if (int rc = make_x_map(ctx, &ml, nsplit == 3 ? xlo : xhi, M, K, p.bnx)) return rc;

  TcArgs a;
  a.qs = ws.qs; a.d = ws.d; a.m = ws.m; a.qh = ws.qh; a.bias = bias; a.res = res; a.y = y; a.status = ctx->d_status; a.act = act;
  a.yhi = ybf.hi; a.ylo = ybf.lo;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.nkb = (int)ws.nkb; a.bnx = p.bnx;
  a.stages = p.stages; a.idesc = p.idesc; a.concat = p.concat;
  a.splits = p.splits; a.cps = p.cps; a.part = nullptr;
  a.cluster = (p.splits > 1 && want_cluster) ? 1 : 0;
  if (p.splits > 1 && !a.cluster) {
    if (int rc = scratch_reserve(ctx, &ctx->wtmp, (size_t)p.splits * p.tiles * p.bnx * TC_BM * sizeof(float))) return rc;
    a.part = (float *)ctx->wtmp.ptr;
  }
  // 1 KB alignment slack + 1 KB bookkeeping + the activation ring (which the split-K staging tile reuses)
  size_t ring = p.stage_bytes * (size_t)p.stages;
  if (a.cluster && ring < (size_t)p.bnx * TC_BM * sizeof(float)) ring = (size_t)p.bnx * TC_BM * sizeof(float);
  const size_t smem = 2048 + ring;
  const dim3 grid((unsigned)p.gx, (unsigned)p.gy, (unsigned)p.splits);
  const int rc = launch_tc(ctx, wt, nsplit, mh, ml, a, grid, smem);
  if (rc || p.splits == 1 || a.cluster) return rc;
  if (defer && act == CATEN_B200_ACT_NONE && !a.yhi && N % 4 == 0) {
    // the consumer of this linear sums the partial tiles itself (and adds bias / residual)
    defer->part = a.part; defer->bias = bias; defer->splits = p.splits; defer->tiles_x = (int)p.gx; defer->bnx = p.bnx;
    defer->zstride = (long long)p.tiles * p.bnx * TC_BM;
    return 0;
  }
  const int64_t total = p.tiles * p.bnx * (TC_BM / 4);
  launch_k(ctx, splitk_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, a.part, p.splits, (int)p.gx, (int)p.tiles, p.bnx, bias,
                                                                              res, y, a.yhi, a.ylo, act, (int)M, (int)N);
  CB_LAUNCH_CHECK(ctx, "splitk_reduce_kernel");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that must not allocate: the same kernels, with the bf16 copy of the
// activations and the split-K partial tiles placed in a buffer that is part of the library image
// instead of a grow-on-demand cudaMalloc.  Every GPU that loads the library holds the buffer
// until the process exits.
// ---------------------------------------------------------------------------------------------
constexpr size_t FIXED_SCRATCH_BYTES = (size_t)32 << 20;  // 32 MiB
static __device__ __align__(256) unsigned char g_fixed_scratch[FIXED_SCRATCH_BYTES];

// The array's name is only a stand-in on the host; its device address is looked up once per
// device (with that device current) and cached.
static int fixed_scratch_ptr(caten_b200_ctx *ctx, uint8_t **out) {
  static std::atomic<uint8_t *> cached[64];  // zero-initialised; host threads of different contexts may race here
  if (ctx->device < 0 || ctx->device >= 64) return fail(ctx, CATEN_B200_EUNSUPPORTED, "linear_noalloc: device index %d", ctx->device);
  uint8_t *have = cached[ctx->device].load(std::memory_order_acquire);
  if (!have) {
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_fixed_scratch);  // the same address whoever asks first
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaGetSymbolAddress(g_fixed_scratch)");
    have = (uint8_t *)p;
    cached[ctx->device].store(have, std::memory_order_release);
  }
  *out = have;
  return 0;
}

int launch_gemm_tc_noalloc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                           const float *res, int act, float *y, int64_t M, int nsplit) {
  const int64_t N = w->rows, K = w->cols;
  if (M <= 0 || N <= 0) return 0;
  TcPlan p;
  if (int rc = tc_plan(ctx, "linear_noalloc", M, N, K, nsplit, 32, &p)) return rc;
  uint8_t *base = nullptr;
  if (int rc = fixed_scratch_ptr(ctx, &base)) return rc;

  // layout of the fixed buffer: [x_hi | x_lo (split-bf16 only) | split-K partial tiles]
  const size_t xb_al = ((size_t)M * K * 2 + 1023) & ~(size_t)1023;
  const size_t x_total = xb_al * (nsplit == 3 ? 2 : 1);
  const size_t part_bytes = p.splits > 1 ? (size_t)p.splits * p.tiles * p.bnx * TC_BM * sizeof(float) : 0;
  if (x_total + part_bytes > FIXED_SCRATCH_BYTES)
    return fail(ctx, CATEN_B200_EUNSUPPORTED,
                "linear_noalloc: M=%lld x %lldx%lld needs %zu bytes of scratch, the built-in buffer holds %zu; use caten_b200_linear",
                (long long)M, (long long)N, (long long)K, x_total + part_bytes, FIXED_SCRATCH_BYTES);
  uint8_t *xhi = base, *xlo = nsplit == 3 ? base + xb_al : nullptr;
  // nothing in the buffer has to start at zero: the used part of x_hi/x_lo and every partial tile
  // that the reduce reads are fully overwritten by this call before they are read
  const int64_t n4 = M * K / 4;
  launch_k(ctx, split_bf16_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, (const float4 *)x, (uint2 *)xhi, (uint2 *)xlo, n4);
  CB_LAUNCH_CHECK(ctx, "split_bf16_kernel");
  CUtensorMap mh, ml;
  if (int rc = make_x_map(ctx, &mh, xhi, M, K, p.bnx)) return rc;
  if (int rc = make_x_map(ctx, &ml, nsplit == 3 ? xlo : xhi, M, K, p.bnx)) return rc;

  TcArgs a;
  a.qs = w->qs; a.d = w->d; a.m = w->m; a.qh = w->qh; a.bias = bias; a.res = res; a.y = y; a.status = ctx->d_status; a.act = act;
  a.yhi = nullptr; a.ylo = nullptr;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.nkb = (int)w->nkb; a.bnx = p.bnx;
  a.stages = p.stages; a.idesc = p.idesc; a.concat = p.concat;
  a.splits = p.splits; a.cps = p.cps; a.cluster = 0;  // partial tiles go through the fixed buffer
  a.part = p.splits > 1 ? (float *)(base + x_total) : nullptr;
  const size_t smem = 2048 + p.stage_bytes * (size_t)p.stages;
  const dim3 grid((unsigned)p.gx, (unsigned)p.gy, (unsigned)p.splits);
  const int rc = launch_tc(ctx, w->type, nsplit, mh, ml, a, grid, smem);
  if (rc || p.splits == 1) return rc;
  const int64_t total = p.tiles * p.bnx * (TC_BM / 4);
  launch_k(ctx, splitk_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, a.part, p.splits, (int)p.gx, (int)p.tiles, p.bnx, bias,
                                                                              res, y, a.yhi, a.ylo, act, (int)M, (int)N);
  CB_LAUNCH_CHECK(ctx, "splitk_reduce_kernel");
  return 0;
}

int launch_gemm_tc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                   const float *res, int act, float *y, int64_t M, int nsplit) {
  return run_tc(ctx, w->type, wsrc_of(w), x, bias, res, act, y, M, w->rows, w->cols, nsplit);
}

int launch_gemm_tc_ex(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const __nv_bfloat16 *xhi,
                      const __nv_bfloat16 *xlo, const float *bias, const float *res, int act, float *y, BfOut ybf, int64_t M,
                      int nsplit, PartIn *defer) {
  return run_tc(ctx, w->type, wsrc_of(w), x, bias, res, act, y, M, w->rows, w->cols, nsplit, xhi, xlo, ybf, defer);
}

int launch_relu_matmul_tc(caten_b200_ctx *ctx, const float *a, const float *b, float *c, int64_t M, int64_t K, int64_t N, int nsplit) {
  return run_tc(ctx, WT_F32_T, WSrc{b, nullptr, nullptr, nullptr, 0}, a, nullptr, nullptr, CATEN_B200_ACT_RELU, c, M, N, K, nsplit);
}

}  // namespace cb

#ifdef DS_TIMING
extern "C" int cb_debug_tc_marks(long long *out, int *n) {
  cudaMemcpyFromSymbol(n, cb::g_tc_marks_n, sizeof(int) * 3);
  return (int)cudaMemcpyFromSymbol(out, cb::g_tc_marks, sizeof(long long) * 3 * 256 * 2);
}
#endif
