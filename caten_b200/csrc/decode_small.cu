// One kernel per token for decode with 1..4 sequences (external/llm/layers.lisp:81-90 with s = 1):
// embedding, every Transformer block, ln_f, lm_head and the arg-max in a single launch of one
// CTA per SM.
//
// Why.  With a handful of sequences every Linear is a dequant-GEMV over a matrix of 0.6..6 MB:
// 0.1..0.9 us of HBM time each.  As separate launches (7 per block) a step is a chain of several
// hundred kernels of 4..8 us whose cost is launch and first-load latency, not bandwidth.  Here
// the chain stays, but its links are cheap:
//
//  * Weights never wait.  A feeder warp streams this CTA's share of every matrix, in step order,
//    into a ring of shared-memory slots with bulk async copies (cp.async.bulk + mbarrier), up to
//    the whole ring (~190 KB per SM) ahead of the arithmetic and independent of any activation.
//  * Activations travel between CTAs as (value, step tag) pairs in 8-byte words written with one
//    64-bit store and read with 64-bit loads.  A consumer polls the words it needs until they
//    carry the tag of the current step; data and "ready" flag are the same word, so a hand-off
//    costs one store and one load through L2 instead of store + fence + flag + load, and there
//    is no grid-wide barrier anywhere.  Every exchange buffer is written once per step (one per
//    layer and kind), so no slot is reused inside a launch; the kernel boundary orders reuse
//    across steps.
//  * Everything a phase needs that does not depend on the exchanged vector (LayerNorm gamma and
//    beta, the biases of the CTA's rows, the K and V rows of an attention chunk) is requested
//    BEFORE the poll, so those loads fly while the CTA waits for its input.
//  * LayerNorm is recomputed by every CTA from the exchanged vector (d <= 2400 values), GELU,
//    bias and residual live in the GEMV epilogues, attention is split over the context so that
//    B x H x C work items fill the SMs, followed by a small combine.
//  * Nothing lives in local memory: with ~220 KB of the SM's 256 KB carved out as shared memory
//    the L1 that would back a stack is tiny, and a spilled value costs an L2 round trip.  Layer
//    descriptors are copied to shared memory once; shared-memory regions are addressed as
//    base + offset taken from the parameter block.
//
// Phases of a block (each ends in tagged stores, the next begins with a poll):
//   P1 ln_1 + c_attn -> qkv      P2 attention partials over context chunks (+ cache append)
//   P3 combine -> att            P4 attn.c_proj + bias + residual -> h2
//   P5 ln_2 + c_fc + GELU -> ff  P6 mlp.c_proj + bias + residual -> h
// then ln_f + lm_head -> logits, per-CTA arg-max candidates -> CTA 0 picks the lowest index of
// the maximum (api/high-level-ops.lisp:314-343), stores the ids and advances position and tag.
//
// All CTAs must be resident at once (they wait for each other's words): the launch is
// cooperative with one CTA per SM.  Every poll and every mbarrier wait is bounded; when one runs
// out the CTA records it in the context's status word, stops requesting weights, waits for the
// bulk copies it has in flight and returns, and the other CTAs run into their own bounds and do
// the same.
#include "common.cuh"
#include "gemv_blocks.cuh"
#include "tcgen05.cuh"

namespace cb {

constexpr int DS_COMPUTE = 480;                 // compute threads (15 warps)
constexpr int DS_THREADS = 512;                 // + the feeder warp: 16 warps, 4 per scheduler, 128 registers each
constexpr int DS_CWARPS = DS_COMPUTE / 32;
constexpr int DS_HALFWARPS = DS_COMPUTE / 16;   // attention: one cache row (64 floats) per half-warp
constexpr int DS_SLOT = 32 * 1024;              // bytes of one ring slot
constexpr int DS_MAX_SLOTS = 6;
constexpr int DS_MAX_B = 4;
constexpr int DS_SLOT_BLOCKS = DS_SLOT / 18 + 1; // most 32-wide blocks one slot can hold (Q4_0: 16 B of codes + 2 B of scale each)
constexpr int DS_MAX_CHUNKS = 32;               // most context chunks per (sequence, head)
constexpr int DS_MISC_FLOATS = 192 + DS_HALFWARPS * 64 + 64;   // q, k, v rows | half-warp partial outputs | two reduction scratch rows
constexpr uint32_t DS_POLL_LIMIT = 1u << 21;    // polls (one L2 round trip each) before giving up: about a second
constexpr float kDsInvLn2 = 1.0f / 0.6931472f;  // (/ (log 2)) in single float, api/function.lisp:437-440

struct DsMatrix {
  const void *qs;      // codes (Q4_0: 16 B / block, Q8_0: 32 B / block) or the fp16 / fp32 matrix
  const __half *d;     // per-block scales, quantised types only
  const float *bias;   // [N] or null
  int type, N, K, nkb;
  int crb, rps;        // bytes of one row of codes; rows of one ring slot
};

struct DsLayer {
  DsMatrix attn, proj, fc, mproj;
  const float *ln1_g, *ln1_b, *ln2_g, *ln2_b;
  float *kc, *vc;      // [B, H, T, 64]
};

struct DsArgs {
  const DsLayer *layers;   // device array [L + 1]; entry L holds lm_head in .attn and ln_f in ln1_g / ln1_b
  const float *wte, *wpe;
  int L, d, H, V, T, B;
  float eps;
  int64_t *ids_io, *out_ids, *hist;   // [B], [B], [T, B]
  int *d_pos;
  unsigned *d_epoch;                  // step tag; starts at 1, the exchange buffers start zeroed
  float *logits;                      // [B, V]
  unsigned long long *xchg;           // tagged exchange words
  long long per_layer_words;
  int *status;
  int nslots, sc_floats, hres_rows, red_floats;
  // byte offsets of the shared-memory regions behind the ring, and word offsets of the exchange sections of a layer
  int off_desc, off_xs, off_red, off_sc, off_hres, off_bias, off_best, off_misc, off_bars, off_flags;
  long long lay_part, lay_att, lay_h2, lay_ff, lay_h;
};

// Exchange words of one layer, in the order they are produced.  One helper for host and device
// so that both agree on the offsets.
struct DsLayout {
  size_t qkv, part, att, h2, ff, h, per_layer;
};
__host__ __device__ inline DsLayout ds_layout(int B, int d, int G, int BH) {
  DsLayout o;
  const size_t items = (size_t)(G > BH ? G : BH);   // B x H x C work items never exceed this (C <= max(1, G / BH))
  o.qkv = 0;
  o.part = o.qkv + (size_t)B * 3 * d;
  o.att = o.part + items * 66;
  o.h2 = o.att + (size_t)B * d;
  o.ff = o.h2 + (size_t)B * d;
  o.h = o.ff + (size_t)B * 4 * d;
  o.per_layer = o.h + (size_t)B * d;
  return o;
}

// Optional per-phase timestamps of one CTA (development builds only: -DDS_TIMING -DDS_TIMING_CTA=n),
// read back with cb_debug_ds_times().
#ifdef DS_TIMING
__device__ unsigned long long g_ds_times[8192];
__device__ __forceinline__ void ds_mark(int &k) {
  if (blockIdx.x == DS_TIMING_CTA && threadIdx.x == 0 && k < 8192) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_ds_times[k] = t;
  }
  ++k;
}
#define DS_MARK() ds_mark(mark_k)
// finer marks (SM cycle counter) inside the building blocks of layer DS_FINE_LAYER
__device__ long long g_ds_fine[512];
__device__ int ds_fine_on;
__device__ int g_ds_fine_n;
// (the mark counter and the on/off switch live in shared memory, flags[4] and flags[5]: a global-memory counter would add an L2 round trip to every mark)
#define DS_FINE(id) do { if (blockIdx.x == DS_TIMING_CTA && threadIdx.x == 0 && sm.flags()[5]) { const int k_ = sm.flags()[4]; if (k_ < 255) { g_ds_fine[2 * k_] = (id); g_ds_fine[2 * k_ + 1] = clock64(); sm.flags()[4] = k_ + 1; g_ds_fine_n = k_ + 1; } } } while (0)
#else
#define DS_MARK() do { } while (0)
#define DS_FINE(id) do { } while (0)
#endif

// ---- tagged words ---------------------------------------------------------------------------------
__device__ __forceinline__ void st_tag(unsigned long long *p, float v, unsigned tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void st_tag_bits(unsigned long long *p, unsigned bits, unsigned tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)bits;
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word(const unsigned long long *p) {
  unsigned long long w;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
__device__ __forceinline__ void ld_word2(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
  asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// position of activation k inside the block-swizzled vector: thread kb reads its 8 float4 without
// bank conflicts against its neighbours (float4 q of block kb sits at slot q ^ (kb & 7))
__device__ __forceinline__ int swz(int k) {
  const int kb = k >> 5, j = k & 31;
  return (kb << 5) + ((((j >> 2) ^ (kb & 7)) << 2) | (j & 3));
}

// first row of CTA `cta` when N rows are cut into G nearly equal runs (N * G < 2^31 is checked by the host)
__device__ __forceinline__ int row_begin(int N, int cta, int G) { return (int)(((unsigned)N * (unsigned)cta) / (unsigned)G); }

__device__ __forceinline__ bool has_scales(int type) { return type == CATEN_B200_Q4_0 || type == CATEN_B200_Q8_0; }

// ---- shared memory -----------------------------------------------------------------------------------
struct Smem {
  uint8_t *base;
  const DsArgs &a;
  __device__ __forceinline__ Smem(uint8_t *b, const DsArgs &args) : base(b), a(args) {}
  __device__ __forceinline__ uint8_t *ring(int slot) const { return base + (size_t)slot * DS_SLOT; }
  __device__ __forceinline__ const DsLayer *layer(int l) const { return reinterpret_cast<const DsLayer *>(base + a.off_desc) + l; }
  __device__ __forceinline__ float *xs() const { return reinterpret_cast<float *>(base + a.off_xs); }
  __device__ __forceinline__ float *red(int buf) const { return reinterpret_cast<float *>(base + a.off_red) + (size_t)buf * a.red_floats; }
  __device__ __forceinline__ float *sc() const { return reinterpret_cast<float *>(base + a.off_sc); }
  __device__ __forceinline__ float *hres(int which) const { return reinterpret_cast<float *>(base + a.off_hres) + (size_t)which * a.B * a.hres_rows; }
  __device__ __forceinline__ float *bias(int which) const { return reinterpret_cast<float *>(base + a.off_bias) + which * DS_COMPUTE; }   // biases of this CTA's rows, two phases
  __device__ __forceinline__ float *misc() const { return reinterpret_cast<float *>(base + a.off_misc); }
  __device__ __forceinline__ float *scratch(int which) const { return misc() + 192 + DS_HALFWARPS * 64 + 32 * which; }
  __device__ __forceinline__ float *best_v() const { return reinterpret_cast<float *>(base + a.off_best); }          // [16 warps][4]
  __device__ __forceinline__ int *best_i() const { return reinterpret_cast<int *>(base + a.off_best) + 64; }          // [16 warps][4]
  __device__ __forceinline__ uint32_t full(int slot) const { return smem_u32(base + a.off_bars) + 8u * (uint32_t)slot; }
  __device__ __forceinline__ uint32_t empty(int slot) const { return smem_u32(base + a.off_bars) + 8u * (uint32_t)(DS_MAX_SLOTS + slot); }
  __device__ __forceinline__ volatile int *flags() const { return reinterpret_cast<volatile int *>(base + a.off_flags); } // [0] abort
};

__device__ __forceinline__ const DsMatrix &layer_matrix(const DsLayer *ly, int ph) {
  return ph == 0 ? ly->attn : ph == 1 ? ly->proj : ph == 2 ? ly->fc : ly->mproj;
}

// Gives up: records the first failure in the context's status word and raises the CTA's abort flag.
__device__ __forceinline__ void ds_fail(const DsArgs &a, volatile int *flags, int site, int detail) {
  if (!flags[0]) {
    flags[0] = 1;
    if (atomicCAS(a.status, 0, DEV_WAIT_TIMEOUT) == 0) { a.status[1] = 100 + site; a.status[2] = detail; a.status[3] = (int)blockIdx.x; }
  }
}

// Polls n (even) consecutive tagged words until all carry `tag` and hands each value to `sink(index, value)`.
// Up to 4 pairs per thread are in flight at once; compute threads only.
template <class Sink>
__device__ __forceinline__ void poll_words(const DsArgs &a, volatile int *flags, const unsigned long long *src, int n, unsigned tag, int site,
                                           Sink sink) {
  const int tid = threadIdx.x, np = n >> 1;
  for (int base = 0; base < np; base += 4 * DS_COMPUTE) {
    unsigned long long va[4], vb[4];
    unsigned pending = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = base + i * DS_COMPUTE + tid;
      if (p < np) {
        ld_word2(src + 2 * (long long)p, va[i], vb[i]);
        if ((unsigned)(va[i] >> 32) != tag || (unsigned)(vb[i] >> 32) != tag) pending |= 1u << i;
      }
    }
    uint32_t spins = 0;
    while (pending) {
      if (++spins > DS_POLL_LIMIT || ((spins & 255u) == 0 && (flags[0] || ((spins & 4095u) == 0 && *(volatile int *)a.status != 0)))) {
        ds_fail(a, flags, site, base);
        break;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (pending & (1u << i)) {
          const int p = base + i * DS_COMPUTE + tid;
          ld_word2(src + 2 * (long long)p, va[i], vb[i]);
          if ((unsigned)(va[i] >> 32) == tag && (unsigned)(vb[i] >> 32) == tag) pending &= ~(1u << i);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = base + i * DS_COMPUTE + tid;
      if (p < np) {
        sink(2 * p, __uint_as_float((unsigned)va[i]));
        sink(2 * p + 1, __uint_as_float((unsigned)vb[i]));
      }
    }
  }
}

// one tagged word, polled by the calling thread
__device__ __forceinline__ unsigned poll_one(const DsArgs &a, volatile int *flags, const unsigned long long *src, unsigned tag, int site) {
  unsigned long long w = ld_word(src);
  uint32_t spins = 0;
  while ((unsigned)(w >> 32) != tag) {
    if (++spins > DS_POLL_LIMIT || ((spins & 255u) == 0 && (flags[0] || ((spins & 4095u) == 0 && *(volatile int *)a.status != 0)))) {
      ds_fail(a, flags, site, 0);
      break;
    }
    w = ld_word(src);
  }
  return (unsigned)w;
}

// barrier over the compute threads (named barrier 1: the feeder warp does not take part)
__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, %0;" ::"n"(DS_COMPUTE) : "memory"); }

// Barrier that also answers "has anyone given up?" with the SAME answer in every compute thread:
// control flow that decides which barriers a thread will reach must only depend on this, never on a
// plain read of the flag (which another warp may be setting at that moment).
__device__ __forceinline__ bool abort_uniform(volatile int *flags) {
  uint32_t r;
  const uint32_t mine = flags[0] ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(mine), "n"(DS_COMPUTE)
      : "memory");
  return r != 0;
}

// Block reductions with ONE barrier each: callers alternate between the two scratch rows, so a row is
// rewritten only after another barrier has passed since it was last read.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  bar_compute();
  float t = scratch[0];
#pragma unroll
  for (int w = 1; w < DS_CWARPS; ++w) t += scratch[w];
  return t;
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  bar_compute();
  float t = scratch[0];
#pragma unroll
  for (int w = 1; w < DS_CWARPS; ++w) t = fmaxf(t, scratch[w]);
  return t;
}

enum { EPI_QKV = 0, EPI_PROJ = 1, EPI_FC = 2, EPI_MPROJ = 3, EPI_LM = 4 };

// ---- feeder warp (lane 0): the bulk copies of every chunk of the step, in consumption order ------------
// layers 0..L-1 x (c_attn, attn.c_proj, c_fc, mlp.c_proj), then lm_head; within a matrix this CTA's rows
// in runs of `rps`.  Chunk i uses slot i % nslots and completes phase (i / nslots) & 1 of its `full`
// mbarrier; a slot is refilled after the compute threads released it through `empty`.
__device__ __forceinline__ void feeder(const DsArgs &a, const Smem &sm) {
  const int G = gridDim.x, cta = blockIdx.x, nslots = a.nslots;
  volatile int *flags = sm.flags();
  int slot = 0, issued = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int l = 0; l <= a.L && ok; ++l) {
    const DsLayer *ly = sm.layer(l);
    for (int ph = 0; ph < (l == a.L ? 1 : 4) && ok; ++ph) {
      const DsMatrix &m = layer_matrix(ly, ph);
      const int r0 = row_begin(m.N, cta, G), r1 = row_begin(m.N, cta + 1, G);
      const int crb = m.crb, rps = m.rps, nkb = m.nkb;
      const bool quant = has_scales(m.type);
      const uint8_t *qs = (const uint8_t *)m.qs, *sd = (const uint8_t *)m.d;
      for (int c0 = r0; c0 < r1; c0 += rps) {
        const int c1 = min(c0 + rps, r1);
        if (!mbar_wait(sm.empty(slot), phase ^ 1u, flags)) { ds_fail(a, flags, 1, c0); ok = false; break; }
        const uint32_t full = sm.full(slot), dst = smem_u32(sm.ring(slot));
        const uint32_t cbytes = (uint32_t)(c1 - c0) * (uint32_t)crb;
        uint32_t sbytes = 0;
        long long sb0 = 0;
        if (quant) {
          sb0 = ((long long)c0 * nkb * 2) & ~15ll;
          sbytes = (uint32_t)((((long long)c1 * nkb * 2 + 15) & ~15ll) - sb0);
        }
        mbar_expect_tx(full, cbytes + sbytes);
        bulk_g2s(dst, qs + (long long)c0 * crb, cbytes, full);
        if (sbytes) bulk_g2s(dst + cbytes, sd + sb0, sbytes, full);
        ++issued;
        if (++slot == nslots) { slot = 0; phase ^= 1u; }
      }
    }
  }
  if (!ok) {
    // the compute warps stopped consuming: let the copies already requested land before the CTA's
    // shared memory is released (a wait on a completed phase returns at once; each wait is bounded)
    volatile int never = 0;
    for (int s = 0; s < nslots; ++s) {
      const int lasti = issued - 1 - ((issued - 1 - s) % nslots + nslots) % nslots;  // last chunk that used slot s
      if (lasti >= 0) mbar_wait(sm.full(s), (uint32_t)(lasti / nslots) & 1u, &never);
    }
  }
}

// ---- one GEMV phase over the CTA's rows, x already in xs ---------------------------------------------
// Thread t < rg * nkb owns the 32-wide column block kb = t % nkb of x (in registers) and walks the rows
// ro, ro + rg, ... of each chunk; per-(row, block) partial sums go through shared memory and a warp per
// row adds them in a fixed order (lane-strided, then a butterfly), as the stand-alone GEMV does.
// Where a thread works in a GEMV over K columns: column block kb, first row ro, rg row groups (rg * nkb <= DS_COMPUTE threads take part)
struct LaneMap {
  int kb, ro, rg;
  bool active;
};
__device__ __forceinline__ LaneMap lane_map(int nkb) {
  LaneMap lm;
  lm.rg = DS_COMPUTE / nkb;
  lm.active = (int)threadIdx.x < lm.rg * nkb;
  lm.kb = lm.active ? (int)threadIdx.x % nkb : 0;
  lm.ro = lm.active ? (int)threadIdx.x / nkb : 0;
  return lm;
}

// ring position of the next chunk this CTA consumes (slot, mbarrier phase), carried across the phases
struct RingPos {
  int slot;
  uint32_t phase;
};

__device__ __forceinline__ void gemv_phase(const DsArgs &a, const Smem &sm, const DsMatrix &m, const LaneMap lm, const int r0, const int r1, RingPos &rp,
                                           int epi, unsigned tag, unsigned long long *out_words, const float *res /* shared [B][hres_rows] or null */) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int type = m.type, nkb = m.nkb, K = m.K, N = m.N, crb = m.crb, rps = m.rps;
  const int rg = lm.rg, kb = lm.kb, ro = lm.ro;
  const bool active = lm.active;
  const bool quant = has_scales(type), with_bias = m.bias != nullptr;
  const float *biasv = sm.bias(epi & 1);
  volatile int *flags = sm.flags();
  BlkQ4 q4;            // x of this thread's block: prepared for Q4_0 (pre-scaled by powers of two),
  float *xr = q4.xs;   // or as it is for the other formats (same registers)
  auto prep = [&](int b) {
    float xv[32];
    const float4 *xp = reinterpret_cast<const float4 *>(sm.xs() + (size_t)b * K + (kb << 5));
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 v = xp[q ^ (kb & 7)];
      xv[4 * q] = v.x; xv[4 * q + 1] = v.y; xv[4 * q + 2] = v.z; xv[4 * q + 3] = v.w;
    }
    if (type == CATEN_B200_Q4_0) q4.prep(xv);
    else {
#pragma unroll
      for (int j = 0; j < 32; ++j) xr[j] = xv[j];
    }
  };
  DS_FINE(1);
  if (a.B == 1 && active && r0 < r1) prep(0);
  DS_FINE(2);
  int buf = 0, slot = rp.slot;
  uint32_t phase = rp.phase;
  for (int c0 = r0; c0 < r1; c0 += rps) {
    const int c1 = min(c0 + rps, r1), nrows = c1 - c0;
    if (!flags[0] && !mbar_wait(sm.full(slot), phase, flags)) ds_fail(a, flags, 2, c0);
    DS_FINE(3);
    const uint8_t *codes = sm.ring(slot);
    const __half *scales = nullptr;
    if (quant) {
      const long long sb0 = ((long long)c0 * nkb * 2) & ~15ll;
      scales = reinterpret_cast<const __half *>(codes + (size_t)nrows * crb + ((long long)c0 * nkb * 2 - sb0));
    }
    float *rb = sm.red(buf);   // [B][nrows][nkb]: at most B x DS_SLOT_BLOCKS values
    if (!flags[0]) {
      for (int b = 0; b < a.B; ++b) {
        if (a.B > 1 && active) prep(b);
        if (active) {
          for (int r = ro; r < nrows; r += rg) {
            const uint8_t *rowp = codes + (size_t)r * crb;
            float part;
            if (type == CATEN_B200_Q4_0) {
              part = q4.dotp(reinterpret_cast<const uint4 *>(rowp) + kb, __half2float(scales[(size_t)r * nkb + kb]));
            } else if (type == CATEN_B200_Q8_0) {
              const uint4 *src = reinterpret_cast<const uint4 *>(rowp) + 2 * kb;
              float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint4 v = src[h];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  // int8 -> float without the (quarter-rate) conversion unit: with the sign bit flipped the byte is
                  // q + 128 in 0..255, and 0x4B0000uu is the float 2^23 + uu; one exact subtraction leaves q
                  const uint32_t u = w[i] ^ 0x80808080u;
                  const float kMagic = 8388736.0f;   // 2^23 + 128
                  a0 = fmaf(xr[16 * h + 4 * i + 0], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - kMagic, a0);
                  a1 = fmaf(xr[16 * h + 4 * i + 1], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - kMagic, a1);
                  a0 = fmaf(xr[16 * h + 4 * i + 2], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - kMagic, a0);
                  a1 = fmaf(xr[16 * h + 4 * i + 3], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - kMagic, a1);
                }
              }
              part = (a0 + a1) * __half2float(scales[(size_t)r * nkb + kb]);
            } else if (type == CATEN_B200_F16) {
              const uint4 *src = reinterpret_cast<const uint4 *>(rowp) + 4 * kb;
              float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 v = src[q];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                  a0 = fmaf(xr[8 * q + 2 * i], f.x, a0);
                  a1 = fmaf(xr[8 * q + 2 * i + 1], f.y, a1);
                }
              }
              part = a0 + a1;
            } else {
              const float4 *src = reinterpret_cast<const float4 *>(rowp) + 8 * kb;
              float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 v = src[q];
                a0 = fmaf(xr[4 * q], v.x, a0);
                a1 = fmaf(xr[4 * q + 1], v.y, a1);
                a0 = fmaf(xr[4 * q + 2], v.z, a0);
                a1 = fmaf(xr[4 * q + 3], v.w, a1);
              }
              part = a0 + a1;
            }
            rb[((size_t)b * nrows + r) * nkb + kb] = part;
          }
        }
      }
    }
    DS_FINE(4);
    bar_compute();                               // partial sums visible; every read of the slot is done
    DS_FINE(5);
    if (tid == 0) mbar_arrive(sm.empty(slot));   // the feeder may refill it
    if (!flags[0]) {
      for (int item = warp; item < nrows * a.B; item += DS_CWARPS) {
        const int b = a.B == 1 ? 0 : item / nrows, r = item - b * nrows, row = c0 + r;
        const float *pr = rb + ((size_t)b * nrows + r) * nkb;
        float s = 0.0f;
        for (int k = lane; k < nkb; k += 32) s += pr[k];
        s = warp_sum(s);
        if (lane == 0) {
          if (with_bias) s = s + biasv[row - r0];
          if (epi == EPI_FC) s = gelu_ref(s);
          if (epi == EPI_PROJ || epi == EPI_MPROJ) s = res[b * a.hres_rows + (row - r0)] + s;
          if (epi == EPI_LM) {
            a.logits[(size_t)b * a.V + row] = s;
            float *bvp = sm.best_v() + warp * DS_MAX_B + b;
            int *bip = sm.best_i() + warp * DS_MAX_B + b;
            if (s > *bvp || (s == *bvp && row < *bip)) { *bvp = s; *bip = row; }
          } else {
            st_tag(out_words + (size_t)b * N + row, s, tag);
          }
        }
      }
    }
    DS_FINE(6);
    buf ^= 1;
    if (++slot == a.nslots) { slot = 0; phase ^= 1u; }
  }
  rp.slot = slot;
  rp.phase = phase;
}

// ---- attention over one context chunk (external/llm/layers.lisp:3-5,19-51) -------------------------
// The K and V rows of the first DS_HALFWARPS x 4 positions of the chunk are requested before the poll
// for q: they do not depend on this step's activations (only position n does, and that row comes from
// the exchanged qkv vector, not from the cache).
struct AttnItem {
  int item, b, h, p0, p1;   // positions [p0, p1) of head h of sequence b
};
__device__ __forceinline__ AttnItem attn_item(int item, int C, int H, int t) {
  AttnItem it;
  const int c = item % C, bh = item / C;
  it.item = item; it.h = bh % H; it.b = bh / H;
  it.p0 = (int)(((unsigned)t * (unsigned)c) / (unsigned)C);
  it.p1 = (int)(((unsigned)t * (unsigned)(c + 1)) / (unsigned)C);
  return it;
}

__device__ __forceinline__ void attention_item(const DsArgs &a, const Smem &sm, const DsLayer *ly, const unsigned long long *qkv_words,
                                               unsigned long long *part_words, const AttnItem it, int n, unsigned tag) {
  constexpr int U = 4;   // cache rows per half-warp in flight
  const int tid = threadIdx.x, d = a.d, H = a.H, t = n + 1;
  const int item = it.item, h = it.h, b = it.b, p0 = it.p0, p1 = it.p1;
  const bool last = p1 == t;
  const int len = p1 - p0;
  float *q = sm.misc(), *kn = q + 64, *vn = q + 128, *part = q + 192, *sc = sm.sc();
  float *kb_ = ly->kc + ((size_t)b * H + h) * a.T * 64;
  float *vb_ = ly->vc + ((size_t)b * H + h) * a.T * 64;
  volatile int *flags = sm.flags();
  const int hw = tid >> 4, l16 = tid & 15;   // DS_HALFWARPS half-warps, 16 lanes x float4 = one 64-float row
  float4 k4[U], v4[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int j = p0 + u * DS_HALFWARPS + hw;
    const bool ok = j < p1 && j != n;
    k4[u] = ok ? __ldcs(reinterpret_cast<const float4 *>(kb_ + (size_t)j * 64) + l16) : make_float4(0.f, 0.f, 0.f, 0.f);
    v4[u] = ok ? __ldcs(reinterpret_cast<const float4 *>(vb_ + (size_t)j * 64) + l16) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  DS_FINE(40);
  bar_compute();  // misc and sc are free (previous item / phase)
  if (tid < 192 && (tid < 64 || last)) {
    const int which = tid >> 6, e = tid & 63;
    const float v = __uint_as_float(poll_one(a, flags, qkv_words + (size_t)b * 3 * d + (size_t)which * d + h * 64 + e, tag, 10 + which));
    if (which == 0) q[e] = v;
    else if (which == 1) { kn[e] = v; kb_[(size_t)n * 64 + e] = v; }   // cache[:, n] = k (layers.lisp:27-33)
    else { vn[e] = v; vb_[(size_t)n * 64 + e] = v; }
  }
  if (abort_uniform(flags)) return;
  DS_FINE(41);
  const float4 q4 = reinterpret_cast<const float4 *>(q)[l16];
  for (int j0 = 0; j0 < len; j0 += DS_HALFWARPS * U) {
    if (j0 > 0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int jj = j0 + u * DS_HALFWARPS + hw, j = p0 + jj;
        k4[u] = (jj < len && j != n) ? __ldcs(reinterpret_cast<const float4 *>(kb_ + (size_t)j * 64) + l16) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int jj = j0 + u * DS_HALFWARPS + hw, j = p0 + jj;
      float4 kk = k4[u];
      if (jj < len && j == n) kk = reinterpret_cast<const float4 *>(kn)[l16];
      float p = fmaf(q4.x, kk.x, fmaf(q4.y, kk.y, fmaf(q4.z, kk.z, q4.w * kk.w)));
      p += __shfl_xor_sync(0xffffffffu, p, 8);
      p += __shfl_xor_sync(0xffffffffu, p, 4);
      p += __shfl_xor_sync(0xffffffffu, p, 2);
      p += __shfl_xor_sync(0xffffffffu, p, 1);
      if (l16 == 0 && jj < len) sc[jj] = p * 0.125f;
    }
  }
  DS_FINE(42);
  bar_compute();
  float m = -INFINITY;
  for (int j = tid; j < len; j += DS_COMPUTE) m = fmaxf(m, sc[j]);
  m = block_max(m, sm.scratch(0));
  float ss = 0.0f;
  for (int j = tid; j < len; j += DS_COMPUTE) {
    const float e = exp2f((sc[j] - m) * kDsInvLn2);
    sc[j] = e;
    ss += e;
  }
  ss = block_sum(ss, sm.scratch(1));   // its barrier also publishes the exponentials
  DS_FINE(43);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < len; j0 += DS_HALFWARPS * U) {
    if (j0 > 0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int jj = j0 + u * DS_HALFWARPS + hw, j = p0 + jj;
        v4[u] = (jj < len && j != n) ? __ldcs(reinterpret_cast<const float4 *>(vb_ + (size_t)j * 64) + l16) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int jj = j0 + u * DS_HALFWARPS + hw, j = p0 + jj;
      const bool ok = jj < len;
      float4 vv = v4[u];
      if (ok && j == n) vv = reinterpret_cast<const float4 *>(vn)[l16];
      const float p = ok ? sc[jj] : 0.0f;
      acc.x = fmaf(p, vv.x, acc.x);
      acc.y = fmaf(p, vv.y, acc.y);
      acc.z = fmaf(p, vv.z, acc.z);
      acc.w = fmaf(p, vv.w, acc.w);
    }
  }
  DS_FINE(44);
  reinterpret_cast<float4 *>(part + hw * 64)[l16] = acc;
  bar_compute();
  DS_FINE(45);
  unsigned long long *dst = part_words + (size_t)item * 66;
  if (tid < 64) {
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < DS_HALFWARPS; ++w) o += part[w * 64 + tid];
    st_tag(dst + 2 + tid, o, tag);
  } else if (tid == 64) {
    st_tag(dst, m, tag);
  } else if (tid == 65) {
    st_tag(dst + 1, ss, tag);
  }
}

// combines the C partial results of one (sequence, head): softmax over the whole context
__device__ __forceinline__ void attention_combine(const DsArgs &a, const Smem &sm, const unsigned long long *part_words,
                                                  unsigned long long *att_words, int bh, int b, int h, int C, unsigned tag) {
  const int tid = threadIdx.x;
  float *buf = sm.misc();   // C x 66 floats: C <= DS_MAX_CHUNKS
  volatile int *flags = sm.flags();
  bar_compute();
  poll_words(a, flags, part_words + (size_t)bh * C * 66, C * 66, tag, 20, [&](int idx, float v) { buf[idx] = v; });
  if (abort_uniform(flags)) return;
  if (tid < 64) {
    float M = -INFINITY;
    for (int c = 0; c < C; ++c) M = fmaxf(M, buf[c * 66]);
    float L = 0.0f, o = 0.0f;
    for (int c = 0; c < C; ++c) {
      const float w = exp2f((buf[c * 66] - M) * kDsInvLn2);
      L += buf[c * 66 + 1] * w;
      o += buf[c * 66 + 2 + tid] * w;
    }
    const float inv = 1.0f / L;
    st_tag(att_words + (size_t)b * a.d + h * 64 + tid, o * inv, tag);
  }
}

__global__ void __launch_bounds__(DS_THREADS, 1) decode_small_kernel(const __grid_constant__ DsArgs a) {
  extern __shared__ uint8_t ds_smem_raw[];
  const Smem sm(reinterpret_cast<uint8_t *>(((uintptr_t)ds_smem_raw + 127) & ~(uintptr_t)127), a);
  const int d = a.d, B = a.B, G = gridDim.x, cta = blockIdx.x, tid = threadIdx.x;
  volatile int *flags = sm.flags();

  // layer descriptors -> shared memory (a global-memory pointer chase per phase would cost more than the phase)
  {
    const uint32_t *src = reinterpret_cast<const uint32_t *>(a.layers);
    uint32_t *dst = reinterpret_cast<uint32_t *>(sm.base + a.off_desc);
    const int words = (int)(sizeof(DsLayer) / 4) * (a.L + 1);
    for (int i = tid; i < words; i += DS_THREADS) dst[i] = src[i];
  }
  if (tid == 0) {
    for (int s = 0; s < a.nslots; ++s) { mbar_init(sm.full(s), 1); mbar_init(sm.empty(s), 1); }
    flags[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 16 * DS_MAX_B) { sm.best_v()[tid] = -INFINITY; sm.best_i()[tid] = 0x7fffffff; }
  __syncthreads();

  if (tid >= DS_COMPUTE) {
    if (tid == DS_COMPUTE) feeder(a, sm);
    return;
  }

  const unsigned tag = *a.d_epoch;
  const int n = *a.d_pos;            // position of this step's token; t = n + 1 keys are attended
  const int L = a.L;
  const int rd0 = row_begin(d, cta, G), rd1 = row_begin(d, cta + 1, G);
  // context chunks per (sequence, head): fill the grid, at least 32 positions each
  const int t = n + 1, BH = B * a.H;
  int C = G / BH;
  if (C < 1) C = 1;
  if (C > (t + 31) / 32) C = (t + 31) / 32;
  if (C > DS_MAX_CHUNKS) C = DS_MAX_CHUNKS;
  const int nitems = BH * C;
  // per-thread and per-CTA constants of the step, computed once: integer divisions are slow and every phase would repeat them
  const LaneMap lm_d = lane_map(d / 32), lm_f = lane_map(d / 8);          // GEMVs over K = d and over K = 4 d columns
  const int rq0 = row_begin(3 * d, cta, G), rq1 = row_begin(3 * d, cta + 1, G);   // rows of c_attn
  const int rf0 = row_begin(4 * d, cta, G), rf1 = row_begin(4 * d, cta + 1, G);   // rows of c_fc
  const int rv0 = row_begin(a.V, cta, G), rv1 = row_begin(a.V, cta + 1, G);       // rows of lm_head
  const AttnItem my_item = attn_item(cta < nitems ? cta : 0, C, a.H, t);
  const int my_b = cta < BH ? cta / a.H : 0, my_h = cta < BH ? cta % a.H : 0;
  RingPos rp;
  rp.slot = 0; rp.phase = 0;
  bool dead = false;
#ifdef DS_TIMING
  int mark_k = 0;
#endif
  DS_MARK();

  // Pseudo-layer L is ln_f + lm_head.  Phase ph of a layer: 0 ln_1 + c_attn, 1 attention + attn.c_proj,
  // 2 ln_2 + c_fc + GELU, 3 mlp.c_proj.  One call site per building block keeps the kernel small.
  for (int l = 0; l <= L && !dead; ++l) {
    unsigned long long *wl = a.xchg + (size_t)l * a.per_layer_words;
    const bool head = l == L;
    const DsLayer *ly = sm.layer(l);
#ifdef DS_TIMING
    if (blockIdx.x == DS_TIMING_CTA && threadIdx.x == 0) { sm.flags()[5] = (l == 1); if (l == 1) sm.flags()[4] = 0; }
#endif
    for (int ph = 0; ph < (head ? 1 : 4) && !dead; ++ph) {
      const DsMatrix &m = layer_matrix(ly, ph);
      DS_FINE(100 + ph);
      const bool ln = ph == 0 || ph == 2;
      // ---- requests that do not depend on this phase's input: LayerNorm parameters, biases of this CTA's rows
      float gg[5], bb[5];
      if (ln) {
        const float *g = ph == 0 ? ly->ln1_g : ly->ln2_g, *bt = ph == 0 ? ly->ln1_b : ly->ln2_b;
#pragma unroll
        for (int i = 0; i < 5; ++i) {
          const int k = tid + i * DS_COMPUTE;
          gg[i] = k < d ? g[k] : 0.0f;
          bb[i] = k < d ? bt[k] : 0.0f;
        }
      }
      const int mr0 = head ? rv0 : ph == 0 ? rq0 : ph == 2 ? rf0 : rd0, mr1 = head ? rv1 : ph == 0 ? rq1 : ph == 2 ? rf1 : rd1;
      const float my_bias = (m.bias && mr0 + tid < mr1) ? m.bias[mr0 + tid] : 0.0f;
      if (ph == 1) {
        // ---- attention partials over context chunks, then the combine
        for (int item = cta; item < nitems; item += G)
          attention_item(a, sm, ly, wl, wl + a.lay_part, item == cta ? my_item : attn_item(item, C, a.H, t), n, tag);
        DS_MARK();
        for (int bh = cta; bh < BH; bh += G)
          attention_combine(a, sm, wl + a.lay_part, wl + a.lay_att, bh, bh == cta ? my_b : bh / a.H, bh == cta ? my_h : bh % a.H, C, tag);
        bar_compute();
        DS_MARK();
      }
      // ---- the input vectors of this phase's GEMV
      float *xs = sm.xs();
      if (ph == 0 && l == 0) {
        // h = wte(tok) + wpe(n): an id outside [0, V) selects no row (source/nn/embedding.lisp:17-25)
        float *keep = sm.hres(0);
        for (int idx = tid; idx < B * d; idx += DS_COMPUTE) {
          const int b = idx / d, k = idx - b * d;
          const int64_t tok = a.ids_io[b];
          float v = (tok >= 0 && tok < a.V) ? a.wte[(size_t)tok * d + k] : 0.0f;
          if (n >= 0 && n < a.T) v += a.wpe[(size_t)n * d + k];
          xs[(size_t)b * d + swz(k)] = v;
          if (k >= rd0 && k < rd1) keep[b * a.hres_rows + (k - rd0)] = v;
        }
      } else {
        const unsigned long long *src = ph == 0 ? wl - a.per_layer_words + a.lay_h : ph == 1 ? wl + a.lay_att : ph == 2 ? wl + a.lay_h2 : wl + a.lay_ff;
        const int nvec = ph == 3 ? 4 * d : d;
        float *keep = (ph == 0 && !head) ? sm.hres(0) : ph == 2 ? sm.hres(1) : nullptr;
        const int hres_rows = a.hres_rows;
        poll_words(a, flags, src, B * nvec, tag, 30 + ph, [&](int idx, float v) {
          const int b = B == 1 ? 0 : idx / nvec, k = idx - b * nvec;
          xs[(size_t)b * nvec + swz(k)] = v;
          if (keep && k >= rd0 && k < rd1) keep[b * hres_rows + (k - rd0)] = v;
        });
      }
      DS_FINE(20);
      if (mr0 + tid < mr1) sm.bias(ph & 1)[tid] = my_bias;   // (two buffers: slow warps may still be adding the previous phase's)
      dead = abort_uniform(flags);   // also the barrier that publishes xs and the biases
      DS_FINE(21);
      DS_MARK();
      if (dead) break;
      if (ln) {
        // LayerNorm in place (source/nn/normalization.lisp:48-58: mean, centred, variance of the centred values, scale, affine)
        const float invd = 1.0f / (float)d;
        for (int b = 0; b < B; ++b) {
          float *x = xs + (size_t)b * d;
          float v[5];
          float sum = 0.0f;
#pragma unroll
          for (int i = 0; i < 5; ++i) {
            const int k = tid + i * DS_COMPUTE;
            v[i] = k < d ? x[swz(k)] : 0.0f;
            sum += v[i];
          }
          DS_FINE(30);
          const float u = block_sum(sum, sm.scratch(0)) * invd;
          DS_FINE(31);
          float sq = 0.0f;
#pragma unroll
          for (int i = 0; i < 5; ++i) {
            const int k = tid + i * DS_COMPUTE;
            if (k < d) { v[i] -= u; sq += v[i] * v[i]; }
          }
          const float var = block_sum(sq, sm.scratch(1)) * invd;
          DS_FINE(32);
          const float rs = 1.0f / sqrtf(var + a.eps);
#pragma unroll
          for (int i = 0; i < 5; ++i) {
            const int k = tid + i * DS_COMPUTE;
            if (k < d) x[swz(k)] = (v[i] * rs) * gg[i] + bb[i];
          }
        }
        bar_compute();
        DS_FINE(33);
      }
      DS_MARK();
      unsigned long long *out = head ? nullptr : ph == 0 ? wl : ph == 1 ? wl + a.lay_h2 : ph == 2 ? wl + a.lay_ff : wl + a.lay_h;
      const float *res = ph == 1 ? sm.hres(0) : ph == 3 ? sm.hres(1) : nullptr;
      gemv_phase(a, sm, m, ph == 3 ? lm_f : lm_d, mr0, mr1, rp, head ? EPI_LM : ph, tag, out, res);
      DS_MARK();
    }
  }
  dead = abort_uniform(flags);
  if (dead) return;   // the feeder notices the flag in its own bounded wait and drains its copies

  // ---- arg-max: per-warp bests -> CTA candidate -> CTA 0 picks
  unsigned long long *w_cand = a.xchg + (size_t)(L + 1) * a.per_layer_words;
  if (tid < B) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int w = 0; w < DS_CWARPS; ++w) {
      const float v = sm.best_v()[w * DS_MAX_B + tid];
      const int i = sm.best_i()[w * DS_MAX_B + tid];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    st_tag(w_cand + ((size_t)cta * B + tid) * 2, bv, tag);
    st_tag_bits(w_cand + ((size_t)cta * B + tid) * 2 + 1, (unsigned)bi, tag);
  }
  if (cta != 0) return;
  // lowest index of the maximum over all CTAs
  float *gv = sm.xs();   // 2 * G * B floats: free now
  bar_compute();
  poll_words(a, flags, w_cand, 2 * G * B, tag, 40, [&](int idx, float v) { gv[idx] = v; });
  if (abort_uniform(flags)) return;
  if (tid < B) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = 0; c < G; ++c) {
      const float v = gv[(c * B + tid) * 2];
      const int i = (int)__float_as_uint(gv[(c * B + tid) * 2 + 1]);
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    const int64_t id = bi == 0x7fffffff ? 0 : bi;
    a.out_ids[tid] = id;
    a.ids_io[tid] = id;
    a.hist[(size_t)n * B + tid] = id;
  }
  bar_compute();
  if (tid == 0) {
    *a.d_pos = n + 1;
    *a.d_epoch = tag + 1u;
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
void decode_small_destroy(DecodeSmall *s);

struct DecodeSmall {
  DsArgs args;
  DsLayer *d_layers = nullptr;
  unsigned long long *d_xchg = nullptr;
  unsigned *d_epoch = nullptr;
  size_t smem = 0;
  int grid = 0;
};

// bytes of one row: codes, and codes + scales
static void ds_row_bytes(int type, int64_t cols, int64_t *codes, int64_t *all) {
  const int64_t nkb = cols / 32;
  switch (type) {
    case CATEN_B200_Q4_0: *codes = nkb * 16; *all = nkb * 18; break;
    case CATEN_B200_Q8_0: *codes = nkb * 32; *all = nkb * 34; break;
    case CATEN_B200_F16: *codes = *all = cols * 2; break;
    default: *codes = *all = cols * 4; break;
  }
}

static DsMatrix ds_matrix(const caten_b200_weight *w, const float *bias) {
  DsMatrix m;
  m.qs = w->qs; m.d = w->d; m.bias = bias; m.type = w->type; m.N = (int)w->rows; m.K = (int)w->cols;
  m.nkb = (int)(w->cols / 32);
  int64_t codes = 0, all = 0;
  ds_row_bytes(w->type, w->cols, &codes, &all);
  m.crb = (int)codes;
  // the scales of a chunk are fetched as the enclosing 16-byte-aligned span: up to 30 bytes of slack
  m.rps = (int)((DS_SLOT - 32) / all);
  if (m.rps < 1) m.rps = 1;
  return m;
}

bool decode_small_supported(const caten_b200_gpt2_desc &c, const caten_b200_weight *const *attn, const caten_b200_weight *const *proj,
                            const caten_b200_weight *const *fc, const caten_b200_weight *const *mproj) {
  if (c.batch < 1 || c.batch > DS_MAX_B) return false;
  if (c.d_model % 32 || c.d_model > 5 * DS_COMPUTE || c.d_model != c.n_heads * 64) return false;
  if (c.max_seq_len > 8192) return false;
  auto ok = [](const caten_b200_weight *w, bool layer) {
    if (!w || w->cols % 32 || w->cols / 32 > DS_COMPUTE) return false;
    // Layer matrices must be block-quantised: dense fp16 / fp32 rows are 4..8 times longer, a CTA's share of a matrix then
    // takes several ring slots and barriers per phase, and the kernel-per-operation path measured faster (GPT-2 small fp32:
    // 473 vs 555 us per step).  lm_head may be dense (files that keep the output matrix in fp16 / fp32).
    if (layer && w->type != CATEN_B200_Q4_0 && w->type != CATEN_B200_Q8_0) return false;
    if (w->type != CATEN_B200_Q4_0 && w->type != CATEN_B200_Q8_0 && w->type != CATEN_B200_F16 && w->type != CATEN_B200_F32) return false;
    if (w->rows > (int64_t)DS_COMPUTE * 128) return false;   // rows x CTAs stays far below 2^31; a CTA's rows fit the bias buffer
    int64_t codes = 0, all = 0;
    ds_row_bytes(w->type, w->cols, &codes, &all);
    return all <= DS_SLOT - 32;   // one row (codes + scales) must fit a ring slot
  };
  if (!ok(c.lm_head, false)) return false;
  for (int l = 0; l < c.n_layers; ++l)
    if (!ok(attn[l], true) || !ok(proj[l], true) || !ok(fc[l], true) || !ok(mproj[l], true)) return false;
  return true;
}

int decode_small_create(caten_b200_ctx *ctx, const caten_b200_gpt2_desc &c, const std::vector<const caten_b200_weight *> &attn,
                        const std::vector<const caten_b200_weight *> &proj, const std::vector<const caten_b200_weight *> &fc,
                        const std::vector<const caten_b200_weight *> &mproj, const std::vector<const float *> *vecs /* 8 tables */,
                        const std::vector<float *> &kc, const std::vector<float *> &vc, int64_t *ids_io, int64_t *out_ids, int64_t *hist,
                        int *d_pos, float *logits, DecodeSmall **out) {
  *out = nullptr;
  DecodeSmall *s = new (std::nothrow) DecodeSmall();
  if (!s) return fail(ctx, CATEN_B200_ECUDA, "out of host memory");
  const int L = c.n_layers, d = c.d_model, B = c.batch, G = ctx->sm_count, BH = B * c.n_heads;
  if ((int64_t)c.vocab > (int64_t)DS_COMPUTE * G || 3 * (int64_t)d > (int64_t)DS_COMPUTE * G) { delete s; return fail(ctx, CATEN_B200_EUNSUPPORTED, "decode step: too few SMs for this model"); }
  std::vector<DsLayer> layers((size_t)L + 1);
  memset(layers.data(), 0, sizeof(DsLayer) * layers.size());
  {
    // entry L: ln_f + lm_head, laid out like phase 0 of a layer
    DsLayer &ly = layers[(size_t)L];
    ly.attn = ds_matrix(c.lm_head, nullptr);
    ly.proj = ly.fc = ly.mproj = ly.attn;
    ly.ln1_g = c.lnf_g; ly.ln1_b = c.lnf_b; ly.ln2_g = c.lnf_g; ly.ln2_b = c.lnf_b;
  }
  for (int l = 0; l < L; ++l) {
    DsLayer &ly = layers[(size_t)l];
    ly.attn = ds_matrix(attn[(size_t)l], vecs[2][(size_t)l]);
    ly.proj = ds_matrix(proj[(size_t)l], vecs[3][(size_t)l]);
    ly.fc = ds_matrix(fc[(size_t)l], vecs[6][(size_t)l]);
    ly.mproj = ds_matrix(mproj[(size_t)l], vecs[7][(size_t)l]);
    ly.ln1_g = vecs[0][(size_t)l]; ly.ln1_b = vecs[1][(size_t)l]; ly.ln2_g = vecs[4][(size_t)l]; ly.ln2_b = vecs[5][(size_t)l];
    ly.kc = kc[(size_t)l]; ly.vc = vc[(size_t)l];
  }
  auto bail = [&](int rc) { decode_small_destroy(s); return rc; };
  cudaError_t e;
  if ((e = cudaMalloc(&s->d_layers, sizeof(DsLayer) * layers.size())) != cudaSuccess) return bail(cuda_fail(ctx, e, "cudaMalloc(decode layers)"));
  if ((e = cudaMemcpyAsync(s->d_layers, layers.data(), sizeof(DsLayer) * layers.size(), cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess)
    return bail(cuda_fail(ctx, e, "cudaMemcpyAsync(decode layers)"));
  cudaStreamSynchronize(ctx->stream);  // `layers` is a local
  const size_t per_layer = ds_layout(B, d, G, BH).per_layer;
  // layers 0..L-1, one unused layer-sized gap for the ln_f + lm_head pseudo-layer (it exchanges nothing), then the
  // arg-max candidates
  const size_t words = per_layer * (size_t)(L + 1) + (size_t)2 * G * B;
  if ((e = cudaMalloc(&s->d_xchg, words * 8)) != cudaSuccess) return bail(cuda_fail(ctx, e, "cudaMalloc(decode exchange)"));
  if ((e = cudaMemsetAsync(s->d_xchg, 0, words * 8, ctx->stream)) != cudaSuccess) return bail(cuda_fail(ctx, e, "cudaMemsetAsync"));
  if ((e = cudaMalloc(&s->d_epoch, sizeof(unsigned))) != cudaSuccess) return bail(cuda_fail(ctx, e, "cudaMalloc(decode tag)"));
  const unsigned one = 1;
  if ((e = cudaMemcpyAsync(s->d_epoch, &one, sizeof one, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) return bail(cuda_fail(ctx, e, "cudaMemcpyAsync"));
  cudaStreamSynchronize(ctx->stream);

  DsArgs &a = s->args;
  a.layers = s->d_layers;
  a.wte = c.wte; a.wpe = c.wpe;
  a.L = L; a.d = d; a.H = c.n_heads; a.V = c.vocab; a.T = c.max_seq_len; a.B = B; a.eps = c.eps;
  a.ids_io = ids_io; a.out_ids = out_ids; a.hist = hist; a.d_pos = d_pos; a.d_epoch = s->d_epoch; a.logits = logits;
  a.xchg = s->d_xchg; a.per_layer_words = (long long)per_layer; a.status = ctx->d_status;
  a.sc_floats = (c.max_seq_len + 3) & ~3;
  a.hres_rows = (d / G + 3) & ~1;   // rows of a d-row matrix one CTA owns, rounded up to an even count
  a.red_floats = (B * DS_SLOT_BLOCKS + 3) & ~3;
  // shared memory: everything but the ring first, the ring takes what is left
  auto up = [](size_t x) { return (x + 127) & ~(size_t)127; };
  const size_t sz_desc = up(sizeof(DsLayer) * layers.size()), sz_xs = up((size_t)B * 4 * d * 4), sz_red = up((size_t)2 * a.red_floats * 4),
               sz_sc = up((size_t)a.sc_floats * 4), sz_hres = up((size_t)2 * B * a.hres_rows * 4), sz_bias = up(2 * DS_COMPUTE * 4),
               sz_best = up(2 * 64 * 4), sz_misc = up(DS_MISC_FLOATS * 4), sz_tail = 256;
  const size_t fixed = 128 + sz_desc + sz_xs + sz_red + sz_sc + sz_hres + sz_bias + sz_best + sz_misc + sz_tail;
  int max_optin = 0;
  cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, ctx->device);
  if ((size_t)max_optin < fixed + 2 * DS_SLOT) return bail(fail(ctx, CATEN_B200_EUNSUPPORTED, "decode step: not enough shared memory for d=%d, B=%d", d, B));
  int nslots = (int)(((size_t)max_optin - fixed) / DS_SLOT);
  if (nslots > DS_MAX_SLOTS) nslots = DS_MAX_SLOTS;
  a.nslots = nslots;
  size_t off = (size_t)nslots * DS_SLOT;
  a.off_desc = (int)off; off += sz_desc;
  a.off_xs = (int)off; off += sz_xs;
  a.off_red = (int)off; off += sz_red;
  a.off_sc = (int)off; off += sz_sc;
  a.off_hres = (int)off; off += sz_hres;
  a.off_bias = (int)off; off += sz_bias;
  a.off_best = (int)off; off += sz_best;
  a.off_misc = (int)off; off += sz_misc;
  a.off_bars = (int)off;            // 2 x DS_MAX_SLOTS x 8 bytes
  a.off_flags = (int)off + 128;
  off += sz_tail;
  s->smem = 128 + off;
  s->grid = G;
  const DsLayout lay = ds_layout(B, d, G, BH);
  a.lay_part = (long long)lay.part; a.lay_att = (long long)lay.att; a.lay_h2 = (long long)lay.h2; a.lay_ff = (long long)lay.ff; a.lay_h = (long long)lay.h;
  if ((e = cudaFuncSetAttribute(decode_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s->smem)) != cudaSuccess)
    return bail(cuda_fail(ctx, e, "cudaFuncSetAttribute(decode_small_kernel)"));
  int per_sm = 0;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_small_kernel, DS_THREADS, s->smem)) != cudaSuccess || per_sm < 1)
    return bail(fail(ctx, CATEN_B200_EUNSUPPORTED, "decode step: the kernel does not fit an SM (%zu bytes of shared memory)", s->smem));
  *out = s;
  return 0;
}

void decode_small_destroy(DecodeSmall *s) {
  if (!s) return;
  if (s->d_layers) cudaFree(s->d_layers);
  if (s->d_xchg) cudaFree(s->d_xchg);
  if (s->d_epoch) cudaFree(s->d_epoch);
  delete s;
}

int decode_small_reset(caten_b200_ctx *ctx, DecodeSmall *s) {
  const DsArgs &a = s->args;
  const size_t words = (size_t)a.per_layer_words * (size_t)(a.L + 1) + (size_t)2 * s->grid * a.B;
  CB_CUDA(ctx, cudaMemsetAsync(s->d_xchg, 0, words * 8, ctx->stream));   // tag 0 never matches a step tag
  return 0;
}

// One decode step from the device-side state (ids_io, d_pos).
int decode_small_launch(caten_b200_ctx *ctx, DecodeSmall *s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)s->grid);
  cfg.blockDim = dim3(DS_THREADS);
  cfg.dynamicSmemBytes = s->smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;   // all CTAs resident at once, or the launch fails
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  ctx->weights_pending = false;  // an ordinary stream-ordered launch
  CB_CUDA(ctx, cudaLaunchKernelEx(&cfg, decode_small_kernel, s->args));
  CB_LAUNCH_CHECK(ctx, "decode_small_kernel");
  return 0;
}

}  // namespace cb

#ifdef DS_TIMING
extern "C" int cb_debug_ds_times(unsigned long long *out, int n) {
  return (int)cudaMemcpyFromSymbol(out, cb::g_ds_times, sizeof(unsigned long long) * (size_t)n);
}
extern "C" int cb_debug_ds_fine(long long *out, int *n) {
  cudaMemcpyFromSymbol(n, cb::g_ds_fine_n, sizeof(int));
  return (int)cudaMemcpyFromSymbol(out, cb::g_ds_fine, sizeof(long long) * 512);
}
#endif
