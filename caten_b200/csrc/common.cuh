// Shared declarations of libcaten_b200: context, weight storage, launch prototypes.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/caten_b200.h"

namespace cb {

// Device-side status word layout (ctx->d_status, 4 ints): [0] error code, [1..3] detail.
enum DevErr : int { DEV_OK = 0, DEV_WAIT_TIMEOUT = 1, DEV_BAD_INDEX = 2 };

// Optional bf16 (hi, lo) destination of a kernel whose output feeds a tensor-core GEMM: when `hi`
// is set the producer writes the split operand itself and the fp32 copy is not needed.
struct BfOut {
  __nv_bfloat16 *hi = nullptr, *lo = nullptr;
};

// Output of a split-K linear that has not been summed yet.  The GEMM leaves its partial tiles
// part[split][tile][column = m % bnx][row = o % 128] in scratch memory and the kernel that
// consumes the result adds them (in split order, then the bias) while it loads its input:
//   y[m, o] = (sum_z part[z][tile(m, o)][m % bnx][o % 128]) + bias[o]
// splits == 0 means "nothing pending": the consumer reads the finished tensor instead.
struct PartIn {
  const float *part = nullptr, *bias = nullptr;
  int splits = 0, tiles_x = 0, bnx = 0;
  long long zstride = 0;  // floats between consecutive splits
};

#ifdef __CUDACC__
// four consecutive output features o..o+3 (o a multiple of 4) of activation row m
__device__ __forceinline__ float4 partin_load4(const PartIn &p, long long m, int o) {
  const long long tile = (m / p.bnx) * p.tiles_x + (o >> 7);
  const float *src = p.part + (tile * p.bnx + (m % p.bnx)) * 128 + (o & 127);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  int z = 0;
  for (; z + 4 <= p.splits; z += 4) {  // four loads in flight, added in split order
    float4 a[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) a[u] = __ldcs(reinterpret_cast<const float4 *>(src + (long long)(z + u) * p.zstride));
#pragma unroll
    for (int u = 0; u < 4; ++u) { v.x += a[u].x; v.y += a[u].y; v.z += a[u].z; v.w += a[u].w; }
  }
  for (; z < p.splits; ++z) {
    const float4 a = __ldcs(reinterpret_cast<const float4 *>(src + (long long)z * p.zstride));
    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
  }
  if (p.bias) {
    const float4 b = *reinterpret_cast<const float4 *>(p.bias + o);
    v.x = v.x + b.x; v.y = v.y + b.y; v.z = v.z + b.z; v.w = v.w + b.w;
  }
  return v;
}
__device__ __forceinline__ float partin_load1(const PartIn &p, long long m, int o) {
  const long long tile = (m / p.bnx) * p.tiles_x + (o >> 7);
  const float *src = p.part + (tile * p.bnx + (m % p.bnx)) * 128 + (o & 127);
  // the bias and up to four partial values are requested together (one round trip to L2 instead of one per split);
  // the additions keep the split order
  const float b = p.bias ? p.bias[o] : 0.f;
  float v = 0.f;
  for (int z = 0; z < p.splits; z += 4) {
    float t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u] = z + u < p.splits ? __ldcs(src + (long long)(z + u) * p.zstride) : 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (z + u < p.splits) v += t[u];
  }
  if (p.bias) v = v + b;
  return v;
}
#endif

struct Scratch {
  void *ptr = nullptr;
  size_t bytes = 0;
};

}  // namespace cb

struct caten_b200_ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;       // where work is queued: own_stream unless the caller supplied one
  cudaStream_t own_stream = nullptr;
  std::string err;
  int *d_status = nullptr;   // device status word written by kernels whose bounded waits run out
  int *h_status = nullptr;   // pinned mirror
  cb::Scratch xbf;           // bf16 copy (hi, lo) of the activation operand of the tensor-core GEMM
  cb::Scratch wtmp;          // split-K partial tiles of the tensor-core GEMM
  cb::Scratch wbf;           // bf16 copy (hi, lo) of the weight operand of the many-row GEMM
  cb::Scratch upload_stage;  // raw blocks of the weight being uploaded, before their re-layout
  void *pin[2] = {nullptr, nullptr};          // pinned bounce buffers for large copies from pageable host memory
  cudaEvent_t pin_ev[2] = {nullptr, nullptr};
  bool pin_busy[2] = {false, false};
  long long attn_prefetch_bytes = 64ll << 20;  // L2 budget of the decode attention's K / V history hint (CATEN_B200_ATTN_PREFETCH_MB; 0 = off)
  bool dense_gemm = true;    // many-row linears expand the weights once and run the TMA-fed GEMM (CATEN_B200_DENSE_GEMM=0: off)
  void *encode_tiled = nullptr;  // cuTensorMapEncodeTiled, resolved at init
  int64_t launches = 0;
  int64_t device_failures = 0;   // kernel-side check failures reported so far
  // split-K partial tiles: reduced by a second kernel through global scratch (default: it overlaps
  // with its neighbours under programmatic dependent launch and measured faster), or inside a
  // thread-block cluster through distributed shared memory (CATEN_B200_SPLITK_CLUSTER=1: every split-K
  // launch; =2: only launches whose epilogue cannot be handed to the consuming kernel)
  int splitk_cluster = 0;
  int attn_tc = 1;           // prefill attention of a tensor-core model on the tensor cores (CATEN_B200_ATTN_TC=0: SIMT kernel)
  bool use_pdl = true;       // programmatic dependent launch between consecutive kernels (CATEN_B200_PDL=0 turns it off)
  // A weight upload queued copy / re-layout kernels on the stream.  The Linear kernels read their
  // weights BEFORE waiting for the preceding kernel (weights are assumed static), so the next launch
  // after an upload is made as an ordinary stream-ordered launch, which completes everything before it.
  bool weights_pending = false;
  // multi-GPU group (caten_b200_dist_init): an NCCL communicator, bound at run time
  void *dist_comm = nullptr;
  int dist_rank = 0, dist_world = 1;
  // per-kernel-class event timing (caten_b200_profile_begin / _end)
  unsigned prof_mask = 0;
  struct ProfRec { int klass; cudaEvent_t a, b; };
  std::vector<ProfRec> prof;
  std::vector<cudaEvent_t> prof_pool;
};

struct caten_b200_weight {
  int type = 0;
  int64_t rows = 0, cols = 0;
  int64_t nkb = 0;          // blocks of 32 per row (quantised types)
  void *qs = nullptr;       // F32: float[rows*cols]; F16: half[rows*cols]; Q8_0: int8[rows*nkb*32]; Q4_x / Q5_x: u8[rows*nkb*16]
  __half *d = nullptr;      // per-block scales [rows*nkb] (quantised types)
  __half *m = nullptr;      // per-block minima [rows*nkb] (Q4_1, Q5_1)
  uint32_t *qh = nullptr;   // per-block fifth code bits [rows*nkb] (Q5_0, Q5_1)
  int64_t device_bytes = 0; // what the arrays above occupy
  caten_b200_ctx *ctx = nullptr;
};

namespace cb {

int fail(caten_b200_ctx *ctx, int code, const char *fmt, ...);
int cuda_fail(caten_b200_ctx *ctx, cudaError_t e, const char *what);
int scratch_reserve(caten_b200_ctx *ctx, Scratch *s, size_t bytes);

#define CB_CUDA(ctx, call)                                          \
  do {                                                              \
    cudaError_t e__ = (call);                                       \
    if (e__ != cudaSuccess) return cb::cuda_fail((ctx), e__, #call); \
  } while (0)
#define CB_LAUNCH_CHECK(ctx, what)                                   \
  do {                                                               \
    cudaError_t e__ = cudaGetLastError();                            \
    if (e__ != cudaSuccess) return cb::cuda_fail((ctx), e__, what);  \
    (ctx)->launches++;                                               \
  } while (0)

// ---- launchers (each returns a status code; all asynchronous on ctx->stream) ----
int launch_repack(caten_b200_ctx *ctx, int type, const uint8_t *d_blocks, int64_t nblocks, void *qs, __half *d, __half *m, uint32_t *qh);
int launch_dequant(caten_b200_ctx *ctx, const caten_b200_weight *w, float *out);
// block formats that are expanded to fp32 at upload (dequant_extra.cu)
int64_t extra_type_nbytes(int type, int64_t n, int64_t cols);
int launch_dequant_extra(caten_b200_ctx *ctx, int type, const uint8_t *d_blocks, int64_t n, float *out);
int launch_layernorm(caten_b200_ctx *ctx, const float *x, const float *g, const float *b, float *y,
                     int64_t rows, int64_t d, float eps);
// src_rows: optional gather — row r of the output reads row (r+1)*src_stride-1 of x when src_stride > 1
int launch_layernorm_strided(caten_b200_ctx *ctx, const float *x, const float *g, const float *b, float *y,
                             int64_t rows, int64_t d, float eps, int64_t src_stride, cb::BfOut bf = cb::BfOut());
// LayerNorm of x = res + pending linear output; also stores x (the new residual stream) to xout
int launch_layernorm_pending(caten_b200_ctx *ctx, const cb::PartIn &pin, const float *res, float *xout, const float *g,
                             const float *b, float *y, int64_t rows, int64_t d, float eps, int64_t src_stride,
                             cb::BfOut bf = cb::BfOut());
int launch_embed(caten_b200_ctx *ctx, const float *ids_f32, const int64_t *ids_i64, const float *wte,
                 const float *wpe, float *out, int64_t B, int64_t s, int64_t n, int64_t d, int64_t V, int64_t T,
                 const int *d_n = nullptr);
int launch_begin_steps(caten_b200_ctx *ctx, const float *ids_f32, const int64_t *ids_i64, int64_t *ids_io, int *d_pos,
                       int64_t n, int64_t B);
int launch_finish_step(caten_b200_ctx *ctx, const int64_t *out_ids, int64_t *ids_io, int64_t *hist, int *d_pos, int64_t B);
int launch_argmax(caten_b200_ctx *ctx, const float *x, int64_t rows, int64_t V, int64_t *out);
int launch_expr(caten_b200_ctx *ctx, const caten_b200_expr *e);
int launch_sample(caten_b200_ctx *ctx, const float *logits, int64_t rows, int64_t V, float temperature, int top_k,
                  const float *uniform, int64_t *out);
int launch_attention(caten_b200_ctx *ctx, const float *qkv, float *kc, float *vc, float *out, int64_t B,
                     int64_t s, int64_t n, int64_t H, int64_t T, const int *d_n = nullptr, cb::BfOut bf = cb::BfOut(),
                     const cb::PartIn *pending_qkv = nullptr, int tensor_cores = 0);
int launch_attention_tc(caten_b200_ctx *ctx, const float *qkv, const float *kc, const float *vc, float *out, int64_t B,
                        int64_t s, int64_t n, int64_t H, int64_t T, cb::BfOut bf);
int launch_gemv(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                const float *res, int act, float *y);
int launch_gemm_simt(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                     const float *res, int act, float *y, int64_t M);
int launch_gemm_tc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                   const float *res, int act, float *y, int64_t M, int nsplit);
// x given as fp32 (split by a pre-pass) or, when xhi is set, already as bf16 hi/lo; output as fp32 y
// or, when ybf.hi is set, as bf16 hi/lo for the next GEMM
int launch_gemm_tc_ex(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const __nv_bfloat16 *xhi,
                      const __nv_bfloat16 *xlo, const float *bias, const float *res, int act, float *y, cb::BfOut ybf,
                      int64_t M, int nsplit, cb::PartIn *defer = nullptr);
// `defer`: when the launch is split-K with no activation, skip the reduction kernel and describe the
// partial tiles in *defer instead (bias and residual are then the consumer's job); otherwise
// defer->splits stays 0 and y is complete
int launch_gemm_tc_noalloc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *x, const float *bias,
                           const float *res, int act, float *y, int64_t M, int nsplit);
// relu(a.b) with b given [K, N] row-major fp32
int launch_relu_matmul_simt(caten_b200_ctx *ctx, const float *a, const float *b, float *c, int64_t M, int64_t K, int64_t N);
int launch_relu_matmul_tc(caten_b200_ctx *ctx, const float *a, const float *b, float *c, int64_t M, int64_t K,
                          int64_t N, int nsplit);

// where a weight operand lives
struct WSrc {
  const void *qs;
  const __half *d, *m;
  const uint32_t *qh;
  int64_t nkb;
};
constexpr int WT_F32_T = 100;  // pseudo weight type: fp32 operand given as [K, N] row-major (relu_matmul's b)
// many-row GEMM with both operands from shared memory (gemm_dense.cu)
bool gemm_dense_applies(const caten_b200_ctx *ctx, int64_t M, int64_t N, int64_t K);
int launch_gemm_dense(caten_b200_ctx *ctx, int wt, const WSrc &ws, const float *x, const __nv_bfloat16 *xhi, const __nv_bfloat16 *xlo,
                      const float *bias, const float *res, int act, float *y, BfOut ybf, int64_t M, int64_t N, int64_t K, int nsplit);

// Whether the next launch may be a programmatic dependent launch; clears the pending-upload mark.
inline bool take_pdl(caten_b200_ctx *ctx) {
  const bool ok = ctx->use_pdl && !ctx->weights_pending;
  ctx->weights_pending = false;
  return ok;
}

// Single-kernel decode step for 1..4 sequences (decode_small.cu)
struct DecodeSmall;
bool decode_small_supported(const caten_b200_gpt2_desc &c, const caten_b200_weight *const *attn, const caten_b200_weight *const *proj,
                            const caten_b200_weight *const *fc, const caten_b200_weight *const *mproj);
// vecs: eight per-layer tables in the order ln1_g, ln1_b, attn_b, proj_b, ln2_g, ln2_b, fc_b, mproj_b
int decode_small_create(caten_b200_ctx *ctx, const caten_b200_gpt2_desc &c, const std::vector<const caten_b200_weight *> &attn,
                        const std::vector<const caten_b200_weight *> &proj, const std::vector<const caten_b200_weight *> &fc,
                        const std::vector<const caten_b200_weight *> &mproj, const std::vector<const float *> *vecs,
                        const std::vector<float *> &kc, const std::vector<float *> &vc, int64_t *ids_io, int64_t *out_ids, int64_t *hist,
                        int *d_pos, float *logits, DecodeSmall **out);
void decode_small_destroy(DecodeSmall *s);
int decode_small_launch(caten_b200_ctx *ctx, DecodeSmall *s);
// after a kernel-side failure the exchange words of the interrupted step are stale: forget them
int decode_small_reset(caten_b200_ctx *ctx, DecodeSmall *s);

// Kernel launch with programmatic dependent launch allowed: the next kernel in the stream may be
// scheduled (and run its prologue) while this one drains; every kernel launched this way calls
// pdl_wait() before it touches memory another kernel produces or still reads.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(caten_b200_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = take_pdl(ctx) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- device helpers ----

// Blocks until the kernels this launch depends on have completed and their writes are visible
// (no-op when the kernel was not launched as a programmatic dependent).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream start being scheduled.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() { pdl_wait(); pdl_launch_dependents(); }


// GeLU exactly as the reference composes it (source/nn/activations.lisp:202-204 with
// tanh(z) = 2*sigmoid(2z) - 1 and sigmoid(y) = 1/(1 + exp2(y * -1/ln2))), every step in fp32.
__device__ __forceinline__ float gelu_ref(float x) {
  const float kC = 0.7978845608028654f, k044 = 0.044715f, kNegInvLn2 = -1.0f / 0.6931472f;
  float x3 = x * x;
  x3 = x3 * x;
  float in = k044 * x3;
  in = x + in;
  const float z = kC * in;
  float a = 2.0f * z;
  a = a * kNegInvLn2;
  float e = exp2f(a);
  e = 1.0f + e;
  const float sg = 1.0f / e;
  float th = 2.0f * sg;
  th = th + (-1.0f);
  const float l = 0.5f * x;
  const float r = 1.0f + th;
  return l * r;
}

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == CATEN_B200_ACT_GELU) return gelu_ref(v);
  if (act == CATEN_B200_ACT_RELU) return v > 0.0f ? v : 0.0f;
  return v;
}

// bf16 operand split used by the tensor-core GEMM: hi = bf16(v), lo = bf16(v - hi)
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);  // .x = a in the low half
  return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ float bf16_lo(float w) { return w - __bfloat162float(__float2bfloat16_rn(w)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace cb
