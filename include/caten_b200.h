/* libcaten_b200.so — C ABI of the B200 (sm_100a) backend for Caten's GPT-2 forward path.
 *
 * Callers: Common Lisp through CFFI (`cffi:foreign-funcall`, the way source/byoc/clang.lisp:197-205
 * calls its gcc-built kernels) and the Python ctypes host in caten_b200/.  Plain pointers and
 * sizes only; every function returns an int status (0 = ok) unless stated, and the message of
 * the last failure is read with caten_b200_last_error().
 *
 * Conventions.  All activations are fp32, row-major.  A Linear weight is W[out, in] row-major
 * and y = x.W^T + b (source/nn/linear.lisp:12-17).  Pointers named d_* are device pointers
 * obtained from caten_b200_malloc (or any CUDA allocation of the context's device); pointers
 * named h_* are host pointers.  Kernels are launched asynchronously on the context's stream;
 * only the functions documented as synchronising wait for the GPU.  A context is driven by one
 * host thread at a time (Caten's VM is single-threaded, source/runtime/runtime.lisp:106-145).
 *
 * Paths below are relative to the hikettei/Caten source tree.
 */
#ifndef CATEN_B200_H
#define CATEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct caten_b200_ctx caten_b200_ctx;
typedef struct caten_b200_weight caten_b200_weight;
typedef struct caten_b200_gpt2 caten_b200_gpt2;

/* status codes */
enum {
  CATEN_B200_OK = 0,
  CATEN_B200_EINVAL = 1,      /* bad argument (null handle, wrong size, misaligned pointer) */
  CATEN_B200_ECUDA = 2,       /* a CUDA runtime/driver call failed */
  CATEN_B200_EUNSUPPORTED = 3,/* shape or type outside what the kernels cover */
  CATEN_B200_EDEVICE = 4      /* a kernel reported a failed internal check (e.g. a bounded wait ran out) */
};

/* ggml tensor type ids as stored in GGUF (external/gguf/tensor-info.lisp:3-34).  F32, F16, Q4_0
 * and Q8_0 weights stay in their file format on the device and the kernels unpack them; the other
 * block formats below (ids the reference lists but does not implement) are expanded to fp32 once
 * at upload, which is what the reference's loader does for every format it knows
 * (external/gguf/dequantize.lisp:14-53). */
enum {
  CATEN_B200_F32 = 0, CATEN_B200_F16 = 1, CATEN_B200_Q4_0 = 2, CATEN_B200_Q8_0 = 8,
  CATEN_B200_Q4_1 = 3, CATEN_B200_Q5_0 = 6, CATEN_B200_Q5_1 = 7,
  CATEN_B200_Q2_K = 10, CATEN_B200_Q3_K = 11, CATEN_B200_Q4_K = 12, CATEN_B200_Q5_K = 13, CATEN_B200_Q6_K = 14
};

/* epilogue applied by the Linear kernels after the bias: the scheduler fuses the activation
 * into the matmul kernel (source/test-suite/test-schedule.lisp:72-74). */
enum { CATEN_B200_ACT_NONE = 0, CATEN_B200_ACT_GELU = 1, CATEN_B200_ACT_RELU = 2 };

/* arithmetic of the Linear kernels when more than a few rows are multiplied at once:
 *   FP32    fp32 operands and accumulation on the CUDA cores (max-abs 1e-3 logit class)
 *   BF16    operands rounded to bf16, fp32 accumulation on tcgen05 tensor cores (rel 2e-2 class)
 *   BF16X3  each operand split into two bf16 terms, three tensor-core products (about 2^-16 rel.)
 * Single-row products (decode with one sequence) always run the fp32 dequant-GEMV. */
enum { CATEN_B200_PREC_FP32 = 0, CATEN_B200_PREC_BF16 = 1, CATEN_B200_PREC_BF16X3 = 2 };

/* ---- context, memory, transfers -------------------------------------------------------------
 * Replaces, for BACKEND=B200, what a Caten backend supplies through define-backend
 * (source/codegen/backend.lisp:22-34): the buffer generics open-buffer / close-buffer /
 * transfer-from-array / transfer-into-array / copy-buffer-value (source/runtime/buffer.lisp:78-89). */

/* Creates a context on CUDA device `device` with its own stream. */
int caten_b200_init(int device, caten_b200_ctx **ctx);
int caten_b200_destroy(caten_b200_ctx *ctx);
/* Message of the last failed call on this context (or of the last failed call without a
 * context when ctx is NULL). Never NULL. The pointer stays valid until the next failing call. */
const char *caten_b200_last_error(caten_b200_ctx *ctx);
/* open-buffer: zero-filled device allocation (source/runtime/buffer.lisp:79). */
int caten_b200_malloc(caten_b200_ctx *ctx, size_t bytes, void **d_ptr);
/* close-buffer. */
int caten_b200_free(caten_b200_ctx *ctx, void *d_ptr);
/* transfer-from-array: host -> device, ordered on the context's stream; returns after the host
 * buffer may be reused. */
int caten_b200_h2d(caten_b200_ctx *ctx, void *d_dst, const void *h_src, size_t bytes);
/* transfer-into-array / bref: device -> host; synchronises. */
int caten_b200_d2h(caten_b200_ctx *ctx, void *h_dst, const void *d_src, size_t bytes);
/* copy-buffer-value: device -> device. */
int caten_b200_d2d(caten_b200_ctx *ctx, void *d_dst, const void *d_src, size_t bytes);
int caten_b200_memset(caten_b200_ctx *ctx, void *d_dst, int byte, size_t bytes);
/* Waits for all work queued on the context and reports kernel-side check failures. */
int caten_b200_sync(caten_b200_ctx *ctx);
/* The context's cudaStream_t, for callers that time or order work themselves. */
void *caten_b200_stream(caten_b200_ctx *ctx);
/* Makes the context queue its work on a stream the caller owns (a cudaStream_t / CUstream of the same device:
 * the host framework's stream, or one bound to a green context, i.e. to a subset of the SMs); NULL returns to
 * the context's own stream. Work already queued is waited for first. The caller keeps the stream alive until
 * the context is destroyed or pointed elsewhere. */
int caten_b200_set_stream(caten_b200_ctx *ctx, void *stream);

/* ---- weights ----------------------------------------------------------------------------------
 * Replaces external/gguf/tensor-info.lisp:71-77,104-120 + external/gguf/dequantize.lisp:14-53,
 * which dequantise every tensor to a fp32 Lisp array at load: here the raw GGUF blocks are
 * uploaded as they are in the file and stay packed in HBM (Q8_0: 34-byte blocks, Q4_0: 18, Q4_1:
 * 20, Q5_0: 22, Q5_1: 24; on the device codes, fp16 scales, fp16 minima and fifth code bits are
 * kept in separate arrays so code loads are 16-byte aligned — same bytes, same values). The
 * 256-weight K formats are expanded to fp32 at upload. `cols` (the `in` dimension) must be a
 * multiple of the block size (32; 256 for the K formats). */
int caten_b200_weight_upload(caten_b200_ctx *ctx, int ggml_type, const void *h_blocks, int64_t rows,
                             int64_t cols, caten_b200_weight **w);
/* Same, from raw blocks already in device memory (e.g. after an NCCL broadcast of the file's
 * tensor data). The blocks are re-laid out into storage owned by the handle; d_blocks may be
 * freed after the call returns and the stream is synchronised. */
int caten_b200_weight_upload_device(caten_b200_ctx *ctx, int ggml_type, const void *d_blocks,
                                    int64_t rows, int64_t cols, caten_b200_weight **w);
int caten_b200_weight_free(caten_b200_ctx *ctx, caten_b200_weight *w);
/* Number of bytes of a rows x cols tensor in GGUF block form; -1 for an unknown type. */
int64_t caten_b200_weight_nbytes(int ggml_type, int64_t rows, int64_t cols);
/* Bytes the uploaded weight occupies in device memory: the file's bytes for the formats the
 * kernels read packed, rows*cols*4 for a format expanded at upload; -1 for a NULL handle. */
int64_t caten_b200_weight_device_nbytes(const caten_b200_weight *w);
/* dequantize (external/gguf/dequantize.lisp:8): writes rows*cols fp32 values, bit-identical to
 * (float)code * (float)scale (Q8_0, Q4_0; the other block formats: to the Python `gguf` package's
 * dequantiser), to d_out. */
int caten_b200_weight_dequant(caten_b200_ctx *ctx, const caten_b200_weight *w, float *d_out);

/* ---- GGUF files ------------------------------------------------------------------------------------
 * Replaces `load-gguf` / `make-gguf` (external/gguf/gguf-file.lisp:48-91), `parse-metadata-kv`
 * (external/gguf/metadata.lisp:3-87) and `parse-tensor-info` (external/gguf/tensor-info.lisp:79-102):
 * the file is memory-mapped and only its header, key/value table and tensor table are decoded;
 * tensor bytes stay where they are until uploaded.  GGUF versions 2 and 3; tensor offsets follow
 * `general.alignment` (default 32).  Returned name/key/data pointers point into the handle and
 * are valid until caten_b200_gguf_close. */
typedef struct caten_b200_gguf caten_b200_gguf;
int caten_b200_gguf_open(const char *path, caten_b200_gguf **g);
int caten_b200_gguf_close(caten_b200_gguf *g);
int caten_b200_gguf_version(const caten_b200_gguf *g);
int64_t caten_b200_gguf_alignment(const caten_b200_gguf *g);
int64_t caten_b200_gguf_tensor_count(const caten_b200_gguf *g);
int64_t caten_b200_gguf_meta_count(const caten_b200_gguf *g);
/* Tensor i: name, ggml type id, number of dims, dims4[4] in file order (dims4[0] is the contiguous
 * dimension; unused entries are 1), pointer to its bytes in the mapping and their count (-1 for
 * a ggml type this library does not hold).  Any out pointer may be NULL. */
int caten_b200_gguf_tensor(const caten_b200_gguf *g, int64_t i, const char **name, int *ggml_type, int *n_dims,
                           int64_t *dims4, const void **data, int64_t *nbytes);
/* Index of the tensor called `name`, or -1. */
int64_t caten_b200_gguf_find_tensor(const caten_b200_gguf *g, const char *name);
/* Metadata entry i: key, value type id (0 u8, 1 i8, 2 u16, 3 i16, 4 u32, 5 i32, 6 f32, 7 bool,
 * 8 string, 9 array, 10 u64, 11 i64, 12 f64), element type and length for arrays, pointer to the
 * little-endian value (strings: first byte, *str_len bytes; arrays: first element; string arrays
 * are sequences of u64 length + bytes). */
int caten_b200_gguf_meta(const caten_b200_gguf *g, int64_t i, const char **key, int *type, int *elem_type,
                         int64_t *count, const void **value, int64_t *str_len);
/* Uploads 2-D tensor i as a Linear weight [dims4[1], dims4[0]] straight from the mapping
 * (`tensor-info->tensor`, external/gguf/tensor-info.lisp:104-120, without dequantising). */
int caten_b200_gguf_upload(caten_b200_ctx *ctx, const caten_b200_gguf *g, int64_t i, caten_b200_weight **w);

/* ---- kernels of the GPT-2 graph -----------------------------------------------------------------
 * One entry per fused kernel the scheduler produces for external/llm/layers.lisp
 * ([Embedding_Embedding_ADD] [LayerNorm] [Matmul+GELU] [Attention], source/codegen/jit.lisp:8);
 * these are what the :b200 renderer's compiled lambdas call in place of the C functions
 * CLANG emits (source/byoc/clang.lisp:163-205). */

/* Linear (source/nn/linear.lisp:12-17; api/high-level-ops.lisp:76-99):
 *   y[m, o] = act(sum_k x[m,k] * W[o,k] + bias[o]) + residual[m, o]
 * x [M, cols], y [M, rows]; d_bias [rows] or NULL; d_residual [M, rows] or NULL (may alias y).
 * M == 1..4 runs the dequant-GEMV; larger M runs the GEMM selected by `precision`. */
int caten_b200_linear(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *d_x,
                      const float *d_bias, const float *d_residual, int act, float *d_y, int64_t M,
                      int precision);
/* (No counterpart in the reference.)  caten_b200_linear for hosts that cannot let the library
 * allocate: a runtime whose memory planner accounts for every device buffer up front, a serving
 * loop that cannot afford cudaMalloc/cudaFree (both can synchronise the whole device) between
 * tokens, or a process that has sized its KV cache to fill HBM so that a late allocation may
 * simply fail.  Same arguments and results as caten_b200_linear; the difference is where the
 * tensor-core path keeps its working memory (the bf16 copy of x and the split-K partial tiles):
 * in a 32 MiB buffer that is part of the library image (resident on every GPU that loads the
 * library until the process exits) instead of a buffer grown with cudaMalloc.  The call makes
 * no allocation of any kind.
 *   - Shapes whose working set exceeds 32 MiB are refused with CATEN_B200_EUNSUPPORTED and a
 *     message stating the bytes needed (M x cols x 2 B, doubled for BF16X3, plus partial tiles);
 *     e.g. 256 rows of a 1600 x 6400 weight in BF16X3 fit, 8192 rows do not.
 *   - The first call on a device looks up the buffer's address (and loads the kernels); make
 *     that call before any stream capture begins.
 *   - All calls on a device share the one buffer, whatever context or stream they use: calls
 *     whose GPU work may overlap race on it. Nothing in it needs to be zero beforehand. */
int caten_b200_linear_noalloc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *d_x,
                              const float *d_bias, const float *d_residual, int act, float *d_y,
                              int64_t M, int precision);
/* `(!relu (!matmul a b))` with a [M,K] and b [K,N], both row-major fp32 (Readme.md:55-60):
 * c = max(a.b, 0).  precision as above (FP32 or BF16X3 keep the reference's 1e-5 tolerance). */
int caten_b200_relu_matmul(caten_b200_ctx *ctx, const float *d_a, const float *d_b, float *d_c,
                           int64_t M, int64_t K, int64_t N, int precision);
/* LayerNorm over the last axis (source/nn/normalization.lisp:48-58). x, y [rows, d]. */
int caten_b200_layernorm(caten_b200_ctx *ctx, const float *d_x, const float *d_gamma,
                         const float *d_beta, float *d_y, int64_t rows, int64_t d, float eps);
/* h = wte(tokens) + wpe(n + arange(s)) (external/llm/layers.lisp:83-85, nn/embedding.lisp:13-25).
 * Exactly one of d_ids_f32 (what apps/gpt2/gpt2.lisp:95 feeds) and d_ids_i64 (what argmax
 * writes) is non-NULL; both are [B, s]. An id that is not an integer in [0, V) selects no row
 * (the one-hot compare of the reference matches nothing): its token embedding is zero. */
int caten_b200_embed(caten_b200_ctx *ctx, const float *d_ids_f32, const int64_t *d_ids_i64,
                     const float *d_wte, const float *d_wpe, float *d_out, int64_t B, int64_t s,
                     int64_t n, int64_t d, int64_t V, int64_t T);
/* Attention core of external/llm/layers.lisp:19-51 for head dim 64: appends this step's K and V
 * rows (columns [d,2d) and [2d,3d) of qkv) at positions [n, n+s) of the caches, then
 * out = softmax(q.K^T * 0.125 + causal mask) . V over positions [0, n+s).
 * qkv [B*s, 3d]; out [B*s, d]; caches are [B, H, T, 64] fp32 (head-major so one head's history
 * is contiguous; the reference's [B, T, H, 64] holds the same values). */
int caten_b200_attention(caten_b200_ctx *ctx, const float *d_qkv, float *d_kcache, float *d_vcache,
                         float *d_out, int64_t B, int64_t s, int64_t n, int64_t H, int64_t T);
/* The same with a precision (CATEN_B200_PREC_*) for steps of more than one token: FP32 is
 * caten_b200_attention; BF16 and BF16X3 run q.K^T and P.V on the tensor cores as bf16 hi/lo split
 * products with fp32 accumulation (within about 2^-16 of the fp32 result; the softmax itself, exp2
 * and the row sums stay fp32).  Single-token steps are the same kernel at every precision. */
int caten_b200_attention_ex(caten_b200_ctx *ctx, const float *d_qkv, float *d_kcache, float *d_vcache,
                            float *d_out, int64_t B, int64_t s, int64_t n, int64_t H, int64_t T,
                            int precision);
/* argmax over the last axis, lowest index on ties (api/high-level-ops.lisp:314-343). */
int caten_b200_argmax(caten_b200_ctx *ctx, const float *d_x, int64_t rows, int64_t V, int64_t *d_out);
/* Temperature / top-k sampling of one id per row.  No counterpart in the reference, whose generate
 * loop is greedy (apps/gpt2/gpt2.lisp:104-107).  Per row: keep the logits >= the top_k-th largest
 * (top_k <= 0 or >= V: all; ties at the threshold are kept), weight them by
 * exp((x - max) / temperature), and return the first index, in index order, whose running weight
 * reaches d_uniform[row] * total (d_uniform: one number in [0, 1) per row, supplied by the caller,
 * so the call is a pure function of its inputs).  temperature <= 0 is the argmax. */
int caten_b200_sample(caten_b200_ctx *ctx, const float *d_logits, int64_t rows, int64_t V, float temperature,
                      int top_k, const float *d_uniform, int64_t *d_out);

/* RMSNorm over the last axis (source/nn/normalization.lisp:70-85):
 *   y = x * (1 / sqrt(eps + mean(x * x))) [* weight]; d_weight [d] or NULL.  x, y [rows, d]; d % 4 == 0, d <= 8192. */
int caten_b200_rmsnorm(caten_b200_ctx *ctx, const float *d_x, const float *d_weight, float *d_y, int64_t rows,
                       int64_t d, float eps);
/* Rotary positional encoding (source/nn/positional-encoding.lisp:3-56, `(!rope x dim)` with dim = head_dim / 2):
 * x, y [B, S, H, head_dim]; the pair (x[2i], x[2i+1]) is rotated by (pos0 + s) * base^(-2i / head_dim); an odd last
 * element is copied.  The reference counts positions from 0 (pos0 = 0); pos0 > 0 serves a step that continues a
 * KV-cached sequence.  In place (d_y == d_x) is allowed. */
int caten_b200_rope(caten_b200_ctx *ctx, const float *d_x, float *d_y, int64_t B, int64_t S, int64_t H,
                    int64_t head_dim, float base, int64_t pos0);

/* ---- whole GPT-2 step ---------------------------------------------------------------------------
 * Replaces one `(forward runtime (x . tokens) (s . len) (n . start-pos))` of
 * apps/gpt2/gpt2.lisp:104 on the GraphRuntime built by make-gpt2 (gpt2.lisp:82-93): the whole
 * kernel sequence of source/runtime/runtime.lisp:106-145 in one call. */
typedef struct {
  int32_t n_layers, d_model, n_heads, vocab, max_seq_len, batch;
  float eps;
  int32_t precision;      /* CATEN_B200_PREC_* for steps with more than 4 rows */
  int32_t max_rows;       /* rows (sequences x tokens) processed at once in prefill; 0 = default */
  /* fp32 device arrays (not owned): */
  const float *wte, *wpe, *lnf_g, *lnf_b;
  const caten_b200_weight *lm_head;
  /* per layer, arrays of n_layers entries (host arrays of device pointers / handles): */
  const float *const *ln1_g, *const *ln1_b, *const *attn_b, *const *proj_b;
  const float *const *ln2_g, *const *ln2_b, *const *fc_b, *const *mproj_b;
  const caten_b200_weight *const *attn_w, *const *proj_w, *const *fc_w, *const *mproj_w;
} caten_b200_gpt2_desc;

/* Allocates the KV caches ([B, H, T, 64] per layer, zero-filled as layers.lisp:25-26 does) and
 * the activation workspace. Weights stay owned by the caller and must outlive the model. */
int caten_b200_gpt2_create(caten_b200_ctx *ctx, const caten_b200_gpt2_desc *desc, caten_b200_gpt2 **m);
int caten_b200_gpt2_destroy(caten_b200_gpt2 *m);
/* One step from host buffers: h_ids_f32 [B, s] token ids as float32, start position n;
 * h_out_ids [B] int64 = argmax of the last position's logits. Copies in, runs, copies out,
 * synchronises. */
int caten_b200_gpt2_step(caten_b200_gpt2 *m, const float *h_ids_f32, int64_t s, int64_t n,
                         int64_t *h_out_ids);
/* Same with device-resident ids: exactly one of d_ids_f32 / d_ids_i64 is non-NULL; d_out_ids
 * [B] int64 (may be the next step's d_ids_i64). Asynchronous. */
int caten_b200_gpt2_step_device(caten_b200_gpt2 *m, const float *d_ids_f32, const int64_t *d_ids_i64,
                                int64_t s, int64_t n, int64_t *d_out_ids);
/* `steps` consecutive single-token steps (the body of the loop of apps/gpt2/gpt2.lisp:102-109 after
 * the prompt) with ids and position kept on the device: step i reads the ids step i-1 produced,
 * starting from d_first_ids [B] at position n.  The launch sequence of one step is captured in a
 * CUDA graph on first use and replayed, so the host issues one call per token instead of several
 * hundred launches.  d_out_ids: NULL or [steps, B] int64 (row i = ids produced by step i).
 * Asynchronous.  While per-kernel timing is on (caten_b200_profile_begin) the steps are launched
 * one kernel at a time instead. */
int caten_b200_gpt2_decode(caten_b200_gpt2 *m, const int64_t *d_first_ids, int64_t n, int64_t steps,
                           int64_t *d_out_ids);
/* Device pointer to the [B, V] fp32 logits of the last step (valid until the next step). */
const float *caten_b200_gpt2_logits(caten_b200_gpt2 *m);
/* Device pointers to layer l's caches, [B, H, T, 64] fp32. */
int caten_b200_gpt2_kv(caten_b200_gpt2 *m, int layer, float **d_k, float **d_v);
/* Number of kernel launches issued by this model's steps since creation. */
int64_t caten_b200_gpt2_launch_count(caten_b200_gpt2 *m);

/* ---- multi-GPU plane -------------------------------------------------------------------------------
 * No counterpart in the reference (multi-device execution is an item of its roadmap, Readme.md:181);
 * these entries let a host that cannot use torch.distributed (Common Lisp through CFFI) run the
 * batch-sharded configurations: one process per GPU, contiguous slices of the batch per rank,
 * weights replicated.  Sequences never interact (external/llm/layers.lisp:35-51), so the only
 * collectives are the two below; both are NCCL calls queued on the context's stream.  NCCL is bound
 * at run time (dlopen of libnccl.so.2); on a host without it only world == 1 works. */
#define CATEN_B200_DIST_ID_BYTES 128
/* Rank 0 creates the group id (an ncclUniqueId, 128 bytes) and hands it to the other ranks by any
 * means the host has (a file, the environment, a socket). */
int caten_b200_dist_unique_id(void *id128);
/* Joins the group: collective over all `world` ranks.  world == 1 needs no id and no NCCL. */
int caten_b200_dist_init(caten_b200_ctx *ctx, int rank, int world, const void *id128);
int caten_b200_dist_finalize(caten_b200_ctx *ctx);
int caten_b200_dist_rank(caten_b200_ctx *ctx);
int caten_b200_dist_world(caten_b200_ctx *ctx);
/* Contiguous slice [*first, *first + *count) of `batch` sequences owned by `rank`; earlier ranks take
 * the remainder. */
int caten_b200_dist_shard(int64_t batch, int world, int rank, int64_t *first, int64_t *count);
/* Broadcasts `bytes` bytes at d_arena (the file's tensor data / the packed weight arena) from rank
 * `root` to every rank, in place; each rank then calls caten_b200_weight_upload_device on its copy. */
int caten_b200_dist_bcast_weights(caten_b200_ctx *ctx, void *d_arena, size_t bytes, int root);
/* All-gather of next-token ids: every rank contributes n_per_rank int64 (slices padded to the largest),
 * d_all receives [world, n_per_rank] in rank order on every rank. */
int caten_b200_dist_gather_ids(caten_b200_ctx *ctx, const int64_t *d_local, int64_t n_per_rank, int64_t *d_all);

/* ---- generic schedule item ------------------------------------------------------------------------
 * One fused element-wise (optionally reducing) kernel of the scheduler, i.e. what
 * source/byoc/clang.lisp:163-205 renders as one C function from a Schedule-Item's :EXPR nodes
 * (source/codegen/renderer.lisp:331-410): a loop nest over an iteration space, strided views of the
 * operands (source/aasm/attrs.lisp:265-283), an expression over the aIR ops of
 * source/aasm/attrs.lisp:42-216, and one store.  Instead of rendering and compiling C at run time
 * the expression is handed over as a short postfix program that one CUDA kernel interprets per
 * element, so any such item runs under BACKEND=B200 without a compiler on the host.
 *
 * Value classes: F32 (fp32), I32 (int32; int64 buffers are read/written through int32), BOOL (0/1).
 * A program word is  opcode | arg << 8 | class << 16.  The classes of the operands must already
 * agree (insert CAST as the reference's graph does).  Float arithmetic is fp32; SIN / EXP2 / LOG2 /
 * SQRT go through double and are rounded once, which is what the C the reference renders computes
 * (double libm functions applied to a float). */
enum {
  CATEN_B200_OP_LOAD = 1,   /* arg = operand index: push the operand's element at the current index */
  CATEN_B200_OP_CONST = 2,  /* arg = index into consts[] (bit pattern of a float or an int32) */
  CATEN_B200_OP_INDEX = 3,  /* arg = axis: push the loop index of that axis as I32 (:INDEX-COMPONENTS of one axis) */
  CATEN_B200_OP_NEG = 10, CATEN_B200_OP_RECIP, CATEN_B200_OP_SIN, CATEN_B200_OP_EXP2, CATEN_B200_OP_LOG2,
  CATEN_B200_OP_SQRT, CATEN_B200_OP_NOT,
  CATEN_B200_OP_CAST,       /* arg = class of the operand; class field = class of the result */
  CATEN_B200_OP_ADD = 30, CATEN_B200_OP_MUL, CATEN_B200_OP_MOD, CATEN_B200_OP_IDIV, CATEN_B200_OP_AND,
  CATEN_B200_OP_OR, CATEN_B200_OP_XOR, CATEN_B200_OP_MAX,
  CATEN_B200_OP_NE, CATEN_B200_OP_LT,   /* (a b -- bool); class field = class of a and b */
  CATEN_B200_OP_WHERE = 50  /* (cond a b -- cond ? a : b) */
};
enum { CATEN_B200_CLS_F32 = 0, CATEN_B200_CLS_I32 = 1, CATEN_B200_CLS_BOOL = 2 };
/* element types of operand and output buffers */
enum { CATEN_B200_DT_F32 = 0, CATEN_B200_DT_I32 = 1, CATEN_B200_DT_I64 = 2, CATEN_B200_DT_U8 = 3 };
enum { CATEN_B200_RED_NONE = 0, CATEN_B200_RED_SUM = 1, CATEN_B200_RED_MAX = 2 };
#define CATEN_B200_EXPR_MAX_DIMS 6
#define CATEN_B200_EXPR_MAX_OPERANDS 8
#define CATEN_B200_EXPR_MAX_CODE 96
#define CATEN_B200_EXPR_MAX_CONSTS 16
typedef struct {
  int32_t ndim;                                   /* loops, outermost first */
  int64_t shape[CATEN_B200_EXPR_MAX_DIMS];
  int32_t n_reduce;                               /* the innermost n_reduce loops are reduced into the output */
  int32_t reduce_op;                              /* CATEN_B200_RED_*; reduction runs in loop order (as the rendered C does) */
  int32_t accumulate;                             /* 1: the output's old value is the first term (the :reduction store) */
  int32_t n_operands;
  const void *operand[CATEN_B200_EXPR_MAX_OPERANDS];           /* device pointers */
  int32_t operand_dtype[CATEN_B200_EXPR_MAX_OPERANDS];
  int64_t operand_offset[CATEN_B200_EXPR_MAX_OPERANDS];        /* in elements */
  int64_t operand_stride[CATEN_B200_EXPR_MAX_OPERANDS][CATEN_B200_EXPR_MAX_DIMS]; /* in elements; 0 = broadcast */
  void *out;
  int32_t out_dtype;
  int64_t out_offset;
  int64_t out_stride[CATEN_B200_EXPR_MAX_DIMS];   /* strides of the reduced loops are ignored */
  int32_t n_code;
  uint32_t code[CATEN_B200_EXPR_MAX_CODE];
  uint32_t consts[CATEN_B200_EXPR_MAX_CONSTS];
} caten_b200_expr;
/* Runs the item.  The program must leave exactly one value; its class is converted to out_dtype. */
int caten_b200_eval_expr(caten_b200_ctx *ctx, const caten_b200_expr *e);

/* ---- per-kernel timing ----------------------------------------------------------------------------
 * Counterpart of PROFILE=1 (source/runtime/profile.lisp:15-39, source/codegen/runner.lisp:28-31),
 * which wall-clocks every node of the VM: here launches of the selected kernel classes are
 * bracketed with CUDA events on the context's stream, so asynchronous execution is kept. */
enum {
  CATEN_B200_K_EMBED = 0, CATEN_B200_K_LAYERNORM = 1, CATEN_B200_K_GEMV = 2, CATEN_B200_K_GEMM = 3,
  CATEN_B200_K_ATTN_DECODE = 4, CATEN_B200_K_ATTN_PREFILL = 5, CATEN_B200_K_ARGMAX = 6,
  CATEN_B200_K_DECODE_STEP = 7,   /* the whole single-token step of 1..4 sequences, which is one kernel */
  CATEN_B200_K_COUNT = 8
};
/* Starts timing the classes whose bit (1 << class) is set in class_mask. */
int caten_b200_profile_begin(caten_b200_ctx *ctx, unsigned class_mask);
/* Stops timing, synchronises, and writes per class the summed device milliseconds and the number
 * of timed calls into ms[CATEN_B200_K_COUNT] and calls[CATEN_B200_K_COUNT]. */
int caten_b200_profile_end(caten_b200_ctx *ctx, double *ms, int64_t *calls);

/* Library build id (sm architecture it was compiled for), e.g. "sm_100a". */
const char *caten_b200_arch(void);

#ifdef __cplusplus
}
#endif
#endif
