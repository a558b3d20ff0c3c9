// C ABI of libcaten_b200: context, device memory, weight handles, per-kernel entry points and
// the whole GPT-2 step.  See include/caten_b200.h for the contract of every function.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <vector>

#include "common.cuh"
#include "blocks32.cuh"

namespace cb {

static thread_local std::string g_err = "";

int fail(caten_b200_ctx *ctx, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  else g_err = buf;
  return code;
}

int cuda_fail(caten_b200_ctx *ctx, cudaError_t e, const char *what) {
  return fail(ctx, CATEN_B200_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

int scratch_reserve(caten_b200_ctx *ctx, Scratch *s, size_t bytes) {
  if (s->bytes >= bytes) return 0;
  if (s->ptr) CB_CUDA(ctx, cudaFree(s->ptr));  // cudaFree waits for work that may still read it
  s->ptr = nullptr;
  s->bytes = 0;
  const size_t want = bytes + bytes / 4;
  CB_CUDA(ctx, cudaMalloc(&s->ptr, want));
  s->bytes = want;
  return 0;
}

static int check_status(caten_b200_ctx *ctx) {
  if (ctx->h_status[0] != DEV_OK) {
    const int code = ctx->h_status[0], where = ctx->h_status[1], detail = ctx->h_status[2];
    ctx->h_status[0] = 0;
    ctx->device_failures++;
    cudaMemsetAsync(ctx->d_status, 0, 4 * sizeof(int), ctx->stream);
    return fail(ctx, CATEN_B200_EDEVICE, "kernel-side check failed: code %d (%s) at site %d, detail %d", code,
                code == DEV_WAIT_TIMEOUT ? "bounded wait ran out" : "bad index", where, detail);
  }
  return 0;
}

// Brackets one kernel-class call with events when that class is being profiled.
struct ProfScope {
  caten_b200_ctx *ctx;
  cudaEvent_t b = nullptr;
  ProfScope(caten_b200_ctx *c, int klass) : ctx(c) {
    if (!(ctx->prof_mask & (1u << klass))) return;
    cudaEvent_t a;
    auto get = [&]() {
      cudaEvent_t e;
      if (!ctx->prof_pool.empty()) { e = ctx->prof_pool.back(); ctx->prof_pool.pop_back(); }
      else cudaEventCreate(&e);
      return e;
    };
    a = get();
    b = get();
    cudaEventRecord(a, ctx->stream);
    ctx->prof.push_back({klass, a, b});
  }
  ~ProfScope() {
    if (b) cudaEventRecord(b, ctx->stream);
  }
};

}  // namespace cb

using namespace cb;

#define NEED_CTX(ctx)                                                              \
  do {                                                                             \
    if (!(ctx)) return cb::fail(nullptr, CATEN_B200_EINVAL, "%s: ctx is NULL", __func__); \
    cudaSetDevice((ctx)->device);                                                  \
  } while (0)

extern "C" {

const char *caten_b200_arch(void) { return "sm_100a"; }

const char *caten_b200_last_error(caten_b200_ctx *ctx) { return ctx ? ctx->err.c_str() : cb::g_err.c_str(); }

int caten_b200_init(int device, caten_b200_ctx **out) {
  if (!out) return fail(nullptr, CATEN_B200_EINVAL, "caten_b200_init: ctx out pointer is NULL");
  *out = nullptr;
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceCount");
  if (device < 0 || device >= ndev) return fail(nullptr, CATEN_B200_EINVAL, "caten_b200_init: device %d of %d", device, ndev);
  if ((e = cudaSetDevice(device)) != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceProperties");
  if (prop.major != 10)
    return fail(nullptr, CATEN_B200_EUNSUPPORTED, "caten_b200_init: device %d is sm_%d%d; this library holds sm_100a code only",
                device, prop.major, prop.minor);
  caten_b200_ctx *ctx = new (std::nothrow) caten_b200_ctx();
  if (!ctx) return fail(nullptr, CATEN_B200_ECUDA, "out of host memory");
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  if (const char *e = getenv("CATEN_B200_PDL")) ctx->use_pdl = atoi(e) != 0;
  if (const char *e = getenv("CATEN_B200_SPLITK_CLUSTER")) ctx->splitk_cluster = atoi(e);
  if (const char *e = getenv("CATEN_B200_DENSE_GEMM")) ctx->dense_gemm = atoi(e) != 0;
  if (const char *e = getenv("CATEN_B200_ATTN_PREFETCH_MB")) ctx->attn_prefetch_bytes = (long long)atoi(e) << 20;
  if (const char *e = getenv("CATEN_B200_ATTN_TC")) ctx->attn_tc = atoi(e);
  if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) { delete ctx; return cuda_fail(nullptr, e, "cudaStreamCreate"); }
  ctx->own_stream = ctx->stream;
  if ((e = cudaMalloc(&ctx->d_status, 4 * sizeof(int))) != cudaSuccess) { delete ctx; return cuda_fail(nullptr, e, "cudaMalloc"); }
  cudaMemset(ctx->d_status, 0, 4 * sizeof(int));

  if ((e = cudaMallocHost(&ctx->h_status, 4 * sizeof(int))) != cudaSuccess) { delete ctx; return cuda_fail(nullptr, e, "cudaMallocHost"); }
  for (int i = 0; i < 4; ++i) ctx->h_status[i] = 0;
  cudaDriverEntryPointQueryResult qres;
  void *fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    ctx->encode_tiled = fn;
  *out = ctx;
  return 0;
}

int caten_b200_destroy(caten_b200_ctx *ctx) {
  if (!ctx) return 0;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  caten_b200_dist_finalize(ctx);
  for (auto &r : ctx->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  for (auto e : ctx->prof_pool) cudaEventDestroy(e);
  if (ctx->xbf.ptr) cudaFree(ctx->xbf.ptr);
  if (ctx->wtmp.ptr) cudaFree(ctx->wtmp.ptr);
  if (ctx->wbf.ptr) cudaFree(ctx->wbf.ptr);
  if (ctx->upload_stage.ptr) cudaFree(ctx->upload_stage.ptr);
  for (int k = 0; k < 2; ++k) {
    if (ctx->pin[k]) cudaFreeHost(ctx->pin[k]);
    if (ctx->pin_ev[k]) cudaEventDestroy(ctx->pin_ev[k]);
  }
  cudaFree(ctx->d_status);
  cudaFreeHost(ctx->h_status);
  cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return 0;
}

void *caten_b200_stream(caten_b200_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int caten_b200_set_stream(caten_b200_ctx *ctx, void *stream) {
  NEED_CTX(ctx);
  CB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stream = stream ? (cudaStream_t)stream : ctx->own_stream;
  return 0;
}

int caten_b200_malloc(caten_b200_ctx *ctx, size_t bytes, void **d_ptr) {
  NEED_CTX(ctx);
  if (!d_ptr) return fail(ctx, CATEN_B200_EINVAL, "malloc: out pointer is NULL");
  *d_ptr = nullptr;
  if (bytes == 0) bytes = 16;
  CB_CUDA(ctx, cudaMalloc(d_ptr, bytes));
  CB_CUDA(ctx, cudaMemsetAsync(*d_ptr, 0, bytes, ctx->stream));
  return 0;
}

int caten_b200_free(caten_b200_ctx *ctx, void *d_ptr) {
  NEED_CTX(ctx);
  if (d_ptr) CB_CUDA(ctx, cudaFree(d_ptr));
  return 0;
}

// Host -> device copy queued on the context's stream.  Large sources (a memory-mapped model file, a numpy array) are
// pageable memory, which the driver copies through its own small staging area at a few GB/s; here they go through two
// 16 MiB pinned buffers of the context in alternation, so that the CPU fills one while the DMA engine drains the other.
// On return the source has been read completely (the copies themselves may still be in flight on the stream).
static constexpr size_t PIN_BYTES = (size_t)16 << 20;
static int h2d_staged(caten_b200_ctx *ctx, void *d_dst, const void *h_src, size_t bytes) {
  if (bytes < ((size_t)4 << 20)) {
    CB_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    CB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // a pageable source may still be read after the call returns otherwise
    return 0;
  }
  for (int k = 0; k < 2; ++k)
    if (!ctx->pin[k]) {
      CB_CUDA(ctx, cudaHostAlloc(&ctx->pin[k], PIN_BYTES, cudaHostAllocDefault));
      CB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->pin_ev[k], cudaEventDisableTiming));
    }
  int k = 0;
  for (size_t off = 0; off < bytes; off += PIN_BYTES, k ^= 1) {
    const size_t n = bytes - off < PIN_BYTES ? bytes - off : PIN_BYTES;
    if (ctx->pin_busy[k]) CB_CUDA(ctx, cudaEventSynchronize(ctx->pin_ev[k]));  // its previous copy has left the buffer
    memcpy(ctx->pin[k], (const char *)h_src + off, n);
    CB_CUDA(ctx, cudaMemcpyAsync((char *)d_dst + off, ctx->pin[k], n, cudaMemcpyHostToDevice, ctx->stream));
    CB_CUDA(ctx, cudaEventRecord(ctx->pin_ev[k], ctx->stream));
    ctx->pin_busy[k] = true;
  }
  return 0;
}

int caten_b200_h2d(caten_b200_ctx *ctx, void *d_dst, const void *h_src, size_t bytes) {
  NEED_CTX(ctx);
  if (bytes && (!d_dst || !h_src)) return fail(ctx, CATEN_B200_EINVAL, "h2d: NULL pointer");
  if (int rc = h2d_staged(ctx, d_dst, h_src, bytes)) return rc;
  CB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return 0;
}

int caten_b200_d2h(caten_b200_ctx *ctx, void *h_dst, const void *d_src, size_t bytes) {
  NEED_CTX(ctx);
  if (bytes && (!h_dst || !d_src)) return fail(ctx, CATEN_B200_EINVAL, "d2h: NULL pointer");
  CB_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return caten_b200_sync(ctx);
}

int caten_b200_d2d(caten_b200_ctx *ctx, void *d_dst, const void *d_src, size_t bytes) {
  NEED_CTX(ctx);
  if (bytes && (!d_dst || !d_src)) return fail(ctx, CATEN_B200_EINVAL, "d2d: NULL pointer");
  CB_CUDA(ctx, cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return 0;
}

int caten_b200_memset(caten_b200_ctx *ctx, void *d_dst, int byte, size_t bytes) {
  NEED_CTX(ctx);
  CB_CUDA(ctx, cudaMemsetAsync(d_dst, byte, bytes, ctx->stream));
  return 0;
}

int caten_b200_sync(caten_b200_ctx *ctx) {
  NEED_CTX(ctx);
  CB_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, 4 * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  CB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return check_status(ctx);
}

int caten_b200_profile_begin(caten_b200_ctx *ctx, unsigned class_mask) {
  NEED_CTX(ctx);
  for (auto &r : ctx->prof) { ctx->prof_pool.push_back(r.a); ctx->prof_pool.push_back(r.b); }
  ctx->prof.clear();
  ctx->prof_mask = class_mask;
  return 0;
}

int caten_b200_profile_end(caten_b200_ctx *ctx, double *ms, int64_t *calls) {
  NEED_CTX(ctx);
  ctx->prof_mask = 0;
  if (!ms || !calls) return fail(ctx, CATEN_B200_EINVAL, "profile_end: NULL output");
  for (int i = 0; i < CATEN_B200_K_COUNT; ++i) { ms[i] = 0.0; calls[i] = 0; }
  CB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto &r : ctx->prof) {
    float t = 0.0f;
    if (cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess) { ms[r.klass] += t; calls[r.klass]++; }
    ctx->prof_pool.push_back(r.a);
    ctx->prof_pool.push_back(r.b);
  }
  ctx->prof.clear();
  return 0;
}

// ------------------------------------------------------------------------------------------------
// weights
// ------------------------------------------------------------------------------------------------
int64_t caten_b200_weight_nbytes(int type, int64_t rows, int64_t cols) {
  const int64_t n = rows * cols;
  switch (type) {
    case CATEN_B200_F32: return n * 4;
    case CATEN_B200_F16: return n * 2;
    case CATEN_B200_Q4_0: case CATEN_B200_Q4_1: case CATEN_B200_Q5_0: case CATEN_B200_Q5_1: case CATEN_B200_Q8_0:
      return cols % 32 ? -1 : n / 32 * cb::type_block_bytes(type);
  }
  return cb::extra_type_nbytes(type, n, cols);
}

int caten_b200_weight_upload_device(caten_b200_ctx *ctx, int type, const void *d_blocks, int64_t rows, int64_t cols,
                                    caten_b200_weight **out) {
  NEED_CTX(ctx);
  if (!out) return fail(ctx, CATEN_B200_EINVAL, "weight_upload: out pointer is NULL");
  *out = nullptr;
  if (!d_blocks || rows <= 0 || cols <= 0) return fail(ctx, CATEN_B200_EINVAL, "weight_upload: NULL data or empty shape %lldx%lld", (long long)rows, (long long)cols);
  const int64_t nbytes = caten_b200_weight_nbytes(type, rows, cols);
  if (nbytes < 0)
    return fail(ctx, CATEN_B200_EUNSUPPORTED, "weight_upload: ggml type %d with cols=%lld (types: F32=0 F16=1 Q4_0=2 Q4_1=3 Q5_0=6 Q5_1=7 Q8_0=8 Q2_K=10 Q3_K=11 Q4_K=12 Q5_K=13 Q6_K=14; cols a multiple of the block size)", type, (long long)cols);
  caten_b200_weight *w = new (std::nothrow) caten_b200_weight();
  if (!w) return fail(ctx, CATEN_B200_ECUDA, "out of host memory");
  w->type = type; w->rows = rows; w->cols = cols; w->ctx = ctx;
  cudaError_t e;
  if (cb::extra_type_nbytes(type, rows * cols, cols) >= 0) {
    // a block format the kernels do not consume packed: expand to fp32 now, keep an fp32 weight
    w->type = CATEN_B200_F32;
    w->device_bytes = rows * cols * (int64_t)sizeof(float);
    if ((e = cudaMalloc(&w->qs, (size_t)(rows * cols) * sizeof(float))) != cudaSuccess) { delete w; return cuda_fail(ctx, e, "cudaMalloc(weight)"); }
    if (int rc = launch_dequant_extra(ctx, type, (const uint8_t *)d_blocks, rows * cols, (float *)w->qs)) { cudaFree(w->qs); delete w; return rc; }
  } else if (type == CATEN_B200_F32 || type == CATEN_B200_F16) {
    w->device_bytes = nbytes;
    if ((e = cudaMalloc(&w->qs, (size_t)nbytes)) != cudaSuccess) { delete w; return cuda_fail(ctx, e, "cudaMalloc(weight)"); }
    if ((e = cudaMemcpyAsync(w->qs, d_blocks, (size_t)nbytes, cudaMemcpyDeviceToDevice, ctx->stream)) != cudaSuccess) {
      cudaFree(w->qs); delete w; return cuda_fail(ctx, e, "cudaMemcpyAsync(weight)");
    }
  } else {
    // the 32-weight block formats stay packed: codes, scales, minima and fifth bits as separate arrays
    w->nkb = cols / 32;
    const int64_t nblocks = rows * w->nkb;
    const size_t qbytes = (size_t)nblocks * cb::type_code_bytes(type);
    auto drop = [&]() { cudaFree(w->qs); cudaFree(w->d); cudaFree(w->m); cudaFree(w->qh); delete w; };
    if ((e = cudaMalloc(&w->qs, qbytes)) != cudaSuccess) { drop(); return cuda_fail(ctx, e, "cudaMalloc(weight codes)"); }
    // 16 spare bytes: the single-kernel decode step fetches scales in whole 16-byte pieces
    if ((e = cudaMalloc((void **)&w->d, (size_t)nblocks * 2 + 16)) != cudaSuccess) { drop(); return cuda_fail(ctx, e, "cudaMalloc(weight scales)"); }
    cudaMemsetAsync((uint8_t *)w->d + (size_t)nblocks * 2, 0, 16, ctx->stream);
    w->device_bytes = (int64_t)qbytes + nblocks * 2;
    if (cb::type_has_min(type)) {
      if ((e = cudaMalloc((void **)&w->m, (size_t)nblocks * 2)) != cudaSuccess) { drop(); return cuda_fail(ctx, e, "cudaMalloc(weight minima)"); }
      w->device_bytes += nblocks * 2;
    }
    if (cb::type_has_qh(type)) {
      if ((e = cudaMalloc((void **)&w->qh, (size_t)nblocks * 4)) != cudaSuccess) { drop(); return cuda_fail(ctx, e, "cudaMalloc(weight fifth bits)"); }
      w->device_bytes += nblocks * 4;
    }
    if (int rc = launch_repack(ctx, type, (const uint8_t *)d_blocks, nblocks, w->qs, w->d, w->m, w->qh)) { drop(); return rc; }
  }
  ctx->weights_pending = true;  // the next kernel launch must not start reading weights early
  *out = w;
  return 0;
}

int caten_b200_weight_upload(caten_b200_ctx *ctx, int type, const void *h_blocks, int64_t rows, int64_t cols,
                             caten_b200_weight **out) {
  NEED_CTX(ctx);
  if (!out) return fail(ctx, CATEN_B200_EINVAL, "weight_upload: out pointer is NULL");
  *out = nullptr;
  if (!h_blocks || rows <= 0 || cols <= 0) return fail(ctx, CATEN_B200_EINVAL, "weight_upload: NULL data or empty shape %lldx%lld", (long long)rows, (long long)cols);
  const int64_t nbytes = caten_b200_weight_nbytes(type, rows, cols);
  if (nbytes < 0)
    return fail(ctx, CATEN_B200_EUNSUPPORTED, "weight_upload: ggml type %d with cols=%lld (types: F32=0 F16=1 Q4_0=2 Q4_1=3 Q5_0=6 Q5_1=7 Q8_0=8 Q2_K=10 Q3_K=11 Q4_K=12 Q5_K=13 Q6_K=14; cols a multiple of the block size)", type, (long long)cols);
  // file / host bytes -> pinned bounce buffers -> a staging area on the device (kept by the context and reused by
  // the next upload: work on the stream is ordered, so the re-layout kernel has read it before it is overwritten)
  if (int rc = scratch_reserve(ctx, &ctx->upload_stage, (size_t)nbytes)) return rc;
  if (int rc = h2d_staged(ctx, ctx->upload_stage.ptr, h_blocks, (size_t)nbytes)) return rc;
  const int rc = caten_b200_weight_upload_device(ctx, type, ctx->upload_stage.ptr, rows, cols, out);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->upload_stage.bytes > ((size_t)128 << 20)) {  // a large dense tensor went through: do not keep that much
    cudaFree(ctx->upload_stage.ptr);
    ctx->upload_stage = cb::Scratch();
  }
  return rc;
}

int caten_b200_weight_free(caten_b200_ctx *ctx, caten_b200_weight *w) {
  NEED_CTX(ctx);
  if (!w) return 0;
  if (w->qs) cudaFree(w->qs);
  if (w->d) cudaFree(w->d);
  if (w->m) cudaFree(w->m);
  if (w->qh) cudaFree(w->qh);
  delete w;
  return 0;
}

int64_t caten_b200_weight_device_nbytes(const caten_b200_weight *w) { return w ? w->device_bytes : -1; }

int caten_b200_weight_dequant(caten_b200_ctx *ctx, const caten_b200_weight *w, float *d_out) {
  NEED_CTX(ctx);
  if (!w || !d_out) return fail(ctx, CATEN_B200_EINVAL, "weight_dequant: NULL argument");
  return launch_dequant(ctx, w, d_out);
}

// ------------------------------------------------------------------------------------------------
// kernels
// ------------------------------------------------------------------------------------------------
static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

int caten_b200_linear(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *d_x, const float *d_bias,
                      const float *d_residual, int act, float *d_y, int64_t M, int precision) {
  NEED_CTX(ctx);
  if (!w || !d_x || !d_y) return fail(ctx, CATEN_B200_EINVAL, "linear: NULL argument");
  if (M < 0) return fail(ctx, CATEN_B200_EINVAL, "linear: M < 0");
  if (M == 0) return 0;
  if (act < 0 || act > 2) return fail(ctx, CATEN_B200_EINVAL, "linear: unknown activation %d", act);
  if (!aligned16(d_x) || !aligned16(d_y)) return fail(ctx, CATEN_B200_EINVAL, "linear: x and y must be 16-byte aligned");
  ProfScope prof(ctx, M <= 4 ? CATEN_B200_K_GEMV : CATEN_B200_K_GEMM);
  if (M <= 4) {
    for (int64_t m = 0; m < M; ++m)
      if (int rc = launch_gemv(ctx, w, d_x + m * w->cols, d_bias, d_residual ? d_residual + m * w->rows : nullptr, act,
                               d_y + m * w->rows))
        return rc;
    return 0;
  }
  switch (precision) {
    case CATEN_B200_PREC_FP32: return launch_gemm_simt(ctx, w, d_x, d_bias, d_residual, act, d_y, M);
    case CATEN_B200_PREC_BF16: return launch_gemm_tc(ctx, w, d_x, d_bias, d_residual, act, d_y, M, 1);
    case CATEN_B200_PREC_BF16X3: return launch_gemm_tc(ctx, w, d_x, d_bias, d_residual, act, d_y, M, 3);
  }
  return fail(ctx, CATEN_B200_EINVAL, "linear: unknown precision %d", precision);
}

int caten_b200_linear_noalloc(caten_b200_ctx *ctx, const caten_b200_weight *w, const float *d_x, const float *d_bias,
                              const float *d_residual, int act, float *d_y, int64_t M, int precision) {
  NEED_CTX(ctx);
  if (!w || !d_x || !d_y) return fail(ctx, CATEN_B200_EINVAL, "linear_noalloc: NULL argument");
  if (M < 0) return fail(ctx, CATEN_B200_EINVAL, "linear_noalloc: M < 0");
  if (M == 0) return 0;
  if (act < 0 || act > 2) return fail(ctx, CATEN_B200_EINVAL, "linear_noalloc: unknown activation %d", act);
  if (!aligned16(d_x) || !aligned16(d_y)) return fail(ctx, CATEN_B200_EINVAL, "linear_noalloc: x and y must be 16-byte aligned");
  ProfScope prof(ctx, M <= 4 ? CATEN_B200_K_GEMV : CATEN_B200_K_GEMM);
  if (M <= 4) {  // the dequant-GEMV uses no scratch memory
    for (int64_t m = 0; m < M; ++m)
      if (int rc = launch_gemv(ctx, w, d_x + m * w->cols, d_bias, d_residual ? d_residual + m * w->rows : nullptr, act,
                               d_y + m * w->rows))
        return rc;
    return 0;
  }
  switch (precision) {
    case CATEN_B200_PREC_FP32: return launch_gemm_simt(ctx, w, d_x, d_bias, d_residual, act, d_y, M);  // no scratch either
    case CATEN_B200_PREC_BF16: return launch_gemm_tc_noalloc(ctx, w, d_x, d_bias, d_residual, act, d_y, M, 1);
    case CATEN_B200_PREC_BF16X3: return launch_gemm_tc_noalloc(ctx, w, d_x, d_bias, d_residual, act, d_y, M, 3);
  }
  return fail(ctx, CATEN_B200_EINVAL, "linear_noalloc: unknown precision %d", precision);
}

int caten_b200_relu_matmul(caten_b200_ctx *ctx, const float *d_a, const float *d_b, float *d_c, int64_t M, int64_t K,
                           int64_t N, int precision) {
  NEED_CTX(ctx);
  if (!d_a || !d_b || !d_c) return fail(ctx, CATEN_B200_EINVAL, "relu_matmul: NULL argument");
  if (M < 0 || K <= 0 || N < 0) return fail(ctx, CATEN_B200_EINVAL, "relu_matmul: bad shape");
  ProfScope prof(ctx, CATEN_B200_K_GEMM);
  switch (precision) {
    case CATEN_B200_PREC_FP32: return launch_relu_matmul_simt(ctx, d_a, d_b, d_c, M, K, N);
    case CATEN_B200_PREC_BF16: return launch_relu_matmul_tc(ctx, d_a, d_b, d_c, M, K, N, 1);
    case CATEN_B200_PREC_BF16X3: return launch_relu_matmul_tc(ctx, d_a, d_b, d_c, M, K, N, 3);
  }
  return fail(ctx, CATEN_B200_EINVAL, "relu_matmul: unknown precision %d", precision);
}

int caten_b200_layernorm(caten_b200_ctx *ctx, const float *d_x, const float *d_gamma, const float *d_beta, float *d_y,
                         int64_t rows, int64_t d, float eps) {
  NEED_CTX(ctx);
  if (!d_x || !d_gamma || !d_beta || !d_y) return fail(ctx, CATEN_B200_EINVAL, "layernorm: NULL argument");
  if (rows < 0 || d <= 0) return fail(ctx, CATEN_B200_EINVAL, "layernorm: bad shape");
  ProfScope prof(ctx, CATEN_B200_K_LAYERNORM);
  return launch_layernorm(ctx, d_x, d_gamma, d_beta, d_y, rows, d, eps);
}

int caten_b200_embed(caten_b200_ctx *ctx, const float *d_ids_f32, const int64_t *d_ids_i64, const float *d_wte,
                     const float *d_wpe, float *d_out, int64_t B, int64_t s, int64_t n, int64_t d, int64_t V, int64_t T) {
  NEED_CTX(ctx);
  if (!d_wte || !d_wpe || !d_out) return fail(ctx, CATEN_B200_EINVAL, "embed: NULL argument");
  if (B < 0 || s < 0 || d <= 0) return fail(ctx, CATEN_B200_EINVAL, "embed: bad shape");
  return launch_embed(ctx, d_ids_f32, d_ids_i64, d_wte, d_wpe, d_out, B, s, n, d, V, T);
}

int caten_b200_attention(caten_b200_ctx *ctx, const float *d_qkv, float *d_kcache, float *d_vcache, float *d_out,
                         int64_t B, int64_t s, int64_t n, int64_t H, int64_t T) {
  NEED_CTX(ctx);
  if (!d_qkv || !d_kcache || !d_vcache || !d_out) return fail(ctx, CATEN_B200_EINVAL, "attention: NULL argument");
  if (B < 0 || s < 0 || H <= 0 || T <= 0) return fail(ctx, CATEN_B200_EINVAL, "attention: bad shape");
  ProfScope prof(ctx, s == 1 ? CATEN_B200_K_ATTN_DECODE : CATEN_B200_K_ATTN_PREFILL);
  return launch_attention(ctx, d_qkv, d_kcache, d_vcache, d_out, B, s, n, H, T);
}

int caten_b200_attention_ex(caten_b200_ctx *ctx, const float *d_qkv, float *d_kcache, float *d_vcache, float *d_out,
                            int64_t B, int64_t s, int64_t n, int64_t H, int64_t T, int precision) {
  NEED_CTX(ctx);
  if (!d_qkv || !d_kcache || !d_vcache || !d_out) return fail(ctx, CATEN_B200_EINVAL, "attention: NULL argument");
  if (B < 0 || s < 0 || H <= 0 || T <= 0) return fail(ctx, CATEN_B200_EINVAL, "attention: bad shape");
  if (precision != CATEN_B200_PREC_FP32 && precision != CATEN_B200_PREC_BF16 && precision != CATEN_B200_PREC_BF16X3)
    return fail(ctx, CATEN_B200_EINVAL, "attention: unknown precision %d", precision);
  ProfScope prof(ctx, s == 1 ? CATEN_B200_K_ATTN_DECODE : CATEN_B200_K_ATTN_PREFILL);
  return launch_attention(ctx, d_qkv, d_kcache, d_vcache, d_out, B, s, n, H, T, nullptr, cb::BfOut(), nullptr,
                          precision != CATEN_B200_PREC_FP32);
}

int caten_b200_argmax(caten_b200_ctx *ctx, const float *d_x, int64_t rows, int64_t V, int64_t *d_out) {
  NEED_CTX(ctx);
  if (!d_x || !d_out) return fail(ctx, CATEN_B200_EINVAL, "argmax: NULL argument");
  return launch_argmax(ctx, d_x, rows, V, d_out);
}

int caten_b200_sample(caten_b200_ctx *ctx, const float *d_logits, int64_t rows, int64_t V, float temperature, int top_k,
                      const float *d_uniform, int64_t *d_out) {
  NEED_CTX(ctx);
  if (!d_logits || !d_out) return fail(ctx, CATEN_B200_EINVAL, "sample: NULL argument");
  if (V <= 0) return fail(ctx, CATEN_B200_EINVAL, "sample: V=%lld", (long long)V);
  if (!(temperature > 0.0f)) return launch_argmax(ctx, d_logits, rows, V, d_out);
  if (!d_uniform) return fail(ctx, CATEN_B200_EINVAL, "sample: uniform numbers are NULL");
  return launch_sample(ctx, d_logits, rows, V, temperature, top_k, d_uniform, d_out);
}

int caten_b200_eval_expr(caten_b200_ctx *ctx, const caten_b200_expr *e) {
  NEED_CTX(ctx);
  if (!e) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: NULL argument");
  return launch_expr(ctx, e);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// whole model
// ------------------------------------------------------------------------------------------------
struct caten_b200_gpt2 {
  caten_b200_ctx *ctx = nullptr;
  caten_b200_gpt2_desc desc;
  std::vector<const float *> ln1_g, ln1_b, attn_b, proj_b, ln2_g, ln2_b, fc_b, mproj_b;
  std::vector<const caten_b200_weight *> attn_w, proj_w, fc_w, mproj_w;
  std::vector<float *> kc, vc;
  int64_t max_rows = 0;
  float *h = nullptr, *h2 = nullptr, *xn = nullptr, *qkv = nullptr, *att = nullptr, *ff = nullptr;
  float *last = nullptr, *logits = nullptr;
  // split bf16 (hi, lo) copies of the activations that feed tensor-core GEMMs, written directly by
  // the kernels that produce them (LayerNorm, attention, the GELU epilogue); unused with PREC_FP32
  cb::BfOut xn_bf, att_bf, ff_bf, last_bf;
  void *bf_arena = nullptr;
  float *ids_f32 = nullptr;  // staging for host ids [B * T]
  int64_t *out_ids = nullptr;
  float *h_ids_pinned = nullptr;
  int64_t *h_out_pinned = nullptr;
  int64_t launches0 = 0;
  // decode replayed from a CUDA graph: position and ids live on the device
  int *d_pos = nullptr, *h_pos_pinned = nullptr;
  int64_t *ids_io = nullptr;   // [B] input ids of the next step
  int64_t *ids_hist = nullptr; // [T, B] row n = ids produced by the step that started at position n
  cudaGraphExec_t graph = nullptr;
  void *graph_xbf = nullptr, *graph_wtmp = nullptr;  // scratch pointers baked into the graph
  int64_t launches_per_step = 0;
  // 1..4 sequences: the whole single-token step is one kernel (decode_small.cu); CATEN_B200_PERSISTENT=0 keeps
  // the kernel-per-operation path
  cb::DecodeSmall *ds = nullptr;
  int64_t ds_failures_seen = 0;
  bool defer_reduce = true;  // CATEN_B200_DEFER_REDUCE=0 keeps a reduction kernel behind every split-K linear
};

// Linear inside the model: with a tensor-core precision and more than 4 rows the input arrives
// already split into bf16 (hi, lo) from its producer and the output can be requested the same way.
static int model_linear(caten_b200_gpt2 *m, const caten_b200_weight *w, const float *x, cb::BfOut xbf, const float *bias,
                        const float *res, int act, float *y, cb::BfOut ybf, int64_t M, cb::PartIn *defer = nullptr) {
  if (defer) *defer = cb::PartIn();
  caten_b200_ctx *ctx = m->ctx;
  const int prec = m->desc.precision;
  if (prec == CATEN_B200_PREC_FP32 || M <= 4) return caten_b200_linear(ctx, w, x, bias, res, act, y, M, prec);
  ProfScope prof(ctx, CATEN_B200_K_GEMM);
  const int nsplit = prec == CATEN_B200_PREC_BF16X3 ? 3 : 1;
  return launch_gemm_tc_ex(ctx, w, nullptr, xbf.hi, nsplit == 3 ? xbf.lo : nullptr, bias, res, act, y, ybf, M, nsplit, defer);
}

extern "C" {

int caten_b200_gpt2_create(caten_b200_ctx *ctx, const caten_b200_gpt2_desc *dsc, caten_b200_gpt2 **out) {
  NEED_CTX(ctx);
  if (!dsc || !out) return fail(ctx, CATEN_B200_EINVAL, "gpt2_create: NULL argument");
  *out = nullptr;
  const int64_t L = dsc->n_layers, d = dsc->d_model, H = dsc->n_heads, V = dsc->vocab, T = dsc->max_seq_len, B = dsc->batch;
  if (L <= 0 || d <= 0 || H <= 0 || V <= 0 || T <= 0 || B <= 0) return fail(ctx, CATEN_B200_EINVAL, "gpt2_create: non-positive size");
  if (d != H * 64) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gpt2_create: head dim %lld/%lld; the attention kernels cover head dim 64 (all GPT-2 sizes)", (long long)d, (long long)H);
  if (!dsc->wte || !dsc->wpe || !dsc->lnf_g || !dsc->lnf_b || !dsc->lm_head) return fail(ctx, CATEN_B200_EINVAL, "gpt2_create: NULL top-level weight");
  if (dsc->lm_head->rows != V || dsc->lm_head->cols != d) return fail(ctx, CATEN_B200_EINVAL, "gpt2_create: lm_head is %lldx%lld, expected %lldx%lld", (long long)dsc->lm_head->rows, (long long)dsc->lm_head->cols, (long long)V, (long long)d);
  caten_b200_gpt2 *m = new (std::nothrow) caten_b200_gpt2();
  if (!m) return fail(ctx, CATEN_B200_ECUDA, "out of host memory");
  m->ctx = ctx;
  if (const char *e = getenv("CATEN_B200_DEFER_REDUCE")) m->defer_reduce = atoi(e) != 0;
  m->desc = *dsc;
  for (int64_t l = 0; l < L; ++l) {
    const caten_b200_weight *ws[4] = {dsc->attn_w[l], dsc->proj_w[l], dsc->fc_w[l], dsc->mproj_w[l]};
    const int64_t er[4] = {3 * d, d, 4 * d, d}, ec[4] = {d, d, d, 4 * d};
    for (int i = 0; i < 4; ++i)
      if (!ws[i] || ws[i]->rows != er[i] || ws[i]->cols != ec[i]) {
        delete m;
        return fail(ctx, CATEN_B200_EINVAL, "gpt2_create: layer %lld weight %d has the wrong shape", (long long)l, i);
      }
    m->ln1_g.push_back(dsc->ln1_g[l]); m->ln1_b.push_back(dsc->ln1_b[l]);
    m->attn_b.push_back(dsc->attn_b[l]); m->proj_b.push_back(dsc->proj_b[l]);
    m->ln2_g.push_back(dsc->ln2_g[l]); m->ln2_b.push_back(dsc->ln2_b[l]);
    m->fc_b.push_back(dsc->fc_b[l]); m->mproj_b.push_back(dsc->mproj_b[l]);
    m->attn_w.push_back(ws[0]); m->proj_w.push_back(ws[1]); m->fc_w.push_back(ws[2]); m->mproj_w.push_back(ws[3]);
  }
  int64_t max_rows = dsc->max_rows > 0 ? dsc->max_rows : 8192;
  if (dsc->max_rows <= 0)
    if (const char *e = getenv("CATEN_B200_MAX_ROWS")) { const long v = atol(e); if (v >= 1 && v <= (1 << 20)) max_rows = v; }
  if (max_rows < B) max_rows = B;  // a decode step processes the whole batch at once
  m->max_rows = max_rows;
  auto alloc = [&](float **p, int64_t n) { return caten_b200_malloc(ctx, (size_t)n * sizeof(float), (void **)p); };
  int rc = 0;
  const int64_t kv = B * H * T * 64;
  for (int64_t l = 0; l < L && !rc; ++l) {
    float *k = nullptr, *v = nullptr;
    rc = alloc(&k, kv);
    if (!rc) rc = alloc(&v, kv);
    m->kc.push_back(k); m->vc.push_back(v);
  }
  if (!rc) rc = alloc(&m->h, max_rows * d);
  if (!rc) rc = alloc(&m->h2, max_rows * d);
  if (!rc) rc = alloc(&m->xn, max_rows * d);
  if (!rc) rc = alloc(&m->qkv, max_rows * 3 * d);
  if (!rc) rc = alloc(&m->att, max_rows * d);
  if (!rc) rc = alloc(&m->ff, max_rows * 4 * d);
  if (!rc) rc = alloc(&m->last, B * d);
  if (!rc) rc = alloc(&m->logits, B * V);
  if (!rc && dsc->precision != CATEN_B200_PREC_FP32) {
    auto al = [](int64_t n) { return (size_t)((n * 2 + 1023) & ~(int64_t)1023); };
    const size_t sz_d = al(max_rows * d), sz_ff = al(max_rows * 4 * d), sz_last = al(B * d);
    rc = caten_b200_malloc(ctx, 4 * sz_d + 2 * sz_ff + 2 * sz_last, &m->bf_arena);
    if (!rc) {
      uint8_t *p = (uint8_t *)m->bf_arena;
      auto take = [&](size_t n) { __nv_bfloat16 *q = (__nv_bfloat16 *)p; p += n; return q; };
      m->xn_bf.hi = take(sz_d); m->xn_bf.lo = take(sz_d);
      m->att_bf.hi = take(sz_d); m->att_bf.lo = take(sz_d);
      m->ff_bf.hi = take(sz_ff); m->ff_bf.lo = take(sz_ff);
      m->last_bf.hi = take(sz_last); m->last_bf.lo = take(sz_last);
    }
  }
  if (!rc) rc = alloc(&m->ids_f32, B * T);
  if (!rc) rc = caten_b200_malloc(ctx, (size_t)B * sizeof(int64_t), (void **)&m->out_ids);
  if (!rc) rc = caten_b200_malloc(ctx, (size_t)B * sizeof(int64_t), (void **)&m->ids_io);
  if (!rc) rc = caten_b200_malloc(ctx, (size_t)B * T * sizeof(int64_t), (void **)&m->ids_hist);
  if (!rc) rc = caten_b200_malloc(ctx, sizeof(int), (void **)&m->d_pos);
  if (!rc && cudaMallocHost(&m->h_pos_pinned, sizeof(int)) != cudaSuccess) rc = fail(ctx, CATEN_B200_ECUDA, "cudaMallocHost(pos)");
  if (!rc && cudaMallocHost(&m->h_ids_pinned, (size_t)B * T * sizeof(float)) != cudaSuccess) rc = fail(ctx, CATEN_B200_ECUDA, "cudaMallocHost(ids)");
  if (!rc && cudaMallocHost(&m->h_out_pinned, (size_t)B * sizeof(int64_t)) != cudaSuccess) rc = fail(ctx, CATEN_B200_ECUDA, "cudaMallocHost(out ids)");
  bool persistent = true;
  if (const char *e = getenv("CATEN_B200_PERSISTENT")) persistent = atoi(e) != 0;
  if (!rc && persistent && cb::decode_small_supported(m->desc, m->attn_w.data(), m->proj_w.data(), m->fc_w.data(), m->mproj_w.data())) {
    const std::vector<const float *> vecs[8] = {m->ln1_g, m->ln1_b, m->attn_b, m->proj_b, m->ln2_g, m->ln2_b, m->fc_b, m->mproj_b};
    rc = cb::decode_small_create(ctx, m->desc, m->attn_w, m->proj_w, m->fc_w, m->mproj_w, vecs, m->kc, m->vc, m->ids_io, m->out_ids,
                                 m->ids_hist, m->d_pos, m->logits, &m->ds);
    m->ds_failures_seen = ctx->device_failures;
  }
  if (rc) { caten_b200_gpt2_destroy(m); return rc; }
  m->launches0 = ctx->launches;
  *out = m;
  return 0;
}

int caten_b200_gpt2_destroy(caten_b200_gpt2 *m) {
  if (!m) return 0;
  caten_b200_ctx *ctx = m->ctx;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (float *p : m->kc) if (p) cudaFree(p);
  for (float *p : m->vc) if (p) cudaFree(p);
  float *bufs[] = {m->h, m->h2, m->xn, m->qkv, m->att, m->ff, m->last, m->logits, m->ids_f32};
  for (float *p : bufs) if (p) cudaFree(p);
  if (m->graph) cudaGraphExecDestroy(m->graph);
  cb::decode_small_destroy(m->ds);
  if (m->bf_arena) cudaFree(m->bf_arena);
  if (m->out_ids) cudaFree(m->out_ids);
  if (m->ids_io) cudaFree(m->ids_io);
  if (m->ids_hist) cudaFree(m->ids_hist);
  if (m->d_pos) cudaFree(m->d_pos);
  if (m->h_pos_pinned) cudaFreeHost(m->h_pos_pinned);
  if (m->h_ids_pinned) cudaFreeHost(m->h_ids_pinned);
  if (m->h_out_pinned) cudaFreeHost(m->h_out_pinned);
  delete m;
  return 0;
}

// Runs the Transformer (external/llm/layers.lisp:81-90) on `nb` sequences [b0, b0+nb) of s tokens.
static int run_chunk(caten_b200_gpt2 *m, const float *ids_f32, const int64_t *ids_i64, int64_t b0, int64_t nb, int64_t s,
                     int64_t n, const int *d_n = nullptr) {
  caten_b200_ctx *ctx = m->ctx;
  const caten_b200_gpt2_desc &c = m->desc;
  const int64_t d = c.d_model, H = c.n_heads, V = c.vocab, T = c.max_seq_len, L = c.n_layers, R = nb * s;
  const int prec = c.precision;
  const float eps = c.eps;
  const int64_t kv_off = b0 * H * T * 64;
  {
    ProfScope prof(ctx, CATEN_B200_K_EMBED);
    if (int rc = launch_embed(ctx, ids_f32 ? ids_f32 + b0 * s : nullptr, ids_i64 ? ids_i64 + b0 * s : nullptr, c.wte, c.wpe,
                              m->h, nb, s, n, d, V, T, d_n))
      return rc;
  }
  // tensor-core precisions: producers write the split bf16 operand of the next GEMM themselves
  const bool fused = prec != CATEN_B200_PREC_FP32 && R > 4;
  const bool x3 = prec == CATEN_B200_PREC_BF16X3;
  auto bf = [&](cb::BfOut b) { cb::BfOut o; if (fused) { o.hi = b.hi; o.lo = x3 ? b.lo : nullptr; } return o; };
  const cb::BfOut none;
  // Single-token steps: a split-K linear whose consumer can sum the partial tiles while loading
  // (LayerNorm for the two projections, attention for qkv) skips its reduction kernel.
  const bool defer_ok = fused && s == 1 && m->defer_reduce;
  cb::PartIn pend_h, pend_qkv, pend_h2;  // pending outputs of mlp.c_proj (-> h), c_attn, attn.c_proj (-> h2)
  auto layernorm = [&](const cb::PartIn &pin, const float *res, float *x, const float *g, const float *b, float *y, int64_t rows,
                       int64_t stride, cb::BfOut o) {
    ProfScope prof(ctx, CATEN_B200_K_LAYERNORM);
    // pending: x = res + linear output is formed (and stored) by the LayerNorm kernel itself
    return pin.splits > 0 ? launch_layernorm_pending(ctx, pin, res, x, g, b, y, rows, d, eps, stride, o)
                          : launch_layernorm_strided(ctx, x, g, b, y, rows, d, eps, stride, o);
  };
  for (int64_t l = 0; l < L; ++l) {
    int rc = layernorm(pend_h, m->h2, m->h, m->ln1_g[l], m->ln1_b[l], m->xn, R, 1, bf(m->xn_bf));
    if (!rc) rc = model_linear(m, m->attn_w[l], m->xn, m->xn_bf, m->attn_b[l], nullptr, CATEN_B200_ACT_NONE, m->qkv, none, R, defer_ok ? &pend_qkv : nullptr);
    if (!rc) { ProfScope prof(ctx, s == 1 ? CATEN_B200_K_ATTN_DECODE : CATEN_B200_K_ATTN_PREFILL); rc = launch_attention(ctx, m->qkv, m->kc[l] + kv_off, m->vc[l] + kv_off, m->att, nb, s, n, H, T, d_n, bf(m->att_bf), &pend_qkv, prec != CATEN_B200_PREC_FP32 && ctx->attn_tc); }
    if (!rc) rc = model_linear(m, m->proj_w[l], m->att, m->att_bf, m->proj_b[l], m->h, CATEN_B200_ACT_NONE, m->h2, none, R, defer_ok ? &pend_h2 : nullptr);
    if (!rc) rc = layernorm(pend_h2, m->h, m->h2, m->ln2_g[l], m->ln2_b[l], m->xn, R, 1, bf(m->xn_bf));
    if (!rc) rc = model_linear(m, m->fc_w[l], m->xn, m->xn_bf, m->fc_b[l], nullptr, CATEN_B200_ACT_GELU, m->ff, bf(m->ff_bf), R);
    if (!rc) rc = model_linear(m, m->mproj_w[l], m->ff, m->ff_bf, m->mproj_b[l], m->h2, CATEN_B200_ACT_NONE, m->h, none, R, defer_ok ? &pend_h : nullptr);
    if (rc) return rc;
  }
  // ln_f on the last position of every sequence only (the reference views the last row of the
  // logits, layers.lisp:90), gathered into rows [b0, b0+nb) of `last`
  cb::BfOut lb;
  if (prec != CATEN_B200_PREC_FP32 && c.batch > 4) { lb.hi = m->last_bf.hi + b0 * d; lb.lo = x3 ? m->last_bf.lo + b0 * d : nullptr; }
  return layernorm(pend_h, m->h2, m->h, c.lnf_g, c.lnf_b, m->last + b0 * d, nb, s, lb);
}

static int decode_step_device_pos(caten_b200_gpt2 *m, int64_t n_host);

int caten_b200_gpt2_step_device(caten_b200_gpt2 *m, const float *d_ids_f32, const int64_t *d_ids_i64, int64_t s, int64_t n,
                                int64_t *d_out_ids) {
  if (!m) return fail(nullptr, CATEN_B200_EINVAL, "gpt2_step: model is NULL");
  caten_b200_ctx *ctx = m->ctx;
  cudaSetDevice(ctx->device);
  const caten_b200_gpt2_desc &c = m->desc;
  if ((d_ids_f32 == nullptr) == (d_ids_i64 == nullptr)) return fail(ctx, CATEN_B200_EINVAL, "gpt2_step: pass exactly one id array");
  if (!d_out_ids) return fail(ctx, CATEN_B200_EINVAL, "gpt2_step: out ids is NULL");
  if (s < 1 || n < 0 || n + s > c.max_seq_len)
    return fail(ctx, CATEN_B200_EINVAL, "gpt2_step: s=%lld n=%lld outside the cache (max_seq_len=%d)", (long long)s, (long long)n, c.max_seq_len);
  const int64_t B = c.batch;
  if (s == 1 && m->ds) {
    // single-token step of a few sequences: the one-kernel path, fed from the device-side state
    if (int rc = launch_begin_steps(ctx, d_ids_f32, d_ids_i64, m->ids_io, m->d_pos, n, B)) return rc;
    if (int rc = decode_step_device_pos(m, n)) return rc;
    if (d_out_ids != m->out_ids)
      CB_CUDA(ctx, cudaMemcpyAsync(d_out_ids, m->out_ids, (size_t)B * sizeof(int64_t), cudaMemcpyDeviceToDevice, ctx->stream));
    return 0;
  }
  int64_t per = m->max_rows / s;
  if (per < 1) return fail(ctx, CATEN_B200_EUNSUPPORTED, "gpt2_step: s=%lld exceeds max_rows=%lld", (long long)s, (long long)m->max_rows);
  if (per > B) per = B;
  for (int64_t b0 = 0; b0 < B; b0 += per) {
    const int64_t nb = B - b0 < per ? B - b0 : per;
    if (int rc = run_chunk(m, d_ids_f32, d_ids_i64, b0, nb, s, n)) return rc;
  }
  // lm_head (no bias, layers.lisp:79) + argmax over the vocabulary
  if (int rc = model_linear(m, c.lm_head, m->last, m->last_bf, nullptr, nullptr, CATEN_B200_ACT_NONE, m->logits, cb::BfOut(), B)) return rc;
  ProfScope prof(ctx, CATEN_B200_K_ARGMAX);
  return launch_argmax(ctx, m->logits, B, c.vocab, d_out_ids);
}

static int decode_run(caten_b200_gpt2 *m, int64_t n, int64_t steps);

int caten_b200_gpt2_step(caten_b200_gpt2 *m, const float *h_ids_f32, int64_t s, int64_t n, int64_t *h_out_ids) {
  if (!m) return fail(nullptr, CATEN_B200_EINVAL, "gpt2_step: model is NULL");
  caten_b200_ctx *ctx = m->ctx;
  cudaSetDevice(ctx->device);
  const int64_t B = m->desc.batch;
  if (!h_ids_f32 || !h_out_ids) return fail(ctx, CATEN_B200_EINVAL, "gpt2_step: NULL host buffer");
  if (s < 1 || s > m->desc.max_seq_len) return fail(ctx, CATEN_B200_EINVAL, "gpt2_step: s=%lld", (long long)s);
  memcpy(m->h_ids_pinned, h_ids_f32, (size_t)(B * s) * sizeof(float));
  CB_CUDA(ctx, cudaMemcpyAsync(m->ids_f32, m->h_ids_pinned, (size_t)(B * s) * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  if (s == 1 && ctx->prof_mask == 0) {
    // single-token step: the captured graph of the step is replayed (ids and position are loaded
    // into the device-side state first); the result is the same as the kernel-by-kernel path
    if (n < 0 || n + 1 > m->desc.max_seq_len)
      return fail(ctx, CATEN_B200_EINVAL, "gpt2_step: s=1 n=%lld outside the cache (max_seq_len=%d)", (long long)n, m->desc.max_seq_len);
    if (int rc = launch_begin_steps(ctx, m->ids_f32, nullptr, m->ids_io, m->d_pos, n, B)) return rc;
    if (int rc = decode_run(m, n, 1)) return rc;
  } else if (int rc = caten_b200_gpt2_step_device(m, m->ids_f32, nullptr, s, n, m->out_ids)) {
    return rc;
  }
  CB_CUDA(ctx, cudaMemcpyAsync(m->h_out_pinned, m->out_ids, (size_t)B * sizeof(int64_t), cudaMemcpyDeviceToHost, ctx->stream));
  if (int rc = caten_b200_sync(ctx)) return rc;
  memcpy(h_out_ids, m->h_out_pinned, (size_t)B * sizeof(int64_t));
  return 0;
}

// One decode step whose position and ids are read from device memory, so that the identical
// launch sequence can be replayed from a CUDA graph.
static int decode_step_device_pos(caten_b200_gpt2 *m, int64_t n_host) {
  caten_b200_ctx *ctx = m->ctx;
  const caten_b200_gpt2_desc &c = m->desc;
  if (m->ds) {
    if (m->ds_failures_seen != ctx->device_failures) {   // an interrupted step left half-written exchange words
      if (int rc = cb::decode_small_reset(ctx, m->ds)) return rc;
      m->ds_failures_seen = ctx->device_failures;
    }
    ProfScope prof(ctx, CATEN_B200_K_DECODE_STEP);
    return cb::decode_small_launch(ctx, m->ds);
  }
  if (int rc = run_chunk(m, nullptr, m->ids_io, 0, c.batch, 1, n_host, m->d_pos)) return rc;
  if (int rc = model_linear(m, c.lm_head, m->last, m->last_bf, nullptr, nullptr, CATEN_B200_ACT_NONE, m->logits, cb::BfOut(), c.batch)) return rc;
  if (int rc = launch_argmax(ctx, m->logits, c.batch, c.vocab, m->out_ids)) return rc;
  return launch_finish_step(ctx, m->out_ids, m->ids_io, m->ids_hist, m->d_pos, c.batch);
}

// Runs `steps` single-token steps from the device-side state (ids_io, d_pos already loaded).
// The launch sequence of a step is captured into a CUDA graph the first time and replayed.
static int decode_run(caten_b200_gpt2 *m, int64_t n, int64_t steps) {
  caten_b200_ctx *ctx = m->ctx;
  const int64_t T = m->desc.max_seq_len;
  int64_t done = 0;
  // event brackets cannot be placed inside a graph; a step that is one kernel already gains nothing from one
  const bool use_graph = ctx->prof_mask == 0 && !m->ds;
  if (use_graph && m->graph && (m->graph_xbf != ctx->xbf.ptr || m->graph_wtmp != ctx->wtmp.ptr)) {
    cudaGraphExecDestroy(m->graph);  // scratch was re-allocated since the capture: its pointers are stale
    m->graph = nullptr;
  }
  if (use_graph && !m->graph) {
    // the first step runs eagerly: it sizes the scratch buffers and sets kernel attributes, which
    // must not happen during capture
    if (int rc = decode_step_device_pos(m, n)) return rc;
    done = 1;
    cudaGraph_t g = nullptr;
    CB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    const int64_t before = ctx->launches;
    const int rc = decode_step_device_pos(m, n + 1 < T ? n + 1 : T - 1);  // host-side position only feeds argument checks
    const cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    m->launches_per_step = ctx->launches - before;
    ctx->launches = before;  // captured, not launched
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaStreamEndCapture");
    const cudaError_t e2 = cudaGraphInstantiate(&m->graph, g, 0);
    cudaGraphDestroy(g);
    if (e2 != cudaSuccess) { m->graph = nullptr; return cuda_fail(ctx, e2, "cudaGraphInstantiate"); }
    m->graph_xbf = ctx->xbf.ptr;
    m->graph_wtmp = ctx->wtmp.ptr;
  }
  for (; done < steps; ++done) {
    if (use_graph && m->graph) {
      CB_CUDA(ctx, cudaGraphLaunch(m->graph, ctx->stream));
      ctx->launches += m->launches_per_step;
    } else if (int rc = decode_step_device_pos(m, n + done)) {
      return rc;
    }
  }
  return 0;
}

int caten_b200_gpt2_decode(caten_b200_gpt2 *m, const int64_t *d_first_ids, int64_t n, int64_t steps, int64_t *d_out_ids) {
  if (!m) return fail(nullptr, CATEN_B200_EINVAL, "gpt2_decode: model is NULL");
  caten_b200_ctx *ctx = m->ctx;
  cudaSetDevice(ctx->device);
  const caten_b200_gpt2_desc &c = m->desc;
  const int64_t B = c.batch;
  if (!d_first_ids) return fail(ctx, CATEN_B200_EINVAL, "gpt2_decode: ids is NULL");
  if (steps < 0 || n < 0 || n + steps > c.max_seq_len)
    return fail(ctx, CATEN_B200_EINVAL, "gpt2_decode: positions [%lld, %lld) outside the cache (max_seq_len=%d)", (long long)n, (long long)(n + steps), c.max_seq_len);
  if (steps == 0) return 0;
  if (int rc = launch_begin_steps(ctx, nullptr, d_first_ids, m->ids_io, m->d_pos, n, B)) return rc;
  if (int rc = decode_run(m, n, steps)) return rc;
  if (d_out_ids)
    CB_CUDA(ctx, cudaMemcpyAsync(d_out_ids, m->ids_hist + n * B, (size_t)(steps * B) * sizeof(int64_t), cudaMemcpyDeviceToDevice, ctx->stream));
  return 0;
}

const float *caten_b200_gpt2_logits(caten_b200_gpt2 *m) { return m ? m->logits : nullptr; }

int caten_b200_gpt2_kv(caten_b200_gpt2 *m, int layer, float **d_k, float **d_v) {
  if (!m) return fail(nullptr, CATEN_B200_EINVAL, "gpt2_kv: model is NULL");
  if (layer < 0 || layer >= m->desc.n_layers || !d_k || !d_v) return fail(m->ctx, CATEN_B200_EINVAL, "gpt2_kv: bad layer or NULL out pointer");
  *d_k = m->kc[layer];
  *d_v = m->vc[layer];
  return 0;
}

int64_t caten_b200_gpt2_launch_count(caten_b200_gpt2 *m) { return m ? m->ctx->launches - m->launches0 : 0; }

}  // extern "C"
