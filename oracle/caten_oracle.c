/* TEST INFRASTRUCTURE — not part of the product.
 *
 * CPU restatement of the path hikettei/Caten runs for GPT-2 with BACKEND=CLANG: GGUF block
 * dequantisation, the Transformer graph of external/llm/layers.lisp and the greedy driver of
 * apps/gpt2/gpt2.lisp.  Only tests, the smoke check and the benchmark's CPU-baseline leg may
 * load this library; the CUDA library never does.
 *
 * The reference itself cannot run where this is built (its host side is Common Lisp and its C
 * kernels are text rendered at JIT time), so this restates the definitions op by op.  It is
 * pinned against what the reference's own tests use as their oracle: PyTorch for the math ops
 * and the Python `gguf` package for Q8_0/F16/F32 dequantisation (64-element arange fixture of
 * source/test-suite/external/test-gguf.lisp).  Whole-model outputs and Q4_0 have no golden
 * vector inside the reference: parity unpinned for those two (Q4_0 is pinned here against
 * `gguf.quants.dequantize`, which implements the ggml layout the reference cites at
 * external/gguf/dequantize.lisp:5-6).
 *
 * Three numeric variants are built from gpt2_impl.inc:
 *   mode 0  strict fp32: every operation rounded to float
 *   mode 1  "C literal promotion": CLANG prints constants without an `f` suffix
 *           (source/codegen/renderer.lisp:319-329) and calls the double exp2/sqrt
 *           (renderer.lisp:362-376), so an element-wise chain that touches a literal is
 *           evaluated in double and rounded when stored; reductions stay sequential fp32
 *   mode 2  everything in double, same constants: measures how far rounding alone moves a logit
 *
 * Build: gcc -O3 -ffp-contract=off -fopenmp -shared -fPIC (no -march=native, no -ffast-math:
 * source/byoc/clang.lisp:127-141,217 compiles its kernels with plain -O3).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
  int32_t n_layers, d_model, n_heads, vocab, max_seq_len, batch;
  float eps;
} orc_gpt2_config;

typedef struct {
  const float *wte, *wpe, *lnf_g, *lnf_b, *lm_head;
  const float **ln1_g, **ln1_b, **attn_w, **attn_b, **proj_w, **proj_b;
  const float **ln2_g, **ln2_b, **fc_w, **fc_b, **mproj_w, **mproj_b;
} orc_gpt2_weights;

/* A single-float constant as C sees it after Lisp printed it: shortest decimal that reads back
 * to the same float (what `(format nil "~a" x)` gives), parsed as a double literal. */
static double orc_lit(float c) {
  char buf[64];
  for (int p = 1; p <= 9; ++p) {
    snprintf(buf, sizeof buf, "%.*g", p, (double)c);
    if (strtof(buf, NULL) == c) break;
  }
  return strtod(buf, NULL);
}

/* (/ (log 2)) and (/ -1 (log 2)) evaluated in single float (api/function.lisp:437-440,
 * nn/activations.lisp:6); (sqrt (/ 2.0 pi)) is a Lisp double (nn/activations.lisp:204). */
#define LN2_F 0.6931472f
#define GELU_C_D 0.7978845608028654

/* ---- mode 0 ---- */
#define REAL float
#define ELT float
#define SFX f32
#define ELT_IS_WIDE 0
#define ELT_SQRT sqrtf
#define ELT_EXP2 exp2f
#define KLIT(c) (c)
static struct { float inv_ln2, neg_inv_ln2, gelu_c, c044; } k_f32;
#include "gpt2_impl.inc"
#undef REAL
#undef ELT
#undef SFX
#undef ELT_IS_WIDE
#undef ELT_SQRT
#undef ELT_EXP2
#undef KLIT

/* ---- mode 1 ---- */
#define REAL float
#define ELT double
#define SFX mix
#define ELT_IS_WIDE 1
#define ELT_SQRT sqrt
#define ELT_EXP2 exp2
#define KLIT(c) orc_lit(c)
static struct { double inv_ln2, neg_inv_ln2, gelu_c, c044; } k_mix;
#include "gpt2_impl.inc"
#undef REAL
#undef ELT
#undef SFX
#undef ELT_IS_WIDE
#undef ELT_SQRT
#undef ELT_EXP2
#undef KLIT

/* ---- mode 2 ---- */
#define REAL double
#define ELT double
#define SFX f64
#define ELT_IS_WIDE 1
#define ELT_SQRT sqrt
#define ELT_EXP2 exp2
#define KLIT(c) ((double)(c))
static struct { double inv_ln2, neg_inv_ln2, gelu_c, c044; } k_f64;
#include "gpt2_impl.inc"
#undef REAL
#undef ELT
#undef SFX
#undef ELT_IS_WIDE
#undef ELT_SQRT
#undef ELT_EXP2
#undef KLIT

__attribute__((constructor)) static void orc_init_constants(void) {
  const float inv = 1.0f / LN2_F, ninv = -1.0f / LN2_F;
  k_f32.inv_ln2 = inv; k_f32.neg_inv_ln2 = ninv; k_f32.gelu_c = (float)GELU_C_D; k_f32.c044 = 0.044715f;
  char buf[64];
  snprintf(buf, sizeof buf, "%.15f", GELU_C_D); /* "~,15f" in renderer.lisp:327-328 */
  k_mix.inv_ln2 = orc_lit(inv); k_mix.neg_inv_ln2 = orc_lit(ninv); k_mix.gelu_c = strtod(buf, NULL);
  k_mix.c044 = orc_lit(0.044715f);
  k_f64.inv_ln2 = inv; k_f64.neg_inv_ln2 = ninv; k_f64.gelu_c = (float)GELU_C_D; k_f64.c044 = 0.044715f;
}

int orc_version(void) { return 1; }

void orc_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n < 1 ? 1 : n);
#else
  (void)n;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---------------- GGUF block formats ---------------- */

/* IEEE binary16 -> binary32, bit exact (source/common/dtype.lisp:159-164 decodes with
 * ieee-floats; external/gguf/helpers.lisp:13 reads the little-endian half). */
float orc_half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | man << 13;
  } else {
    bits = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* ggml type ids as stored in GGUF tensor infos (external/gguf/tensor-info.lisp:3-34). */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q4_1 = 3, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8 };

/* external/gguf/dequantize.lisp:14-53.  Q8_0: 34-byte blocks = fp16 scale + 32 int8,
 * w = (float)q * (float)scale.  Q4_0 is not implemented by the reference
 * (tensor-info.lisp:41 signals "Not ready"); layout per ggml: 18-byte blocks = fp16 scale +
 * 16 bytes, byte j holds element j in its low nibble and element j+16 in its high nibble,
 * w = (float)(nibble - 8) * (float)scale.  Q4_1 (d, m, 16 bytes: w = q*d + m), Q5_0 (d, 4 bytes
 * of fifth bits, 16 bytes: w = (q - 16)*d) and Q5_1 (d, m, fifth bits, 16 bytes: w = q*d + m)
 * are ggml's other 32-weight formats, which the reference lists (tensor-info.lisp:3-34) but does
 * not implement; each value is a rounded product followed by a rounded sum, as the Python `gguf`
 * package computes it.  n = number of elements (multiple of 32 for Q*). */
int orc_dequant(int ggml_type, const uint8_t *src, int64_t n, float *out) {
  if (ggml_type == ORC_F32) {
    memcpy(out, src, (size_t)n * 4);
  } else if (ggml_type == ORC_F16) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_half_to_float((uint16_t)(src[2 * i] | src[2 * i + 1] << 8));
  } else if (ggml_type == ORC_Q8_0) {
    const int64_t nb = (n + 31) / 32;
    for (int64_t b = 0; b < nb; ++b) {
      const uint8_t *blk = src + b * 34;
      const float sc = orc_half_to_float((uint16_t)(blk[0] | blk[1] << 8));
      const int64_t lim = (n - b * 32) < 32 ? (n - b * 32) : 32;
      for (int64_t i = 0; i < lim; ++i) out[b * 32 + i] = (float)(int8_t)blk[2 + i] * sc;
    }
  } else if (ggml_type == ORC_Q4_0) {
    if (n % 32) return 2;
    for (int64_t b = 0; b < n / 32; ++b) {
      const uint8_t *blk = src + b * 18;
      const float sc = orc_half_to_float((uint16_t)(blk[0] | blk[1] << 8));
      for (int i = 0; i < 16; ++i) {
        out[b * 32 + i] = (float)((int)(blk[2 + i] & 0x0F) - 8) * sc;
        out[b * 32 + i + 16] = (float)((int)(blk[2 + i] >> 4) - 8) * sc;
      }
    }
  } else if (ggml_type == ORC_Q4_1 || ggml_type == ORC_Q5_0 || ggml_type == ORC_Q5_1) {
    if (n % 32) return 2;
    const int has_m = ggml_type != ORC_Q5_0, has_h = ggml_type != ORC_Q4_1;
    const int head = 2 + 2 * has_m + 4 * has_h;
    for (int64_t b = 0; b < n / 32; ++b) {
      const uint8_t *blk = src + b * (head + 16);
      const float sc = orc_half_to_float((uint16_t)(blk[0] | blk[1] << 8));
      const float mn = has_m ? orc_half_to_float((uint16_t)(blk[2] | blk[3] << 8)) : 0.0f;
      const uint8_t *h = blk + 2 + 2 * has_m;
      const uint32_t qh = has_h ? ((uint32_t)h[0] | (uint32_t)h[1] << 8 | (uint32_t)h[2] << 16 | (uint32_t)h[3] << 24) : 0u;
      const uint8_t *qs = blk + head;
      for (int e = 0; e < 32; ++e) {
        const int nib = e < 16 ? (qs[e] & 0x0F) : (qs[e - 16] >> 4);
        const int q = nib | (int)((qh >> e) & 1u) << 4;
        volatile float prod;  /* keeps the product and the sum separately rounded at any -O level */
        if (has_m) {
          prod = (float)q * sc;
          out[b * 32 + e] = prod + mn;
        } else {
          out[b * 32 + e] = (float)(q - 16) * sc;
        }
      }
    }
  } else {
    return 1;
  }
  return 0;
}

/* ---------------- single ops, float in / float out ---------------- */

static double *to_d(const float *p, int64_t n) {
  if (!p) return NULL;
  double *q = (double *)malloc(sizeof(double) * (size_t)n);
  for (int64_t i = 0; i < n; ++i) q[i] = p[i];
  return q;
}
static void from_d(const double *q, int64_t n, float *p) {
  for (int64_t i = 0; i < n; ++i) p[i] = (float)q[i];
}

void orc_embedding(const float *tok, int64_t B, int64_t s, int64_t n, const float *wte,
                   const float *wpe, int64_t V, int64_t T, int64_t d, float *out) {
  embed_f32(tok, B, s, n, wte, wpe, V, T, d, out);
}

void orc_layernorm(int mode, const float *x, const float *g, const float *b, int64_t rows,
                   int64_t d, float eps, float *y) {
  if (mode == 0) layernorm_f32(x, g, b, rows, d, eps, y);
  else if (mode == 1) layernorm_mix(x, g, b, rows, d, eps, y);
  else {
    double *xd = to_d(x, rows * d), *gd = to_d(g, d), *bd = to_d(b, d);
    double *yd = (double *)malloc(sizeof(double) * (size_t)(rows * d));
    layernorm_f64(xd, gd, bd, rows, d, eps, yd);
    from_d(yd, rows * d, y);
    free(xd); free(gd); free(bd); free(yd);
  }
}

void orc_linear(int mode, const float *x, const float *W, const float *bias, const float *res,
                int act, int64_t M, int64_t N, int64_t K, float *y) {
  if (mode == 0) linear_f32(x, W, bias, res, act, M, N, K, y);
  else if (mode == 1) linear_mix(x, W, bias, res, act, M, N, K, y);
  else {
    double *xd = to_d(x, M * K), *wd = to_d(W, N * K), *bd = to_d(bias, N), *rd = to_d(res, M * N);
    double *yd = (double *)malloc(sizeof(double) * (size_t)(M * N));
    linear_f64(xd, wd, bd, rd, act, M, N, K, yd);
    from_d(yd, M * N, y);
    free(xd); free(wd); free(bd); free(rd); free(yd);
  }
}

/* Readme.md:55-60 example `(!relu (!matmul a b))` with a [M,K] and b [K,N] both row-major:
 * c[m,o] = max(sum_k a[m,k]*b[k,o], 0), k sequential. */
void orc_relu_matmul(int mode, const float *a, const float *b, int64_t M, int64_t K, int64_t N,
                     float *c) {
#pragma omp parallel for if (M * N * K > 262144)
  for (int64_t m = 0; m < M; ++m) {
    if (mode == 2) {
      double *acc = (double *)calloc((size_t)N, sizeof(double));
      for (int64_t k = 0; k < K; ++k) {
        const double av = a[m * K + k];
        for (int64_t o = 0; o < N; ++o) acc[o] = acc[o] + av * (double)b[k * N + o];
      }
      for (int64_t o = 0; o < N; ++o) c[m * N + o] = (float)(acc[o] > 0 ? acc[o] : 0);
      free(acc);
    } else {
      float *acc = (float *)calloc((size_t)N, sizeof(float));
      for (int64_t k = 0; k < K; ++k) {
        const float av = a[m * K + k];
        for (int64_t o = 0; o < N; ++o) acc[o] = acc[o] + (float)(av * b[k * N + o]);
      }
      for (int64_t o = 0; o < N; ++o) c[m * N + o] = acc[o] > 0 ? acc[o] : 0;
      free(acc);
    }
  }
}

void orc_gelu(int mode, const float *x, int64_t n, float *y) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = mode == 0 ? gelu1_f32(x[i]) : mode == 1 ? gelu1_mix(x[i]) : (float)gelu1_f64(x[i]);
}

/* qkv [B*s, 3d] -> out [B*s, d]; kc, vc are caches of layout [B, T, H, hd], updated in place. */
void orc_attention(int mode, const float *qkv, float *kc, float *vc, int64_t B, int64_t s,
                   int64_t n, int64_t H, int64_t hd, int64_t T, float *out) {
  if (mode == 0) attention_f32(qkv, kc, vc, B, s, n, H, hd, T, out);
  else if (mode == 1) attention_mix(qkv, kc, vc, B, s, n, H, hd, T, out);
  else {
    const int64_t d = H * hd;
    double *qd = to_d(qkv, B * s * 3 * d), *kd = to_d(kc, B * T * d), *vd = to_d(vc, B * T * d);
    double *od = (double *)malloc(sizeof(double) * (size_t)(B * s * d));
    attention_f64(qd, kd, vd, B, s, n, H, hd, T, od);
    from_d(od, B * s * d, out); from_d(kd, B * T * d, kc); from_d(vd, B * T * d, vc);
    free(qd); free(kd); free(vd); free(od);
  }
}

/* source/nn/normalization.lisp:70-85: norm = x * recip(sqrt(eps + mean(x * x))), then * weight.
 * mode 0: every step in fp32 (sequential sum); mode 2: all in double. */
void orc_rmsnorm(int mode, const float *x, const float *w, int64_t rows, int64_t d, float eps, float *y) {
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * d;
    float *yr = y + r * d;
    if (mode == 2) {
      double sq = 0;
      for (int64_t k = 0; k < d; ++k) sq += (double)xr[k] * (double)xr[k];
      const double rs = 1.0 / sqrt((double)eps + sq / (double)d);
      for (int64_t k = 0; k < d; ++k) yr[k] = (float)((double)xr[k] * rs * (w ? (double)w[k] : 1.0));
    } else {
      float sq = 0;
      for (int64_t k = 0; k < d; ++k) sq = sq + xr[k] * xr[k];
      const float mean = sq * (1.0f / (float)d);
      const float rs = 1.0f / sqrtf(eps + mean);
      for (int64_t k = 0; k < d; ++k) {
        float v = xr[k] * rs;
        if (w) v = v * w[k];
        yr[k] = v;
      }
    }
  }
}

/* source/nn/positional-encoding.lisp:3-56 on x [B, S, H, hd] with dim = hd / 2:
 *   theta_i = exp(-((2 i) / hd) * log(base)); angle = (pos0 + s) * theta_i;
 *   out[2i] = x[2i] * cos - x[2i+1] * sin; out[2i+1] = x[2i] * sin + x[2i+1] * cos; an odd last element is copied.
 * exp = exp2(x * 1/ln2), log = log2(x) * ln2 (api/function.lisp:437-448), cos(a) = sin(a + pi/2)
 * (api/high-level-ops.lisp:119-122); transcendentals are the double libm functions applied to floats, as the
 * rendered C calls them (source/codegen/renderer.lisp:362-370).  mode 2: everything in double, cos as cos. */
void orc_rope(int mode, const float *x, int64_t B, int64_t S, int64_t H, int64_t hd, float base, int64_t pos0, float *y) {
  const int64_t half = hd / 2;
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t h = 0; h < H; ++h) {
        const float *xp = x + ((b * S + s) * H + h) * hd;
        float *yp = y + ((b * S + s) * H + h) * hd;
        for (int64_t i = 0; i < half; ++i) {
          if (mode == 2) {
            const double theta = exp(-((double)(2 * i) / (double)hd) * log((double)base));
            const double ang = (double)(pos0 + s) * theta;
            yp[2 * i] = (float)((double)xp[2 * i] * cos(ang) - (double)xp[2 * i + 1] * sin(ang));
            yp[2 * i + 1] = (float)((double)xp[2 * i] * sin(ang) + (double)xp[2 * i + 1] * cos(ang));
          } else {
            const float expo = (float)(2 * i) * (1.0f / (float)hd);
            const float logb = (float)log2((double)base) * 0.6931472f;
            const float theta = (float)exp2((double)(-(expo * logb)) * (double)(1.0f / 0.6931472f));
            const float ang = (float)(pos0 + s) * theta;
            const float sn = (float)sin((double)ang), cs = (float)sin((double)(ang + 1.5707964f));
            yp[2 * i] = xp[2 * i] * cs + (-(xp[2 * i + 1] * sn));
            yp[2 * i + 1] = xp[2 * i] * sn + xp[2 * i + 1] * cs;
          }
        }
        if (hd & 1) yp[hd - 1] = xp[hd - 1];
      }
}

void orc_argmax(const float *x, int64_t rows, int64_t V, int64_t *out) {
  for (int64_t r = 0; r < rows; ++r) out[r] = argmax_f32(x + r * V, V);
}

/* ---------------- whole model ---------------- */

typedef struct { int mode; void *impl; } orc_model;

void *orc_gpt2_create(const orc_gpt2_config *c, const orc_gpt2_weights *w, int mode) {
  if (c->d_model % c->n_heads) return NULL;
  orc_model *m = (orc_model *)malloc(sizeof(*m));
  m->mode = mode;
  m->impl = mode == 0 ? create_f32(c, w) : mode == 1 ? create_mix(c, w) : create_f64(c, w);
  return m;
}

/* tok: [B, s] token ids as float32 (apps/gpt2/gpt2.lisp:95); n: start position.
 * out_ids: [B] int64; logits: NULL or [B, V] (last position). Returns 0 on success. */
int orc_gpt2_step(void *mp, const float *tok, int64_t s, int64_t n, int64_t *out_ids, float *logits) {
  orc_model *m = (orc_model *)mp;
  return m->mode == 0   ? step_f32(m->impl, tok, s, n, out_ids, logits)
         : m->mode == 1 ? step_mix(m->impl, tok, s, n, out_ids, logits)
                        : step_f64(m->impl, tok, s, n, out_ids, logits);
}

/* Fill the KV caches of every layer with a value pattern (benchmark only: lets the CPU
 * baseline time a decode step at a long context without running the prefill on the CPU). */
void orc_gpt2_fill_cache(void *mp, float value) {
  orc_model *m = (orc_model *)mp;
  if (m->mode == 2) return;
  model_f32 *f = (model_f32 *)m->impl; /* mode 0 and 1 share the float layout */
  const int64_t cnt = (int64_t)f->cfg.batch * f->cfg.max_seq_len * f->cfg.d_model;
  for (int64_t l = 0; l < f->cfg.n_layers; ++l)
    for (int64_t i = 0; i < cnt; ++i) f->kc[l][i] = f->vc[l][i] = value * (float)((i % 17) - 8);
}

void orc_gpt2_destroy(void *mp) {
  orc_model *m = (orc_model *)mp;
  if (m->mode == 0) destroy_f32(m->impl);
  else if (m->mode == 1) destroy_mix(m->impl);
  else destroy_f64(m->impl);
  free(m);
}
