// Generic schedule item: one kernel that interprets a fused element-wise (optionally reducing)
// expression per element.  It stands where the reference renders one C function per
// Schedule-Item (source/byoc/clang.lisp:163-205, op by op as in source/codegen/renderer.lisp:331-410)
// and compiles it with gcc at run time; here nothing is compiled on the host.
//
// One thread owns one output element.  It decodes its multi-index, then walks the reduced loops
// (if any) in loop order, exactly like the rendered loop nest, so a float sum is added in the
// reference's order.  The program is postfix over a small value stack; the stack lives in
// registers / local memory, the program and the views in the kernel's constant parameter space.
#include "common.cuh"

namespace cb {

__device__ __forceinline__ uint32_t expr_load(const void *p, int dtype, int64_t at) {
  switch (dtype) {
    case CATEN_B200_DT_F32: return __float_as_uint(reinterpret_cast<const float *>(p)[at]);
    case CATEN_B200_DT_I32: return (uint32_t) reinterpret_cast<const int32_t *>(p)[at];
    case CATEN_B200_DT_I64: return (uint32_t)(int32_t) reinterpret_cast<const int64_t *>(p)[at];
    default: return reinterpret_cast<const uint8_t *>(p)[at] ? 1u : 0u;
  }
}

// value of class `cls` -> the output buffer's element type (C conversion rules)
__device__ __forceinline__ void expr_store(void *p, int dtype, int64_t at, uint32_t v, int cls) {
  const bool is_f = cls == CATEN_B200_CLS_F32;
  switch (dtype) {
    case CATEN_B200_DT_F32: reinterpret_cast<float *>(p)[at] = is_f ? __uint_as_float(v) : (float)(int32_t)v; break;
    case CATEN_B200_DT_I32: reinterpret_cast<int32_t *>(p)[at] = is_f ? (int32_t)__uint_as_float(v) : (int32_t)v; break;
    case CATEN_B200_DT_I64: reinterpret_cast<int64_t *>(p)[at] = is_f ? (int64_t)__uint_as_float(v) : (int64_t)(int32_t)v; break;
    default: reinterpret_cast<uint8_t *>(p)[at] = is_f ? (__uint_as_float(v) != 0.0f) : (v != 0u); break;
  }
}

__device__ __forceinline__ uint32_t expr_cast(uint32_t v, int from, int to) {
  if (from == to) return v;
  if (to == CATEN_B200_CLS_F32) return __float_as_uint((float)(int32_t)v);          // I32 / BOOL -> float
  if (from == CATEN_B200_CLS_F32) {
    const float f = __uint_as_float(v);
    return to == CATEN_B200_CLS_BOOL ? (f != 0.0f ? 1u : 0u) : (uint32_t)(int32_t)f;  // C truncation
  }
  return to == CATEN_B200_CLS_BOOL ? (v != 0u ? 1u : 0u) : v;                          // I32 <-> BOOL
}

__device__ __forceinline__ uint32_t expr_run(const caten_b200_expr &e, const int64_t *off, const int64_t *index) {
  uint32_t st[16];
  int sp = 0;
  for (int pc = 0; pc < e.n_code; ++pc) {
    const uint32_t w = e.code[pc];
    const int op = w & 255, arg = (w >> 8) & 255, cls = (w >> 16) & 255;
    const bool f = cls == CATEN_B200_CLS_F32;
    if (op == CATEN_B200_OP_LOAD) {
      st[sp++] = expr_load(e.operand[arg], e.operand_dtype[arg], off[arg]);
    } else if (op == CATEN_B200_OP_CONST) {
      st[sp++] = e.consts[arg];
    } else if (op == CATEN_B200_OP_INDEX) {
      st[sp++] = (uint32_t)(int32_t)index[arg];
    } else if (op < CATEN_B200_OP_ADD) {  // unary
      const uint32_t a = st[sp - 1];
      const float fa = __uint_as_float(a);
      const int32_t ia = (int32_t)a;
      uint32_t r;
      switch (op) {
        case CATEN_B200_OP_NEG: r = f ? __float_as_uint(-fa) : (uint32_t)(-ia); break;
        case CATEN_B200_OP_RECIP: r = f ? __float_as_uint(1.0f / fa) : (ia == 0 ? 0u : (uint32_t)(1 / ia)); break;
        case CATEN_B200_OP_SIN: r = __float_as_uint((float)sin((double)fa)); break;
        case CATEN_B200_OP_EXP2: r = __float_as_uint((float)exp2((double)fa)); break;
        case CATEN_B200_OP_LOG2: r = __float_as_uint((float)log2((double)fa)); break;
        case CATEN_B200_OP_SQRT: r = __float_as_uint((float)sqrt((double)fa)); break;
        case CATEN_B200_OP_NOT: r = f ? (fa == 0.0f ? 1u : 0u) : (a == 0u ? 1u : 0u); break;
        default: r = expr_cast(a, arg, cls); break;  // CAST
      }
      st[sp - 1] = r;
    } else if (op < CATEN_B200_OP_WHERE) {  // binary
      const uint32_t b = st[--sp], a = st[sp - 1];
      const float fa = __uint_as_float(a), fb = __uint_as_float(b);
      const int32_t ia = (int32_t)a, ib = (int32_t)b;
      uint32_t r;
      switch (op) {
        case CATEN_B200_OP_ADD: r = f ? __float_as_uint(fa + fb) : (uint32_t)(ia + ib); break;
        case CATEN_B200_OP_MUL: r = f ? __float_as_uint(fa * fb) : (uint32_t)(ia * ib); break;
        case CATEN_B200_OP_MOD: r = ib == 0 ? 0u : (uint32_t)(ia % ib); break;
        case CATEN_B200_OP_IDIV: r = ib == 0 ? 0u : (uint32_t)(ia / ib); break;
        case CATEN_B200_OP_AND: r = a & b; break;
        case CATEN_B200_OP_OR: r = a | b; break;
        case CATEN_B200_OP_XOR: r = a ^ b; break;
        case CATEN_B200_OP_MAX: r = f ? (fa > fb ? a : b) : (ia > ib ? a : b); break;
        case CATEN_B200_OP_NE: r = f ? (fa != fb ? 1u : 0u) : (a != b ? 1u : 0u); break;
        default: r = f ? (fa < fb ? 1u : 0u) : (ia < ib ? 1u : 0u); break;  // LT
      }
      st[sp - 1] = r;
    } else {  // WHERE
      const uint32_t b = st[--sp], a = st[--sp], c = st[sp - 1];
      st[sp - 1] = c != 0u ? a : b;
    }
  }
  return st[0];
}

__global__ void __launch_bounds__(256) expr_kernel(const __grid_constant__ caten_b200_expr e, const int64_t n_out, const int64_t n_red,
                                                   const int result_cls) {
  pdl_enter();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out) return;
  const int nd_out = e.ndim - e.n_reduce;
  int64_t index[CATEN_B200_EXPR_MAX_DIMS];
  int64_t base[CATEN_B200_EXPR_MAX_OPERANDS], off[CATEN_B200_EXPR_MAX_OPERANDS];
  int64_t rem = idx, out_at = e.out_offset;
  for (int d = nd_out - 1; d >= 0; --d) {
    index[d] = rem % e.shape[d];
    rem /= e.shape[d];
    out_at += index[d] * e.out_stride[d];
  }
  for (int i = 0; i < e.n_operands; ++i) {
    int64_t o = e.operand_offset[i];
    for (int d = 0; d < nd_out; ++d) o += index[d] * e.operand_stride[i][d];
    base[i] = o;
  }
  const bool f = result_cls == CATEN_B200_CLS_F32;
  if (e.n_reduce == 0) {
    for (int i = 0; i < e.n_operands; ++i) off[i] = base[i];
    expr_store(e.out, e.out_dtype, out_at, expr_run(e, off, index), result_cls);
    return;
  }
  float facc = e.reduce_op == CATEN_B200_RED_MAX ? -INFINITY : 0.0f;
  int32_t iacc = e.reduce_op == CATEN_B200_RED_MAX ? INT32_MIN : 0;
  bool have = false;
  if (e.accumulate) {
    const uint32_t old = expr_load(e.out, e.out_dtype, out_at);
    // the buffer's element type decides how its old value reads
    if (f) facc = e.out_dtype == CATEN_B200_DT_F32 ? __uint_as_float(old) : (float)(int32_t)old;
    else iacc = e.out_dtype == CATEN_B200_DT_F32 ? (int32_t)__uint_as_float(old) : (int32_t)old;
    have = true;
  }
  for (int64_t r = 0; r < n_red; ++r) {
    int64_t rr = r;
    for (int d = e.ndim - 1; d >= nd_out; --d) {
      index[d] = rr % e.shape[d];
      rr /= e.shape[d];
    }
    for (int i = 0; i < e.n_operands; ++i) {
      int64_t o = base[i];
      for (int d = nd_out; d < e.ndim; ++d) o += index[d] * e.operand_stride[i][d];
      off[i] = o;
    }
    const uint32_t v = expr_run(e, off, index);
    if (f) {
      const float x = __uint_as_float(v);
      if (e.reduce_op == CATEN_B200_RED_SUM) facc = facc + x;
      else facc = (have || r > 0) ? (facc > x ? facc : x) : x;
    } else {
      const int32_t x = (int32_t)v;
      if (e.reduce_op == CATEN_B200_RED_SUM) iacc = iacc + x;
      else iacc = (have || r > 0) ? (iacc > x ? iacc : x) : x;
    }
  }
  expr_store(e.out, e.out_dtype, out_at, f ? __float_as_uint(facc) : (uint32_t)iacc, result_cls);
}

// Checks the program on the host (operand indices, stack discipline, classes) and returns the
// class of the value it leaves.
static int expr_validate(caten_b200_ctx *ctx, const caten_b200_expr *e, int *result_cls) {
  if (e->ndim < 1 || e->ndim > CATEN_B200_EXPR_MAX_DIMS) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: ndim %d outside 1..%d", e->ndim, CATEN_B200_EXPR_MAX_DIMS);
  if (e->n_reduce < 0 || e->n_reduce > e->ndim) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: n_reduce %d", e->n_reduce);
  if ((e->n_reduce > 0) != (e->reduce_op != CATEN_B200_RED_NONE) || e->reduce_op < 0 || e->reduce_op > CATEN_B200_RED_MAX)
    return fail(ctx, CATEN_B200_EINVAL, "eval_expr: reduce_op %d with %d reduced loops", e->reduce_op, e->n_reduce);
  if (e->n_operands < 0 || e->n_operands > CATEN_B200_EXPR_MAX_OPERANDS) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: %d operands", e->n_operands);
  if (e->n_code < 1 || e->n_code > CATEN_B200_EXPR_MAX_CODE) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: program of %d words", e->n_code);
  if (!e->out || e->out_dtype < 0 || e->out_dtype > CATEN_B200_DT_U8) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: output");
  for (int d = 0; d < e->ndim; ++d)
    if (e->shape[d] < 0) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: negative extent");
  for (int i = 0; i < e->n_operands; ++i)
    if (!e->operand[i] || e->operand_dtype[i] < 0 || e->operand_dtype[i] > CATEN_B200_DT_U8)
      return fail(ctx, CATEN_B200_EINVAL, "eval_expr: operand %d", i);
  int cls_stack[16], sp = 0;
  for (int pc = 0; pc < e->n_code; ++pc) {
    const uint32_t w = e->code[pc];
    const int op = w & 255, arg = (w >> 8) & 255, cls = (w >> 16) & 255;
    if (cls > CATEN_B200_CLS_BOOL) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: class %d", pc, cls);
    if (op == CATEN_B200_OP_LOAD || op == CATEN_B200_OP_CONST || op == CATEN_B200_OP_INDEX) {
      if (op == CATEN_B200_OP_LOAD && arg >= e->n_operands) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d loads operand %d", pc, arg);
      if (op == CATEN_B200_OP_CONST && arg >= CATEN_B200_EXPR_MAX_CONSTS) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: constant %d", pc, arg);
      if (op == CATEN_B200_OP_INDEX && (arg >= e->ndim || cls != CATEN_B200_CLS_I32)) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: index of axis %d", pc, arg);
      if (op == CATEN_B200_OP_LOAD) {
        const int dt = e->operand_dtype[arg];
        const int want = dt == CATEN_B200_DT_F32 ? CATEN_B200_CLS_F32 : dt == CATEN_B200_DT_U8 ? CATEN_B200_CLS_BOOL : CATEN_B200_CLS_I32;
        if (cls != want) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: class %d for an operand of type %d", pc, cls, dt);
      }
      if (sp >= 16) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: stack deeper than 16");
      cls_stack[sp++] = cls;
    } else if (op >= CATEN_B200_OP_NEG && op <= CATEN_B200_OP_CAST) {
      if (sp < 1) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: empty stack", pc);
      const int have = cls_stack[sp - 1];
      if (op == CATEN_B200_OP_CAST) {
        if (arg != have) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: CAST from class %d, stack holds %d", pc, arg, have);
      } else {
        if (cls != have) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: class %d, stack holds %d", pc, cls, have);
        if (op >= CATEN_B200_OP_SIN && op <= CATEN_B200_OP_SQRT && cls != CATEN_B200_CLS_F32)
          return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: float-only op on class %d", pc, cls);
      }
      cls_stack[sp - 1] = op == CATEN_B200_OP_NOT ? CATEN_B200_CLS_BOOL : cls;
    } else if (op >= CATEN_B200_OP_ADD && op <= CATEN_B200_OP_LT) {
      if (sp < 2) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: needs two values", pc);
      if (cls_stack[sp - 1] != cls || cls_stack[sp - 2] != cls) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: operand classes differ from %d", pc, cls);
      if (op >= CATEN_B200_OP_MOD && op <= CATEN_B200_OP_XOR && cls == CATEN_B200_CLS_F32)
        return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: integer op on floats", pc);
      --sp;
      cls_stack[sp - 1] = (op == CATEN_B200_OP_NE || op == CATEN_B200_OP_LT) ? CATEN_B200_CLS_BOOL : cls;
    } else if (op == CATEN_B200_OP_WHERE) {
      if (sp < 3) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: needs three values", pc);
      if (cls_stack[sp - 1] != cls || cls_stack[sp - 2] != cls) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: branch classes differ from %d", pc, cls);
      sp -= 2;
      cls_stack[sp - 1] = cls;
    } else {
      return fail(ctx, CATEN_B200_EINVAL, "eval_expr: word %d: unknown opcode %d", pc, op);
    }
  }
  if (sp != 1) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: the program leaves %d values", sp);
  *result_cls = cls_stack[0];
  return 0;
}

int launch_expr(caten_b200_ctx *ctx, const caten_b200_expr *e) {
  int result_cls = 0;
  if (int rc = expr_validate(ctx, e, &result_cls)) return rc;
  const int nd_out = e->ndim - e->n_reduce;
  int64_t n_out = 1, n_red = 1;
  for (int d = 0; d < nd_out; ++d) n_out *= e->shape[d];
  for (int d = nd_out; d < e->ndim; ++d) n_red *= e->shape[d];
  if (n_out == 0) return 0;
  if (e->n_reduce > 0 && n_red == 0 && !e->accumulate && e->reduce_op == CATEN_B200_RED_MAX)
    return fail(ctx, CATEN_B200_EINVAL, "eval_expr: max over an empty range");
  const int64_t blocks = (n_out + 255) / 256;
  if (blocks > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "eval_expr: %lld output elements", (long long)n_out);
  launch_k(ctx, expr_kernel, dim3((unsigned)blocks), dim3(256), 0, *e, n_out, n_red, result_cls);
  CB_LAUNCH_CHECK(ctx, "expr_kernel");
  return 0;
}

}  // namespace cb
