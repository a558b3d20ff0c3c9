// Generic schedule item: one kernel that interprets a fused element-wise (optionally reducing)
// expression per element.  It stands where the reference renders one C function per
// Schedule-Item (source/byoc/clang.lisp:163-205, op by op as in source/codegen/renderer.lisp:331-410)
// and compiles it with gcc at run time; here nothing is compiled on the host.
//
// One thread owns four output elements of the innermost kept loop (32 apart, so that a warp's
// accesses are coalesced).  It decodes its multi-index once, then walks the reduced loops (if
// any) in loop order, exactly like the rendered loop nest, so a float sum is added in the
// reference's order.  The program is postfix over a small value stack whose slots hold the four
// elements side by side, so decoding a program word is paid once per four elements; the top of
// the stack is in registers, the rest in shared memory, the program and the views in the
// kernel's constant parameter space.  Contiguous row reductions use a second kernel with the
// lanes along the reduced loop and an in-order accumulation across lanes.
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

constexpr int EV = 4;          // output elements per thread (32 apart along the strip)
constexpr int EXPR_THREADS = 256;
constexpr int MAXD = CATEN_B200_EXPR_MAX_DIMS;

// Per-thread state is kept out of local memory: with 2048 threads per SM a few hundred bytes of
// local arrays each overflow L1 and turn every stack access into L2 traffic.  The loop indices
// are MAXD registers (all loops over them are fully unrolled), operand offsets are recomputed
// from them at each LOAD (strides come from the kernel's parameter space), the top of the value
// stack is EV registers and the values under it live in shared memory, [slot][element][thread].
struct ExprIx {
  int v[MAXD];
};

// Runs the program for EV elements at once: the decode of a word is shared.  Element j of the
// thread is 32 j further along loop `vec_axis` (vec_axis < 0: a single element); for j >= lanes
// element 0 is re-read, so nothing outside the views is touched.
__device__ __forceinline__ void expr_run(const caten_b200_expr &e, const ExprIx &ix, const int vec_axis, const int lanes, uint32_t *tos,
                                         uint32_t *sm) {
  int sp = 0;  // values on the stack, the top one (registers) included
  auto slot = [&](int s, int j) -> uint32_t & { return sm[(s * EV + j) * EXPR_THREADS]; };
#define EXPR_PUSH(VALUE)                                                           \
  {                                                                                \
    if (sp > 0) {                                                                  \
      _Pragma("unroll") for (int j = 0; j < EV; ++j) slot(sp - 1, j) = tos[j];     \
    }                                                                              \
    _Pragma("unroll") for (int j = 0; j < EV; ++j) tos[j] = (VALUE);               \
    ++sp;                                                                          \
    break;                                                                         \
  }
#define EXPR_UN(EXPR_F, EXPR_I)                                                    \
  {                                                                                \
    _Pragma("unroll") for (int j = 0; j < EV; ++j) {                               \
      const uint32_t a = tos[j];                                                   \
      const float fa = __uint_as_float(a);                                         \
      const int32_t ia = (int32_t)a;                                               \
      (void)fa; (void)ia;                                                          \
      tos[j] = f ? (EXPR_F) : (EXPR_I);                                            \
    }                                                                              \
    break;                                                                         \
  }
#define EXPR_BIN(EXPR_F, EXPR_I)                                                   \
  {                                                                                \
    --sp;                                                                          \
    _Pragma("unroll") for (int j = 0; j < EV; ++j) {                               \
      const uint32_t b = tos[j], a = slot(sp - 1, j);                              \
      const float fa = __uint_as_float(a), fb = __uint_as_float(b);                \
      const int32_t ia = (int32_t)a, ib = (int32_t)b;                              \
      (void)fa; (void)fb; (void)ia; (void)ib;                                      \
      tos[j] = f ? (EXPR_F) : (EXPR_I);                                            \
    }                                                                              \
    break;                                                                         \
  }
  for (int pc = 0; pc < e.n_code; ++pc) {
    const uint32_t w = e.code[pc];
    const int op = w & 255, arg = (w >> 8) & 255, cls = (w >> 16) & 255;
    const bool f = cls == CATEN_B200_CLS_F32;
    switch (op) {
      case CATEN_B200_OP_LOAD: {
        const void *p = e.operand[arg];
        const int dt = e.operand_dtype[arg];
        int64_t o = e.operand_offset[arg];
#pragma unroll
        for (int d = 0; d < MAXD; ++d)
          if (d < e.ndim) o += (int64_t)ix.v[d] * e.operand_stride[arg][d];
        const int64_t step = vec_axis >= 0 ? 32 * e.operand_stride[arg][vec_axis] : 0;
        if (dt == CATEN_B200_DT_F32) {  // the common case without the per-element type switch
          const float *fp = reinterpret_cast<const float *>(p) + o;
          EXPR_PUSH(__float_as_uint(fp[(j < lanes ? j : 0) * step]))
        }
        EXPR_PUSH(expr_load(p, dt, o + (j < lanes ? j : 0) * step))
      }
      case CATEN_B200_OP_CONST: EXPR_PUSH(e.consts[arg])
      case CATEN_B200_OP_INDEX: {
        int base = 0;
#pragma unroll
        for (int d = 0; d < MAXD; ++d)
          if (d == arg) base = ix.v[d];
        EXPR_PUSH((uint32_t)(base + (arg == vec_axis ? 32 * j : 0)))
      }
      case CATEN_B200_OP_NEG: EXPR_UN(__float_as_uint(-fa), (uint32_t)(-ia))
      case CATEN_B200_OP_RECIP: EXPR_UN(__float_as_uint(1.0f / fa), (ia == 0 ? 0u : (uint32_t)(1 / ia)))
      case CATEN_B200_OP_SIN: EXPR_UN(__float_as_uint((float)sin((double)fa)), a)
      case CATEN_B200_OP_EXP2: EXPR_UN(__float_as_uint((float)exp2((double)fa)), a)
      case CATEN_B200_OP_LOG2: EXPR_UN(__float_as_uint((float)log2((double)fa)), a)
      case CATEN_B200_OP_SQRT: EXPR_UN(__float_as_uint((float)sqrt((double)fa)), a)
      case CATEN_B200_OP_NOT: EXPR_UN((fa == 0.0f ? 1u : 0u), (a == 0u ? 1u : 0u))
      case CATEN_B200_OP_CAST: {
#pragma unroll
        for (int j = 0; j < EV; ++j) tos[j] = expr_cast(tos[j], arg, cls);
        break;
      }
      case CATEN_B200_OP_ADD: EXPR_BIN(__float_as_uint(fa + fb), (uint32_t)(ia + ib))
      case CATEN_B200_OP_MUL: EXPR_BIN(__float_as_uint(fa * fb), (uint32_t)(ia * ib))
      case CATEN_B200_OP_MOD: EXPR_BIN(a, (ib == 0 ? 0u : (uint32_t)(ia % ib)))
      case CATEN_B200_OP_IDIV: EXPR_BIN(a, (ib == 0 ? 0u : (uint32_t)(ia / ib)))
      case CATEN_B200_OP_AND: EXPR_BIN(a & b, a & b)
      case CATEN_B200_OP_OR: EXPR_BIN(a | b, a | b)
      case CATEN_B200_OP_XOR: EXPR_BIN(a ^ b, a ^ b)
      case CATEN_B200_OP_MAX: EXPR_BIN((fa > fb ? a : b), (ia > ib ? a : b))
      case CATEN_B200_OP_NE: EXPR_BIN((fa != fb ? 1u : 0u), (a != b ? 1u : 0u))
      case CATEN_B200_OP_LT: EXPR_BIN((fa < fb ? 1u : 0u), (ia < ib ? 1u : 0u))
      default: {  // WHERE: (cond a b) with b on top
        sp -= 2;
#pragma unroll
        for (int j = 0; j < EV; ++j) tos[j] = slot(sp - 1, j) != 0u ? slot(sp, j) : tos[j];
        break;
      }
    }
  }
#undef EXPR_PUSH
#undef EXPR_UN
#undef EXPR_BIN
}

// loop indices of flat position `pos` over loops [first, last) -> ix (innermost fastest)
__device__ __forceinline__ void expr_decode(const caten_b200_expr &e, int64_t pos, const int first, const int last, ExprIx &ix) {
#pragma unroll
  for (int d = MAXD - 1; d >= 0; --d) {
    if (d >= first && d < last) {
      ix.v[d] = (int)(pos % e.shape[d]);
      pos /= e.shape[d];
    }
  }
}

__device__ __forceinline__ int64_t expr_out_at(const caten_b200_expr &e, const ExprIx &ix, const int nd_out) {
  int64_t at = e.out_offset;
#pragma unroll
  for (int d = 0; d < MAXD; ++d)
    if (d < nd_out) at += (int64_t)ix.v[d] * e.out_stride[d];
  return at;
}

struct ExprAcc {  // reduction state of one output element
  float f;
  int32_t i;
};

__device__ __forceinline__ ExprAcc expr_acc_init(const caten_b200_expr &e, const bool is_f, const int64_t out_at, const bool valid) {
  ExprAcc a;
  a.f = e.reduce_op == CATEN_B200_RED_MAX ? -INFINITY : 0.0f;
  a.i = e.reduce_op == CATEN_B200_RED_MAX ? INT32_MIN : 0;
  if (e.accumulate && valid) {  // the buffer's element type decides how its old value reads
    const uint32_t old = expr_load(e.out, e.out_dtype, out_at);
    if (is_f) a.f = e.out_dtype == CATEN_B200_DT_F32 ? __uint_as_float(old) : (float)(int32_t)old;
    else a.i = e.out_dtype == CATEN_B200_DT_F32 ? (int32_t)__uint_as_float(old) : (int32_t)old;
  }
  return a;
}

// acc <- acc (op) x; `first` = no value has entered a MAX yet
__device__ __forceinline__ void expr_acc_add(ExprAcc &a, const uint32_t x, const bool is_f, const bool is_sum, const bool first) {
  if (is_f) {
    const float xf = __uint_as_float(x);
    a.f = is_sum ? a.f + xf : (first ? xf : (a.f > xf ? a.f : xf));
  } else {
    const int32_t xi = (int32_t)x;
    a.i = is_sum ? a.i + xi : (first ? xi : (a.i > xi ? a.i : xi));
  }
}

// A warp owns strips of 32 * EV consecutive elements of the innermost kept loop; lane l takes
// elements l, l + 32, ... of a strip, so every load and store of the warp is coalesced.  Each
// warp takes `spw` consecutive strips of one row, so the index decoding (64-bit divisions) is
// paid once per warp.  Reduced loops (if any) are walked by each thread in loop order, exactly
// like the rendered loop nest, so a float sum is added in the reference's order.
__global__ void __launch_bounds__(EXPR_THREADS) expr_kernel(const __grid_constant__ caten_b200_expr e, const int64_t n_groups, const int spw,
                                                            const int64_t n_red, const int result_cls) {
  extern __shared__ uint32_t expr_smem[];
  pdl_enter();
  const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (group >= n_groups) return;
  uint32_t *sm = expr_smem + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const int nd_out = e.ndim - e.n_reduce;
  const int va = nd_out - 1;  // the loop the strips run along (-1: a single output element)
  const int64_t vlen = va >= 0 ? e.shape[va] : 1;
  const int64_t strips_per_row = (vlen + 32 * EV - 1) / (32 * EV);
  const int64_t groups_per_row = (strips_per_row + spw - 1) / spw;
  ExprIx ix;
#pragma unroll
  for (int d = 0; d < MAXD; ++d) ix.v[d] = 0;
  expr_decode(e, group / groups_per_row, 0, va, ix);
  int64_t j0 = (group % groups_per_row) * spw * (32 * EV) + lane;  // this thread's first element; the others follow 32 apart
  const bool is_f = result_cls == CATEN_B200_CLS_F32, is_sum = e.reduce_op == CATEN_B200_RED_SUM;
  const int64_t ovs = va >= 0 ? 32 * e.out_stride[va] : 0;
  for (int s = 0; s < spw && j0 < vlen; ++s, j0 += 32 * EV) {
    const int lanes = (int)((vlen - j0 + 31) / 32 < EV ? (vlen - j0 + 31) / 32 : EV);  // elements of this thread in this strip
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d == va) ix.v[d] = (int)j0;
    const int64_t out_at = expr_out_at(e, ix, nd_out);
    uint32_t val[EV];
    if (e.n_reduce == 0) {
      expr_run(e, ix, va, lanes, val, sm);
#pragma unroll
      for (int j = 0; j < EV; ++j)
        if (j < lanes) expr_store(e.out, e.out_dtype, out_at + j * ovs, val[j], result_cls);
      continue;
    }
    ExprAcc acc[EV];
#pragma unroll
    for (int j = 0; j < EV; ++j) acc[j] = expr_acc_init(e, is_f, out_at + j * ovs, j < lanes);
    for (int64_t r = 0; r < n_red; ++r) {
      expr_decode(e, r, nd_out, e.ndim, ix);
      expr_run(e, ix, va, lanes, val, sm);
#pragma unroll
      for (int j = 0; j < EV; ++j) expr_acc_add(acc[j], val[j], is_f, is_sum, !e.accumulate && r == 0);
    }
#pragma unroll
    for (int j = 0; j < EV; ++j)
      if (j < lanes) expr_store(e.out, e.out_dtype, out_at + j * ovs, is_f ? __float_as_uint(acc[j].f) : (uint32_t)acc[j].i, result_cls);
  }
}

// Reduction whose single reduced loop is the contiguous one (row sums, softmax statistics): one
// warp per output element, lanes along the reduced loop so that loads are coalesced.  The warp
// evaluates 32 * EV elements at a time and then adds them in loop order - element r0, r0 + 1, ... -
// by walking the lanes with shuffles, so the result has the reference's order of additions
// although the loads are parallel.
__global__ void __launch_bounds__(EXPR_THREADS) expr_rowreduce_kernel(const __grid_constant__ caten_b200_expr e, const int64_t n_out,
                                                                      const int result_cls) {
  extern __shared__ uint32_t expr_smem[];
  pdl_enter();
  const int64_t o_idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (o_idx >= n_out) return;  // whole warps leave together
  uint32_t *sm = expr_smem + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const int nd_out = e.ndim - 1, ra = e.ndim - 1;
  const int64_t n_red = e.shape[ra];
  ExprIx ix;
#pragma unroll
  for (int d = 0; d < MAXD; ++d) ix.v[d] = 0;
  expr_decode(e, o_idx, 0, nd_out, ix);
  const int64_t out_at = expr_out_at(e, ix, nd_out);
  const bool is_f = result_cls == CATEN_B200_CLS_F32, is_sum = e.reduce_op == CATEN_B200_RED_SUM;
  ExprAcc acc = expr_acc_init(e, is_f, out_at, true);
  uint32_t val[EV];
  for (int64_t r0 = 0; r0 < n_red; r0 += 32 * EV) {
    const int64_t mine = r0 + lane;  // this lane's elements: mine, mine + 32, ...
    // elements of this lane in this round; a lane past the end re-reads element 0 of the row
    const int mine_n = mine >= n_red ? 0 : (int)((n_red - mine + 31) / 32 < EV ? (n_red - mine + 31) / 32 : EV);
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d == ra) ix.v[d] = mine_n > 0 ? (int)mine : 0;
    expr_run(e, ix, ra, mine_n, val, sm);
#pragma unroll
    for (int j = 0; j < EV; ++j) {
      const int64_t first = r0 + 32 * j;  // element of lane 0 in this round
      if (first >= n_red) break;
      const int n_here = (int)(n_red - first < 32 ? n_red - first : 32);
#pragma unroll
      for (int k = 0; k < 32; ++k) {       // loop order: lane 0, 1, ..., 31
        const uint32_t x = __shfl_sync(0xffffffffu, val[j], k);
        if (k < n_here) expr_acc_add(acc, x, is_f, is_sum, !e.accumulate && first + k == 0);
      }
    }
  }
  if (lane == 0) expr_store(e.out, e.out_dtype, out_at, is_f ? __float_as_uint(acc.f) : (uint32_t)acc.i, result_cls);
}

// Checks the program on the host (operand indices, stack discipline, classes) and returns the
// class of the value it leaves.
static int expr_validate(caten_b200_ctx *ctx, const caten_b200_expr *e, int *result_cls, int *max_depth) {
  *max_depth = 1;
  if (e->ndim < 1 || e->ndim > CATEN_B200_EXPR_MAX_DIMS) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: ndim %d outside 1..%d", e->ndim, CATEN_B200_EXPR_MAX_DIMS);
  if (e->n_reduce < 0 || e->n_reduce > e->ndim) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: n_reduce %d", e->n_reduce);
  if ((e->n_reduce > 0) != (e->reduce_op != CATEN_B200_RED_NONE) || e->reduce_op < 0 || e->reduce_op > CATEN_B200_RED_MAX)
    return fail(ctx, CATEN_B200_EINVAL, "eval_expr: reduce_op %d with %d reduced loops", e->reduce_op, e->n_reduce);
  if (e->n_operands < 0 || e->n_operands > CATEN_B200_EXPR_MAX_OPERANDS) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: %d operands", e->n_operands);
  if (e->n_code < 1 || e->n_code > CATEN_B200_EXPR_MAX_CODE) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: program of %d words", e->n_code);
  if (!e->out || e->out_dtype < 0 || e->out_dtype > CATEN_B200_DT_U8) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: output");
  for (int d = 0; d < e->ndim; ++d)
    if (e->shape[d] < 0 || e->shape[d] > 0x7fffffff) return fail(ctx, CATEN_B200_EINVAL, "eval_expr: extent %lld of loop %d", (long long)e->shape[d], d);
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
      if (sp > *max_depth) *max_depth = sp;
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

// Merges neighbouring loops that every view walks as one contiguous run (stride[d] ==
// stride[d+1] * extent[d+1], which also holds for two broadcast axes) and drops loops of extent
// 1, so that the strip a warp works on is as long as the data allows.  Kept and reduced loops
// are only merged among themselves; the visiting order of the elements does not change.
static void expr_collapse(caten_b200_expr *c) {
  for (int pc = 0; pc < c->n_code; ++pc)
    if ((c->code[pc] & 255) == CATEN_B200_OP_INDEX) return;  // loop indices are observable: keep the nest
  auto remove_loop = [&](int d) {
    for (int k = d; k + 1 < c->ndim; ++k) {
      c->shape[k] = c->shape[k + 1];
      c->out_stride[k] = c->out_stride[k + 1];
      for (int i = 0; i < c->n_operands; ++i) c->operand_stride[i][k] = c->operand_stride[i][k + 1];
    }
    --c->ndim;
  };
  int d = 0;
  while (d + 1 < c->ndim) {
    const int nd_out = c->ndim - c->n_reduce;
    const bool kept = d + 1 < nd_out, reduced = d >= nd_out;
    bool ok = kept || reduced;
    if (ok && c->shape[d + 1] != 1 && c->shape[d] != 1) {
      for (int i = 0; i < c->n_operands && ok; ++i) ok = c->operand_stride[i][d] == c->operand_stride[i][d + 1] * c->shape[d + 1];
      if (ok && kept) ok = c->out_stride[d] == c->out_stride[d + 1] * c->shape[d + 1];
    }
    // the kernels index a loop with an int: never build a fused loop longer than that
    if (ok && c->shape[d] > 1 && c->shape[d + 1] > 1 && c->shape[d] > (int64_t)INT32_MAX / c->shape[d + 1]) ok = false;
    if (!ok) { ++d; continue; }
    if (c->shape[d] == 1) {          // drop loop d
      remove_loop(d);
    } else if (c->shape[d + 1] == 1) {  // drop loop d + 1
      remove_loop(d + 1);
    } else {                         // fuse d + 1 into d: the fused loop steps with the inner stride
      c->shape[d] *= c->shape[d + 1];
      c->out_stride[d] = c->out_stride[d + 1];
      for (int i = 0; i < c->n_operands; ++i) c->operand_stride[i][d] = c->operand_stride[i][d + 1];
      remove_loop(d + 1);
    }
    if (reduced) --c->n_reduce;
  }
}

int launch_expr(caten_b200_ctx *ctx, const caten_b200_expr *given) {
  int result_cls = 0, max_depth = 1;
  if (int rc = expr_validate(ctx, given, &result_cls, &max_depth)) return rc;
  // values under the top of the stack: [slot][element][thread] in shared memory
  const size_t smem = (size_t)(max_depth > 1 ? max_depth - 1 : 1) * EV * EXPR_THREADS * sizeof(uint32_t);
  if (smem > 48 * 1024) {
    CB_CUDA(ctx, cudaFuncSetAttribute(expr_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CB_CUDA(ctx, cudaFuncSetAttribute(expr_rowreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  caten_b200_expr collapsed = *given;
  expr_collapse(&collapsed);
  const caten_b200_expr *e = &collapsed;
  const int nd_out = e->ndim - e->n_reduce;
  int64_t n_out = 1, n_red = 1;
  for (int d = 0; d < nd_out; ++d) n_out *= e->shape[d];
  for (int d = nd_out; d < e->ndim; ++d) n_red *= e->shape[d];
  if (n_out == 0) return 0;
  if (e->n_reduce > 0 && n_red == 0 && !e->accumulate && e->reduce_op == CATEN_B200_RED_MAX)
    return fail(ctx, CATEN_B200_EINVAL, "eval_expr: max over an empty range");
  if (e->n_reduce == 1 && n_red >= 64) {
    // lanes along the reduced loop when that is where the operands are contiguous (or nothing else is left)
    bool unit_red = false, unit_kept = false;
    for (int i = 0; i < e->n_operands; ++i) {
      if (e->operand_stride[i][e->ndim - 1] == 1) unit_red = true;
      if (nd_out > 0 && e->operand_stride[i][nd_out - 1] == 1) unit_kept = true;
    }
    if (nd_out == 0 || (unit_red && !unit_kept)) {
      const int64_t blocks = (n_out + 7) / 8;  // one warp per output element
      if (blocks > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "eval_expr: %lld output elements", (long long)n_out);
      launch_k(ctx, expr_rowreduce_kernel, dim3((unsigned)blocks), dim3(EXPR_THREADS), smem, *e, n_out, result_cls);
      CB_LAUNCH_CHECK(ctx, "expr_rowreduce_kernel");
      return 0;
    }
  }
  const int64_t vlen = nd_out > 0 ? e->shape[nd_out - 1] : 1;
  const int64_t strips_per_row = (vlen + 32 * EV - 1) / (32 * EV), rows = n_out / vlen;
  // strips per warp: as many as still leave every SM a full complement of warps, at most 16
  int64_t spw = (rows * strips_per_row) / ((int64_t)ctx->sm_count * 64);
  spw = spw < 1 ? 1 : spw > 16 ? 16 : spw;
  if (spw > strips_per_row) spw = strips_per_row;
  const int64_t n_groups = rows * ((strips_per_row + spw - 1) / spw);  // one warp each
  const int64_t blocks = (n_groups + 7) / 8;
  if (blocks > 0x7fffffff) return fail(ctx, CATEN_B200_EUNSUPPORTED, "eval_expr: %lld output elements", (long long)n_out);
  launch_k(ctx, expr_kernel, dim3((unsigned)blocks), dim3(EXPR_THREADS), smem, *e, n_groups, (int)spw, n_red, result_cls);
  CB_LAUNCH_CHECK(ctx, "expr_kernel");
  return 0;
}

}  // namespace cb
