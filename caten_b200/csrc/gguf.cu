// GGUF file reader: header, metadata key/values, tensor infos and the alignment rule, over a
// read-only memory map, so that packed tensor blocks go file -> device without being touched on
// the host.  Replaces the per-element Lisp reader of external/gguf/gguf-file.lisp:48-81,
// metadata.lisp:3-87 and tensor-info.lisp:79-102 (which dequantises every tensor to fp32 while
// parsing).  Host code only; compiled with the rest of the library.
//
// File layout (the structure make-gguf documents at gguf-file.lisp:53-60):
//   "GGUF" | version u32 | tensor_count u64 | metadata_kv_count u64 | kv... | tensor_info... | pad | data
// A tensor's bytes start at align_up(end of tensor infos, alignment) + its relative offset, with
// alignment = metadata "general.alignment" or 32 (gguf-file.lisp:71-72, tensor-info.lisp:88-98).
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

enum MetaType : uint32_t { U8 = 0, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 };

struct Meta {
  std::string key;
  uint32_t type = 0, elem_type = 0;
  uint64_t count = 0;        // array length (1 for scalars)
  const uint8_t *value = nullptr;  // scalars: the little-endian bytes; strings: first byte; arrays: first element
  uint64_t str_len = 0;
};

struct Tensor {
  std::string name;
  int type = 0, n_dims = 0;
  int64_t dims[4] = {1, 1, 1, 1};  // GGUF order: dims[0] is the innermost (contiguous) dimension
  uint64_t rel_offset = 0;
  const uint8_t *data = nullptr;
  int64_t nbytes = 0;
};

struct Cursor {
  const uint8_t *p, *end;
  bool ok = true;
  template <typename T> T get() {
    T v{};
    if ((size_t)(end - p) < sizeof(T)) { ok = false; p = end; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  const uint8_t *skip(uint64_t n) {
    if ((uint64_t)(end - p) < n) { ok = false; p = end; return nullptr; }
    const uint8_t *q = p;
    p += n;
    return q;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    const uint8_t *q = skip(n);
    return q ? std::string((const char *)q, (size_t)n) : std::string();
  }
};

int scalar_size(uint32_t t) {
  switch (t) {
    case U8: case I8: case BOOL: return 1;
    case U16: case I16: return 2;
    case U32: case I32: case F32: return 4;
    case U64: case I64: case F64: return 8;
  }
  return 0;
}

}  // namespace

struct caten_b200_gguf {
  int fd = -1;
  const uint8_t *base = nullptr;
  size_t size = 0;
  uint32_t version = 0;
  uint64_t alignment = 32;
  std::vector<Meta> meta;
  std::vector<Tensor> tensors;
};

static bool skip_value(Cursor &c, uint32_t type, Meta *m) {
  if (type == STR) {
    const uint64_t n = c.get<uint64_t>();
    const uint8_t *q = c.skip(n);
    if (m) { m->value = q; m->str_len = n; }
    return c.ok;
  }
  if (type == ARR) {
    const uint32_t et = c.get<uint32_t>();
    const uint64_t n = c.get<uint64_t>();
    if (et == ARR) { c.ok = false; return false; }  // nested arrays are not part of the format
    if (m) { m->elem_type = et; m->count = n; m->value = c.p; }
    if (et == STR) {
      for (uint64_t i = 0; i < n && c.ok; ++i) c.skip(c.get<uint64_t>());
    } else {
      const int sz = scalar_size(et);
      if (!sz || (n && (uint64_t)(c.end - c.p) / sz < n)) { c.ok = false; return false; }
      c.skip(n * sz);
    }
    return c.ok;
  }
  const int sz = scalar_size(type);
  if (!sz) { c.ok = false; return false; }
  const uint8_t *q = c.skip(sz);
  if (m) m->value = q;
  return c.ok;
}

extern "C" {

int caten_b200_gguf_open(const char *path, caten_b200_gguf **out) {
  using cb::fail;
  if (!path || !out) return fail(nullptr, CATEN_B200_EINVAL, "gguf_open: NULL argument");
  *out = nullptr;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return fail(nullptr, CATEN_B200_EINVAL, "gguf_open: cannot open %s", path);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 24) { close(fd); return fail(nullptr, CATEN_B200_EINVAL, "gguf_open: %s is too short to be a GGUF file", path); }
  void *map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (map == MAP_FAILED) { close(fd); return fail(nullptr, CATEN_B200_EINVAL, "gguf_open: mmap of %s failed", path); }
  caten_b200_gguf *g = new (std::nothrow) caten_b200_gguf();
  if (!g) { munmap(map, (size_t)st.st_size); close(fd); return fail(nullptr, CATEN_B200_ECUDA, "out of host memory"); }
  g->fd = fd; g->base = (const uint8_t *)map; g->size = (size_t)st.st_size;
  auto bad = [&](const char *why) {
    const int rc = fail(nullptr, CATEN_B200_EINVAL, "gguf_open: %s: %s", path, why);
    munmap((void *)g->base, g->size); close(g->fd); delete g;
    return rc;
  };
  Cursor c{g->base, g->base + g->size};
  if (memcmp(c.skip(4), "GGUF", 4) != 0) return bad("the magic is not \"GGUF\"");
  g->version = c.get<uint32_t>();
  if (g->version < 2 || g->version > 3) return bad("unsupported GGUF version (2 and 3 are read)");
  const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
  if (n_tensors > (1u << 24) || n_kv > (1u << 24)) return bad("implausible tensor or metadata count");
  for (uint64_t i = 0; i < n_kv; ++i) {
    Meta m;
    m.key = c.str();
    m.type = c.get<uint32_t>();
    m.count = 1;
    if (!c.ok || !skip_value(c, m.type, &m)) return bad("truncated or malformed metadata");
    if (m.key == "general.alignment" && m.type == U32) { uint32_t a; memcpy(&a, m.value, 4); if (a) g->alignment = a; }
    g->meta.push_back(std::move(m));
  }
  for (uint64_t i = 0; i < n_tensors; ++i) {
    Tensor t;
    t.name = c.str();
    t.n_dims = (int)c.get<uint32_t>();
    if (!c.ok || t.n_dims < 1 || t.n_dims > 4) return bad("tensor with an unsupported number of dimensions");
    for (int k = 0; k < t.n_dims; ++k) {
      const uint64_t dim = c.get<uint64_t>();
      if (dim == 0 || dim > (uint64_t)1 << 31) return bad("tensor dimension is zero or larger than 2^31");
      t.dims[k] = (int64_t)dim;
    }
    t.type = (int)c.get<uint32_t>();
    t.rel_offset = c.get<uint64_t>();
    if (!c.ok) return bad("truncated tensor table");
    g->tensors.push_back(std::move(t));
  }
  const uint64_t table_end = (uint64_t)(c.p - g->base);
  const uint64_t data_start = (table_end + g->alignment - 1) / g->alignment * g->alignment;
  for (Tensor &t : g->tensors) {
    int64_t rows = 1, count = 0;
    for (int k = 1; k < t.n_dims; ++k)
      if (__builtin_mul_overflow(rows, t.dims[k], &rows)) return bad("tensor element count overflows");
    if (__builtin_mul_overflow(rows, t.dims[0], &count) || count > INT64_MAX / 8) return bad("tensor element count overflows");
    t.nbytes = caten_b200_weight_nbytes(t.type, rows, t.dims[0]);  // -1: a ggml type this library does not hold
    uint64_t off = 0;
    if (__builtin_add_overflow(data_start, t.rel_offset, &off)) return bad("tensor offset overflows");
    if (t.rel_offset % g->alignment) return bad("tensor offset is not a multiple of the alignment");
    if (t.nbytes >= 0 && (off > g->size || (uint64_t)t.nbytes > g->size - off)) return bad("tensor data runs past the end of the file");
    t.data = off <= g->size ? g->base + off : nullptr;
  }
  *out = g;
  return 0;
}

int caten_b200_gguf_close(caten_b200_gguf *g) {
  if (!g) return 0;
  munmap((void *)g->base, g->size);
  close(g->fd);
  delete g;
  return 0;
}

int64_t caten_b200_gguf_tensor_count(const caten_b200_gguf *g) { return g ? (int64_t)g->tensors.size() : -1; }
int64_t caten_b200_gguf_meta_count(const caten_b200_gguf *g) { return g ? (int64_t)g->meta.size() : -1; }
int64_t caten_b200_gguf_alignment(const caten_b200_gguf *g) { return g ? (int64_t)g->alignment : -1; }
int caten_b200_gguf_version(const caten_b200_gguf *g) { return g ? (int)g->version : -1; }

int caten_b200_gguf_tensor(const caten_b200_gguf *g, int64_t i, const char **name, int *ggml_type, int *n_dims,
                           int64_t *dims4, const void **data, int64_t *nbytes) {
  if (!g || i < 0 || i >= (int64_t)g->tensors.size()) return cb::fail(nullptr, CATEN_B200_EINVAL, "gguf_tensor: index out of range");
  const Tensor &t = g->tensors[(size_t)i];
  if (name) *name = t.name.c_str();
  if (ggml_type) *ggml_type = t.type;
  if (n_dims) *n_dims = t.n_dims;
  if (dims4) for (int k = 0; k < 4; ++k) dims4[k] = t.dims[k];
  if (data) *data = t.data;
  if (nbytes) *nbytes = t.nbytes;
  return 0;
}

int64_t caten_b200_gguf_find_tensor(const caten_b200_gguf *g, const char *name) {
  if (!g || !name) return -1;
  for (size_t i = 0; i < g->tensors.size(); ++i)
    if (g->tensors[i].name == name) return (int64_t)i;
  return -1;
}

int caten_b200_gguf_meta(const caten_b200_gguf *g, int64_t i, const char **key, int *type, int *elem_type, int64_t *count,
                         const void **value, int64_t *str_len) {
  if (!g || i < 0 || i >= (int64_t)g->meta.size()) return cb::fail(nullptr, CATEN_B200_EINVAL, "gguf_meta: index out of range");
  const Meta &m = g->meta[(size_t)i];
  if (key) *key = m.key.c_str();
  if (type) *type = (int)m.type;
  if (elem_type) *elem_type = (int)m.elem_type;
  if (count) *count = (int64_t)m.count;
  if (value) *value = m.value;
  if (str_len) *str_len = (int64_t)m.str_len;
  return 0;
}

int caten_b200_gguf_upload(caten_b200_ctx *ctx, const caten_b200_gguf *g, int64_t i, caten_b200_weight **w) {
  if (!ctx) return cb::fail(nullptr, CATEN_B200_EINVAL, "gguf_upload: ctx is NULL");
  if (!g || i < 0 || i >= (int64_t)g->tensors.size()) return cb::fail(ctx, CATEN_B200_EINVAL, "gguf_upload: index out of range");
  const Tensor &t = g->tensors[(size_t)i];
  if (t.n_dims != 2) return cb::fail(ctx, CATEN_B200_EUNSUPPORTED, "gguf_upload: %s has %d dimensions; Linear weights are 2-D", t.name.c_str(), t.n_dims);
  if (t.nbytes < 0) return cb::fail(ctx, CATEN_B200_EUNSUPPORTED, "gguf_upload: %s has ggml type %d (held: F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K)", t.name.c_str(), t.type);
  // GGUF lists the contiguous dimension first: [cols, rows] (tensor-info.lisp:108 reverses it on load)
  return caten_b200_weight_upload(ctx, t.type, t.data, t.dims[1], t.dims[0], w);
}

}  // extern "C"
