// Errors, arena, tensor storage and the eager tensor ops of the C API.
// Reference surface: include/cg_tensor.h, include/cg_arena.h, src/core/tensor.c,
// src/core/tensor_ops.c, src/utils/arena.c; error strings: src/core/tensor.c:443.
#include <algorithm>
#include <atomic>

#include "internal.hpp"

namespace {
thread_local cg_error g_err = CG_SUCCESS;
std::atomic<int> g_live{0};
std::atomic<uint64_t> g_seed{1}, g_layer_counter{0};

void fill_strides(cg_tensor* t) {
  int s = 1;
  for (int i = t->ndim - 1; i >= 0; --i) { t->strides[i] = s; s *= t->shape[i]; }
}
int numel(const int* shape, int ndim) {
  long n = 1;
  for (int i = 0; i < ndim; ++i) { if (shape[i] < 0) return -1; n *= shape[i]; if (n > 0x7fffffffL) return -1; }
  return (int)n;
}
cg_tensor* header(const int* shape, int ndim, bool rg) {
  if (ndim < 0 || ndim > CG_MAX_DIMS || (ndim > 0 && !shape)) return cgi::fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  int n = numel(shape, ndim);
  if (n < 0) return cgi::fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  cg_tensor* t = (cg_tensor*)std::calloc(1, sizeof(cg_tensor));
  if (!t) return cgi::fail(CG_ERROR_OUT_OF_MEMORY, (cg_tensor*)nullptr);
  for (int i = 0; i < ndim; ++i) t->shape[i] = shape[i];
  t->ndim = ndim; t->size = n; t->requires_grad = rg; t->ref_count = 1;
  fill_strides(t);
  g_live.fetch_add(1);
  return t;
}
}  // namespace

namespace cgi {
void set_error(cg_error e) { g_err = e; }
uint64_t next_layer_seed() { return g_seed.load() * 0x100000001B3ull + 0x9E37ull * (g_layer_counter.fetch_add(1) + 1); }

cg_tensor* make_header(const int* shape, int ndim, bool rg) { return header(shape, ndim, rg); }
cg_tensor* make(const int* shape, int ndim, bool rg) {
  cg_tensor* t = header(shape, ndim, rg);
  if (!t) return nullptr;
  t->data = (float*)std::calloc(t->size > 0 ? t->size : 1, sizeof(float));
  if (!t->data) { std::free(t); g_live.fetch_sub(1); return fail(CG_ERROR_OUT_OF_MEMORY, (cg_tensor*)nullptr); }
  if (rg) ensure_grad(t);
  return t;
}
cg_tensor* make_like(const cg_tensor* t, bool rg) { return make(t->shape, t->ndim, rg); }
void ensure_grad(cg_tensor* t) {
  if (t->grad) return;
  if (t->arena) t->grad = (float*)cg_arena_alloc(t->arena, sizeof(float) * (t->size ? t->size : 1), 16);
  else t->grad = (float*)std::calloc(t->size > 0 ? t->size : 1, sizeof(float));
  if (t->arena && t->grad) std::memset(t->grad, 0, sizeof(float) * t->size);
}

// The host GEMM: C[M,N] (+)= op(A) op(B).  Every case is brought to the form "row of C += a * row of B"
// with unit stride along the row (B^T is transposed into a scratch buffer first); the loops themselves are
// in host_simd.cpp.
void gemm(const float* A, const float* B, float* C, int M, int N, int K, bool ta, bool tb, bool acc) {
  if (!acc) std::memset(C, 0, sizeof(float) * (size_t)M * N);
  if (M <= 0 || N <= 0 || K <= 0) return;
  if (!tb) { gemm_rows(A, B, C, M, N, K, ta); return; }
  if (!ta && M < 4) { gemm_dots(A, B, C, M, N, K); return; }
  // B is [N, K]: transpose it once (N * K moves against 2 * M * N * K flops)
  static thread_local std::vector<float> bt;
  if (bt.size() < (size_t)N * K) bt.resize((size_t)N * K);
  float* t = bt.data();
  for (int j0 = 0; j0 < N; j0 += 32)
    for (int k0 = 0; k0 < K; k0 += 32) {
      const int j1 = std::min(N, j0 + 32), k1 = std::min(K, k0 + 32);
      for (int j = j0; j < j1; ++j)
        for (int k = k0; k < k1; ++k) t[(size_t)k * N + j] = B[(size_t)j * K + k];
    }
  gemm_rows(A, t, C, M, N, K, ta);
  if (bt.size() > ((size_t)1 << 24)) std::vector<float>().swap(bt);      // a one-off large product does not pin 64 MB
}
}  // namespace cgi

using namespace cgi;

// ------------------------------------------------------------------ errors
CG_EXPORT const char* cg_error_string(cg_error e) {
  switch (e) {
    case CG_SUCCESS: return "success";
    case CG_ERROR_NULL_POINTER: return "null pointer";
    case CG_ERROR_SHAPE_MISMATCH: return "shape mismatch";
    case CG_ERROR_OUT_OF_MEMORY: return "out of memory";
    case CG_ERROR_INVALID_ARGUMENT: return "invalid argument";
    case CG_ERROR_FILE_NOT_FOUND: return "file not found";
    case CG_ERROR_INVALID_FORMAT: return "invalid format";
    case CG_ERROR_TIMEOUT: return "timeout";
  }
  return "unknown error";
}
CG_EXPORT cg_error cg_last_error(void) { cg_error e = g_err; g_err = CG_SUCCESS; return e; }
CG_EXPORT void cg_manual_seed(unsigned int seed) { g_seed.store((uint64_t)seed + 1); g_layer_counter.store(0); }

// ------------------------------------------------------------------- arena
static cg_arena_block* new_block(size_t size) {
  cg_arena_block* b = (cg_arena_block*)std::malloc(sizeof(cg_arena_block));
  if (!b) return nullptr;
  b->data = (unsigned char*)std::malloc(size);
  if (!b->data) { std::free(b); return nullptr; }
  b->size = size; b->used = 0; b->next = nullptr;
  return b;
}
CG_EXPORT cg_arena* cg_arena_new(size_t initial_size) {
  if (initial_size == 0) initial_size = 1 << 20;
  cg_arena* a = (cg_arena*)std::calloc(1, sizeof(cg_arena));
  if (!a) return fail(CG_ERROR_OUT_OF_MEMORY, (cg_arena*)nullptr);
  a->first = a->current = new_block(initial_size);
  if (!a->first) { std::free(a); return fail(CG_ERROR_OUT_OF_MEMORY, (cg_arena*)nullptr); }
  a->default_block_size = initial_size; a->total_allocated = initial_size;
  return a;
}
CG_EXPORT void* cg_arena_alloc(cg_arena* a, size_t size, size_t alignment) {
  if (!a) return fail(CG_ERROR_NULL_POINTER, (void*)nullptr);
  if (alignment == 0 || (alignment & (alignment - 1))) return fail(CG_ERROR_INVALID_ARGUMENT, (void*)nullptr);
  for (;;) {
    cg_arena_block* b = a->current;
    uintptr_t base = (uintptr_t)b->data + b->used;
    size_t pad = (alignment - (base & (alignment - 1))) & (alignment - 1);
    if (b->used + pad + size <= b->size) {
      b->used += pad + size; a->total_used += pad + size;
      return (void*)(base + pad);
    }
    if (b->next) { a->current = b->next; continue; }          // blocks kept by cg_arena_clear
    size_t want = size + alignment > a->default_block_size ? size + alignment : a->default_block_size;
    cg_arena_block* nb = new_block(want);
    if (!nb) return fail(CG_ERROR_OUT_OF_MEMORY, (void*)nullptr);
    b->next = nb; a->current = nb; a->total_allocated += want;
  }
}
CG_EXPORT void cg_arena_clear(cg_arena* a) {
  if (!a) return;
  for (cg_arena_block* b = a->first; b; b = b->next) b->used = 0;
  a->current = a->first; a->total_used = 0;
}
CG_EXPORT void cg_arena_free(cg_arena* a) {
  if (!a) return;
  for (cg_arena_block* b = a->first; b;) { cg_arena_block* n = b->next; std::free(b->data); std::free(b); b = n; }
  std::free(a);
}
CG_EXPORT size_t cg_arena_total_allocated(cg_arena* a) { return a ? a->total_allocated : 0; }
CG_EXPORT size_t cg_arena_total_used(cg_arena* a) { return a ? a->total_used : 0; }

// ---------------------------------------------------------------- creation
CG_EXPORT cg_tensor* cg_tensor_new(int* shape, int ndim, bool rg) { return make(shape, ndim, rg); }
CG_EXPORT cg_tensor* cg_tensor_zeros(int* shape, int ndim, bool rg) { return make(shape, ndim, rg); }
CG_EXPORT cg_tensor* cg_tensor_full(int* shape, int ndim, float v, bool rg) {
  cg_tensor* t = make(shape, ndim, rg);
  if (t) for (int i = 0; i < t->size; ++i) t->data[i] = v;
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_ones(int* shape, int ndim, bool rg) { return cg_tensor_full(shape, ndim, 1.0f, rg); }
CG_EXPORT cg_tensor* cg_tensor_rand(int* shape, int ndim, unsigned int seed, bool rg) {
  cg_tensor* t = make(shape, ndim, rg);
  if (t) { Rng r(seed); for (int i = 0; i < t->size; ++i) t->data[i] = r.uniform(); }
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_randn(int* shape, int ndim, unsigned int seed, bool rg) {
  cg_tensor* t = make(shape, ndim, rg);
  if (t) { Rng r(seed); for (int i = 0; i < t->size; ++i) t->data[i] = r.normal(); }
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_from_data(float* data, int* shape, int ndim, bool rg) {
  if (!data) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* t = make(shape, ndim, rg);
  if (t) std::memcpy(t->data, data, sizeof(float) * t->size);
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_clone(cg_tensor* s) {
  if (!s) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* t = make(s->shape, s->ndim, s->requires_grad);
  if (t) std::memcpy(t->data, s->data, sizeof(float) * s->size);
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_zeros_arena(cg_arena* arena, int* shape, int ndim, bool rg) {
  if (!arena) return make(shape, ndim, rg);
  int n = numel(shape, ndim);
  if (n < 0 || ndim > CG_MAX_DIMS) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  cg_tensor* t = (cg_tensor*)cg_arena_alloc(arena, sizeof(cg_tensor), 16);
  if (!t) return nullptr;
  std::memset(t, 0, sizeof(*t));
  for (int i = 0; i < ndim; ++i) t->shape[i] = shape[i];
  t->ndim = ndim; t->size = n; t->requires_grad = rg; t->ref_count = 1; t->arena = arena;
  fill_strides(t);
  t->data = (float*)cg_arena_alloc(arena, sizeof(float) * (n ? n : 1), 16);
  if (!t->data) return nullptr;
  std::memset(t->data, 0, sizeof(float) * n);
  if (rg) ensure_grad(t);
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_randn_arena(cg_arena* arena, int* shape, int ndim, unsigned int seed, bool rg) {
  cg_tensor* t = cg_tensor_zeros_arena(arena, shape, ndim, rg);
  if (t) { Rng r(seed); for (int i = 0; i < t->size; ++i) t->data[i] = r.normal(); }
  return t;
}
CG_EXPORT void cg_tensor_retain(cg_tensor* t) { if (t) ++t->ref_count; }
CG_EXPORT void cg_tensor_release(cg_tensor* t) {
  if (!t) return;
  if (t->ref_count > 1) { --t->ref_count; return; }     // the common case: somebody else still holds it
  // iterative: a long chain of parents must not recurse once per node.  The first entries of the
  // work list live on the stack; training loops free a handful of nodes per call.
  cg_tensor* first[32];
  int nfirst = 0;
  std::vector<cg_tensor*> more;
  first[nfirst++] = t;
  while (nfirst > 0 || !more.empty()) {
    cg_tensor* x;
    if (!more.empty()) { x = more.back(); more.pop_back(); } else x = first[--nfirst];
    if (--x->ref_count > 0) continue;
    for (int i = 0; i < x->num_parents; ++i) {
      if (!x->parents[i]) continue;
      if (nfirst < 32 && more.empty()) first[nfirst++] = x->parents[i]; else more.push_back(x->parents[i]);
    }
    if (x->backward_ctx) {
      BackCtx* c = (BackCtx*)x->backward_ctx; x->backward_ctx = nullptr;
      delete c;
    }
    if (x->arena) continue;                        // storage belongs to the arena
    if (!x->is_view) free_storage(x->data);      // host or device memory
    free_storage(x->grad);
    std::free(x);
    g_live.fetch_sub(1);
  }
}
CG_EXPORT void cg_tensor_free(cg_tensor* t) { cg_tensor_release(t); }
CG_EXPORT int cg_tensor_live_count(void) { return g_live.load(); }

// ------------------------------------------------------------- elementwise
static bool same3(cg_tensor* a, cg_tensor* b, cg_tensor* o) {
  if (!a || !b || !o) { set_error(CG_ERROR_NULL_POINTER); return false; }
  if (a->size != b->size || a->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return false; }
  return true;
}
static bool same2(cg_tensor* a, cg_tensor* o) {
  if (!a || !o) { set_error(CG_ERROR_NULL_POINTER); return false; }
  if (a->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return false; }
  return true;
}
static void trace2(cg_ir_opcode op, cg_tensor* a, cg_tensor* b, cg_tensor* o) {
  if (cg_jit_is_tracing()) { cg_tensor* in[2] = {a, b}; cg_jit_record(op, in, 2, o, nullptr, 0); }
}
static void trace1(cg_ir_opcode op, cg_tensor* a, cg_tensor* o, const void* attr = nullptr, size_t n = 0) {
  if (cg_jit_is_tracing()) { cg_tensor* in[1] = {a}; cg_jit_record(op, in, 1, o, attr, n); }
}
#define CG_BINARY(NAME, OP, IROP)                                                      \
  CG_EXPORT void NAME(cg_tensor* a, cg_tensor* b, cg_tensor* o) {                      \
    if (!same3(a, b, o)) return;                                                       \
    for (int i = 0; i < o->size; ++i) o->data[i] = a->data[i] OP b->data[i];           \
    trace2(IROP, a, b, o);                                                             \
  }
CG_BINARY(cg_tensor_add, +, OP_ADD)
CG_BINARY(cg_tensor_sub, -, OP_SUB)
CG_BINARY(cg_tensor_mul, *, OP_MUL)
CG_BINARY(cg_tensor_div, /, OP_DIV)
CG_EXPORT void cg_tensor_scale(cg_tensor* a, float s, cg_tensor* o) {
  if (!same2(a, o)) return;
  for (int i = 0; i < o->size; ++i) o->data[i] = a->data[i] * s;
}
CG_EXPORT void cg_tensor_exp(cg_tensor* a, cg_tensor* o) {
  if (!same2(a, o)) return;
  for (int i = 0; i < o->size; ++i) o->data[i] = std::exp(a->data[i]);
  trace1(OP_EXP, a, o);
}
CG_EXPORT void cg_tensor_log(cg_tensor* a, cg_tensor* o) {
  if (!same2(a, o)) return;
  for (int i = 0; i < o->size; ++i) o->data[i] = std::log(a->data[i]);
  trace1(OP_LOG, a, o);
}
CG_EXPORT void cg_tensor_pow(cg_tensor* a, float p, cg_tensor* o) {
  if (!same2(a, o)) return;
  for (int i = 0; i < o->size; ++i) o->data[i] = std::pow(a->data[i], p);
}

// ------------------------------------------------------------------ matmul
// a [..., M, K] times b [K, N] (shared) or b [..., K, N] (batched, equal leading size).
CG_EXPORT void cg_tensor_matmul(cg_tensor* a, cg_tensor* b, cg_tensor* o) {
  if (!a || !b || !o) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (a->ndim < 2 || b->ndim < 2) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int M = a->shape[a->ndim - 2], K = a->shape[a->ndim - 1];
  const int Kb = b->shape[b->ndim - 2], N = b->shape[b->ndim - 1];
  const int batch = a->size / (M * K), bbatch = b->size / (Kb * N);
  if (K != Kb || (bbatch != 1 && bbatch != batch) || o->size != batch * M * N) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  for (int i = 0; i < batch; ++i)
    gemm(a->data + (size_t)i * M * K, b->data + (bbatch == 1 ? 0 : (size_t)i * K * N), o->data + (size_t)i * M * N,
         M, N, K, false, false, false);
  trace2(OP_MATMUL, a, b, o);
}
CG_EXPORT void cg_tensor_transpose(cg_tensor* a, cg_tensor* o) {
  if (!same2(a, o)) return;
  if (a->ndim != 2) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int R = a->shape[0], C = a->shape[1];
  for (int i = 0; i < R; ++i) for (int j = 0; j < C; ++j) o->data[(size_t)j * R + i] = a->data[(size_t)i * C + j];
  trace1(OP_TRANSPOSE, a, o);
}

// -------------------------------------------------------------- reductions
enum RedKind { R_SUM, R_MEAN, R_MAX };
static void reduce(cg_tensor* a, int axis, cg_tensor* o, RedKind kind) {
  if (!a || !o) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (axis >= a->ndim) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  int outer = 1, len = a->size, inner = 1;
  if (axis >= 0) {
    len = a->shape[axis];
    for (int i = 0; i < axis; ++i) outer *= a->shape[i];
    for (int i = axis + 1; i < a->ndim; ++i) inner *= a->shape[i];
  }
  if (o->size != outer * inner || len == 0) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  for (int x = 0; x < outer; ++x)
    for (int z = 0; z < inner; ++z) {
      const float* p = a->data + (size_t)x * len * inner + z;
      double acc = kind == R_MAX ? p[0] : 0.0;
      for (int k = 0; k < len; ++k) {
        const float v = p[(size_t)k * inner];
        if (kind == R_MAX) { if (v > acc) acc = v; } else acc += v;
      }
      if (kind == R_MEAN) acc /= len;
      o->data[(size_t)x * inner + z] = (float)acc;
    }
  static const cg_ir_opcode ops[3] = {OP_SUM, OP_MEAN, OP_MAX};
  trace1(ops[kind], a, o, &axis, sizeof(axis));
}
CG_EXPORT void cg_tensor_sum(cg_tensor* a, int axis, cg_tensor* o) { reduce(a, axis, o, R_SUM); }
CG_EXPORT void cg_tensor_mean(cg_tensor* a, int axis, cg_tensor* o) { reduce(a, axis, o, R_MEAN); }
CG_EXPORT void cg_tensor_max(cg_tensor* a, int axis, cg_tensor* o) { reduce(a, axis, o, R_MAX); }

// --------------------------------------------------------------- utilities
CG_EXPORT void cg_tensor_zero_grad(cg_tensor* t) { if (t && t->grad) std::memset(t->grad, 0, sizeof(float) * t->size); }
CG_EXPORT void cg_tensor_print(cg_tensor* t, const char* name) {
  if (!t) { std::printf("%s: (null)\n", name ? name : "tensor"); return; }
  std::printf("%s: shape=[", name ? name : "tensor");
  for (int i = 0; i < t->ndim; ++i) std::printf(i ? ", %d" : "%d", t->shape[i]);
  std::printf("] data=[");
  const int n = t->size < 16 ? t->size : 16;
  for (int i = 0; i < n; ++i) std::printf(i ? ", %.6g" : "%.6g", t->data[i]);
  std::printf(t->size > n ? ", ...]\n" : "]\n");
}
static long flat_index(cg_tensor* t, int* idx) {
  long off = 0;
  for (int i = 0; i < t->ndim; ++i) { if (idx[i] < 0 || idx[i] >= t->shape[i]) return -1; off += (long)idx[i] * t->strides[i]; }
  return off;
}
CG_EXPORT float cg_tensor_get(cg_tensor* t, int* idx) {
  if (!t || !idx) return fail(CG_ERROR_NULL_POINTER, 0.0f);
  long o = flat_index(t, idx);
  return o < 0 ? fail(CG_ERROR_INVALID_ARGUMENT, 0.0f) : t->data[o];
}
CG_EXPORT void cg_tensor_set(cg_tensor* t, int* idx, float v) {
  if (!t || !idx) { set_error(CG_ERROR_NULL_POINTER); return; }
  long o = flat_index(t, idx);
  if (o < 0) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  t->data[o] = v;
}
CG_EXPORT void cg_tensor_reshape(cg_tensor* t, int* shape, int ndim) {
  if (!t || !shape) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (ndim > CG_MAX_DIMS || numel(shape, ndim) != t->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  for (int i = 0; i < ndim; ++i) t->shape[i] = shape[i];
  t->ndim = ndim;
  fill_strides(t);
}
CG_EXPORT bool cg_tensor_shape_equal(cg_tensor* a, cg_tensor* b) {
  if (!a || !b || a->ndim != b->ndim) return false;
  for (int i = 0; i < a->ndim; ++i) if (a->shape[i] != b->shape[i]) return false;
  return true;
}

// --------------------------------------------------------------- broadcast
CG_EXPORT bool cg_broadcast_shapes(int* sa, int na, int* sb, int nb, int* out, int* nout) {
  const int n = na > nb ? na : nb;
  if (n > CG_MAX_DIMS) return false;
  for (int i = 0; i < n; ++i) {
    const int da = i < n - na ? 1 : sa[i - (n - na)], db = i < n - nb ? 1 : sb[i - (n - nb)];
    if (da != db && da != 1 && db != 1) return false;
    out[i] = da == 1 ? db : da;
  }
  *nout = n;
  return true;
}
CG_EXPORT void cg_broadcast_strides(int* shape, int ndim, int* out_shape, int out_ndim, int* out_strides) {
  int s = 1;
  for (int i = out_ndim - 1; i >= 0; --i) {
    const int j = i - (out_ndim - ndim);
    if (j < 0 || shape[j] == 1) { out_strides[i] = 0; if (j >= 0) s *= shape[j]; }
    else { out_strides[i] = s; s *= shape[j]; }
  }
  (void)out_shape;
}
template <class F> static cg_tensor* broadcast_op(cg_tensor* a, cg_tensor* b, F f) {
  if (!a || !b) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  int shape[CG_MAX_DIMS], nd;
  if (!cg_broadcast_shapes(a->shape, a->ndim, b->shape, b->ndim, shape, &nd)) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  cg_tensor* o = make(shape, nd, false);
  if (!o) return nullptr;
  int sa[CG_MAX_DIMS], sb[CG_MAX_DIMS], idx[CG_MAX_DIMS] = {0};
  cg_broadcast_strides(a->shape, a->ndim, shape, nd, sa);
  cg_broadcast_strides(b->shape, b->ndim, shape, nd, sb);
  long oa = 0, ob = 0;
  for (int i = 0; i < o->size; ++i) {
    o->data[i] = f(a->data[oa], b->data[ob]);
    for (int d = nd - 1; d >= 0; --d) {          // odometer
      ++idx[d]; oa += sa[d]; ob += sb[d];
      if (idx[d] < shape[d]) break;
      oa -= (long)sa[d] * shape[d]; ob -= (long)sb[d] * shape[d]; idx[d] = 0;
    }
  }
  return o;
}
CG_EXPORT cg_tensor* cg_tensor_add_broadcast(cg_tensor* a, cg_tensor* b) { return broadcast_op(a, b, [](float x, float y) { return x + y; }); }
CG_EXPORT cg_tensor* cg_tensor_sub_broadcast(cg_tensor* a, cg_tensor* b) { return broadcast_op(a, b, [](float x, float y) { return x - y; }); }
CG_EXPORT cg_tensor* cg_tensor_mul_broadcast(cg_tensor* a, cg_tensor* b) { return broadcast_op(a, b, [](float x, float y) { return x * y; }); }
CG_EXPORT cg_tensor* cg_tensor_div_broadcast(cg_tensor* a, cg_tensor* b) { return broadcast_op(a, b, [](float x, float y) { return x / y; }); }

CG_EXPORT cg_tensor* cg_tensor_stack(cg_tensor** ts, int count) {
  if (!ts || count <= 0 || !ts[0]) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  if (ts[0]->ndim + 1 > CG_MAX_DIMS) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  int shape[CG_MAX_DIMS];
  shape[0] = count;
  for (int i = 0; i < ts[0]->ndim; ++i) shape[i + 1] = ts[0]->shape[i];
  for (int i = 1; i < count; ++i) if (!cg_tensor_shape_equal(ts[0], ts[i])) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  cg_tensor* o = make(shape, ts[0]->ndim + 1, false);
  if (o) for (int i = 0; i < count; ++i) std::memcpy(o->data + (size_t)i * ts[0]->size, ts[i]->data, sizeof(float) * ts[0]->size);
  return o;
}
CG_EXPORT cg_tensor* cg_tensor_cat(cg_tensor** ts, int count, int dim) {
  if (!ts || count <= 0 || !ts[0]) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  const int nd = ts[0]->ndim;
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  int shape[CG_MAX_DIMS];
  for (int i = 0; i < nd; ++i) shape[i] = ts[0]->shape[i];
  shape[dim] = 0;
  for (int t = 0; t < count; ++t) {
    if (!ts[t] || ts[t]->ndim != nd) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
    for (int i = 0; i < nd; ++i) if (i != dim && ts[t]->shape[i] != shape[i]) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
    shape[dim] += ts[t]->shape[dim];
  }
  cg_tensor* o = make(shape, nd, false);
  if (!o) return nullptr;
  int outer = 1, inner = 1;
  for (int i = 0; i < dim; ++i) outer *= shape[i];
  for (int i = dim + 1; i < nd; ++i) inner *= shape[i];
  size_t col = 0;
  for (int t = 0; t < count; ++t) {
    const size_t w = (size_t)ts[t]->shape[dim] * inner;
    for (int x = 0; x < outer; ++x)
      std::memcpy(o->data + (size_t)x * shape[dim] * inner + col, ts[t]->data + x * w, sizeof(float) * w);
    col += w;
  }
  return o;
}
