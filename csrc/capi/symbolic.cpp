// Symbolic dimensions, integer expressions over named variables, symbolic shapes with
// broadcast / matmul inference, and shape guards for specialised kernels.
// Reference surface: include/cg_symbolic.h, src/core/symbolic.c.
#include <string>

#include "internal.hpp"

using namespace cgi;

static cg_symbolic_expr* new_expr(cg_expr_type t) { cg_symbolic_expr* e = (cg_symbolic_expr*)std::calloc(1, sizeof(cg_symbolic_expr)); e->type = t; return e; }
CG_EXPORT cg_symbolic_expr* cg_expr_const(int64_t v) { cg_symbolic_expr* e = new_expr(EXPR_CONST); e->data.constant = v; return e; }
CG_EXPORT cg_symbolic_expr* cg_expr_var(const char* name) {
  if (!name) return fail(CG_ERROR_NULL_POINTER, (cg_symbolic_expr*)nullptr);
  cg_symbolic_expr* e = new_expr(EXPR_VAR); e->data.variable = strdup(name); return e;
}
// Takes ownership of both operands; constant operands fold.
CG_EXPORT cg_symbolic_expr* cg_expr_binary(cg_expr_type t, cg_symbolic_expr* l, cg_symbolic_expr* r) {
  if (!l || !r || t == EXPR_CONST || t == EXPR_VAR) { cg_expr_free(l); cg_expr_free(r); return fail(CG_ERROR_INVALID_ARGUMENT, (cg_symbolic_expr*)nullptr); }
  cg_symbolic_expr* e = new_expr(t);
  e->data.binary.left = l; e->data.binary.right = r;
  if (l->type == EXPR_CONST && r->type == EXPR_CONST) {
    int64_t v;
    if (cg_expr_try_eval(e, nullptr, nullptr, 0, &v)) { cg_expr_free(e); return cg_expr_const(v); }
  }
  return e;
}
CG_EXPORT cg_symbolic_expr* cg_expr_add(cg_symbolic_expr* l, cg_symbolic_expr* r) { return cg_expr_binary(EXPR_ADD, l, r); }
CG_EXPORT cg_symbolic_expr* cg_expr_sub(cg_symbolic_expr* l, cg_symbolic_expr* r) { return cg_expr_binary(EXPR_SUB, l, r); }
CG_EXPORT cg_symbolic_expr* cg_expr_mul(cg_symbolic_expr* l, cg_symbolic_expr* r) { return cg_expr_binary(EXPR_MUL, l, r); }
CG_EXPORT cg_symbolic_expr* cg_expr_div(cg_symbolic_expr* l, cg_symbolic_expr* r) { return cg_expr_binary(EXPR_DIV, l, r); }
CG_EXPORT cg_symbolic_expr* cg_expr_floordiv(cg_symbolic_expr* l, cg_symbolic_expr* r) { return cg_expr_binary(EXPR_FLOORDIV, l, r); }
static cg_symbolic_expr* expr_clone(const cg_symbolic_expr* e) {
  if (!e) return nullptr;
  if (e->type == EXPR_CONST) return cg_expr_const(e->data.constant);
  if (e->type == EXPR_VAR) return cg_expr_var(e->data.variable);
  cg_symbolic_expr* c = new_expr(e->type);
  c->data.binary.left = expr_clone(e->data.binary.left); c->data.binary.right = expr_clone(e->data.binary.right);
  return c;
}
CG_EXPORT bool cg_expr_try_eval(cg_symbolic_expr* e, int64_t* vals, const char** names, int n, int64_t* out) {
  if (!e || !out) return false;
  if (e->type == EXPR_CONST) { *out = e->data.constant; return true; }
  if (e->type == EXPR_VAR) {
    for (int i = 0; i < n; ++i) if (names[i] && !std::strcmp(names[i], e->data.variable)) { *out = vals[i]; return true; }
    return false;
  }
  int64_t a, b;
  if (!cg_expr_try_eval(e->data.binary.left, vals, names, n, &a) || !cg_expr_try_eval(e->data.binary.right, vals, names, n, &b)) return false;
  switch (e->type) {
    case EXPR_ADD: *out = a + b; return true;
    case EXPR_SUB: *out = a - b; return true;
    case EXPR_MUL: *out = a * b; return true;
    case EXPR_DIV: if (b == 0) return false; *out = a / b; return true;
    case EXPR_FLOORDIV: if (b == 0) return false; *out = a / b - ((a % b != 0) && ((a < 0) != (b < 0))); return true;
    case EXPR_MOD: if (b == 0) return false; *out = ((a % b) + b) % b; return true;
    case EXPR_MAX: *out = a > b ? a : b; return true;
    case EXPR_MIN: *out = a < b ? a : b; return true;
    default: return false;
  }
}
// The reference's evaluator (include/cg_symbolic.h, src/core/symbolic.c:88-140): the value, or -1 for an unbound
// variable or an operation it cannot carry out (it prints "Unbound variable" there; here the error code says so).
CG_EXPORT int64_t cg_expr_eval(cg_symbolic_expr* e, int64_t* vals, const char** names, int n) {
  int64_t v = -1;
  if (!cg_expr_try_eval(e, vals, names, n, &v)) { set_error(CG_ERROR_INVALID_ARGUMENT); return -1; }
  return v;
}
static void expr_str(const cg_symbolic_expr* e, std::string& s) {
  if (!e) { s += "?"; return; }
  if (e->type == EXPR_CONST) { s += std::to_string(e->data.constant); return; }
  if (e->type == EXPR_VAR) { s += e->data.variable; return; }
  static const char* ops[] = {"", "", " + ", " - ", " * ", " / ", " // ", " % ", "", ""};
  if (e->type == EXPR_MAX || e->type == EXPR_MIN) {
    s += e->type == EXPR_MAX ? "max(" : "min(";
    expr_str(e->data.binary.left, s); s += ", "; expr_str(e->data.binary.right, s); s += ")";
    return;
  }
  s += "("; expr_str(e->data.binary.left, s); s += ops[e->type]; expr_str(e->data.binary.right, s); s += ")";
}
CG_EXPORT char* cg_expr_to_string(cg_symbolic_expr* e) { std::string s; expr_str(e, s); return strdup(s.c_str()); }
CG_EXPORT void cg_expr_free(cg_symbolic_expr* e) {
  if (!e) return;
  if (e->type == EXPR_VAR) std::free(e->data.variable);
  else if (e->type != EXPR_CONST) { cg_expr_free(e->data.binary.left); cg_expr_free(e->data.binary.right); }
  std::free(e);
}

// -------------------------------------------------------------------- dims
static cg_symbolic_dim* new_dim(cg_dim_type t) {
  cg_symbolic_dim* d = (cg_symbolic_dim*)std::calloc(1, sizeof(cg_symbolic_dim));
  d->type = t; d->min_value = 1; d->max_value = INT64_MAX; d->divisor = 1;
  return d;
}
CG_EXPORT cg_symbolic_dim* cg_dim_const(int64_t v) { cg_symbolic_dim* d = new_dim(DIM_CONSTANT); d->value = v; d->min_value = d->max_value = v; return d; }
CG_EXPORT cg_symbolic_dim* cg_dim_var(const char* name) {
  if (!name) return fail(CG_ERROR_NULL_POINTER, (cg_symbolic_dim*)nullptr);
  cg_symbolic_dim* d = new_dim(DIM_SYMBOLIC); d->name = strdup(name); return d;
}
CG_EXPORT cg_symbolic_dim* cg_dim_inferred(cg_symbolic_expr* e) {
  if (!e) return fail(CG_ERROR_NULL_POINTER, (cg_symbolic_dim*)nullptr);
  if (e->type == EXPR_CONST) { cg_symbolic_dim* d = cg_dim_const(e->data.constant); cg_expr_free(e); return d; }
  cg_symbolic_dim* d = new_dim(DIM_INFERRED); d->expr = e; return d;
}
static cg_symbolic_dim* dim_clone(const cg_symbolic_dim* s) {
  cg_symbolic_dim* d = new_dim(s->type);
  *d = *s;
  d->name = s->name ? strdup(s->name) : nullptr;
  d->expr = expr_clone(s->expr);
  return d;
}
CG_EXPORT void cg_dim_constrain(cg_symbolic_dim* d, int64_t lo, int64_t hi) { if (d) { d->min_value = lo; d->max_value = hi; } }
CG_EXPORT void cg_dim_set_divisor(cg_symbolic_dim* d, int64_t k) { if (d && k > 0) { d->divisible_by = k > 1; d->divisor = k; } }
static bool same_expr(const cg_symbolic_expr* a, const cg_symbolic_expr* b) {
  if (!a || !b) return a == b;
  if (a->type != b->type) return false;
  if (a->type == EXPR_CONST) return a->data.constant == b->data.constant;
  if (a->type == EXPR_VAR) return !std::strcmp(a->data.variable, b->data.variable);
  return same_expr(a->data.binary.left, b->data.binary.left) && same_expr(a->data.binary.right, b->data.binary.right);
}
// Can the two dimensions denote the same extent?  Constants must be equal; a variable is
// compatible with a constant inside its range (and divisor), with the same variable, or with
// another variable whose range overlaps.
CG_EXPORT bool cg_dim_compatible(cg_symbolic_dim* a, cg_symbolic_dim* b) {
  if (!a || !b) return false;
  if (a->type == DIM_CONSTANT && b->type == DIM_CONSTANT) return a->value == b->value;
  if (a->type == DIM_CONSTANT) { cg_symbolic_dim* t = a; a = b; b = t; }
  if (b->type == DIM_CONSTANT) return b->value >= a->min_value && b->value <= a->max_value && (!a->divisible_by || b->value % a->divisor == 0);
  if (a->type == DIM_SYMBOLIC && b->type == DIM_SYMBOLIC && !std::strcmp(a->name, b->name)) return true;
  if (a->type == DIM_INFERRED && b->type == DIM_INFERRED && same_expr(a->expr, b->expr)) return true;
  return a->min_value <= b->max_value && b->min_value <= a->max_value;
}
CG_EXPORT int64_t cg_dim_resolve(cg_symbolic_dim* d, int64_t* vals, const char** names, int n) {
  if (!d) return -1;
  int64_t v = -1;
  if (d->type == DIM_CONSTANT) v = d->value;
  else if (d->type == DIM_INFERRED) { if (!cg_expr_try_eval(d->expr, vals, names, n, &v)) return -1; }
  else {
    bool found = false;
    for (int i = 0; i < n && d->name; ++i) if (names[i] && !std::strcmp(names[i], d->name)) { v = vals[i]; found = true; break; }
    if (!found) return -1;
  }
  if (v < d->min_value || v > d->max_value || (d->divisible_by && v % d->divisor)) return -1;
  return v;
}
CG_EXPORT void cg_dim_free(cg_symbolic_dim* d) { if (d) { std::free(d->name); cg_expr_free(d->expr); std::free(d); } }

// ------------------------------------------------------------------ shapes
static uint64_t hash_bytes(uint64_t h, const void* p, size_t n) { const unsigned char* b = (const unsigned char*)p; for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 0x100000001B3ull; } return h; }
static uint64_t hash_expr(uint64_t h, const cg_symbolic_expr* e) {
  if (!e) return h;
  h = hash_bytes(h, &e->type, sizeof(e->type));
  if (e->type == EXPR_CONST) return hash_bytes(h, &e->data.constant, 8);
  if (e->type == EXPR_VAR) return hash_bytes(h, e->data.variable, std::strlen(e->data.variable));
  return hash_expr(hash_expr(h, e->data.binary.left), e->data.binary.right);
}
CG_EXPORT uint64_t cg_shape_hash(cg_symbolic_shape* s) {
  if (!s) return 0;
  uint64_t h = 0xCBF29CE484222325ull;
  h = hash_bytes(h, &s->ndim, sizeof(int));
  for (int i = 0; i < s->ndim; ++i) {
    const cg_symbolic_dim* d = s->dims[i];
    h = hash_bytes(h, &d->type, sizeof(d->type));
    if (d->type == DIM_CONSTANT) h = hash_bytes(h, &d->value, 8);
    else if (d->name) h = hash_bytes(h, d->name, std::strlen(d->name));
    h = hash_expr(h, d->expr);
  }
  return h;
}
CG_EXPORT cg_symbolic_shape* cg_shape_new(cg_symbolic_dim** dims, int ndim) {
  if (ndim < 0 || ndim > CG_MAX_DIMS || (ndim && !dims)) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_symbolic_shape*)nullptr);
  cg_symbolic_shape* s = (cg_symbolic_shape*)std::calloc(1, sizeof(cg_symbolic_shape));
  s->ndim = ndim; s->dims = (cg_symbolic_dim**)std::calloc(ndim ? ndim : 1, sizeof(cg_symbolic_dim*));
  for (int i = 0; i < ndim; ++i) s->dims[i] = dims[i];
  s->hash = cg_shape_hash(s);
  return s;
}
CG_EXPORT cg_symbolic_shape* cg_shape_from_ints(int* dims, int ndim) {
  if (ndim < 0 || ndim > CG_MAX_DIMS || (ndim && !dims)) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_symbolic_shape*)nullptr);
  cg_symbolic_dim* ds[CG_MAX_DIMS];
  for (int i = 0; i < ndim; ++i) ds[i] = cg_dim_const(dims[i]);
  return cg_shape_new(ds, ndim);
}
static bool is_one(const cg_symbolic_dim* d) { return d->type == DIM_CONSTANT && d->value == 1; }
CG_EXPORT cg_symbolic_shape* cg_shape_broadcast(cg_symbolic_shape* a, cg_symbolic_shape* b) {
  if (!a || !b) return fail(CG_ERROR_NULL_POINTER, (cg_symbolic_shape*)nullptr);
  const int n = a->ndim > b->ndim ? a->ndim : b->ndim;
  cg_symbolic_dim* out[CG_MAX_DIMS];
  for (int i = 0; i < n; ++i) {
    const cg_symbolic_dim* da = i < n - a->ndim ? nullptr : a->dims[i - (n - a->ndim)];
    const cg_symbolic_dim* db = i < n - b->ndim ? nullptr : b->dims[i - (n - b->ndim)];
    const cg_symbolic_dim* pick;
    if (!da || is_one(da)) pick = db ? db : da;
    else if (!db || is_one(db)) pick = da;
    else if (cg_dim_compatible((cg_symbolic_dim*)da, (cg_symbolic_dim*)db)) pick = da->type == DIM_CONSTANT ? da : db->type == DIM_CONSTANT ? db : da;
    else { for (int k = 0; k < i; ++k) cg_dim_free(out[k]); return fail(CG_ERROR_SHAPE_MISMATCH, (cg_symbolic_shape*)nullptr); }
    out[i] = dim_clone(pick);
  }
  return cg_shape_new(out, n);
}
// [..., M, K] x [..., K, N] -> [..., M, N] with broadcast leading dimensions
CG_EXPORT cg_symbolic_shape* cg_shape_matmul(cg_symbolic_shape* a, cg_symbolic_shape* b) {
  if (!a || !b) return fail(CG_ERROR_NULL_POINTER, (cg_symbolic_shape*)nullptr);
  if (a->ndim < 2 || b->ndim < 2 || !cg_dim_compatible(a->dims[a->ndim - 1], b->dims[b->ndim - 2])) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_symbolic_shape*)nullptr);
  cg_symbolic_shape la = {a->dims, a->ndim - 2, 0}, lb = {b->dims, b->ndim - 2, 0};
  cg_symbolic_shape* lead = cg_shape_broadcast(&la, &lb);
  if (!lead) return nullptr;
  cg_symbolic_dim* out[CG_MAX_DIMS];
  for (int i = 0; i < lead->ndim; ++i) out[i] = lead->dims[i];
  const int n = lead->ndim;
  std::free(lead->dims); std::free(lead);
  out[n] = dim_clone(a->dims[a->ndim - 2]); out[n + 1] = dim_clone(b->dims[b->ndim - 1]);
  return cg_shape_new(out, n + 2);
}
// [N, C, H, W] -> [N, out_channels, (H + 2p - k) / s + 1, (W + 2p - k) / s + 1] for a square kernel;
// a symbolic extent gives an inferred dimension carrying that expression
// (include/cg_symbolic.h:161 in the reference, where it is declared and never defined).
CG_EXPORT cg_symbolic_shape* cg_shape_conv2d(cg_symbolic_shape* in, int out_channels, int kernel_size, int stride, int padding) {
  if (!in) return fail(CG_ERROR_NULL_POINTER, (cg_symbolic_shape*)nullptr);
  if (in->ndim != 4 || out_channels <= 0 || kernel_size <= 0 || stride <= 0 || padding < 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_symbolic_shape*)nullptr);
  auto spatial = [&](cg_symbolic_dim* d) -> cg_symbolic_dim* {
    const int64_t off = 2 * (int64_t)padding - kernel_size;
    if (d->type == DIM_CONSTANT) {
      const int64_t v = d->value + off;
      return v < 0 ? nullptr : cg_dim_const(v / stride + 1);
    }
    cg_symbolic_expr* base = d->expr ? expr_clone(d->expr) : cg_expr_var(d->name ? d->name : "?");
    cg_symbolic_expr* e = cg_expr_add(cg_expr_floordiv(cg_expr_add(base, cg_expr_const(off)), cg_expr_const(stride)), cg_expr_const(1));
    cg_symbolic_dim* out = cg_dim_inferred(e);
    if (out && d->min_value > 0 && d->min_value + off >= 0) out->min_value = (d->min_value + off) / stride + 1;
    if (out && d->max_value > 0 && d->max_value < INT64_MAX / 2 && d->max_value + off >= 0) out->max_value = (d->max_value + off) / stride + 1;
    return out;
  };
  cg_symbolic_dim* out[4] = {dim_clone(in->dims[0]), cg_dim_const(out_channels), spatial(in->dims[2]), spatial(in->dims[3])};
  if (!out[0] || !out[2] || !out[3]) {
    for (cg_symbolic_dim* d : out) if (d) cg_dim_free(d);
    return fail(CG_ERROR_SHAPE_MISMATCH, (cg_symbolic_shape*)nullptr);
  }
  return cg_shape_new(out, 4);
}
CG_EXPORT bool cg_shape_is_dynamic(cg_symbolic_shape* s) {
  if (s) for (int i = 0; i < s->ndim; ++i) if (s->dims[i]->type != DIM_CONSTANT) return true;
  return false;
}
CG_EXPORT bool cg_shape_to_ints(cg_symbolic_shape* s, int* out, int* ndim) {
  if (!s || !out || cg_shape_is_dynamic(s)) return false;
  for (int i = 0; i < s->ndim; ++i) out[i] = (int)s->dims[i]->value;
  if (ndim) *ndim = s->ndim;
  return true;
}
CG_EXPORT bool cg_shape_resolve(cg_symbolic_shape* s, int64_t* vals, const char** names, int n, int* out) {
  if (!s || !out) return false;
  for (int i = 0; i < s->ndim; ++i) { const int64_t v = cg_dim_resolve(s->dims[i], vals, names, n); if (v < 0) return false; out[i] = (int)v; }
  return true;
}
CG_EXPORT void cg_shape_free(cg_symbolic_shape* s) {
  if (!s) return;
  for (int i = 0; i < s->ndim; ++i) cg_dim_free(s->dims[i]);
  std::free(s->dims); std::free(s);
}
CG_EXPORT void cg_shape_print(cg_symbolic_shape* s) {
  if (!s) { std::printf("(null shape)\n"); return; }
  std::printf("[");
  for (int i = 0; i < s->ndim; ++i) {
    const cg_symbolic_dim* d = s->dims[i];
    if (i) std::printf(", ");
    if (d->type == DIM_CONSTANT) std::printf("%lld", (long long)d->value);
    else if (d->type == DIM_INFERRED) { char* t = cg_expr_to_string(d->expr); std::printf("%s", t); std::free(t); }
    else std::printf("%s", d->name ? d->name : "?");
  }
  std::printf("]\n");
}
// Guards: the variable bindings a kernel was specialised for.
static void collect_vars(const cg_symbolic_expr* e, std::vector<std::string>& out) {
  if (!e) return;
  if (e->type == EXPR_VAR) { for (auto& s : out) if (s == e->data.variable) return; out.push_back(e->data.variable); }
  else if (e->type != EXPR_CONST) { collect_vars(e->data.binary.left, out); collect_vars(e->data.binary.right, out); }
}
CG_EXPORT cg_shape_specialization* cg_shape_specialize(cg_symbolic_shape* s, int64_t* vals, const char** names, int n) {
  if (!s) return fail(CG_ERROR_NULL_POINTER, (cg_shape_specialization*)nullptr);
  std::vector<std::string> vars;
  for (int i = 0; i < s->ndim; ++i) {
    const cg_symbolic_dim* d = s->dims[i];
    if (d->type == DIM_SYMBOLIC || d->type == DIM_BROADCAST) { bool have = false; for (auto& v : vars) have = have || v == d->name; if (!have) vars.push_back(d->name); }
    collect_vars(d->expr, vars);
  }
  cg_shape_specialization* sp = (cg_shape_specialization*)std::calloc(1, sizeof(cg_shape_specialization));
  sp->guards = (cg_shape_guard*)std::calloc(vars.size() ? vars.size() : 1, sizeof(cg_shape_guard));
  for (auto& v : vars) {
    bool found = false;
    for (int i = 0; i < n; ++i) if (names[i] && v == names[i]) { sp->guards[sp->num_guards].dim_name = strdup(v.c_str()); sp->guards[sp->num_guards++].expected_value = vals[i]; found = true; break; }
    if (!found) { cg_shape_specialization_free(sp); return fail(CG_ERROR_INVALID_ARGUMENT, (cg_shape_specialization*)nullptr); }
  }
  return sp;
}
CG_EXPORT bool cg_shape_guards_hold(cg_shape_specialization* sp, int64_t* vals, const char** names, int n) {
  if (!sp) return false;
  for (int g = 0; g < sp->num_guards; ++g) {
    bool ok = false;
    for (int i = 0; i < n; ++i) if (names[i] && !std::strcmp(names[i], sp->guards[g].dim_name)) { ok = vals[i] == sp->guards[g].expected_value; break; }
    if (!ok) return false;
  }
  return true;
}
// The reference's name for the same check (include/cg_symbolic.h:200).
CG_EXPORT bool cg_guards_check(cg_shape_specialization* sp, int64_t* vals, const char** names, int n) { return cg_shape_guards_hold(sp, vals, names, n); }
CG_EXPORT void cg_shape_specialization_free(cg_shape_specialization* sp) {
  if (!sp) return;
  for (int i = 0; i < sp->num_guards; ++i) std::free(sp->guards[i].dim_name);
  std::free(sp->guards); std::free(sp);
}
