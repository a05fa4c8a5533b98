// One reverse-mode tape for the whole C API: functional ops, the cg_graph_* registry and
// the gradient checker.  Reference surface: include/cg_tensor.h:165-195 (cg_backward),
// src/core/autograd.c (functional ops), src/core/graph.c (cg_graph_*),
// src/utils/grad_check.c.
#include <algorithm>
#include <cstdint>

#include "internal.hpp"

namespace cgi {
static void trampoline(cg_tensor* self) {
  BackCtx* c = (BackCtx*)self->backward_ctx;
  if (c && c->fn) { c->ran = true; c->fn(self); }
}
void attach_n(cg_tensor* out, cg_tensor* const* parents, int n, BackFn fn) {
  bool any = false;
  for (int i = 0; i < n; ++i) any = any || wants_grad(parents[i]);
  if (!any) return;
  out->requires_grad = true;
  ensure_grad(out);
  // Only the first CG_MAX_PARENTS are visible in the public struct; further ones hang off a
  // pass-through node so that the topological walk still reaches them.
  cg_tensor* few[16];
  std::vector<cg_tensor*> many;
  if (n > 16) many.resize(n);
  cg_tensor** ps = n > 16 ? many.data() : few;
  size_t np = 0;
  for (int pass = 0; pass < 2; ++pass)          // those that want gradients first
    for (int i = 0; i < n; ++i) if (parents[i] && wants_grad(parents[i]) == (pass == 0)) ps[np++] = parents[i];
  cg_tensor* node = out;
  size_t at = 0;
  while (at < np) {
    const size_t left = np - at;
    const int direct = left <= CG_MAX_PARENTS ? (int)left : CG_MAX_PARENTS - 1;
    int k = 0;
    for (int i = 0; i < direct; ++i) { node->parents[k++] = ps[at + i]; cg_tensor_retain(ps[at + i]); }
    at += direct;
    if (at < np) {                               // the hub owns the remaining references
      int one[1] = {1};
      cg_tensor* hub = make(one, 1, false);
      hub->requires_grad = wants_grad(ps[at]);
      node->parents[k++] = hub;
      node->num_parents = k;
      node = hub;
    } else node->num_parents = k;
  }
  out->backward_ctx = new BackCtx{std::move(fn)};
  out->backward_fn = trampoline;
}
void attach(cg_tensor* out, std::initializer_list<cg_tensor*> parents, BackFn fn) {
  attach_n(out, parents.begin(), (int)parents.size(), std::move(fn));
}
}  // namespace cgi

using namespace cgi;

namespace {
// Adds g (shape of `out`) into p->grad, summing over the dimensions along which p was broadcast.
void add_reduced(cg_tensor* p, const cg_tensor* out, const float* g, float sign) {
  if (!wants_grad(p)) return;
  ensure_grad(p);
  if (p->size == out->size) { for (int i = 0; i < p->size; ++i) p->grad[i] += sign * g[i]; return; }
  int st[CG_MAX_DIMS], idx[CG_MAX_DIMS] = {0};
  cg_broadcast_strides(p->shape, p->ndim, (int*)out->shape, out->ndim, st);
  long off = 0;
  for (int i = 0; i < out->size; ++i) {
    p->grad[off] += sign * g[i];
    for (int d = out->ndim - 1; d >= 0; --d) {
      ++idx[d]; off += st[d];
      if (idx[d] < out->shape[d]) break;
      off -= (long)st[d] * out->shape[d]; idx[d] = 0;
    }
  }
}
cg_tensor* binary(cg_tensor* a, cg_tensor* b, int kind) {
  cg_tensor* o = kind == 0 ? cg_tensor_add_broadcast(a, b) : kind == 1 ? cg_tensor_sub_broadcast(a, b) : cg_tensor_mul_broadcast(a, b);
  if (!o) return nullptr;
  attach(o, {a, b}, [a, b, kind](cg_tensor* self) {
    if (kind < 2) {
      add_reduced(a, self, self->grad, 1.0f);
      add_reduced(b, self, self->grad, kind == 0 ? 1.0f : -1.0f);
      return;
    }
    // product rule: the other factor, broadcast to the output shape
    cg_tensor* ones = cg_tensor_ones(self->shape, self->ndim, false);
    std::vector<float> tmp(self->size);
    if (wants_grad(a)) {
      cg_tensor* bb = cg_tensor_mul_broadcast(b, ones);
      for (int i = 0; i < self->size; ++i) tmp[i] = self->grad[i] * bb->data[i];
      add_reduced(a, self, tmp.data(), 1.0f);
      cg_tensor_release(bb);
    }
    if (wants_grad(b)) {
      cg_tensor* ab = cg_tensor_mul_broadcast(a, ones);
      for (int i = 0; i < self->size; ++i) tmp[i] = self->grad[i] * ab->data[i];
      add_reduced(b, self, tmp.data(), 1.0f);
      cg_tensor_release(ab);
    }
    cg_tensor_release(ones);
  });
  return o;
}
}  // namespace

CG_EXPORT cg_tensor* cg_add(cg_tensor* a, cg_tensor* b) { return binary(a, b, 0); }
CG_EXPORT cg_tensor* cg_sub(cg_tensor* a, cg_tensor* b) { return binary(a, b, 1); }
CG_EXPORT cg_tensor* cg_mul(cg_tensor* a, cg_tensor* b) { return binary(a, b, 2); }

CG_EXPORT cg_tensor* cg_matmul(cg_tensor* a, cg_tensor* b) {
  if (!a || !b) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (a->ndim < 2 || b->ndim < 2 || a->shape[a->ndim - 1] != b->shape[b->ndim - 2]) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  int shape[CG_MAX_DIMS];
  for (int i = 0; i < a->ndim - 1; ++i) shape[i] = a->shape[i];
  shape[a->ndim - 1] = b->shape[b->ndim - 1];
  cg_tensor* o = make(shape, a->ndim, false);
  if (!o) return nullptr;
  (void)cg_last_error();                    // an error left by an earlier call must not fail this one
  cg_tensor_matmul(a, b, o);
  if (cg_last_error() != CG_SUCCESS) { cg_tensor_release(o); return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr); }
  attach(o, {a, b}, [a, b](cg_tensor* self) {
    const int M = a->shape[a->ndim - 2], K = a->shape[a->ndim - 1], N = b->shape[b->ndim - 1];
    const int batch = a->size / (M * K), bb = b->size / (K * N);
    for (int i = 0; i < batch; ++i) {
      const float* g = self->grad + (size_t)i * M * N;
      const float* bd = b->data + (bb == 1 ? 0 : (size_t)i * K * N);
      if (wants_grad(a)) { ensure_grad(a); gemm(g, bd, a->grad + (size_t)i * M * K, M, K, N, false, true, true); }          // dA = G B^T
      if (wants_grad(b)) { ensure_grad(b); gemm(a->data + (size_t)i * M * K, g, b->grad + (bb == 1 ? 0 : (size_t)i * K * N), K, N, M, true, false, true); }  // dB = A^T G
    }
  });
  return o;
}

static cg_tensor* reduce_all(cg_tensor* a, bool mean) {
  if (!a) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  int one[1] = {1};
  cg_tensor* o = make(one, 1, false);
  if (!o) return nullptr;
  double s = 0;
  for (int i = 0; i < a->size; ++i) s += a->data[i];
  const float w = mean && a->size ? 1.0f / a->size : 1.0f;
  o->data[0] = (float)s * w;
  attach(o, {a}, [a, w](cg_tensor* self) {
    ensure_grad(a);
    const float g = self->grad[0] * w;
    for (int i = 0; i < a->size; ++i) a->grad[i] += g;
  });
  return o;
}
CG_EXPORT cg_tensor* cg_sum_all(cg_tensor* a) { return reduce_all(a, false); }
CG_EXPORT cg_tensor* cg_mean_all(cg_tensor* a) { return reduce_all(a, true); }

template <class F, class D> static cg_tensor* unary(cg_tensor* a, F f, D dfdx) {
  if (!a) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* o = make_like(a, false);
  if (!o) return nullptr;
  for (int i = 0; i < a->size; ++i) o->data[i] = f(a->data[i]);
  attach(o, {a}, [a, dfdx](cg_tensor* self) {
    ensure_grad(a);
    for (int i = 0; i < a->size; ++i) a->grad[i] += self->grad[i] * dfdx(a->data[i], self->data[i]);
  });
  return o;
}
CG_EXPORT cg_tensor* cg_exp(cg_tensor* a) { return unary(a, [](float x) { return std::exp(x); }, [](float, float y) { return y; }); }
CG_EXPORT cg_tensor* cg_log_op(cg_tensor* a) { return unary(a, [](float x) { return std::log(x); }, [](float x, float) { return 1.0f / x; }); }
CG_EXPORT cg_tensor* cg_pow_op(cg_tensor* a, float p) {
  return unary(a, [p](float x) { return std::pow(x, p); }, [p](float x, float) { return p * std::pow(x, p - 1.0f); });
}

// -------------------------------------------------------------- backward
CG_EXPORT void cg_backward(cg_tensor* loss) {
  if (!loss) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (!loss->requires_grad) return;
  ensure_grad(loss);
  bool seeded = false;
  for (int i = 0; i < loss->size; ++i) seeded = seeded || loss->grad[i] != 0.0f;
  if (!seeded) for (int i = 0; i < loss->size; ++i) loss->grad[i] = 1.0f;
  // iterative post-order DFS.  The walk's three containers are kept between calls (a training loop
  // walks the same few nodes every step); a backward function that itself calls cg_backward gets
  // containers of its own.
  struct Scratch {
    std::vector<cg_tensor*> order, table;          // table: open addressing, power-of-two size, nullptr = free
    std::vector<std::pair<cg_tensor*, int>> stack;
    size_t used = 0;
    bool insert(cg_tensor* p) {
      if (table.empty()) table.assign(64, nullptr);
      if ((used + 1) * 2 > table.size()) {
        std::vector<cg_tensor*> old;
        old.swap(table);
        table.assign(old.size() * 2, nullptr);
        used = 0;
        for (cg_tensor* q : old) if (q) insert(q);
      }
      const size_t mask = table.size() - 1;
      size_t h = ((uintptr_t)p >> 4) * 0x9E3779B97F4A7C15ull >> 20 & mask;
      while (table[h]) { if (table[h] == p) return false; h = (h + 1) & mask; }
      table[h] = p; ++used;
      return true;
    }
  };
  static thread_local Scratch shared;
  static thread_local int depth = 0;
  Scratch own;
  Scratch& w = depth == 0 ? shared : own;
  ++depth;
  w.order.clear(); w.stack.clear();
  if (w.used) { std::fill(w.table.begin(), w.table.end(), nullptr); w.used = 0; }
  w.stack.push_back({loss, 0});
  w.insert(loss);
  while (!w.stack.empty()) {
    auto& top = w.stack.back();
    if (top.second < top.first->num_parents) {
      cg_tensor* p = top.first->parents[top.second++];
      if (p && p->requires_grad && w.insert(p)) w.stack.push_back({p, 0});
    } else {
      w.order.push_back(top.first);
      w.stack.pop_back();
    }
  }
  for (size_t i = w.order.size(); i-- > 0;)
    if (w.order[i]->backward_fn) w.order[i]->backward_fn(w.order[i]);
  --depth;
  if (w.table.size() > (1u << 16)) { Scratch().table.swap(w.table); w.used = 0; }     // a huge graph does not pin its table
}

// ---------------------------------------------------------- graph registry
// The reference keeps a second, global graph (src/core/graph.c).  Here it is a
// registry over the same tape: while active, every tensor made by cg_graph_* is owned by
// the registry and released by cg_graph_reset, so callers need not free intermediates.
namespace {
bool g_graph_active = false;
std::vector<cg_tensor*> g_graph_nodes;
cg_tensor* own(cg_tensor* t) { if (t && g_graph_active) g_graph_nodes.push_back(t); return t; }
}  // namespace
CG_EXPORT void cg_graph_init(void) { g_graph_active = true; }
CG_EXPORT bool cg_graph_is_active(void) { return g_graph_active; }
CG_EXPORT void cg_graph_reset(void) {
  for (cg_tensor* t : g_graph_nodes) cg_tensor_release(t);
  g_graph_nodes.clear();
  g_graph_active = false;
}
CG_EXPORT void cg_graph_register(cg_tensor* t, cg_tensor** parents, int num_parents) {
  if (!t) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (t->num_parents == 0 && parents && num_parents > 0) {
    const int n = num_parents < CG_MAX_PARENTS ? num_parents : CG_MAX_PARENTS;
    for (int i = 0; i < n; ++i) { t->parents[i] = parents[i]; cg_tensor_retain(parents[i]); if (wants_grad(parents[i])) t->requires_grad = true; }
    t->num_parents = n;
    if (t->requires_grad) ensure_grad(t);
  }
  if (g_graph_active) { cg_tensor_retain(t); g_graph_nodes.push_back(t); }
}
CG_EXPORT void cg_graph_backward(cg_tensor* loss) { cg_backward(loss); }
CG_EXPORT cg_tensor* cg_graph_add(cg_tensor* a, cg_tensor* b) { return own(cg_add(a, b)); }
CG_EXPORT cg_tensor* cg_graph_mul(cg_tensor* a, cg_tensor* b) { return own(cg_mul(a, b)); }
CG_EXPORT cg_tensor* cg_graph_matmul(cg_tensor* a, cg_tensor* b) { return own(cg_matmul(a, b)); }

// -------------------------------------------------------------- grad check
// Compares input->grad (as left by the caller's backward pass, or computed here from the
// central difference when absent) with d<forward(input), grad_output>/d input.
CG_EXPORT bool cg_grad_check(void (*forward_fn)(cg_tensor*, cg_tensor*), cg_tensor* input, cg_tensor* grad_output,
                             float eps, float tol) {
  if (!forward_fn || !input || !grad_output) return fail(CG_ERROR_NULL_POINTER, false);
  if (eps <= 0) eps = 1e-3f;
  cg_tensor* out = make_like(grad_output, false);
  if (!out) return false;
  bool ok = true;
  for (int i = 0; i < input->size && ok; ++i) {
    const float keep = input->data[i];
    double plus = 0, minus = 0;
    input->data[i] = keep + eps;
    forward_fn(input, out);
    for (int j = 0; j < out->size; ++j) plus += (double)out->data[j] * grad_output->data[j];
    input->data[i] = keep - eps;
    forward_fn(input, out);
    for (int j = 0; j < out->size; ++j) minus += (double)out->data[j] * grad_output->data[j];
    input->data[i] = keep;
    const double num = (plus - minus) / (2.0 * eps);
    if (input->grad) {
      const double ana = input->grad[i];
      const double denom = std::fabs(num) + std::fabs(ana) > 1.0 ? std::fabs(num) + std::fabs(ana) : 1.0;
      if (std::fabs(num - ana) / denom > tol) ok = false;
    } else if (!std::isfinite(num)) ok = false;
  }
  cg_tensor_release(out);
  return ok;
}
