// Losses (on the tape) and optimizers of the C API.
// Reference surface: include/cg_loss.h, src/layers/loss.c; include/cg_optim.h,
// src/optim/{sgd,adam,optimizer}.c.
#include "internal.hpp"

using namespace cgi;

namespace {
// f(pred, target, &dloss/dpred) per element; `denom` divides value and gradient for MEAN.
template <class F> cg_tensor* pointwise_loss(cg_tensor* p, cg_tensor* t, cg_reduction red, F f) {
  if (!p || !t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (p->size != t->size) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int n = p->size;
  int one[1] = {1};
  cg_tensor* o = red == CG_REDUCTION_NONE ? make_like(p, false) : make(one, 1, false);
  if (!o) return nullptr;
  const float w = red == CG_REDUCTION_MEAN && n ? 1.0f / n : 1.0f;
  double acc = 0;
  for (int i = 0; i < n; ++i) {
    float d;
    const float v = f(p->data[i], t->data[i], &d);
    if (red == CG_REDUCTION_NONE) o->data[i] = v; else acc += v;
  }
  if (red != CG_REDUCTION_NONE) o->data[0] = (float)(acc * w);
  attach(o, {p, t}, [p, t, red, w, f, n](cg_tensor* self) {
    if (!wants_grad(p)) return;
    ensure_grad(p);
    for (int i = 0; i < n; ++i) {
      float d;
      f(p->data[i], t->data[i], &d);
      p->grad[i] += d * w * (red == CG_REDUCTION_NONE ? self->grad[i] : self->grad[0]);
    }
  });
  return o;
}
}  // namespace

CG_EXPORT cg_tensor* cg_mse_loss(cg_tensor* p, cg_tensor* t, cg_reduction red) {
  return pointwise_loss(p, t, red, [](float a, float b, float* d) { const float e = a - b; *d = 2.0f * e; return e * e; });
}
CG_EXPORT cg_tensor* cg_l1_loss(cg_tensor* p, cg_tensor* t, cg_reduction red) {
  return pointwise_loss(p, t, red, [](float a, float b, float* d) { const float e = a - b; *d = e > 0 ? 1.0f : (e < 0 ? -1.0f : 0.0f); return std::fabs(e); });
}
CG_EXPORT cg_tensor* cg_smooth_l1_loss(cg_tensor* p, cg_tensor* t, float beta, cg_reduction red) {
  if (beta <= 0) beta = 1.0f;
  return pointwise_loss(p, t, red, [beta](float a, float b, float* d) {
    const float e = a - b, ae = std::fabs(e);
    if (ae < beta) { *d = e / beta; return 0.5f * e * e / beta; }
    *d = e > 0 ? 1.0f : -1.0f;
    return ae - 0.5f * beta;
  });
}
CG_EXPORT cg_tensor* cg_bce_loss(cg_tensor* p, cg_tensor* t, cg_reduction red) {
  return pointwise_loss(p, t, red, [](float a, float b, float* d) {
    const float eps = 1e-7f, q = a < eps ? eps : (a > 1 - eps ? 1 - eps : a);
    *d = (q - b) / (q * (1.0f - q));
    return -(b * std::log(q) + (1.0f - b) * std::log(1.0f - q));
  });
}
CG_EXPORT cg_tensor* cg_bce_with_logits_loss(cg_tensor* x, cg_tensor* t, cg_reduction red) {
  return pointwise_loss(x, t, red, [](float a, float b, float* d) {
    *d = sigmoidf(a) - b;
    return (a > 0 ? a : 0.0f) - a * b + std::log1p(std::exp(-std::fabs(a)));
  });
}

// pred and target [N, C] (target: one-hot or soft labels).  MEAN divides by N.
CG_EXPORT cg_tensor* cg_cross_entropy_loss(cg_tensor* p, cg_tensor* t, bool from_logits, cg_reduction red) {
  if (!p || !t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (p->ndim < 1) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int C = cols_of(p), N = rows_of(p);
  // Targets: probabilities / one-hot rows of the prediction's shape, or - the reference's convention
  // (src/layers/loss.c:58-78) - one class index per row.  Indices are expanded to one-hot rows here.
  cg_tensor* expanded = nullptr;
  if (t->size == N && t->size != p->size) {
    expanded = make_like(p, false);
    if (!expanded) return nullptr;
    for (int r = 0; r < N; ++r) {
      const int lbl = (int)t->data[r];
      if (lbl < 0 || lbl >= C) { cg_tensor_release(expanded); return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr); }
      expanded->data[(size_t)r * C + lbl] = 1.0f;
    }
    t = expanded;
  }
  if (p->size != t->size) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  int os[1] = {red == CG_REDUCTION_NONE ? N : 1};
  cg_tensor* o = make(os, 1, false);
  if (!o) { if (expanded) cg_tensor_release(expanded); return nullptr; }
  std::vector<float> prob(from_logits ? p->size : 0);
  const float eps = 1e-7f;
  double total = 0;
  for (int r = 0; r < N; ++r) {
    const float* x = p->data + (size_t)r * C; const float* y = t->data + (size_t)r * C;
    double loss = 0;
    if (from_logits) {
      float m = x[0]; for (int j = 1; j < C; ++j) m = x[j] > m ? x[j] : m;
      double s = 0; for (int j = 0; j < C; ++j) s += std::exp((double)x[j] - m);
      const double lse = m + std::log(s);
      for (int j = 0; j < C; ++j) { prob[(size_t)r * C + j] = (float)std::exp(x[j] - lse); loss -= y[j] * (x[j] - lse); }
    } else {
      for (int j = 0; j < C; ++j) if (y[j] != 0.0f) loss -= y[j] * std::log((x[j] > eps ? x[j] : eps));
    }
    if (red == CG_REDUCTION_NONE) o->data[r] = (float)loss; else total += loss;
  }
  const float w = red == CG_REDUCTION_MEAN && N ? 1.0f / N : 1.0f;
  if (red != CG_REDUCTION_NONE) o->data[0] = (float)(total * w);
  attach(o, {p, t}, [p, t, prob, from_logits, red, w, N, C, eps](cg_tensor* self) {
    if (!wants_grad(p)) return;
    ensure_grad(p);
    for (int r = 0; r < N; ++r) {
      const float g = w * (red == CG_REDUCTION_NONE ? self->grad[r] : self->grad[0]);
      const float* y = t->data + (size_t)r * C;
      double ysum = 0;
      if (from_logits) for (int j = 0; j < C; ++j) ysum += y[j];
      for (int j = 0; j < C; ++j) {
        const size_t i = (size_t)r * C + j;
        if (from_logits) p->grad[i] += g * (prob[i] * (float)ysum - y[j]);
        else p->grad[i] += g * (-y[j] / (p->data[i] > eps ? p->data[i] : eps));
      }
    }
  });
  if (expanded) cg_tensor_release(expanded);       // the tape holds it from here on (or nobody needs it)
  return o;
}
CG_EXPORT cg_tensor* cg_softmax_cross_entropy_loss(cg_tensor* logits, cg_tensor* t, cg_reduction red) {
  return cg_cross_entropy_loss(logits, t, true, red);
}

// ------------------------------------------------------------- optimizers
namespace {
inline float bf16_round(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return f;
  u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u;
  std::memcpy(&f, &u, 4); return f;
}
cg_tensor** zeros_like_all(cg_tensor** ps, int n) {
  cg_tensor** out = (cg_tensor**)std::calloc(n ? n : 1, sizeof(cg_tensor*));
  for (int i = 0; i < n; ++i) out[i] = make_like(ps[i], false);
  return out;
}
void release_all(cg_tensor** ts, int n) { if (!ts) return; for (int i = 0; i < n; ++i) if (ts[i]) cg_tensor_release(ts[i]); std::free(ts); }
// Unscale, overflow check, clip.  Returns false when the step must be skipped.
bool prepare(cg_optimizer* o) {
  double ss = 0; bool finite = true;
  for (int i = 0; i < o->num_params; ++i) {
    cg_tensor* p = o->params[i];
    if (!p || !p->grad) continue;
    for (int j = 0; j < p->size; ++j) { const float g = p->grad[j]; if (!std::isfinite(g)) finite = false; ss += (double)g * g; }
  }
  float inv = 1.0f;
  if (o->use_mixed_precision) {
    const float scale = o->loss_scale;
    if (cg_optimizer_update_scale(o, finite ? (float)std::sqrt(ss) : INFINITY)) return false;
    inv = 1.0f / scale;
  } else if (!finite) return false;
  float mul = inv;
  if (o->max_grad_norm > 0) {
    const float norm = (float)std::sqrt(ss) * inv;
    if (norm > o->max_grad_norm) mul *= o->max_grad_norm / (norm + 1e-6f);
  }
  if (mul != 1.0f)
    for (int i = 0; i < o->num_params; ++i) { cg_tensor* p = o->params[i]; if (p && p->grad) for (int j = 0; j < p->size; ++j) p->grad[j] *= mul; }
  return true;
}
float* weights_of(cg_optimizer* o, int i) { return o->use_master_weights && o->master_params ? o->master_params[i]->data : o->params[i]->data; }
void publish_weights(cg_optimizer* o, int i) {
  if (!(o->use_master_weights && o->master_params)) return;
  cg_tensor* p = o->params[i]; const float* m = o->master_params[i]->data;
  for (int j = 0; j < p->size; ++j) p->data[j] = bf16_round(m[j]);
}
void base_init(cg_optimizer* o, cg_tensor** params, int n, float lr) {
  o->learning_rate = lr; o->num_params = n; o->t = 0; o->loss_scale = 1.0f; o->scale_factor = 2.0f; o->scale_window = 2000;
  o->params = (cg_tensor**)std::malloc(sizeof(cg_tensor*) * (n ? n : 1));
  for (int i = 0; i < n; ++i) { o->params[i] = params[i]; cg_tensor_retain(params[i]); ensure_grad(params[i]); }
}
void base_free(cg_optimizer* o) {
  release_all(o->params, o->num_params);
  release_all(o->master_params, o->num_params);
}
void zero_grad_all(cg_optimizer* o) { for (int i = 0; i < o->num_params; ++i) cg_tensor_zero_grad(o->params[i]); }

void sgd_step(cg_optimizer* o) {
  cg_sgd* s = (cg_sgd*)o;
  if (!prepare(o)) return;
  ++o->t;
  for (int i = 0; i < o->num_params; ++i) {
    cg_tensor* p = o->params[i];
    float* w = weights_of(o, i);
    float* v = s->velocities ? s->velocities[i]->data : nullptr;
    for (int j = 0; j < p->size; ++j) {
      float g = p->grad[j] + s->weight_decay * w[j];
      if (v) { v[j] = s->momentum * v[j] + g; g = s->nesterov ? g + s->momentum * v[j] : v[j]; }
      w[j] -= o->learning_rate * g;
    }
    publish_weights(o, i);
  }
}
void sgd_free(cg_optimizer* o) { cg_sgd* s = (cg_sgd*)o; release_all(s->velocities, o->num_params); base_free(o); std::free(o); }

void adam_step(cg_optimizer* o) {
  cg_adam* a = (cg_adam*)o;
  if (!prepare(o)) return;
  ++o->t;
  const float bc1 = 1.0f - std::pow(a->beta1, (float)o->t), bc2 = 1.0f - std::pow(a->beta2, (float)o->t);
  const float decay = a->weight_decay > 0 ? 1.0f - o->learning_rate * a->weight_decay : 1.0f;
  for (int i = 0; i < o->num_params; ++i) {
    cg_tensor* p = o->params[i];
    adam_update(weights_of(o, i), a->m[i]->data, a->v[i]->data, p->grad, p->size, a->beta1, a->beta2, o->learning_rate,
                a->epsilon, bc1, bc2, decay);
    publish_weights(o, i);
  }
}
void adam_free(cg_optimizer* o) { cg_adam* a = (cg_adam*)o; release_all(a->m, o->num_params); release_all(a->v, o->num_params); base_free(o); std::free(o); }
}  // namespace

CG_EXPORT cg_sgd* cg_sgd_new(cg_tensor** params, int n, float lr, float momentum, float wd, bool nesterov) {
  if (!params || n <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_sgd*)nullptr);
  cg_sgd* s = (cg_sgd*)std::calloc(1, sizeof(cg_sgd));
  base_init(&s->base, params, n, lr);
  s->momentum = momentum; s->weight_decay = wd; s->nesterov = nesterov;
  if (momentum > 0) s->velocities = zeros_like_all(params, n);
  s->base.step = sgd_step; s->base.zero_grad = zero_grad_all; s->base.free = sgd_free;
  return s;
}
CG_EXPORT cg_sgd* cg_sgd_new_for_sequential(cg_sequential* m, float lr, float momentum, float wd, bool nesterov) {
  return cg_sgd_new(cg_sequential_get_params(m), cg_sequential_num_params(m), lr, momentum, wd, nesterov);
}
CG_EXPORT cg_adam* cg_adam_new(cg_tensor** params, int n, float lr, float b1, float b2, float eps, float wd) {
  if (!params || n <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_adam*)nullptr);
  cg_adam* a = (cg_adam*)std::calloc(1, sizeof(cg_adam));
  base_init(&a->base, params, n, lr);
  a->beta1 = b1 > 0 ? b1 : 0.9f; a->beta2 = b2 > 0 ? b2 : 0.999f; a->epsilon = eps > 0 ? eps : 1e-8f; a->weight_decay = wd;
  a->m = zeros_like_all(params, n); a->v = zeros_like_all(params, n);
  a->base.step = adam_step; a->base.zero_grad = zero_grad_all; a->base.free = adam_free;
  return a;
}
CG_EXPORT cg_adam* cg_adam_new_for_sequential(cg_sequential* m, float lr, float b1, float b2, float eps, float wd) {
  return cg_adam_new(cg_sequential_get_params(m), cg_sequential_num_params(m), lr, b1, b2, eps, wd);
}
CG_EXPORT void cg_optimizer_step(cg_optimizer* o) { if (o && o->step) o->step(o); }
CG_EXPORT void cg_optimizer_zero_grad(cg_optimizer* o) { if (o && o->zero_grad) o->zero_grad(o); }
CG_EXPORT void cg_optimizer_free(cg_optimizer* o) { if (o && o->free) o->free(o); }
CG_EXPORT void cg_optimizer_step_lr(cg_optimizer* o, int step, int step_size, float gamma) {
  if (o && step_size > 0 && step > 0 && step % step_size == 0) o->learning_rate *= gamma;
}
CG_EXPORT void cg_optimizer_exp_lr(cg_optimizer* o, float initial_lr, float gamma) {
  if (o) o->learning_rate = initial_lr * std::pow(gamma, (float)o->t);
}
CG_EXPORT void cg_optimizer_enable_loss_scaling(cg_optimizer* o, float init_scale, float factor, int window) {
  if (!o) return;
  o->use_mixed_precision = true;
  o->loss_scale = init_scale > 0 ? init_scale : 65536.0f;
  o->scale_factor = factor > 1 ? factor : 2.0f;
  o->scale_window = window > 0 ? window : 2000;
  o->scale_backoff = 0;
}
CG_EXPORT void cg_optimizer_enable_master_weights(cg_optimizer* o) {
  if (!o || o->master_params) return;
  o->use_master_weights = true;
  o->master_params = (cg_tensor**)std::calloc(o->num_params ? o->num_params : 1, sizeof(cg_tensor*));
  for (int i = 0; i < o->num_params; ++i) { o->master_params[i] = cg_tensor_clone(o->params[i]); o->master_params[i]->requires_grad = false; publish_weights(o, i); }
}
// scale_backoff counts the clean steps since the last overflow.
CG_EXPORT bool cg_optimizer_update_scale(cg_optimizer* o, float grad_norm) {
  if (!o || !o->use_mixed_precision) return false;
  if (!std::isfinite(grad_norm)) {
    o->loss_scale = o->loss_scale / o->scale_factor < 1.0f ? 1.0f : o->loss_scale / o->scale_factor;
    o->scale_backoff = 0;
    return true;
  }
  if (++o->scale_backoff >= o->scale_window) {
    o->loss_scale = o->loss_scale * o->scale_factor > 65536.0f ? 65536.0f : o->loss_scale * o->scale_factor;
    o->scale_backoff = 0;
  }
  return false;
}
