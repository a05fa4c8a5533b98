// Layers of the C API.  Every forward records itself on the tape (parents: input,
// weights, bias), so cg_backward(loss) reaches every parameter; the per-layer
// backward(self, grad_output) entry point runs the same closure for one layer.
// Reference surface: include/cg_layers.h; src/layers/{linear,activations,dropout,
// batchnorm,normalization,conv2d,sequential}.c.
#include "internal.hpp"

using namespace cgi;

namespace {
template <class T> T* new_layer(const char* name) {
  T* l = (T*)std::calloc(1, sizeof(T));
  if (!l) return fail(CG_ERROR_OUT_OF_MEMORY, (T*)nullptr);
  l->base.name = name;
  return l;
}
// Takes ownership of `out`; keeps `in` alive for the per-layer backward.
// The reference's ownership rule (src/layers/linear.c:60-97): the layer keeps a reference to its input and one to
// its output, and the output's first reference goes to the caller, who releases it when done.
cg_tensor* publish(cg_layer* L, cg_tensor* in, cg_tensor* out) {
  if (in) cg_tensor_retain(in);
  if (out) cg_tensor_retain(out);
  if (L->input) cg_tensor_release(L->input);
  if (L->output) cg_tensor_release(L->output);
  L->input = in; L->output = out;
  return out;
}
void base_free(cg_layer* L) {
  if (L->input) cg_tensor_release(L->input);
  if (L->output) cg_tensor_release(L->output);
  if (L->weights) cg_tensor_release(L->weights);
  if (L->bias) cg_tensor_release(L->bias);
}
void plain_free(cg_layer* L) { base_free(L); std::free(L); }
int zero_params(cg_layer*) { return 0; }
cg_tensor** no_params(cg_layer*) { return nullptr; }
const float* upstream(cg_tensor* g) { return g->grad ? g->grad : g->data; }
// Shared per-layer backward: seed output->grad from grad_output and run the node's closure.
void layer_backward(cg_layer* L, cg_tensor* grad_output) {
  if (!L || !L->output || !grad_output) { set_error(CG_ERROR_NULL_POINTER); return; }
  cg_tensor* o = L->output;
  if (!o->backward_fn || tape_ran(o)) return;
  if (grad_output->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (grad_output != o || !o->grad) { ensure_grad(o); std::memcpy(o->grad, upstream(grad_output), sizeof(float) * o->size); }
  if (L->input && !L->input->grad) ensure_grad(L->input);      // lets a chain of manual backward calls read input->grad
  o->backward_fn(o);
}
void finish(cg_layer* L, cg_tensor* (*fwd)(cg_layer*, cg_tensor*), void (*fr)(cg_layer*), int (*np)(cg_layer*), cg_tensor** (*gp)(cg_layer*)) {
  L->forward = fwd; L->backward = layer_backward; L->free = fr; L->num_params = np; L->get_params = gp;
}
// An input that nobody asked gradients for still gets one when a manual backward chain needs it.
bool in_grad(cg_tensor* in) { return in->grad != nullptr; }
}  // namespace

CG_EXPORT void cg_layer_free(cg_layer* l) { if (l && l->free) l->free(l); }
CG_EXPORT void cg_layer_zero_grad(cg_layer* l) {
  if (!l) return;
  const int n = l->num_params ? l->num_params(l) : 0;
  cg_tensor** p = n ? l->get_params(l) : nullptr;
  for (int i = 0; i < n; ++i) cg_tensor_zero_grad(p[i]);
}

// ------------------------------------------------------------------ linear
static cg_tensor* linear_forward(cg_layer* L, cg_tensor* x) {
  cg_linear* l = (cg_linear*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  const int in = l->in_features, out = l->out_features;
  if (x->ndim < 1 || cols_of(x) != in) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  int shape[CG_MAX_DIMS];
  for (int i = 0; i < x->ndim; ++i) shape[i] = x->shape[i];
  shape[x->ndim - 1] = out;
  cg_tensor* y = make(shape, x->ndim, false);
  if (!y) return nullptr;
  const int rows = rows_of(x);
  cg_tensor* W = L->weights; cg_tensor* b = L->bias;
  gemm(x->data, W->data, y->data, rows, out, in, false, false, false);
  if (b) for (int r = 0; r < rows; ++r) for (int j = 0; j < out; ++j) y->data[(size_t)r * out + j] += b->data[j];
  attach(y, {x, W, b}, [x, W, b, rows, in, out](cg_tensor* self) {
    const float* g = self->grad;
    gemm(x->data, g, W->grad, in, out, rows, true, false, true);                        // dW += X^T G
    if (b) for (int r = 0; r < rows; ++r) for (int j = 0; j < out; ++j) b->grad[j] += g[(size_t)r * out + j];
    if (in_grad(x)) gemm(g, W->data, x->grad, rows, in, out, false, true, true);        // dX += G W^T
  });
  return publish(L, x, y);
}
static int linear_np(cg_layer* L) { return L->bias ? 2 : 1; }
static cg_tensor** linear_gp(cg_layer* L) { return ((cg_linear*)L)->param_ptrs; }
CG_EXPORT cg_linear* cg_linear_new(int in, int out, bool bias) {
  if (in <= 0 || out <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_linear*)nullptr);
  cg_linear* l = new_layer<cg_linear>("Linear");
  if (!l) return nullptr;
  l->in_features = in; l->out_features = out;
  int ws[2] = {in, out};
  l->base.weights = make(ws, 2, true);
  Rng rng(next_layer_seed());
  const float limit = std::sqrt(6.0f / (in + out));            // Xavier uniform
  for (int i = 0; i < in * out; ++i) l->base.weights->data[i] = (2.0f * rng.uniform() - 1.0f) * limit;
  if (bias) { int bs[1] = {out}; l->base.bias = make(bs, 1, true); }
  l->param_ptrs[0] = l->base.weights; l->param_ptrs[1] = l->base.bias;
  finish(&l->base, linear_forward, plain_free, linear_np, linear_gp);
  return l;
}

// ------------------------------------------------------------- activations
template <class F, class D> static cg_tensor* act_forward(cg_layer* L, cg_tensor* x, F f, D d) {
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* y = make_like(x, false);
  if (!y) return nullptr;
  for (int i = 0; i < x->size; ++i) y->data[i] = f(x->data[i]);
  attach(y, {x}, [x, d](cg_tensor* self) {
    if (!in_grad(x)) return;
    for (int i = 0; i < x->size; ++i) x->grad[i] += self->grad[i] * d(x->data[i], self->data[i]);
  });
  return publish(L, x, y);
}
static cg_tensor* relu_forward(cg_layer* L, cg_tensor* x) {
  return act_forward(L, x, [](float v) { return v > 0 ? v : 0.0f; }, [](float v, float) { return v > 0 ? 1.0f : 0.0f; });
}
static cg_tensor* sigmoid_forward(cg_layer* L, cg_tensor* x) {
  return act_forward(L, x, [](float v) { return sigmoidf(v); }, [](float, float y) { return y * (1.0f - y); });
}
static cg_tensor* tanh_forward(cg_layer* L, cg_tensor* x) {
  return act_forward(L, x, [](float v) { return std::tanh(v); }, [](float, float y) { return 1.0f - y * y; });
}
CG_EXPORT cg_relu* cg_relu_new(void) { auto* l = new_layer<cg_relu>("ReLU"); if (l) finish(&l->base, relu_forward, plain_free, zero_params, no_params); return l; }
CG_EXPORT cg_sigmoid* cg_sigmoid_new(void) { auto* l = new_layer<cg_sigmoid>("Sigmoid"); if (l) finish(&l->base, sigmoid_forward, plain_free, zero_params, no_params); return l; }
CG_EXPORT cg_tanh_layer* cg_tanh_new(void) { auto* l = new_layer<cg_tanh_layer>("Tanh"); if (l) finish(&l->base, tanh_forward, plain_free, zero_params, no_params); return l; }

static cg_tensor* softmax_forward(cg_layer* L, cg_tensor* x) {
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* y = make_like(x, false);
  if (!y) return nullptr;
  const int C = cols_of(x), R = rows_of(x);
  for (int r = 0; r < R; ++r) {
    const float* p = x->data + (size_t)r * C; float* q = y->data + (size_t)r * C;
    float m = p[0]; for (int j = 1; j < C; ++j) m = p[j] > m ? p[j] : m;
    double s = 0; for (int j = 0; j < C; ++j) { q[j] = std::exp(p[j] - m); s += q[j]; }
    const float inv = (float)(1.0 / s); for (int j = 0; j < C; ++j) q[j] *= inv;
  }
  attach(y, {x}, [x, R, C](cg_tensor* self) {
    if (!in_grad(x)) return;
    for (int r = 0; r < R; ++r) {
      const float* yv = self->data + (size_t)r * C; const float* g = self->grad + (size_t)r * C;
      double dot = 0; for (int j = 0; j < C; ++j) dot += (double)g[j] * yv[j];
      for (int j = 0; j < C; ++j) x->grad[(size_t)r * C + j] += yv[j] * (g[j] - (float)dot);
    }
  });
  return publish(L, x, y);
}
CG_EXPORT cg_softmax* cg_softmax_new(void) { auto* l = new_layer<cg_softmax>("Softmax"); if (l) finish(&l->base, softmax_forward, plain_free, zero_params, no_params); return l; }

// ----------------------------------------------------------------- dropout
static cg_tensor* dropout_forward(cg_layer* L, cg_tensor* x) {
  cg_dropout* l = (cg_dropout*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* y = make_like(x, false);
  if (!y) return nullptr;
  if (!l->training || l->p <= 0.0f) {
    std::memcpy(y->data, x->data, sizeof(float) * x->size);
    attach(y, {x}, [x](cg_tensor* self) { if (in_grad(x)) for (int i = 0; i < x->size; ++i) x->grad[i] += self->grad[i]; });
    return publish(L, x, y);
  }
  if (l->mask) cg_tensor_release(l->mask);
  cg_tensor* mask = l->mask = make_like(x, false);
  static thread_local Rng rng(next_layer_seed());
  const float keep = 1.0f - l->p, scale = keep > 0 ? 1.0f / keep : 0.0f;
  for (int i = 0; i < x->size; ++i) { mask->data[i] = rng.uniform() < keep ? scale : 0.0f; y->data[i] = x->data[i] * mask->data[i]; }
  cg_tensor_retain(mask);
  attach(y, {x, mask}, [x, mask](cg_tensor* self) {
    if (in_grad(x)) for (int i = 0; i < x->size; ++i) x->grad[i] += self->grad[i] * mask->data[i];
  });
  cg_tensor_release(mask);
  return publish(L, x, y);
}
static void dropout_free(cg_layer* L) { cg_dropout* l = (cg_dropout*)L; if (l->mask) cg_tensor_release(l->mask); plain_free(L); }
CG_EXPORT cg_dropout* cg_dropout_new(float p) {
  if (p < 0.0f || p >= 1.0f) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_dropout*)nullptr);
  auto* l = new_layer<cg_dropout>("Dropout");
  if (!l) return nullptr;
  l->p = p; l->training = true;
  finish(&l->base, dropout_forward, dropout_free, zero_params, no_params);
  return l;
}
CG_EXPORT void cg_dropout_set_training(cg_dropout* l, bool t) { if (l) l->training = t; }

// --------------------------------------------------------------- batchnorm
// Input [N, F] or [N, C, H, W] (statistics per feature / channel).
static cg_tensor* batchnorm_forward(cg_layer* L, cg_tensor* x) {
  cg_batchnorm* l = (cg_batchnorm*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  const int F = l->num_features;
  if (x->ndim < 2 || x->shape[1] != F) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int N = x->shape[0], S = x->size / (N * F);        // spatial size
  const int cnt = N * S;
  cg_tensor* y = make_like(x, false);
  if (!y) return nullptr;
  cg_tensor* gamma = L->weights; cg_tensor* beta = L->bias;
  if (l->x_norm) cg_tensor_release(l->x_norm);
  if (l->std_inv) cg_tensor_release(l->std_inv);
  cg_tensor* xn = l->x_norm = make_like(x, false);
  int fs[1] = {F};
  cg_tensor* si = l->std_inv = make(fs, 1, false);
  if (!l->batch_mean) { l->batch_mean = make(fs, 1, false); l->batch_var = make(fs, 1, false); }
  auto at = [=](int n, int f, int s) { return ((size_t)n * F + f) * S + s; };
  for (int f = 0; f < F; ++f) {
    float mean, var;
    if (l->training) {
      double m = 0, v = 0;
      for (int n = 0; n < N; ++n) for (int s = 0; s < S; ++s) m += x->data[at(n, f, s)];
      m /= cnt;
      for (int n = 0; n < N; ++n) for (int s = 0; s < S; ++s) { const double d = x->data[at(n, f, s)] - m; v += d * d; }
      v /= cnt;
      mean = (float)m; var = (float)v;
      l->running_mean->data[f] = l->momentum * l->running_mean->data[f] + (1 - l->momentum) * mean;   // the reference's rule
      l->running_var->data[f] = l->momentum * l->running_var->data[f] + (1 - l->momentum) * var;
    } else { mean = l->running_mean->data[f]; var = l->running_var->data[f]; }
    const float inv = 1.0f / std::sqrt(var + l->epsilon);
    si->data[f] = inv;
    l->batch_mean->data[f] = mean; l->batch_var->data[f] = var;        // the statistics this pass normalised with
    for (int n = 0; n < N; ++n) for (int s = 0; s < S; ++s) {
      const size_t i = at(n, f, s);
      xn->data[i] = (x->data[i] - mean) * inv;
      y->data[i] = xn->data[i] * gamma->data[f] + beta->data[f];
    }
  }
  const bool training = l->training;
  const std::vector<float> inv_std(si->data, si->data + F);
  attach(y, {x, gamma, beta, xn}, [=](cg_tensor* self) {
    for (int f = 0; f < F; ++f) {
      double sg = 0, sgx = 0;
      for (int n = 0; n < N; ++n) for (int s = 0; s < S; ++s) { const size_t i = at(n, f, s); sg += self->grad[i]; sgx += (double)self->grad[i] * xn->data[i]; }
      gamma->grad[f] += (float)sgx; beta->grad[f] += (float)sg;
      if (!in_grad(x)) continue;
      const float k = gamma->data[f] * inv_std[f];
      for (int n = 0; n < N; ++n) for (int s = 0; s < S; ++s) {
        const size_t i = at(n, f, s);
        x->grad[i] += training ? k * (self->grad[i] - (float)(sg / cnt) - xn->data[i] * (float)(sgx / cnt)) : k * self->grad[i];
      }
    }
  });
  return publish(L, x, y);
}
static void batchnorm_free(cg_layer* L) {
  cg_batchnorm* l = (cg_batchnorm*)L;
  cg_tensor* ts[6] = {l->running_mean, l->running_var, l->x_norm, l->std_inv, l->batch_mean, l->batch_var};
  for (cg_tensor* t : ts) if (t) cg_tensor_release(t);
  plain_free(L);
}
static int two_params(cg_layer*) { return 2; }
static cg_tensor** batchnorm_gp(cg_layer* L) { return ((cg_batchnorm*)L)->param_ptrs; }
CG_EXPORT cg_batchnorm* cg_batchnorm_new(int F, float eps, float momentum) {
  if (F <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_batchnorm*)nullptr);
  auto* l = new_layer<cg_batchnorm>("BatchNorm");
  if (!l) return nullptr;
  l->num_features = F; l->epsilon = eps > 0 ? eps : 1e-5f; l->momentum = momentum > 0 ? momentum : 0.1f; l->training = true;
  int fs[1] = {F};
  l->base.weights = cg_tensor_ones(fs, 1, true);
  l->base.bias = make(fs, 1, true);
  l->running_mean = make(fs, 1, false);
  l->running_var = cg_tensor_ones(fs, 1, false);
  l->param_ptrs[0] = l->base.weights; l->param_ptrs[1] = l->base.bias;
  finish(&l->base, batchnorm_forward, batchnorm_free, two_params, batchnorm_gp);
  return l;
}
CG_EXPORT void cg_batchnorm_set_training(cg_batchnorm* l, bool t) { if (l) l->training = t; }

// ----------------------------------------------------------------- rmsnorm
static cg_tensor* rmsnorm_forward(cg_layer* L, cg_tensor* x) {
  cg_rmsnorm* l = (cg_rmsnorm*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  const int C = l->normalized_shape;
  if (cols_of(x) != C) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int R = rows_of(x);
  cg_tensor* y = make_like(x, false);
  if (!y) return nullptr;
  if (l->inv_rms) cg_tensor_release(l->inv_rms);
  int rs[1] = {R};
  cg_tensor* inv = l->inv_rms = make(rs, 1, false);
  cg_tensor* g = L->weights;
  for (int r = 0; r < R; ++r) {
    const float* p = x->data + (size_t)r * C;
    double ss = 0; for (int j = 0; j < C; ++j) ss += (double)p[j] * p[j];
    const float iv = 1.0f / std::sqrt((float)(ss / C) + l->epsilon);
    inv->data[r] = iv;
    for (int j = 0; j < C; ++j) y->data[(size_t)r * C + j] = p[j] * iv * g->data[j];
  }
  cg_tensor_retain(inv);
  attach(y, {x, g, inv}, [x, g, inv, R, C](cg_tensor* self) {
    for (int r = 0; r < R; ++r) {
      const float* p = x->data + (size_t)r * C; const float* go = self->grad + (size_t)r * C;
      const float iv = inv->data[r];
      double dot = 0;
      for (int j = 0; j < C; ++j) { g->grad[j] += go[j] * p[j] * iv; dot += (double)go[j] * g->data[j] * p[j]; }
      if (!in_grad(x)) continue;
      const float c = (float)(dot / C) * iv * iv * iv;
      for (int j = 0; j < C; ++j) x->grad[(size_t)r * C + j] += go[j] * g->data[j] * iv - p[j] * c;
    }
  });
  cg_tensor_release(inv);
  return publish(L, x, y);
}
static void rmsnorm_free(cg_layer* L) { cg_rmsnorm* l = (cg_rmsnorm*)L; if (l->inv_rms) cg_tensor_release(l->inv_rms); plain_free(L); }
static int one_param(cg_layer*) { return 1; }
static cg_tensor** rmsnorm_gp(cg_layer* L) { return ((cg_rmsnorm*)L)->param_ptrs; }
CG_EXPORT cg_rmsnorm* cg_rmsnorm_new(int C, float eps) {
  if (C <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_rmsnorm*)nullptr);
  auto* l = new_layer<cg_rmsnorm>("RMSNorm");
  if (!l) return nullptr;
  l->normalized_shape = C; l->epsilon = eps > 0 ? eps : 1e-6f;
  int cs[1] = {C};
  l->base.weights = cg_tensor_ones(cs, 1, true);
  l->param_ptrs[0] = l->base.weights;
  finish(&l->base, rmsnorm_forward, rmsnorm_free, one_param, rmsnorm_gp);
  return l;
}

// ------------------------------------------------------------------ swiglu
// [..., 2H] -> [..., H]: silu(x[..., :H]) * x[..., H:]
static cg_tensor* swiglu_apply(cg_tensor* x) {
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  const int C2 = cols_of(x);
  if (C2 % 2) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int H = C2 / 2, R = rows_of(x);
  int shape[CG_MAX_DIMS];
  for (int i = 0; i < x->ndim; ++i) shape[i] = x->shape[i];
  shape[x->ndim - 1] = H;
  cg_tensor* y = make(shape, x->ndim, false);
  if (!y) return nullptr;
  for (int r = 0; r < R; ++r) for (int j = 0; j < H; ++j)
    y->data[(size_t)r * H + j] = siluf(x->data[(size_t)r * C2 + j]) * x->data[(size_t)r * C2 + H + j];
  attach(y, {x}, [x, R, H, C2](cg_tensor* self) {
    if (!in_grad(x)) return;
    for (int r = 0; r < R; ++r) for (int j = 0; j < H; ++j) {
      const float a = x->data[(size_t)r * C2 + j], b = x->data[(size_t)r * C2 + H + j], g = self->grad[(size_t)r * H + j];
      const float s = sigmoidf(a);
      x->grad[(size_t)r * C2 + j] += g * b * s * (1.0f + a * (1.0f - s));
      x->grad[(size_t)r * C2 + H + j] += g * a * s;
    }
  });
  return y;
}
static cg_tensor* swiglu_forward(cg_layer* L, cg_tensor* x) { cg_tensor* y = swiglu_apply(x); return y ? publish(L, x, y) : nullptr; }
CG_EXPORT cg_swiglu* cg_swiglu_new(void) { auto* l = new_layer<cg_swiglu>("SwiGLU"); if (l) finish(&l->base, swiglu_forward, plain_free, zero_params, no_params); return l; }
CG_EXPORT cg_tensor* cg_swiglu_forward_split(cg_tensor* x) { return swiglu_apply(x); }

// ------------------------------------------------------------------ conv2d
static void im2col(const float* img, int C, int H, int W, int k, int stride, int pad, int OH, int OW, float* col) {
  for (int c = 0; c < C; ++c) for (int ky = 0; ky < k; ++ky) for (int kx = 0; kx < k; ++kx) {
    float* dst = col + (((size_t)c * k + ky) * k + kx) * OH * OW;
    for (int oy = 0; oy < OH; ++oy) {
      const int iy = oy * stride - pad + ky;
      for (int ox = 0; ox < OW; ++ox) {
        const int ix = ox * stride - pad + kx;
        dst[(size_t)oy * OW + ox] = (iy >= 0 && iy < H && ix >= 0 && ix < W) ? img[((size_t)c * H + iy) * W + ix] : 0.0f;
      }
    }
  }
}
static void col2im_add(const float* col, int C, int H, int W, int k, int stride, int pad, int OH, int OW, float* img) {
  for (int c = 0; c < C; ++c) for (int ky = 0; ky < k; ++ky) for (int kx = 0; kx < k; ++kx) {
    const float* src = col + (((size_t)c * k + ky) * k + kx) * OH * OW;
    for (int oy = 0; oy < OH; ++oy) {
      const int iy = oy * stride - pad + ky;
      if (iy < 0 || iy >= H) continue;
      for (int ox = 0; ox < OW; ++ox) {
        const int ix = ox * stride - pad + kx;
        if (ix >= 0 && ix < W) img[((size_t)c * H + iy) * W + ix] += src[(size_t)oy * OW + ox];
      }
    }
  }
}
static cg_tensor* conv2d_forward(cg_layer* L, cg_tensor* x) {
  cg_conv2d* l = (cg_conv2d*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (x->ndim != 4 || x->shape[1] != l->in_channels) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int N = x->shape[0], C = l->in_channels, H = x->shape[2], W = x->shape[3], k = l->kernel_size, st = l->stride, pd = l->padding;
  const int OH = (H + 2 * pd - k) / st + 1, OW = (W + 2 * pd - k) / st + 1, OC = l->out_channels, CK = C * k * k, P = OH * OW;
  if (OH <= 0 || OW <= 0) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  int ys[4] = {N, OC, OH, OW};
  cg_tensor* y = make(ys, 4, false);
  if (!y) return nullptr;
  if (l->col_buffer) cg_tensor_release(l->col_buffer);
  int cs[3] = {N, CK, P};
  cg_tensor* col = l->col_buffer = make(cs, 3, false);
  cg_tensor* Wt = L->weights; cg_tensor* b = L->bias;
  for (int n = 0; n < N; ++n) {
    float* cn = col->data + (size_t)n * CK * P;
    im2col(x->data + (size_t)n * C * H * W, C, H, W, k, st, pd, OH, OW, cn);
    float* yn = y->data + (size_t)n * OC * P;
    gemm(Wt->data, cn, yn, OC, P, CK, false, false, false);
    if (b) for (int o = 0; o < OC; ++o) for (int p = 0; p < P; ++p) yn[(size_t)o * P + p] += b->data[o];
  }
  cg_tensor_retain(col);
  attach(y, {x, Wt, b, col}, [=](cg_tensor* self) {
    std::vector<float> dcol(in_grad(x) ? (size_t)CK * P : 0);
    for (int n = 0; n < N; ++n) {
      const float* g = self->grad + (size_t)n * OC * P;
      const float* cn = col->data + (size_t)n * CK * P;
      gemm(g, cn, Wt->grad, OC, CK, P, false, true, true);                        // dW += G col^T
      if (b) for (int o = 0; o < OC; ++o) { double s = 0; for (int p = 0; p < P; ++p) s += g[(size_t)o * P + p]; b->grad[o] += (float)s; }
      if (in_grad(x)) {
        gemm(Wt->data, g, dcol.data(), CK, P, OC, true, false, false);           // dcol = W^T G
        col2im_add(dcol.data(), C, H, W, k, st, pd, OH, OW, x->grad + (size_t)n * C * H * W);
      }
    }
  });
  cg_tensor_release(col);
  return publish(L, x, y);
}
static void conv2d_free(cg_layer* L) { cg_conv2d* l = (cg_conv2d*)L; if (l->col_buffer) cg_tensor_release(l->col_buffer); plain_free(L); }
static cg_tensor** conv2d_gp(cg_layer* L) { return ((cg_conv2d*)L)->param_ptrs; }
CG_EXPORT cg_conv2d* cg_conv2d_new(int ic, int oc, int k, int stride, int padding, bool use_bias) {
  if (ic <= 0 || oc <= 0 || k <= 0 || stride <= 0 || padding < 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_conv2d*)nullptr);
  auto* l = new_layer<cg_conv2d>("Conv2D");
  if (!l) return nullptr;
  l->in_channels = ic; l->out_channels = oc; l->kernel_size = k; l->stride = stride; l->padding = padding;
  int ws[2] = {oc, ic * k * k};
  l->base.weights = make(ws, 2, true);
  Rng rng(next_layer_seed());
  const float std_ = std::sqrt(2.0f / (ic * k * k));            // Kaiming normal
  for (int i = 0; i < l->base.weights->size; ++i) l->base.weights->data[i] = rng.normal() * std_;
  int bs[1] = {oc};
  l->base.bias = use_bias ? make(bs, 1, true) : nullptr;
  l->param_ptrs[0] = l->base.weights; l->param_ptrs[1] = l->base.bias;
  finish(&l->base, conv2d_forward, conv2d_free, linear_np, conv2d_gp);       // one or two parameters, like Linear
  return l;
}

// --------------------------------------------------------------- maxpool2d
static cg_tensor* maxpool_forward(cg_layer* L, cg_tensor* x) {
  cg_maxpool2d* l = (cg_maxpool2d*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (x->ndim != 4) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3], k = l->kernel_size, st = l->stride;
  const int OH = (H - k) / st + 1, OW = (W - k) / st + 1;
  if (OH <= 0 || OW <= 0) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  int ys[4] = {N, C, OH, OW};
  cg_tensor* y = make(ys, 4, false);
  if (!y) return nullptr;
  std::free(l->max_indices);
  int* idx = l->max_indices = (int*)std::malloc(sizeof(int) * (y->size ? y->size : 1));
  for (int nc = 0; nc < N * C; ++nc) {
    const float* img = x->data + (size_t)nc * H * W;
    for (int oy = 0; oy < OH; ++oy) for (int ox = 0; ox < OW; ++ox) {
      int best = (oy * st) * W + ox * st;
      for (int ky = 0; ky < k; ++ky) for (int kx = 0; kx < k; ++kx) {
        const int i = (oy * st + ky) * W + ox * st + kx;
        if (img[i] > img[best]) best = i;
      }
      const size_t o = ((size_t)nc * OH + oy) * OW + ox;
      y->data[o] = img[best]; idx[o] = nc * H * W + best;
    }
  }
  std::vector<int> saved(idx, idx + y->size);
  attach(y, {x}, [x, saved](cg_tensor* self) {
    if (!in_grad(x)) return;
    for (int i = 0; i < self->size; ++i) x->grad[saved[i]] += self->grad[i];
  });
  return publish(L, x, y);
}
static void maxpool_free(cg_layer* L) { std::free(((cg_maxpool2d*)L)->max_indices); plain_free(L); }
CG_EXPORT cg_maxpool2d* cg_maxpool2d_new(int k, int stride) {
  if (k <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_maxpool2d*)nullptr);
  auto* l = new_layer<cg_maxpool2d>("MaxPool2D");
  if (!l) return nullptr;
  l->kernel_size = k; l->stride = stride > 0 ? stride : k;
  finish(&l->base, maxpool_forward, maxpool_free, zero_params, no_params);
  return l;
}

// ----------------------------------------------------------------- flatten
static cg_tensor* flatten_forward(cg_layer* L, cg_tensor* x) {
  cg_flatten* l = (cg_flatten*)L;
  if (!x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  l->input_ndim = x->ndim;
  for (int i = 0; i < x->ndim; ++i) l->input_shape[i] = x->shape[i];
  const int N = x->ndim ? x->shape[0] : 1;
  int ys[2] = {N, N ? x->size / N : 0};
  cg_tensor* y = make(ys, 2, false);
  if (!y) return nullptr;
  std::memcpy(y->data, x->data, sizeof(float) * x->size);
  attach(y, {x}, [x](cg_tensor* self) { if (in_grad(x)) for (int i = 0; i < x->size; ++i) x->grad[i] += self->grad[i]; });
  return publish(L, x, y);
}
CG_EXPORT cg_flatten* cg_flatten_new(void) { auto* l = new_layer<cg_flatten>("Flatten"); if (l) finish(&l->base, flatten_forward, plain_free, zero_params, no_params); return l; }

// -------------------------------------------------------------- sequential
static cg_tensor* seq_forward(cg_layer* L, cg_tensor* x) { return cg_sequential_forward((cg_sequential*)L, x); }
static void seq_backward(cg_layer* L, cg_tensor* g) { cg_sequential_backward((cg_sequential*)L, g); }
static void seq_free(cg_layer* L) { cg_sequential_free((cg_sequential*)L); }
static int seq_np(cg_layer* L) { return cg_sequential_num_params((cg_sequential*)L); }
static cg_tensor** seq_gp(cg_layer* L) { return cg_sequential_get_params((cg_sequential*)L); }
CG_EXPORT cg_sequential* cg_sequential_new(void) {
  auto* s = new_layer<cg_sequential>("Sequential");
  if (!s) return nullptr;
  s->base.forward = seq_forward; s->base.backward = seq_backward; s->base.free = seq_free;
  s->base.num_params = seq_np; s->base.get_params = seq_gp;
  return s;
}
CG_EXPORT void cg_sequential_add(cg_sequential* s, cg_layer* layer) {
  if (!s || !layer) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (s->num_layers == s->capacity) {
    const int cap = s->capacity ? s->capacity * 2 : 8;
    cg_layer** nl = (cg_layer**)std::realloc(s->layers, sizeof(cg_layer*) * cap);
    if (!nl) { set_error(CG_ERROR_OUT_OF_MEMORY); return; }
    s->layers = nl; s->capacity = cap;
  }
  s->layers[s->num_layers++] = layer;
  std::free(s->param_cache); s->param_cache = nullptr;
}
CG_EXPORT cg_tensor* cg_sequential_forward(cg_sequential* s, cg_tensor* x) {
  if (!s || !x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  // Every layer hands its output to us and keeps references to its input and output itself: an intermediate can go
  // once the next layer has taken it; the last output is the caller's.
  cg_tensor* cur = x; cg_tensor* mine = nullptr;
  for (int i = 0; i < s->num_layers && cur; ++i) {
    cg_tensor* next = s->layers[i]->forward(s->layers[i], cur);
    if (mine) cg_tensor_release(mine);
    mine = cur = next;
  }
  if (s->num_layers == 0) cg_tensor_retain(x);      // nothing ran: the caller still gets a reference of its own
  s->base.output = cur;     // not counted: the last layer holds it
  return cur;
}
CG_EXPORT void cg_sequential_backward(cg_sequential* s, cg_tensor* grad_output) {
  if (!s || !grad_output || s->num_layers == 0) { set_error(CG_ERROR_NULL_POINTER); return; }
  cg_tensor* o = s->layers[s->num_layers - 1]->output;
  if (!o || !o->backward_fn || tape_ran(o)) return;
  if (grad_output->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  ensure_grad(o);
  if (grad_output != o) std::memcpy(o->grad, upstream(grad_output), sizeof(float) * o->size);
  else { bool any = false; for (int i = 0; i < o->size; ++i) any = any || o->grad[i] != 0.0f; if (!any) return; }
  cg_backward(o);
}
CG_EXPORT void cg_sequential_free(cg_sequential* s) {
  if (!s) return;
  for (int i = 0; i < s->num_layers; ++i) cg_layer_free(s->layers[i]);
  std::free(s->layers); std::free(s->param_cache); std::free(s);
}
CG_EXPORT int cg_sequential_num_params(cg_sequential* s) {
  int n = 0;
  if (s) for (int i = 0; i < s->num_layers; ++i) n += s->layers[i]->num_params ? s->layers[i]->num_params(s->layers[i]) : 0;
  return n;
}
CG_EXPORT cg_tensor** cg_sequential_get_params(cg_sequential* s) {
  if (!s) return nullptr;
  const int n = cg_sequential_num_params(s);
  std::free(s->param_cache);
  s->param_cache = (cg_tensor**)std::malloc(sizeof(cg_tensor*) * (n ? n : 1));
  int k = 0;
  for (int i = 0; i < s->num_layers; ++i) {
    cg_layer* l = s->layers[i];
    const int m = l->num_params ? l->num_params(l) : 0;
    cg_tensor** p = m ? l->get_params(l) : nullptr;
    for (int j = 0; j < m; ++j) s->param_cache[k++] = p[j];
  }
  return s->param_cache;
}
CG_EXPORT void cg_sequential_zero_grad(cg_sequential* s) {
  if (!s) return;
  for (int i = 0; i < s->num_layers; ++i) cg_layer_zero_grad(s->layers[i]);
}
