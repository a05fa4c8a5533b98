// Host attention: tiled online-softmax forward and backward (the oracle of the GPU flash
// kernels), RoPE, ALiBi, launch heuristics, and the transformer block built on them.
// Reference surface: include/cg_flash_attn.h, src/attention/flash_attn.c,
// include/cg_transformer.h, src/layers/transformer.c.
#include <algorithm>

#include "internal.hpp"

using namespace cgi;

namespace {
struct Dims { int B, Tq, Tk, H, Hk, D; };
bool dims_of(const cg_flash_attn_params* p, Dims* d) {
  if (!p || !p->Q || !p->K || !p->V || p->Q->ndim != 4 || p->K->ndim != 4 || p->V->ndim != 4) return false;
  d->B = p->Q->shape[0]; d->Tq = p->Q->shape[1]; d->H = p->Q->shape[2]; d->D = p->Q->shape[3];
  d->Tk = p->K->shape[1]; d->Hk = p->K->shape[2];
  return p->K->shape[0] == d->B && p->K->shape[3] == d->D && p->V->size == p->K->size && d->Hk > 0 && d->H % d->Hk == 0;
}
// Additive bias / visibility of key k for query q.
inline bool visible(const cg_flash_attn_params* p, int q, int k, int shift) {
  const int rel = k - (q + shift);
  if ((p->mask_type == CG_MASK_CAUSAL || p->mask_type == CG_MASK_SLIDING_WINDOW) && rel > 0) return false;
  if (p->mask_type == CG_MASK_SLIDING_WINDOW && p->window_size > 0 && -rel >= p->window_size) return false;
  return true;
}
inline float bias_of(const cg_flash_attn_params* p, const Dims& d, int b, int h, int q, int k, int shift) {
  float v = 0.0f;
  if (p->alibi_slopes) v += p->alibi_slopes[h] * (float)(k - (q + shift));
  if (p->mask_type == CG_MASK_CUSTOM && p->mask) {
    const cg_tensor* m = p->mask;
    const size_t per = (size_t)d.Tq * d.Tk;
    size_t off = (size_t)q * d.Tk + k;
    if ((size_t)m->size == per * d.B * d.H) off += ((size_t)b * d.H + h) * per;
    else if ((size_t)m->size == per * d.B) off += (size_t)b * per;
    v += m->data[off];
  }
  return v;
}
cg_tensor* ensure_like(cg_tensor*& slot, const cg_tensor* like) { if (!slot) slot = make_like(like, false); return slot; }

// A parameter block filled the reference's way (include/cg_flash_attn.h:51-88): raw fp32 arrays in the operand slots.
// The arrays are wrapped in tensor headers that do not own them, the tensor path runs, the headers go.
struct RawBlock {
  cg_flash_attn_params t;
  std::vector<cg_tensor*> headers;
  bool ok = false;
  cg_tensor* wrap(void* data, int a, int b, int c, int d4) {
    if (!data) return nullptr;
    int shape[4] = {a, b, c, d4};
    cg_tensor* h = make_header(shape, d4 > 0 ? 4 : (c > 0 ? 3 : 2), false);
    if (!h) return nullptr;
    h->data = (float*)data; h->is_view = true;
    headers.push_back(h);
    return h;
  }
  RawBlock(const cg_flash_attn_params* p, bool backward) {
    std::memset(&t, 0, sizeof(t));
    const int B = p->batch_size, Tq = p->seqlen_q, Tk = p->seqlen_k > 0 ? p->seqlen_k : p->seqlen_q, H = p->n_heads;
    const int Hk = p->n_kv_heads > 0 ? p->n_kv_heads : H, D = p->d_head;
    if (B <= 0 || Tq <= 0 || H <= 0 || D <= 0 || !p->Q || !p->K || !p->V || !p->O) return;
    t.operand_mode = CG_FLASH_TENSOR_MODE;
    t.Q = wrap(p->Q, B, Tq, H, D); t.K = wrap(p->K, B, Tk, Hk, D); t.V = wrap(p->V, B, Tk, Hk, D); t.O = wrap(p->O, B, Tq, H, D);
    if (p->softmax_lse) t.L = wrap(p->softmax_lse, B, H, Tq, 0);
    if (p->mask_type == CG_MASK_CUSTOM && p->mask) t.mask = wrap(p->mask, Tq, Tk, 0, 0);
    if (backward) { t.dO = wrap(p->dO, B, Tq, H, D); t.dQ = wrap(p->dQ, B, Tq, H, D); t.dK = wrap(p->dK, B, Tk, Hk, D); t.dV = wrap(p->dV, B, Tk, Hk, D); }
    t.batch_size = B; t.seqlen_q = Tq; t.seqlen_k = Tk; t.n_heads = H; t.n_kv_heads = Hk; t.d_head = D;
    t.softmax_scale = p->softmax_scale; t.dropout_prob = p->dropout_prob; t.mask_type = p->mask_type; t.window_size = p->window_size;
    t.alibi_slopes = p->alibi_slopes; t.config = p->config;
    ok = t.Q && t.K && t.V && t.O && (!backward || (t.dO && t.dQ && t.dK && t.dV && t.L));
  }
  ~RawBlock() {
    if (t.L && std::find(headers.begin(), headers.end(), t.L) == headers.end()) cg_tensor_release(t.L);   // made by the forward pass
    for (cg_tensor* h : headers) cg_tensor_release(h);
  }
};
inline bool raw_block(const cg_flash_attn_params* p) { return p && p->operand_mode != CG_FLASH_TENSOR_MODE; }
}  // namespace
namespace cgi { bool flash_raw_block(const cg_flash_attn_params* p) { return raw_block(p); } }

CG_EXPORT void cg_flash_attention_forward_cpu(cg_flash_attn_params* p) {
  if (raw_block(p)) {
    RawBlock r(p, false);
    if (!r.ok) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
    cg_flash_attention_forward_cpu(&r.t);
    return;
  }
  Dims d;
  if (!dims_of(p, &d)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  ensure_like(p->O, p->Q);
  if (!p->L) { int ls[3] = {d.B, d.H, d.Tq}; p->L = make(ls, 3, false); }
  const float scale = p->softmax_scale > 0 ? p->softmax_scale : 1.0f / std::sqrt((float)d.D);
  const int bn = p->config.block_n > 0 ? p->config.block_n : 64, rep = d.H / d.Hk, shift = d.Tk - d.Tq;
  std::vector<float> s(bn), acc(d.D);
  for (int b = 0; b < d.B; ++b) for (int h = 0; h < d.H; ++h) for (int q = 0; q < d.Tq; ++q) {
    const float* qv = p->Q->data + (((size_t)b * d.Tq + q) * d.H + h) * d.D;
    float m = -INFINITY, l = 0.0f;
    std::fill(acc.begin(), acc.end(), 0.0f);
    for (int k0 = 0; k0 < d.Tk; k0 += bn) {
      const int kn = d.Tk - k0 < bn ? d.Tk - k0 : bn;
      float tile_max = -INFINITY;
      for (int j = 0; j < kn; ++j) {
        const int k = k0 + j;
        if (!visible(p, q, k, shift)) { s[j] = -INFINITY; continue; }
        const float* kv = p->K->data + (((size_t)b * d.Tk + k) * d.Hk + h / rep) * d.D;
        float dot = 0; for (int e = 0; e < d.D; ++e) dot += qv[e] * kv[e];
        s[j] = dot * scale + bias_of(p, d, b, h, q, k, shift);
        tile_max = s[j] > tile_max ? s[j] : tile_max;
      }
      if (tile_max == -INFINITY) continue;
      const float mn = tile_max > m ? tile_max : m, corr = std::exp(m - mn);
      l *= corr;
      for (int e = 0; e < d.D; ++e) acc[e] *= corr;
      for (int j = 0; j < kn; ++j) {
        if (s[j] == -INFINITY) continue;
        const float pj = std::exp(s[j] - mn);
        l += pj;
        const float* vv = p->V->data + (((size_t)b * d.Tk + k0 + j) * d.Hk + h / rep) * d.D;
        for (int e = 0; e < d.D; ++e) acc[e] += pj * vv[e];
      }
      m = mn;
    }
    float* o = p->O->data + (((size_t)b * d.Tq + q) * d.H + h) * d.D;
    const float inv = l > 0 ? 1.0f / l : 0.0f;
    for (int e = 0; e < d.D; ++e) o[e] = acc[e] * inv;
    p->L->data[((size_t)b * d.H + h) * d.Tq + q] = l > 0 ? m + std::log(l) : -INFINITY;
  }
}

// Needs O and L from the forward pass and dO; fills (overwrites) dQ, dK, dV.
CG_EXPORT void cg_flash_attention_backward_cpu(cg_flash_attn_params* p) {
  if (raw_block(p)) {
    RawBlock r(p, true);
    if (!r.ok) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
    cg_flash_attention_backward_cpu(&r.t);
    return;
  }
  Dims d;
  if (!dims_of(p, &d) || !p->O || !p->L || !p->dO || p->dO->size != p->Q->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  ensure_like(p->dQ, p->Q); ensure_like(p->dK, p->K); ensure_like(p->dV, p->V);
  std::memset(p->dQ->data, 0, sizeof(float) * p->dQ->size);
  std::memset(p->dK->data, 0, sizeof(float) * p->dK->size);
  std::memset(p->dV->data, 0, sizeof(float) * p->dV->size);
  const float scale = p->softmax_scale > 0 ? p->softmax_scale : 1.0f / std::sqrt((float)d.D);
  const int rep = d.H / d.Hk, shift = d.Tk - d.Tq;
  for (int b = 0; b < d.B; ++b) for (int h = 0; h < d.H; ++h) for (int q = 0; q < d.Tq; ++q) {
    const size_t qo = (((size_t)b * d.Tq + q) * d.H + h) * d.D;
    const float* qv = p->Q->data + qo; const float* dov = p->dO->data + qo; const float* ov = p->O->data + qo;
    float* dq = p->dQ->data + qo;
    const float lse = p->L->data[((size_t)b * d.H + h) * d.Tq + q];
    if (lse == -INFINITY) continue;
    float delta = 0; for (int e = 0; e < d.D; ++e) delta += dov[e] * ov[e];
    for (int k = 0; k < d.Tk; ++k) {
      if (!visible(p, q, k, shift)) continue;
      const size_t ko = (((size_t)b * d.Tk + k) * d.Hk + h / rep) * d.D;
      const float* kv = p->K->data + ko; const float* vv = p->V->data + ko;
      float dot = 0, dp = 0;
      for (int e = 0; e < d.D; ++e) { dot += qv[e] * kv[e]; dp += dov[e] * vv[e]; }
      const float pj = std::exp(dot * scale + bias_of(p, d, b, h, q, k, shift) - lse);
      const float ds = pj * (dp - delta) * scale;
      float* dk = p->dK->data + ko; float* dv = p->dV->data + ko;
      for (int e = 0; e < d.D; ++e) { dv[e] += pj * dov[e]; dq[e] += ds * kv[e]; dk[e] += ds * qv[e]; }
    }
  }
}
// In this host library the device-less entry points run the host kernels; the GPU package
// routes the same parameter block to the sm_100a kernels.
CG_EXPORT void cg_flash_attention_forward(cg_flash_attn_params* p) { cg_flash_attention_forward_cpu(p); }
CG_EXPORT void cg_flash_attention_backward(cg_flash_attn_params* p) { cg_flash_attention_backward_cpu(p); }
CG_EXPORT void cg_flash_attention_mqa(cg_flash_attn_params* p) {
  if (raw_block(p)) { if (p->n_kv_heads != 1) { set_error(CG_ERROR_SHAPE_MISMATCH); return; } cg_flash_attention_forward(p); return; }
  if (!p || !p->K || p->K->ndim != 4 || p->K->shape[2] != 1) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  p->n_kv_heads = 1;
  cg_flash_attention_forward(p);
}
CG_EXPORT void cg_flash_attention_gqa(cg_flash_attn_params* p, int num_kv_groups) {
  if (raw_block(p)) { if (num_kv_groups <= 0) { set_error(CG_ERROR_SHAPE_MISMATCH); return; } p->n_kv_heads = num_kv_groups; cg_flash_attention_forward(p); return; }
  if (!p || !p->K || p->K->ndim != 4 || num_kv_groups <= 0 || p->K->shape[2] != num_kv_groups) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  p->n_kv_heads = num_kv_groups;
  cg_flash_attention_forward(p);
}
CG_EXPORT cg_flash_attn_params* cg_flash_attn_params_new(cg_tensor* Q, cg_tensor* K, cg_tensor* V, cg_attention_mask_type mt, float dropout) {
  if (!Q || !K || !V) return fail(CG_ERROR_NULL_POINTER, (cg_flash_attn_params*)nullptr);
  cg_flash_attn_params* p = (cg_flash_attn_params*)std::calloc(1, sizeof(cg_flash_attn_params));
  p->Q = Q; p->K = K; p->V = V; p->mask_type = mt; p->dropout_prob = dropout;
  p->operand_mode = CG_FLASH_TENSOR_MODE;
  Dims d;
  if (!dims_of(p, &d)) { std::free(p); return fail(CG_ERROR_SHAPE_MISMATCH, (cg_flash_attn_params*)nullptr); }
  p->batch_size = d.B; p->seqlen_q = d.Tq; p->seqlen_k = d.Tk; p->n_heads = d.H; p->n_kv_heads = d.Hk; p->d_head = d.D;
  p->softmax_scale = 1.0f / std::sqrt((float)d.D);
  p->config = cg_flash_attn_autotune(d.Tq, d.Tk, d.D, 148);
  p->O = make_like(Q, false);
  int ls[3] = {d.B, d.H, d.Tq};
  p->L = make(ls, 3, false);
  p->softmax_lse = p->L ? p->L->data : nullptr;
  p->is_training = Q->requires_grad || K->requires_grad || V->requires_grad;
  return p;
}
// Frees the block and the tensors it created (O, L, dQ, dK, dV); Q, K, V, dO, mask stay the caller's.
CG_EXPORT void cg_flash_attn_params_free(cg_flash_attn_params* p) {
  if (!p) return;
  cg_tensor* owned[5] = {p->O, p->L, p->dQ, p->dK, p->dV};
  for (cg_tensor* t : owned) if (t) cg_tensor_release(t);
  std::free(p);
}
// Tile shapes of the sm_100a kernels: two 128-row query tiles per CTA against 128-key tiles,
// a 4-deep (d<=64) or 3-deep K/V ring; short-query decode splits the keys over the SMs.
CG_EXPORT cg_flash_attn_config cg_flash_attn_autotune(int tq, int tk, int d, int sm_count) {
  cg_flash_attn_config c{};
  c.block_m = tq >= 256 ? 256 : 128; c.block_n = 128; c.num_warps = 12;
  c.num_stages = d <= 64 ? 4 : 3; c.use_register_tiling = true; c.split_k = 1;
  c.sm_count = sm_count;
  c.use_persistent = sm_count > 0 && (tq + c.block_m - 1) / c.block_m > sm_count;
  if (tq <= 16 && sm_count > 0) {
    const int tiles = (tk + c.block_n - 1) / c.block_n;
    int split = tiles < sm_count ? tiles : sm_count;
    c.split_k = split < 1 ? 1 : split;
  }
  return c;
}
CG_EXPORT size_t cg_flash_attn_shared_mem(int bm, int bn, int d) {
  const int stages = d <= 64 ? 4 : 3;
  return ((size_t)bm * d + (size_t)stages * 2 * bn * d) * 2 /* bf16 */ + 1024;
}

// ------------------------------------------------------------ RoPE / ALiBi
CG_EXPORT void cg_rope_precompute_freqs(float* cos_cache, float* sin_cache, int max_seqlen, int d_head, float theta) {
  if (!cos_cache || !sin_cache) { set_error(CG_ERROR_NULL_POINTER); return; }
  const int half = d_head / 2;
  for (int t = 0; t < max_seqlen; ++t) for (int i = 0; i < half; ++i) {
    const float a = t * std::pow(theta, -2.0f * i / d_head);
    cos_cache[(size_t)t * half + i] = std::cos(a); sin_cache[(size_t)t * half + i] = std::sin(a);
  }
}
static void rope_rows(float* x, int T, int H, int D, int offset, float theta, float sign) {
  const int half = D / 2;
  for (int t = 0; t < T; ++t) for (int i = 0; i < half; ++i) {
    const float a = (t + offset) * std::pow(theta, -2.0f * i / D), c = std::cos(a), s = sign * std::sin(a);
    for (int h = 0; h < H; ++h) {
      float* v = x + ((size_t)t * H + h) * D;
      const float x0 = v[i], x1 = v[i + half];
      v[i] = x0 * c - x1 * s; v[i + half] = x0 * s + x1 * c;
    }
  }
}
// Q and K are [seqlen, n_heads, d_head]; element i is paired with i + d_head/2.
CG_EXPORT void cg_apply_rope(float* Q, float* K, int T, int H, int D, int offset, float theta) {
  if (theta <= 0) theta = 10000.0f;
  if (Q) rope_rows(Q, T, H, D, offset, theta, 1.0f);
  if (K) rope_rows(K, T, H, D, offset, theta, 1.0f);
}
CG_EXPORT void cg_alibi_slopes(float* slopes, int H) {
  if (!slopes || H <= 0) return;
  int p2 = 1; while (p2 * 2 <= H) p2 *= 2;
  const float base = std::pow(2.0f, -8.0f / p2);
  for (int i = 0; i < p2 && i < H; ++i) slopes[i] = std::pow(base, (float)(i + 1));
  if (p2 < H) { const float eb = std::pow(2.0f, -4.0f / p2); for (int i = p2; i < H; ++i) slopes[i] = std::pow(eb, (float)(2 * (i - p2) + 1)); }
}
// bias [n_heads, seqlen_q, seqlen_k] = slope_h * (k - (q + seqlen_k - seqlen_q))
CG_EXPORT void cg_alibi_bias(float* bias, int Tq, int Tk, int H, float* slopes) {
  if (!bias) { set_error(CG_ERROR_NULL_POINTER); return; }
  std::vector<float> own;
  if (!slopes) { own.resize(H); cg_alibi_slopes(own.data(), H); slopes = own.data(); }
  for (int h = 0; h < H; ++h) for (int q = 0; q < Tq; ++q) for (int k = 0; k < Tk; ++k)
    bias[((size_t)h * Tq + q) * Tk + k] = slopes[h] * (float)(k - (q + Tk - Tq));
}

// ------------------------------------------------------- transformer block
// x [T, hidden].  pre-norm:  x += attn(norm1(x));  x += mlp(norm2(x))   (post-norm: norm after the add).
// attention: q/k/v projections, grouped-query heads, optional additive mask [T, T] (else causal).
namespace {
cg_tensor* attention_op(cg_tensor* q, cg_tensor* k, cg_tensor* v, cg_tensor* mask, int H, int Hk, int D) {
  const int T = rows_of(q);
  auto setup = [=](cg_flash_attn_params* p, cg_tensor* Q4, cg_tensor* K4, cg_tensor* V4) {
    std::memset(p, 0, sizeof(*p));
    p->Q = Q4; p->K = K4; p->V = V4;
    p->mask_type = mask ? CG_MASK_CUSTOM : CG_MASK_CAUSAL; p->mask = mask;
    p->softmax_scale = 1.0f / std::sqrt((float)D);
    p->operand_mode = CG_FLASH_TENSOR_MODE;
  };
  auto view4 = [T, D](cg_tensor* t, int heads) { cg_tensor w = *t; w.ndim = 4; w.shape[0] = 1; w.shape[1] = T; w.shape[2] = heads; w.shape[3] = D; return w; };
  cg_tensor Q4 = view4(q, H), K4 = view4(k, Hk), V4 = view4(v, Hk);
  cg_flash_attn_params p;
  setup(&p, &Q4, &K4, &V4);
  cg_flash_attention_forward_cpu(&p);
  cg_tensor* O = p.O; cg_tensor* L = p.L;
  int os[2] = {T, H * D};
  cg_tensor_reshape(O, os, 2);
  attach(O, {q, k, v, L, mask}, [=](cg_tensor* self) {
    cg_tensor Q4b = view4(q, H), K4b = view4(k, Hk), V4b = view4(v, Hk), O4 = view4(self, H);
    cg_tensor dO = O4; dO.data = self->grad;
    cg_flash_attn_params pb;
    setup(&pb, &Q4b, &K4b, &V4b);
    pb.O = &O4; pb.L = L; pb.dO = &dO;
    cg_flash_attention_backward_cpu(&pb);
    cg_tensor* gs[3] = {pb.dQ, pb.dK, pb.dV}; cg_tensor* ts[3] = {q, k, v};
    for (int i = 0; i < 3; ++i) { if (ts[i]->grad) for (int j = 0; j < ts[i]->size; ++j) ts[i]->grad[j] += gs[i]->data[j]; cg_tensor_release(gs[i]); }
  });
  cg_tensor_release(L);          // the node holds its own reference when it was attached
  return O;
}
cg_tensor* gelu_op(cg_tensor* x) {
  cg_tensor* y = make_like(x, false);
  for (int i = 0; i < x->size; ++i) y->data[i] = geluf(x->data[i]);
  attach(y, {x}, [x](cg_tensor* self) {
    if (!x->grad) return;
    for (int i = 0; i < x->size; ++i) {
      const float v = x->data[i], u = 0.7978845608f * (v + 0.044715f * v * v * v), t = std::tanh(u);
      x->grad[i] += self->grad[i] * (0.5f * (1 + t) + 0.5f * v * (1 - t * t) * 0.7978845608f * (1 + 3 * 0.044715f * v * v));
    }
  });
  return y;
}
cg_tensor* layernorm_fwd(cg_layer* L, cg_tensor* x);
}  // namespace

// LayerNorm as a layer (used when use_rms_norm is false): weights = gamma, bias = beta.
namespace {
struct LayerNormLayer { cg_layer base; int C; float eps; cg_tensor* params[2]; };
cg_tensor* layernorm_fwd(cg_layer* Lr, cg_tensor* x) {
  LayerNormLayer* l = (LayerNormLayer*)Lr;
  const int C = l->C, R = rows_of(x);
  if (cols_of(x) != C) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  cg_tensor* y = make_like(x, false);
  cg_tensor* g = Lr->weights; cg_tensor* b = Lr->bias;
  std::vector<float> mean(R), inv(R);
  for (int r = 0; r < R; ++r) {
    const float* p = x->data + (size_t)r * C;
    double m = 0, v = 0;
    for (int j = 0; j < C; ++j) m += p[j];
    m /= C;
    for (int j = 0; j < C; ++j) { const double dd = p[j] - m; v += dd * dd; }
    mean[r] = (float)m; inv[r] = 1.0f / std::sqrt((float)(v / C) + l->eps);
    for (int j = 0; j < C; ++j) y->data[(size_t)r * C + j] = (p[j] - mean[r]) * inv[r] * g->data[j] + b->data[j];
  }
  attach(y, {x, g, b}, [=](cg_tensor* self) {
    for (int r = 0; r < R; ++r) {
      const float* p = x->data + (size_t)r * C; const float* go = self->grad + (size_t)r * C;
      double s1 = 0, s2 = 0;
      for (int j = 0; j < C; ++j) {
        const float xh = (p[j] - mean[r]) * inv[r], gg = go[j] * g->data[j];
        g->grad[j] += go[j] * xh; b->grad[j] += go[j];
        s1 += gg; s2 += (double)gg * xh;
      }
      if (!x->grad) continue;
      for (int j = 0; j < C; ++j) {
        const float xh = (p[j] - mean[r]) * inv[r], gg = go[j] * g->data[j];
        x->grad[(size_t)r * C + j] += inv[r] * (gg - (float)(s1 / C) - xh * (float)(s2 / C));
      }
    }
  });
  if (x) cg_tensor_retain(x);
  if (y) cg_tensor_retain(y);                       // the layer's reference; the first one is the caller's
  if (Lr->input) cg_tensor_release(Lr->input);
  if (Lr->output) cg_tensor_release(Lr->output);
  Lr->input = x; Lr->output = y;
  return y;
}
void layernorm_free(cg_layer* L) {
  if (L->input) cg_tensor_release(L->input);
  if (L->output) cg_tensor_release(L->output);
  cg_tensor_release(L->weights); cg_tensor_release(L->bias);
  std::free(L);
}
int ln_np(cg_layer*) { return 2; }
cg_tensor** ln_gp(cg_layer* L) { return ((LayerNormLayer*)L)->params; }
cg_layer* layernorm_new(int C, float eps) {
  LayerNormLayer* l = (LayerNormLayer*)std::calloc(1, sizeof(LayerNormLayer));
  l->base.name = "LayerNorm"; l->C = C; l->eps = eps > 0 ? eps : 1e-5f;
  int cs[1] = {C};
  l->base.weights = cg_tensor_ones(cs, 1, true); l->base.bias = make(cs, 1, true);
  l->params[0] = l->base.weights; l->params[1] = l->base.bias;
  l->base.forward = layernorm_fwd; l->base.free = layernorm_free; l->base.num_params = ln_np; l->base.get_params = ln_gp;
  return &l->base;
}

cg_tensor* block_forward_default(cg_layer* L, cg_tensor* x) { return cg_transformer_forward(L, x, nullptr); }
void block_backward(cg_layer* L, cg_tensor* g) {
  cg_tensor* o = L->output;
  if (!o || !g || !o->backward_fn || tape_ran(o) || g->size != o->size) return;
  ensure_grad(o);
  if (g != o) std::memcpy(o->grad, g->grad ? g->grad : g->data, sizeof(float) * o->size);
  cg_backward(o);
}
void block_free(cg_layer* L) {
  cg_transformer_block* b = (cg_transformer_block*)L;
  cg_layer* subs[9] = {b->norm1, b->norm2, (cg_layer*)b->q_proj, (cg_layer*)b->k_proj, (cg_layer*)b->v_proj, (cg_layer*)b->o_proj,
                       (cg_layer*)b->gate_proj, (cg_layer*)b->up_proj, (cg_layer*)b->down_proj};
  for (cg_layer* s : subs) if (s) cg_layer_free(s);
  if (L->input) cg_tensor_release(L->input);
  if (L->output) cg_tensor_release(L->output);
  std::free(b->param_cache); std::free(b);
}
int block_np(cg_layer* L) { return ((cg_transformer_block*)L)->n_params; }
cg_tensor** block_gp(cg_layer* L) { return ((cg_transformer_block*)L)->param_cache; }
}  // namespace

CG_EXPORT cg_transformer_block* cg_transformer_block_new(cg_transformer_config c) {
  if (c.hidden_size <= 0 || c.num_heads <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_transformer_block*)nullptr);
  if (c.num_kv_heads <= 0) c.num_kv_heads = c.num_heads;
  if (c.head_dim <= 0) c.head_dim = c.hidden_size / c.num_heads;
  if (c.intermediate_size <= 0) c.intermediate_size = 4 * c.hidden_size;
  if (c.norm_eps <= 0) c.norm_eps = c.use_rms_norm ? 1e-6f : 1e-5f;
  if (c.num_heads % c.num_kv_heads) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_transformer_block*)nullptr);
  cg_transformer_block* b = (cg_transformer_block*)std::calloc(1, sizeof(cg_transformer_block));
  b->base.name = "TransformerBlock"; b->config = c;
  auto norm = [&]() { return c.use_rms_norm ? (cg_layer*)cg_rmsnorm_new(c.hidden_size, c.norm_eps) : layernorm_new(c.hidden_size, c.norm_eps); };
  b->norm1 = norm(); b->norm2 = norm();
  const int qd = c.num_heads * c.head_dim, kd = c.num_kv_heads * c.head_dim;
  b->q_proj = cg_linear_new(c.hidden_size, qd, c.use_bias);
  b->k_proj = cg_linear_new(c.hidden_size, kd, c.use_bias);
  b->v_proj = cg_linear_new(c.hidden_size, kd, c.use_bias);
  b->o_proj = cg_linear_new(qd, c.hidden_size, c.use_bias);
  if (c.use_swiglu) b->gate_proj = cg_linear_new(c.hidden_size, c.intermediate_size, c.use_bias);
  b->up_proj = cg_linear_new(c.hidden_size, c.intermediate_size, c.use_bias);
  b->down_proj = cg_linear_new(c.intermediate_size, c.hidden_size, c.use_bias);
  cg_layer* subs[9] = {b->norm1, b->norm2, (cg_layer*)b->q_proj, (cg_layer*)b->k_proj, (cg_layer*)b->v_proj, (cg_layer*)b->o_proj,
                       (cg_layer*)b->gate_proj, (cg_layer*)b->up_proj, (cg_layer*)b->down_proj};
  int n = 0;
  for (cg_layer* s : subs) if (s) n += s->num_params(s);
  b->param_cache = (cg_tensor**)std::malloc(sizeof(cg_tensor*) * n);
  b->n_params = 0;
  for (cg_layer* s : subs) if (s) { cg_tensor** ps = s->get_params(s); for (int i = 0; i < s->num_params(s); ++i) b->param_cache[b->n_params++] = ps[i]; }
  b->base.forward = block_forward_default; b->base.backward = block_backward; b->base.free = block_free;
  b->base.num_params = block_np; b->base.get_params = block_gp;
  return b;
}
CG_EXPORT cg_tensor* cg_transformer_forward(cg_layer* layer, cg_tensor* x, cg_tensor* mask) {
  cg_transformer_block* b = (cg_transformer_block*)layer;
  if (!b || !x) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  const cg_transformer_config& c = b->config;
  if (x->ndim != 2 || x->shape[1] != c.hidden_size) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  const int T = x->shape[0];
  if (mask && mask->size != T * T) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  std::vector<cg_tensor*> temps;        // functional results owned here; the tape keeps what it needs
  auto keep = [&](cg_tensor* t) { temps.push_back(t); return t; };
  auto fwd = [&](void* l, cg_tensor* in) { cg_layer* L = (cg_layer*)l; return keep(L->forward(L, in)); };   // sub-layer outputs are ours to release
  cg_tensor* h = c.pre_norm ? fwd(b->norm1, x) : x;
  cg_tensor* q = fwd(b->q_proj, h); cg_tensor* k = fwd(b->k_proj, h); cg_tensor* v = fwd(b->v_proj, h);
  cg_tensor* a = keep(attention_op(q, k, v, mask, c.num_heads, c.num_kv_heads, c.head_dim));
  cg_tensor* o = fwd(b->o_proj, a);
  cg_tensor* x1 = keep(cg_add(x, o));
  if (!c.pre_norm) x1 = fwd(b->norm1, x1);
  cg_tensor* h2 = c.pre_norm ? fwd(b->norm2, x1) : x1;
  cg_tensor* up = fwd(b->up_proj, h2);
  cg_tensor* act;
  if (c.use_swiglu) {
    cg_tensor* gate = fwd(b->gate_proj, h2);
    cg_tensor* pair[2] = {gate, up};
    cg_tensor* cat = keep(cg_tensor_cat(pair, 2, 1));
    // concatenation on the tape: split the gradient back to gate and up
    attach(cat, {gate, up}, [gate, up](cg_tensor* self) {
      const int R = rows_of(gate), I = cols_of(gate);
      for (int r = 0; r < R; ++r) for (int j = 0; j < I; ++j) {
        gate->grad[(size_t)r * I + j] += self->grad[(size_t)r * 2 * I + j];
        up->grad[(size_t)r * I + j] += self->grad[(size_t)r * 2 * I + I + j];
      }
    });
    act = keep(cg_swiglu_forward_split(cat));
  } else act = keep(gelu_op(up));
  cg_tensor* down = fwd(b->down_proj, act);
  cg_tensor* y = cg_add(x1, down);
  if (!c.pre_norm) { temps.push_back(y); y = fwd(b->norm2, y); cg_tensor_retain(y); }   // the caller's reference
  cg_tensor_retain(y);                              // the block's own
  cg_tensor_retain(x);
  if (layer->input) cg_tensor_release(layer->input);
  if (layer->output) cg_tensor_release(layer->output);
  layer->input = x; layer->output = y;
  for (cg_tensor* t : temps) cg_tensor_release(t);
  return y;
}
