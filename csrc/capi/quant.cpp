// 4-bit quantisation: INT4 / NF4 / GPTQ / AWQ weights, dequant matmul / gemv, the INT4
// KV cache with attention over it, activation calibration.
// Reference surface: include/cg_quantize.h, src/quantize/int4.c.
// Packed format (bit-exact with the reference): symmetric, groups of `group_size`
// consecutive elements of the row-major tensor, scale = absmax/7 (1 when < 1e-10),
// q = clamp(round(x/scale), -8, 7), two values per byte with the even index in the low nibble.
#include "internal.hpp"

using namespace cgi;

namespace {
const float kNF4[16] = {-1.0f, -0.6961928f, -0.5250730f, -0.3949175f, -0.2844414f, -0.1848449f, -0.0910500f, 0.0f,
                        0.0795803f, 0.1609302f, 0.2461123f, 0.3379152f, 0.4407098f, 0.5626170f, 0.7229568f, 1.0f};
inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
inline void put_nibble(uint8_t* d, size_t i, int q) {
  uint8_t& b = d[i >> 1];
  b = (i & 1) ? (uint8_t)((b & 0x0f) | ((q & 0xf) << 4)) : (uint8_t)((b & 0xf0) | (q & 0xf));
}
inline int get_nibble_s(const uint8_t* d, size_t i) { int v = (i & 1) ? d[i >> 1] >> 4 : d[i >> 1] & 0xf; return v >= 8 ? v - 16 : v; }
inline int get_nibble_u(const uint8_t* d, size_t i) { return (i & 1) ? d[i >> 1] >> 4 : d[i >> 1] & 0xf; }
inline float group_scale(const float* x, int n) {
  float m = 0; for (int i = 0; i < n; ++i) { const float a = std::fabs(x[i]); m = a > m ? a : m; }
  return m < 1e-10f ? 1.0f : m / 7.0f;
}
cg_tensor_quant* new_quant(const cg_tensor* t, int group, cg_quant_type type, int extra_scales) {
  if (!t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor_quant*)nullptr);
  if (group <= 0) group = 128;
  cg_tensor_quant* q = (cg_tensor_quant*)std::calloc(1, sizeof(cg_tensor_quant));
  q->ndim = t->ndim; q->size = t->size; q->quant_type = type; q->group_size = group; q->symmetric = true;
  q->num_groups = (t->size + group - 1) / group;
  q->shape = (int*)std::malloc(sizeof(int) * (t->ndim ? t->ndim : 1));
  for (int i = 0; i < t->ndim; ++i) q->shape[i] = t->shape[i];
  q->data = (uint8_t*)std::calloc((t->size + 1) / 2 + 1, 1);
  q->scales = (float*)std::calloc(q->num_groups + extra_scales + 1, sizeof(float));
  q->zeros = (float*)std::calloc(q->num_groups + 1, sizeof(float));
  return q;
}
void quantize_groups(const float* x, cg_tensor_quant* q) {
  for (int g = 0; g < q->num_groups; ++g) {
    const int lo = g * q->group_size, n = q->size - lo < q->group_size ? q->size - lo : q->group_size;
    const float s = group_scale(x + lo, n);
    q->scales[g] = s;
    for (int i = 0; i < n; ++i) put_nibble(q->data, lo + i, clampi((int)std::round(x[lo + i] / s), -8, 7));
  }
}
// dst[0..n) = dequantised elements [start, start+n)
void dequant_range(const cg_tensor_quant* q, size_t start, int n, float* dst) {
  const int cols = q->ndim ? q->shape[q->ndim - 1] : 1;
  for (int i = 0; i < n; ++i) {
    const size_t e = start + i;
    const float s = q->scales[e / q->group_size];
    float v;
    if (q->quant_type == QUANT_NF4) v = kNF4[get_nibble_u(q->data, e)] * s;
    else if (!q->symmetric) v = (get_nibble_u(q->data, e) - q->zeros[e / q->group_size]) * s;
    else v = get_nibble_s(q->data, e) * s;
    if (q->quant_type == QUANT_AWQ) v /= q->scales[q->num_groups + (int)(e % cols)];
    dst[i] = v;
  }
}
}  // namespace

CG_EXPORT cg_tensor_quant* cg_quantize_int4(cg_tensor* t, int group) {
  cg_tensor_quant* q = new_quant(t, group, QUANT_INT4, 0);
  if (q) quantize_groups(t->data, q);
  return q;
}
CG_EXPORT cg_tensor_quant* cg_quantize_nf4(cg_tensor* t, int group) {
  cg_tensor_quant* q = new_quant(t, group, QUANT_NF4, 0);
  if (!q) return nullptr;
  for (int g = 0; g < q->num_groups; ++g) {
    const int lo = g * q->group_size, n = q->size - lo < q->group_size ? q->size - lo : q->group_size;
    float m = 0; for (int i = 0; i < n; ++i) { const float a = std::fabs(t->data[lo + i]); m = a > m ? a : m; }
    const float s = m < 1e-10f ? 1.0f : m;
    q->scales[g] = s;
    for (int i = 0; i < n; ++i) {
      const float v = t->data[lo + i] / s;
      int best = 0;
      for (int c = 1; c < 16; ++c) if (std::fabs(kNF4[c] - v) < std::fabs(kNF4[best] - v)) best = c;
      put_nibble(q->data, lo + i, best);
    }
  }
  return q;
}

// GPTQ on a [R, C] weight with the [C, C] Hessian of its inputs: columns are quantised in
// order and the rounding error of each is pushed onto the not-yet-quantised columns through
// the upper Cholesky factor of H^-1.  Without a Hessian this is plain group quantisation.
CG_EXPORT cg_tensor_quant* cg_quantize_gptq(cg_tensor* t, cg_tensor* hessian, int group, int bits) {
  if (!t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor_quant*)nullptr);
  if (bits <= 0) bits = 4;
  if (bits < 2 || bits > 4) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor_quant*)nullptr);
  cg_tensor_quant* q = new_quant(t, group, QUANT_GPTQ, 0);
  if (!q) return nullptr;
  const int C = cols_of(t), R = rows_of(t);
  if (!hessian || hessian->size != C * C || C % q->group_size != 0 || bits != 4) {
    if (bits == 4) { quantize_groups(t->data, q); return q; }
    const int qmax = (1 << (bits - 1)) - 1;
    for (int g = 0; g < q->num_groups; ++g) {
      const int lo = g * q->group_size, n = q->size - lo < q->group_size ? q->size - lo : q->group_size;
      float m = 0; for (int i = 0; i < n; ++i) { const float a = std::fabs(t->data[lo + i]); m = a > m ? a : m; }
      const float s = m < 1e-10f ? 1.0f : m / qmax;
      q->scales[g] = s;
      for (int i = 0; i < n; ++i) put_nibble(q->data, lo + i, clampi((int)std::round(t->data[lo + i] / s), -qmax - 1, qmax));
    }
    return q;
  }
  // H + damping, inverse by Cholesky, then the upper Cholesky factor U of the inverse (Hinv = U^T U)
  std::vector<double> H(hessian->data, hessian->data + (size_t)C * C), L((size_t)C * C, 0.0), Hinv((size_t)C * C, 0.0), U((size_t)C * C, 0.0);
  double mean_diag = 0; for (int i = 0; i < C; ++i) mean_diag += H[(size_t)i * C + i];
  mean_diag = mean_diag / C; if (mean_diag <= 0) mean_diag = 1.0;
  for (int i = 0; i < C; ++i) H[(size_t)i * C + i] += 0.01 * mean_diag;
  auto cholesky = [C](const std::vector<double>& A, std::vector<double>& Lo) {
    for (int i = 0; i < C; ++i) for (int j = 0; j <= i; ++j) {
      double s = A[(size_t)i * C + j];
      for (int k = 0; k < j; ++k) s -= Lo[(size_t)i * C + k] * Lo[(size_t)j * C + k];
      if (i == j) { if (s <= 1e-12) return false; Lo[(size_t)i * C + i] = std::sqrt(s); }
      else Lo[(size_t)i * C + j] = s / Lo[(size_t)j * C + j];
    }
    return true;
  };
  bool ok = cholesky(H, L);
  if (ok) {
    for (int c = 0; c < C; ++c) {                    // solve H x = e_c
      std::vector<double> y(C, 0.0);
      for (int i = 0; i < C; ++i) { double s = i == c ? 1.0 : 0.0; for (int k = 0; k < i; ++k) s -= L[(size_t)i * C + k] * y[k]; y[i] = s / L[(size_t)i * C + i]; }
      for (int i = C - 1; i >= 0; --i) { double s = y[i]; for (int k = i + 1; k < C; ++k) s -= L[(size_t)k * C + i] * Hinv[(size_t)k * C + c]; Hinv[(size_t)i * C + c] = s / L[(size_t)i * C + i]; }
    }
    // upper factor: reverse-order Cholesky so that Hinv = U^T U with U upper triangular
    std::vector<double> Lr((size_t)C * C, 0.0);
    ok = cholesky(Hinv, Lr);
    if (ok) for (int i = 0; i < C; ++i) for (int j = i; j < C; ++j) U[(size_t)i * C + j] = Lr[(size_t)j * C + i];
  }
  if (!ok) { quantize_groups(t->data, q); return q; }
  std::vector<float> W(t->data, t->data + t->size);
  for (int j = 0; j < C; ++j) {
    if (j % q->group_size == 0)
      for (int r = 0; r < R; ++r) q->scales[((size_t)r * C + j) / q->group_size] = group_scale(&W[(size_t)r * C + j], q->group_size);
    const double d = U[(size_t)j * C + j];
    for (int r = 0; r < R; ++r) {
      const size_t e = (size_t)r * C + j;
      const float s = q->scales[e / q->group_size];
      const int qi = clampi((int)std::round(W[e] / s), -8, 7);
      put_nibble(q->data, e, qi);
      const double err = (W[e] - qi * s) / d;
      for (int k = j + 1; k < C; ++k) W[(size_t)r * C + k] -= (float)(err * U[(size_t)j * C + k]);
    }
  }
  return q;
}

// AWQ on a [R, C] weight: per-input-channel scales s_c = mean|act_c|^alpha protect the
// channels that see large activations; alpha is chosen on a grid to minimise the
// activation-weighted reconstruction error.  The channel scales are stored after the group
// scales (scales[num_groups + c]) and divided out again on dequantisation.
CG_EXPORT cg_tensor_quant* cg_quantize_awq(cg_tensor* t, cg_tensor* act, int group) {
  if (!t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor_quant*)nullptr);
  const int C = cols_of(t);
  cg_tensor_quant* q = new_quant(t, group, QUANT_AWQ, C);
  if (!q) return nullptr;
  std::vector<float> mag(C, 1.0f);
  if (act && cols_of(act) == C && act->size >= C) {
    const int S = act->size / C;
    for (int c = 0; c < C; ++c) { double s = 0; for (int r = 0; r < S; ++r) s += std::fabs(act->data[(size_t)r * C + c]); mag[c] = (float)(s / S) + 1e-8f; }
  }
  std::vector<float> scaled(t->size), deq(t->size), best_s(C, 1.0f);
  double best_err = -1;
  std::vector<uint8_t> best_data; std::vector<float> best_scales;
  for (int a = 0; a <= 4; ++a) {
    const float alpha = 0.25f * a;
    std::vector<float> s(C);
    double gm = 0;
    for (int c = 0; c < C; ++c) { s[c] = std::pow(mag[c], alpha); gm += std::log(s[c]); }
    const float norm = (float)std::exp(gm / C);
    for (int c = 0; c < C; ++c) s[c] /= norm;
    for (int i = 0; i < t->size; ++i) scaled[i] = t->data[i] * s[i % C];
    quantize_groups(scaled.data(), q);
    double err = 0;
    for (int i = 0; i < t->size; ++i) {
      const float v = get_nibble_s(q->data, i) * q->scales[i / q->group_size] / s[i % C];
      const double d = (double)(v - t->data[i]) * mag[i % C];
      err += d * d;
    }
    if (best_err < 0 || err < best_err) {
      best_err = err; best_s = s;
      best_data.assign(q->data, q->data + (t->size + 1) / 2);
      best_scales.assign(q->scales, q->scales + q->num_groups);
    }
  }
  std::memcpy(q->data, best_data.data(), best_data.size());
  std::memcpy(q->scales, best_scales.data(), sizeof(float) * q->num_groups);
  for (int c = 0; c < C; ++c) q->scales[q->num_groups + c] = best_s[c];
  return q;
}

CG_EXPORT cg_tensor* cg_dequantize(cg_tensor_quant* q) {
  if (!q) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* t = make(q->shape, q->ndim, false);
  if (t) dequant_range(q, 0, q->size, t->data);
  return t;
}
CG_EXPORT void cg_tensor_quant_free(cg_tensor_quant* q) {
  if (!q) return;
  std::free(q->data); std::free(q->scales); std::free(q->zeros); std::free(q->shape); std::free(q);
}
// input [M, K] x weight [K, N] -> output [M, N]; one weight row is dequantised at a time
CG_EXPORT void cg_matmul_int4(cg_tensor* x, cg_tensor_quant* w, cg_tensor* out) {
  if (!x || !w || !out) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (w->ndim != 2) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int K = w->shape[0], N = w->shape[1];
  if (cols_of(x) != K || out->size != rows_of(x) * N) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int M = rows_of(x);
  std::memset(out->data, 0, sizeof(float) * out->size);
  std::vector<float> row(N);
  for (int k = 0; k < K; ++k) {
    dequant_range(w, (size_t)k * N, N, row.data());
    for (int m = 0; m < M; ++m) {
      const float a = x->data[(size_t)m * K + k];
      if (a == 0.0f) continue;
      float* o = out->data + (size_t)m * N;
      for (int n = 0; n < N; ++n) o[n] += a * row[n];
    }
  }
}
CG_EXPORT void cg_gemv_int4(cg_tensor* x, cg_tensor_quant* w, cg_tensor* out) {
  if (!x || !w || !out) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (w->ndim != 2 || x->size != w->shape[0] || out->size != w->shape[1]) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  int xs[2] = {1, x->size};
  cg_tensor view = *x;
  view.ndim = 2; view.shape[0] = xs[0]; view.shape[1] = xs[1];
  cg_matmul_int4(&view, w, out);
}

// ---------------------------------------------------------------- KV cache
// k_cache / v_cache: [layers, max_seq, heads, head_dim/2] bytes; scales
// [layers, max_seq, heads, head_dim/group] fp32.
CG_EXPORT cg_kv_cache_int4* cg_kv_cache_int4_new(int layers, int max_seq, int heads, int head_dim, int group) {
  if (layers <= 0 || max_seq <= 0 || heads <= 0 || head_dim <= 0 || head_dim % 2) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_kv_cache_int4*)nullptr);
  if (group <= 0 || group > head_dim) group = head_dim;
  if (head_dim % group) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_kv_cache_int4*)nullptr);
  cg_kv_cache_int4* c = (cg_kv_cache_int4*)std::calloc(1, sizeof(cg_kv_cache_int4));
  c->num_layers = layers; c->max_seq_len = max_seq; c->n_heads = heads; c->head_dim = head_dim; c->group_size = group;
  const size_t bytes = (size_t)layers * max_seq * heads * head_dim / 2, ns = (size_t)layers * max_seq * heads * (head_dim / group);
  c->k_cache = (uint8_t*)std::calloc(bytes, 1); c->v_cache = (uint8_t*)std::calloc(bytes, 1);
  c->k_scales = (float*)std::calloc(ns, sizeof(float)); c->v_scales = (float*)std::calloc(ns, sizeof(float));
  if (!c->k_cache || !c->v_cache || !c->k_scales || !c->v_scales) { cg_kv_cache_int4_free(c); return fail(CG_ERROR_OUT_OF_MEMORY, (cg_kv_cache_int4*)nullptr); }
  return c;
}
static void quantize_token(const float* src, int heads, int D, int group, uint8_t* bytes, float* scales) {
  const int G = D / group;
  for (int h = 0; h < heads; ++h) for (int g = 0; g < G; ++g) {
    const float* x = src + (size_t)h * D + g * group;
    const float s = group_scale(x, group);
    scales[h * G + g] = s;
    for (int i = 0; i < group; ++i) put_nibble(bytes, (size_t)h * D + g * group + i, clampi((int)std::round(x[i] / s), -8, 7));
  }
}
// new_k / new_v hold T >= 1 tokens of [heads * head_dim].  Layer 0 advances the length;
// the other layers write the same T positions.
CG_EXPORT void cg_kv_cache_int4_append(cg_kv_cache_int4* c, int layer, cg_tensor* nk, cg_tensor* nv) {
  if (!c || !nk || !nv) { set_error(CG_ERROR_NULL_POINTER); return; }
  const int HD = c->n_heads * c->head_dim, G = c->head_dim / c->group_size;
  if (layer < 0 || layer >= c->num_layers || nk->size % HD || nk->size != nv->size || nk->size == 0) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  const int T = nk->size / HD;
  int pos;
  if (layer == 0) { pos = c->current_len; if (pos + T > c->max_seq_len) { set_error(CG_ERROR_OUT_OF_MEMORY); return; } c->current_len += T; }
  else { pos = c->current_len - T; if (pos < 0) { set_error(CG_ERROR_INVALID_ARGUMENT); return; } }
  for (int t = 0; t < T; ++t) {
    const size_t tok = (size_t)layer * c->max_seq_len + pos + t;
    quantize_token(nk->data + (size_t)t * HD, c->n_heads, c->head_dim, c->group_size, c->k_cache + tok * HD / 2, c->k_scales + tok * c->n_heads * G);
    quantize_token(nv->data + (size_t)t * HD, c->n_heads, c->head_dim, c->group_size, c->v_cache + tok * HD / 2, c->v_scales + tok * c->n_heads * G);
  }
}
static void dequant_token(const cg_kv_cache_int4* c, const uint8_t* bytes, const float* scales, float* dst) {
  const int D = c->head_dim, G = D / c->group_size;
  for (int h = 0; h < c->n_heads; ++h) for (int d = 0; d < D; ++d)
    dst[(size_t)h * D + d] = get_nibble_s(bytes, (size_t)h * D + d) * scales[h * G + d / c->group_size];
}
CG_EXPORT void cg_kv_cache_int4_get(cg_kv_cache_int4* c, int layer, cg_tensor* k_out, cg_tensor* v_out) {
  if (!c || !k_out || !v_out) { set_error(CG_ERROR_NULL_POINTER); return; }
  const int HD = c->n_heads * c->head_dim, G = c->head_dim / c->group_size;
  if (layer < 0 || layer >= c->num_layers || k_out->size < c->current_len * HD || v_out->size < c->current_len * HD) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  for (int t = 0; t < c->current_len; ++t) {
    const size_t tok = (size_t)layer * c->max_seq_len + t;
    dequant_token(c, c->k_cache + tok * HD / 2, c->k_scales + tok * c->n_heads * G, k_out->data + (size_t)t * HD);
    dequant_token(c, c->v_cache + tok * HD / 2, c->v_scales + tok * c->n_heads * G, v_out->data + (size_t)t * HD);
  }
}
CG_EXPORT void cg_kv_cache_int4_reset(cg_kv_cache_int4* c) { if (c) c->current_len = 0; }
// Drop the newest positions (rejected speculative tokens).
CG_EXPORT void cg_kv_cache_int4_truncate(cg_kv_cache_int4* c, int new_len) { if (c && new_len >= 0 && new_len <= c->current_len) c->current_len = new_len; }
CG_EXPORT void cg_kv_cache_int4_free(cg_kv_cache_int4* c) {
  if (!c) return;
  std::free(c->k_cache); std::free(c->v_cache); std::free(c->k_scales); std::free(c->v_scales); std::free(c);
}
// Q holds the Tq newest positions, [Tq, Hq * head_dim] (Hq a multiple of the cache's heads:
// grouped-query attention).  Query i sees keys 0 .. len - Tq + i.  One streaming pass per
// (query, head) with an online softmax; keys and values are dequantised one token at a time.
CG_EXPORT void cg_attention_int4_kv(cg_tensor* Q, cg_kv_cache_int4* c, int layer, cg_tensor* out) {
  if (!Q || !c || !out) { set_error(CG_ERROR_NULL_POINTER); return; }
  const int D = c->head_dim, Hk = c->n_heads, G = D / c->group_size, L = c->current_len;
  const int Tq = Q->ndim >= 2 ? Q->shape[0] : 1;
  if (layer < 0 || layer >= c->num_layers || Q->size % (Tq * D) || out->size != Q->size || Tq > L) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  const int Hq = Q->size / (Tq * D);
  if (Hq % Hk) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int rep = Hq / Hk;
  const float scale = 1.0f / std::sqrt((float)D);
  std::vector<float> kf((size_t)Hk * D), vf((size_t)Hk * D), m((size_t)Tq * Hq, -INFINITY), l((size_t)Tq * Hq, 0.0f);
  std::memset(out->data, 0, sizeof(float) * out->size);
  for (int t = 0; t < L; ++t) {
    const size_t tok = (size_t)layer * c->max_seq_len + t;
    dequant_token(c, c->k_cache + tok * Hk * D / 2, c->k_scales + tok * Hk * G, kf.data());
    dequant_token(c, c->v_cache + tok * Hk * D / 2, c->v_scales + tok * Hk * G, vf.data());
    for (int i = 0; i < Tq; ++i) {
      if (t > L - Tq + i) continue;
      for (int h = 0; h < Hq; ++h) {
        const float* q = Q->data + ((size_t)i * Hq + h) * D; const float* k = kf.data() + (size_t)(h / rep) * D; const float* v = vf.data() + (size_t)(h / rep) * D;
        float s = 0; for (int d = 0; d < D; ++d) s += q[d] * k[d];
        s *= scale;
        float& mi = m[(size_t)i * Hq + h]; float& li = l[(size_t)i * Hq + h];
        float* o = out->data + ((size_t)i * Hq + h) * D;
        const float mn = s > mi ? s : mi, corr = std::exp(mi - mn), p = std::exp(s - mn);
        for (int d = 0; d < D; ++d) o[d] = o[d] * corr + p * v[d];
        li = li * corr + p; mi = mn;
      }
    }
  }
  for (int i = 0; i < Tq * Hq; ++i) { const float inv = l[i] > 0 ? 1.0f / l[i] : 0.0f; for (int d = 0; d < D; ++d) out->data[(size_t)i * D + d] *= inv; }
}

// ------------------------------------------------------------- calibration
CG_EXPORT cg_quant_calibration* cg_calibration_new(int channels) {
  if (channels <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_quant_calibration*)nullptr);
  cg_quant_calibration* c = (cg_quant_calibration*)std::calloc(1, sizeof(cg_quant_calibration));
  c->channels = channels;
  c->min_vals = (float*)std::malloc(sizeof(float) * channels); c->max_vals = (float*)std::malloc(sizeof(float) * channels);
  c->abs_max = (float*)std::calloc(channels, sizeof(float));
  for (int i = 0; i < channels; ++i) { c->min_vals[i] = INFINITY; c->max_vals[i] = -INFINITY; }
  return c;
}
CG_EXPORT void cg_calibration_update(cg_quant_calibration* c, cg_tensor* act) {
  if (!c || !act) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (act->size % c->channels) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int R = act->size / c->channels;
  for (int r = 0; r < R; ++r) for (int j = 0; j < c->channels; ++j) {
    const float v = act->data[(size_t)r * c->channels + j];
    if (v < c->min_vals[j]) c->min_vals[j] = v;
    if (v > c->max_vals[j]) c->max_vals[j] = v;
    if (std::fabs(v) > c->abs_max[j]) c->abs_max[j] = std::fabs(v);
  }
  c->num_samples += R;
}
// Asymmetric 4-bit parameters per group of `group_size` channels: x ~ (q - zero) * scale, q in [0, 15].
CG_EXPORT void cg_calibration_compute_scales(cg_quant_calibration* c, float* scales, float* zeros, int group) {
  if (!c || !scales) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (group <= 0) group = 1;
  const int G = (c->channels + group - 1) / group;
  for (int g = 0; g < G; ++g) {
    float lo = INFINITY, hi = -INFINITY;
    for (int j = g * group; j < c->channels && j < (g + 1) * group; ++j) { lo = c->min_vals[j] < lo ? c->min_vals[j] : lo; hi = c->max_vals[j] > hi ? c->max_vals[j] : hi; }
    if (!(hi >= lo)) { lo = 0; hi = 0; }
    if (lo > 0) lo = 0;
    if (hi < 0) hi = 0;
    const float s = hi - lo < 1e-10f ? 1.0f : (hi - lo) / 15.0f;
    scales[g] = s;
    if (zeros) zeros[g] = std::round(-lo / s);
  }
}
CG_EXPORT void cg_calibration_free(cg_quant_calibration* c) {
  if (!c) return;
  std::free(c->min_vals); std::free(c->max_vals); std::free(c->abs_max); std::free(c);
}
