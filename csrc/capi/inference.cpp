// Samplers, draft/verify speculative decoding, token trees, tree-attention masks, the
// EAGLE-style tree drafter.  Reference surface: include/cg_speculative.h,
// src/inference/speculative.c.
#include <algorithm>
#include <numeric>

#include "internal.hpp"

using namespace cgi;

namespace {
Rng g_rng(0x5A3Dull);
void softmax_t(const float* logits, int V, float temperature, std::vector<float>& p) {
  p.resize(V);
  const float invT = temperature > 0 ? 1.0f / temperature : 1.0f;
  float m = logits[0];
  for (int i = 1; i < V; ++i) m = logits[i] > m ? logits[i] : m;
  double s = 0;
  for (int i = 0; i < V; ++i) { p[i] = std::exp((logits[i] - m) * invT); s += p[i]; }
  const float inv = (float)(1.0 / s);
  for (int i = 0; i < V; ++i) p[i] *= inv;
}
int sample_from(const float* p, int V, Rng& rng) {
  double total = 0;
  for (int i = 0; i < V; ++i) total += p[i];
  if (!(total > 0)) return 0;
  double u = rng.uniform() * total, acc = 0;
  int last = 0;
  for (int i = 0; i < V; ++i) { if (p[i] <= 0) continue; acc += p[i]; last = i; if (u < acc) return i; }
  return last;
}
int argmax(const float* x, int V) { int b = 0; for (int i = 1; i < V; ++i) if (x[i] > x[b]) b = i; return b; }
// Keeps the smallest set of most probable tokens whose mass reaches top_p (in place, renormalised).
void nucleus(std::vector<float>& p, float top_p) {
  if (top_p <= 0 || top_p >= 1) return;
  std::vector<int> idx(p.size());
  std::iota(idx.begin(), idx.end(), 0);
  std::sort(idx.begin(), idx.end(), [&](int a, int b) { return p[a] > p[b] || (p[a] == p[b] && a < b); });
  double acc = 0; size_t keep = 0;
  while (keep < idx.size()) { acc += p[idx[keep++]]; if (acc >= top_p) break; }
  for (size_t i = keep; i < idx.size(); ++i) p[idx[i]] = 0;
  const float inv = (float)(1.0 / acc);
  for (size_t i = 0; i < keep; ++i) p[idx[i]] *= inv;
}
void keep_top_k(std::vector<float>& p, int k) {
  if (k <= 0 || k >= (int)p.size()) return;
  std::vector<float> s(p);
  std::nth_element(s.begin(), s.begin() + (k - 1), s.end(), std::greater<float>());
  const float cut = s[k - 1];
  int kept = 0; double acc = 0;
  for (size_t i = 0; i < p.size(); ++i) { if (p[i] >= cut && kept < k) { ++kept; acc += p[i]; } else p[i] = 0; }
  const float inv = (float)(1.0 / acc);
  for (auto& v : p) v *= inv;
}
}  // namespace

CG_EXPORT void cg_sample_seed(unsigned int seed) { g_rng = Rng(seed); }
CG_EXPORT int cg_sample_temperature(float* logits, int V, float temperature) {
  if (!logits || V <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  if (temperature <= 0) return argmax(logits, V);
  std::vector<float> p; softmax_t(logits, V, temperature, p);
  return sample_from(p.data(), V, g_rng);
}
CG_EXPORT int cg_sample_top_p(float* logits, int V, float top_p) {
  if (!logits || V <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  std::vector<float> p; softmax_t(logits, V, 1.0f, p);
  nucleus(p, top_p);
  return sample_from(p.data(), V, g_rng);
}
CG_EXPORT int cg_sample_top_k(float* logits, int V, int top_k) {
  if (!logits || V <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  std::vector<float> p; softmax_t(logits, V, 1.0f, p);
  keep_top_k(p, top_k);
  return sample_from(p.data(), V, g_rng);
}
// Locally typical sampling: keep the tokens whose surprisal is closest to the entropy until
// their mass reaches typical_p.
CG_EXPORT int cg_sample_typical(float* logits, int V, float typical_p) {
  if (!logits || V <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  std::vector<float> p; softmax_t(logits, V, 1.0f, p);
  if (typical_p > 0 && typical_p < 1) {
    double H = 0;
    for (int i = 0; i < V; ++i) if (p[i] > 0) H -= p[i] * std::log(p[i]);
    std::vector<int> idx(V);
    std::iota(idx.begin(), idx.end(), 0);
    auto dev = [&](int i) { return p[i] > 0 ? std::fabs(-std::log(p[i]) - H) : 1e30; };
    std::sort(idx.begin(), idx.end(), [&](int a, int b) { const double da = dev(a), db = dev(b); return da < db || (da == db && a < b); });
    double acc = 0; int keep = 0;
    while (keep < V) { acc += p[idx[keep++]]; if (acc >= typical_p) break; }
    for (int i = keep; i < V; ++i) p[idx[i]] = 0;
  }
  return sample_from(p.data(), V, g_rng);
}
CG_EXPORT float cg_acceptance_prob(float draft, float target) {
  if (draft <= 0) return 1.0f;
  const float r = target / draft;
  return r < 1.0f ? (r > 0 ? r : 0.0f) : 1.0f;
}
// Sample from norm(max(0, target - draft)); falls back to target when the residual is empty.
CG_EXPORT int cg_sample_corrected(float* draft, float* target, int V) {
  if (!draft || !target || V <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  std::vector<float> r(V);
  double s = 0;
  for (int i = 0; i < V; ++i) { r[i] = target[i] > draft[i] ? target[i] - draft[i] : 0.0f; s += r[i]; }
  return s > 1e-12 ? sample_from(r.data(), V, g_rng) : sample_from(target, V, g_rng);
}

// -------------------------------------------------------------- token tree
CG_EXPORT cg_token_tree* cg_token_tree_new(int depth) {
  cg_token_tree* t = (cg_token_tree*)std::calloc(1, sizeof(cg_token_tree));
  t->depth = depth > 0 ? depth : 0;
  t->capacity = depth > 0 ? depth : 4;
  t->tokens = (int*)std::calloc(t->capacity, sizeof(int));
  t->parents = (int*)std::calloc(t->capacity, sizeof(int));
  t->probs = (float**)std::calloc(t->capacity, sizeof(float*));
  return t;
}
// parent = -1 hangs the token off the last prefix token.  probs (vocab_size floats) is copied
// when the tree's vocab_size is set.
CG_EXPORT int cg_token_tree_add_child(cg_token_tree* t, int parent, int token, float* probs) {
  if (!t || parent >= t->num_tokens || parent < -1) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  if (t->num_tokens == t->capacity) {
    const int cap = t->capacity * 2;
    t->tokens = (int*)std::realloc(t->tokens, sizeof(int) * cap);
    t->parents = (int*)std::realloc(t->parents, sizeof(int) * cap);
    t->probs = (float**)std::realloc(t->probs, sizeof(float*) * cap);
    for (int i = t->capacity; i < cap; ++i) t->probs[i] = nullptr;
    t->capacity = cap;
  }
  const int id = t->num_tokens++;
  t->tokens[id] = token; t->parents[id] = parent; t->probs[id] = nullptr;
  if (probs && t->vocab_size > 0) { t->probs[id] = (float*)std::malloc(sizeof(float) * t->vocab_size); std::memcpy(t->probs[id], probs, sizeof(float) * t->vocab_size); }
  int d = 1; for (int p = parent; p >= 0; p = t->parents[p]) ++d;
  if (d > t->depth) t->depth = d;
  return id;
}
CG_EXPORT void cg_token_tree_add_token(cg_token_tree* t, int token, float* probs) { if (t) cg_token_tree_add_child(t, t->num_tokens - 1, token, probs); }
CG_EXPORT cg_tensor* cg_token_tree_to_tensor(cg_token_tree* t) {
  if (!t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  int s[1] = {t->num_tokens};
  cg_tensor* o = make(s, 1, false);
  if (o) for (int i = 0; i < t->num_tokens; ++i) o->data[i] = (float)t->tokens[i];
  return o;
}
CG_EXPORT void cg_token_tree_free(cg_token_tree* t) {
  if (!t) return;
  for (int i = 0; i < t->capacity; ++i) std::free(t->probs[i]);
  std::free(t->probs); std::free(t->tokens); std::free(t->parents); std::free(t);
}
// [1, 1, L+g, L+g] additive mask: the prefix is causal; tree token i sees the whole prefix,
// its ancestors and itself.
CG_EXPORT cg_tensor* cg_tree_attention_mask(cg_token_tree* t, int L) {
  if (!t || L < 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  const int g = t->num_tokens, T = L + g;
  int s[4] = {1, 1, T, T};
  cg_tensor* m = cg_tensor_full(s, 4, -1e9f, false);
  if (!m) return nullptr;
  for (int i = 0; i < L; ++i) for (int j = 0; j <= i; ++j) m->data[(size_t)i * T + j] = 0.0f;
  for (int i = 0; i < g; ++i) {
    float* row = m->data + (size_t)(L + i) * T;
    for (int j = 0; j < L; ++j) row[j] = 0.0f;
    for (int a = i; a >= 0; a = t->parents[a]) row[L + a] = 0.0f;
  }
  return m;
}
// `model` is a transformer block (cg_layer*); tree_mask is [1,1,T,T] or [T,T].
CG_EXPORT cg_tensor* cg_forward_tree_attention(void* model, cg_tensor* input, cg_tensor* tree_mask) {
  if (!model || !input) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  return cg_transformer_forward((cg_layer*)model, input, tree_mask);
}

// ---------------------------------------------------------------- decoder
CG_EXPORT cg_speculative_decoder* cg_speculative_decoder_new(void* draft, void* target, int gamma) {
  cg_speculative_decoder* d = (cg_speculative_decoder*)std::calloc(1, sizeof(cg_speculative_decoder));
  d->draft_model = draft; d->target_model = target; d->gamma = gamma > 0 ? gamma : 4;
  d->temperature = 1.0f; d->top_p = 1.0f; d->top_k = 0; d->rng_state = 0x5A3D;
  return d;
}
CG_EXPORT void cg_speculative_set_models(cg_speculative_decoder* d, cg_logits_fn draft_fn, cg_logits_fn target_fn, int V) {
  if (d) { d->draft_fn = draft_fn; d->target_fn = target_fn; d->vocab_size = V; }
}
CG_EXPORT void cg_speculative_decoder_free(cg_speculative_decoder* d) { std::free(d); }

namespace {
// The sampling distribution both models are compared under: temperature, then top-k, then top-p.
void shaped_probs(const cg_speculative_decoder* d, const float* logits, std::vector<float>& p) {
  const int V = d->vocab_size;
  if (d->temperature <= 0) { p.assign(V, 0.0f); p[argmax(logits, V)] = 1.0f; return; }
  softmax_t(logits, V, d->temperature, p);
  keep_top_k(p, d->top_k);
  nucleus(p, d->top_p);
}
std::vector<int> ids_of(cg_tensor* t) { std::vector<int> v(t->size); for (int i = 0; i < t->size; ++i) v[i] = (int)t->data[i]; return v; }
bool ready(cg_speculative_decoder* d) { return d && d->draft_fn && d->target_fn && d->vocab_size > 0; }
}  // namespace

CG_EXPORT cg_token_tree* cg_draft_generate(cg_speculative_decoder* d, cg_tensor* input_ids) {
  if (!ready(d) || !input_ids) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_token_tree*)nullptr);
  const int V = d->vocab_size;
  std::vector<int> ids = ids_of(input_ids);
  cg_token_tree* tree = cg_token_tree_new(d->gamma);
  tree->vocab_size = V;
  std::vector<float> logits(V), p;
  Rng rng(((uint64_t)d->rng_state << 20) ^ 0xD4AF7ull ^ (uint64_t)ids.size());
  for (int i = 0; i < d->gamma; ++i) {
    d->draft_fn(d->draft_model, ids.data(), (int)ids.size(), 1, logits.data());
    shaped_probs(d, logits.data(), p);
    const int tok = sample_from(p.data(), V, rng);
    cg_token_tree_add_token(tree, tok, p.data());
    ids.push_back(tok);
  }
  d->rng_state = d->rng_state * 1664525u + 1013904223u;
  d->total_draft_tokens += d->gamma;
  return tree;
}
// Scores the chain with one target call over gamma+1 positions, accepts each draft token with
// probability min(1, p_target/p_draft), replaces the first rejected one by a sample of the
// residual distribution, or appends a bonus token when all were accepted.  On return the tree
// holds the tokens to append (accepted ones, then the corrected / bonus token).
CG_EXPORT int cg_target_verify(cg_speculative_decoder* d, cg_tensor* input_ids, cg_token_tree* tree) {
  if (!ready(d) || !input_ids || !tree) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  const int V = d->vocab_size, g = tree->num_tokens;
  std::vector<int> ids = ids_of(input_ids);
  for (int i = 0; i < g; ++i) ids.push_back(tree->tokens[i]);
  std::vector<float> logits((size_t)(g + 1) * V), pt;
  d->target_fn(d->target_model, ids.data(), (int)ids.size(), g + 1, logits.data());
  Rng rng(((uint64_t)d->rng_state << 20) ^ 0x7E21Full ^ (uint64_t)ids.size());
  d->rng_state = d->rng_state * 1664525u + 1013904223u;
  int n = 0;
  for (; n < g; ++n) {
    shaped_probs(d, logits.data() + (size_t)n * V, pt);
    const int tok = tree->tokens[n];
    const float pd = tree->probs[n] ? tree->probs[n][tok] : 1.0f;
    if (rng.uniform() < cg_acceptance_prob(pd, pt[tok])) continue;
    // rejected: resample position n from the residual
    std::vector<float> r(V); double s = 0;
    for (int i = 0; i < V; ++i) { const float q = tree->probs[n] ? tree->probs[n][i] : 0.0f; r[i] = pt[i] > q ? pt[i] - q : 0.0f; s += r[i]; }
    tree->tokens[n] = s > 1e-12 ? sample_from(r.data(), V, rng) : sample_from(pt.data(), V, rng);
    tree->num_tokens = n + 1;
    d->accepted_draft_tokens += n;
    return n;
  }
  shaped_probs(d, logits.data() + (size_t)g * V, pt);
  tree->vocab_size = 0;                                   // the bonus token carries no draft distribution
  cg_token_tree_add_token(tree, sample_from(pt.data(), V, rng), nullptr);
  tree->vocab_size = V;
  d->accepted_draft_tokens += g;
  return g;
}
CG_EXPORT int cg_speculative_step(cg_speculative_decoder* d, cg_tensor* input_ids, cg_token_tree* tree) {
  if (!ready(d) || !input_ids) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  cg_token_tree* drafted = cg_draft_generate(d, input_ids);
  if (!drafted) return -1;
  const int n = cg_target_verify(d, input_ids, drafted);
  ++d->num_steps;
  d->avg_acceptance_rate = d->total_draft_tokens ? (float)d->accepted_draft_tokens / d->total_draft_tokens : 0.0f;
  if (tree) {                                             // hand the result to the caller's tree
    for (int i = 0; i < tree->capacity; ++i) { std::free(tree->probs[i]); tree->probs[i] = nullptr; }
    tree->num_tokens = 0; tree->vocab_size = 0;
    for (int i = 0; i < drafted->num_tokens; ++i) cg_token_tree_add_token(tree, drafted->tokens[i], nullptr);
  }
  cg_token_tree_free(drafted);
  return n;
}
CG_EXPORT cg_tensor* cg_speculative_generate(cg_speculative_decoder* d, cg_tensor* input_ids, int max_new, float temperature, float top_p) {
  if (!ready(d) || !input_ids || max_new < 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  d->temperature = temperature; d->top_p = top_p > 0 ? top_p : 1.0f;
  std::vector<int> ids = ids_of(input_ids);
  const size_t start = ids.size();
  cg_token_tree* out = cg_token_tree_new(d->gamma + 1);
  while ((int)(ids.size() - start) < max_new) {
    int s[1] = {(int)ids.size()};
    cg_tensor* cur = make(s, 1, false);
    for (size_t i = 0; i < ids.size(); ++i) cur->data[i] = (float)ids[i];
    const int n = cg_speculative_step(d, cur, out);
    cg_tensor_release(cur);
    if (n < 0) break;
    for (int i = 0; i < out->num_tokens && (int)(ids.size() - start) < max_new; ++i) ids.push_back(out->tokens[i]);
  }
  cg_token_tree_free(out);
  int s[1] = {(int)ids.size()};
  cg_tensor* r = make(s, 1, false);
  if (r) for (size_t i = 0; i < ids.size(); ++i) r->data[i] = (float)ids[i];
  return r;
}

// ------------------------------------------------------------------- EAGLE
// base_draft is a cg_speculative_decoder whose draft model proposes the tokens.
CG_EXPORT cg_eagle_draft* cg_eagle_draft_new(void* base_draft) {
  cg_eagle_draft* e = (cg_eagle_draft*)std::calloc(1, sizeof(cg_eagle_draft));
  e->base_draft = base_draft; e->max_branch = 4;
  return e;
}
CG_EXPORT void cg_eagle_draft_free(cg_eagle_draft* e) { if (e) { std::free(e->branching); std::free(e); } }
// features: [depth, vocab] (or [vocab]) probability rows; the branching factor of a level is
// the number of tokens needed to cover 80 % of its mass, between 1 and max_branch.
CG_EXPORT int* cg_eagle_compute_branching(cg_eagle_draft* e, cg_tensor* features) {
  if (!e || !features) return fail(CG_ERROR_NULL_POINTER, (int*)nullptr);
  const int V = cols_of(features), depth = rows_of(features);
  std::free(e->branching);
  e->branching = (int*)std::malloc(sizeof(int) * (depth ? depth : 1));
  for (int r = 0; r < depth; ++r) {
    std::vector<float> p(features->data + (size_t)r * V, features->data + (size_t)(r + 1) * V);
    std::sort(p.begin(), p.end(), std::greater<float>());
    double total = 0; for (float v : p) total += v;
    double acc = 0; int k = 0;
    while (k < V && k < e->max_branch) { acc += p[k++]; if (acc >= 0.8 * total) break; }
    e->branching[r] = k < 1 ? 1 : k;
  }
  return e->branching;
}
// Level by level: the most probable node of a level is expanded, its top-b tokens become the
// next level (b from the entropy rule above); the other nodes stay as alternative leaves.
CG_EXPORT cg_token_tree* cg_eagle_generate_tree(cg_eagle_draft* e, cg_tensor* input, int max_depth) {
  cg_speculative_decoder* d = e ? (cg_speculative_decoder*)e->base_draft : nullptr;
  if (!d || !d->draft_fn || d->vocab_size <= 0 || !input || max_depth <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_token_tree*)nullptr);
  const int V = d->vocab_size;
  std::vector<int> ids = ids_of(input);
  cg_token_tree* tree = cg_token_tree_new(max_depth);
  tree->vocab_size = V;
  std::vector<float> logits(V), p;
  int parent = -1;
  for (int level = 0; level < max_depth; ++level) {
    d->draft_fn(d->draft_model, ids.data(), (int)ids.size(), 1, logits.data());
    softmax_t(logits.data(), V, d->temperature > 0 ? d->temperature : 1.0f, p);
    int s[2] = {1, V};
    cg_tensor* f = cg_tensor_from_data(p.data(), s, 2, false);
    const int b = cg_eagle_compute_branching(e, f)[0];
    cg_tensor_release(f);
    std::vector<int> idx(V);
    std::iota(idx.begin(), idx.end(), 0);
    std::partial_sort(idx.begin(), idx.begin() + b, idx.end(), [&](int a, int c) { return p[a] > p[c] || (p[a] == p[c] && a < c); });
    int first = -1;
    for (int k = 0; k < b; ++k) { const int id = cg_token_tree_add_child(tree, parent, idx[k], p.data()); if (k == 0) first = id; }
    parent = first;
    ids.push_back(idx[0]);
  }
  return tree;
}
