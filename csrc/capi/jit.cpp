// JIT intermediate representation: tracing of the eager tensor ops, graph construction,
// dead-code elimination, common-subexpression elimination, fusion marks and an interpreter.
// Reference surface: include/cg_jit.h, src/jit/graph_capture.c.
#include <map>
#include <set>
#include <string>

#include "internal.hpp"
#include "jit_internal.hpp"

using namespace cgi;

namespace {
cg_ir_graph* g_trace = nullptr;
const char* kNames[] = {"noop", "add", "sub", "mul", "div", "neg", "exp", "log", "sqrt", "rsqrt", "relu", "sigmoid", "tanh", "gelu",
                        "softmax", "matmul", "transpose", "conv2d", "maxpool2d", "sum", "mean", "max", "min", "copy", "reshape", "broadcast",
                        "fused_attention", "fused_layernorm", "fused_layernorm_gelu_linear", "fused_softmax_dropout_residual", "fused_qkv_rope", "custom"};
static_assert(sizeof(kNames) / sizeof(kNames[0]) == OP_CUSTOM + 1, "one name per opcode");
}  // namespace

namespace cgjit {
bool is_elementwise(cg_ir_opcode op) { return (op >= OP_ADD && op <= OP_GELU) || op == OP_COPY; }
bool is_binary(cg_ir_opcode op) { return op >= OP_ADD && op <= OP_DIV; }
bool is_reduction(cg_ir_opcode op) { return op >= OP_SUM && op <= OP_MIN; }
int tensor_size(const cg_ir_graph* g, int id) { return id >= 0 && id < g->num_tensors && g->tensors[id] ? g->tensors[id]->size : 0; }
std::vector<std::vector<int>> consumers(const cg_ir_graph* g) {
  std::vector<std::vector<int>> c(g->num_tensors);
  for (int i = 0; i < g->num_nodes; ++i) {
    const cg_ir_node* n = g->nodes[i];
    if (n->dead) continue;
    for (int k = 0; k < n->num_inputs; ++k) if (n->input_ids[k] >= 0 && n->input_ids[k] < g->num_tensors) c[n->input_ids[k]].push_back(i);
  }
  return c;
}
bool is_graph_output(const cg_ir_graph* g, int tensor_id) {
  for (int i = 0; i < g->num_outputs; ++i) if (g->output_node_ids[i] == tensor_id) return true;
  return false;
}
}  // namespace cgjit
using namespace cgjit;

CG_EXPORT const char* cg_ir_opcode_name(cg_ir_opcode op) { return op >= 0 && op <= OP_CUSTOM ? kNames[op] : "invalid"; }
CG_EXPORT cg_ir_graph* cg_ir_graph_new(void) { return (cg_ir_graph*)std::calloc(1, sizeof(cg_ir_graph)); }
CG_EXPORT cg_ir_node* cg_ir_node_new(cg_ir_opcode op) {
  cg_ir_node* n = (cg_ir_node*)std::calloc(1, sizeof(cg_ir_node));
  n->opcode = op; n->id = -1; n->output_id = -1;
  return n;
}
CG_EXPORT void cg_ir_node_free(cg_ir_node* n) { if (n) { std::free(n->input_ids); std::free(n->attributes); std::free(n); } }
CG_EXPORT void cg_ir_graph_free(cg_ir_graph* g) {
  if (!g) return;
  for (int i = 0; i < g->num_nodes; ++i) cg_ir_node_free(g->nodes[i]);
  for (int i = 0; i < g->num_tensors; ++i) if (g->tensors[i]) cg_tensor_release(g->tensors[i]);
  std::free(g->nodes); std::free(g->tensors); std::free(g->input_node_ids); std::free(g->output_node_ids); std::free(g);
}
CG_EXPORT int cg_ir_graph_tensor_id(cg_ir_graph* g, cg_tensor* t) {
  if (!g || !t) return fail(CG_ERROR_NULL_POINTER, -1);
  for (int i = 0; i < g->num_tensors; ++i) if (g->tensors[i] == t) return i;
  if (g->num_tensors == g->tensor_capacity) {
    g->tensor_capacity = g->tensor_capacity ? g->tensor_capacity * 2 : 16;
    g->tensors = (cg_tensor**)std::realloc(g->tensors, sizeof(cg_tensor*) * g->tensor_capacity);
  }
  cg_tensor_retain(t);
  g->tensors[g->num_tensors] = t;
  return g->num_tensors++;
}
CG_EXPORT cg_ir_node* cg_ir_graph_add_node(cg_ir_graph* g, cg_ir_opcode op, const int* in, int n_in, int out, const void* attr, size_t attr_size) {
  if (!g || n_in < 0 || (n_in && !in)) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_ir_node*)nullptr);
  cg_ir_node* n = cg_ir_node_new(op);
  n->id = g->num_nodes; n->schedule_order = g->num_nodes;
  n->input_ids = (int*)std::malloc(sizeof(int) * (n_in ? n_in : 1));
  for (int i = 0; i < n_in; ++i) n->input_ids[i] = in[i];
  n->num_inputs = n_in; n->output_id = out;
  if (out >= 0 && out < g->num_tensors) { n->output_ndim = g->tensors[out]->ndim; for (int i = 0; i < n->output_ndim; ++i) n->output_shape[i] = g->tensors[out]->shape[i]; }
  if (attr && attr_size) { n->attributes = std::malloc(attr_size); std::memcpy(n->attributes, attr, attr_size); n->attr_size = attr_size; }
  if (g->num_nodes == g->capacity) { g->capacity = g->capacity ? g->capacity * 2 : 16; g->nodes = (cg_ir_node**)std::realloc(g->nodes, sizeof(cg_ir_node*) * g->capacity); }
  g->nodes[g->num_nodes++] = n;
  return n;
}
CG_EXPORT void cg_ir_graph_mark_output(cg_ir_graph* g, cg_tensor* t) {
  if (!g || !t) return;
  const int id = cg_ir_graph_tensor_id(g, t);
  if (is_graph_output(g, id)) return;
  g->output_node_ids = (int*)std::realloc(g->output_node_ids, sizeof(int) * (g->num_outputs + 1));
  g->output_node_ids[g->num_outputs++] = id;
}
CG_EXPORT int cg_ir_graph_live_nodes(cg_ir_graph* g) { int n = 0; if (g) for (int i = 0; i < g->num_nodes; ++i) n += !g->nodes[i]->dead; return n; }

// ----------------------------------------------------------------- tracing
CG_EXPORT void cg_jit_begin_trace(void) { if (g_trace) cg_ir_graph_free(g_trace); g_trace = cg_ir_graph_new(); }
CG_EXPORT bool cg_jit_is_tracing(void) { return g_trace != nullptr; }
CG_EXPORT void cg_jit_record(cg_ir_opcode op, cg_tensor** inputs, int n_in, cg_tensor* output, const void* attr, size_t attr_size) {
  if (!g_trace || !output) return;
  std::vector<int> ids(n_in);
  for (int i = 0; i < n_in; ++i) ids[i] = cg_ir_graph_tensor_id(g_trace, inputs[i]);
  cg_ir_graph_add_node(g_trace, op, ids.data(), n_in, cg_ir_graph_tensor_id(g_trace, output), attr, attr_size);
}
static void find_inputs(cg_ir_graph* g) {
  std::set<int> produced, ins;
  for (int i = 0; i < g->num_nodes; ++i) if (!g->nodes[i]->dead) produced.insert(g->nodes[i]->output_id);
  for (int i = 0; i < g->num_nodes; ++i) if (!g->nodes[i]->dead) for (int k = 0; k < g->nodes[i]->num_inputs; ++k) if (!produced.count(g->nodes[i]->input_ids[k])) ins.insert(g->nodes[i]->input_ids[k]);
  std::free(g->input_node_ids);
  g->input_node_ids = (int*)std::malloc(sizeof(int) * (ins.size() ? ins.size() : 1));
  g->num_inputs = 0;
  for (int id : ins) g->input_node_ids[g->num_inputs++] = id;
}
// Results nobody consumed inside the trace become the graph outputs unless some were marked.
CG_EXPORT cg_ir_graph* cg_jit_end_trace(void) {
  cg_ir_graph* g = g_trace;
  g_trace = nullptr;
  if (!g) return nullptr;
  find_inputs(g);
  if (g->num_outputs == 0) {
    auto cons = consumers(g);
    for (int i = 0; i < g->num_nodes; ++i) { const int o = g->nodes[i]->output_id; if (cons[o].empty()) cg_ir_graph_mark_output(g, g->tensors[o]); }
  }
  return g;
}

// ------------------------------------------------------------------ passes
CG_EXPORT void cg_ir_dce(cg_ir_graph* g) {
  if (!g) return;
  std::map<int, int> producer;                       // tensor id -> last live node writing it
  for (int i = 0; i < g->num_nodes; ++i) if (!g->nodes[i]->dead) producer[g->nodes[i]->output_id] = i;
  std::vector<char> live(g->num_nodes, 0);
  std::vector<int> work;
  for (int i = 0; i < g->num_outputs; ++i) { auto it = producer.find(g->output_node_ids[i]); if (it != producer.end()) work.push_back(it->second); }
  while (!work.empty()) {
    const int i = work.back(); work.pop_back();
    if (live[i]) continue;
    live[i] = 1;
    for (int k = 0; k < g->nodes[i]->num_inputs; ++k) { auto it = producer.find(g->nodes[i]->input_ids[k]); if (it != producer.end() && it->second < i) work.push_back(it->second); }
  }
  for (int i = 0; i < g->num_nodes; ++i) if (!live[i]) g->nodes[i]->dead = true;
  find_inputs(g);
}
CG_EXPORT void cg_ir_cse(cg_ir_graph* g) {
  if (!g) return;
  std::map<std::string, int> seen;                   // key -> output tensor id of the first occurrence
  std::map<int, int> rename;
  for (int i = 0; i < g->num_nodes; ++i) {
    cg_ir_node* n = g->nodes[i];
    if (n->dead) continue;
    for (int k = 0; k < n->num_inputs; ++k) { auto it = rename.find(n->input_ids[k]); if (it != rename.end()) n->input_ids[k] = it->second; }
    std::vector<int> in(n->input_ids, n->input_ids + n->num_inputs);
    if ((n->opcode == OP_ADD || n->opcode == OP_MUL) && in.size() == 2 && in[0] > in[1]) std::swap(in[0], in[1]);
    std::string key((const char*)&n->opcode, sizeof(n->opcode));
    key.append((const char*)in.data(), in.size() * sizeof(int));
    if (n->attributes) key.append((const char*)n->attributes, n->attr_size);
    key.append((const char*)n->output_shape, sizeof(int) * n->output_ndim);
    auto it = seen.find(key);
    if (it == seen.end()) { seen[key] = n->output_id; continue; }
    if (is_graph_output(g, n->output_id)) continue;   // a named result keeps its own storage
    rename[n->output_id] = it->second;
    n->dead = true;
  }
}
// Marks producer -> single elementwise consumer pairs (vertical) and independent elementwise
// nodes that read the same tensor (horizontal).
CG_EXPORT void cg_ir_fuse_ops(cg_ir_graph* g) {
  if (!g) return;
  auto cons = consumers(g);
  for (int i = 0; i < g->num_nodes; ++i) {
    cg_ir_node* n = g->nodes[i];
    n->can_fuse = false; n->fusion_type = NODE_FUSION_NONE; n->fused_with = nullptr;
  }
  for (int i = 0; i < g->num_nodes; ++i) {
    cg_ir_node* n = g->nodes[i];
    if (n->dead) continue;
    const auto& c = cons[n->output_id];
    if (c.size() == 1 && !is_graph_output(g, n->output_id)) {
      cg_ir_node* m = g->nodes[c[0]];
      if (cg_fusion_can_fuse(n, m)) { n->can_fuse = true; n->fusion_type = NODE_FUSION_VERTICAL; n->fused_with = m; continue; }
    }
    if (!is_elementwise(n->opcode) || n->num_inputs == 0) continue;
    for (int j : cons[n->input_ids[0]]) {
      cg_ir_node* m = g->nodes[j];
      if (j <= i || m->dead || !is_elementwise(m->opcode) || m->fusion_type != NODE_FUSION_NONE) continue;
      if (tensor_size(g, m->output_id) != tensor_size(g, n->output_id)) continue;
      bool dependent = false;
      for (int k = 0; k < m->num_inputs; ++k) dependent = dependent || m->input_ids[k] == n->output_id;
      if (dependent) continue;
      n->can_fuse = true; n->fusion_type = NODE_FUSION_HORIZONTAL; n->fused_with = m;
      break;
    }
  }
}
CG_EXPORT void cg_ir_optimize(cg_ir_graph* g, int level) {
  if (!g) return;
  g->opt_level = level;
  if (level <= 0) return;
  cg_ir_cse(g);
  cg_ir_dce(g);
  if (level >= 2) cg_ir_fuse_ops(g);
}
CG_EXPORT void cg_ir_graph_print(cg_ir_graph* g) {
  if (!g) { std::printf("(null graph)\n"); return; }
  std::printf("graph: %d nodes (%d live), %d tensors, %d inputs, %d outputs, opt level %d\n", g->num_nodes, cg_ir_graph_live_nodes(g), g->num_tensors, g->num_inputs, g->num_outputs, g->opt_level);
  for (int i = 0; i < g->num_nodes; ++i) {
    const cg_ir_node* n = g->nodes[i];
    std::printf("  %%%d = %s(", n->output_id, cg_ir_opcode_name(n->opcode));
    for (int k = 0; k < n->num_inputs; ++k) std::printf(k ? ", %%%d" : "%%%d", n->input_ids[k]);
    std::printf(") [");
    for (int k = 0; k < n->output_ndim; ++k) std::printf(k ? "x%d" : "%d", n->output_shape[k]);
    std::printf("]%s%s\n", n->dead ? " dead" : "", n->fusion_type == NODE_FUSION_VERTICAL ? " fuse-down" : n->fusion_type == NODE_FUSION_HORIZONTAL ? " fuse-across" : "");
  }
}

// ------------------------------------------------------------- interpreter
static float apply_unary(cg_ir_opcode op, float x) {
  switch (op) {
    case OP_NEG: return -x;
    case OP_EXP: return std::exp(x);
    case OP_LOG: return std::log(x);
    case OP_SQRT: return std::sqrt(x);
    case OP_RSQRT: return 1.0f / std::sqrt(x);
    case OP_RELU: return x > 0 ? x : 0.0f;
    case OP_SIGMOID: return sigmoidf(x);
    case OP_TANH: return std::tanh(x);
    case OP_GELU: return geluf(x);
    default: return x;
  }
}
static void softmax_rows(const float* x, float* y, int R, int C, float scale) {
  for (int r = 0; r < R; ++r) {
    const float* p = x + (size_t)r * C; float* q = y + (size_t)r * C;
    float m = p[0] * scale; for (int j = 1; j < C; ++j) m = p[j] * scale > m ? p[j] * scale : m;
    double s = 0; for (int j = 0; j < C; ++j) { q[j] = std::exp(p[j] * scale - m); s += q[j]; }
    const float inv = (float)(1.0 / s); for (int j = 0; j < C; ++j) q[j] *= inv;
  }
}
static bool run_node(cg_ir_graph* g, cg_ir_node* n) {
  auto T = [&](int k) -> cg_tensor* { const int id = n->input_ids[k]; return id >= 0 && id < g->num_tensors ? g->tensors[id] : nullptr; };
  cg_tensor* o = n->output_id >= 0 && n->output_id < g->num_tensors ? g->tensors[n->output_id] : nullptr;
  if (!o) return false;
  for (int k = 0; k < n->num_inputs; ++k) if (!T(k)) return false;
  const cg_ir_opcode op = n->opcode;
  if (is_binary(op)) {
    if (n->num_inputs != 2 || T(0)->size != o->size || T(1)->size != o->size) return false;
    const float* a = T(0)->data; const float* b = T(1)->data;
    for (int i = 0; i < o->size; ++i) o->data[i] = op == OP_ADD ? a[i] + b[i] : op == OP_SUB ? a[i] - b[i] : op == OP_MUL ? a[i] * b[i] : a[i] / b[i];
    return true;
  }
  if ((op >= OP_NEG && op <= OP_GELU) || op == OP_COPY || op == OP_RESHAPE || op == OP_NOOP) {
    if (n->num_inputs < 1 || T(0)->size != o->size) return false;
    for (int i = 0; i < o->size; ++i) o->data[i] = apply_unary(op, T(0)->data[i]);
    return true;
  }
  switch (op) {
    case OP_SOFTMAX: if (T(0)->size != o->size) return false; softmax_rows(T(0)->data, o->data, rows_of(o), cols_of(o), 1.0f); return true;
    case OP_MATMUL: {
      cg_tensor *a = T(0), *b = T(1);
      if (a->ndim < 2 || b->ndim < 2) return false;
      const int M = a->shape[a->ndim - 2], K = a->shape[a->ndim - 1], N = b->shape[b->ndim - 1];
      if (b->shape[b->ndim - 2] != K) return false;
      const int batch = a->size / (M * K), bb = b->size / (K * N);
      if (o->size != batch * M * N || (bb != 1 && bb != batch)) return false;
      for (int i = 0; i < batch; ++i) gemm(a->data + (size_t)i * M * K, b->data + (bb == 1 ? 0 : (size_t)i * K * N), o->data + (size_t)i * M * N, M, N, K, false, false, false);
      return true;
    }
    case OP_TRANSPOSE: {
      cg_tensor* a = T(0);
      if (a->ndim != 2 || o->size != a->size) return false;
      for (int i = 0; i < a->shape[0]; ++i) for (int j = 0; j < a->shape[1]; ++j) o->data[(size_t)j * a->shape[0] + i] = a->data[(size_t)i * a->shape[1] + j];
      return true;
    }
    case OP_SUM: case OP_MEAN: case OP_MAX: case OP_MIN: {
      cg_tensor* a = T(0);
      int axis = -1;
      if (n->attributes && n->attr_size >= sizeof(int)) std::memcpy(&axis, n->attributes, sizeof(int));
      int outer = 1, len = a->size, inner = 1;
      if (axis >= 0 && axis < a->ndim) { len = a->shape[axis]; for (int i = 0; i < axis; ++i) outer *= a->shape[i]; for (int i = axis + 1; i < a->ndim; ++i) inner *= a->shape[i]; }
      if (o->size != outer * inner || len <= 0) return false;
      for (int x = 0; x < outer; ++x) for (int z = 0; z < inner; ++z) {
        const float* p = a->data + (size_t)x * len * inner + z;
        double acc = (op == OP_MAX || op == OP_MIN) ? p[0] : 0.0;
        for (int k = 0; k < len; ++k) { const float v = p[(size_t)k * inner]; if (op == OP_MAX) acc = v > acc ? v : acc; else if (op == OP_MIN) acc = v < acc ? v : acc; else acc += v; }
        o->data[(size_t)x * inner + z] = (float)(op == OP_MEAN ? acc / len : acc);
      }
      return true;
    }
    case OP_BROADCAST: {
      cg_tensor* a = T(0);
      int st[CG_MAX_DIMS], idx[CG_MAX_DIMS] = {0};
      cg_broadcast_strides(a->shape, a->ndim, o->shape, o->ndim, st);
      long off = 0;
      for (int i = 0; i < o->size; ++i) {
        o->data[i] = a->data[off];
        for (int d = o->ndim - 1; d >= 0; --d) { ++idx[d]; off += st[d]; if (idx[d] < o->shape[d]) break; off -= (long)st[d] * o->shape[d]; idx[d] = 0; }
      }
      return true;
    }
    case OP_FUSED_LAYERNORM: {          // inputs: x [, gamma [, beta]]; attr: float eps
      cg_tensor* x = T(0);
      float eps = 1e-5f;
      if (n->attributes && n->attr_size >= sizeof(float)) std::memcpy(&eps, n->attributes, sizeof(float));
      const int C = cols_of(x), R = rows_of(x);
      for (int r = 0; r < R; ++r) {
        const float* p = x->data + (size_t)r * C;
        double m = 0, v = 0;
        for (int j = 0; j < C; ++j) m += p[j];
        m /= C;
        for (int j = 0; j < C; ++j) { const double d = p[j] - m; v += d * d; }
        const float inv = 1.0f / std::sqrt((float)(v / C) + eps);
        for (int j = 0; j < C; ++j) {
          float y = (p[j] - (float)m) * inv;
          if (n->num_inputs > 1) y *= T(1)->data[j];
          if (n->num_inputs > 2) y += T(2)->data[j];
          o->data[(size_t)r * C + j] = y;
        }
      }
      return true;
    }
    case OP_FUSED_ATTENTION: {          // inputs: q [T,D], k^T [D,S], v [S,Dv]; attr: float scale
      if (n->num_inputs != 3) return false;
      cg_tensor *q = T(0), *kt = T(1), *v = T(2);
      if (q->ndim != 2 || kt->ndim != 2 || v->ndim != 2 || q->shape[1] != kt->shape[0] || kt->shape[1] != v->shape[0]) return false;
      float scale = 1.0f;
      if (n->attributes && n->attr_size >= sizeof(float)) std::memcpy(&scale, n->attributes, sizeof(float));
      const int Tq = q->shape[0], D = q->shape[1], S = kt->shape[1], Dv = v->shape[1];
      if (o->size != Tq * Dv) return false;
      std::vector<float> s((size_t)Tq * S);
      gemm(q->data, kt->data, s.data(), Tq, S, D, false, false, false);
      softmax_rows(s.data(), s.data(), Tq, S, scale);
      gemm(s.data(), v->data, o->data, Tq, Dv, S, false, false, false);
      return true;
    }
    default: return false;
  }
}
CG_EXPORT bool cg_ir_execute(cg_ir_graph* g) {
  if (!g) return fail(CG_ERROR_NULL_POINTER, false);
  for (int i = 0; i < g->num_nodes; ++i) {
    if (g->nodes[i]->dead) continue;
    if (!run_node(g, g->nodes[i])) return fail(CG_ERROR_INVALID_ARGUMENT, false);
  }
  return true;
}
