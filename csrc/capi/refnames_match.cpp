// Second part of the reference-named entry points: the LayerNorm and attention pattern matchers
// (include/cg_fusion.h:140-147, declared there and defined nowhere), the shape-mismatch report
// (src/core/symbolic.c:490) and the attention call of the transformer block
// (cg_flash_attn_forward, src/layers/transformer.c:62, defined nowhere in the reference).
#include <string>

#include "internal.hpp"
#include "jit_internal.hpp"

using namespace cgi;

namespace {

struct Walk {
  cg_ir_graph* g;
  std::vector<std::vector<int>> cons;
  explicit Walk(cg_ir_graph* graph) : g(graph), cons(cgjit::consumers(graph)) {}
  cg_ir_node* node(int idx) const { return idx >= 0 && idx < g->num_nodes && !g->nodes[idx]->dead ? g->nodes[idx] : nullptr; }
  bool reads(const cg_ir_node* n, int tensor) const {
    for (int k = 0; k < n->num_inputs; ++k) if (n->input_ids[k] == tensor) return true;
    return false;
  }
  // the only live reader of `tensor` if it has opcode `op` (and also reads `also` when >= 0)
  cg_ir_node* sole(int tensor, cg_ir_opcode op, int also = -1) const {
    if (tensor < 0 || tensor >= (int)cons.size() || cons[tensor].size() != 1) return nullptr;
    cg_ir_node* n = node(cons[tensor][0]);
    return n && n->opcode == op && (also < 0 || reads(n, also)) ? n : nullptr;
  }
  // a reader of `tensor` with opcode `op` that also reads `also` (the tensor may have other readers)
  cg_ir_node* any(int tensor, cg_ir_opcode op, int also = -1) const {
    if (tensor < 0 || tensor >= (int)cons.size()) return nullptr;
    for (int idx : cons[tensor]) {
      cg_ir_node* n = node(idx);
      if (n && n->opcode == op && (also < 0 || reads(n, also))) return n;
    }
    return nullptr;
  }
  // follows `tensor` through an OP_BROADCAST node that is its only reader (the node joins `nodes`)
  int through_bcast(int tensor, std::vector<cg_ir_node*>& nodes) const {
    if (cg_ir_node* b = sole(tensor, OP_BROADCAST)) { nodes.push_back(b); return b->output_id; }
    return tensor;
  }
};

bool emit(std::vector<cg_ir_node*>& nodes, cg_fusion_type type, const char* name, cg_fusion_group** out) {
  if (out) {
    cg_fusion_group* grp = cg_fusion_group_new(nodes.data(), (int)nodes.size());
    if (!grp) return false;
    grp->fusion_type = type;
    std::free(grp->kernel_name);
    grp->kernel_name = strdup(name);
    grp->is_valid = true;
    *out = grp;
  }
  return true;
}

}  // namespace

// LayerNorm written out in primitive operations, starting at the node that takes the row mean:
//   mu = MEAN(x);  c = SUB(x, mu);  sq = MUL(c, c);  var = MEAN(sq);  [ve = ADD(var, eps)];
//   then  r = RSQRT(ve); y = MUL(c, r)   or   s = SQRT(ve); y = DIV(c, s);
//   [y = MUL(y, gamma)];  [y = ADD(y, beta)]
// with an optional OP_BROADCAST between a row statistic and the operation that applies it.
// A single OP_FUSED_LAYERNORM node matches too.  On success *out_group (when given) is a new
// group of type FUSION_LAYERNORM holding the matched nodes in program order.
CG_EXPORT bool cg_fusion_match_layernorm(cg_ir_graph* g, int start_idx, cg_fusion_group** out_group) {
  if (out_group) *out_group = nullptr;
  if (!g) { set_error(CG_ERROR_NULL_POINTER); return false; }
  Walk w(g);
  cg_ir_node* mu = w.node(start_idx);
  if (!mu) return false;
  std::vector<cg_ir_node*> nodes{mu};
  if (mu->opcode == OP_FUSED_LAYERNORM) return emit(nodes, FUSION_LAYERNORM, "fused_layernorm", out_group);
  if (mu->opcode != OP_MEAN || mu->num_inputs < 1) return false;
  const int x = mu->input_ids[0];
  cg_ir_node* c = w.sole(w.through_bcast(mu->output_id, nodes), OP_SUB, x);
  if (!c || c->input_ids[0] != x) return false;
  cg_ir_node* sq = w.any(c->output_id, OP_MUL);
  if (!sq || sq->num_inputs != 2 || sq->input_ids[0] != c->output_id || sq->input_ids[1] != c->output_id) return false;
  cg_ir_node* var = w.sole(sq->output_id, OP_MEAN);
  if (!var) return false;
  nodes.insert(nodes.end(), {c, sq, var});
  int stat = var->output_id;
  if (cg_ir_node* ve = w.sole(stat, OP_ADD)) { nodes.push_back(ve); stat = ve->output_id; }
  cg_ir_node* y = nullptr;
  if (cg_ir_node* r = w.sole(stat, OP_RSQRT)) {
    nodes.push_back(r);
    y = w.sole(w.through_bcast(r->output_id, nodes), OP_MUL, c->output_id);
    if (!y) return false;
    nodes.push_back(y);
  } else if (cg_ir_node* s = w.sole(stat, OP_SQRT)) {
    nodes.push_back(s);
    y = w.sole(w.through_bcast(s->output_id, nodes), OP_DIV, c->output_id);
    if (!y || y->input_ids[0] != c->output_id) return false;
    nodes.push_back(y);
  } else {
    return false;
  }
  if (cg_ir_node* sc = w.sole(y->output_id, OP_MUL)) {
    nodes.push_back(sc);
    y = sc;
  }
  if (cg_ir_node* sh = w.sole(y->output_id, OP_ADD)) nodes.push_back(sh);
  return emit(nodes, FUSION_LAYERNORM, "fused_layernorm", out_group);
}

// Attention written out in primitive operations, starting at the score product:
//   s = MATMUL(q, kT);  [s = MUL(s, scale) | DIV(s, scale)];  [s = ADD(s, mask)];
//   p = SOFTMAX(s);  o = MATMUL(p, v)
// where kT may itself be the result of a TRANSPOSE node read only here (it joins the group).
// A single OP_FUSED_ATTENTION node matches too.  Group type FUSION_ATTENTION.
CG_EXPORT bool cg_fusion_match_attention(cg_ir_graph* g, int start_idx, cg_fusion_group** out_group) {
  if (out_group) *out_group = nullptr;
  if (!g) { set_error(CG_ERROR_NULL_POINTER); return false; }
  Walk w(g);
  cg_ir_node* qk = w.node(start_idx);
  if (!qk) return false;
  std::vector<cg_ir_node*> nodes;
  if (qk->opcode == OP_FUSED_ATTENTION) { nodes.push_back(qk); return emit(nodes, FUSION_ATTENTION, "fused_attention", out_group); }
  if (qk->opcode != OP_MATMUL || qk->num_inputs != 2) return false;
  // a transpose that feeds only this product belongs to the pattern
  for (int i = 0; i < g->num_nodes; ++i) {
    cg_ir_node* t = w.node(i);
    if (t && t->opcode == OP_TRANSPOSE && t->output_id == qk->input_ids[1] && w.cons[t->output_id].size() == 1) nodes.push_back(t);
  }
  nodes.push_back(qk);
  int s = qk->output_id;
  cg_ir_node* sc = w.sole(s, OP_MUL);
  if (!sc) sc = w.sole(s, OP_DIV);
  if (sc) { nodes.push_back(sc); s = sc->output_id; }
  if (cg_ir_node* m = w.sole(s, OP_ADD)) { nodes.push_back(m); s = m->output_id; }
  cg_ir_node* p = w.sole(s, OP_SOFTMAX);
  if (!p) return false;
  cg_ir_node* o = w.sole(p->output_id, OP_MATMUL);
  if (!o || o->input_ids[0] != p->output_id) return false;
  nodes.insert(nodes.end(), {p, o});
  return emit(nodes, FUSION_ATTENTION, "fused_attention", out_group);
}

// MATMUL -> [ADD bias (through an optional OP_BROADCAST of the bias)] -> activation
// (RELU, SIGMOID, TANH or GELU), each result read only by the next node: the shape the tcgen05
// GEMM's epilogue covers (bias, activation).  A product followed by the bias alone matches too.
// Group type FUSION_EPILOGUE.  (Declared at include/cg_fusion.h:128 in the reference.)
CG_EXPORT bool cg_fusion_match_matmul_epilogue(cg_ir_graph* g, int start_idx, cg_fusion_group** out_group) {
  if (out_group) *out_group = nullptr;
  if (!g) { set_error(CG_ERROR_NULL_POINTER); return false; }
  Walk w(g);
  cg_ir_node* mm = w.node(start_idx);
  if (!mm || mm->opcode != OP_MATMUL) return false;
  std::vector<cg_ir_node*> nodes{mm};
  int t = mm->output_id;
  if (cg_ir_node* bias = w.sole(t, OP_ADD)) { nodes.push_back(bias); t = bias->output_id; }
  cg_ir_node* act = nullptr;
  for (cg_ir_opcode op : {OP_RELU, OP_SIGMOID, OP_TANH, OP_GELU}) if (!act) act = w.sole(t, op);
  if (act) nodes.push_back(act);
  if (nodes.size() < 2) return false;
  return emit(nodes, FUSION_EPILOGUE, "fused_matmul_epilogue", out_group);
}

// RELU -> elementwise MUL (the dropout mask, already scaled) -> ADD (the residual), each result
// read only by the next node.  Group type FUSION_ELEMENTWISE.  (include/cg_fusion.h:134.)
CG_EXPORT bool cg_fusion_match_relu_dropout_add(cg_ir_graph* g, int start_idx, cg_fusion_group** out_group) {
  if (out_group) *out_group = nullptr;
  if (!g) { set_error(CG_ERROR_NULL_POINTER); return false; }
  Walk w(g);
  cg_ir_node* relu = w.node(start_idx);
  if (!relu || relu->opcode != OP_RELU) return false;
  cg_ir_node* drop = w.sole(relu->output_id, OP_MUL);
  cg_ir_node* add = drop ? w.sole(drop->output_id, OP_ADD) : nullptr;
  if (!add) return false;
  std::vector<cg_ir_node*> nodes{relu, drop, add};
  return emit(nodes, FUSION_ELEMENTWISE, "fused_relu_dropout_add", out_group);
}

// Prints both shapes and names the first dimension at which they cannot be unified (or the rank
// difference) to stderr, prefixed with the caller's context.
CG_EXPORT void cg_symbolic_report_mismatch(cg_symbolic_shape* a, cg_symbolic_shape* b, const char* context) {
  if (!a || !b) { set_error(CG_ERROR_NULL_POINTER); return; }
  auto dim_text = [](const cg_symbolic_dim* d) -> std::string {
    if (!d) return "?";
    if (d->name) return d->name;
    if (d->expr) { char* s = cg_expr_to_string(d->expr); std::string r = s ? s : "?"; std::free(s); return r; }
    return std::to_string((long long)d->value);
  };
  auto shape_text = [&](const cg_symbolic_shape* s) {
    std::string r = "[";
    for (int i = 0; i < s->ndim; ++i) r += (i ? ", " : "") + dim_text(s->dims[i]);
    return r + "]";
  };
  std::fprintf(stderr, "shape mismatch in %s: %s vs %s\n", context ? context : "(no context)", shape_text(a).c_str(), shape_text(b).c_str());
  const int n = a->ndim < b->ndim ? a->ndim : b->ndim;
  for (int i = 1; i <= n; ++i) {                     // aligned from the last dimension, as broadcasting does
    cg_symbolic_dim* da = a->dims[a->ndim - i]; cg_symbolic_dim* db = b->dims[b->ndim - i];
    if (!cg_dim_compatible(da, db)) {
      std::fprintf(stderr, "  dimension -%d: %s is not compatible with %s\n", i, dim_text(da).c_str(), dim_text(db).c_str());
      return;
    }
  }
  if (a->ndim != b->ndim) std::fprintf(stderr, "  ranks differ: %d vs %d\n", a->ndim, b->ndim);
}

// Attention of [batch, seq, heads, d_head] tensors; returns a new tensor (the caller frees it).
// The name under which the reference's transformer block calls attention.
CG_EXPORT cg_tensor* cg_flash_attn_forward(cg_tensor* q, cg_tensor* k, cg_tensor* v, float dropout_prob, float softmax_scale, bool causal) {
  cg_flash_attn_params* p = cg_flash_attn_params_new(q, k, v, causal ? CG_MASK_CAUSAL : CG_MASK_NONE, dropout_prob);
  if (!p) return nullptr;
  if (softmax_scale > 0) p->softmax_scale = softmax_scale;
  cg_flash_attention_forward(p);
  cg_tensor* out = p->O;
  p->O = nullptr;
  cg_flash_attn_params_free(p);
  return out;
}
