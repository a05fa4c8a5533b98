// Entry points under the names the reference's headers and sources use, for programs written
// against them: cg_jit_record_op / cg_jit_execute (include/cg_jit.h:169,209, the second never
// defined there), cg_opcode_name and cg_ir_allocate_registers (src/jit/graph_capture.c:54,321),
// cg_fusion_match_layernorm / cg_fusion_match_attention (include/cg_fusion.h:140,146, never
// defined there), cg_symbolic_report_mismatch (src/core/symbolic.c:490) and cg_flash_attn_forward
// (called by src/layers/transformer.c:62 but defined nowhere).  Each is a full implementation on
// top of this library's IR, interpreter and attention.
#include <map>
#include <mutex>
#include <string>

#include "internal.hpp"
#include "jit_internal.hpp"

using namespace cgi;

CG_EXPORT const char* cg_opcode_name(cg_ir_opcode op) { return cg_ir_opcode_name(op); }

// ------------------------------------------------------------------ tracing by hand
// Allocates the result tensor of `op` on `inputs`, records the node when a trace is open and
// returns the (zero-filled) result; cg_ir_execute / cg_jit_execute compute the values.
// Shape rule: matmul [.., M, K] x [.., K, N] -> [.., M, N]; transpose swaps the last two
// dimensions; reductions take an int axis attribute (absent or < 0: all -> [1]); binary
// operations broadcast; everything else keeps the first input's shape.
CG_EXPORT cg_tensor* cg_jit_record_op(cg_ir_opcode op, cg_tensor** inputs, int num_inputs, void* attributes, size_t attr_size) {
  if (!inputs || num_inputs <= 0 || !inputs[0]) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  const cg_tensor* a = inputs[0];
  int shape[CG_MAX_DIMS], nd = a->ndim;
  for (int i = 0; i < nd; ++i) shape[i] = a->shape[i];
  if (op == OP_MATMUL) {
    if (num_inputs < 2 || !inputs[1] || a->ndim < 2 || inputs[1]->ndim < 2 ||
        inputs[1]->shape[inputs[1]->ndim - 2] != a->shape[a->ndim - 1])
      return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
    shape[nd - 1] = inputs[1]->shape[inputs[1]->ndim - 1];
  } else if (op == OP_TRANSPOSE) {
    if (nd < 2) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
    std::swap(shape[nd - 1], shape[nd - 2]);
  } else if (cgjit::is_reduction(op)) {
    int axis = -1;
    if (attributes && attr_size >= sizeof(int)) std::memcpy(&axis, attributes, sizeof(int));
    if (axis >= nd) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
    if (axis < 0) { nd = 1; shape[0] = 1; }
    else { for (int i = axis; i + 1 < nd; ++i) shape[i] = shape[i + 1]; nd = nd > 1 ? nd - 1 : 1; if (a->ndim == 1) shape[0] = 1; }
  } else if (cgjit::is_binary(op) && num_inputs >= 2 && inputs[1]) {
    const cg_tensor* b = inputs[1];
    const int out_nd = a->ndim > b->ndim ? a->ndim : b->ndim;
    for (int i = 0; i < out_nd; ++i) {
      const int da = i < out_nd - a->ndim ? 1 : a->shape[i - (out_nd - a->ndim)];
      const int db = i < out_nd - b->ndim ? 1 : b->shape[i - (out_nd - b->ndim)];
      if (da != db && da != 1 && db != 1) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
      shape[i] = da > db ? da : db;
    }
    nd = out_nd;
  }
  cg_tensor* out = make(shape, nd, false);
  if (!out || !cg_jit_is_tracing()) return out;
  if (cgjit::is_binary(op) && num_inputs == 2 && (inputs[0]->size != out->size || inputs[1]->size != out->size)) {
    // the IR's binary nodes take equal shapes: an operand that broadcasts gets an explicit
    // OP_BROADCAST node in front (its result tensor is kept alive by the graph)
    cg_tensor* ops[2] = {inputs[0], inputs[1]};
    cg_tensor* tmp[2] = {nullptr, nullptr};
    for (int k = 0; k < 2; ++k) {
      if (ops[k]->size == out->size) continue;
      tmp[k] = make(shape, nd, false);
      if (!tmp[k]) { cg_tensor_release(out); if (tmp[0]) cg_tensor_release(tmp[0]); return nullptr; }
      cg_jit_record(OP_BROADCAST, &ops[k], 1, tmp[k], nullptr, 0);
      ops[k] = tmp[k];
    }
    cg_jit_record(op, ops, 2, out, attributes, attr_size);
    for (cg_tensor* t : tmp) if (t) cg_tensor_release(t);
    return out;
  }
  cg_jit_record(op, inputs, num_inputs, out, attributes, attr_size);
  return out;
}

// Runs the compiler's graph on caller-provided tensors: inputs[i] is copied into the graph's i-th
// input (order of graph->input_node_ids), the compiled CPU module runs (the interpreter when
// nothing was compiled or the back end has no loader in this library), and the graph's j-th
// output is copied into outputs[j].
CG_EXPORT void cg_jit_execute(cg_jit_compiler* c, cg_tensor** inputs, int num_inputs, cg_tensor** outputs, int num_outputs) {
  if (!c || !c->graph) { set_error(CG_ERROR_NULL_POINTER); return; }
  cg_ir_graph* g = c->graph;
  if (num_inputs > g->num_inputs || num_outputs > g->num_outputs || (num_inputs && !inputs) || (num_outputs && !outputs)) {
    set_error(CG_ERROR_INVALID_ARGUMENT); return;
  }
  for (int i = 0; i < num_inputs; ++i) {
    cg_tensor* dst = g->tensors[g->input_node_ids[i]];
    if (!inputs[i] || inputs[i]->size != dst->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
    if (inputs[i] != dst) std::memcpy(dst->data, inputs[i]->data, sizeof(float) * (size_t)dst->size);
  }
  const bool compiled = c->is_compiled && c->backend == JIT_BACKEND_CPU && c->compiled_kernel;
  if (!(compiled ? cg_jit_run(c) : cg_ir_execute(g))) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  for (int j = 0; j < num_outputs; ++j) {
    const cg_tensor* src = g->tensors[g->output_node_ids[j]];
    if (!outputs[j] || outputs[j]->size != src->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
    if (outputs[j] != src) std::memcpy(outputs[j]->data, src->data, sizeof(float) * (size_t)src->size);
  }
}

// ------------------------------------------------------------------ register allocation
// Linear scan over the live nodes in program order: a tensor's interval runs from its producer to
// its last reader (graph outputs stay live to the end); a freed register is reused by the next
// definition; with more than max_regs values live the value whose interval ends last is spilled.
// The reference computes such an assignment and throws it away (src/jit/graph_capture.c:321-377);
// here it is kept per graph and can be read back.
namespace {
struct RegPlan { std::map<int, int> reg; int spills = 0, used = 0; };
std::mutex g_plan_mu;
std::map<const cg_ir_graph*, RegPlan> g_plans;
}  // namespace

CG_EXPORT void cg_ir_allocate_registers(cg_ir_graph* g, int max_regs) {
  if (!g) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (max_regs <= 0) max_regs = 1;
  std::vector<int> order;
  for (int i = 0; i < g->num_nodes; ++i) if (!g->nodes[i]->dead) order.push_back(i);
  std::map<int, int> last_use;                                  // tensor id -> position of the last reader
  for (size_t pos = 0; pos < order.size(); ++pos) {
    const cg_ir_node* n = g->nodes[order[pos]];
    for (int k = 0; k < n->num_inputs; ++k) last_use[n->input_ids[k]] = (int)pos;
  }
  for (int j = 0; j < g->num_outputs; ++j) last_use[g->output_node_ids[j]] = (int)order.size();
  RegPlan plan;
  std::vector<int> free_regs;
  std::map<int, int> live;                                      // register -> tensor id
  for (size_t pos = 0; pos < order.size(); ++pos) {
    const cg_ir_node* n = g->nodes[order[pos]];
    // registers whose value was read for the last time before this node are free again
    for (auto it = live.begin(); it != live.end();) {
      auto lu = last_use.find(it->second);
      if (lu == last_use.end() || lu->second < (int)pos) { free_regs.push_back(it->first); it = live.erase(it); }
      else ++it;
    }
    int r;
    if (!free_regs.empty()) { r = free_regs.back(); free_regs.pop_back(); }
    else if (plan.used < max_regs) r = plan.used++;
    else {
      // spill the live value that is needed last (or this one, when it outlives them all)
      int victim = -1, far = last_use.count(n->output_id) ? last_use[n->output_id] : (int)pos;
      for (auto& kv : live) if (last_use[kv.second] > far) { far = last_use[kv.second]; victim = kv.first; }
      ++plan.spills;
      if (victim < 0) { plan.reg[n->output_id] = -1; continue; }
      plan.reg[live[victim]] = -1;
      live.erase(victim);
      r = victim;
    }
    live[r] = n->output_id;
    plan.reg[n->output_id] = r;
  }
  std::lock_guard<std::mutex> lock(g_plan_mu);
  g_plans[g] = plan;
}
// Register of a tensor id after cg_ir_allocate_registers: >= 0, -1 spilled, -2 unknown / not planned.
CG_EXPORT int cg_ir_register_of(cg_ir_graph* g, int tensor_id) {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  auto p = g_plans.find(g);
  if (p == g_plans.end()) return -2;
  auto r = p->second.reg.find(tensor_id);
  return r == p->second.reg.end() ? -2 : r->second;
}
CG_EXPORT int cg_ir_spill_count(cg_ir_graph* g) {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  auto p = g_plans.find(g);
  return p == g_plans.end() ? -1 : p->second.spills;
}
CG_EXPORT int cg_ir_registers_used(cg_ir_graph* g) {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  auto p = g_plans.find(g);
  return p == g_plans.end() ? -1 : p->second.used;
}
