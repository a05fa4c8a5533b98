// Code generation from the IR (C for the host, CUDA for NVRTC), the host compile-and-load
// path, and the pattern-based fusion pass.
// Reference surface: include/cg_jit.h (codegen, compiler), include/cg_fusion.h,
// src/jit/graph_capture.c:383-660, src/jit/fusion.c.
#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <spawn.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <set>
#include <sstream>
#include <string>

extern char** environ;

#include "internal.hpp"
#include "jit_internal.hpp"

using namespace cgi;
using namespace cgjit;

namespace {
std::string expr_of(cg_ir_opcode op, const std::string& a, const std::string& b, bool cuda) {
  switch (op) {
    case OP_ADD: return "(" + a + " + " + b + ")";
    case OP_SUB: return "(" + a + " - " + b + ")";
    case OP_MUL: return "(" + a + " * " + b + ")";
    case OP_DIV: return "(" + a + " / " + b + ")";
    case OP_NEG: return "(-" + a + ")";
    case OP_EXP: return "expf(" + a + ")";
    case OP_LOG: return "logf(" + a + ")";
    case OP_SQRT: return "sqrtf(" + a + ")";
    case OP_RSQRT: return cuda ? "rsqrtf(" + a + ")" : "(1.0f / sqrtf(" + a + "))";
    case OP_RELU: return "fmaxf(" + a + ", 0.0f)";
    case OP_SIGMOID: return "(1.0f / (1.0f + expf(-" + a + ")))";
    case OP_TANH: return "tanhf(" + a + ")";
    case OP_GELU: return "(0.5f * " + a + " * (1.0f + tanhf(0.7978845608f * (" + a + " + 0.044715f * " + a + " * " + a + " * " + a + "))))";
    default: return a;
  }
}
// Maximal sequences of live elementwise nodes over the same number of elements.
std::vector<std::vector<int>> split_runs(const cg_ir_graph* g, std::vector<int>* others) {
  std::vector<std::vector<int>> runs;
  std::vector<int> cur; int cur_size = -1;
  for (int i = 0; i < g->num_nodes; ++i) {
    const cg_ir_node* n = g->nodes[i];
    if (n->dead) continue;
    bool ew = is_elementwise(n->opcode);
    const int sz = tensor_size(g, n->output_id);
    for (int k = 0; ew && k < n->num_inputs; ++k) ew = tensor_size(g, n->input_ids[k]) == sz;
    if (ew && (cur.empty() || sz == cur_size)) { cur.push_back(i); cur_size = sz; continue; }
    if (!cur.empty()) { runs.push_back(cur); cur.clear(); }
    if (ew) { cur.push_back(i); cur_size = sz; }
    else { if (others) others->push_back(i); runs.push_back({-1 - i}); }   // marker: a non-elementwise node sits here
  }
  if (!cur.empty()) runs.push_back(cur);
  return runs;
}
// Body of one fused loop over index i.  Values defined in the run stay in registers; a store
// is emitted only for tensors that are read outside the run or are graph outputs.
std::string run_body(const cg_ir_graph* g, const std::vector<int>& run, const std::vector<std::vector<int>>& cons, bool cuda, const char* indent) {
  std::set<int> defined, in_run(run.begin(), run.end());
  std::ostringstream s;
  for (int idx : run) {
    const cg_ir_node* n = g->nodes[idx];
    auto operand = [&](int k) { const int id = n->input_ids[k]; return defined.count(id) ? "v" + std::to_string(id) : "t[" + std::to_string(id) + "][i]"; };
    const std::string a = n->num_inputs > 0 ? operand(0) : "0.0f", b = n->num_inputs > 1 ? operand(1) : "0.0f";
    s << indent << "const float v" << n->output_id << " = " << expr_of(n->opcode, a, b, cuda) << ";\n";
    defined.insert(n->output_id);
    bool store = is_graph_output(g, n->output_id);
    for (int c : cons[n->output_id]) store = store || !in_run.count(c);
    if (store) s << indent << "t[" << n->output_id << "][i] = v" << n->output_id << ";\n";
  }
  return s.str();
}
int axis_of(const cg_ir_node* n) { int a = -1; if (n->attributes && n->attr_size >= sizeof(int)) std::memcpy(&a, n->attributes, sizeof(int)); return a; }
// Plain C loops for the non-elementwise nodes the host module supports; false = unsupported.
bool emit_c_node(const cg_ir_graph* g, const cg_ir_node* n, std::ostringstream& s) {
  auto T = [&](int k) { return g->tensors[n->input_ids[k]]; };
  const cg_tensor* o = g->tensors[n->output_id];
  const int out = n->output_id;
  switch (n->opcode) {
    case OP_MATMUL: {
      const cg_tensor *a = T(0), *b = T(1);
      if (a->ndim < 2 || b->ndim < 2) return false;
      const int M = a->shape[a->ndim - 2], K = a->shape[a->ndim - 1], N = b->shape[b->ndim - 1];
      const int batch = a->size / (M * K), bb = b->size / (K * N);
      s << "  for (long z = 0; z < " << batch << "; ++z) {\n    const float* A = t[" << n->input_ids[0] << "] + z * " << (long)M * K << ";\n"
        << "    const float* B = t[" << n->input_ids[1] << "] + " << (bb == 1 ? "0" : "z * " + std::to_string((long)K * N)) << ";\n"
        << "    float* C = t[" << out << "] + z * " << (long)M * N << ";\n"
        << "    for (int i = 0; i < " << M << "; ++i) {\n      for (int j = 0; j < " << N << "; ++j) C[i * " << N << " + j] = 0.0f;\n"
        << "      for (int k = 0; k < " << K << "; ++k) { const float a = A[i * " << K << " + k]; for (int j = 0; j < " << N << "; ++j) C[i * " << N << " + j] += a * B[k * " << N << " + j]; }\n    }\n  }\n";
      return true;
    }
    case OP_TRANSPOSE: {
      const cg_tensor* a = T(0);
      if (a->ndim != 2) return false;
      s << "  for (int i = 0; i < " << a->shape[0] << "; ++i) for (int j = 0; j < " << a->shape[1] << "; ++j) t[" << out << "][j * " << a->shape[0] << " + i] = t[" << n->input_ids[0] << "][i * " << a->shape[1] << " + j];\n";
      return true;
    }
    case OP_SOFTMAX: {
      const int C = o->ndim ? o->shape[o->ndim - 1] : 1, R = C ? o->size / C : 0;
      s << "  for (int r = 0; r < " << R << "; ++r) {\n    const float* x = t[" << n->input_ids[0] << "] + (long)r * " << C << "; float* y = t[" << out << "] + (long)r * " << C << ";\n"
        << "    float m = x[0]; for (int j = 1; j < " << C << "; ++j) m = x[j] > m ? x[j] : m;\n    float sum = 0.0f; for (int j = 0; j < " << C << "; ++j) { y[j] = expf(x[j] - m); sum += y[j]; }\n"
        << "    for (int j = 0; j < " << C << "; ++j) y[j] /= sum;\n  }\n";
      return true;
    }
    case OP_SUM: case OP_MEAN: case OP_MAX: case OP_MIN: {
      const cg_tensor* a = T(0);
      const int axis = axis_of(n);
      int outer = 1, len = a->size, inner = 1;
      if (axis >= 0 && axis < a->ndim) { len = a->shape[axis]; for (int i = 0; i < axis; ++i) outer *= a->shape[i]; for (int i = axis + 1; i < a->ndim; ++i) inner *= a->shape[i]; }
      const bool mx = n->opcode == OP_MAX, mn = n->opcode == OP_MIN;
      s << "  for (long x = 0; x < " << outer << "; ++x) for (long z = 0; z < " << inner << "; ++z) {\n    const float* p = t[" << n->input_ids[0] << "] + x * " << (long)len * inner << " + z;\n"
        << "    float acc = " << ((mx || mn) ? "p[0]" : "0.0f") << ";\n    for (long k = 0; k < " << len << "; ++k) { const float v = p[k * " << inner << "]; "
        << (mx ? "acc = v > acc ? v : acc;" : mn ? "acc = v < acc ? v : acc;" : "acc += v;") << " }\n    t[" << out << "][x * " << inner << " + z] = acc"
        << (n->opcode == OP_MEAN ? " / " + std::to_string(len) + ".0f" : "") << ";\n  }\n";
      return true;
    }
    case OP_RESHAPE: case OP_NOOP:
      s << "  memcpy(t[" << out << "], t[" << n->input_ids[0] << "], sizeof(float) * " << o->size << ");\n";
      return true;
    case OP_BROADCAST: {
      cg_tensor* a = T(0);
      int st[CG_MAX_DIMS];
      cg_broadcast_strides(a->shape, a->ndim, const_cast<int*>(o->shape), o->ndim, st);
      s << "  for (long i = 0; i < " << o->size << "; ++i) {\n    long r = i, off = 0;\n";
      for (int d = o->ndim - 1; d >= 0; --d) {
        if (st[d]) s << "    off += (r % " << o->shape[d] << ") * " << st[d] << ";";
        s << "    r /= " << o->shape[d] << ";\n";
      }
      s << "    t[" << out << "][i] = t[" << n->input_ids[0] << "][off];\n  }\n";
      return true;
    }
    default: return false;
  }
}
uint64_t fnv(uint64_t h, const void* p, size_t n) { const unsigned char* b = (const unsigned char*)p; for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 0x100000001B3ull; } return h; }
std::atomic<int> g_module_counter{0};
typedef int (*jit_entry)(float**);
}  // namespace

// int jit_kernel(float** t): t[id] is the storage of tensor id; sizes are baked in.  Returns 0,
// or 1 + the index of the first node the host generator cannot express.
CG_EXPORT char* cg_jit_codegen_c(cg_ir_graph* g) {
  if (!g) return fail(CG_ERROR_NULL_POINTER, (char*)nullptr);
  auto cons = consumers(g);
  std::ostringstream s;
  s << "/* generated: " << cg_ir_graph_live_nodes(g) << " live nodes */\n#include <math.h>\n#include <string.h>\nint jit_kernel(float** t) {\n";
  for (auto& run : split_runs(g, nullptr)) {
    if (run[0] < 0) {
      const cg_ir_node* n = g->nodes[-1 - run[0]];
      s << "  /* node " << n->id << ": " << cg_ir_opcode_name(n->opcode) << " */\n";
      if (!emit_c_node(g, n, s)) s << "  return " << n->id + 1 << ";\n";
      continue;
    }
    s << "  /* fused elementwise: " << run.size() << " ops */\n  for (long i = 0; i < " << tensor_size(g, g->nodes[run[0]]->output_id) << "; ++i) {\n" << run_body(g, run, cons, false, "    ") << "  }\n";
  }
  s << "  return 0;\n}\n";
  return strdup(s.str().c_str());
}
// One grid-stride kernel per fused elementwise run: jit_kernel, jit_kernel_1, ...
// (float* const* t, long n).  Contractions and reductions are left to the library kernels and
// appear as comments in program order.
CG_EXPORT char* cg_jit_codegen_cuda(cg_ir_graph* g) {
  if (!g) return fail(CG_ERROR_NULL_POINTER, (char*)nullptr);
  auto cons = consumers(g);
  std::ostringstream s;
  s << "// generated for sm_100a: " << cg_ir_graph_live_nodes(g) << " live nodes\n";
  int k = 0;
  for (auto& run : split_runs(g, nullptr)) {
    if (run[0] < 0) { const cg_ir_node* n = g->nodes[-1 - run[0]]; s << "// node " << n->id << ": " << cg_ir_opcode_name(n->opcode) << " -> library kernel\n"; continue; }
    s << "// elements: " << tensor_size(g, g->nodes[run[0]]->output_id) << "\nextern \"C\" __global__ void jit_kernel" << (k ? "_" + std::to_string(k) : std::string()) << "(float* const* t, long n) {\n"
      << "  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {\n" << run_body(g, run, cons, true, "    ") << "  }\n}\n";
    ++k;
  }
  return strdup(s.str().c_str());
}

CG_EXPORT cg_jit_compiler* cg_jit_compiler_new(cg_ir_graph* g, cg_jit_backend backend) {
  if (!g) return fail(CG_ERROR_NULL_POINTER, (cg_jit_compiler*)nullptr);
  cg_jit_compiler* c = (cg_jit_compiler*)std::calloc(1, sizeof(cg_jit_compiler));
  c->graph = g; c->backend = backend;
  uint64_t ph = 0xCBF29CE484222325ull, sh = ph;
  for (int i = 0; i < g->num_nodes; ++i) {
    const cg_ir_node* n = g->nodes[i];
    if (n->dead) continue;
    ph = fnv(ph, &n->opcode, sizeof(n->opcode)); ph = fnv(ph, n->input_ids, sizeof(int) * n->num_inputs); ph = fnv(ph, &n->output_id, sizeof(int));
    sh = fnv(sh, n->output_shape, sizeof(int) * n->output_ndim);
  }
  c->pattern_hash = ph; c->shape_hash = sh;
  return c;
}
CG_EXPORT bool cg_jit_compile(cg_jit_compiler* c) {
  if (!c || !c->graph) return fail(CG_ERROR_NULL_POINTER, false);
  std::free(c->source_code); c->source_code = nullptr;
  if (c->backend == JIT_BACKEND_CUDA) {
    c->source_code = cg_jit_codegen_cuda(c->graph);
    c->source_len = std::strlen(c->source_code);
    return true;                                     // compiled by NVRTC in the GPU package
  }
  if (c->backend != JIT_BACKEND_CPU) { std::fprintf(stderr, "JIT: Unsupported backend\n"); return fail(CG_ERROR_INVALID_ARGUMENT, false); }
  c->source_code = cg_jit_codegen_c(c->graph);
  c->source_len = std::strlen(c->source_code);
  // The source and the shared object live in a directory of their own that only this user can
  // enter (mkdtemp, mode 0700), so nobody can plant a file or a link at the paths used here; the
  // compiler is started directly with an argument vector (no shell: TMPDIR and CC are never parsed).
  const char* tmp = getenv("TMPDIR");
  std::string dir = std::string(tmp && *tmp ? tmp : "/tmp") + "/cogito_jit_XXXXXX";
  if (!mkdtemp(&dir[0])) return fail(CG_ERROR_FILE_NOT_FOUND, false);
  const std::string src = dir + "/kernel.c", lib = dir + "/kernel.so";
  auto cleanup = [&]() { unlink(src.c_str()); unlink(lib.c_str()); rmdir(dir.c_str()); };
  const int fd = open(src.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0600);
  if (fd < 0) { cleanup(); return fail(CG_ERROR_FILE_NOT_FOUND, false); }
  FILE* f = fdopen(fd, "w");
  if (!f) { close(fd); cleanup(); return fail(CG_ERROR_FILE_NOT_FOUND, false); }
  std::fwrite(c->source_code, 1, c->source_len, f);
  std::fclose(f);
  const char* cc = getenv("CC");
  const std::string compiler = cc && *cc ? cc : "cc";
  std::vector<std::string> args = {compiler, "-O2", "-shared", "-fPIC", "-o", lib, src, "-lm"};
  std::vector<char*> argv;
  for (auto& a : args) argv.push_back(&a[0]);
  argv.push_back(nullptr);
  posix_spawn_file_actions_t fa;
  posix_spawn_file_actions_init(&fa);
  posix_spawn_file_actions_addopen(&fa, 2, "/dev/null", O_WRONLY, 0);      // a missing compiler is not an error worth printing
  pid_t pid = 0;
  int rc = posix_spawnp(&pid, compiler.c_str(), &fa, nullptr, argv.data(), environ);
  posix_spawn_file_actions_destroy(&fa);
  if (rc == 0) {
    int status = 0;
    while (waitpid(pid, &status, 0) < 0 && errno == EINTR) {}
    rc = (WIFEXITED(status) && WEXITSTATUS(status) == 0) ? 0 : 1;
  }
  if (rc != 0) { cleanup(); return false; }           // no compiler here: cg_jit_run interprets instead
  void* h = dlopen(lib.c_str(), RTLD_NOW | RTLD_LOCAL);
  cleanup();
  if (!h) return false;
  c->compiled_module = h; c->compiled_kernel = dlsym(h, "jit_kernel"); c->is_compiled = c->compiled_kernel != nullptr;
  return c->is_compiled;
}
CG_EXPORT bool cg_jit_run(cg_jit_compiler* c) {
  if (!c || !c->graph) return fail(CG_ERROR_NULL_POINTER, false);
  if (!c->is_compiled || c->backend != JIT_BACKEND_CPU) return cg_ir_execute(c->graph);
  std::vector<float*> t(c->graph->num_tensors);
  for (int i = 0; i < c->graph->num_tensors; ++i) t[i] = c->graph->tensors[i] ? c->graph->tensors[i]->data : nullptr;
  const int rc = ((jit_entry)c->compiled_kernel)(t.data());
  return rc == 0 ? true : cg_ir_execute(c->graph);  // a node the generator left out: interpret
}
CG_EXPORT void cg_jit_compiler_free(cg_jit_compiler* c) {
  if (!c) return;
  if (c->compiled_module) dlclose(c->compiled_module);
  std::free(c->source_code); std::free(c);
}

// ------------------------------------------------------------------ fusion
CG_EXPORT bool cg_fusion_can_fuse(cg_ir_node* a, cg_ir_node* b) {
  if (!a || !b || a->dead || b->dead || a == b) return false;
  bool reads = false;
  for (int k = 0; k < b->num_inputs; ++k) reads = reads || b->input_ids[k] == a->output_id;
  if (!reads) return false;
  long sa = 1, sb = 1;
  for (int i = 0; i < a->output_ndim; ++i) sa *= a->output_shape[i];
  for (int i = 0; i < b->output_ndim; ++i) sb *= b->output_shape[i];
  if (is_elementwise(a->opcode) && is_elementwise(b->opcode)) return sa == sb;
  if (is_elementwise(a->opcode) && is_reduction(b->opcode)) return true;
  if (a->opcode == OP_MATMUL && is_elementwise(b->opcode)) return sa == sb;       // epilogue
  return false;
}
CG_EXPORT cg_fusion_group* cg_fusion_group_new(cg_ir_node** nodes, int count) {
  cg_fusion_group* gr = (cg_fusion_group*)std::calloc(1, sizeof(cg_fusion_group));
  gr->capacity = count > 4 ? count : 4;
  gr->nodes = (cg_ir_node**)std::calloc(gr->capacity, sizeof(cg_ir_node*));
  gr->is_valid = true;
  for (int i = 0; i < count; ++i) cg_fusion_group_add(gr, nodes[i]);
  return gr;
}
CG_EXPORT void cg_fusion_group_add(cg_fusion_group* gr, cg_ir_node* n) {
  if (!gr || !n) return;
  if (gr->num_nodes == gr->capacity) { gr->capacity *= 2; gr->nodes = (cg_ir_node**)std::realloc(gr->nodes, sizeof(cg_ir_node*) * gr->capacity); }
  gr->nodes[gr->num_nodes++] = n;
  std::free(gr->output_shape);
  gr->output_ndim = n->output_ndim;
  gr->output_shape = (int*)std::malloc(sizeof(int) * (n->output_ndim ? n->output_ndim : 1));
  for (int i = 0; i < n->output_ndim; ++i) gr->output_shape[i] = n->output_shape[i];
}
CG_EXPORT void cg_fusion_group_free(cg_fusion_group* gr) {
  if (!gr) return;
  std::free(gr->nodes); std::free(gr->kernel_name); std::free(gr->kernel_code); std::free(gr->output_shape); std::free(gr);
}
static long elems(const cg_ir_node* n) { long s = 1; for (int i = 0; i < n->output_ndim; ++i) s *= n->output_shape[i]; return s; }
static void finish_group(cg_fusion_group* gr, cg_fusion_type type, const char* name) {
  gr->fusion_type = type;
  std::free(gr->kernel_name); gr->kernel_name = strdup(name);
  // every intermediate that no longer goes through memory saves one write and one read
  size_t saved = 0, flops = 0;
  for (int i = 0; i < gr->num_nodes; ++i) {
    const cg_ir_node* n = gr->nodes[i];
    if (i + 1 < gr->num_nodes) saved += 2 * sizeof(float) * (size_t)elems(n);
    flops += (size_t)elems(n) * (n->opcode == OP_MATMUL ? 2 : 1);
  }
  gr->memory_saved = saved; gr->flops = flops;
  const size_t bytes = sizeof(float) * (size_t)(elems(gr->nodes[0]) + elems(gr->nodes[gr->num_nodes - 1]));
  gr->arithmetic_intensity = bytes ? (float)flops / bytes : 0.0f;
  gr->schedule_priority = type == FUSION_ATTENTION ? 3 : type == FUSION_EPILOGUE || type == FUSION_CUSTOM ? 2 : 1;
}
// Patterns, most specific first; a node joins at most one group:
//   matmul -> softmax -> matmul                      fused_attention
//   fused_layernorm -> gelu -> matmul                fused_ln_gelu_linear
//   softmax -> mul -> add                            fused_softmax_dropout_residual
//   matmul -> [add] -> [relu|gelu|sigmoid|tanh]      fused_matmul_epilogue
//   elementwise chain -> sum|mean|max|min            fused_reduce
//   elementwise chain of two or more                 fused_elementwise
CG_EXPORT cg_fusion_group** cg_fusion_find_patterns(cg_ir_graph* g, int* num_groups) {
  if (num_groups) *num_groups = 0;
  if (!g) return fail(CG_ERROR_NULL_POINTER, (cg_fusion_group**)nullptr);
  auto cons = consumers(g);
  std::vector<char> used(g->num_nodes, 0);
  std::vector<cg_fusion_group*> out;
  auto next_of = [&](int i) -> int {                  // the single live consumer of node i's result, or -1
    const cg_ir_node* n = g->nodes[i];
    if (is_graph_output(g, n->output_id) || cons[n->output_id].size() != 1) return -1;
    const int j = cons[n->output_id][0];
    return used[j] || g->nodes[j]->dead ? -1 : j;
  };
  auto is_act = [](cg_ir_opcode op) { return op == OP_RELU || op == OP_GELU || op == OP_SIGMOID || op == OP_TANH; };
  auto take = [&](std::vector<int> idx, cg_fusion_type type, const char* name) {
    std::vector<cg_ir_node*> ns;
    for (int i : idx) { used[i] = 1; ns.push_back(g->nodes[i]); }
    cg_fusion_group* gr = cg_fusion_group_new(ns.data(), (int)ns.size());
    finish_group(gr, type, name);
    out.push_back(gr);
  };
  auto op_at = [&](int i) { return i < 0 ? OP_NOOP : g->nodes[i]->opcode; };
  for (int i = 0; i < g->num_nodes; ++i) {            // three-node patterns
    if (used[i] || g->nodes[i]->dead) continue;
    const int j = next_of(i), k = j >= 0 ? next_of(j) : -1;
    if (k < 0) continue;
    const cg_ir_opcode a = op_at(i), b = op_at(j), c = op_at(k);
    if (a == OP_MATMUL && b == OP_SOFTMAX && c == OP_MATMUL && g->nodes[k]->input_ids[0] == g->nodes[j]->output_id) take({i, j, k}, FUSION_ATTENTION, "fused_attention");
    else if (a == OP_FUSED_LAYERNORM && b == OP_GELU && c == OP_MATMUL) take({i, j, k}, FUSION_CUSTOM, "fused_ln_gelu_linear");
    else if (a == OP_SOFTMAX && b == OP_MUL && c == OP_ADD) take({i, j, k}, FUSION_CUSTOM, "fused_softmax_dropout_residual");
  }
  for (int i = 0; i < g->num_nodes; ++i) {            // GEMM epilogues
    if (used[i] || g->nodes[i]->dead || op_at(i) != OP_MATMUL) continue;
    std::vector<int> idx{i};
    int j = next_of(i);
    if (j >= 0 && op_at(j) == OP_ADD && cg_fusion_can_fuse(g->nodes[i], g->nodes[j])) { idx.push_back(j); j = next_of(j); }
    if (j >= 0 && is_act(op_at(j)) && cg_fusion_can_fuse(g->nodes[idx.back()], g->nodes[j])) idx.push_back(j);
    if (idx.size() > 1) take(idx, FUSION_EPILOGUE, "fused_matmul_epilogue");
  }
  for (int i = 0; i < g->num_nodes; ++i) {            // elementwise chains, optionally ending in a reduction
    if (used[i] || g->nodes[i]->dead || !is_elementwise(op_at(i))) continue;
    std::vector<int> idx{i};
    int j = next_of(i);
    while (j >= 0 && is_elementwise(op_at(j)) && cg_fusion_can_fuse(g->nodes[idx.back()], g->nodes[j])) { idx.push_back(j); j = next_of(j); }
    if (j >= 0 && is_reduction(op_at(j))) { idx.push_back(j); take(idx, FUSION_REDUCTION, "fused_reduce"); }
    else if (idx.size() > 1) take(idx, FUSION_ELEMENTWISE, "fused_elementwise");
  }
  if (num_groups) *num_groups = (int)out.size();
  cg_fusion_group** arr = (cg_fusion_group**)std::calloc(out.size() ? out.size() : 1, sizeof(cg_fusion_group*));
  std::copy(out.begin(), out.end(), arr);
  return arr;
}
// CUDA source for elementwise (and elementwise + reduction prologue) groups; for the groups
// that map onto library kernels, the plan of calls that replaces them.
CG_EXPORT char* cg_fusion_generate_kernel(cg_fusion_group* gr) {
  if (!gr || gr->num_nodes == 0) return fail(CG_ERROR_INVALID_ARGUMENT, (char*)nullptr);
  std::ostringstream s;
  const char* name = gr->kernel_name ? gr->kernel_name : "fused";
  if (gr->fusion_type == FUSION_ELEMENTWISE || gr->fusion_type == FUSION_REDUCTION) {
    const int ew = gr->fusion_type == FUSION_REDUCTION ? gr->num_nodes - 1 : gr->num_nodes;
    std::set<int> defined;
    s << "extern \"C\" __global__ void " << name << "(float* const* t, long n) {\n  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {\n";
    for (int i = 0; i < ew; ++i) {
      const cg_ir_node* n = gr->nodes[i];
      auto operand = [&](int k) { const int id = n->input_ids[k]; return defined.count(id) ? "v" + std::to_string(id) : "t[" + std::to_string(id) + "][i]"; };
      s << "    const float v" << n->output_id << " = " << expr_of(n->opcode, n->num_inputs > 0 ? operand(0) : "0.0f", n->num_inputs > 1 ? operand(1) : "0.0f", true) << ";\n";
      defined.insert(n->output_id);
    }
    s << "    t[" << gr->nodes[ew - 1]->output_id << "][i] = v" << gr->nodes[ew - 1]->output_id << ";\n  }\n}\n";
    if (gr->fusion_type == FUSION_REDUCTION) s << "// then: " << cg_ir_opcode_name(gr->nodes[ew]->opcode) << " over t[" << gr->nodes[ew - 1]->output_id << "] (cgk_reduce_axis)\n";
  } else if (gr->fusion_type == FUSION_EPILOGUE) {
    s << "// " << name << ": one tcgen05 GEMM (cgk_gemm_bf16) with epilogue";
    for (int i = 1; i < gr->num_nodes; ++i) s << (i == 1 ? " " : " -> ") << (gr->nodes[i]->opcode == OP_ADD ? "bias" : cg_ir_opcode_name(gr->nodes[i]->opcode));
    s << "\n";
  } else if (gr->fusion_type == FUSION_ATTENTION) s << "// " << name << ": cgk_flash_forward (QK^T, online softmax and PV in one kernel)\n";
  else if (!std::strcmp(name, "fused_ln_gelu_linear")) s << "// " << name << ": cgk_norm_forward, then cgk_gemm_bf16 whose A-operand pass applies GELU\n";
  else s << "// " << name << ": " << gr->num_nodes << " nodes\n";
  std::free(gr->kernel_code);
  gr->kernel_code = strdup(s.str().c_str());
  return strdup(gr->kernel_code);
}
CG_EXPORT cg_fusion_pass* cg_fusion_pass_new(cg_ir_graph* g) {
  if (!g) return fail(CG_ERROR_NULL_POINTER, (cg_fusion_pass*)nullptr);
  cg_fusion_pass* p = (cg_fusion_pass*)std::calloc(1, sizeof(cg_fusion_pass));
  p->graph = g; p->max_fusion_depth = 8; p->enable_epilogue = true; p->enable_attention = true;
  return p;
}
CG_EXPORT void cg_fusion_analyze(cg_fusion_pass* p) {
  if (!p) return;
  for (int i = 0; i < p->num_groups; ++i) cg_fusion_group_free(p->groups[i]);
  std::free(p->groups);
  p->groups = cg_fusion_find_patterns(p->graph, &p->num_groups);
  p->max_groups = p->num_groups;
  for (int i = 0; i < p->num_groups; ++i) {
    cg_fusion_group* gr = p->groups[i];
    if ((gr->fusion_type == FUSION_EPILOGUE && !p->enable_epilogue) || (gr->fusion_type == FUSION_ATTENTION && !p->enable_attention) || gr->num_nodes > p->max_fusion_depth) gr->is_valid = false;
  }
}
// Rewrites the graph: matmul -> softmax -> matmul becomes one OP_FUSED_ATTENTION node
// (inputs q, k^T, v); the members of every other valid group are chained through fused_with
// so that the code generators emit them as one kernel.
CG_EXPORT void cg_fusion_apply(cg_fusion_pass* p) {
  if (!p) return;
  if (!p->groups) cg_fusion_analyze(p);
  for (int i = 0; i < p->num_groups; ++i) {
    cg_fusion_group* gr = p->groups[i];
    if (!gr->is_valid) continue;
    for (int k = 0; k + 1 < gr->num_nodes; ++k) { gr->nodes[k]->can_fuse = true; gr->nodes[k]->fusion_type = NODE_FUSION_VERTICAL; gr->nodes[k]->fused_with = gr->nodes[k + 1]; }
    if (gr->fusion_type == FUSION_ATTENTION && gr->num_nodes == 3) {
      cg_ir_node *qk = gr->nodes[0], *sm = gr->nodes[1], *pv = gr->nodes[2];
      if (qk->num_inputs != 2 || pv->num_inputs != 2) continue;
      int* in = (int*)std::malloc(sizeof(int) * 3);
      in[0] = qk->input_ids[0]; in[1] = qk->input_ids[1]; in[2] = pv->input_ids[1];
      std::free(pv->input_ids);
      pv->input_ids = in; pv->num_inputs = 3; pv->opcode = OP_FUSED_ATTENTION;
      qk->dead = true; sm->dead = true;
    }
  }
}
CG_EXPORT void cg_fusion_pass_free(cg_fusion_pass* p) {
  if (!p) return;
  for (int i = 0; i < p->num_groups; ++i) cg_fusion_group_free(p->groups[i]);
  std::free(p->groups); std::free(p);
}
