/* cogito_jit.h — symbolic shapes, the JIT IR (trace, DCE, CSE, fusion, code generation,
 * execution) and the fusion pass.  Included by cogito.h.
 *
 * The reference declares two different enums named cg_fusion_type (include/cg_jit.h:65
 * and include/cg_fusion.h:17), so its two headers cannot be included together; here the
 * per-node mark is cg_node_fusion and cg_fusion_type is the group-level enum. */
#ifndef COGITO_JIT_H
#define COGITO_JIT_H

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------ symbolic */
typedef enum { DIM_CONSTANT, DIM_SYMBOLIC, DIM_INFERRED, DIM_BROADCAST } cg_dim_type;
typedef enum { EXPR_CONST, EXPR_VAR, EXPR_ADD, EXPR_SUB, EXPR_MUL, EXPR_DIV, EXPR_FLOORDIV,
               EXPR_MOD, EXPR_MAX, EXPR_MIN } cg_expr_type;
typedef struct cg_symbolic_expr {
  cg_expr_type type;
  union {
    int64_t constant;
    char* variable;
    struct { struct cg_symbolic_expr* left; struct cg_symbolic_expr* right; } binary;
  } data;
} cg_symbolic_expr;
typedef struct {
  cg_dim_type type; int64_t value; char* name; cg_symbolic_expr* expr;
  int64_t min_value, max_value; bool divisible_by; int64_t divisor;
} cg_symbolic_dim;
typedef struct { cg_symbolic_dim** dims; int ndim; uint64_t hash; } cg_symbolic_shape;
typedef struct { char* dim_name; int64_t expected_value; } cg_shape_guard;
typedef struct { cg_shape_guard* guards; int num_guards; void* specialized_kernel; } cg_shape_specialization;

cg_symbolic_dim* cg_dim_const(int64_t value);
cg_symbolic_dim* cg_dim_var(const char* name);
cg_symbolic_dim* cg_dim_inferred(cg_symbolic_expr* expr);        /* takes ownership of expr */
void cg_dim_constrain(cg_symbolic_dim* dim, int64_t min, int64_t max);
void cg_dim_set_divisor(cg_symbolic_dim* dim, int64_t divisor);
bool cg_dim_compatible(cg_symbolic_dim* a, cg_symbolic_dim* b);
int64_t cg_dim_resolve(cg_symbolic_dim* dim, int64_t* bindings, const char** binding_names, int num_bindings); /* -1: unbound or out of range */
void cg_dim_free(cg_symbolic_dim* dim);
cg_symbolic_expr* cg_expr_const(int64_t value);
cg_symbolic_expr* cg_expr_var(const char* name);
cg_symbolic_expr* cg_expr_add(cg_symbolic_expr* left, cg_symbolic_expr* right);
cg_symbolic_expr* cg_expr_sub(cg_symbolic_expr* left, cg_symbolic_expr* right);
cg_symbolic_expr* cg_expr_mul(cg_symbolic_expr* left, cg_symbolic_expr* right);
cg_symbolic_expr* cg_expr_div(cg_symbolic_expr* left, cg_symbolic_expr* right);
cg_symbolic_expr* cg_expr_floordiv(cg_symbolic_expr* left, cg_symbolic_expr* right);
cg_symbolic_expr* cg_expr_binary(cg_expr_type type, cg_symbolic_expr* left, cg_symbolic_expr* right);
/* the value; -1 (and CG_ERROR_INVALID_ARGUMENT) for an unbound variable or a division by zero, as in the reference */
int64_t cg_expr_eval(cg_symbolic_expr* expr, int64_t* bindings, const char** binding_names, int num_bindings);
/* the same with the outcome separate from the value: false when the expression cannot be evaluated */
bool cg_expr_try_eval(cg_symbolic_expr* expr, int64_t* bindings, const char** binding_names, int num_bindings, int64_t* out);
char* cg_expr_to_string(cg_symbolic_expr* expr);                 /* caller frees */
void cg_expr_free(cg_symbolic_expr* expr);
cg_symbolic_shape* cg_shape_new(cg_symbolic_dim** dims, int ndim);   /* takes ownership of the dims */
cg_symbolic_shape* cg_shape_from_ints(int* dims, int ndim);
cg_symbolic_shape* cg_shape_broadcast(cg_symbolic_shape* a, cg_symbolic_shape* b);
cg_symbolic_shape* cg_shape_matmul(cg_symbolic_shape* a, cg_symbolic_shape* b);
/* [N, C, H, W] -> [N, out_channels, (H + 2p - k) / s + 1, (W + 2p - k) / s + 1], square kernel */
cg_symbolic_shape* cg_shape_conv2d(cg_symbolic_shape* input, int out_channels, int kernel_size, int stride, int padding);
bool cg_shape_is_dynamic(cg_symbolic_shape* shape);
uint64_t cg_shape_hash(cg_symbolic_shape* shape);
bool cg_shape_to_ints(cg_symbolic_shape* shape, int* out_dims, int* out_ndim);
bool cg_shape_resolve(cg_symbolic_shape* shape, int64_t* bindings, const char** binding_names, int num_bindings, int* out_dims);
void cg_shape_free(cg_symbolic_shape* shape);
void cg_shape_print(cg_symbolic_shape* shape);
cg_shape_specialization* cg_shape_specialize(cg_symbolic_shape* shape, int64_t* bindings, const char** binding_names, int num_bindings);
bool cg_shape_guards_hold(cg_shape_specialization* spec, int64_t* bindings, const char** binding_names, int num_bindings);
bool cg_guards_check(cg_shape_specialization* spec, int64_t* bindings, const char** binding_names, int num_bindings);   /* same check, the reference's name */
void cg_shape_specialization_free(cg_shape_specialization* spec);

/* ----------------------------------------------------------------- JIT */
typedef enum {
  OP_NOOP = 0, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_NEG, OP_EXP, OP_LOG, OP_SQRT, OP_RSQRT,
  OP_RELU, OP_SIGMOID, OP_TANH, OP_GELU, OP_SOFTMAX, OP_MATMUL, OP_TRANSPOSE, OP_CONV2D, OP_MAXPOOL2D,
  OP_SUM, OP_MEAN, OP_MAX, OP_MIN, OP_COPY, OP_RESHAPE, OP_BROADCAST,
  OP_FUSED_ATTENTION, OP_FUSED_LAYERNORM, OP_FUSED_LAYERNORM_GELU_LINEAR,
  OP_FUSED_SOFTMAX_DROPOUT_RESIDUAL, OP_FUSED_QKV_ROPE, OP_CUSTOM
} cg_ir_opcode;
typedef enum { NODE_FUSION_NONE = 0, NODE_FUSION_VERTICAL, NODE_FUSION_HORIZONTAL, NODE_FUSION_CUSTOM,
               FUSION_VERTICAL = 1, FUSION_HORIZONTAL = 2 /* the reference's names for the two marks (include/cg_jit.h:65-70) */
} cg_node_fusion;
typedef enum { FUSION_NONE = 0, FUSION_ELEMENTWISE, FUSION_REDUCTION, FUSION_EPILOGUE, FUSION_ATTENTION,
               FUSION_LAYERNORM, FUSION_CUSTOM } cg_fusion_type;
typedef struct cg_ir_node {
  cg_ir_opcode opcode; int id;
  int* input_ids; int num_inputs;          /* tensor ids */
  int output_id; int output_shape[CG_MAX_DIMS]; int output_ndim;
  void* attributes; size_t attr_size;
  int schedule_order; bool can_fuse; cg_node_fusion fusion_type; struct cg_ir_node* fused_with;
  bool dead;
} cg_ir_node;
typedef struct {
  cg_ir_node** nodes; int num_nodes; int capacity;
  cg_tensor** tensors; int num_tensors; int tensor_capacity;     /* tensor id -> tensor (retained) */
  int* input_node_ids; int num_inputs;                           /* tensor ids with no producer */
  int* output_node_ids; int num_outputs;                         /* tensor ids marked as results */
  int opt_level;
} cg_ir_graph;
typedef enum { JIT_BACKEND_CPU, JIT_BACKEND_CUDA, JIT_BACKEND_METAL, JIT_BACKEND_VULKAN } cg_jit_backend;
typedef struct {
  cg_ir_graph* graph; cg_jit_backend backend;
  char* source_code; size_t source_len;
  void* compiled_module; void* compiled_kernel;
  bool is_compiled; int shared_memory_bytes; int registers_per_thread; int occupancy;
  uint64_t shape_hash; uint64_t pattern_hash;
} cg_jit_compiler;

void cg_jit_begin_trace(void);
cg_ir_graph* cg_jit_end_trace(void);
bool cg_jit_is_tracing(void);
/* Called by the tensor ops while tracing; also usable to build a graph by hand. */
void cg_jit_record(cg_ir_opcode op, cg_tensor** inputs, int num_inputs, cg_tensor* output, const void* attr, size_t attr_size);
cg_ir_graph* cg_ir_graph_new(void);
void cg_ir_graph_free(cg_ir_graph* graph);
cg_ir_node* cg_ir_node_new(cg_ir_opcode op);
void cg_ir_node_free(cg_ir_node* node);
int cg_ir_graph_tensor_id(cg_ir_graph* graph, cg_tensor* t);    /* registers t when unknown */
cg_ir_node* cg_ir_graph_add_node(cg_ir_graph* graph, cg_ir_opcode op, const int* input_ids, int num_inputs,
                                 int output_id, const void* attr, size_t attr_size);
void cg_ir_graph_mark_output(cg_ir_graph* graph, cg_tensor* t);
int cg_ir_graph_live_nodes(cg_ir_graph* graph);
void cg_ir_optimize(cg_ir_graph* graph, int opt_level);          /* 0 none, 1 dce+cse, >=2 + fusion marks */
void cg_ir_fuse_ops(cg_ir_graph* graph);
void cg_ir_dce(cg_ir_graph* graph);
void cg_ir_cse(cg_ir_graph* graph);
void cg_ir_graph_print(cg_ir_graph* graph);
const char* cg_ir_opcode_name(cg_ir_opcode op);
/* Interpreter over the graph's own tensors: recomputes every live node in order. */
bool cg_ir_execute(cg_ir_graph* graph);
cg_jit_compiler* cg_jit_compiler_new(cg_ir_graph* graph, cg_jit_backend backend);
bool cg_jit_compile(cg_jit_compiler* compiler);   /* CPU: cc + dlopen; CUDA: source only (the GPU package compiles it with NVRTC) */
bool cg_jit_run(cg_jit_compiler* compiler);       /* run the compiled CPU module over the graph's tensors */
void cg_jit_compiler_free(cg_jit_compiler* compiler);
char* cg_jit_codegen_c(cg_ir_graph* graph);
char* cg_jit_codegen_cuda(cg_ir_graph* graph);

/* -------------------------------------------------------------- fusion */
typedef struct cg_fusion_group {
  cg_ir_node** nodes; int num_nodes; int capacity;
  cg_fusion_type fusion_type; char* kernel_name; char* kernel_code;
  int* output_shape; int output_ndim;
  size_t memory_saved; size_t flops; float arithmetic_intensity;
  int schedule_priority; bool is_valid;
} cg_fusion_group;
typedef struct {
  cg_ir_graph* graph; cg_fusion_group** groups; int num_groups; int max_groups;
  int max_fusion_depth; bool enable_epilogue; bool enable_attention; bool aggressive;
} cg_fusion_pass;
cg_fusion_pass* cg_fusion_pass_new(cg_ir_graph* graph);
void cg_fusion_analyze(cg_fusion_pass* pass);
cg_fusion_group** cg_fusion_find_patterns(cg_ir_graph* graph, int* num_groups);
bool cg_fusion_can_fuse(cg_ir_node* a, cg_ir_node* b);
cg_fusion_group* cg_fusion_group_new(cg_ir_node** nodes, int count);
void cg_fusion_group_add(cg_fusion_group* group, cg_ir_node* node);
char* cg_fusion_generate_kernel(cg_fusion_group* group);
void cg_fusion_apply(cg_fusion_pass* pass);
void cg_fusion_group_free(cg_fusion_group* group);
void cg_fusion_pass_free(cg_fusion_pass* pass);
/* Pattern matchers anchored at one node (start_idx = index into graph->nodes): LayerNorm spelled
 * as MEAN, SUB, MUL, MEAN, [ADD], RSQRT+MUL or SQRT+DIV, [MUL], [ADD]; attention spelled as
 * [TRANSPOSE], MATMUL, [MUL | DIV], [ADD], SOFTMAX, MATMUL.  On a match *out_group (may be NULL)
 * receives a new group (FUSION_LAYERNORM / FUSION_ATTENTION) that the caller frees. */
bool cg_fusion_match_layernorm(cg_ir_graph* graph, int start_idx, cg_fusion_group** out_group);
bool cg_fusion_match_attention(cg_ir_graph* graph, int start_idx, cg_fusion_group** out_group);
/* MATMUL, [ADD bias], [RELU | SIGMOID | TANH | GELU] (FUSION_EPILOGUE); RELU, MUL mask, ADD (FUSION_ELEMENTWISE) */
bool cg_fusion_match_matmul_epilogue(cg_ir_graph* graph, int start_idx, cg_fusion_group** out_group);
bool cg_fusion_match_relu_dropout_add(cg_ir_graph* graph, int start_idx, cg_fusion_group** out_group);

/* ---- the reference's names for entry points that this library also has under other names ---- */
const char* cg_opcode_name(cg_ir_opcode op);                      /* = cg_ir_opcode_name */
/* Allocates the result of `op` (shape inferred), records the node when a trace is open, returns it. */
cg_tensor* cg_jit_record_op(cg_ir_opcode op, cg_tensor** inputs, int num_inputs, void* attributes, size_t attr_size);
/* Copies inputs into the graph's inputs, runs the compiled module (or the interpreter), copies the
 * graph's outputs out. */
void cg_jit_execute(cg_jit_compiler* compiler, cg_tensor** inputs, int num_inputs, cg_tensor** outputs, int num_outputs);
/* Linear-scan register assignment over the live nodes; results via the three readers below. */
void cg_ir_allocate_registers(cg_ir_graph* graph, int max_regs);
int cg_ir_register_of(cg_ir_graph* graph, int tensor_id);         /* >= 0, -1 spilled, -2 not planned */
int cg_ir_spill_count(cg_ir_graph* graph);
int cg_ir_registers_used(cg_ir_graph* graph);
void cg_symbolic_report_mismatch(cg_symbolic_shape* a, cg_symbolic_shape* b, const char* context);   /* to stderr */
/* Attention of [batch, seq, heads, d_head] tensors; the caller frees the result. */
cg_tensor* cg_flash_attn_forward(cg_tensor* q, cg_tensor* k, cg_tensor* v, float dropout_prob, float softmax_scale, bool causal);

#ifdef __cplusplus
}
#endif
#endif /* COGITO_JIT_H */
