/* cogito.h — C API of the host runtime (libcogito.so).
 *
 * One header for the whole cg_* surface: tensors, arena, autograd, layers, losses,
 * optimizers, data, checkpoints, quantisation, sampling / speculative decoding,
 * pipeline schedules, memory pools, symbolic shapes, the JIT IR, the profiler.
 * Function names, argument orders and the documented struct fields follow the
 * reference library so that programs written against it recompile against this one.
 *
 * Semantics that differ on purpose (each fixes a defect of the reference):
 *  - there is ONE autograd: layers record themselves on the tensor tape, so
 *    cg_backward(loss) reaches every parameter of a cg_sequential;
 *  - the upstream gradient of every backward function is read from ->grad;
 *  - cg_tensor_matmul honours leading batch dimensions, cg_tensor_cat any dimension;
 *  - every layer draws its initial weights from its own random stream;
 *  - cg_kv_cache_int4_append advances the length once per token (layer 0), not per call.
 */
#ifndef COGITO_H
#define COGITO_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COGITO_VERSION_MAJOR 1
#define COGITO_VERSION_MINOR 0
#define COGITO_VERSION_PATCH 0
#define COGITO_API_VERSION 1
/* binds an exported function to a symbol version (GNU toolchains); a no-op elsewhere */
#if defined(__linux__) && defined(__GNUC__)
#define CG_API_VERSIONed(func, ver) __asm__(".symver " #func "," #func "@" #ver)
#else
#define CG_API_VERSIONed(func, ver)
#endif

typedef enum {
  CG_SUCCESS = 0, CG_ERROR_NULL_POINTER, CG_ERROR_SHAPE_MISMATCH, CG_ERROR_OUT_OF_MEMORY,
  CG_ERROR_INVALID_ARGUMENT, CG_ERROR_FILE_NOT_FOUND, CG_ERROR_INVALID_FORMAT, CG_ERROR_TIMEOUT
} cg_error;
const char* cg_error_string(cg_error err);
cg_error cg_last_error(void);              /* of the calling thread; reading it clears it */
void cg_manual_seed(unsigned int seed);    /* seeds the per-layer initialisation streams */

/* ------------------------------------------------------------------ arena */
#define CG_ARENA_DEFAULT_ALIGNMENT 16
typedef struct cg_arena_block {
  unsigned char* data; size_t size; size_t used; struct cg_arena_block* next;
} cg_arena_block;
typedef struct cg_arena {
  cg_arena_block* first; cg_arena_block* current;
  size_t default_block_size; size_t total_allocated; size_t total_used;
} cg_arena;
cg_arena* cg_arena_new(size_t initial_size);
void* cg_arena_alloc(cg_arena* arena, size_t size, size_t alignment);
#define cg_arena_alloc_default(arena, size) cg_arena_alloc(arena, size, CG_ARENA_DEFAULT_ALIGNMENT)
void cg_arena_clear(cg_arena* arena);
void cg_arena_free(cg_arena* arena);
size_t cg_arena_total_allocated(cg_arena* arena);
size_t cg_arena_total_used(cg_arena* arena);

/* ----------------------------------------------------------------- tensor */
#define CG_MAX_DIMS 8
#define CG_MAX_PARENTS 4
typedef struct cg_tensor cg_tensor;
typedef void (*cg_backward_fn)(cg_tensor* self);
struct cg_tensor {
  float* data; float* grad;
  int shape[CG_MAX_DIMS]; int strides[CG_MAX_DIMS]; int ndim; int size;
  bool requires_grad; cg_backward_fn backward_fn;
  cg_tensor* parents[CG_MAX_PARENTS]; int num_parents; void* backward_ctx;
  int ref_count; bool is_view; cg_arena* arena;
};
cg_tensor* cg_tensor_new(int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_zeros(int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_ones(int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_full(int* shape, int ndim, float value, bool requires_grad);
cg_tensor* cg_tensor_rand(int* shape, int ndim, unsigned int seed, bool requires_grad);
cg_tensor* cg_tensor_randn(int* shape, int ndim, unsigned int seed, bool requires_grad);
cg_tensor* cg_tensor_from_data(float* data, int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_clone(cg_tensor* t);
cg_tensor* cg_tensor_zeros_arena(cg_arena* arena, int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_randn_arena(cg_arena* arena, int* shape, int ndim, unsigned int seed, bool requires_grad);
void cg_tensor_retain(cg_tensor* t);
void cg_tensor_release(cg_tensor* t);
void cg_tensor_free(cg_tensor* t);
int cg_tensor_live_count(void);            /* live tensors (leak check) */
void cg_tensor_add(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_tensor_sub(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_tensor_mul(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_tensor_div(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_tensor_scale(cg_tensor* a, float scalar, cg_tensor* out);
void cg_tensor_matmul(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_tensor_transpose(cg_tensor* a, cg_tensor* out);
void cg_tensor_sum(cg_tensor* a, int axis, cg_tensor* out);   /* axis < 0: all */
void cg_tensor_mean(cg_tensor* a, int axis, cg_tensor* out);
void cg_tensor_max(cg_tensor* a, int axis, cg_tensor* out);
void cg_tensor_exp(cg_tensor* a, cg_tensor* out);
void cg_tensor_log(cg_tensor* a, cg_tensor* out);
void cg_tensor_pow(cg_tensor* a, float power, cg_tensor* out);
void cg_tensor_zero_grad(cg_tensor* t);
void cg_tensor_print(cg_tensor* t, const char* name);
float cg_tensor_get(cg_tensor* t, int* indices);
void cg_tensor_set(cg_tensor* t, int* indices, float value);
void cg_tensor_reshape(cg_tensor* t, int* new_shape, int new_ndim);
bool cg_tensor_shape_equal(cg_tensor* a, cg_tensor* b);
bool cg_broadcast_shapes(int* shape_a, int ndim_a, int* shape_b, int ndim_b, int* out_shape, int* out_ndim);
void cg_broadcast_strides(int* shape, int ndim, int* out_shape, int out_ndim, int* out_strides);
cg_tensor* cg_tensor_add_broadcast(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_tensor_sub_broadcast(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_tensor_mul_broadcast(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_tensor_div_broadcast(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_tensor_stack(cg_tensor** tensors, int count);
cg_tensor* cg_tensor_cat(cg_tensor** tensors, int count, int dim);

/* --------------------------------------------------------------- autograd */
cg_tensor* cg_add(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_sub(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_mul(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_matmul(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_sum_all(cg_tensor* a);
cg_tensor* cg_mean_all(cg_tensor* a);
cg_tensor* cg_exp(cg_tensor* a);
cg_tensor* cg_log_op(cg_tensor* a);
cg_tensor* cg_pow_op(cg_tensor* a, float p);
void cg_backward(cg_tensor* loss);
void cg_graph_init(void);
void cg_graph_reset(void);
bool cg_graph_is_active(void);
void cg_graph_register(cg_tensor* t, cg_tensor** parents, int num_parents);
void cg_graph_backward(cg_tensor* loss);
cg_tensor* cg_graph_add(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_graph_mul(cg_tensor* a, cg_tensor* b);
cg_tensor* cg_graph_matmul(cg_tensor* a, cg_tensor* b);
/* Central-difference check of forward_fn's input gradient (fp64 accumulation). */
bool cg_grad_check(void (*forward_fn)(cg_tensor* in, cg_tensor* out), cg_tensor* input,
                   cg_tensor* grad_output, float epsilon, float tolerance);

/* ----------------------------------------------------------------- layers */
/* Ownership, as in the reference (src/layers/linear.c:60-97): forward() returns a tensor whose first reference is
 * the caller's (release it when done); the layer keeps references of its own to its last input and output until the
 * next forward() or cg_layer_free().  cg_sequential_forward releases the intermediate outputs itself and hands the last
 * one to the caller. */
typedef struct cg_layer cg_layer;
struct cg_layer {
  const char* name;
  cg_tensor* weights; cg_tensor* bias;
  cg_tensor* input; cg_tensor* output;
  cg_tensor* (*forward)(cg_layer* self, cg_tensor* input);
  void (*backward)(cg_layer* self, cg_tensor* grad_output);
  void (*free)(cg_layer* self);
  int (*num_params)(cg_layer* self);
  cg_tensor** (*get_params)(cg_layer* self);
};
void cg_layer_free(cg_layer* layer);
void cg_layer_zero_grad(cg_layer* layer);
typedef struct { cg_layer base; int in_features; int out_features; cg_tensor* param_ptrs[2]; } cg_linear;
typedef struct { cg_layer base; cg_tensor* mask; } cg_relu;
typedef struct { cg_layer base; } cg_sigmoid;
typedef struct { cg_layer base; } cg_tanh_layer;
typedef struct { cg_layer base; } cg_softmax;
typedef struct { cg_layer base; float p; bool training; cg_tensor* mask; } cg_dropout;
typedef struct {
  cg_layer base; int num_features; float epsilon; float momentum;
  cg_tensor* running_mean; cg_tensor* running_var;
  union { cg_tensor* x_norm; cg_tensor* input_normalized; };    /* input_normalized: the reference's name */
  cg_tensor* std_inv;
  bool training; cg_tensor* param_ptrs[2];
  cg_tensor* batch_mean; cg_tensor* batch_var;                   /* reference fields: mean / biased variance of the last pass */
} cg_batchnorm;
typedef struct { cg_layer base; int normalized_shape; float epsilon; cg_tensor* inv_rms; cg_tensor* param_ptrs[1]; } cg_rmsnorm;
typedef struct { cg_layer base; } cg_swiglu;
typedef struct {
  cg_layer base; int in_channels, out_channels, kernel_size, stride, padding;
  cg_tensor* col_buffer; cg_tensor* param_ptrs[2];
} cg_conv2d;
typedef struct { cg_layer base; int kernel_size, stride; int* max_indices; } cg_maxpool2d;
typedef struct { cg_layer base; int input_shape[CG_MAX_DIMS]; int input_ndim; } cg_flatten;
typedef struct { cg_layer base; cg_layer** layers; int num_layers; int capacity; cg_tensor** param_cache; } cg_sequential;
cg_linear* cg_linear_new(int in_features, int out_features, bool bias);
cg_relu* cg_relu_new(void);
cg_sigmoid* cg_sigmoid_new(void);
cg_tanh_layer* cg_tanh_new(void);
cg_softmax* cg_softmax_new(void);
cg_dropout* cg_dropout_new(float p);
void cg_dropout_set_training(cg_dropout* layer, bool training);
cg_batchnorm* cg_batchnorm_new(int num_features, float epsilon, float momentum);
void cg_batchnorm_set_training(cg_batchnorm* layer, bool training);
cg_rmsnorm* cg_rmsnorm_new(int normalized_shape, float epsilon);
cg_swiglu* cg_swiglu_new(void);
cg_tensor* cg_swiglu_forward_split(cg_tensor* input);
cg_conv2d* cg_conv2d_new(int in_channels, int out_channels, int kernel_size, int stride, int padding, bool use_bias);
cg_maxpool2d* cg_maxpool2d_new(int kernel_size, int stride);
cg_flatten* cg_flatten_new(void);
cg_sequential* cg_sequential_new(void);
void cg_sequential_add(cg_sequential* seq, cg_layer* layer);
cg_tensor* cg_sequential_forward(cg_sequential* seq, cg_tensor* input);
void cg_sequential_backward(cg_sequential* seq, cg_tensor* grad_output);
void cg_sequential_free(cg_sequential* seq);
void cg_sequential_zero_grad(cg_sequential* seq);
int cg_sequential_num_params(cg_sequential* seq);
cg_tensor** cg_sequential_get_params(cg_sequential* seq);

typedef struct {
  /* hidden_dim / intermediate_dim are the reference's names (include/cg_transformer.h:19-34); hidden_size /
   * intermediate_size name the same two fields */
  union { int hidden_dim; int hidden_size; };
  int num_heads, num_kv_heads, head_dim;
  union { int intermediate_dim; int intermediate_size; };
  float norm_eps, dropout_prob;
  bool use_bias, pre_norm, use_rms_norm, use_swiglu;
} cg_transformer_config;
typedef struct {
  cg_layer base; cg_transformer_config config;
  cg_layer* norm1; cg_layer* norm2;
  /* attn_*_proj / mlp_* are the reference's names (include/cg_transformer.h); a cg_linear starts with its cg_layer */
  union { cg_linear* q_proj; cg_layer* attn_q_proj; }; union { cg_linear* k_proj; cg_layer* attn_k_proj; };
  union { cg_linear* v_proj; cg_layer* attn_v_proj; }; union { cg_linear* o_proj; cg_layer* attn_o_proj; };
  union { cg_linear* gate_proj; cg_layer* mlp_gate; }; union { cg_linear* up_proj; cg_layer* mlp_up; };
  union { cg_linear* down_proj; cg_layer* mlp_down; };
  cg_tensor** param_cache; int n_params;
  /* reference fields; the block applies its activation and dropout itself and leaves these null */
  cg_layer* act_fn; cg_layer* drop1; cg_layer* drop2;
} cg_transformer_block;
cg_transformer_block* cg_transformer_block_new(cg_transformer_config config);
cg_tensor* cg_transformer_forward(cg_layer* layer, cg_tensor* input, cg_tensor* mask);   /* input [seq, hidden] */

/* ----------------------------------------------------------------- losses */
typedef enum { CG_REDUCTION_NONE = 0, CG_REDUCTION_MEAN = 1, CG_REDUCTION_SUM = 2 } cg_reduction;
cg_tensor* cg_mse_loss(cg_tensor* pred, cg_tensor* target, cg_reduction reduction);
cg_tensor* cg_cross_entropy_loss(cg_tensor* pred, cg_tensor* target, bool from_logits, cg_reduction reduction);
cg_tensor* cg_softmax_cross_entropy_loss(cg_tensor* logits, cg_tensor* target, cg_reduction reduction);
cg_tensor* cg_bce_loss(cg_tensor* pred, cg_tensor* target, cg_reduction reduction);
cg_tensor* cg_bce_with_logits_loss(cg_tensor* logits, cg_tensor* target, cg_reduction reduction);
cg_tensor* cg_l1_loss(cg_tensor* pred, cg_tensor* target, cg_reduction reduction);
cg_tensor* cg_smooth_l1_loss(cg_tensor* pred, cg_tensor* target, float beta, cg_reduction reduction);

/* ------------------------------------------------------------- optimizers */
typedef struct cg_optimizer cg_optimizer;
struct cg_optimizer {
  float learning_rate; cg_tensor** params; int num_params; int t;
  bool use_mixed_precision; float loss_scale; int scale_window; float scale_factor; int scale_backoff;
  bool use_master_weights; cg_tensor** master_params; float max_grad_norm;
  void (*step)(cg_optimizer* self); void (*zero_grad)(cg_optimizer* self); void (*free)(cg_optimizer* self);
};
typedef struct { cg_optimizer base; float momentum; float weight_decay; bool nesterov; cg_tensor** velocities; } cg_sgd;
typedef struct { cg_optimizer base; float beta1, beta2, epsilon, weight_decay; cg_tensor** m; cg_tensor** v; } cg_adam;
cg_sgd* cg_sgd_new(cg_tensor** params, int num_params, float lr, float momentum, float weight_decay, bool nesterov);
cg_sgd* cg_sgd_new_for_sequential(cg_sequential* model, float lr, float momentum, float weight_decay, bool nesterov);
cg_adam* cg_adam_new(cg_tensor** params, int num_params, float lr, float beta1, float beta2, float epsilon, float weight_decay);
cg_adam* cg_adam_new_for_sequential(cg_sequential* model, float lr, float beta1, float beta2, float epsilon, float weight_decay);
void cg_optimizer_step(cg_optimizer* opt);
void cg_optimizer_zero_grad(cg_optimizer* opt);
void cg_optimizer_free(cg_optimizer* opt);
void cg_optimizer_step_lr(cg_optimizer* opt, int current_step, int step_size, float gamma);
void cg_optimizer_exp_lr(cg_optimizer* opt, float initial_lr, float gamma);
void cg_optimizer_enable_loss_scaling(cg_optimizer* opt, float init_scale, float factor, int window);
void cg_optimizer_enable_master_weights(cg_optimizer* opt);
bool cg_optimizer_update_scale(cg_optimizer* opt, float grad_norm);   /* true: skip this step */

#ifdef __cplusplus
}
#endif

#include "cogito_ext.h"
#include "cogito_cuda.h"

#endif /* COGITO_H */
