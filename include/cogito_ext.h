/* cogito_ext.h — second half of the C API (included by cogito.h): precision,
 * quantisation, attention helpers, data, checkpoints, inference, parallel schedules,
 * memory pools, symbolic shapes, JIT, profiler.  See cogito.h for conventions. */
#ifndef COGITO_EXT_H
#define COGITO_EXT_H

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------- bf16 */
typedef uint16_t cg_bf16;
typedef uint8_t cg_fp8_e4m3;
typedef uint8_t cg_fp8_e5m2;
cg_bf16 cg_fp32_to_bf16(float f);          /* round to nearest even */
float cg_bf16_to_fp32(cg_bf16 h);
/* the reference's spellings (static inline there, include/cg_bf16.h:22-32) */
static inline cg_bf16 cg_float_to_bf16(float f) { return cg_fp32_to_bf16(f); }
static inline float cg_bf16_to_float(cg_bf16 b) { return cg_bf16_to_fp32(b); }
/* The reference's layout (include/cg_bf16.h:38-50): bf16 values and gradient, fp32 master copy and fp32 gradient
 * accumulator of a trainable tensor (null otherwise); `master` names data_fp32. */
typedef struct {
  cg_bf16* data; cg_bf16* grad;
  union { float* data_fp32; float* master; };
  float* grad_fp32;
  int shape[CG_MAX_DIMS]; int ndim; int size; bool requires_grad; bool has_master_copy;
} cg_tensor_bf16;
typedef struct {
  /* second names: the reference's (include/cg_bf16.h) */
  union { cg_tensor** params; cg_tensor** master_params; };
  cg_tensor_bf16** model_params; int num_params;
  float loss_scale;
  union { float min_loss_scale; float loss_scale_min; };
  union { float max_loss_scale; float loss_scale_max; };
  float scale_factor;
  union { int scale_window; int scale_growth_interval; };
  union { int steps_since_overflow; int steps_since_update; };
  bool found_overflow; float max_grad_norm; float learning_rate;
  union { int num_skipped; int overflow_count; };
  int num_steps;
  void* optimizer;              /* the caller's; cg_mp_step applies its own update rule */
} cg_mixed_precision;
cg_tensor_bf16* cg_tensor_bf16_new(int* shape, int ndim, bool requires_grad);
cg_tensor_bf16* cg_tensor_bf16_from_fp32(cg_tensor* fp32);
cg_tensor* cg_tensor_bf16_to_fp32(cg_tensor_bf16* bf16);
void cg_tensor_bf16_free(cg_tensor_bf16* t);
cg_mixed_precision* cg_mixed_precision_new(cg_tensor** params, int num_params);
cg_tensor_bf16* cg_mp_forward(cg_mixed_precision* mp, cg_tensor_bf16* (*model_fn)(void*, cg_tensor_bf16*),
                              void* model, cg_tensor_bf16* input);
bool cg_mp_backward(cg_mixed_precision* mp, cg_tensor_bf16* loss);   /* false on overflow */
void cg_mp_step(cg_mixed_precision* mp);
bool cg_mp_check_overflow(cg_mixed_precision* mp);
void cg_mixed_precision_free(cg_mixed_precision* mp);
void cg_bf16_add(cg_tensor_bf16* a, cg_tensor_bf16* b, cg_tensor_bf16* out);
void cg_bf16_mul(cg_tensor_bf16* a, cg_tensor_bf16* b, cg_tensor_bf16* out);
void cg_bf16_matmul(cg_tensor_bf16* a, cg_tensor_bf16* b, cg_tensor_bf16* out);
void cg_bf16_gelu(cg_tensor_bf16* a, cg_tensor_bf16* out);
void cg_bf16_layernorm(cg_tensor_bf16* x, cg_tensor_bf16* gamma, cg_tensor_bf16* beta, float eps, cg_tensor_bf16* out);

/* ----------------------------------------------------------- quantisation */
typedef enum { QUANT_NONE = 0, QUANT_INT8, QUANT_INT4, QUANT_NF4, QUANT_FP8_E4M3, QUANT_FP8_E5M2,
               QUANT_GPTQ, QUANT_AWQ, QUANT_GGML } cg_quant_type;
typedef struct {
  uint8_t* data; float* scales; float* zeros;
  int* shape; int ndim; int size;
  cg_quant_type quant_type; int group_size; int num_groups; bool symmetric;
} cg_tensor_quant;
typedef struct {
  uint8_t* k_cache; uint8_t* v_cache; float* k_scales; float* v_scales;
  int current_len, max_seq_len, num_layers, n_heads, head_dim, group_size;
} cg_kv_cache_int4;
typedef struct { float* min_vals; float* max_vals; union { float* abs_max; float* absmax; }; int channels; int num_samples; } cg_quant_calibration;
cg_tensor_quant* cg_quantize_int4(cg_tensor* tensor, int group_size);
cg_tensor_quant* cg_quantize_gptq(cg_tensor* tensor, cg_tensor* hessian, int group_size, int bits);
cg_tensor_quant* cg_quantize_awq(cg_tensor* tensor, cg_tensor* activations, int group_size);
cg_tensor_quant* cg_quantize_nf4(cg_tensor* tensor, int group_size);
cg_tensor* cg_dequantize(cg_tensor_quant* quant);
void cg_tensor_quant_free(cg_tensor_quant* quant);
void cg_matmul_int4(cg_tensor* input, cg_tensor_quant* weight, cg_tensor* output);   /* weight [K, N] */
void cg_gemv_int4(cg_tensor* input, cg_tensor_quant* weight, cg_tensor* output);
void cg_attention_int4_kv(cg_tensor* Q, cg_kv_cache_int4* kv_cache, int layer_idx, cg_tensor* output);
cg_kv_cache_int4* cg_kv_cache_int4_new(int num_layers, int max_seq_len, int n_heads, int head_dim, int group_size);
void cg_kv_cache_int4_append(cg_kv_cache_int4* cache, int layer_idx, cg_tensor* new_k, cg_tensor* new_v);
void cg_kv_cache_int4_get(cg_kv_cache_int4* cache, int layer_idx, cg_tensor* k_out, cg_tensor* v_out);
void cg_kv_cache_int4_reset(cg_kv_cache_int4* cache);
void cg_kv_cache_int4_truncate(cg_kv_cache_int4* cache, int new_len);   /* roll back rejected positions */
void cg_kv_cache_int4_free(cg_kv_cache_int4* cache);
cg_quant_calibration* cg_calibration_new(int channels);
void cg_calibration_update(cg_quant_calibration* calib, cg_tensor* activations);
void cg_calibration_compute_scales(cg_quant_calibration* calib, float* scales, float* zeros, int group_size);
void cg_calibration_free(cg_quant_calibration* calib);

/* -------------------------------------------------------------- attention */
/* ATTN_MASK_* are the reference's enumerators (include/cg_flash_attn.h:40-45); CG_MASK_* name the same values */
typedef enum { ATTN_MASK_NONE = 0, ATTN_MASK_CAUSAL = 1, ATTN_MASK_SLIDING_WINDOW = 2, ATTN_MASK_CUSTOM = 3,
               CG_MASK_NONE = 0, CG_MASK_CAUSAL = 1, CG_MASK_SLIDING_WINDOW = 2, CG_MASK_CUSTOM = 3 } cg_attention_mask_type;
/* Tile shape of the sm_100a attention kernels, under the reference's macro names (64 x 64 tiles and 4 / 8 warps there,
 * include/cg_flash_attn.h:18-21, include/cg_flash_attn_kernels.h:24-30): 128 query rows x 128 keys per tile (two query
 * tiles per CTA), the whole head dimension (up to 128) in one piece, 12 warps. */
#define FLASH_BLOCK_M_DEFAULT 128
#define FLASH_BLOCK_N_DEFAULT 128
#define FLASH_BLOCK_M FLASH_BLOCK_M_DEFAULT
#define FLASH_BLOCK_N FLASH_BLOCK_N_DEFAULT
#define FLASH_BLOCK_K 128
#define FLASH_WARPS 12
#define FA_BLOCK_M 128
#define FA_BLOCK_N 128
#define FA_BLOCK_K 128
#define FA_THREADS 384
#define FA_WARPS 12
/* use_register_tile, use_persistent and sm_count are the reference's names (include/cg_flash_attn.h:27-35) */
typedef struct {
  int block_m, block_n, num_warps, num_stages;
  union { bool use_register_tiling; bool use_register_tile; };
  int split_k;
  bool use_persistent;          /* more query tiles than SMs: a CTA loops over tiles */
  int sm_count;
} cg_flash_attn_config;
typedef struct {
  cg_tensor* Q; cg_tensor* K; cg_tensor* V; cg_tensor* O;        /* [batch, seq, heads, d_head] */
  cg_tensor* dO; cg_tensor* dQ; cg_tensor* dK; cg_tensor* dV;
  cg_tensor* L;                                                   /* logsumexp [batch, heads, seq] */
  cg_tensor* mask;
  int batch_size, seqlen_q, seqlen_k, n_heads;
  union { int n_kv_heads; int n_heads_k; };                      /* n_heads_k, scale: the reference's names */
  int d_head;
  union { float softmax_scale; float scale; };
  float dropout_prob;
  cg_attention_mask_type mask_type; int window_size;
  float* alibi_slopes;
  cg_flash_attn_config config;
  /* reference fields (include/cg_flash_attn.h:51-88): softmax_lse points at L's values; the attention functions carry
   * dropout_prob but apply no dropout, so the mask stays null */
  bool is_training; float* softmax_lse; float* dropout_mask;
  /* CG_FLASH_TENSOR_MODE (set by cg_flash_attn_params_new): the operand slots hold tensors.  Anything else - a block a
   * caller zero-filled and set up the reference's way - means they hold raw fp32 arrays [batch, seq, heads, d_head],
   * described by batch_size .. d_head, with the output in O and the log-sum-exp rows in softmax_lse (host memory). */
  unsigned int operand_mode;
} cg_flash_attn_params;
#define CG_FLASH_TENSOR_MODE 0x43475450u
void cg_flash_attention_forward(cg_flash_attn_params* params);
void cg_flash_attention_forward_cpu(cg_flash_attn_params* params);
void cg_flash_attention_backward(cg_flash_attn_params* params);
void cg_flash_attention_backward_cpu(cg_flash_attn_params* params);
void cg_flash_attention_mqa(cg_flash_attn_params* params);
void cg_flash_attention_gqa(cg_flash_attn_params* params, int num_kv_groups);
cg_flash_attn_params* cg_flash_attn_params_new(cg_tensor* Q, cg_tensor* K, cg_tensor* V,
                                               cg_attention_mask_type mask_type, float dropout_prob);
cg_flash_attn_config cg_flash_attn_autotune(int seqlen_q, int seqlen_k, int d_head, int sm_count);
size_t cg_flash_attn_shared_mem(int block_m, int block_n, int d_head);
void cg_flash_attn_params_free(cg_flash_attn_params* params);
void cg_apply_rope(float* Q, float* K, int seqlen, int n_heads, int d_head, int position_offset, float rope_theta);
void cg_rope_precompute_freqs(float* cos_cache, float* sin_cache, int max_seqlen, int d_head, float theta);
void cg_alibi_bias(float* bias, int seqlen_q, int seqlen_k, int n_heads, float* slopes);
void cg_alibi_slopes(float* slopes, int n_heads);

/* ------------------------------------------------------------------- data */
typedef struct { cg_tensor* images; cg_tensor* labels; int num_samples; int rows, cols; } cg_mnist;
typedef struct {
  cg_tensor* data; cg_tensor* labels; int batch_size; bool shuffle; unsigned int seed;
  int* indices; union { int position; int current_idx; }; int num_samples; cg_tensor* batch_data; cg_tensor* batch_labels;
} cg_data_iter;
typedef cg_data_iter cg_dataloader_state;
typedef struct { cg_data_iter it; int epoch; } cg_dataloader;
cg_mnist* cg_mnist_load(const char* images_path, const char* labels_path);
void cg_mnist_free(cg_mnist* mnist);
void cg_mnist_get_batch(cg_mnist* mnist, int start_idx, int batch_size, cg_tensor* images_out, cg_tensor* labels_out);
cg_tensor* cg_labels_to_onehot(cg_tensor* labels, int num_classes);
void cg_augment_gaussian_noise(cg_tensor* t, float std, unsigned int seed);
void cg_augment_horizontal_flip(cg_tensor* t, float prob, unsigned int seed);   /* [N, rows*cols] square images */
cg_data_iter* cg_data_iter_new(cg_tensor* data, cg_tensor* labels, int batch_size, bool shuffle, unsigned int seed);
bool cg_data_iter_next(cg_data_iter* iter, cg_tensor** batch_data, cg_tensor** batch_labels);
void cg_data_iter_reset(cg_data_iter* iter, unsigned int seed);
void cg_data_iter_free(cg_data_iter* iter);
cg_dataloader* cg_dataloader_new(cg_tensor* data, cg_tensor* labels, int batch_size, bool shuffle, unsigned int seed);
bool cg_dataloader_next(cg_dataloader* loader, cg_tensor** batch_data, cg_tensor** batch_labels, int* actual_batch_size);
void cg_dataloader_reset(cg_dataloader* loader);
int cg_dataloader_num_batches(cg_dataloader* loader);
void cg_dataloader_free(cg_dataloader* loader);
cg_tensor* cg_tensor_onehot(cg_tensor* labels, int num_classes);
int cg_tensor_argmax(cg_tensor* t, int sample_idx, int num_classes);
float cg_compute_accuracy(cg_tensor* logits, cg_tensor* labels, int num_classes);

/* ------------------------------------------------------------ checkpoints */
#define CG_MODEL_MAGIC 0x434F4731u   /* "COG1" */
typedef struct { uint32_t magic; uint32_t version; uint32_t num_tensors; uint64_t total_size; } cg_model_header;
typedef struct { char name[64]; int32_t ndim; int32_t shape[8]; int32_t dtype; uint64_t offset; uint64_t size_bytes; } cg_tensor_entry;
void cg_save_model(const char* filename, cg_tensor** tensors, const char** names, int count);
void cg_load_model(const char* filename, cg_tensor*** out_tensors, char*** out_names, int* out_count);

/* ------------------------------------------------ sampling / speculative */
/* The second line holds the reference's fields (include/cg_speculative.h); its tree functions are declared only, and the
 * functions of this library keep parents and one distribution per node instead and leave them null / 0. */
typedef struct cg_token_tree {
  int* tokens; float** probs; int* parents; int depth; int num_tokens; int capacity; int vocab_size;
  float* draft_probs; float* target_probs; bool* accepted; cg_tensor* hidden_states; int* branch_points; int num_branches;
} cg_token_tree;
/* A model is a callback: logits_out[n_positions * vocab] for the LAST n_positions of ids. */
typedef void (*cg_logits_fn)(void* model, const int* ids, int len, int n_positions, float* logits_out);
typedef struct {
  void* draft_model; void* target_model; int gamma;
  float temperature, top_p; int top_k;
  int total_draft_tokens, accepted_draft_tokens, num_steps; float avg_acceptance_rate;
  cg_logits_fn draft_fn; cg_logits_fn target_fn; int vocab_size; unsigned int rng_state;
  /* reference fields (include/cg_speculative.h:37-50), kept so that code written against it compiles: the reference
   * sets accept_threshold to 0 and reads none of the four (src/inference/speculative.c:40); neither does this library */
  float accept_threshold; bool use_typical_sampling; void* draft_kv_cache; void* target_kv_cache;
} cg_speculative_decoder;
/* feature_proj, uncertainty_head and feature_cache are the reference's fields (include/cg_speculative.h); its EAGLE
 * functions are declared only and nothing reads them there or here */
typedef struct { void* base_draft; int max_branch; int* branching; void* feature_proj; void* uncertainty_head; float* feature_cache; } cg_eagle_draft;
cg_speculative_decoder* cg_speculative_decoder_new(void* draft_model, void* target_model, int gamma);
void cg_speculative_set_models(cg_speculative_decoder* d, cg_logits_fn draft_fn, cg_logits_fn target_fn, int vocab_size);
cg_tensor* cg_speculative_generate(cg_speculative_decoder* decoder, cg_tensor* input_ids, int max_new_tokens,
                                   float temperature, float top_p);
int cg_speculative_step(cg_speculative_decoder* decoder, cg_tensor* input_ids, cg_token_tree* tree);
cg_token_tree* cg_draft_generate(cg_speculative_decoder* decoder, cg_tensor* input_ids);
int cg_target_verify(cg_speculative_decoder* decoder, cg_tensor* input_ids, cg_token_tree* tree);
void cg_speculative_decoder_free(cg_speculative_decoder* decoder);
cg_token_tree* cg_token_tree_new(int depth);
void cg_token_tree_add_token(cg_token_tree* tree, int token, float* probs);          /* child of the newest token */
int cg_token_tree_add_child(cg_token_tree* tree, int parent, int token, float* probs); /* parent -1 = prefix; returns the node id */
cg_tensor* cg_token_tree_to_tensor(cg_token_tree* tree);
void cg_token_tree_free(cg_token_tree* tree);
cg_tensor* cg_tree_attention_mask(cg_token_tree* tree, int seqlen);     /* [1,1,L+g,L+g], 0 / -1e9 */
cg_tensor* cg_forward_tree_attention(void* model, cg_tensor* input, cg_tensor* tree_mask);
cg_eagle_draft* cg_eagle_draft_new(void* base_draft);
cg_token_tree* cg_eagle_generate_tree(cg_eagle_draft* eagle, cg_tensor* input, int max_depth);
int* cg_eagle_compute_branching(cg_eagle_draft* eagle, cg_tensor* features);
void cg_eagle_draft_free(cg_eagle_draft* eagle);
void cg_sample_seed(unsigned int seed);
int cg_sample_temperature(float* logits, int vocab_size, float temperature);
int cg_sample_top_p(float* logits, int vocab_size, float top_p);
int cg_sample_top_k(float* logits, int vocab_size, int top_k);
int cg_sample_typical(float* logits, int vocab_size, float typical_p);
float cg_acceptance_prob(float draft_prob, float target_prob);
int cg_sample_corrected(float* draft_probs, float* target_probs, int vocab_size);

/* ---------------------------------------------------- parallel schedules */
typedef enum { PARALLEL_DATA, PARALLEL_TENSOR, PARALLEL_PIPELINE } cg_parallel_mode;
/* cg_schedule_op with its eight operations and the `op` field are the reference's (include/cg_pipeline.h:121-136);
 * SCHEDULE_OPTIMIZER closes a rank's program here, and `action` / cg_schedule_action name the same field and type. */
typedef enum { SCHEDULE_FORWARD = 0, SCHEDULE_BACKWARD, SCHEDULE_SEND_FWD, SCHEDULE_RECV_FWD,
               SCHEDULE_SEND_BWD, SCHEDULE_RECV_BWD, SCHEDULE_WAIT, SCHEDULE_SYNC, SCHEDULE_OPTIMIZER } cg_schedule_op;
typedef cg_schedule_op cg_schedule_action;
typedef struct { union { cg_schedule_op op; cg_schedule_op action; }; int microbatch_id; int stage_id; } cg_schedule_step;
typedef struct { cg_parallel_mode mode; int world_size; int rank; int* ranks; void* comm; void* stream; } cg_distributed_group;
/* The double-buffer and event fields are the reference's (include/cg_pipeline.h:33-58); the in-process executor of this
 * library keeps its buffers in `impl` of the pipeline and leaves them null. */
typedef struct {
  int stage_id; void* layers; int num_layers;
  cg_tensor** send_buffers_a; cg_tensor** send_buffers_b; cg_tensor** recv_buffers_a; cg_tensor** recv_buffers_b;
  cg_tensor** grad_send_a; cg_tensor** grad_send_b; cg_tensor** grad_recv_a; cg_tensor** grad_recv_b;
  void* compute_event; void* comm_stream; void* send_event_a; void* send_event_b; void* recv_event_a; void* recv_event_b;
} cg_pipeline_stage;
typedef struct {
  int num_stages, micro_batch_size, num_microbatches, global_batch_size;
  cg_pipeline_stage* stages; cg_schedule_step* schedule;
  union { int schedule_len; int schedule_length; };              /* schedule_length: the reference's name */
  cg_distributed_group* pp_group; cg_distributed_group* dp_group;
  bool use_recompute; void* activation_cache;
  float last_loss; void* impl;
  cg_distributed_group* tp_group; int local_stage_id;            /* reference fields (include/cg_pipeline.h:72-77) */
} cg_pipeline_parallel;
typedef struct { cg_distributed_group* group; int shard_dim; bool input_is_parallel; bool output_is_parallel; } cg_tensor_parallel_linear;
typedef struct {
  int dp_size, tp_size, pp_size; int dp_rank, tp_rank, pp_rank; int world_size, world_rank;
  cg_distributed_group* dp_group; cg_distributed_group* tp_group; cg_distributed_group* pp_group;
  cg_pipeline_parallel* pipeline;                                /* reference field (include/cg_pipeline.h:200) */
} cg_3d_parallel;
cg_pipeline_parallel* cg_pipeline_new(int num_stages, int num_microbatches);
void cg_pipeline_set_stage(cg_pipeline_parallel* pp, int stage_id, void* layers, int num_layers);   /* layers: cg_sequential* */
void cg_pipeline_forward_backward(cg_pipeline_parallel* pp, cg_tensor* input, cg_tensor* target);
void cg_pipeline_allreduce_grads(cg_pipeline_parallel* pp);
void cg_pipeline_free(cg_pipeline_parallel* pp);
/* Schedule of ONE stage (stage_id of the returned steps): warm-up = S-1-stage forwards. */
cg_schedule_step* cg_pipeline_gen_1f1b_stage(int num_stages, int num_microbatches, int stage, int* schedule_len);
cg_schedule_step* cg_pipeline_gen_1f1b(int num_stages, int num_microbatches, int* schedule_len);   /* stage 0 */
cg_schedule_step* cg_pipeline_gen_interleaved(int num_stages, int num_virtual, int num_microbatches, int* schedule_len);
/* stage_id of the returned steps is the virtual stage chunk * num_stages + rank */
cg_schedule_step* cg_pipeline_gen_interleaved_stage(int num_stages, int num_virtual, int num_microbatches, int rank, int* schedule_len);
void cg_pipeline_set_loss(cg_pipeline_parallel* pp, int kind);     /* 0 MSE (default), 1 softmax cross-entropy */
void cg_pipeline_send_activation(cg_pipeline_parallel* pp, int dest_stage, cg_tensor* activation, int microbatch_id);
void cg_pipeline_recv_activation(cg_pipeline_parallel* pp, int src_stage, cg_tensor* buffer, int microbatch_id);
void cg_pipeline_send_gradient(cg_pipeline_parallel* pp, int dest_stage, cg_tensor* gradient, int microbatch_id);
void cg_pipeline_recv_gradient(cg_pipeline_parallel* pp, int src_stage, cg_tensor* buffer, int microbatch_id);
cg_tensor* cg_tp_column_parallel_forward(cg_tensor_parallel_linear* tp, cg_tensor* input, cg_tensor* weight);
cg_tensor* cg_tp_row_parallel_forward(cg_tensor_parallel_linear* tp, cg_tensor* input, cg_tensor* weight);
cg_3d_parallel* cg_3d_parallel_new(int dp_size, int tp_size, int pp_size);
void cg_3d_parallel_init_from_world(cg_3d_parallel* ctx, int world_size, int world_rank);
void cg_3d_parallel_free(cg_3d_parallel* ctx);

/* ---------------------------------------------------------------- memory */
/* The reference's four arenas (include/cg_memory.h:48-53) all live in the device pool here; CG_ARENA_HOST
 * selects the pinned-host pool of the planner. */
typedef enum { CG_ARENA_DEFAULT = 0, CG_ARENA_PARAM, CG_ARENA_ACTIVATION, CG_ARENA_GRADIENT,
               CG_ARENA_DEVICE = 0, CG_ARENA_HOST = 4 } cg_arena_type;
/* Size classes of the caching pool: powers of two from 2^CG_MIN_BIN to 2^CG_MAX_BIN bytes plus the three exact sizes
 * (the reference stops at 2^36, include/cg_memory.h:32-35,84-86).  The buddy allocator hands out blocks from
 * 2^CG_BUDDY_MIN_ORDER bytes up to the largest power of two that fits its region; CG_BUDDY_MAX_ORDER bounds that. */
#define CG_SUBBIN_768 768
#define CG_SUBBIN_1024 1024
#define CG_SUBBIN_4096 4096
#define CG_NUM_SUBBINS 3
#define CG_MIN_BIN 5
#define CG_MAX_BIN 40
#define CG_NUM_BINS (CG_MAX_BIN - CG_MIN_BIN + 1)
#define CG_BUDDY_MIN_ORDER 8
#define CG_BUDDY_MAX_ORDER 40
#define CG_BUDDY_NUM_ORDERS (CG_BUDDY_MAX_ORDER - CG_BUDDY_MIN_ORDER + 1)
/* The counters and pointers the reference exposes (include/cg_memory.h:73-133), kept current by the functions below;
 * the bins, free lists and lifetime tables themselves are private to the library (created by the *_new functions only). */
typedef struct cg_buddy_allocator {
  void* base_ptr; size_t total_size; size_t allocated; size_t buddy_splits; size_t buddy_coalesces;
} cg_buddy_allocator;
typedef struct cg_memory_pool {
  cg_buddy_allocator* buddy;                  /* null: the pool caches whole blocks; the buddy allocator is used on its own */
  size_t total_allocated, total_in_use, peak_usage, num_allocs, num_frees, cache_hits, cache_misses, subbin_hits, buddy_coalesces;
} cg_memory_pool;
typedef struct cg_memory_planner {
  cg_memory_pool* device_pool; cg_memory_pool* host_pool;
  bool graph_captured; float frag_threshold; bool defrag_enabled; int num_tensors;
} cg_memory_planner;
typedef struct {
  size_t total_allocated, total_cached, peak_allocated; int num_allocs, num_frees, cache_hits, cache_misses;
  int buddy_splits, buddy_coalesces; float fragmentation;
  /* the reference's names (include/cg_memory.h:303-310): bytes handed out, their peak, hits per 100 requests, size
   * classes that hold cached blocks */
  size_t total_in_use, peak_usage, cache_hit_rate; int num_bins_used;
} cg_memory_stats;
cg_memory_pool* cg_memory_pool_new(void);
void* cg_pool_alloc(cg_memory_pool* pool, size_t size);
void cg_pool_free(cg_memory_pool* pool, void* ptr);
void cg_pool_trim(cg_memory_pool* pool);
void cg_memory_pool_free(cg_memory_pool* pool);
void* cg_pool_alloc_subbin(cg_memory_pool* pool, size_t size);
int cg_subbin_index(size_t size);                        /* 768 -> 0, 1024 -> 1, 4096 -> 2, else -1 */
void* cg_pool_alloc_arena(cg_memory_pool* pool, size_t size, cg_arena_type arena);
void cg_pool_free_arena(cg_memory_pool* pool, void* ptr, cg_arena_type arena);
cg_buddy_allocator* cg_buddy_new(void* base, size_t size);
void* cg_buddy_alloc(cg_buddy_allocator* buddy, size_t size);
void cg_buddy_free(cg_buddy_allocator* buddy, void* ptr, size_t size);
void cg_buddy_destroy(cg_buddy_allocator* buddy);
int cg_buddy_splits(cg_buddy_allocator* buddy);
int cg_buddy_coalesces(cg_buddy_allocator* buddy);
cg_memory_planner* cg_memory_planner_new(void);
void cg_memory_plan_analyze(cg_memory_planner* planner, void* ir_graph);
void* cg_planned_alloc(cg_memory_planner* planner, size_t size, int tensor_id);
void cg_planned_free(cg_memory_planner* planner, void* ptr, int tensor_id);
void cg_memory_planner_free(cg_memory_planner* planner);
void cg_memory_sliding_compact(cg_memory_planner* planner);
bool cg_memory_needs_compact(cg_memory_pool* pool, float threshold);
void cg_cuda_graph_capture_begin(cg_memory_planner* planner);
void cg_cuda_graph_capture_end(cg_memory_planner* planner);
void cg_cuda_graph_replay(cg_memory_planner* planner);
bool cg_cuda_graph_needs_update(cg_memory_planner* planner);
float cg_memory_fragmentation(cg_memory_pool* pool);
void cg_memory_defrag(cg_memory_planner* planner);
void cg_memory_maybe_defrag(cg_memory_planner* planner);
cg_memory_stats cg_memory_get_stats(cg_memory_planner* planner);
void cg_memory_print_stats(cg_memory_planner* planner);
void cg_analyze_tensor_lifetimes(cg_memory_planner* planner, void* ir_graph);
void cg_find_reuse_opportunities(cg_memory_planner* planner);
bool cg_can_reuse_memory(cg_memory_planner* planner, int tensor_a, int tensor_b);
cg_memory_pool* cg_memory_planner_pool(cg_memory_planner* planner, cg_arena_type arena);
size_t cg_memory_plan_bytes(cg_memory_planner* planner);                 /* slab size of the current plan */
size_t cg_memory_plan_offset(cg_memory_planner* planner, int tensor_id); /* (size_t)-1 when unplanned */
void* cg_planned_lookup(cg_memory_planner* planner, int tensor_id);      /* current address (moves on compaction) */

/* --------------------------------------------------------------- profiler */
/* The reference's public profiler state (include/cg_profiler.h:13-30): one entry per named region in first-use order,
 * kept current by the functions below (the event slots stay null: regions are timed on the host clock here, device
 * time per layer is the Python profiler's job).  g_profiler names the library's instance. */
typedef struct { char name[64]; void* start_event; void* stop_event; float total_ms; int count; } cg_layer_stat;
typedef struct { cg_layer_stat* layers; int num_layers; int capacity; bool enabled; int current_epoch; } cg_profiler;
cg_profiler* cg_profiler_state(void);
#define g_profiler (*cg_profiler_state())
void cg_profiler_init(void);
void cg_profiler_enable(bool enable);
void cg_profiler_begin_layer(const char* name);
void cg_profiler_end_layer(const char* name);
void cg_profiler_step_end(void);
void cg_profiler_report(void);
void cg_profiler_reset(void);
double cg_profiler_total_ms(const char* name);
int cg_profiler_count(const char* name);

#ifdef __cplusplus
}
#endif

#include "cogito_jit.h"

#endif /* COGITO_EXT_H */
