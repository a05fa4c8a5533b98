/* Device layer of the cg_* C API: device discovery, memory, device tensors and the fp32 tensor
 * operations on them.  Surface of the reference's include/cg_cuda.h, cg_tensor_kernels.h and
 * cg_flash_attn_kernels.h.
 *
 * Two modes, chosen by cg_cuda_init():
 *  - device mode: the kernel library (libcogito_kernels.so, next to libcogito.so) was opened and
 *    reports at least one GPU.  cg_cuda_malloc is device memory, device tensors hold device
 *    pointers, every cg_cuda_* operation launches sm_100a kernels on the context's stream.
 *  - host mode (no GPU, no driver or no kernel library): the same calls work on host memory and
 *    compute with the host implementations, like the reference's simulation build
 *    (src/cuda/cg_cuda.c:56-171), so programs and tests run unchanged without a GPU.
 * cg_cuda_device_mode() tells which.  Setting the environment variable COGITO_FORCE_HOST=1 before
 * cg_cuda_init() keeps host mode on a machine that has a GPU. */
#ifndef COGITO_CUDA_H
#define COGITO_CUDA_H

#include "cogito.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { CG_DEVICE_CPU = 0, CG_DEVICE_CUDA = 1 } cg_device_type;

typedef struct {
  int device_id;
  int compute_capability_major, compute_capability_minor;
  size_t total_memory, free_memory;
  int multiprocessor_count, max_threads_per_block, warp_size;
  size_t shared_memory_per_block;
  char device_name[256];
  bool is_available;
} cg_cuda_device_info;

typedef struct {
  void* stream;          /* cudaStream_t of every launch and asynchronous copy of this API */
  void* cublas_handle;   /* always NULL: matrix products run on this library's tcgen05 GEMM */
  int device_id;
  bool initialized;
} cg_cuda_context;

typedef enum { CG_MEMCPY_HOST_TO_DEVICE, CG_MEMCPY_DEVICE_TO_HOST, CG_MEMCPY_DEVICE_TO_DEVICE } cg_memcpy_kind;

bool cg_cuda_init(void);
void cg_cuda_shutdown(void);
bool cg_cuda_is_available(void);
bool cg_cuda_device_mode(void);            /* true: a real GPU executes; false: host mode */
int cg_cuda_device_count(void);
cg_cuda_device_info cg_cuda_get_device_info(int device_id);
void cg_cuda_set_device(int device_id);
int cg_cuda_get_device(void);
cg_cuda_context* cg_cuda_get_context(void);

void* cg_cuda_malloc(size_t size);
void cg_cuda_free(void* ptr);
void* cg_cuda_malloc_host(size_t size);    /* page-locked in device mode */
void cg_cuda_free_host(void* ptr);
void cg_cuda_memcpy(void* dst, const void* src, size_t size, cg_memcpy_kind kind);
void cg_cuda_memcpy_async(void* dst, const void* src, size_t size, cg_memcpy_kind kind, void* stream);
void cg_cuda_memset(void* ptr, int value, size_t size);
void cg_cuda_device_synchronize(void);
void cg_cuda_stream_synchronize(void* stream);

/* Device tensors: the cg_tensor header lives on the host, data (and grad) on the device.
 * cg_tensor_free releases them like any other tensor. */
cg_tensor* cg_tensor_cuda_new(int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_cuda_zeros(int* shape, int ndim, bool requires_grad);
cg_tensor* cg_tensor_to_cuda(cg_tensor* t);
cg_tensor* cg_tensor_to_cpu(cg_tensor* t);
bool cg_tensor_is_cuda(cg_tensor* t);

const char* cg_cuda_get_last_error(void);
void cg_cuda_clear_error(void);
void cg_cuda_calculate_launch_dims(int n_elements, int* grid_size, int* block_size);
void cg_cuda_calculate_launch_dims_2d(int rows, int cols, int* grid_x, int* grid_y, int* block_x, int* block_y);

/* ---- fp32 tensor operations (operands made by cg_tensor_cuda_* / cg_tensor_to_cuda) ---- */
void cg_cuda_tensor_add(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_cuda_tensor_sub(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_cuda_tensor_mul(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_cuda_tensor_div(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_cuda_tensor_scale(cg_tensor* a, float scalar, cg_tensor* out);
void cg_cuda_tensor_exp(cg_tensor* a, cg_tensor* out);
void cg_cuda_tensor_log(cg_tensor* a, cg_tensor* out);
void cg_cuda_tensor_pow(cg_tensor* a, float power, cg_tensor* out);
void cg_cuda_tensor_sqrt(cg_tensor* a, cg_tensor* out);
void cg_cuda_tensor_abs(cg_tensor* a, cg_tensor* out);
/* axis < 0 reduces everything to out[0]; otherwise out has the shape of a without that axis */
void cg_cuda_tensor_sum(cg_tensor* a, int axis, cg_tensor* out);
void cg_cuda_tensor_mean(cg_tensor* a, int axis, cg_tensor* out);
void cg_cuda_tensor_max(cg_tensor* a, int axis, cg_tensor* out);
void cg_cuda_tensor_min(cg_tensor* a, int axis, cg_tensor* out);
/* [M,K] x [K,N]; in device mode three bf16 tensor-core products of a two-term split of each
 * operand (hi*hi + hi*lo + lo*hi, fp32 accumulation) give fp32-class accuracy.
 * cg_cuda_set_matmul_precision(1) uses one bf16 product instead (faster, ~3 significant digits). */
void cg_cuda_tensor_matmul(cg_tensor* a, cg_tensor* b, cg_tensor* out);
void cg_cuda_tensor_bmm(cg_tensor* a, cg_tensor* b, cg_tensor* out);    /* [B,M,K] x [B,K,N] */
void cg_cuda_tensor_transpose(cg_tensor* a, cg_tensor* out);            /* 2-D */
void cg_cuda_set_matmul_precision(int bf16_products);                   /* 3 (default) or 1 */

void cg_cuda_relu_forward(cg_tensor* input, cg_tensor* output);
void cg_cuda_relu_backward(cg_tensor* input, cg_tensor* grad_output, cg_tensor* grad_input);
void cg_cuda_sigmoid_forward(cg_tensor* input, cg_tensor* output);
void cg_cuda_sigmoid_backward(cg_tensor* output, cg_tensor* grad_output, cg_tensor* grad_input);
void cg_cuda_tanh_forward(cg_tensor* input, cg_tensor* output);
void cg_cuda_tanh_backward(cg_tensor* output, cg_tensor* grad_output, cg_tensor* grad_input);
void cg_cuda_gelu_forward(cg_tensor* input, cg_tensor* output);
void cg_cuda_gelu_backward(cg_tensor* input, cg_tensor* grad_output, cg_tensor* grad_input);
void cg_cuda_softmax_forward(cg_tensor* input, cg_tensor* output, int axis);
void cg_cuda_softmax_backward(cg_tensor* output, cg_tensor* grad_output, cg_tensor* grad_input, int axis);
/* rows of normalized_shape elements; mean / rstd ([rows]) may be NULL in the forward pass */
void cg_cuda_layernorm_forward(cg_tensor* input, cg_tensor* gamma, cg_tensor* beta, cg_tensor* output,
                               cg_tensor* mean, cg_tensor* rstd, float eps, int normalized_shape);
void cg_cuda_layernorm_backward(cg_tensor* grad_output, cg_tensor* input, cg_tensor* gamma, cg_tensor* mean,
                                cg_tensor* rstd, cg_tensor* grad_input, cg_tensor* grad_gamma, cg_tensor* grad_beta,
                                int normalized_shape);
void cg_cuda_rmsnorm_forward(cg_tensor* input, cg_tensor* weight, cg_tensor* output, float eps);

/* ---- attention on device tensors ([batch, seq, heads, d_head], fp32 in and out; the tcgen05
 * flash kernels compute in bf16 with fp32 accumulation; d_head 64 or 128 in device mode) ---- */
void cg_flash_attention_forward_cuda(cg_flash_attn_params* params);
void cg_flash_attention_forward_rope_cuda(cg_flash_attn_params* params, float* cos_cache, float* sin_cache,
                                          int position_offset);
void cg_flash_attention_backward_cuda(cg_flash_attn_params* params);
void cg_flash_attention_mqa_cuda(cg_flash_attn_params* params);
void cg_flash_attention_gqa_cuda(cg_flash_attn_params* params, int num_kv_groups);
void cg_flash_attention_sliding_window_cuda(cg_flash_attn_params* params, int window_size);
/* K / V are block pools [num_blocks, block_size, kv_heads, d_head]; block_tables is
 * [batch, ceil(max_context_len / block_size)] on the host */
void cg_flash_attention_paged_cuda(cg_flash_attn_params* params, int* block_tables, int block_size,
                                   int max_context_len);
/* x: [batch, seqlen, n_heads, d_head] in device memory, caches [positions, d_head/2] likewise */
void cg_rope_forward_cuda(float* x, int batch, int seqlen, int n_heads, int d_head, float* cos_cache,
                          float* sin_cache, int position_offset);
void cg_rope_backward_cuda(float* dx, int batch, int seqlen, int n_heads, int d_head, float* cos_cache,
                           float* sin_cache, int position_offset);
void cg_flash_attn_get_tile_sizes(int d_head, int sm_version, int* block_m, int* block_n);
size_t cg_flash_attn_estimate_shmem(int block_m, int block_n, int d_head);
bool cg_flash_attn_check_config(int block_m, int block_n, int d_head, size_t max_shmem);

#ifdef __cplusplus
}
#endif
#endif /* COGITO_CUDA_H */
