/* C interface of the sm_100a kernel library (libcogito_kernels.so).
 *
 * All functions take raw device pointers and a cudaStream_t passed as void*.
 * They return 0 on success or a negative code; cgk_last_error() gives the text.
 * The Python package calls these through ctypes; C and C++ callers include this
 * header and link the shared library.
 */
#ifndef COGITO_KERNELS_H
#define COGITO_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* cgk_last_error(void);
int cgk_version(void);
/* out[4] = {code, where, block, aux}; synchronises `stream`; clears the word. */
int cgk_read_status(int* out, void* stream);

/* ---- GEMM ------------------------------------------------------------- */
enum { CGK_ACT_NONE = 0, CGK_ACT_GELU = 1, CGK_ACT_RELU = 2, CGK_ACT_SILU = 3,
       CGK_ACT_SIGMOID = 4, CGK_ACT_TANH = 5 };

/* out[b,m,n] = epilogue( alpha * sum_k A(b,m,k) * B(b,n,k) )
 *   a_mn = 0: A is [M rows, K cols] with leading dimension lda   (K contiguous)
 *   a_mn = 1: A is [K rows, M cols] with leading dimension lda   (M contiguous)
 *   b_mn = 0: B is [N rows, K cols] with leading dimension ldb   (K contiguous)
 *   b_mn = 1: B is [K rows, N cols] with leading dimension ldb   (N contiguous)
 * epilogue, in this order:
 *   v = alpha*acc (+ bias[n]);  aux_out[m,n] = v (if given);  v = act(v);
 *   v *= act'(aux_in[m,n]) where act' is the derivative selected by dact (if given);
 *   v += residual[m,n] (if given);  out = accumulate ? out + v : v
 * bias / residual / aux tensors are bf16 unless bias_fp32 is set for the bias. */
typedef struct {
  const void* A;
  const void* B;
  void* out;
  int32_t M, N, K, batch;
  int64_t lda, ldb, ldc;
  int64_t strideA, strideB, strideC; /* batch strides, elements */
  int32_t a_mn, b_mn;
  int32_t out_fp32;
  int32_t accumulate;
  float alpha;
  const void* bias;
  int32_t bias_fp32;
  int32_t act;
  const void* residual;
  int64_t ldr;
  void* aux_out;
  int64_t ldaux;
  const void* aux_in;
  int64_t ldauxin;
  int32_t dact;
  int32_t force_simt; /* testing: use the CUDA-core fallback */
  int32_t max_ctas;   /* 0 = one persistent CTA per SM */
  /* Rotary embedding in the epilogue (the QKV projection): output columns [0, rope_cols) are heads of
   * rope_D (64 or 128) elements; element pairs (i, i + rope_D / 2) of a head are rotated by the angle
   * of position (row % rope_T) + rope_pos0, taken from fp32 tables [positions][rope_D / 2]
   * (rope_inverse: by the negative angle).  bf16 output only, no activation / residual / aux. */
  const float* rope_cos; const float* rope_sin;
  int32_t rope_cols, rope_D, rope_T, rope_pos0, rope_inverse;
  int32_t split_k;    /* fp32 accumulating outputs only: 0 = split the K range over idle SMs when the
                         output has few tiles (partial sums meet in the output through fp32 reductions,
                         so their order, and the last bits, can differ between runs), 1 = never, n = n slices */
} cgk_gemm_args;

int cgk_gemm_bf16(const cgk_gemm_args* args, void* stream);

/* ---- Fused tensor-parallel kernels (csrc/comm/fused_tp.cu) -------------------- */
/* All pointer tables are indexed by rank and hold addresses valid on THIS GPU
 * (peer mappings of symmetric memory); entry [rank] is the local buffer. */
typedef struct {
  int32_t rank, ranks;
  int32_t epoch;            /* > 0; one more than on the previous call with this workspace */
  int32_t chunk_rows;       /* rows per readiness flag, a multiple of 128 */
  const void* shard_ptrs[8];   /* [M/ranks, K] bf16 activation shard of each rank */
  void* signal_ptrs[8];        /* int32[2*ranks] per rank: ready words, then done words */
  void* chunk_flag_ptrs[8];    /* per rank: int32[ranks * ceil(rows/chunk_rows)] in symmetric memory */
  int32_t* done_count;         /* local int32[ranks], zero on entry, zero on exit */
  int32_t n_copy_ctas;         /* 0 = default */
  void* mc_gathered;           /* NVSwitch multicast address of the gathered buffer (which then must
                                  sit at the same offset of a symmetric buffer on every rank), or
                                  null: the shards are pulled with peer loads.  In multicast mode
                                  only shard_ptrs[rank] is read and it may be any local memory. */
} cgk_ag_args;

typedef struct {
  int32_t rank, ranks;
  int32_t queue_base;       /* value of *queue when the call starts: the sum over earlier calls
                               of (row blocks + CTAs of the launch); see cgk_gemm_rs_queue_step */
  void* partial_ptrs[8];    /* per rank: bf16 [M][ld] buffer that rank writes its partial product to */
  void* flag_ptrs[8];       /* per rank: int32[(M/ranks)/128] arrival counters, zero on entry and on exit */
  int64_t ld;               /* leading dimension of a partial row */
  const void* bias;         /* bf16 [N] or null, added after the reduction */
  const void* residual;     /* bf16 [M/ranks, ldr] or null */
  int64_t ldr;
  void* out;                /* bf16 [M/ranks, ldo] */
  int64_t ldo;
  int32_t n_reduce_ctas;    /* 0 = default */
  int32_t* queue;           /* local int32 work counter, zero before the first call */
  const void* mc_partial;   /* NVSwitch multicast address of the partial buffers (sum in the switch), or null */
} cgk_rs_args;

/* g->A is the LOCAL gathered buffer [M, K] (filled by the kernel, M = ranks * shard rows). */
int cgk_ag_gemm(const cgk_gemm_args* g, const cgk_ag_args* x, void* stream);
/* g describes this rank's partial product [M, N]; g->out is ignored; g->max_ctas > 0 caps the grid. */
int cgk_gemm_rs(const cgk_gemm_args* g, const cgk_rs_args* x, void* stream);
/* By how much one cgk_gemm_rs call with M rows advances *queue on the current device. */
int cgk_gemm_rs_queue_step(int M, int ranks, int max_ctas);

/* ---- Fused data-parallel optimizer step in buckets (csrc/comm/dp_adam.cu) --------- */
/* The flat parameter space [0, n) is cut into buckets of bucket_len elements (the last may be
 * shorter; n and bucket_len are multiples of 8 * ranks).  Inside bucket b of length len_b rank r
 * owns [b * bucket_len + r * len_b / ranks, + len_b / ranks); its reduced gradients, Adam moments
 * and fp32 master weights are stored bucket after bucket (n / ranks elements in all).  Pointer
 * tables are indexed by rank (peer mappings of symmetric memory). */
#define CGK_DP_MAX_BUCKETS 64
#define CGK_DP_MAX_CTAS 1024
typedef struct {
  int32_t rank, ranks;
  int32_t epoch;                   /* > 0, the same for all buckets of a step, +1 per step */
  int32_t bucket;                  /* index of the bucket */
  int32_t grid_ctas;               /* CTAs of this launch (a few: it runs beside the backward pass) */
  const void* grad_ptrs[8];        /* fp32 flat gradients of every rank */
  void* signal_ptrs[8];            /* cgk_dp_signal_bytes(ranks) bytes per rank, zero before the first call */
  float* gsum;                     /* local out: reduced gradients of the owned part of this bucket */
  int64_t begin, count;            /* the owned part: flat offset and length */
  float* block_part;               /* local scratch [2 * grid_ctas] for this bucket */
  void* arrive;                    /* local uint32 counter for this bucket, zero before the first call */
  float* stats;                    /* local out [2]: sum of squares and overflow flag of the owned part */
} cgk_dp_bucket_args;

typedef struct {
  int32_t rank, ranks, epoch, nbuckets;
  int32_t grid_ctas;               /* 0 = default */
  void* param_lp_ptrs[8];          /* bf16 flat parameters of every rank, or all null */
  void* param_fp_ptrs[8];          /* fp32 flat parameters of every rank (used when no bf16 copy) */
  void* signal_ptrs[8];
  float* master;                   /* local fp32 master weights of the owned parts [n / ranks], or null */
  float* m; float* v;              /* local Adam moments [n / ranks] */
  const float* gsum;               /* local reduced gradients [n / ranks] (from cgk_dp_bucket_reduce) */
  int64_t n, bucket_len;
  float lr, beta1, beta2, eps, weight_decay, max_grad_norm;
  float grad_mul;                  /* multiplies the summed gradient (1/ranks = mean) */
  float growth, backoff, min_scale, max_scale;
  int32_t window;
  void* scaler;                    /* local scaler state (cgk_scaler_state_bytes) */
  const float* bucket_stats;       /* local [nbuckets][2], written by cgk_dp_bucket_reduce */
  const float* ext_stats;          /* device {sum of squares, overflow} agreed by a larger group (tensor /
                                      pipeline parallel replica), or null: the group of this call decides */
  void* arrive;                    /* local uint32 counter, zero before the first call */
} cgk_dp_finish_args;

int cgk_dp_bucket_reduce(const cgk_dp_bucket_args* args, void* stream);
int cgk_dp_adam_finish(const cgk_dp_finish_args* args, void* stream);
int cgk_dp_signal_bytes(int ranks);

/* Tensor-parallel serving: x[t,:] += sum over ranks of partial_p[t,:], then (w given)
 * h = rmsnorm(x) * w, in one launch over peer memory (one-shot all-reduce, sums in rank order).
 * partial[p] / sig[p]: rank p's slot of this call and its flag array (ranks ints) as mapped
 * here; slots alternate between two buffers; counters: two local ints, zero before the first
 * call, in which the kernel numbers the calls (so that a CUDA graph can replay it). */
int cgk_serve_allreduce(const void* const* partial, int* const* sig, int rank, int ranks, int* counters, void* x,
                        const void* w, void* h, int rows, int cols, float eps, void* stream);

/* ---- Flash attention ------------------------------------------------------ */
/* Tensors are bf16 [batch, seq, heads, head_dim] with head_dim contiguous and the
 * given element strides (batch, token, head), all multiples of 8.  lse is fp32
 * [batch, heads_q, seq_q].  head_dim 64 or 128.  Key k is visible to query q iff
 * (!causal || k <= q + Tk - Tq) and (window < 0 || |k - (q + Tk - Tq)| <= window).
 * alibi_slopes: fp32 [heads_q] or null; bias = slope * (k - (q + Tk - Tq)). */
typedef struct {
  const void* q; const void* k; const void* v;
  void* o;
  float* lse;
  int32_t B, Hq, Hk, Tq, Tk, D;
  int64_t q_bs, q_ts, q_hs;
  int64_t k_bs, k_ts, k_hs;
  int64_t v_bs, v_ts, v_hs;
  int64_t o_bs, o_ts, o_hs;
  float scale;
  int32_t causal;
  int32_t window;
  const float* alibi_slopes;
  /* backward only */
  const void* d_o;            /* same layout as o */
  void* dq; void* dk; void* dv;
  int64_t dq_bs, dq_ts, dq_hs;
  int64_t dk_bs, dk_ts, dk_hs;
  int64_t dv_bs, dv_ts, dv_hs;
  float* delta;               /* scratch fp32 [B, Hq, Tq] */
  float* dq_accum;            /* scratch fp32 [B, Tq, Hq, D] */
} cgk_flash_args;

int cgk_flash_forward(const cgk_flash_args* args, void* stream);
int cgk_flash_backward(const cgk_flash_args* args, void* stream);

/* ---- Serving: INT4 weights, paged INT4 KV cache, sampling, speculative decoding ---- */
/* Packed INT4 format: groups of `group` consecutive elements of the row-major tensor,
 * scale = absmax / 7 (1 when < 1e-10), q = clamp(round(x / scale), -8, 7), two values per
 * byte with the even index in the low nibble, fp32 scales. */
int cgk_int4_quantize(const float* x, long long n, int group, void* packed, float* scales, void* stream);
int cgk_int4_dequantize(const void* packed, const float* scales, long long n, int group, float* out_f32,
                        void* out_bf16, void* stream);
/* Tile-major reordering of reference-format weights for cgk_int4_gemm: packed [K, N/2] bytes +
 * fp32 scales per flat group -> [N/128][K/64][4608] (64 rows of 64 bytes, then fp32 scales
 * [64][2]).  N % 128 == 0, K % 64 == 0, group a multiple of 64 dividing N. */
long long cgk_int4_tiles_bytes(int K, int N);
int cgk_int4_tile_weights(const void* packed, const float* scales, int K, int N, int group, void* tiles, void* stream);
/* out[M,N] (bf16, leading dimension ldo) = x[M,K] (bf16) . dequant(w)[K,N] (+ bias).
 * acc (fp32 [M, N]) and counters (int32 [cgk_int4_gemm_counters(M, N)]) serve split-K: zero
 * before the first call, left zero by every call; both may be null, which forces one split.
 * splits 0 = pick so that the SMs are covered in whole waves. */
long long cgk_int4_gemm_counters(int M, int N);
int cgk_int4_gemm(const void* x, long long ldx, const void* w_tiles, float* acc, int* counters, void* out,
                  long long ldo, const void* bias, int M, int N, int K, int splits, void* stream);
/* The same product with the weights on the M side of the tensor core (time grows with the rows
 * of x instead of always paying for 128), the group scale folded into x and a bit-trick-only
 * nibble conversion.  Needs group % 128 == 0.  Tiles: [N/128][K/64][4352] (4096 bytes of
 * nibbles [feature][8 words], then 64 fp32 scales); acc / counters as for cgk_int4_gemm. */
long long cgk_int4_wa_tiles_bytes(int K, int N);
int cgk_int4_wa_tile_weights(const void* packed, const float* scales, int K, int N, int group, void* tiles, void* stream);
int cgk_int4_wa_gemm(const void* x, long long ldx, const void* tiles, float* acc, int* counters, void* out,
                     long long ldo, const void* bias, int M, int N, int K, int splits, void* stream);

/* One layer of a paged INT4 KV cache: pages[num_pages][page_size][heads][D/2] bytes and
 * scales[num_pages][page_size][heads][D/group] fp32 for K and V; page_table[batch][max_pages]
 * maps logical to pool pages; lengths[batch] tokens are valid.  D 64 or 128. */
typedef struct {
  void* k_pages; void* v_pages; float* k_scales; float* v_scales;
  const int32_t* page_table; const int32_t* lengths;
  int32_t batch, heads, D, group, page_size, max_pages;
} cgk_kv_args;
/* k_new, v_new: bf16 [batch, T, heads, D]; written at positions lengths[b] .. lengths[b]+T-1
 * (lengths is not changed: cgk_spec_accept or the caller commits). */
int cgk_kv_int4_append(const cgk_kv_args* a, const void* k_new, const void* v_new, int T, void* stream);
long long cgk_kv_int4_attention_scratch_floats(int batch, int Hq, int Tq, int D, int splits);
/* q, out: bf16 [batch, Tq, Hq, D]; the Tq newest tokens are already in the cache; query t sees
 * keys 0 .. lengths[b] + t.  Hq a multiple of heads (grouped-query attention). */
int cgk_kv_int4_attention(const cgk_kv_args* a, const void* q, void* out, int Tq, int Hq, float scale,
                          int splits, float* scratch, void* stream);
/* Per row: logits / temperature -> top_k (1..1024, 0 = 1024) -> top_p -> sample.  temperature
 * <= 0: argmax.  Random stream = (seed, row, *step).  probs_out: fp32 [rows, V] or null. */
int cgk_sample(const void* logits, int logits_bf16, long long ld, int rows, int V, float temperature, int top_k,
               float top_p, unsigned long long seed, const long long* step, int* tokens, float* probs_out,
               void* stream);
/* draft_tokens [B, gamma]; q [B, gamma, V]; p [B, gamma+1, V].  Accept token i with probability
 * min(1, p/q); replace the first rejected one by a sample of max(0, p - q); append a bonus token
 * when all pass.  out_tokens [B, gamma+1]; lengths[b] += n_accepted[b] + 1 (null: untouched);
 * stats[0] += gamma, stats[1] += accepted (null: untouched). */
int cgk_spec_accept(const int* draft_tokens, const float* q, const float* p, int batch, int gamma, int V,
                    unsigned long long seed, const long long* step, int* n_accepted, int* out_tokens,
                    int* lengths, int* stats, void* stream);
/* Self-test of the bounded waits: one thread waits until *flag >= want or budget_ns (<= 5 s)
 * passes; on a timeout the status word reads {2, 900, 0, want} and *reached (optional) is 0. */
int cgk_selftest_bounded_wait(const int* flag, int want, unsigned long long budget_ns, int* reached, void* stream);
/* mask [(L+n), (L+n)], 0 or -1e9: causal prefix; tree node i sees the prefix, its ancestors, itself. */
int cgk_tree_mask(const int* parents, int n, int L, float* mask_f32, void* mask_bf16, void* stream);

/* ---- Fused row kernel of the fusion pass (csrc/kernels/softmax_ce.cu) --------------------- */
/* out = softmax(x) * w + residual per row, w = mul (tensor) or the dropout mask of (seed, index)
 * scaled by 1 / (1 - p); dtype 0 fp32, 1 bf16; mul / residual may be null.  This is the kernel
 * behind the "fused_softmax_dropout_residual" group (softmax -> mul -> add). */
int cgk_softmax_dropout_residual(int dtype, const void* x, const void* mul, const void* residual, void* out,
                                 int R, int V, float p, unsigned long long seed, void* stream);
int cgk_softmax_dropout_residual_backward(int dtype, const void* x, const void* mul, const void* dy, void* dx,
                                          int R, int V, float p, unsigned long long seed, void* stream);

#ifdef __cplusplus
}
#endif
#endif
