/* A walk through the host runtime's subsystems, compiled and run under AddressSanitizer and
 * UndefinedBehaviorSanitizer by tests/test_capi_sanitizers_cpu.py: tensors and the tape, the
 * memory pool and buddy allocator, INT4 quantisation and the KV cache, tracing and both code
 * generators, symbolic shapes, samplers, the 1F1B schedule, checkpoints and the device layer in
 * host mode.  Exit code 0 = every check held (the sanitizers abort on their own findings). */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "cogito.h"

#define CHECK(cond) do { if (!(cond)) { fprintf(stderr, "check failed at line %d: %s\n", __LINE__, #cond); return 1; } } while (0)

static int tensors_and_tape(void) {
  int sa[2] = {5, 7}, sb[2] = {7, 3};
  cg_tensor* a = cg_tensor_randn(sa, 2, 1, true);
  cg_tensor* b = cg_tensor_randn(sb, 2, 2, true);
  cg_tensor* y = cg_matmul(a, b);
  CHECK(y && y->shape[0] == 5 && y->shape[1] == 3);
  cg_tensor* sq = cg_mul(y, y);
  cg_tensor* loss = cg_mean_all(sq);
  CHECK(loss && loss->size == 1);
  cg_backward(loss);
  CHECK(a->grad && b->grad);
  float g = 0;
  for (int i = 0; i < a->size; ++i) g += fabsf(a->grad[i]);
  CHECK(g > 0);
  /* every node keeps a reference to its parents: the caller drops its own */
  cg_tensor_free(loss); cg_tensor_free(sq); cg_tensor_free(y); cg_tensor_free(a); cg_tensor_free(b);
  cg_arena* arena = cg_arena_new(1024);
  for (int i = 0; i < 50; ++i) CHECK(cg_arena_alloc_default(arena, 100 + i) != NULL);
  cg_tensor* t = cg_tensor_zeros_arena(arena, sa, 2, false);
  CHECK(t && t->data[34] == 0.0f);
  cg_arena_clear(arena);
  cg_arena_free(arena);
  return 0;
}

static int pools(void) {
  cg_memory_pool* pool = cg_memory_pool_new();
  void* p[64];
  for (int round = 0; round < 3; ++round) {
    for (int i = 0; i < 64; ++i) { p[i] = cg_pool_alloc(pool, (size_t)32 << (i % 12)); CHECK(p[i]); memset(p[i], i, (size_t)32 << (i % 12)); }
    for (int i = 0; i < 64; i += 2) cg_pool_free(pool, p[i]);
    for (int i = 1; i < 64; i += 2) cg_pool_free(pool, p[i]);
  }
  cg_pool_trim(pool);
  cg_memory_pool_free(pool);
  const size_t span = 1 << 16;
  void* base = malloc(span);
  cg_buddy_allocator* buddy = cg_buddy_new(base, span);
  void* x = cg_buddy_alloc(buddy, 100), *y = cg_buddy_alloc(buddy, 5000), *z = cg_buddy_alloc(buddy, 64);
  CHECK(x && y && z);
  memset(x, 1, 100); memset(y, 2, 5000); memset(z, 3, 64);
  cg_buddy_free(buddy, y, 5000); cg_buddy_free(buddy, x, 100); cg_buddy_free(buddy, z, 64);
  CHECK(cg_buddy_splits(buddy) > 0 && cg_buddy_coalesces(buddy) == cg_buddy_splits(buddy));
  void* whole = cg_buddy_alloc(buddy, span);
  CHECK(whole == base);
  cg_buddy_free(buddy, whole, span);
  cg_buddy_destroy(buddy);
  free(base);
  return 0;
}

static int quant_and_cache(void) {
  int sw[2] = {64, 128}, sx[2] = {3, 64}, so[2] = {3, 128};
  cg_tensor* w = cg_tensor_randn(sw, 2, 3, false);
  cg_tensor* x = cg_tensor_randn(sx, 2, 4, false);
  cg_tensor* out = cg_tensor_zeros(so, 2, false);
  cg_tensor_quant* q = cg_quantize_int4(w, 128);
  CHECK(q);
  cg_matmul_int4(x, q, out);
  cg_tensor* deq = cg_dequantize(q);
  cg_tensor* ref = cg_tensor_zeros(so, 2, false);
  cg_tensor_matmul(x, deq, ref);
  for (int i = 0; i < out->size; ++i) CHECK(fabsf(out->data[i] - ref->data[i]) < 1e-3f);
  cg_tensor_quant* nf = cg_quantize_nf4(w, 64);
  CHECK(nf);
  cg_tensor_quant_free(nf);
  cg_tensor_quant_free(q);
  cg_tensor_free(deq); cg_tensor_free(ref); cg_tensor_free(out); cg_tensor_free(x); cg_tensor_free(w);
  cg_kv_cache_int4* kv = cg_kv_cache_int4_new(2, 8, 2, 32, 32);
  int st[2] = {2, 32}, sk[3] = {8, 2, 32};
  for (int t = 0; t < 8; ++t) for (int layer = 0; layer < 2; ++layer) {
    cg_tensor* k = cg_tensor_randn(st, 2, 10 + t, false);
    cg_kv_cache_int4_append(kv, layer, k, k);
    cg_tensor_free(k);
  }
  cg_tensor* ko = cg_tensor_zeros(sk, 3, false), *vo = cg_tensor_zeros(sk, 3, false);
  cg_kv_cache_int4_get(kv, 1, ko, vo);
  CHECK(fabsf(ko->data[0] - vo->data[0]) < 1e-6f);
  cg_kv_cache_int4_truncate(kv, 5);
  cg_kv_cache_int4_reset(kv);
  cg_tensor_free(ko); cg_tensor_free(vo);
  cg_kv_cache_int4_free(kv);
  return 0;
}

static int tracing_and_shapes(void) {
  int s[2] = {6, 6};
  cg_tensor* a = cg_tensor_randn(s, 2, 5, false), *b = cg_tensor_randn(s, 2, 6, false);
  cg_jit_begin_trace();
  cg_tensor* in2[2] = {a, b};
  cg_tensor* mm = cg_jit_record_op(OP_MATMUL, in2, 2, NULL, 0);
  cg_tensor* in1[2] = {mm, a};
  cg_tensor* ad = cg_jit_record_op(OP_ADD, in1, 2, NULL, 0);
  cg_tensor* in0[1] = {ad};
  cg_tensor* re = cg_jit_record_op(OP_RELU, in0, 1, NULL, 0);
  cg_tensor* in3[1] = {re};
  cg_tensor* dead = cg_jit_record_op(OP_EXP, in3, 1, NULL, 0);
  cg_ir_graph* g = cg_jit_end_trace();
  CHECK(g && g->num_nodes == 4);
  cg_fusion_group* grp = NULL;
  CHECK(cg_fusion_match_matmul_epilogue(g, 0, &grp) && grp->num_nodes == 3);
  cg_fusion_group_free(grp);
  cg_ir_allocate_registers(g, 2);
  CHECK(cg_ir_registers_used(g) <= 2);
  cg_ir_optimize(g, 2);
  char* c_src = cg_jit_codegen_c(g), *cu_src = cg_jit_codegen_cuda(g);
  CHECK(c_src && cu_src && strstr(c_src, "jit_kernel") && strstr(cu_src, "__global__"));
  free(c_src); free(cu_src);
  CHECK(cg_ir_execute(g));
  cg_ir_graph_free(g);
  cg_tensor_free(mm); cg_tensor_free(ad); cg_tensor_free(re); cg_tensor_free(dead);
  cg_tensor_free(a); cg_tensor_free(b);
  cg_symbolic_dim* dims[4] = {cg_dim_var("N"), cg_dim_const(3), cg_dim_var("H"), cg_dim_const(28)};
  cg_symbolic_shape* in = cg_shape_new(dims, 4);
  cg_symbolic_shape* out = cg_shape_conv2d(in, 8, 5, 1, 2);
  CHECK(out && out->ndim == 4 && out->dims[3]->value == 28);
  int64_t vals[2] = {4, 30}; const char* names[2] = {"N", "H"}; int resolved[4];
  CHECK(cg_shape_resolve(out, vals, names, 2, resolved) && resolved[2] == 30);
  cg_shape_free(out); cg_shape_free(in);
  return 0;
}

static int sampling_schedule_checkpoint(const char* path) {
  float logits[50];
  for (int i = 0; i < 50; ++i) logits[i] = sinf((float)i);
  cg_sample_seed(7);
  for (int i = 0; i < 20; ++i) {
    int t = cg_sample_temperature(logits, 50, 0.8f), p = cg_sample_top_p(logits, 50, 0.9f), k = cg_sample_top_k(logits, 50, 5);
    CHECK(t >= 0 && t < 50 && p >= 0 && p < 50 && k >= 0 && k < 50);
  }
  int n = 0;
  cg_schedule_step* steps = cg_pipeline_gen_1f1b(4, 8, &n);
  CHECK(steps && n > 16);
  free(steps);
  int s[2] = {4, 9};
  cg_tensor* a = cg_tensor_randn(s, 2, 8, false), *b = cg_tensor_randn(s, 2, 9, false);
  cg_tensor* ts[2] = {a, b}; const char* names[2] = {"layer0.weight", "layer1.weight"};
  cg_save_model(path, ts, names, 2);
  cg_tensor** back = NULL; char** back_names = NULL; int count = 0;
  cg_load_model(path, &back, &back_names, &count);
  CHECK(count == 2 && !strcmp(back_names[1], "layer1.weight") && back[0]->data[35] == a->data[35]);
  for (int i = 0; i < count; ++i) { cg_tensor_free(back[i]); free(back_names[i]); }
  free(back); free(back_names);
  cg_tensor_free(a); cg_tensor_free(b);
  remove(path);
  return 0;
}

static int device_layer_host_mode(void) {
  CHECK(cg_cuda_init() && !cg_cuda_device_mode());     /* the test sets COGITO_FORCE_HOST=1 */
  int s[2] = {9, 20};
  cg_tensor* h = cg_tensor_randn(s, 2, 11, false);
  cg_tensor* d = cg_tensor_to_cuda(h), *y = cg_tensor_cuda_zeros(s, 2, false);
  cg_cuda_softmax_forward(d, y, 0);
  cg_cuda_gelu_forward(y, y);
  int sr[1] = {9};
  cg_tensor* r = cg_tensor_cuda_zeros(sr, 1, false);
  cg_cuda_tensor_sum(y, 1, r);
  cg_tensor* back = cg_tensor_to_cpu(r);
  CHECK(back && back->data[8] > 0);
  void* raw = cg_cuda_malloc(333);
  cg_cuda_memset(raw, 0, 333);
  cg_cuda_free(raw);
  cg_tensor_free(back); cg_tensor_free(r); cg_tensor_free(y); cg_tensor_free(d); cg_tensor_free(h);
  cg_cuda_shutdown();
  return 0;
}

int main(int argc, char** argv) {
  const char* path = argc > 1 ? argv[1] : "capi_stress.cog";
  if (tensors_and_tape() || pools() || quant_and_cache() || tracing_and_shapes() || sampling_schedule_checkpoint(path) ||
      device_layer_host_mode())
    return 1;
  if (cg_tensor_live_count() != 0) { fprintf(stderr, "%d tensors still live\n", cg_tensor_live_count()); return 2; }
  printf("ok\n");
  return 0;
}
