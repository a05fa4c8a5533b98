/* A transformer block trained in a loop the way a caller of the C API does it: the output of every forward pass is
 * released by the caller, the tape by releasing the loss; the number of live tensors must settle and end at zero.
 * Built and run by tests/test_capi_core_cpu.py. */
#include <stdio.h>
#include "cogito.h"
int main(void) {
  cg_transformer_config c = {0};
  c.hidden_dim = 32; c.num_heads = 4; c.num_kv_heads = 2; c.head_dim = 8; c.intermediate_dim = 64; c.norm_eps = 1e-5f;
  c.pre_norm = true; c.use_rms_norm = true; c.use_swiglu = true;
  for (int variant = 0; variant < 2; ++variant) {
    c.pre_norm = variant == 0; c.use_swiglu = variant == 0; c.use_rms_norm = variant == 0;
    cg_transformer_block* b = cg_transformer_block_new(c);
    int xs[2] = {6, 32};
    cg_tensor* x = cg_tensor_randn(xs, 2, 3u, true);
    int base = -1;
    for (int it = 0; it < 50; ++it) {
      cg_tensor* y = cg_transformer_forward(&b->base, x, NULL);
      cg_tensor* l = cg_mean_all(y);
      cg_backward(l);
      cg_tensor_release(l);
      cg_tensor_release(y);
      if (it == 5) base = cg_tensor_live_count();
      if (it > 5 && cg_tensor_live_count() != base) { printf("leak: %d vs %d at %d\n", cg_tensor_live_count(), base, it); return 1; }
    }
    cg_tensor_release(x);
    cg_layer_free(&b->base);
  }
  printf("live %d\n", cg_tensor_live_count());
  return cg_tensor_live_count() != 0;
}
