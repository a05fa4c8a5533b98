/* XOR with the C API: Linear(2,4) -> ReLU -> Linear(4,1) -> Sigmoid, MSE, SGD lr 0.5 momentum 0.9.
 * Build:  cc -std=c11 -Iinclude examples/xor.c -Lcogito_b200/lib -lcogito -lm -o xor
 * Counterpart of the reference's examples/xor.c. */
#include <stdio.h>
#include <stdlib.h>

#include "cogito.h"

int main(int argc, char** argv) {
  const int epochs = argc > 1 ? atoi(argv[1]) : 5000;
  cg_manual_seed(argc > 2 ? (unsigned)atoi(argv[2]) : 0u);
  float xs[8] = {0, 0, 0, 1, 1, 0, 1, 1}, ys[4] = {0, 1, 1, 0};
  int xshape[2] = {4, 2}, yshape[2] = {4, 1};
  cg_tensor* x = cg_tensor_from_data(xs, xshape, 2, false);
  cg_tensor* y = cg_tensor_from_data(ys, yshape, 2, false);

  cg_sequential* model = cg_sequential_new();
  cg_sequential_add(model, (cg_layer*)cg_linear_new(2, 4, true));
  cg_sequential_add(model, (cg_layer*)cg_relu_new());
  cg_sequential_add(model, (cg_layer*)cg_linear_new(4, 1, true));
  cg_sequential_add(model, (cg_layer*)cg_sigmoid_new());
  cg_sgd* opt = cg_sgd_new_for_sequential(model, 0.5f, 0.9f, 0.0f, false);

  float last = 0.0f;
  for (int e = 0; e < epochs; ++e) {
    cg_optimizer_zero_grad(&opt->base);
    cg_tensor* pred = cg_sequential_forward(model, x);
    cg_tensor* loss = cg_mse_loss(pred, y, CG_REDUCTION_MEAN);
    cg_backward(loss);                      /* reaches every parameter: layers are on the tape */
    cg_optimizer_step(&opt->base);
    last = loss->data[0];
    if (e % 1000 == 0) printf("epoch %d loss %.6f\n", e, last);
    cg_tensor_release(loss);
    cg_tensor_release(pred);               /* a layer's output is handed to the caller, who releases it */
  }
  cg_tensor* pred = cg_sequential_forward(model, x);
  for (int i = 0; i < 4; ++i) printf("%g xor %g -> %.4f\n", xs[2 * i], xs[2 * i + 1], pred->data[i]);
  printf("final loss %.6f\n", last);
  cg_tensor_release(pred);
  cg_optimizer_free(&opt->base);
  cg_sequential_free(model);
  cg_tensor_release(x);
  cg_tensor_release(y);
  printf("live tensors %d\n", cg_tensor_live_count());
  return last < 0.01f ? 0 : 1;
}
