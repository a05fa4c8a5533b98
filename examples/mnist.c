/* MNIST-shaped classifier with the C API: 784 -> 128 -> 64 -> 10, ReLU, softmax cross-entropy, Adam.
 * Build:  cc -std=c11 -Iinclude examples/mnist.c -Lcogito_b200/lib -lcogito -lm -o mnist
 * Run:    ./mnist [train-images-idx3-ubyte train-labels-idx1-ubyte]   (no files: synthetic digits)
 * Counterpart of the reference's examples/mnist.c, which hand-codes the same network because its
 * library path could not train; here the layers, the loader and the optimizer are the library's. */
#include <stdio.h>
#include <stdlib.h>
#include <time.h>

#include "cogito.h"
#include "cogito_ext.h"

/* ten random prototypes plus noise: separable, so the accuracy shows whether training works */
static void synthetic(int n, cg_tensor** images, cg_tensor** labels) {
  int ishape[2] = {n, 784}, lshape[1] = {n}, pshape[2] = {10, 784};
  cg_tensor* proto = cg_tensor_randn(pshape, 2, 7u, false);
  cg_tensor* noise = cg_tensor_randn(ishape, 2, 11u, false);
  *images = cg_tensor_zeros(ishape, 2, false);
  *labels = cg_tensor_zeros(lshape, 1, false);
  for (int i = 0; i < n; ++i) {
    const int c = (i * 7 + i / 10) % 10;
    (*labels)->data[i] = (float)c;
    for (int j = 0; j < 784; ++j) (*images)->data[i * 784 + j] = 0.5f * proto->data[c * 784 + j] + 0.7f * noise->data[i * 784 + j];
  }
  cg_tensor_release(proto);
  cg_tensor_release(noise);
}

int main(int argc, char** argv) {
  cg_manual_seed(0u);
  cg_tensor *images = NULL, *labels = NULL;
  cg_mnist* mnist = NULL;
  if (argc > 2 && (mnist = cg_mnist_load(argv[1], argv[2])) != NULL) {
    images = mnist->images;
    labels = mnist->labels;
    printf("loaded %d images of %d x %d\n", mnist->num_samples, mnist->rows, mnist->cols);
  } else {
    synthetic(2000, &images, &labels);
    printf("synthetic data: 2000 samples, 10 classes\n");
  }
  cg_tensor* onehot = cg_labels_to_onehot(labels, 10);

  cg_sequential* model = cg_sequential_new();
  cg_sequential_add(model, (cg_layer*)cg_linear_new(784, 128, true));
  cg_sequential_add(model, (cg_layer*)cg_relu_new());
  cg_sequential_add(model, (cg_layer*)cg_linear_new(128, 64, true));
  cg_sequential_add(model, (cg_layer*)cg_relu_new());
  cg_sequential_add(model, (cg_layer*)cg_linear_new(64, 10, true));
  cg_adam* opt = cg_adam_new_for_sequential(model, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.0f);
  cg_dataloader* loader = cg_dataloader_new(images, onehot, 32, true, 1u);

  const clock_t t0 = clock();
  float acc = 0.0f, mean = 0.0f;
  for (int epoch = 0; epoch < 5; ++epoch) {
    double total = 0.0, hits = 0.0;
    int batches = 0, seen = 0, n = 0;
    cg_tensor *bx, *by;                                  /* owned by the loader, valid until the next call */
    while (cg_dataloader_next(loader, &bx, &by, &n)) {
      cg_optimizer_zero_grad(&opt->base);
      cg_tensor* logits = cg_sequential_forward(model, bx);
      cg_tensor* loss = cg_softmax_cross_entropy_loss(logits, by, CG_REDUCTION_MEAN);
      cg_backward(loss);
      cg_optimizer_step(&opt->base);
      total += loss->data[0];
      hits += cg_compute_accuracy(logits, by, 10) * n;
      seen += n;
      ++batches;
      cg_tensor_release(loss);
      cg_tensor_release(logits);                         /* a layer's output is handed to the caller, who releases it */
    }
    cg_dataloader_reset(loader);
    mean = (float)(total / batches);
    acc = (float)(hits / seen);
    printf("epoch %d  loss %.4f  accuracy %.3f\n", epoch + 1, mean, acc);
  }
  printf("training time %.2f s\n", (double)(clock() - t0) / CLOCKS_PER_SEC);

  cg_dataloader_free(loader);
  cg_optimizer_free(&opt->base);
  cg_sequential_free(model);
  cg_tensor_release(onehot);
  if (mnist) cg_mnist_free(mnist);
  else { cg_tensor_release(images); cg_tensor_release(labels); }
  return acc > 0.9f ? 0 : 1;
}
