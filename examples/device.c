/* The device layer of the C API from a plain C program: the same binary runs its tensor
 * operations on a B200 (sm_100a kernels, tcgen05 GEMM) when one is present and on the host when
 * not.  Counterpart of the reference's tests/test_cuda.c walk (init, device info, a copy round
 * trip, elementwise, a matrix product, an activation, softmax rows).
 *
 *   cc examples/device.c -Iinclude -Lcogito_b200/lib -lcogito -lm -o device
 *   LD_LIBRARY_PATH=cogito_b200/lib ./device
 */
#include <math.h>
#include <stdio.h>

#include "cogito.h"

static int close_to(float a, float b, float tol) { return fabsf(a - b) <= tol * (1.0f + fabsf(b)); }

int main(void) {
  if (!cg_cuda_init()) { fprintf(stderr, "cg_cuda_init failed: %s\n", cg_cuda_get_last_error()); return 1; }
  cg_cuda_device_info info = cg_cuda_get_device_info(cg_cuda_get_device());
  printf("mode: %s\ndevice: %s (cc %d.%d, %d SMs, %.1f GB)\n", cg_cuda_device_mode() ? "GPU" : "host", info.device_name,
         info.compute_capability_major, info.compute_capability_minor, info.multiprocessor_count, info.total_memory / 1e9);

  enum { M = 192, K = 256, N = 128 };
  int sa[2] = {M, K}, sb[2] = {K, N}, sc[2] = {M, N};
  cg_tensor* a = cg_tensor_randn(sa, 2, 1, false);
  cg_tensor* b = cg_tensor_randn(sb, 2, 2, false);
  cg_tensor* da = cg_tensor_to_cuda(a), *db = cg_tensor_to_cuda(b);
  cg_tensor* dc = cg_tensor_cuda_zeros(sc, 2, false), *dp = cg_tensor_cuda_zeros(sc, 2, false);
  if (!da || !db || !dc || !dp) { fprintf(stderr, "allocation failed: %s\n", cg_cuda_get_last_error()); return 1; }

  cg_cuda_tensor_matmul(da, db, dc);          /* [M,K] x [K,N] */
  cg_cuda_gelu_forward(dc, dc);
  cg_cuda_softmax_forward(dc, dp, 1);         /* rows sum to one */
  cg_cuda_device_synchronize();
  if (cg_last_error() != CG_SUCCESS) { fprintf(stderr, "device operation failed: %s\n", cg_cuda_get_last_error()); return 1; }

  /* the same on the host, as the check */
  cg_tensor* c = cg_tensor_zeros(sc, 2, false);
  cg_tensor_matmul(a, b, c);
  cg_tensor* p = cg_tensor_to_cpu(dp);
  int bad = 0;
  for (int i = 0; i < M && !bad; ++i) {
    float mx = -INFINITY, z = 0.0f, row = 0.0f;
    for (int j = 0; j < N; ++j) {
      const float x = c->data[i * N + j];
      const float g = 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
      c->data[i * N + j] = g;
      mx = g > mx ? g : mx;
    }
    for (int j = 0; j < N; ++j) z += expf(c->data[i * N + j] - mx);
    for (int j = 0; j < N; ++j) {
      const float want = expf(c->data[i * N + j] - mx) / z;
      row += p->data[i * N + j];
      if (!close_to(p->data[i * N + j], want, 2e-3f)) { fprintf(stderr, "mismatch at (%d, %d): %g vs %g\n", i, j, p->data[i * N + j], want); bad = 1; break; }
    }
    if (!bad && !close_to(row, 1.0f, 1e-4f)) { fprintf(stderr, "row %d sums to %g\n", i, row); bad = 1; }
  }
  printf("softmax(gelu(A x B)): %s\n", bad ? "MISMATCH" : "matches the host computation");

  cg_tensor_free(p); cg_tensor_free(c);
  cg_tensor_free(dp); cg_tensor_free(dc); cg_tensor_free(db); cg_tensor_free(da);
  cg_tensor_free(b); cg_tensor_free(a);
  cg_cuda_shutdown();
  return bad;
}
