// The hot loops of the host runtime: GEMM inner kernels and the Adam update.  This file is compiled with
// -O3 -fno-math-errno (the rest of the library with -O2, which vectorises only loops whose trip count is
// known when compiling and keeps sqrt scalar because it may set errno), and on x86-64 every function here
// is built twice, the second time for AVX2 + FMA; the loader picks the copy the CPU can run.
#include "internal.hpp"

#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__) && !defined(__SANITIZE_ADDRESS__)
#define CGI_SIMD_CLONES __attribute__((target_clones("arch=haswell", "default")))
#else
#define CGI_SIMD_CLONES
#endif

namespace cgi {
// C[M,N] += op(A) B with B [K,N] row-major: "row of C += a * row of B", four rows of C at a time so that a
// row of B is loaded once for four multiply-adds.  op(A)(i,k) = ta ? A[k*M+i] : A[i*K+k].
CGI_SIMD_CLONES void gemm_rows(const float* __restrict A, const float* __restrict B, float* __restrict C,
                                      int M, int N, int K, bool ta) {
  int i = 0;
  for (; i + 4 <= M; i += 4) {
    float* __restrict c0 = C + (size_t)i * N;
    float* __restrict c1 = c0 + N;
    float* __restrict c2 = c1 + N;
    float* __restrict c3 = c2 + N;
    for (int k = 0; k < K; ++k) {
      float a0, a1, a2, a3;
      if (ta) {
        const float* a = A + (size_t)k * M + i;
        a0 = a[0]; a1 = a[1]; a2 = a[2]; a3 = a[3];
      } else {
        const float* a = A + (size_t)i * K + k;
        a0 = a[0]; a1 = a[K]; a2 = a[2 * (size_t)K]; a3 = a[3 * (size_t)K];
      }
      if (a0 == 0.0f && a1 == 0.0f && a2 == 0.0f && a3 == 0.0f) continue;      // rows behind a ReLU are half zeros
      const float* __restrict b = B + (size_t)k * N;
      for (int j = 0; j < N; ++j) {
        const float bv = b[j];
        c0[j] += a0 * bv; c1[j] += a1 * bv; c2[j] += a2 * bv; c3[j] += a3 * bv;
      }
    }
  }
  for (; i < M; ++i) {
    float* __restrict c = C + (size_t)i * N;
    for (int k = 0; k < K; ++k) {
      const float a = ta ? A[(size_t)k * M + i] : A[(size_t)i * K + k];
      if (a == 0.0f) continue;
      const float* __restrict b = B + (size_t)k * N;
      for (int j = 0; j < N; ++j) c[j] += a * b[j];
    }
  }
}
// C[i,j] += sum_k A[i,k] B[j,k] for a few rows of A: eight partial sums per dot product
CGI_SIMD_CLONES void gemm_dots(const float* __restrict A, const float* __restrict B, float* __restrict C,
                                      int M, int N, int K) {
  for (int i = 0; i < M; ++i) {
    const float* __restrict a = A + (size_t)i * K;
    for (int j = 0; j < N; ++j) {
      const float* __restrict b = B + (size_t)j * K;
      float p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      int k = 0;
      for (; k + 8 <= K; k += 8)
        for (int u = 0; u < 8; ++u) p[u] += a[k + u] * b[k + u];
      float s = ((p[0] + p[4]) + (p[1] + p[5])) + ((p[2] + p[6]) + (p[3] + p[7]));
      for (; k < K; ++k) s += a[k] * b[k];
      C[(size_t)i * N + j] += s;
    }
  }
}

// w, m, v updated in place from the gradient g; decay = 1 - lr * weight_decay (1 when off).
CGI_SIMD_CLONES void adam_update(float* __restrict w, float* __restrict m, float* __restrict v, const float* __restrict g, int n,
                                 float b1, float b2, float lr, float eps, float bc1, float bc2, float decay) {
  for (int j = 0; j < n; ++j) {
    const float gj = g[j];
    float wj = w[j] * decay;                                                              // decoupled decay (1 when off)
    const float mj = b1 * m[j] + (1 - b1) * gj;
    const float vj = b2 * v[j] + (1 - b2) * gj * gj;
    m[j] = mj; v[j] = vj;
    wj -= lr * (mj / bc1) / (__builtin_sqrtf(vj / bc2) + eps);
    w[j] = wj;
  }
}
}  // namespace cgi
