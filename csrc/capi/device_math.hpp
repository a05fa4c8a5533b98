// Part of device.cpp (included at its end; uses its file-local state and helpers): matrix
// products, activation gradients, softmax and the normalisations of the cg_cuda_* API.
// Reference counterparts: src/cuda/tensor_kernels.c:523-601 (matmul, transpose, bmm),
// :607-806 (activations, softmax), :812-909 (LayerNorm, RMSNorm).
#pragma once
#include "cogito_kernels.h"      // plain C declarations of the kernel library (argument structs)

namespace {

// out[b] = A[b] (M x K, row-major) * B[b] (K x N, row-major), fp32 in and out.
bool device_matmul(const float* A, const float* B, float* out, int batch, int M, int N, int K) {
  State& s = S();
  cgdev::Scratch sc;
  const size_t na = (size_t)batch * M * K, nb = (size_t)batch * K * N;
  const int terms = s.matmul_products == 1 ? 1 : 3;
  char* ah = (char*)sc.get(na * 2), *bh = (char*)sc.get(nb * 2);
  char* al = terms == 3 ? (char*)sc.get(na * 2) : nullptr, *bl = terms == 3 ? (char*)sc.get(nb * 2) : nullptr;
  if (!ah || !bh || (terms == 3 && (!al || !bl))) return false;
  if (terms == 3) {
    if (!ok(s.k.split_bf16(A, ah, al, (long long)na, stream()), "operand split")) return false;
    if (!ok(s.k.split_bf16(B, bh, bl, (long long)nb, stream()), "operand split")) return false;
  } else {
    if (!ok(s.k.cast(A, ah, (long long)na, 1, stream()), "operand cast")) return false;
    if (!ok(s.k.cast(B, bh, (long long)nb, 1, stream()), "operand cast")) return false;
  }
  cgk_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.out = out; g.M = M; g.N = N; g.K = K; g.batch = batch;
  g.lda = K; g.ldb = N; g.ldc = N;
  g.strideA = (int64_t)M * K; g.strideB = (int64_t)K * N; g.strideC = (int64_t)M * N;
  g.a_mn = 0; g.b_mn = 1;                   // B is [K rows, N cols], N contiguous
  g.out_fp32 = 1; g.alpha = 1.0f;
  // smallest terms first, so that the large product is added last
  const char* as[3] = {al, ah, ah};
  const char* bs[3] = {bh, bl, bh};
  for (int t = terms == 3 ? 0 : 2; t < 3; ++t) {
    g.A = as[t]; g.B = bs[t];
    g.accumulate = (terms == 3 && t > 0) ? 1 : 0;
    if (!ok(s.k.gemm(&g, stream()), "tensor-core GEMM")) return false;
  }
  return true;
}

void matmul_impl(cg_tensor* a, cg_tensor* b, cg_tensor* o, bool batched) {
  if (!operands_ok({a, b, o})) return;
  const int need = batched ? 3 : 2;
  if (a->ndim != need || b->ndim != need) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int B = batched ? a->shape[0] : 1;
  const int M = a->shape[need - 2], K = a->shape[need - 1], N = b->shape[need - 1];
  if (b->shape[need - 2] != K || (batched && b->shape[0] != B) || o->size != B * M * N) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (dev()) { device_matmul(a->data, b->data, o->data, B, M, N, K); return; }
  for (int i = 0; i < B; ++i)
    gemm(a->data + (size_t)i * M * K, b->data + (size_t)i * K * N, o->data + (size_t)i * M * N, M, N, K, false, false, false);
}

// grad_in = grad_out * f'(.), the derivative written in terms of the saved tensor
void act_backward(int op, bool from_output, cg_tensor* saved, cg_tensor* gy, cg_tensor* gx) {
  if (!operands_ok({saved, gy, gx}) || !same_size(saved, gy) || !same_size(saved, gx)) return;
  const long long n = saved->size;
  if (dev()) {
    State& s = S();
    if (!from_output) { ok(s.k.unary_backward(op, 0, saved->data, gy->data, gx->data, n, 0.0f, stream()), "activation gradient"); return; }
    // sigmoid: y (1 - y);  tanh: 1 - y^2  -- composed from elementwise kernels on the saved output
    cgdev::Scratch sc;
    float* t = (float*)sc.get(sizeof(float) * (size_t)n);
    if (!t) return;
    if (op == UN_SIGMOID) {
      if (!dun(UN_SQUARE, saved->data, t, n) || !dbin(BIN_SUB, saved->data, t, FULL, t, 1, n)) return;      // y - y^2
    } else {
      if (!dun(UN_SQUARE, saved->data, t, n) || !dun(UN_SCALE, t, t, n, -1.0f) || !dun(UN_ADDS, t, t, n, 1.0f)) return;
    }
    dbin(BIN_MUL, gy->data, t, FULL, gx->data, 1, n);
    return;
  }
  for (long long i = 0; i < n; ++i) {
    const float v = saved->data[i];
    float d;
    if (op == UN_RELU) d = v > 0 ? 1.0f : 0.0f;
    else if (op == UN_SIGMOID) d = from_output ? v * (1 - v) : sigmoidf(v) * (1 - sigmoidf(v));
    else if (op == UN_TANH) d = from_output ? 1 - v * v : 1 - std::tanh(v) * std::tanh(v);
    else {  // tanh-approximated GELU
      const float c = 0.7978845608f, u = c * (v + 0.044715f * v * v * v), th = std::tanh(u);
      d = 0.5f * (1 + th) + 0.5f * v * (1 - th * th) * c * (1 + 3 * 0.044715f * v * v);
    }
    gx->data[i] = gy->data[i] * d;
  }
}

// Softmax over `axis` of a tensor viewed as [outer, red, inner]; backward when y/dy are given.
void softmax_impl(cg_tensor* x_or_y, cg_tensor* dy, cg_tensor* out, int axis) {
  if (dy ? !operands_ok({x_or_y, dy, out}) : !operands_ok({x_or_y, out})) return;
  if (!same_size(x_or_y, out) || (dy && !same_size(x_or_y, dy))) return;
  if (axis < 0) axis += x_or_y->ndim;
  long long outer, red, inner;
  if (axis < 0 || !split_axis(x_or_y, axis, &outer, &red, &inner)) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (dev()) {
    State& s = S();
    if (inner == 1) {
      if (dy) ok(s.k.softmax_rows_backward(x_or_y->data, dy->data, out->data, (int)outer, (int)red, stream()), "softmax gradient");
      else ok(s.k.softmax_rows(x_or_y->data, out->data, (int)outer, (int)red, 1.0f, stream()), "softmax");
      return;
    }
    // reduced axis is not the last: bring it last with a transpose per outer slice
    cgdev::Scratch sc;
    const size_t slice = (size_t)red * inner;
    float* t0 = (float*)sc.get(sizeof(float) * slice), *t1 = (float*)sc.get(sizeof(float) * slice);
    float* t2 = dy ? (float*)sc.get(sizeof(float) * slice) : nullptr;
    if (!t0 || !t1 || (dy && !t2)) return;
    for (long long u = 0; u < outer; ++u) {
      if (!ok(s.k.transpose2d(0, x_or_y->data + u * slice, t0, (int)red, (int)inner, stream()), "transpose")) return;
      if (dy) {
        if (!ok(s.k.transpose2d(0, dy->data + u * slice, t2, (int)red, (int)inner, stream()), "transpose")) return;
        if (!ok(s.k.softmax_rows_backward(t0, t2, t1, (int)inner, (int)red, stream()), "softmax gradient")) return;
      } else if (!ok(s.k.softmax_rows(t0, t1, (int)inner, (int)red, 1.0f, stream()), "softmax")) return;
      if (!ok(s.k.transpose2d(0, t1, out->data + u * slice, (int)inner, (int)red, stream()), "transpose")) return;
    }
    return;
  }
  for (long long u = 0; u < outer; ++u) for (long long v = 0; v < inner; ++v) {
    const size_t base = u * red * inner + v;
    if (!dy) {
      const float* x = x_or_y->data + base;
      float m = x[0];
      for (long long r = 1; r < red; ++r) m = std::fmax(m, x[r * inner]);
      double z = 0;
      for (long long r = 0; r < red; ++r) z += std::exp(x[r * inner] - m);
      for (long long r = 0; r < red; ++r) out->data[base + r * inner] = (float)(std::exp(x[r * inner] - m) / z);
    } else {
      const float* y = x_or_y->data + base; const float* g = dy->data + base;
      double dot = 0;
      for (long long r = 0; r < red; ++r) dot += (double)y[r * inner] * g[r * inner];
      for (long long r = 0; r < red; ++r) out->data[base + r * inner] = y[r * inner] * (g[r * inner] - (float)dot);
    }
  }
}

}  // namespace

CG_EXPORT void cg_cuda_set_matmul_precision(int products) { S().matmul_products = products == 1 ? 1 : 3; }
CG_EXPORT void cg_cuda_tensor_matmul(cg_tensor* a, cg_tensor* b, cg_tensor* o) { matmul_impl(a, b, o, false); }
CG_EXPORT void cg_cuda_tensor_bmm(cg_tensor* a, cg_tensor* b, cg_tensor* o) { matmul_impl(a, b, o, true); }
CG_EXPORT void cg_cuda_tensor_transpose(cg_tensor* a, cg_tensor* o) {
  if (!operands_ok({a, o}) || !same_size(a, o)) return;
  if (a->ndim != 2) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int R = a->shape[0], C = a->shape[1];
  if (dev()) { ok(S().k.transpose2d(0, a->data, o->data, R, C, stream()), "transpose"); return; }
  for (int i = 0; i < R; ++i) for (int j = 0; j < C; ++j) o->data[(size_t)j * R + i] = a->data[(size_t)i * C + j];
}

CG_EXPORT void cg_cuda_relu_backward(cg_tensor* x, cg_tensor* gy, cg_tensor* gx) { act_backward(UN_RELU, false, x, gy, gx); }
CG_EXPORT void cg_cuda_sigmoid_backward(cg_tensor* y, cg_tensor* gy, cg_tensor* gx) { act_backward(UN_SIGMOID, true, y, gy, gx); }
CG_EXPORT void cg_cuda_tanh_backward(cg_tensor* y, cg_tensor* gy, cg_tensor* gx) { act_backward(UN_TANH, true, y, gy, gx); }
CG_EXPORT void cg_cuda_gelu_backward(cg_tensor* x, cg_tensor* gy, cg_tensor* gx) { act_backward(UN_GELU, false, x, gy, gx); }
CG_EXPORT void cg_cuda_softmax_forward(cg_tensor* x, cg_tensor* y, int axis) { softmax_impl(x, nullptr, y, axis); }
CG_EXPORT void cg_cuda_softmax_backward(cg_tensor* y, cg_tensor* gy, cg_tensor* gx, int axis) { softmax_impl(y, gy, gx, axis); }
