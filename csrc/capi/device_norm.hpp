// Part of device.cpp (included at its end): LayerNorm forward / backward and RMSNorm forward of
// the cg_cuda_* API, in fp32 for any row length.  On the device each is a short chain of the
// fp32 reduction and broadcast kernels (the fused one-pass bf16 norm kernels serve the training
// path of the Python framework, not this fp32 tier).
// Reference counterparts: src/cuda/tensor_kernels.c:812-909 (host loops only).
#pragma once

namespace {

// mean / rstd of each row of x [rows, D]; rms: mean is not computed and rstd = rsqrt(mean(x^2)+eps)
bool device_row_stats(const float* x, float* xc, float* mean, float* rstd, float* tmp, long long rows, long long D, float eps,
                      bool rms) {
  if (!rms) {
    if (!dred(RED_MEAN, x, mean, rows, D, 1) || !dbin(BIN_SUB, x, mean, PER_ROW, xc, rows, D)) return false;
  }
  const float* c = rms ? x : xc;
  return dun(UN_SQUARE, c, tmp, rows * D) && dred(RED_MEAN, tmp, rstd, rows, D, 1) && dun(UN_ADDS, rstd, rstd, rows, eps) &&
         dun(UN_RSQRT, rstd, rstd, rows);
}

void layernorm_forward_impl(cg_tensor* x, cg_tensor* gamma, cg_tensor* beta, cg_tensor* y, cg_tensor* mean, cg_tensor* rstd,
                            float eps, int D, bool rms) {
  if (!operands_ok({x, gamma, y}) || (beta && !operands_ok({beta})) || (mean && !operands_ok({mean})) ||
      (rstd && !operands_ok({rstd})) || !same_size(x, y))
    return;
  if (D <= 0 || x->size % D || gamma->size != D || (beta && beta->size != D)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const long long rows = x->size / D;
  if ((mean && mean->size != rows) || (rstd && rstd->size != rows)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (eps <= 0) eps = 1e-5f;
  if (dev()) {
    cgdev::Scratch sc;
    float* xc = (float*)sc.get(sizeof(float) * (size_t)x->size), *tmp = (float*)sc.get(sizeof(float) * (size_t)x->size);
    float* m = mean ? mean->data : (float*)sc.get(sizeof(float) * (size_t)rows);
    float* r = rstd ? rstd->data : (float*)sc.get(sizeof(float) * (size_t)rows);
    if (!xc || !tmp || !m || !r) return;
    if (!device_row_stats(x->data, xc, m, r, tmp, rows, D, eps, rms)) return;
    if (!dbin(BIN_MUL, rms ? x->data : xc, r, PER_ROW, y->data, rows, D)) return;
    if (!dbin(BIN_MUL, y->data, gamma->data, PER_COL, y->data, rows, D)) return;
    if (beta && !rms) dbin(BIN_ADD, y->data, beta->data, PER_COL, y->data, rows, D);
    return;
  }
  for (long long i = 0; i < rows; ++i) {
    const float* xr = x->data + i * D;
    double mu = 0, var = 0;
    if (!rms) { for (int j = 0; j < D; ++j) mu += xr[j]; mu /= D; }
    for (int j = 0; j < D; ++j) var += (xr[j] - mu) * (xr[j] - mu);
    const float rs = 1.0f / std::sqrt((float)(var / D) + eps);
    if (mean) mean->data[i] = (float)mu;
    if (rstd) rstd->data[i] = rs;
    for (int j = 0; j < D; ++j) y->data[i * D + j] = (xr[j] - (float)mu) * rs * gamma->data[j] + (beta && !rms ? beta->data[j] : 0.0f);
  }
}

}  // namespace

CG_EXPORT void cg_cuda_layernorm_forward(cg_tensor* x, cg_tensor* gamma, cg_tensor* beta, cg_tensor* y, cg_tensor* mean,
                                         cg_tensor* rstd, float eps, int normalized_shape) {
  layernorm_forward_impl(x, gamma, beta, y, mean, rstd, eps, normalized_shape, false);
}
CG_EXPORT void cg_cuda_rmsnorm_forward(cg_tensor* x, cg_tensor* weight, cg_tensor* y, float eps) {
  if (!weight) { set_error(CG_ERROR_NULL_POINTER); return; }
  layernorm_forward_impl(x, weight, nullptr, y, nullptr, nullptr, eps > 0 ? eps : 1e-6f, weight->size, true);
}

// dx = rstd * (g - mean_D(g) - xhat * mean_D(g * xhat)) with g = dy * gamma, xhat = (x - mean) * rstd;
// dgamma = sum_rows(dy * xhat), dbeta = sum_rows(dy).  grad_gamma / grad_beta may be NULL.
CG_EXPORT void cg_cuda_layernorm_backward(cg_tensor* dy, cg_tensor* x, cg_tensor* gamma, cg_tensor* mean, cg_tensor* rstd,
                                          cg_tensor* dx, cg_tensor* dgamma, cg_tensor* dbeta, int D) {
  if (!operands_ok({dy, x, gamma, mean, rstd, dx}) || (dgamma && !operands_ok({dgamma})) || (dbeta && !operands_ok({dbeta})) ||
      !same_size(dy, x) || !same_size(dx, x))
    return;
  if (D <= 0 || x->size % D || gamma->size != D || mean->size != x->size / D || rstd->size != x->size / D ||
      (dgamma && dgamma->size != D) || (dbeta && dbeta->size != D)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const long long rows = x->size / D, n = x->size;
  if (dev()) {
    cgdev::Scratch sc;
    float* xhat = (float*)sc.get(sizeof(float) * (size_t)n), *g = (float*)sc.get(sizeof(float) * (size_t)n);
    float* t = (float*)sc.get(sizeof(float) * (size_t)n), *r1 = (float*)sc.get(sizeof(float) * (size_t)rows);
    float* r2 = (float*)sc.get(sizeof(float) * (size_t)rows);
    if (!xhat || !g || !t || !r1 || !r2) return;
    if (!dbin(BIN_SUB, x->data, mean->data, PER_ROW, xhat, rows, D) || !dbin(BIN_MUL, xhat, rstd->data, PER_ROW, xhat, rows, D)) return;
    if (dgamma && (!dbin(BIN_MUL, dy->data, xhat, FULL, t, rows, D) || !dred(RED_SUM, t, dgamma->data, 1, rows, D))) return;
    if (dbeta && !dred(RED_SUM, dy->data, dbeta->data, 1, rows, D)) return;
    if (!dbin(BIN_MUL, dy->data, gamma->data, PER_COL, g, rows, D)) return;
    if (!dred(RED_MEAN, g, r1, rows, D, 1)) return;                                       // mean_D(g)
    if (!dbin(BIN_MUL, g, xhat, FULL, t, rows, D) || !dred(RED_MEAN, t, r2, rows, D, 1)) return;   // mean_D(g xhat)
    if (!dbin(BIN_MUL, xhat, r2, PER_ROW, t, rows, D)) return;
    if (!dbin(BIN_SUB, g, r1, PER_ROW, g, rows, D) || !dbin(BIN_SUB, g, t, FULL, g, rows, D)) return;
    dbin(BIN_MUL, g, rstd->data, PER_ROW, dx->data, rows, D);
    return;
  }
  if (dgamma) std::fill(dgamma->data, dgamma->data + D, 0.0f);
  if (dbeta) std::fill(dbeta->data, dbeta->data + D, 0.0f);
  std::vector<float> xh(D), gv(D);
  for (long long i = 0; i < rows; ++i) {
    const float mu = mean->data[i], rs = rstd->data[i];
    double m1 = 0, m2 = 0;
    for (int j = 0; j < D; ++j) {
      xh[j] = (x->data[i * D + j] - mu) * rs;
      gv[j] = dy->data[i * D + j] * gamma->data[j];
      m1 += gv[j]; m2 += (double)gv[j] * xh[j];
      if (dgamma) dgamma->data[j] += dy->data[i * D + j] * xh[j];
      if (dbeta) dbeta->data[j] += dy->data[i * D + j];
    }
    m1 /= D; m2 /= D;
    for (int j = 0; j < D; ++j) dx->data[i * D + j] = rs * (gv[j] - (float)m1 - xh[j] * (float)m2);
  }
}
