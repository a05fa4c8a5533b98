// Optimizer kernels on flat fp32 buffers with a device-resident loss-scaler, so
// a mixed-precision step needs no host round trip:
//
//   cgk_grad_stats   : sum of squares of the (still scaled) gradients + inf/nan flag
//   cgk_adam_step    : unscale, optional global-norm clip, AdamW update of the fp32
//                      masters, bf16 copy of the new weights; skipped when the
//                      flag is set
//   cgk_sgd_step     : SGD with momentum / Nesterov / L2 decay, same skip rule
//   cgk_scaler_update: halve on overflow, double after `window` clean steps,
//                      advance the step counter, clear the flag
//
// Update rules follow the reference: Adam increments t first, applies decoupled
// decay p -= lr*wd*p, then p -= lr * m_hat / (sqrt(v_hat) + eps)
// (src/optim/adam.c:10-46); SGD does g += wd*p, v = mu*v + g, Nesterov
// p -= lr*(mu*v + g) else p -= lr*v (src/optim/sgd.c:10-44); the scaler starts
// at 65536, stays in [1, 65536], doubles every 2000 clean steps and halves on
// overflow (src/core/bf16.c:88-94,115-198; src/optim/optimizer.c:66-88).
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cgk {

// Layout of the scaler state in device memory (8 x 4 bytes).
struct ScalerState {
  float scale;       // current loss scale
  int good_steps;    // clean steps since the last change
  int found_inf;     // set by grad_stats (or by a fused reduce kernel)
  int step;          // optimizer steps actually applied (Adam's t)
  int skipped;       // steps dropped because of overflow
  float norm_sq;     // sum of squares of the scaled gradients of this step
  float pad0, pad1;
};

constexpr int STAT_THREADS = 256;

__global__ void __launch_bounds__(STAT_THREADS)
grad_stats_partial_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial,
                          int* __restrict__ inf_partial) {
  float s = 0.0f;
  int bad = 0;
  const long long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 v = g4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    bad |= !isfinite(v.x) | !isfinite(v.y) | !isfinite(v.z) | !isfinite(v.w);
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float v = g[i];
    s += v * v;
    bad |= !isfinite(v);
  }
  __shared__ float sh[STAT_THREADS / 32];
  __shared__ int shb[STAT_THREADS / 32];
  s = warp_sum(s);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) { sh[threadIdx.x >> 5] = s; shb[threadIdx.x >> 5] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    int b = 0;
    for (int w = 0; w < STAT_THREADS / 32; ++w) { t += sh[w]; b |= shb[w]; }
    partial[blockIdx.x] = t;
    inf_partial[blockIdx.x] = b;
  }
}

__global__ void grad_stats_final_kernel(const float* __restrict__ partial,
                                        const int* __restrict__ inf_partial, int nparts,
                                        ScalerState* st, int accumulate) {
  __shared__ float sh[STAT_THREADS / 32];
  __shared__ int shb[STAT_THREADS / 32];
  float s = 0.0f;
  int bad = 0;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) { s += partial[i]; bad |= inf_partial[i]; }
  s = warp_sum(s);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) { sh[threadIdx.x >> 5] = s; shb[threadIdx.x >> 5] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    int b = 0;
    for (int w = 0; w < STAT_THREADS / 32; ++w) { t += sh[w]; b |= shb[w]; }
    if (!isfinite(t)) b = 1;
    st->norm_sq = accumulate ? st->norm_sq + t : t;
    st->found_inf = accumulate ? (st->found_inf | b) : b;
  }
}

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay;
  float max_grad_norm;  // <= 0: no clipping
};

__global__ void __launch_bounds__(256)
adam_step_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                 const float* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n,
                 AdamHyper h, const ScalerState* __restrict__ st) {
  float inv_scale = 1.0f;
  int t = 1;
  if (st) {
    if (st->found_inf) return;
    inv_scale = 1.0f / st->scale;
    t = st->step + 1;
    if (h.max_grad_norm > 0.0f) {
      float norm = sqrtf(st->norm_sq) * inv_scale;
      if (norm > h.max_grad_norm) inv_scale *= h.max_grad_norm / (norm + 1e-6f);
    }
  }
  const float bc1 = 1.0f - powf(h.beta1, (float)t);
  const float bc2 = 1.0f - powf(h.beta2, (float)t);
  const float decay = 1.0f - h.lr * h.weight_decay;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gr = g[i] * inv_scale;
    float pv = p[i];
    if (h.weight_decay > 0.0f) pv *= decay;
    const float mi = h.beta1 * m[i] + (1.0f - h.beta1) * gr;
    const float vi = h.beta2 * v[i] + (1.0f - h.beta2) * gr * gr;
    m[i] = mi;
    v[i] = vi;
    pv -= h.lr * (mi / bc1) / (sqrtf(vi / bc2) + h.eps);
    p[i] = pv;
    if (p16) p16[i] = __float2bfloat16(pv);
  }
}

__global__ void __launch_bounds__(256)
sgd_step_kernel(float* __restrict__ p, float* __restrict__ vel, const float* __restrict__ g,
                __nv_bfloat16* __restrict__ p16, long long n, float lr, float momentum,
                float weight_decay, int nesterov, float max_grad_norm,
                const ScalerState* __restrict__ st) {
  float inv_scale = 1.0f;
  if (st) {
    if (st->found_inf) return;
    inv_scale = 1.0f / st->scale;
    if (max_grad_norm > 0.0f) {
      float norm = sqrtf(st->norm_sq) * inv_scale;
      if (norm > max_grad_norm) inv_scale *= max_grad_norm / (norm + 1e-6f);
    }
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float gr = g[i] * inv_scale;
    float pv = p[i];
    if (weight_decay > 0.0f) gr += weight_decay * pv;
    if (momentum > 0.0f && vel) {
      float vv = momentum * vel[i] + gr;
      vel[i] = vv;
      pv -= nesterov ? lr * (momentum * vv + gr) : lr * vv;
    } else {
      pv -= lr * gr;
    }
    p[i] = pv;
    if (p16) p16[i] = __float2bfloat16(pv);
  }
}

__global__ void scaler_update_kernel(ScalerState* st, float growth, float backoff, int window,
                                     float min_scale, float max_scale) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (st->found_inf) {
    st->scale = fmaxf(st->scale * backoff, min_scale);
    st->good_steps = 0;
    st->skipped += 1;
  } else {
    st->step += 1;
    st->good_steps += 1;
    if (st->good_steps >= window) {
      st->scale = fminf(st->scale * growth, max_scale);
      st->good_steps = 0;
    }
  }
  st->found_inf = 0;
  st->norm_sq = 0.0f;
}

__global__ void scaler_init_kernel(ScalerState* st, float scale) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  st->scale = scale;
  st->good_steps = 0;
  st->found_inf = 0;
  st->step = 0;
  st->skipped = 0;
  st->norm_sq = 0.0f;
  st->pad0 = st->pad1 = 0.0f;
}

}  // namespace cgk

using namespace cgk;

static int flat_grid(long long n, int threads) {
  int dev = 0;
  cudaGetDevice(&dev);
  long long want = (n + threads - 1) / threads;
  long long cap = (long long)sm_count(dev) * 8;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

// The scaler state is 8 x 4 bytes of device memory owned by the caller.
CGK_API int cgk_scaler_state_bytes() { return (int)sizeof(ScalerState); }

CGK_API int cgk_scaler_init(void* state, float scale, void* stream) {
  CGK_REQUIRE(state, "cgk_scaler_init: null state");
  scaler_init_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((ScalerState*)state, scale);
  CGK_LAUNCH_CHECK();
  return 0;
}

// Number of fp32 + int32 scratch elements cgk_grad_stats needs (one of each per CTA).
CGK_API int cgk_grad_stats_scratch_elems(long long n) { return 2 * flat_grid(n, STAT_THREADS); }

// scratch: cgk_grad_stats_scratch_elems(n) 4-byte words.  accumulate != 0 adds to
// the state's norm_sq / ORs into found_inf (several buffers per step).
CGK_API int cgk_grad_stats(const float* g, long long n, void* state, void* scratch, int accumulate,
                           void* stream) {
  CGK_REQUIRE(g && state && scratch, "cgk_grad_stats: null pointer");
  CGK_REQUIRE(((uintptr_t)g & 15) == 0, "cgk_grad_stats: gradient buffer must be 16-byte aligned");
  int grid = flat_grid(n, STAT_THREADS);
  float* partial = (float*)scratch;
  int* infp = (int*)scratch + grid;
  grad_stats_partial_kernel<<<grid, STAT_THREADS, 0, (cudaStream_t)stream>>>(g, n, partial, infp);
  CGK_LAUNCH_CHECK();
  grad_stats_final_kernel<<<1, STAT_THREADS, 0, (cudaStream_t)stream>>>(partial, infp, grid,
                                                                        (ScalerState*)state, accumulate);
  CGK_LAUNCH_CHECK();
  return 0;
}

// state may be null (no loss scaling, t taken as 1 is then wrong for bias
// correction: pass a state initialised with scale 1 for plain fp32 training).
CGK_API int cgk_adam_step(float* p, float* m, float* v, const float* g, void* p16, long long n,
                          float lr, float beta1, float beta2, float eps, float weight_decay,
                          float max_grad_norm, const void* state, void* stream) {
  CGK_REQUIRE(p && m && v && g, "cgk_adam_step: null pointer");
  if (n == 0) return 0;
  AdamHyper h{lr, beta1, beta2, eps, weight_decay, max_grad_norm};
  adam_step_kernel<<<flat_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(
      p, m, v, g, (__nv_bfloat16*)p16, n, h, (const ScalerState*)state);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_sgd_step(float* p, float* vel, const float* g, void* p16, long long n, float lr,
                         float momentum, float weight_decay, int nesterov, float max_grad_norm,
                         const void* state, void* stream) {
  CGK_REQUIRE(p && g, "cgk_sgd_step: null pointer");
  if (n == 0) return 0;
  sgd_step_kernel<<<flat_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(
      p, vel, g, (__nv_bfloat16*)p16, n, lr, momentum, weight_decay, nesterov, max_grad_norm,
      (const ScalerState*)state);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_scaler_update(void* state, float growth, float backoff, int window,
                              float min_scale, float max_scale, void* stream) {
  CGK_REQUIRE(state, "cgk_scaler_update: null state");
  scaler_update_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((ScalerState*)state, growth, backoff,
                                                           window, min_scale, max_scale);
  CGK_LAUNCH_CHECK();
  return 0;
}
