// Data-parallel optimizer step as ONE kernel: gradient all-reduce over NVLink peer
// memory fused with the loss-scale unscale / overflow check, the global-norm clip,
// the Adam update and the broadcast of the new weights.
//
// Every rank owns one contiguous slice of the flat parameter space (and only that
// slice of the fp32 master weights and Adam moments).  One launch, all SMs:
//   1. handshake: "my gradients are complete" (epoch word in every peer's memory);
//   2. reduce-scatter: each rank sums its slice over all ranks' gradient buffers with
//      plain P2P loads in rank order (bitwise reproducible), keeps the sum locally
//      and accumulates sum-of-squares and an inf/nan flag;
//   3. the per-rank (norm^2, overflow) pairs are exchanged through peer memory, so
//      every rank takes the same skip / clip decision without the host;
//   4. Adam on the owned slice, then the new compute-precision weights are stored
//      into every rank's parameter buffer (P2P stores = the all-gather);
//   5. closing handshake, loss-scaler update.
// A grid-wide barrier separates the phases; the grid is one CTA per SM so all CTAs
// are resident.  All waits are bounded.
//
// Reference counterparts: cg_pipeline_allreduce_grads (declared, undefined,
// include/cg_pipeline.h:113), adam_step (src/optim/adam.c:10-46), cg_mp_step and the
// scaler rule (src/core/bf16.c:115-198, src/optim/optimizer.c:66-88).
#include "../../include/cogito_kernels.h"
#include "../kernels/host_common.h"
#include "comm_device.cuh"

namespace cgk {

struct ScalerStateDP {   // same layout as ScalerState in optim.cu
  float scale;
  int good_steps, found_inf, step, skipped;
  float norm_sq, pad0, pad1;
};

struct DpAdamDev {
  int rank, ranks, epoch;
  const float* grad[8];        // every rank's flat gradient buffer
  void* param_lp[8];           // every rank's flat compute-precision parameters (bf16), or null
  float* param_fp[8];          // every rank's flat fp32 parameters when there is no bf16 copy
  int* sig[8];                 // every rank's signal words: [0..P) ready, [P..2P) done, then stats
  float* master;               // local fp32 master slice (null: param_fp[rank] slice is the master)
  float* m; float* v;          // local Adam moments of the slice
  float* gsum;                 // local reduced gradient slice
  long long begin, count;      // slice of this rank
  float lr, beta1, beta2, eps, weight_decay, max_grad_norm, grad_mul;
  float growth, backoff, min_scale, max_scale;
  int window;
  ScalerStateDP* scaler;       // local
  float* block_part;           // local [gridDim.x * 2]
  unsigned int* grid_bar;      // local, monotonically increasing
  unsigned int grid_bar_base;
  int* status;
};

__device__ __forceinline__ bool grid_barrier(unsigned int* bar, unsigned int target, int* status, int where) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(bar, 1u);
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (*reinterpret_cast<volatile unsigned int*>(bar) < target) {
      if ((++it & 63u) == 0u) {
        if (globaltimer_ns() - t0 > CGK_PEER_WAIT_BUDGET_NS) { ok = false; report_status(status, KST_FLAG_TIMEOUT, where, (int)target); break; }
        __nanosleep(64);
      }
    }
    __threadfence();
  }
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = ok ? 1 : 0;
  __syncthreads();
  return ok_s != 0;
}

__global__ void __launch_bounds__(256)
dp_adam_kernel(const DpAdamDev d) {
  const int P = d.ranks, me = d.rank;
  const unsigned int G = gridDim.x;
  int* my_sig = d.sig[me];
  __shared__ float sh_a[8];
  __shared__ int sh_b[8];
  __shared__ int ok_s;
  // ---- 1. opening handshake ----
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < P; ++p)
      if (p != me) st_release_sys(d.sig[p] + me, d.epoch);
  }
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int p = 0; p < P && ok; ++p)
      if (p != me) ok = flag_wait_ge_sys(my_sig + p, d.epoch, d.status, 4000 + p, CGK_PEER_WAIT_BUDGET_NS);
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (!ok_s) return;
  // ---- 2. reduce-scatter of the owned slice ----
  float sq = 0.0f;
  int bad = 0;
  const long long n4 = d.count >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)G * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int p = 0; p < P; ++p) {
      const float4 g = __ldcg(reinterpret_cast<const float4*>(d.grad[p] + d.begin) + i);
      acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
    }
    reinterpret_cast<float4*>(d.gsum)[i] = acc;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    bad |= !isfinite(acc.x) | !isfinite(acc.y) | !isfinite(acc.z) | !isfinite(acc.w);
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.count;
       i += (long long)G * blockDim.x) {
    float acc = 0.0f;
    for (int p = 0; p < P; ++p) acc += __ldcg(d.grad[p] + d.begin + i);
    d.gsum[i] = acc;
    sq += acc * acc;
    bad |= !isfinite(acc);
  }
  sq = warp_sum(sq);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) { sh_a[threadIdx.x >> 5] = sq; sh_b[threadIdx.x >> 5] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    int b = 0;
    for (int w = 0; w < 8; ++w) { t += sh_a[w]; b |= sh_b[w]; }
    d.block_part[2 * blockIdx.x] = t;
    d.block_part[2 * blockIdx.x + 1] = b ? 1.0f : 0.0f;
  }
  if (!grid_barrier(d.grid_bar, d.grid_bar_base + G, d.status, 4100)) return;
  // ---- 3. exchange (norm^2, overflow) ----
  float* stats = reinterpret_cast<float*>(my_sig + 2 * P);      // [P][2] floats + [P] epoch words after
  int* stat_ep = my_sig + 2 * P + 2 * P;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    float t = 0.0f, b = 0.0f;
    for (unsigned int k = 0; k < G; ++k) { t += d.block_part[2 * k]; b += d.block_part[2 * k + 1]; }
    if (!isfinite(t)) b = 1.0f;
    for (int p = 0; p < P; ++p) {
      float* ps = reinterpret_cast<float*>(d.sig[p] + 2 * P);
      ps[2 * me] = t;
      ps[2 * me + 1] = b;
    }
    __threadfence_system();
    for (int p = 0; p < P; ++p) st_release_sys(d.sig[p] + 4 * P + me, d.epoch);
  }
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int p = 0; p < P && ok; ++p) ok = flag_wait_ge_sys(stat_ep + p, d.epoch, d.status, 4200 + p, CGK_PEER_WAIT_BUDGET_NS);
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (!ok_s) return;
  float norm_sq = 0.0f, any_bad = 0.0f;
  for (int p = 0; p < P; ++p) {
    norm_sq += __ldcg(stats + 2 * p);
    any_bad += __ldcg(stats + 2 * p + 1);
  }
  const bool skip = any_bad > 0.0f;
  // ---- 4. Adam on the slice + broadcast of the new weights ----
  const float scale = d.scaler->scale;
  const int t_step = d.scaler->step + 1;
  if (!skip) {
    float inv = d.grad_mul / scale;     // grad_mul = 1 / ranks turns the sum into a mean
    if (d.max_grad_norm > 0.0f) {
      const float norm = sqrtf(norm_sq) * inv;
      if (norm > d.max_grad_norm) inv *= d.max_grad_norm / (norm + 1e-6f);
    }
    const float bc1 = 1.0f - powf(d.beta1, (float)t_step);
    const float bc2 = 1.0f - powf(d.beta2, (float)t_step);
    const float decay = 1.0f - d.lr * d.weight_decay;
    float* master = d.master ? d.master : d.param_fp[me] + d.begin;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.count;
         i += (long long)G * blockDim.x) {
      const float gr = d.gsum[i] * inv;
      float pv = master[i];
      if (d.weight_decay > 0.0f) pv *= decay;
      const float mi = d.beta1 * d.m[i] + (1.0f - d.beta1) * gr;
      const float vi = d.beta2 * d.v[i] + (1.0f - d.beta2) * gr * gr;
      d.m[i] = mi;
      d.v[i] = vi;
      pv -= d.lr * (mi / bc1) / (sqrtf(vi / bc2) + d.eps);
      master[i] = pv;
      if (d.param_lp[0]) {
        const __nv_bfloat16 h = __float2bfloat16(pv);
        for (int p = 0; p < P; ++p) reinterpret_cast<__nv_bfloat16*>(d.param_lp[p])[d.begin + i] = h;
      } else {
        for (int p = 0; p < P; ++p)
          if (p != me || d.master) d.param_fp[p][d.begin + i] = pv;
      }
    }
  }
  __threadfence_system();
  if (!grid_barrier(d.grid_bar, d.grid_bar_base + 2 * G, d.status, 4300)) return;
  // ---- 5. closing handshake + scaler ----
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int p = 0; p < P; ++p)
      if (p != me) st_release_sys(d.sig[p] + P + me, d.epoch);
    bool ok = true;
    for (int p = 0; p < P && ok; ++p)
      if (p != me) ok = flag_wait_ge_sys(my_sig + P + p, d.epoch, d.status, 4400 + p, CGK_PEER_WAIT_BUDGET_NS);
    ScalerStateDP* st = d.scaler;
    if (skip) {
      st->scale = fmaxf(st->scale * d.backoff, d.min_scale);
      st->good_steps = 0;
      st->skipped += 1;
    } else {
      st->step += 1;
      st->good_steps += 1;
      if (st->good_steps >= d.window) { st->scale = fminf(st->scale * d.growth, d.max_scale); st->good_steps = 0; }
    }
    st->found_inf = 0;
    st->norm_sq = norm_sq;
  }
}

}  // namespace cgk

using namespace cgk;

CGK_API int cgk_dp_adam_step(const cgk_dp_adam_args* px, void* stream) {
  CGK_REQUIRE(px, "cgk_dp_adam_step: null args");
  const cgk_dp_adam_args& x = *px;
  CGK_REQUIRE(x.ranks >= 1 && x.ranks <= 8 && x.rank >= 0 && x.rank < x.ranks, "cgk_dp_adam_step: bad rank");
  CGK_REQUIRE(x.epoch > 0 && x.count >= 0 && x.begin % 4 == 0, "cgk_dp_adam_step: bad epoch / slice");
  CGK_REQUIRE(x.m && x.v && x.gsum && x.scaler && x.block_part && x.grid_bar, "cgk_dp_adam_step: null pointer");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  DpAdamDev d{};
  d.rank = x.rank; d.ranks = x.ranks; d.epoch = x.epoch;
  for (int p = 0; p < x.ranks; ++p) {
    d.grad[p] = (const float*)x.grad_ptrs[p];
    d.param_lp[p] = x.param_lp_ptrs[p];
    d.param_fp[p] = (float*)x.param_fp_ptrs[p];
    d.sig[p] = (int*)x.signal_ptrs[p];
  }
  d.master = x.master; d.m = x.m; d.v = x.v; d.gsum = x.gsum;
  d.begin = x.begin; d.count = x.count;
  d.lr = x.lr; d.beta1 = x.beta1; d.beta2 = x.beta2; d.eps = x.eps; d.weight_decay = x.weight_decay;
  d.max_grad_norm = x.max_grad_norm;
  d.grad_mul = x.grad_mul;
  d.growth = x.growth; d.backoff = x.backoff; d.min_scale = x.min_scale; d.max_scale = x.max_scale;
  d.window = x.window;
  d.scaler = (ScalerStateDP*)x.scaler;
  d.block_part = x.block_part;
  d.grid_bar = (unsigned int*)x.grid_bar;
  d.grid_bar_base = (unsigned int)x.grid_bar_base;
  d.status = device_status(dev);
  const int grid = x.grid_ctas;
  CGK_REQUIRE(grid > 0 && grid <= sm_count(dev), "cgk_dp_adam_step: grid_ctas must be in 1..%d", sm_count(dev));
  dp_adam_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_dp_adam_max_ctas() {
  int dev = 0;
  cudaGetDevice(&dev);
  return sm_count(dev);
}
