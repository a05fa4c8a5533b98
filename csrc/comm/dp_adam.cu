// Data-parallel optimizer step over NVLink peer memory, in buckets that overlap the
// backward pass: gradient all-reduce fused with the loss-scale unscale / overflow check,
// the global-norm clip, the Adam update and the broadcast of the new weights.
//
// The flat parameter space is cut into buckets of `bucket_len` elements (the last one may
// be shorter); inside every bucket rank r owns the r-th of P equal parts, and only that
// part of the fp32 master weights and Adam moments (sharded optimizer state, stored bucket
// after bucket).  Two kernels:
//
//  cgk_dp_bucket_reduce  (one launch per bucket, on a side stream, as soon as the backward
//      pass has produced the bucket's gradients; a few CTAs, so backward keeps its SMs)
//        1. handshake: "my gradients of bucket b are complete" (epoch word on every peer);
//        2. reduce-scatter: the rank sums its part of the bucket over all ranks' gradient
//           buffers with plain P2P loads in rank order (bitwise reproducible), sixteen
//           16-byte loads in flight per thread, keeps the sum locally and accumulates
//           sum-of-squares and an inf/nan flag; the last CTA to finish adds up the
//           per-CTA partials in CTA order and leaves the bucket's (norm^2, overflow).
//  cgk_dp_adam_finish  (once, after the last bucket)
//        3. the per-rank (norm^2, overflow) pairs are exchanged through peer memory (or
//           taken from `ext_stats` when a larger group than this one decides, as under
//           tensor / pipeline parallelism), so every rank takes the same skip / clip
//           decision without the host;
//        4. Adam on the owned parts, then the new compute-precision weights are stored
//           into every rank's parameter buffer with 16-byte P2P stores (the all-gather);
//        5. the last CTA to finish closes the step: handshake "my stores into your
//           parameters are done", loss-scaler update.
// No grid-wide barrier anywhere (nothing requires all CTAs to be resident): phases are
// separated by kernel boundaries, by flags, or by a last-arriver counter.  All waits are
// bounded; a wait that runs out leaves a code in the device status word, which
// DPFusedAdam reads back with the loss.
//
// Gradients cross NVLink in fp32 (the buffers the backward GEMMs accumulate into): the
// transfer hides under the backward pass, so halving it would buy nothing and cost bits.
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

constexpr int DP_MAX_BUCKETS = CGK_DP_MAX_BUCKETS;

// Signal words of one rank (int32), written by its peers:
//   [b * P + p]                  bucket b of rank p is complete (epoch)      b < DP_MAX_BUCKETS
//   [S0 + p]                     rank p has published its statistics (epoch)
//   [S0 + P + p]                 rank p has finished storing into my parameters (epoch)
//   [S0 + 2P + 2p], [.. + 1]     rank p's (norm^2, overflow) as floats
__host__ __device__ __forceinline__ int dp_sig_s0(int P) { return DP_MAX_BUCKETS * P; }

struct DpBucketDev {
  int rank, ranks, epoch, bucket;
  const float* grad[8];        // every rank's flat gradient buffer
  int* sig[8];                 // every rank's signal words
  float* gsum;                 // local reduced gradients of the owned part of this bucket
  long long begin, count;      // owned part: flat offset and length (multiple of 4)
  float* block_part;           // local scratch [2 * gridDim.x] of this bucket
  unsigned int* arrive;        // local counter of this bucket (zero between launches)
  float* stats;                // local out: {norm^2, overflow} of this bucket
  int* status;
};

template <int P>
__device__ __forceinline__ void dp_reduce_range(const DpBucketDev& d, float& sq, int& bad) {
  constexpr int U = P >= 8 ? 2 : (P >= 4 ? 4 : 8);
  const long long n4 = d.count >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * U) {
    float4 g[U][P];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < n4) {
#pragma unroll
        for (int p = 0; p < P; ++p) g[u][p] = __ldcg(reinterpret_cast<const float4*>(d.grad[p] + d.begin) + i);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) break;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < P; ++p) { acc.x += g[u][p].x; acc.y += g[u][p].y; acc.z += g[u][p].z; acc.w += g[u][p].w; }
      reinterpret_cast<float4*>(d.gsum)[i] = acc;
      sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
      bad |= !isfinite(acc.x) | !isfinite(acc.y) | !isfinite(acc.z) | !isfinite(acc.w);
    }
  }
}

__global__ void __launch_bounds__(256)
dp_bucket_reduce_kernel(const DpBucketDev d) {
  const int P = d.ranks, me = d.rank;
  __shared__ float sh_a[8];
  __shared__ int sh_b[8];
  __shared__ int ok_s;
  // ---- 1. handshake for this bucket ----
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int p = 0; p < P; ++p)
        if (p != me) st_release_sys(d.sig[p] + d.bucket * P + me, d.epoch);
    }
    bool ok = true;
    for (int p = 0; p < P && ok; ++p)
      if (p != me) ok = flag_wait_ge_sys(d.sig[me] + d.bucket * P + p, d.epoch, d.status, 4000 + p, CGK_PEER_WAIT_BUDGET_NS);
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (!ok_s) return;
  // ---- 2. reduce-scatter of the owned part ----
  float sq = 0.0f;
  int bad = 0;
  switch (P) {
    case 1: dp_reduce_range<1>(d, sq, bad); break;
    case 2: dp_reduce_range<2>(d, sq, bad); break;
    case 3: dp_reduce_range<3>(d, sq, bad); break;
    case 4: dp_reduce_range<4>(d, sq, bad); break;
    case 5: dp_reduce_range<5>(d, sq, bad); break;
    case 6: dp_reduce_range<6>(d, sq, bad); break;
    case 7: dp_reduce_range<7>(d, sq, bad); break;
    default: dp_reduce_range<8>(d, sq, bad); break;
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
    __threadfence();
    // the last CTA to arrive adds the partials in CTA order: the same bits every run
    if (atomicAdd(d.arrive, 1u) == gridDim.x - 1) {
      __threadfence();
      float tt = 0.0f, bb = 0.0f;
      for (unsigned int k = 0; k < gridDim.x; ++k) {
        tt += __ldcg(d.block_part + 2 * k);
        bb += __ldcg(d.block_part + 2 * k + 1);
      }
      d.stats[0] = tt;
      d.stats[1] = bb;
      *d.arrive = 0u;
    }
  }
}

struct DpFinishDev {
  int rank, ranks, epoch, nbuckets;
  void* param_lp[8];           // every rank's flat compute-precision parameters (bf16), or null
  float* param_fp[8];          // every rank's flat fp32 parameters when there is no bf16 copy
  int* sig[8];
  float* master;               // local fp32 master weights of the owned parts (null: fp32 parameters are the master)
  float* m; float* v;          // local Adam moments of the owned parts
  const float* gsum;           // local reduced gradients of the owned parts
  long long n, bucket_len;     // flat length and bucket length (both multiples of 8 * P)
  float lr, beta1, beta2, eps, weight_decay, max_grad_norm, grad_mul;
  float growth, backoff, min_scale, max_scale;
  int window;
  ScalerStateDP* scaler;       // local
  const float* bucket_stats;   // local [nbuckets][2]
  const float* ext_stats;      // {norm^2, overflow} decided by a larger group, or null
  unsigned int* arrive;        // local counter (zero between launches)
  int* status;
};

__global__ void __launch_bounds__(256)
dp_adam_finish_kernel(const DpFinishDev d) {
  const int P = d.ranks, me = d.rank;
  const int S0 = dp_sig_s0(P);
  int* my_sig = d.sig[me];
  __shared__ int ok_s;
  __shared__ float sh_norm, sh_bad;
  // ---- 3. statistics of the whole group ----
  if (threadIdx.x == 0) {
    bool ok = true;
    float norm_sq = 0.0f, any_bad = 0.0f;
    if (d.ext_stats != nullptr) {
      norm_sq = d.ext_stats[0];
      any_bad = d.ext_stats[1];
    } else {
      if (blockIdx.x == 0) {
        float t = 0.0f, b = 0.0f;
        for (int k = 0; k < d.nbuckets; ++k) { t += d.bucket_stats[2 * k]; b += d.bucket_stats[2 * k + 1]; }
        if (!isfinite(t)) b = 1.0f;
        for (int p = 0; p < P; ++p) {
          float* ps = reinterpret_cast<float*>(d.sig[p] + S0 + 2 * P);
          ps[2 * me] = t;
          ps[2 * me + 1] = b;
        }
        __threadfence_system();
        for (int p = 0; p < P; ++p) st_release_sys(d.sig[p] + S0 + me, d.epoch);
      }
      for (int p = 0; p < P && ok; ++p)
        ok = flag_wait_ge_sys(my_sig + S0 + p, d.epoch, d.status, 4200 + p, CGK_PEER_WAIT_BUDGET_NS);
      const float* stats = reinterpret_cast<const float*>(my_sig + S0 + 2 * P);
      for (int p = 0; p < P; ++p) {           // rank order: every rank and every CTA gets the same bits
        norm_sq += __ldcg(stats + 2 * p);
        any_bad += __ldcg(stats + 2 * p + 1);
      }
    }
    sh_norm = norm_sq;
    sh_bad = any_bad;
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (!ok_s) return;
  const float norm_sq = sh_norm;
  const bool skip = sh_bad > 0.0f || !isfinite(norm_sq);
  // ---- 4. Adam on the owned parts + broadcast of the new weights ----
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
    const long long owned = d.n / P;                       // elements this rank owns, stored bucket after bucket
    const long long part = d.bucket_len / P;               // owned elements per full bucket
    float* master = d.master;
    for (long long j = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; j < owned;
         j += (long long)gridDim.x * blockDim.x * 8) {
      // local position j -> flat position: bucket b, my part of it, offset inside the part
      long long b = j / part;
      if (b >= d.nbuckets) b = d.nbuckets - 1;
      const long long len_b = (b == d.nbuckets - 1) ? d.n - b * d.bucket_len : d.bucket_len;
      const long long flat = b * d.bucket_len + me * (len_b / P) + (j - b * part);
      float pv[8];
      const float4 g0 = *reinterpret_cast<const float4*>(d.gsum + j), g1 = *reinterpret_cast<const float4*>(d.gsum + j + 4);
      const float gr[8] = {g0.x * inv, g0.y * inv, g0.z * inv, g0.w * inv, g1.x * inv, g1.y * inv, g1.z * inv, g1.w * inv};
      float* mp = master ? master + j : d.param_fp[me] + flat;
      float4 p0 = *reinterpret_cast<const float4*>(mp), p1 = *reinterpret_cast<const float4*>(mp + 4);
      pv[0] = p0.x; pv[1] = p0.y; pv[2] = p0.z; pv[3] = p0.w; pv[4] = p1.x; pv[5] = p1.y; pv[6] = p1.z; pv[7] = p1.w;
      float4 m0 = *reinterpret_cast<const float4*>(d.m + j), m1 = *reinterpret_cast<const float4*>(d.m + j + 4);
      float4 v0 = *reinterpret_cast<const float4*>(d.v + j), v1 = *reinterpret_cast<const float4*>(d.v + j + 4);
      float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (d.weight_decay > 0.0f) pv[e] *= decay;
        mm[e] = d.beta1 * mm[e] + (1.0f - d.beta1) * gr[e];
        vv[e] = d.beta2 * vv[e] + (1.0f - d.beta2) * gr[e] * gr[e];
        pv[e] -= d.lr * (mm[e] / bc1) / (sqrtf(vv[e] / bc2) + d.eps);
      }
      *reinterpret_cast<float4*>(d.m + j) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(d.m + j + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
      *reinterpret_cast<float4*>(d.v + j) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(d.v + j + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
      const float4 q0 = make_float4(pv[0], pv[1], pv[2], pv[3]), q1 = make_float4(pv[4], pv[5], pv[6], pv[7]);
      if (master) {
        *reinterpret_cast<float4*>(master + j) = q0;
        *reinterpret_cast<float4*>(master + j + 4) = q1;
      }
      if (d.param_lp[0]) {
        uint4 h;                                           // eight bf16 weights: one 16-byte store per rank
        h.x = pack_bf16x2(pv[0], pv[1]); h.y = pack_bf16x2(pv[2], pv[3]);
        h.z = pack_bf16x2(pv[4], pv[5]); h.w = pack_bf16x2(pv[6], pv[7]);
        for (int p = 0; p < P; ++p)
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(d.param_lp[p]) + flat) = h;
      } else {
        for (int p = 0; p < P; ++p) {                      // without a separate master the own copy is the master
          *reinterpret_cast<float4*>(d.param_fp[p] + flat) = q0;
          *reinterpret_cast<float4*>(d.param_fp[p] + flat + 4) = q1;
        }
      }
    }
  }
  // ---- 5. the last CTA closes the step ----
  __threadfence_system();            // my stores into the peers' parameters are performed
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(d.arrive, 1u) == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < P; ++p)
        if (p != me) st_release_sys(d.sig[p] + S0 + P + me, d.epoch);
      bool ok = true;
      for (int p = 0; p < P && ok; ++p)
        if (p != me) ok = flag_wait_ge_sys(my_sig + S0 + P + p, d.epoch, d.status, 4400 + p, CGK_PEER_WAIT_BUDGET_NS);
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
      *d.arrive = 0u;
    }
  }
}

}  // namespace cgk

using namespace cgk;

CGK_API int cgk_dp_bucket_reduce(const cgk_dp_bucket_args* px, void* stream) {
  CGK_REQUIRE(px, "cgk_dp_bucket_reduce: null args");
  const cgk_dp_bucket_args& x = *px;
  CGK_REQUIRE(x.ranks >= 1 && x.ranks <= 8 && x.rank >= 0 && x.rank < x.ranks, "cgk_dp_bucket_reduce: bad rank");
  CGK_REQUIRE(x.epoch > 0 && x.bucket >= 0 && x.bucket < DP_MAX_BUCKETS, "cgk_dp_bucket_reduce: bad epoch / bucket");
  CGK_REQUIRE(x.count >= 0 && x.count % 4 == 0 && x.begin % 4 == 0, "cgk_dp_bucket_reduce: the owned part must be a multiple of 4 elements");
  CGK_REQUIRE(x.gsum && x.block_part && x.arrive && x.stats, "cgk_dp_bucket_reduce: null pointer");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  DpBucketDev d{};
  d.rank = x.rank; d.ranks = x.ranks; d.epoch = x.epoch; d.bucket = x.bucket;
  for (int p = 0; p < x.ranks; ++p) { d.grad[p] = (const float*)x.grad_ptrs[p]; d.sig[p] = (int*)x.signal_ptrs[p]; }
  d.gsum = x.gsum; d.begin = x.begin; d.count = x.count;
  d.block_part = x.block_part; d.arrive = (unsigned int*)x.arrive; d.stats = x.stats;
  d.status = device_status(dev);
  CGK_REQUIRE(x.grid_ctas > 0 && x.grid_ctas <= CGK_DP_MAX_CTAS, "cgk_dp_bucket_reduce: grid_ctas must be in 1..%d", CGK_DP_MAX_CTAS);
  dp_bucket_reduce_kernel<<<x.grid_ctas, 256, 0, (cudaStream_t)stream>>>(d);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_dp_adam_finish(const cgk_dp_finish_args* px, void* stream) {
  CGK_REQUIRE(px, "cgk_dp_adam_finish: null args");
  const cgk_dp_finish_args& x = *px;
  CGK_REQUIRE(x.ranks >= 1 && x.ranks <= 8 && x.rank >= 0 && x.rank < x.ranks, "cgk_dp_adam_finish: bad rank");
  CGK_REQUIRE(x.epoch > 0 && x.nbuckets >= 1 && x.nbuckets <= DP_MAX_BUCKETS, "cgk_dp_adam_finish: bad epoch / bucket count");
  CGK_REQUIRE(x.n > 0 && x.bucket_len > 0 && x.n % (8 * x.ranks) == 0 && x.bucket_len % (8 * x.ranks) == 0 &&
                  (x.n + x.bucket_len - 1) / x.bucket_len == x.nbuckets,
              "cgk_dp_adam_finish: flat length and bucket length must be multiples of 8 * ranks and agree with nbuckets");
  CGK_REQUIRE(x.m && x.v && x.gsum && x.scaler && x.bucket_stats && x.arrive, "cgk_dp_adam_finish: null pointer");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  DpFinishDev d{};
  d.rank = x.rank; d.ranks = x.ranks; d.epoch = x.epoch; d.nbuckets = x.nbuckets;
  for (int p = 0; p < x.ranks; ++p) {
    d.param_lp[p] = x.param_lp_ptrs[p];
    d.param_fp[p] = (float*)x.param_fp_ptrs[p];
    d.sig[p] = (int*)x.signal_ptrs[p];
  }
  d.master = x.master; d.m = x.m; d.v = x.v; d.gsum = x.gsum;
  d.n = x.n; d.bucket_len = x.bucket_len;
  d.lr = x.lr; d.beta1 = x.beta1; d.beta2 = x.beta2; d.eps = x.eps; d.weight_decay = x.weight_decay;
  d.max_grad_norm = x.max_grad_norm; d.grad_mul = x.grad_mul;
  d.growth = x.growth; d.backoff = x.backoff; d.min_scale = x.min_scale; d.max_scale = x.max_scale;
  d.window = x.window;
  d.scaler = (ScalerStateDP*)x.scaler;
  d.bucket_stats = x.bucket_stats; d.ext_stats = x.ext_stats;
  d.arrive = (unsigned int*)x.arrive;
  d.status = device_status(dev);
  int grid = x.grid_ctas > 0 ? x.grid_ctas : 2 * sm_count(dev);
  const long long units = x.n / x.ranks / 8;
  if ((long long)grid * 256 > units) grid = (int)((units + 255) / 256);
  if (grid < 1) grid = 1;
  dp_adam_finish_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d);
  CGK_LAUNCH_CHECK();
  return 0;
}

// Bytes of signal words each rank must provide (zero before the first call).
CGK_API int cgk_dp_signal_bytes(int ranks) {
  return (dp_sig_s0(ranks) + 4 * ranks) * 4;
}
