// Tensor-parallel serving: sum of a row-parallel projection's partial results over the ranks,
// fused with the residual add and, optionally, with the RMSNorm that feeds the next projection.
//
//   x[t, :] += sum_p partial_p[t, :]            (every rank ends with the same x)
//   h[t, :]  = x[t, :] * rsqrt(mean(x[t, :]^2) + eps) * w        (when w is given)
//
// The partials are a few hundred KiB (16 .. 128 tokens x d_model bf16), so the step is bound by
// latency, not bandwidth: one launch, one signal round, then every rank reads every peer's
// partial directly over NVLink (one-shot all-reduce) with all its loads in flight at once.
// Each rank's projection writes its partial into a buffer of symmetric memory, in one of two
// slots used alternately; the kernel
//   1. tells every peer "my partial of this epoch is complete" (release store into the peer's
//      flag array; the projection kernel ran before this one in the same stream),
//   2. waits (bounded) until all peers have said so,
//   3. one CTA per token row: 16-byte loads from the P slots, fp32 sum in rank order (every rank
//      adds in the same order, so the replicas of x stay bit-identical), residual, norm.
// A slot is rewritten two epochs later.  By then every peer has signalled the epoch in between,
// which it does only after its reads of the older epoch have finished, so no closing handshake
// is needed.
//
// Reference counterpart: cg_tp_row_parallel_forward's all-reduce (src/pipeline/tensor_parallel.c:
// 81-105, ncclAllReduce in place), which the reference calls through an uninitialised communicator.
#include <cuda_bf16.h>

#include "../../include/cogito_kernels.h"
#include "../kernels/host_common.h"
#include "comm_device.cuh"

namespace cgk {
namespace {

struct ServeArDev {
  const __nv_bfloat16* partial[8];   // every rank's slot of this epoch
  int* sig[8];                       // every rank's flag array: sig[r][p] = last epoch rank p completed
  __nv_bfloat16* x;                  // [rows, cols] residual stream, updated in place
  const __nv_bfloat16* w;            // [cols] RMSNorm weight or null
  __nv_bfloat16* h;                  // [rows, cols] normalised output (when w)
  int* counters;                     // local: [0] calls completed (the epoch of this call is that + 1), [1] CTAs done in this call
  int rank, ranks, rows, cols;
  float eps;
  int* status;
};

constexpr int SAR_THREADS = 512, SAR_MAX_VEC = 4;     // up to 512 * 4 * 8 = 16384 columns

__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void reduce_row(const ServeArDev& d, int row, int tid, float* red_s);

__global__ void __launch_bounds__(SAR_THREADS)
serve_allreduce_kernel(const ServeArDev d) {
  __shared__ int ok_s, epoch_s;
  __shared__ float red_s[SAR_THREADS / 32];
  const int P = d.ranks, row = blockIdx.x, tid = threadIdx.x;
  // The epoch is counted on the device (a launch replayed from a CUDA graph cannot take it as an
  // argument): every CTA reads the count of completed calls; the CTA that finishes last raises it,
  // which is after every CTA of this launch has read it.
  if (tid == 0) { epoch_s = *reinterpret_cast<volatile int*>(d.counters) + 1; ok_s = 1; }
  __syncthreads();
  const int epoch = epoch_s;
  // 1. signal (one CTA is enough: the partial was complete before this kernel started)
  if (blockIdx.x == 0 && tid < P) {
    __threadfence_system();
    st_release_sys(d.sig[tid] + d.rank, epoch);
  }
  // 2. wait for every peer's signal in my own flag array
  if (tid < P && !flag_wait_ge_sys(d.sig[d.rank] + tid, epoch, d.status, 4000 + tid, CGK_PEER_WAIT_BUDGET_NS)) ok_s = 0;
  __syncthreads();
  if (ok_s) reduce_row(d, row, tid, red_s);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(d.counters + 1, 1) == (int)gridDim.x - 1) {
      d.counters[1] = 0;
      __threadfence();
      atomicAdd(d.counters, 1);
    }
  }
}

// 3. sum, residual, norm of one row by one CTA
__device__ __forceinline__ void reduce_row(const ServeArDev& d, int row, int tid, float* red_s) {
  const int P = d.ranks;
  const int vecs = d.cols / 8;                         // 16-byte pieces per row
  float acc[SAR_MAX_VEC][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < SAR_MAX_VEC; ++i) {
    const int v = tid + i * SAR_THREADS;
    if (v < vecs) {
      const long long off = (long long)row * d.cols + v * 8;
      uint4 part[8];
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < P) part[p] = ld_peer_16(d.partial[p] + off);
      const uint4 xr = *reinterpret_cast<const uint4*>(d.x + off);
      const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(xw[j]); acc[i][2 * j] = f.x; acc[i][2 * j + 1] = f.y; }
      float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        if (p < P) {
          const uint32_t pw[4] = {part[p].x, part[p].y, part[p].z, part[p].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(pw[j]); sum[2 * j] += f.x; sum[2 * j + 1] += f.y; }
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = pack_bf16x2(acc[i][2 * j] + sum[2 * j], acc[i][2 * j + 1] + sum[2 * j + 1]);
        const float2 r = unpack_bf16x2(o[j]);          // the norm sees the stored (rounded) x
        acc[i][2 * j] = r.x; acc[i][2 * j + 1] = r.y;
        ss += r.x * r.x + r.y * r.y;
      }
      *reinterpret_cast<uint4*>(d.x + off) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (!d.w) return;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red_s[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < SAR_THREADS / 32; ++i) tot += red_s[i];
  const float inv = rsqrtf(tot / (float)d.cols + d.eps);
#pragma unroll
  for (int i = 0; i < SAR_MAX_VEC; ++i) {
    const int v = tid + i * SAR_THREADS;
    if (v < vecs) {
      const long long off = (long long)row * d.cols + v * 8;
      const uint4 wr = *reinterpret_cast<const uint4*>(d.w + v * 8);
      const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(ww[j]);
        o[j] = pack_bf16x2(acc[i][2 * j] * inv * f.x, acc[i][2 * j + 1] * inv * f.y);
      }
      *reinterpret_cast<uint4*>(d.h + off) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}
}  // namespace
}  // namespace cgk

// partial[p], sig[p]: the addresses of rank p's slot / flag array as mapped in THIS process.
// x, h: [rows, cols] bf16, local.  cols a multiple of 8, at most 16384.  counters: two local ints, zero
// before the first call (the kernel numbers the calls itself; every rank makes the same calls in the
// same order).  w null: no norm.
CGK_API int cgk_serve_allreduce(const void* const* partial, int* const* sig, int rank, int ranks, int* counters, void* x,
                                const void* w, void* h, int rows, int cols, float eps, void* stream) {
  using namespace cgk;
  CGK_REQUIRE(partial && sig && x && ranks >= 1 && ranks <= 8 && rank >= 0 && rank < ranks && counters, "cgk_serve_allreduce: bad argument");
  CGK_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0 && cols <= SAR_THREADS * SAR_MAX_VEC * 8, "cgk_serve_allreduce: cols must be a multiple of 8, at most 16384");
  CGK_REQUIRE(!w || h, "cgk_serve_allreduce: a norm weight needs an output");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  ServeArDev d{};
  for (int p = 0; p < ranks; ++p) {
    CGK_REQUIRE(partial[p] && sig[p] && ((uintptr_t)partial[p] & 15) == 0, "cgk_serve_allreduce: null or misaligned peer buffer");
    d.partial[p] = (const __nv_bfloat16*)partial[p];
    d.sig[p] = sig[p];
  }
  d.x = (__nv_bfloat16*)x; d.w = (const __nv_bfloat16*)w; d.h = (__nv_bfloat16*)h;
  d.rank = rank; d.ranks = ranks; d.counters = counters; d.rows = rows; d.cols = cols; d.eps = eps;
  d.status = device_status(dev);
  serve_allreduce_kernel<<<rows, SAR_THREADS, 0, (cudaStream_t)stream>>>(d);
  CGK_LAUNCH_CHECK();
  return 0;
}
