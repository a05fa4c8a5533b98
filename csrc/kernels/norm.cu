// Fused LayerNorm / RMSNorm forward and backward, bf16 in/out, fp32 statistics,
// optional residual add fused into the forward (writes the sum as a second
// output so the next residual branch can reuse it).
//
// One warp per row, the row held in registers between the statistics pass and
// the normalisation pass.  Backward keeps per-column partial sums of
// dgamma / dbeta in registers across all rows a warp handles, combines the
// warps of a CTA through shared memory and writes one fp32 partial row per CTA
// into a scratch buffer that a second kernel reduces.
//
// Reference counterparts: cg_cuda_layernorm_forward/backward and
// cg_cuda_rmsnorm_forward (src/cuda/tensor_kernels.c:812-909, host loops there),
// cg_bf16_layernorm (src/core/bf16.c:267), rmsnorm_forward/backward
// (src/layers/normalization.c:14-105).
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cgk {

constexpr int NORM_WARPS = 4;

__device__ __forceinline__ void unpack8(const uint4& a, float (&f)[8]) {
  float2 t;
  t = unpack_bf16x2(a.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16x2(a.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16x2(a.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16x2(a.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}

// MAXV = uint4 vectors (8 bf16 each) per lane; a row of D elements needs
// ceil(D / 256) of them.  The row stays in registers as packed bf16.
template <int MAXV, bool RMS>
__global__ void __launch_bounds__(NORM_WARPS * 32)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int D,
                float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;  // uint4 vectors per row
  for (long long row = (long long)blockIdx.x * NORM_WARPS + warp; row < rows;
       row += (long long)gridDim.x * NORM_WARPS) {
    const uint4* xp = reinterpret_cast<const uint4*>(x + row * D);
    const uint4* rp = residual ? reinterpret_cast<const uint4*>(residual + row * D) : nullptr;
    uint4 v[MAXV];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        uint4 a = xp[c];
        if (rp) {
          // the sum is what later layers see, so statistics use its bf16 rounding
          float fa[8], fb[8];
          unpack8(a, fa);
          unpack8(rp[c], fb);
#pragma unroll
          for (int j = 0; j < 8; ++j) fa[j] += fb[j];
          a = pack8(fa);
          if (sum_out) reinterpret_cast<uint4*>(sum_out + row * D)[c] = a;
        }
        v[i] = a;
        float f[8];
        unpack8(a, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += RMS ? f[j] * f[j] : f[j];
      }
    }
    s = warp_sum(s);
    float mean = 0.0f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / D + eps);
    } else {
      mean = s / D;
      float q = 0.0f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        if (lane + i * 32 < nvec) {
          float f[8];
          unpack8(v[i], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = f[j] - mean; q += d * d; }
        }
      }
      q = warp_sum(q);
      rstd = rsqrtf(q / D + eps);
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    const uint4* gp = reinterpret_cast<const uint4*>(gamma);
    const uint4* bp = beta ? reinterpret_cast<const uint4*>(beta) : nullptr;
    uint4* yp = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float f[8], g[8], b[8];
        unpack8(v[i], f);
        unpack8(__ldg(gp + c), g);
        if (bp) {
          unpack8(__ldg(bp + c), b);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) b[j] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * g[j] + b[j];
        yp[c] = pack8(f);
      }
    }
  }
}

// Backward.  partial: [gridDim.x, 2, D] fp32 (dgamma row, dbeta row per CTA).
// Each warp keeps its dgamma / dbeta sums in a private slice of shared memory
// (each lane owns its columns, so no atomics).
template <int MAXV, bool RMS>
__global__ void __launch_bounds__(NORM_WARPS * 32)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres_in,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int D) {
  extern __shared__ float sm_part[];  // [NORM_WARPS][2][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  float* mine = sm_part + (size_t)warp * 2 * D;
  for (int i = lane; i < 2 * D; i += 32) mine[i] = 0.0f;
  __syncwarp();
  const uint4* gp = reinterpret_cast<const uint4*>(gamma);
  // A lane sees the same columns in every row, so for rows of up to 1024 elements its partial
  // sums of dgamma / dbeta stay in registers across all rows the warp handles and reach shared
  // memory once, at the end (a read-modify-write of shared memory per row was the kernel's bottleneck).
  constexpr bool REGACC = MAXV <= 4;
  float accg[REGACC ? MAXV * 8 : 1], accb[REGACC ? MAXV * 8 : 1];
  if (REGACC) {
#pragma unroll
    for (int i = 0; i < (REGACC ? MAXV * 8 : 1); ++i) { accg[i] = 0.0f; accb[i] = 0.0f; }
  }
  for (long long row = (long long)blockIdx.x * NORM_WARPS + warp; row < rows;
       row += (long long)gridDim.x * NORM_WARPS) {
    const float mean = RMS ? 0.0f : mean_in[row];
    const float rstd = rstd_in[row];
    const uint4* xp = reinterpret_cast<const uint4*>(x + row * D);
    const uint4* dp = reinterpret_cast<const uint4*>(dy + row * D);
    uint4 xr[MAXV], dr[MAXV];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        xr[i] = xp[c];
        dr[i] = dp[c];
        float xv[8], dv[8], g[8];
        unpack8(xr[i], xv);
        unpack8(dr[i], dv);
        unpack8(__ldg(gp + c), g);
        float h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          h[j] = (xv[j] - mean) * rstd;
          float t = dv[j] * g[j];
          s1 += t;
          s2 += t * h[j];
        }
        if (REGACC) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { accg[(REGACC ? i : 0) * 8 + j] += dv[j] * h[j]; accb[(REGACC ? i : 0) * 8 + j] += dv[j]; }
        } else {
          float4* pg = reinterpret_cast<float4*>(mine + c * 8);
          float4* pb = reinterpret_cast<float4*>(mine + D + c * 8);
          float4 g0 = pg[0], g1 = pg[1], b0 = pb[0], b1 = pb[1];
          g0.x += dv[0] * h[0]; g0.y += dv[1] * h[1]; g0.z += dv[2] * h[2]; g0.w += dv[3] * h[3];
          g1.x += dv[4] * h[4]; g1.y += dv[5] * h[5]; g1.z += dv[6] * h[6]; g1.w += dv[7] * h[7];
          b0.x += dv[0]; b0.y += dv[1]; b0.z += dv[2]; b0.w += dv[3];
          b1.x += dv[4]; b1.y += dv[5]; b1.z += dv[6]; b1.w += dv[7];
          pg[0] = g0; pg[1] = g1; pb[0] = b0; pb[1] = b1;
        }
      }
    }
    s1 = RMS ? 0.0f : warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    uint4* op = reinterpret_cast<uint4*>(dx + row * D);
    const uint4* rp = dres_in ? reinterpret_cast<const uint4*>(dres_in + row * D) : nullptr;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float xv[8], dv[8], g[8], o[8];
        unpack8(xr[i], xv);
        unpack8(dr[i], dv);
        unpack8(__ldg(gp + c), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float h = (xv[j] - mean) * rstd;
          o[j] = rstd * (dv[j] * g[j] - s1 - h * s2);
        }
        if (rp) {
          float r[8];
          unpack8(rp[c], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        op[c] = pack8(o);
      }
    }
  }
  if (REGACC) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { mine[c * 8 + j] = accg[(REGACC ? i : 0) * 8 + j]; mine[D + c * 8 + j] = accb[(REGACC ? i : 0) * 8 + j]; }
      }
    }
  }
  __syncthreads();
  float* out = partial + (size_t)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < NORM_WARPS; ++w) a += sm_part[(size_t)w * 2 * D + i];
    out[i] = a;
  }
}

// The same backward pass for rows of up to 1024 elements, fed by bulk copies.  Each warp owns a
// ring of row slots in shared memory (x, dy and the residual gradient of a row per slot); lane 0
// keeps `stages` rows of copies in flight, so the loads of later rows never wait for the arithmetic
// of the current one and the number of bytes in flight per SM no longer depends on registers.
// One CTA of NORM_RING_WARPS warps per SM; dgamma / dbeta partials stay in registers and are
// combined through the ring's memory at the end.  partial: [gridDim.x, 2, D] fp32.
constexpr int NORM_RING_WARPS = 8;
template <int MAXV, bool RMS>
__global__ void __launch_bounds__(NORM_RING_WARPS * 32, 1)
norm_bwd_ring_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres_in,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int D,
                     int stages, int* status) {
  extern __shared__ __align__(128) uint8_t ring_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  const int nt = dres_in ? 3 : 2;                      // tensors per slot
  const uint32_t row_bytes = (uint32_t)D * 2u;
  const uint32_t slot_bytes = 3u * row_bytes;
  const uint32_t ring_bytes = (uint32_t)NORM_RING_WARPS * stages * slot_bytes;
  uint8_t* my_ring = ring_raw + (size_t)warp * stages * slot_bytes;
  const uint32_t bar0 = smem_u32(ring_raw) + ring_bytes + (uint32_t)warp * stages * 8u;
  volatile int* dead = reinterpret_cast<volatile int*>(ring_raw + ring_bytes + NORM_RING_WARPS * stages * 8);
  if (threadIdx.x == 0) *dead = 0;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(bar0 + 8u * s, 1);
    mbar_fence_init();
  }
  __syncthreads();
  const long long first = (long long)blockIdx.x * NORM_RING_WARPS + warp;
  const long long stride = (long long)gridDim.x * NORM_RING_WARPS;
  auto post = [&](long long row, int s) {               // lane 0 only
    const uint32_t bar = bar0 + 8u * s;
    const uint32_t dst = smem_u32(my_ring) + (uint32_t)s * slot_bytes;
    mbar_expect_tx(bar, (uint32_t)nt * row_bytes);
    bulk_load_1d(dst, x + row * D, row_bytes, bar);
    bulk_load_1d(dst + row_bytes, dy + row * D, row_bytes, bar);
    if (dres_in) bulk_load_1d(dst + 2u * row_bytes, dres_in + row * D, row_bytes, bar);
  };
  if (lane == 0)
    for (int s = 0; s < stages; ++s)
      if (first + s * stride < rows) post(first + s * stride, s);
  const uint4* gp = reinterpret_cast<const uint4*>(gamma);
  float accg[MAXV * 8], accb[MAXV * 8];
  uint4 gr[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    gr[i] = (lane + i * 32 < nvec) ? __ldg(gp + lane + i * 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < 8; ++j) { accg[i * 8 + j] = 0.0f; accb[i * 8 + j] = 0.0f; }
  }
  bool ok = true;
  uint32_t k = 0;
  // the row statistics are fetched one row ahead as well
  float mean_next = 0.0f, rstd_next = 0.0f;
  if (first < rows) { mean_next = RMS ? 0.0f : mean_in[first]; rstd_next = rstd_in[first]; }
  for (long long row = first; row < rows && ok; row += stride, ++k) {
    const int s = (int)(k % (uint32_t)stages);
    const float mean = mean_next, rstd = rstd_next;
    if (row + stride < rows) { mean_next = RMS ? 0.0f : mean_in[row + stride]; rstd_next = rstd_in[row + stride]; }
    if (!mbar_wait(bar0 + 8u * s, (k / (uint32_t)stages) & 1u, dead, status, 3100)) { ok = false; break; }
    const uint4* slot = reinterpret_cast<const uint4*>(my_ring + (size_t)s * slot_bytes);
    uint4 xr[MAXV], dr[MAXV], rr[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        xr[i] = slot[c];
        dr[i] = slot[nvec + c];
        rr[i] = dres_in ? slot[2 * nvec + c] : make_uint4(0, 0, 0, 0);
      }
    }
    // every lane holds its part of the row: the slot can take the row `stages` ahead
    __syncwarp();
    if (lane == 0 && row + (long long)stages * stride < rows) post(row + (long long)stages * stride, s);
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      if (lane + i * 32 < nvec) {
        float xv[8], dv[8], g[8];
        unpack8(xr[i], xv);
        unpack8(dr[i], dv);
        unpack8(gr[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float h = (xv[j] - mean) * rstd;
          const float t = dv[j] * g[j];
          s1 += t;
          s2 += t * h;
          accg[i * 8 + j] += dv[j] * h;
          accb[i * 8 + j] += dv[j];
        }
      }
    }
    s1 = RMS ? 0.0f : warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    uint4* op = reinterpret_cast<uint4*>(dx + row * D);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float xv[8], dv[8], g[8], r[8], o[8];
        unpack8(xr[i], xv);
        unpack8(dr[i], dv);
        unpack8(gr[i], g);
        unpack8(rr[i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float h = (xv[j] - mean) * rstd;
          o[j] = rstd * (dv[j] * g[j] - s1 - h * s2) + r[j];
        }
        op[c] = pack8(o);
      }
    }
  }
  // no copy is in flight any more (every posted row was waited for, unless a wait gave up, in
  // which case the ring is left alone): the ring's memory now combines the warps' partial sums
  __syncthreads();
  if (*dead) { __nanosleep(100000); return; }
  float* sm_part = reinterpret_cast<float*>(ring_raw);   // [NORM_RING_WARPS][2][D]
  float* mine = sm_part + (size_t)warp * 2 * D;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[c * 8 + j] = accg[i * 8 + j]; mine[D + c * 8 + j] = accb[i * 8 + j]; }
    }
  }
  __syncthreads();
  float* out = partial + (size_t)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < NORM_RING_WARPS; ++w) a += sm_part[(size_t)w * 2 * D + i];
    out[i] = a;
  }
}

// dgamma[c] (+)= sum_p partial[p][0][c]; dbeta likewise.  fp32 outputs.
// One CTA per 32 columns of the [2, D] partial rows: 32 x 8 threads, each sums every 8th partial.
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(const float* __restrict__ partial, int nparts, int D,
                       float* __restrict__ dgamma, float* __restrict__ dbeta, int accumulate) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;                 // column of the concatenated [dgamma | dbeta] row
  float a = 0.0f;
  if (c < 2 * D)
    for (int p = py; p < nparts; p += 8) a += partial[(size_t)p * 2 * D + c];
  sh[py][cx] = a;
  __syncthreads();
  if (py == 0 && c < 2 * D) {
#pragma unroll
    for (int w = 1; w < 8; ++w) a += sh[w][cx];
    float* dst = c < D ? dgamma : dbeta;
    const int cc = c < D ? c : c - D;
    if (dst) dst[cc] = accumulate ? dst[cc] + a : a;
  }
}

}  // namespace cgk

using namespace cgk;

// CTAs of the backward kernel: as many as fit an SM by shared memory (each holds 2 * D floats per
// warp), up to eight per SM: a streaming kernel needs that many warps to keep the memory pipe full.
static int norm_bwd_cap(int dev, int D) {
  const size_t smem = (size_t)NORM_WARPS * 2 * D * sizeof(float);
  int per_sm = (int)((200 * 1024) / (smem + 1024));
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  return sm_count(dev) * per_sm;
}

// rms = 0: LayerNorm (beta may be null), rms = 1: RMSNorm (beta ignored, mean unused).
// residual / sum_out / mean / rstd may be null.  D must be a multiple of 8, D <= 8192.
CGK_API int cgk_norm_forward(const void* x, const void* residual, const void* gamma,
                             const void* beta, void* y, void* sum_out, float* mean, float* rstd,
                             int rows, int D, float eps, int rms, void* stream_) {
  CGK_REQUIRE(x && gamma && y, "cgk_norm_forward: null pointer");
  CGK_REQUIRE(D > 0 && D % 8 == 0 && D <= 8192, "cgk_norm_forward: D=%d must be a multiple of 8, <= 8192", D);
  if (rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream_;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  int grid = (rows + NORM_WARPS - 1) / NORM_WARPS;
  int cap = sm_count(dev) * 16;
  if (grid > cap) grid = cap;
  const int need = (D / 8 + 31) / 32;
#define LAUNCH(MAXV)                                                                          \
  if (rms)                                                                                    \
    norm_fwd_kernel<MAXV, true><<<grid, NORM_WARPS * 32, 0, st>>>(                            \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)gamma, \
        nullptr, (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, mean, rstd, rows, D, eps);       \
  else                                                                                        \
    norm_fwd_kernel<MAXV, false><<<grid, NORM_WARPS * 32, 0, st>>>(                           \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)gamma, \
        (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, mean, rstd,   \
        rows, D, eps);
  if (need <= 1) { LAUNCH(1) }
  else if (need <= 2) { LAUNCH(2) }
  else if (need <= 4) { LAUNCH(4) }
  else if (need <= 8) { LAUNCH(8) }
  else if (need <= 16) { LAUNCH(16) }
  else { LAUNCH(32) }
#undef LAUNCH
  CGK_LAUNCH_CHECK();
  return 0;
}

// Number of fp32 elements the backward needs in `scratch`.
CGK_API long long cgk_norm_backward_scratch_elems(int rows, int D) {
  int dev = 0;
  cudaGetDevice(&dev);
  int grid = (rows + NORM_WARPS - 1) / NORM_WARPS;
  int cap = norm_bwd_cap(dev, D);
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return (long long)grid * 2 * D;
}

// dx = norm backward (+ dres_in if given).  dgamma / dbeta are fp32 and are
// overwritten, or added to when accumulate != 0.  scratch: see above.
CGK_API int cgk_norm_backward(const void* dy, const void* x, const void* gamma, const float* mean,
                              const float* rstd, const void* dres_in, void* dx, float* dgamma,
                              float* dbeta, float* scratch, int rows, int D, int rms,
                              int accumulate, void* stream_) {
  CGK_REQUIRE(dy && x && gamma && rstd && dx && scratch, "cgk_norm_backward: null pointer");
  CGK_REQUIRE(rms || mean, "cgk_norm_backward: LayerNorm needs the saved mean");
  CGK_REQUIRE(D > 0 && D % 8 == 0 && D <= 8192, "cgk_norm_backward: D=%d must be a multiple of 8, <= 8192", D);
  if (rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream_;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const int need = (D / 8 + 31) / 32;
  const bool aligned = (((uintptr_t)dy | (uintptr_t)x | (uintptr_t)dres_in) & 15u) == 0;
  if (need <= 4 && aligned) {
    // rows of up to 1024 elements: the bulk-copy ring kernel, one CTA per SM
    int stages = (int)((200 * 1024 - 1024) / ((size_t)NORM_RING_WARPS * 3 * D * 2));
    if (stages > 6) stages = 6;
    int grid = (rows + NORM_RING_WARPS - 1) / NORM_RING_WARPS;
    if (grid > sm_count(dev)) grid = sm_count(dev);
    const size_t smem = (size_t)NORM_RING_WARPS * stages * 3 * D * 2 + NORM_RING_WARPS * stages * 8 + 16;
#define LAUNCH_RING(MAXV)                                                                          \
  {                                                                                                \
    if (rms) {                                                                                     \
      CGK_CUDA_CHECK(cudaFuncSetAttribute(norm_bwd_ring_kernel<MAXV, true>,                        \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      norm_bwd_ring_kernel<MAXV, true><<<grid, NORM_RING_WARPS * 32, smem, st>>>(                  \
          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean,    \
          rstd, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, scratch, rows, D, stages,       \
          device_status(dev));                                                                     \
    } else {                                                                                       \
      CGK_CUDA_CHECK(cudaFuncSetAttribute(norm_bwd_ring_kernel<MAXV, false>,                       \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      norm_bwd_ring_kernel<MAXV, false><<<grid, NORM_RING_WARPS * 32, smem, st>>>(                 \
          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean,    \
          rstd, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, scratch, rows, D, stages,       \
          device_status(dev));                                                                     \
    }                                                                                              \
  }
    if (need <= 1) LAUNCH_RING(1)
    else if (need <= 2) LAUNCH_RING(2)
    else if (need <= 3) LAUNCH_RING(3)
    else LAUNCH_RING(4)
#undef LAUNCH_RING
    CGK_LAUNCH_CHECK();
    norm_bwd_reduce_kernel<<<(2 * D + 31) / 32, 256, 0, st>>>(scratch, grid, D, dgamma, dbeta, accumulate);
    CGK_LAUNCH_CHECK();
    return 0;
  }
  int grid = (rows + NORM_WARPS - 1) / NORM_WARPS;
  int cap = norm_bwd_cap(dev, D);
  if (grid > cap) grid = cap;
  const size_t smem = (size_t)NORM_WARPS * 2 * D * sizeof(float);
#define LAUNCH(MAXV)                                                                              \
  {                                                                                               \
    if (rms) {                                                                                    \
      CGK_CUDA_CHECK(cudaFuncSetAttribute(norm_bwd_kernel<MAXV, true>,                            \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      norm_bwd_kernel<MAXV, true><<<grid, NORM_WARPS * 32, smem, st>>>(                           \
          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean,   \
          rstd, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, scratch, rows, D);             \
    } else {                                                                                      \
      CGK_CUDA_CHECK(cudaFuncSetAttribute(norm_bwd_kernel<MAXV, false>,                           \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      norm_bwd_kernel<MAXV, false><<<grid, NORM_WARPS * 32, smem, st>>>(                          \
          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean,   \
          rstd, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, scratch, rows, D);             \
    }                                                                                             \
  }
  if (need <= 1) LAUNCH(1)
  else if (need <= 2) LAUNCH(2)
  else if (need <= 4) LAUNCH(4)
  else if (need <= 8) LAUNCH(8)
  else if (need <= 16) LAUNCH(16)
  else LAUNCH(32)
#undef LAUNCH
  CGK_LAUNCH_CHECK();
  norm_bwd_reduce_kernel<<<(2 * D + 31) / 32, 256, 0, st>>>(scratch, grid, D, dgamma, dbeta, accumulate);
  CGK_LAUNCH_CHECK();
  return 0;
}
