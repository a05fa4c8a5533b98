// Row softmax and fused softmax-cross-entropy for large vocabularies
// (50 304 / 32 000 columns), bf16 logits, fp32 statistics.
//
//  * cgk_softmax_ce_fused: one CTA per row; pass 1 = online max / sum-exp,
//    pass 2 (row re-read from L2) writes d(logits) in place or to a second
//    buffer.  Loss per row goes to an fp32 vector.
//  * cgk_ce_stats + cgk_ce_backward: the same split in two so a vocabulary-
//    parallel run can all-reduce (max, sum-exp, target-logit) between them.
//  * cgk_softmax_rows / cgk_softmax_rows_backward: plain row softmax, fp32.
//  * cgk_softmax_dropout_residual (+ backward): out = dropout(softmax(x)) + residual in one
//    pass over the row, fp32 or bf16; the multiplier is either a tensor (the reference's
//    softmax -> mul -> add pattern, src/jit/fusion.c:152-190) or a keep mask drawn from
//    (seed, element index), which the backward pass regenerates.
//
// Reference counterparts: cg_cross_entropy_loss (src/layers/loss.c:44-78, always
// applies softmax, clamps p at 1e-7), cg_cuda_softmax_forward/backward
// (src/cuda/tensor_kernels.c:699-771, host loops).
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"
#include <cuda_fp16.h>

namespace cgk {

constexpr int CE_THREADS = 256;

struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  MaxSum r;
  r.m = fmaxf(a.m, b.m);
  if (r.m == -INFINITY) { r.s = 0.0f; return r; }
  r.s = a.s * __expf(a.m - r.m) + b.s * __expf(b.m - r.m);
  return r;
}
__device__ __forceinline__ void ms_push(MaxSum& a, float x) {
  if (x > a.m) {
    a.s = a.s * __expf(a.m - x) + 1.0f;
    a.m = x;
  } else {
    a.s += __expf(x - a.m);
  }
}

__device__ MaxSum block_maxsum(MaxSum v, MaxSum* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t;
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v = ms_combine(v, t);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  MaxSum r = sh[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = ms_combine(r, sh[w]);
  __syncthreads();
  return r;
}

__device__ __forceinline__ MaxSum row_maxsum_bf16(const __nv_bfloat16* row, int V) {
  MaxSum a;
  a.m = -INFINITY;
  a.s = 0.0f;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int nvec = V >> 3;
    const uint4* p = reinterpret_cast<const uint4*>(row);
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      uint4 u = p[c];
      float2 f;
      f = unpack_bf16x2(u.x); ms_push(a, f.x); ms_push(a, f.y);
      f = unpack_bf16x2(u.y); ms_push(a, f.x); ms_push(a, f.y);
      f = unpack_bf16x2(u.z); ms_push(a, f.x); ms_push(a, f.y);
      f = unpack_bf16x2(u.w); ms_push(a, f.x); ms_push(a, f.y);
    }
    for (int c = (nvec << 3) + threadIdx.x; c < V; c += blockDim.x) ms_push(a, __bfloat162float(row[c]));
  } else {
    for (int c = threadIdx.x; c < V; c += blockDim.x) ms_push(a, __bfloat162float(row[c]));
  }
  return a;
}

// dl[c] = (exp(l[c] - lse) - [c == tgt]) * scale   for one row
__device__ __forceinline__ void row_ce_grad(const __nv_bfloat16* row, __nv_bfloat16* drow, int V,
                                            float lse, int tgt, float scale) {
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(drow) & 15) == 0);
  int done = 0;
  if (vec) {
    const int nvec = V >> 3;
    const uint4* p = reinterpret_cast<const uint4*>(row);
    uint4* q = reinterpret_cast<uint4*>(drow);
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      uint4 u = p[c];
      float f[8];
      float2 t;
      t = unpack_bf16x2(u.x); f[0] = t.x; f[1] = t.y;
      t = unpack_bf16x2(u.y); f[2] = t.x; f[3] = t.y;
      t = unpack_bf16x2(u.z); f[4] = t.x; f[5] = t.y;
      t = unpack_bf16x2(u.w); f[6] = t.x; f[7] = t.y;
      const int base = c << 3;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float pr = __expf(f[j] - lse);
        if (base + j == tgt) pr -= 1.0f;
        f[j] = pr * scale;
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
      q[c] = o;
    }
    done = nvec << 3;
  }
  for (int c = done + threadIdx.x; c < V; c += blockDim.x) {
    float pr = __expf(__bfloat162float(row[c]) - lse);
    if (c == tgt) pr -= 1.0f;
    drow[c] = __float2bfloat16(pr * scale);
  }
}

__global__ void __launch_bounds__(CE_THREADS)
softmax_ce_fused_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                        float* __restrict__ loss_rows, __nv_bfloat16* dlogits, int R, int V,
                        long long ld, float scale_f, const float* __restrict__ scale_ptr,
                        long long ignore_index) {
  __shared__ MaxSum sh[CE_THREADS / 32];
  const float scale = scale_f * (scale_ptr ? *scale_ptr : 1.0f);
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const __nv_bfloat16* row = logits + (long long)r * ld;
    const long long tgt = targets[r];
    if (tgt != ignore_index) (void)CGK_IDX(tgt, V);        // debug build: a label outside the vocabulary is reported, not just skipped
    const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
    MaxSum ms = block_maxsum(row_maxsum_bf16(row, V), sh);
    const float lse = ms.m + __logf(ms.s);
    if (threadIdx.x == 0 && loss_rows)
      loss_rows[r] = ignored ? 0.0f : (lse - __bfloat162float(row[tgt]));
    __syncthreads();  // loss reads the target logit before it is overwritten in place
    if (dlogits) row_ce_grad(row, dlogits + (long long)r * ld, V, lse, ignored ? -1 : (int)tgt,
                             ignored ? 0.0f : scale);
  }
}

// The fused kernel for rows that fit shared memory twice (V * 2 bytes <= ~110 KB: vocabularies up to
// ~56 000): one persistent CTA per SM, rows arrive by bulk copy one row ahead of the arithmetic, and
// every pass after the first reads shared memory, so each logit crosses HBM once in and once out.
// Pass A: row maximum.  Pass B: e = exp(x - max), summed in fp32 and written back over the row as
// fp16 (values in (0, 1]: 11 bits of mantissa, more than the bf16 gradient keeps), so that the
// exponential is taken once per element - at 16 per clock and SM a second one would cost as much
// as the memory traffic.  Pass C: d(logit) = (e / sum - [c == target]) * scale, 16 bytes per store.
constexpr int CE_SMEM_THREADS = 512;
__global__ void __launch_bounds__(CE_SMEM_THREADS, 1)
softmax_ce_smem_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                       float* __restrict__ loss_rows, __nv_bfloat16* dlogits, int R, int V, long long ld,
                       float scale_f, const float* __restrict__ scale_ptr, long long ignore_index,
                       int row_stride_bytes, int* status) {
  extern __shared__ __align__(128) uint8_t ce_raw[];
  __shared__ float red[CE_SMEM_THREADS / 32];
  __shared__ float bcast;
  const uint32_t bar0 = smem_u32(ce_raw) + 2u * (uint32_t)row_stride_bytes;
  volatile int* dead = reinterpret_cast<volatile int*>(ce_raw + 2 * (size_t)row_stride_bytes + 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)V * 2u;
  if (threadIdx.x == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const float scale = scale_f * (scale_ptr ? *scale_ptr : 1.0f);
  auto post = [&](long long r, int s) {     // thread 0 only
    mbar_expect_tx(bar0 + 8u * s, row_bytes);
    bulk_load_1d(smem_u32(ce_raw) + (uint32_t)s * (uint32_t)row_stride_bytes, logits + r * ld, row_bytes, bar0 + 8u * s);
  };
  const long long first = blockIdx.x, stride = gridDim.x;
  if (threadIdx.x == 0) {
    if (first < R) post(first, 0);
    if (first + stride < R) post(first + stride, 1);
  }
  auto block_max = [&](float v) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = red[0];
      for (int w = 1; w < CE_SMEM_THREADS / 32; ++w) a = fmaxf(a, red[w]);
      bcast = a;
    }
    __syncthreads();
    return bcast;
  };
  auto block_sum = [&](float v) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                        // everyone has read the previous broadcast
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.0f;
      for (int w = 0; w < CE_SMEM_THREADS / 32; ++w) a += red[w];
      bcast = a;
    }
    __syncthreads();
    return bcast;
  };
  const int nvec = V >> 3;
  const float LOG2E = 1.4426950408889634f;
  uint32_t k = 0;
  for (long long r = first; r < R; r += stride, ++k) {
    const int s = (int)(k & 1u);
    uint4* buf = reinterpret_cast<uint4*>(ce_raw + (size_t)s * row_stride_bytes);
    const long long tgt = targets[r];
    if (tgt != ignore_index) (void)CGK_IDX(tgt, V);        // debug build: a label outside the vocabulary is reported, not just skipped
    const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
    if (!mbar_wait(bar0 + 8u * s, (k >> 1) & 1u, dead, status, 3200)) break;
    const float x_t = ignored ? 0.0f : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(buf)[tgt]);
    // pass A: maximum
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < nvec; c += CE_SMEM_THREADS) {
      const uint4 u = buf[c];
      float2 f;
      f = unpack_bf16x2(u.x); mx = fmaxf(mx, fmaxf(f.x, f.y));
      f = unpack_bf16x2(u.y); mx = fmaxf(mx, fmaxf(f.x, f.y));
      f = unpack_bf16x2(u.z); mx = fmaxf(mx, fmaxf(f.x, f.y));
      f = unpack_bf16x2(u.w); mx = fmaxf(mx, fmaxf(f.x, f.y));
    }
    mx = block_max(mx);                      // (its barriers also order x_t's read before pass B's writes)
    const float neg = (mx == -INFINITY) ? 0.0f : -mx * LOG2E;
    // pass B: exponentials, once per element, kept as fp16 in place
    float sum = 0.0f;
    for (int c = threadIdx.x; c < nvec; c += CE_SMEM_THREADS) {
      const uint4 u = buf[c];
      float e[8];
      float2 f;
      f = unpack_bf16x2(u.x); e[0] = fast_exp2(fmaf(f.x, LOG2E, neg)); e[1] = fast_exp2(fmaf(f.y, LOG2E, neg));
      f = unpack_bf16x2(u.y); e[2] = fast_exp2(fmaf(f.x, LOG2E, neg)); e[3] = fast_exp2(fmaf(f.y, LOG2E, neg));
      f = unpack_bf16x2(u.z); e[4] = fast_exp2(fmaf(f.x, LOG2E, neg)); e[5] = fast_exp2(fmaf(f.y, LOG2E, neg));
      f = unpack_bf16x2(u.w); e[6] = fast_exp2(fmaf(f.x, LOG2E, neg)); e[7] = fast_exp2(fmaf(f.y, LOG2E, neg));
      sum += ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
      uint4 o;
      __half2 h;
      h = __floats2half2_rn(e[0], e[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2half2_rn(e[2], e[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2half2_rn(e[4], e[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2half2_rn(e[6], e[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
      buf[c] = o;
    }
    sum = block_sum(sum);
    const float lse = mx + __logf(sum);
    if (threadIdx.x == 0 && loss_rows) loss_rows[r] = ignored ? 0.0f : (lse - x_t);
    // pass C: gradient
    if (dlogits) {
      const float inv = ignored ? 0.0f : scale / sum;
      const float hot = ignored ? 0.0f : scale;
      uint4* q = reinterpret_cast<uint4*>(dlogits + r * ld);
      const int tv = ignored ? -1 : (int)(tgt >> 3), tj = (int)(tgt & 7);
      for (int c = threadIdx.x; c < nvec; c += CE_SMEM_THREADS) {
        const uint4 u = buf[c];
        float g[8];
        float2 f;
        f = __half22float2(*reinterpret_cast<const __half2*>(&u.x)); g[0] = f.x * inv; g[1] = f.y * inv;
        f = __half22float2(*reinterpret_cast<const __half2*>(&u.y)); g[2] = f.x * inv; g[3] = f.y * inv;
        f = __half22float2(*reinterpret_cast<const __half2*>(&u.z)); g[4] = f.x * inv; g[5] = f.y * inv;
        f = __half22float2(*reinterpret_cast<const __half2*>(&u.w)); g[6] = f.x * inv; g[7] = f.y * inv;
        if (c == tv) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j == tj) g[j] -= hot;
        }
        uint4 o;
        o.x = pack_bf16x2(g[0], g[1]); o.y = pack_bf16x2(g[2], g[3]);
        o.z = pack_bf16x2(g[4], g[5]); o.w = pack_bf16x2(g[6], g[7]);
        q[c] = o;
      }
    }
    // every thread is done with this buffer: it can take the row two steps ahead
    __syncthreads();
    if (threadIdx.x == 0 && r + 2 * stride < R) post(r + 2 * stride, s);
  }
  if (*dead) __nanosleep(100000);
}

// Per-row partial statistics of a vocabulary shard [vocab_start, vocab_start+V).
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                long long vocab_start, float* __restrict__ rowmax, float* __restrict__ rowsum,
                float* __restrict__ tgt_logit, int R, int V, long long ld) {
  __shared__ MaxSum sh[CE_THREADS / 32];
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const __nv_bfloat16* row = logits + (long long)r * ld;
    MaxSum ms = block_maxsum(row_maxsum_bf16(row, V), sh);
    if (threadIdx.x == 0) {
      rowmax[r] = ms.m;
      rowsum[r] = ms.s;
      const long long t = targets[r] - vocab_start;
      tgt_logit[r] = (t >= 0 && t < V) ? __bfloat162float(row[t]) : 0.0f;
    }
  }
}

__global__ void __launch_bounds__(CE_THREADS)
ce_backward_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                   long long vocab_start, const float* __restrict__ lse,
                   __nv_bfloat16* dlogits, int R, int V, long long ld, float scale_f,
                   const float* __restrict__ scale_ptr, long long ignore_index) {
  const float scale = scale_f * (scale_ptr ? *scale_ptr : 1.0f);
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const long long tg = targets[r];
    const bool ignored = (tg == ignore_index);
    const long long t = tg - vocab_start;
    row_ce_grad(logits + (long long)r * ld, dlogits + (long long)r * ld, V, lse[r],
                (t >= 0 && t < V) ? (int)t : -1, ignored ? 0.0f : scale);
  }
}

// fp32 row softmax.  y may alias x.
__global__ void __launch_bounds__(CE_THREADS)
softmax_rows_kernel(const float* __restrict__ x, float* y, int R, int V, float inv_temp) {
  __shared__ MaxSum sh[CE_THREADS / 32];
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const float* row = x + (long long)r * V;
    float* out = y + (long long)r * V;
    MaxSum a;
    a.m = -INFINITY;
    a.s = 0.0f;
    for (int c = threadIdx.x; c < V; c += blockDim.x) ms_push(a, row[c] * inv_temp);
    MaxSum ms = block_maxsum(a, sh);
    const float inv = 1.0f / ms.s;
    for (int c = threadIdx.x; c < V; c += blockDim.x) out[c] = __expf(row[c] * inv_temp - ms.m) * inv;
    __syncthreads();
  }
}

// dx = y * (dy - sum(dy * y))
__global__ void __launch_bounds__(CE_THREADS)
softmax_rows_bwd_kernel(const float* __restrict__ y, const float* __restrict__ dy, float* dx, int R,
                        int V) {
  __shared__ float sh[CE_THREADS / 32];
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const float* yr = y + (long long)r * V;
    const float* dr = dy + (long long)r * V;
    float s = 0.0f;
    for (int c = threadIdx.x; c < V; c += blockDim.x) s += yr[c] * dr[c];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < CE_THREADS / 32; ++w) tot += sh[w];
    __syncthreads();
    for (int c = threadIdx.x; c < V; c += blockDim.x) dx[(long long)r * V + c] = yr[c] * (dr[c] - tot);
  }
}

template <typename T> __device__ __forceinline__ float ldv(const T* p, long long i);
template <> __device__ __forceinline__ float ldv<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldv<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stv(T* p, long long i, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stv<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// out[r, c] = softmax(x[r, :])[c] * w(r, c) + residual[r, c], with w = mul[r, c] when a multiplier
// tensor is given, else keep(seed, r * V + c) / (1 - p) (1 when p == 0).  One CTA per row at a time.
template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
softmax_dropout_residual_kernel(const T* __restrict__ x, const T* __restrict__ mul, const T* __restrict__ residual,
                                T* __restrict__ out, int R, int V, float p, unsigned long long seed) {
  __shared__ MaxSum sh[CE_THREADS / 32];
  const float keep_scale = 1.0f / (1.0f - p);
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const long long base = (long long)r * V;
    MaxSum a;
    a.m = -INFINITY;
    a.s = 0.0f;
    for (int c = threadIdx.x; c < V; c += blockDim.x) ms_push(a, ldv<T>(x, base + c));
    const MaxSum ms = block_maxsum(a, sh);
    const float inv = 1.0f / ms.s;
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
      float v = __expf(ldv<T>(x, base + c) - ms.m) * inv;
      if (mul) v *= ldv<T>(mul, base + c);
      else if (p > 0.0f) v = dropout_keep(seed, base + c, thresh) ? v * keep_scale : 0.0f;
      if (residual) v += ldv<T>(residual, base + c);
      stv<T>(out, base + c, v);
    }
    __syncthreads();
  }
}

// dx = s * (g - sum(g * s)) with s = softmax(x) recomputed from x and g = dy * w.
template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
softmax_dropout_residual_bwd_kernel(const T* __restrict__ x, const T* __restrict__ mul, const T* __restrict__ dy,
                                    T* __restrict__ dx, int R, int V, float p, unsigned long long seed) {
  __shared__ MaxSum sh[CE_THREADS / 32];
  __shared__ float shf[CE_THREADS / 32];
  const float keep_scale = 1.0f / (1.0f - p);
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const long long base = (long long)r * V;
    MaxSum a;
    a.m = -INFINITY;
    a.s = 0.0f;
    for (int c = threadIdx.x; c < V; c += blockDim.x) ms_push(a, ldv<T>(x, base + c));
    const MaxSum ms = block_maxsum(a, sh);
    const float inv = 1.0f / ms.s;
    auto weight = [&](int c) {
      if (mul) return ldv<T>(mul, base + c);
      if (p > 0.0f) return dropout_keep(seed, base + c, thresh) ? keep_scale : 0.0f;
      return 1.0f;
    };
    float dot = 0.0f;
    for (int c = threadIdx.x; c < V; c += blockDim.x)
      dot += ldv<T>(dy, base + c) * weight(c) * __expf(ldv<T>(x, base + c) - ms.m) * inv;
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) shf[threadIdx.x >> 5] = dot;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < CE_THREADS / 32; ++w) tot += shf[w];
    __syncthreads();
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
      const float s = __expf(ldv<T>(x, base + c) - ms.m) * inv;
      stv<T>(dx, base + c, s * (ldv<T>(dy, base + c) * weight(c) - tot));
    }
  }
}

}  // namespace cgk

using namespace cgk;

static int ce_grid(int R) {
  int dev = 0;
  cudaGetDevice(&dev);
  int cap = sm_count(dev) * 8;
  return R < cap ? (R < 1 ? 1 : R) : cap;
}

// loss_rows[r] = lse(row r) - logit[r, target[r]] (0 for ignored rows).
// dlogits (may be null, may alias logits) = (softmax - onehot) * scale_f * (*scale_ptr).
CGK_API int cgk_softmax_ce_fused(const void* logits, const long long* targets, float* loss_rows,
                                 void* dlogits, int R, int V, long long ld, float scale_f,
                                 const float* scale_ptr, long long ignore_index, void* stream) {
  CGK_REQUIRE(logits && targets, "cgk_softmax_ce_fused: null pointer");
  CGK_REQUIRE(R >= 0 && V > 0 && ld >= V, "cgk_softmax_ce_fused: bad shape");
  if (R == 0) return 0;
  // rows that fit shared memory twice take the single-read kernel
  const long long row_stride = ((long long)V * 2 + 127) / 128 * 128;
  const bool aligned = (V % 8) == 0 && (ld % 8) == 0 && (((uintptr_t)logits) & 15) == 0 &&
                       (!dlogits || (((uintptr_t)dlogits) & 15) == 0);
  if (aligned && 2 * row_stride + 64 <= 220 * 1024 && V >= 4096) {
    int dev = 0;
    CGK_CUDA_CHECK(cudaGetDevice(&dev));
    const int smem = (int)(2 * row_stride + 64);
    CGK_CUDA_CHECK(cudaFuncSetAttribute(softmax_ce_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    int grid = sm_count(dev);
    if (grid > R) grid = R;
    softmax_ce_smem_kernel<<<grid, CE_SMEM_THREADS, smem, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)logits, targets, loss_rows, (__nv_bfloat16*)dlogits, R, V, ld, scale_f, scale_ptr,
        ignore_index, (int)row_stride, device_status(dev));
    CGK_LAUNCH_CHECK();
    return 0;
  }
  softmax_ce_fused_kernel<<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, targets, loss_rows, (__nv_bfloat16*)dlogits, R, V, ld, scale_f,
      scale_ptr, ignore_index);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_ce_stats(const void* logits, const long long* targets, long long vocab_start,
                         float* rowmax, float* rowsum, float* tgt_logit, int R, int V, long long ld,
                         void* stream) {
  CGK_REQUIRE(logits && targets && rowmax && rowsum && tgt_logit, "cgk_ce_stats: null pointer");
  if (R == 0) return 0;
  ce_stats_kernel<<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, targets, vocab_start, rowmax, rowsum, tgt_logit, R, V, ld);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_ce_backward(const void* logits, const long long* targets, long long vocab_start,
                            const float* lse, void* dlogits, int R, int V, long long ld,
                            float scale_f, const float* scale_ptr, long long ignore_index,
                            void* stream) {
  CGK_REQUIRE(logits && targets && lse && dlogits, "cgk_ce_backward: null pointer");
  if (R == 0) return 0;
  ce_backward_kernel<<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, targets, vocab_start, lse, (__nv_bfloat16*)dlogits, R, V, ld,
      scale_f, scale_ptr, ignore_index);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_softmax_rows(const float* x, float* y, int R, int V, float inv_temp, void* stream) {
  CGK_REQUIRE(x && y && V > 0, "cgk_softmax_rows: bad argument");
  if (R == 0) return 0;
  softmax_rows_kernel<<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(x, y, R, V, inv_temp);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_softmax_rows_backward(const float* y, const float* dy, float* dx, int R, int V,
                                      void* stream) {
  CGK_REQUIRE(y && dy && dx && V > 0, "cgk_softmax_rows_backward: bad argument");
  if (R == 0) return 0;
  softmax_rows_bwd_kernel<<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(y, dy, dx, R, V);
  CGK_LAUNCH_CHECK();
  return 0;
}

// dtype: 0 fp32, 1 bf16 (all four tensors alike).  mul and residual may be null; with mul == null and
// p > 0 the multiplier is the dropout mask of (seed, element index).  out may alias residual.
CGK_API int cgk_softmax_dropout_residual(int dtype, const void* x, const void* mul, const void* residual, void* out,
                                         int R, int V, float p, unsigned long long seed, void* stream) {
  CGK_REQUIRE(x && out && V > 0 && R >= 0 && p >= 0.0f && p < 1.0f && (dtype == 0 || dtype == 1),
              "cgk_softmax_dropout_residual: bad argument");
  if (R == 0) return 0;
  if (dtype == 0)
    softmax_dropout_residual_kernel<float><<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
        (const float*)x, (const float*)mul, (const float*)residual, (float*)out, R, V, p, seed);
  else
    softmax_dropout_residual_kernel<__nv_bfloat16><<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)mul, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, R, V, p, seed);
  CGK_LAUNCH_CHECK();
  return 0;
}

// dx for the call above (the gradient of the residual is dy itself; that of mul is not produced).
CGK_API int cgk_softmax_dropout_residual_backward(int dtype, const void* x, const void* mul, const void* dy, void* dx,
                                                  int R, int V, float p, unsigned long long seed, void* stream) {
  CGK_REQUIRE(x && dy && dx && V > 0 && R >= 0 && p >= 0.0f && p < 1.0f && (dtype == 0 || dtype == 1),
              "cgk_softmax_dropout_residual_backward: bad argument");
  if (R == 0) return 0;
  if (dtype == 0)
    softmax_dropout_residual_bwd_kernel<float><<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
        (const float*)x, (const float*)mul, (const float*)dy, (float*)dx, R, V, p, seed);
  else
    softmax_dropout_residual_bwd_kernel<__nv_bfloat16><<<ce_grid(R), CE_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)mul, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, R, V, p, seed);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_BOUNDS_READER(softmax_ce)
