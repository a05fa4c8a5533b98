// Elementwise, reduction, gather/scatter and small layer kernels.
//
// dtype codes used by this file: 0 = fp32, 1 = bf16.  All kernels are
// grid-stride (the reference caps its grid at 65 535 blocks without a stride
// loop, src/cuda/cg_cuda.c:355-363, and so mis-computes tensors above 16.7 M
// elements; these do not).
//
// Reference counterparts: ker_add/sub/mul/div/scale and the unary kernels
// (src/cuda/tensor_kernels.c:26-94), activation forward/backward kernels
// (:135-188), ker_sum_reduce and the host reductions (:97-132, :399-517),
// broadcast ops (src/core/broadcast.c:18-283), dropout / SwiGLU / BatchNorm
// (src/layers/activations.c:17-62,360-642), im2col / max-pool
// (src/layers/conv2d.c:23-421).
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cgk {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}

enum { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_DIV = 3, BIN_MAX = 4, BIN_MIN = 5 };
enum {
  UN_EXP = 0, UN_LOG = 1, UN_SQRT = 2, UN_ABS = 3, UN_NEG = 4, UN_RSQRT = 5, UN_RELU = 6,
  UN_SIGMOID = 7, UN_TANH = 8, UN_GELU = 9, UN_SILU = 10, UN_POW = 11, UN_SCALE = 12,
  UN_ADDS = 13, UN_COPY = 14, UN_SQUARE = 15, UN_RECIP = 16
};

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
  switch (op) {
    case BIN_ADD: return a + b;
    case BIN_SUB: return a - b;
    case BIN_MUL: return a * b;
    case BIN_DIV: return a / b;
    case BIN_MAX: return fmaxf(a, b);
    default: return fminf(a, b);
  }
}
__device__ __forceinline__ float un_apply(int op, float x, float s) {
  switch (op) {
    case UN_EXP: return expf(x);
    case UN_LOG: return logf(x);
    case UN_SQRT: return sqrtf(x);
    case UN_ABS: return fabsf(x);
    case UN_NEG: return -x;
    case UN_RSQRT: return rsqrtf(x);
    case UN_RELU: return fmaxf(x, 0.0f);
    case UN_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case UN_TANH: return tanhf(x);
    case UN_GELU: return gelu_tanh_precise(x);
    case UN_SILU: return silu_f(x);
    case UN_POW: return powf(x, s);
    case UN_SCALE: return x * s;
    case UN_ADDS: return x + s;
    case UN_SQUARE: return x * x;
    case UN_RECIP: return 1.0f / x;
    default: return x;
  }
}
// derivative of the activation given the forward INPUT x (and output y where cheaper)
__device__ __forceinline__ float un_grad(int op, float x, float s) {
  switch (op) {
    case UN_EXP: return expf(x);
    case UN_LOG: return 1.0f / x;
    case UN_SQRT: return 0.5f * rsqrtf(x);
    case UN_ABS: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f);
    case UN_NEG: return -1.0f;
    case UN_RSQRT: return -0.5f * rsqrtf(x) / x;
    case UN_RELU: return x > 0.0f ? 1.0f : 0.0f;
    case UN_SIGMOID: { float y = 1.0f / (1.0f + expf(-x)); return y * (1.0f - y); }
    case UN_TANH: { float y = tanhf(x); return 1.0f - y * y; }
    case UN_GELU: return dgelu_tanh_precise(x);
    case UN_SILU: return dsilu_f(x);
    case UN_POW: return s * powf(x, s - 1.0f);
    case UN_SCALE: return s;
    case UN_SQUARE: return 2.0f * x;
    case UN_RECIP: return -1.0f / (x * x);
    default: return 1.0f;
  }
}

struct BcastDims {
  int nd;
  int shape[8];        // output shape
  long long sa[8];     // element strides of a (0 where broadcast)
  long long sb[8];
};

template <typename T>
__global__ void binary_contig_kernel(const T* __restrict__ a, const T* __restrict__ b, T* out,
                                     long long n, int op) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    stf<T>(out, i, bin_apply(op, ldf<T>(a, i), ldf<T>(b, i)));
}

template <typename T>
__global__ void binary_bcast_kernel(const T* __restrict__ a, const T* __restrict__ b, T* out,
                                    long long n, int op, BcastDims d) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i, oa = 0, ob = 0;
#pragma unroll 1
    for (int k = d.nd - 1; k >= 0; --k) {
      const long long idx = r % d.shape[k];
      r /= d.shape[k];
      oa += idx * d.sa[k];
      ob += idx * d.sb[k];
    }
    stf<T>(out, i, bin_apply(op, ldf<T>(a, oa), ldf<T>(b, ob)));
  }
}

template <typename T>
__global__ void unary_kernel(const T* __restrict__ x, T* out, long long n, int op, float s) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    stf<T>(out, i, un_apply(op, ldf<T>(x, i), s));
}

// dx = dy * f'(x)
template <typename T>
__global__ void unary_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* dx,
                                 long long n, int op, float s) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    stf<T>(dx, i, ldf<T>(dy, i) * un_grad(op, ldf<T>(x, i), s));
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    stf<TO>(out, i, ldf<TI>(x, i));
}

// x = hi + lo with both halves in bf16: the two-term split that lets three bf16 tensor-core
// products (hi*hi + hi*lo + lo*hi) stand in for an fp32 product.
__global__ void split_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* hi, __nv_bfloat16* lo, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = x[i];
    const __nv_bfloat16 h = __float2bfloat16(v);
    hi[i] = h;
    lo[i] = __float2bfloat16(v - __bfloat162float(h));
  }
}

// ---- reductions ---------------------------------------------------------
enum { RED_SUM = 0, RED_MEAN = 1, RED_MAX = 2, RED_MIN = 3 };
__device__ __forceinline__ float red_identity(int op) {
  return op == RED_MAX ? -INFINITY : (op == RED_MIN ? INFINITY : 0.0f);
}
__device__ __forceinline__ float red_combine(int op, float a, float b) {
  return op == RED_MAX ? fmaxf(a, b) : (op == RED_MIN ? fminf(a, b) : a + b);
}
__device__ float block_reduce(int op, float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine(op, v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red_identity(op);
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) r = red_combine(op, r, sh[w]);
  __syncthreads();
  return r;
}

// x viewed as [outer, red, inner]; out[outer, inner].  One CTA per output when
// inner == 1 (row reduction); otherwise one thread per output, looping over red.
template <typename T>
__global__ void reduce_rows_kernel(const T* __restrict__ x, float* __restrict__ out, long long outer,
                                   long long red, int op) {
  __shared__ float sh[32];
  for (long long o = blockIdx.x; o < outer; o += gridDim.x) {
    float v = red_identity(op);
    for (long long i = threadIdx.x; i < red; i += blockDim.x)
      v = red_combine(op, v, ldf<T>(x, o * red + i));
    v = block_reduce(op, v, sh);
    if (threadIdx.x == 0) out[o] = op == RED_MEAN ? v / (float)red : v;
  }
}
template <typename T>
__global__ void reduce_strided_kernel(const T* __restrict__ x, float* __restrict__ out,
                                      long long outer, long long red, long long inner, int op) {
  const long long total = outer * inner;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long o = t / inner, in = t - o * inner;
    float v = red_identity(op);
    for (long long i = 0; i < red; ++i) v = red_combine(op, v, ldf<T>(x, (o * red + i) * inner + in));
    out[t] = op == RED_MEAN ? v / (float)red : v;
  }
}
// Two-stage full reduction: stage 1 writes one partial per CTA into scratch.
template <typename T>
__global__ void reduce_all_partial_kernel(const T* __restrict__ x, long long n, float* partial, int op) {
  __shared__ float sh[32];
  float v = red_identity(op);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    v = red_combine(op, v, ldf<T>(x, i));
  v = block_reduce(op, v, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = v;
}
__global__ void reduce_all_final_kernel(const float* partial, int nparts, float* out, int op,
                                        long long n) {
  __shared__ float sh[32];
  float v = red_identity(op);
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) v = red_combine(op, v, partial[i]);
  v = block_reduce(op, v, sh);
  if (threadIdx.x == 0) out[0] = op == RED_MEAN ? v / (float)n : v;
}

// Column sums of a bf16 matrix [M, N] (leading dimension ld) into fp32 [N]:
// the bias gradient of a linear layer.  grid.x covers 64-column strips,
// grid.y splits M; partial[grid.y][N] is reduced by a second kernel.
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long M, int N, long long ld,
                      float* __restrict__ partial) {
  __shared__ float sh[4][64];
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int rlane = threadIdx.x >> 6;  // 0..3
  float s = 0.0f;
  if (c < N) {
    for (long long r = (long long)blockIdx.y * 4 + rlane; r < M; r += (long long)gridDim.y * 4)
      s += __bfloat162float(x[r * ld + c]);
  }
  sh[rlane][threadIdx.x & 63] = s;
  __syncthreads();
  if (rlane == 0 && c < N)
    partial[(long long)blockIdx.y * N + c] = sh[0][threadIdx.x] + sh[1][threadIdx.x] +
                                             sh[2][threadIdx.x] + sh[3][threadIdx.x];
}
// The same for rows whose columns come in aligned groups of eight: a thread owns one 16-byte
// column vector and every 8th row of the CTA's share, four loads in flight; a warp reads 512
// contiguous bytes of a row.  grid.x covers 256-column strips, grid.y splits M.
__global__ void __launch_bounds__(256)
colsum_partial_vec_kernel(const __nv_bfloat16* __restrict__ x, long long M, int N, long long ld,
                          float* __restrict__ partial) {
  __shared__ float sh[8][32][9];
  const int cx = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + cx) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  if (c < N) {
    const long long step = (long long)gridDim.y * 8;
    long long r = (long long)blockIdx.y * 8 + rl;
    const __nv_bfloat16* col = x + c;
    for (; r + 3 * step < M; r += 4 * step) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldg(reinterpret_cast<const uint4*>(col + (r + u * step) * ld));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float2 t;
        t = unpack_bf16x2(v[u].x); acc[0] += t.x; acc[1] += t.y;
        t = unpack_bf16x2(v[u].y); acc[2] += t.x; acc[3] += t.y;
        t = unpack_bf16x2(v[u].z); acc[4] += t.x; acc[5] += t.y;
        t = unpack_bf16x2(v[u].w); acc[6] += t.x; acc[7] += t.y;
      }
    }
    for (; r < M; r += step) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(col + r * ld));
      float2 t;
      t = unpack_bf16x2(v.x); acc[0] += t.x; acc[1] += t.y;
      t = unpack_bf16x2(v.y); acc[2] += t.x; acc[3] += t.y;
      t = unpack_bf16x2(v.z); acc[4] += t.x; acc[5] += t.y;
      t = unpack_bf16x2(v.w); acc[6] += t.x; acc[7] += t.y;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[rl][cx][j] = acc[j];
  __syncthreads();
  // 256 threads = 256 columns of the strip
  const int oc = blockIdx.x * 256 + threadIdx.x;
  if (oc < N) {
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += sh[w][threadIdx.x >> 3][threadIdx.x & 7];
    partial[(long long)blockIdx.y * N + oc] = a;
  }
}
// One CTA per 32 columns: 32 x 8 threads, each sums every 8th partial row.
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, int nparts, int N, float* __restrict__ out,
                    int accumulate) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.0f;
  if (c < N)
    for (int p = py; p < nparts; p += 8) s += partial[(long long)p * N + c];
  sh[py][cx] = s;
  __syncthreads();
  if (py == 0 && c < N) {
#pragma unroll
    for (int w = 1; w < 8; ++w) s += sh[w][cx];
    out[c] = accumulate ? out[c] + s : s;
  }
}

// ---- embedding ------------------------------------------------------------
// out[r, :] = wte[ids[r], :] (+ wpe[r % T, :] when wpe != null)
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe,
                                     __nv_bfloat16* __restrict__ out, long long rows, int D, int T,
                                     long long id_offset, long long vocab_local) {
  const int nvec = D >> 3;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long id = ids[r] - id_offset;
    const bool have = id >= 0 && id < vocab_local;
    const uint4* a = reinterpret_cast<const uint4*>(wte + (have ? id : 0) * D);
    const uint4* p = wpe ? reinterpret_cast<const uint4*>(wpe + (r % T) * D) : nullptr;
    uint4* o = reinterpret_cast<uint4*>(out + r * D);
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      uint4 u = have ? a[c] : make_uint4(0, 0, 0, 0);
      if (p) {
        uint4 w = p[c];
        float2 x, y;
        x = unpack_bf16x2(u.x); y = unpack_bf16x2(w.x); u.x = pack_bf16x2(x.x + y.x, x.y + y.y);
        x = unpack_bf16x2(u.y); y = unpack_bf16x2(w.y); u.y = pack_bf16x2(x.x + y.x, x.y + y.y);
        x = unpack_bf16x2(u.z); y = unpack_bf16x2(w.z); u.z = pack_bf16x2(x.x + y.x, x.y + y.y);
        x = unpack_bf16x2(u.w); y = unpack_bf16x2(w.w); u.w = pack_bf16x2(x.x + y.x, x.y + y.y);
      }
      o[c] = u;
    }
  }
}
// dwte[ids[r], :] += dout[r, :]; dwpe[r % T, :] += dout[r, :]   (fp32 grads, atomics)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dwte, float* __restrict__ dwpe,
                                     long long rows, int D, int T, long long id_offset,
                                     long long vocab_local) {
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long id = ids[r] - id_offset;
    const bool have = id >= 0 && id < vocab_local;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const float g = __bfloat162float(dout[r * D + c]);
      if (have && dwte) atomicAdd(dwte + id * D + c, g);
      if (dwpe) atomicAdd(dwpe + (r % T) * D + c, g);
    }
  }
}

// ---- dropout (counter-based RNG) --------------------------------------------
// y = x * keep / (1 - p) with keep decided by hash(seed, index); the backward
// pass calls the same kernel on dy with the same seed, so no mask is stored.
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* out, long long n, float p,
                               unsigned long long seed) {
  const float scale = 1.0f / (1.0f - p);
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const uint32_t h = mix32(seed * 0x100000001B3ull + (uint64_t)i);
    stf<T>(out, i, h >= thresh ? ldf<T>(x, i) * scale : 0.0f);
  }
}

// ---- SwiGLU: x = [rows, 2H] as (gate | value); y = silu(gate) * value ----------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int H) {
  const long long n = rows * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / H;
    const int c = (int)(i - r * H);
    const float g = ldf<T>(x, r * 2 * H + c), v = ldf<T>(x, r * 2 * H + H + c);
    stf<T>(y, i, silu_f(g) * v);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                  T* __restrict__ dx, long long rows, int H) {
  const long long n = rows * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / H;
    const int c = (int)(i - r * H);
    const float g = ldf<T>(x, r * 2 * H + c), v = ldf<T>(x, r * 2 * H + H + c);
    const float d = ldf<T>(dy, i);
    stf<T>(dx, r * 2 * H + c, d * v * dsilu_f(g));
    stf<T>(dx, r * 2 * H + H + c, d * silu_f(g));
  }
}

// ---- 2-D transpose (fp32 / bf16), tiled through shared memory ------------------
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
  __shared__ float tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = by + j, c = bx + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = ldf<T>(x, (long long)r * cols + c);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = bx + j, r = by + threadIdx.x;
    if (r < rows && c < cols) stf<T>(y, (long long)c * rows + r, tile[threadIdx.x][j]);
  }
}

// ---- BatchNorm-1D over [B, F], fp32 ----------------------------------------------
// One CTA per feature.  Biased batch variance; running = mom*running + (1-mom)*batch
// (the reference's convention, src/layers/activations.c:496-499).
__global__ void batchnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, float* __restrict__ y,
                                     float* running_mean, float* running_var,
                                     float* __restrict__ save_mean, float* __restrict__ save_rstd,
                                     int B, int F, float eps, float momentum, int training) {
  __shared__ float sh[32];
  const int f = blockIdx.x;
  float mean, var;
  if (training) {
    float s = 0.0f;
    for (int b = threadIdx.x; b < B; b += blockDim.x) s += x[(long long)b * F + f];
    mean = block_reduce(RED_SUM, s, sh) / B;
    float q = 0.0f;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
      float d = x[(long long)b * F + f] - mean;
      q += d * d;
    }
    var = block_reduce(RED_SUM, q, sh) / B;
    if (threadIdx.x == 0) {
      running_mean[f] = momentum * running_mean[f] + (1.0f - momentum) * mean;
      running_var[f] = momentum * running_var[f] + (1.0f - momentum) * var;
    }
  } else {
    mean = running_mean[f];
    var = running_var[f];
  }
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0 && save_mean) { save_mean[f] = mean; save_rstd[f] = rstd; }
  const float g = gamma ? gamma[f] : 1.0f, bt = beta ? beta[f] : 0.0f;
  for (int b = threadIdx.x; b < B; b += blockDim.x)
    y[(long long)b * F + f] = (x[(long long)b * F + f] - mean) * rstd * g + bt;
}
__global__ void batchnorm_bwd_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                     const float* __restrict__ gamma,
                                     const float* __restrict__ save_mean,
                                     const float* __restrict__ save_rstd, float* __restrict__ dx,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta, int B,
                                     int F) {
  __shared__ float sh[32];
  const int f = blockIdx.x;
  const float mean = save_mean[f], rstd = save_rstd[f], g = gamma ? gamma[f] : 1.0f;
  float s1 = 0.0f, s2 = 0.0f;
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const float d = dy[(long long)b * F + f];
    s1 += d;
    s2 += d * (x[(long long)b * F + f] - mean) * rstd;
  }
  s1 = block_reduce(RED_SUM, s1, sh);
  s2 = block_reduce(RED_SUM, s2, sh);
  if (threadIdx.x == 0) {
    if (dgamma) dgamma[f] += s2;
    if (dbeta) dbeta[f] += s1;
  }
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const float h = (x[(long long)b * F + f] - mean) * rstd;
    dx[(long long)b * F + f] = g * rstd * (dy[(long long)b * F + f] - s1 / B - h * s2 / B);
  }
}

// ---- im2col / col2im / max-pool (NCHW, square kernel) -----------------------------
// col: [N*OH*OW, C*KH*KW]
template <typename T>
__global__ void im2col_kernel(const T* __restrict__ x, T* __restrict__ col, int N, int C, int H,
                              int W, int K, int stride, int pad, int OH, int OW, long long ldcol) {
  const long long total = (long long)N * OH * OW * C * K * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int kw = r % K; r /= K;
    const int kh = r % K; r /= K;
    const int c = r % C; r /= C;
    const int ow = r % OW; r /= OW;
    const int oh = r % OH; r /= OH;
    const int n = (int)r;
    const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
    float v = 0.0f;
    if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = ldf<T>(x, (((long long)n * C + c) * H + ih) * W + iw);
    const long long row = ((long long)n * OH + oh) * OW + ow;
    stf<T>(col, row * ldcol + ((long long)c * K + kh) * K + kw, v);
  }
}
// dx (fp32, pre-zeroed) += scatter of dcol
template <typename T>
__global__ void col2im_kernel(const T* __restrict__ dcol, float* __restrict__ dx, int N, int C, int H,
                              int W, int K, int stride, int pad, int OH, int OW, long long ldcol) {
  const long long total = (long long)N * OH * OW * C * K * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int kw = r % K; r /= K;
    const int kh = r % K; r /= K;
    const int c = r % C; r /= C;
    const int ow = r % OW; r /= OW;
    const int oh = r % OH; r /= OH;
    const int n = (int)r;
    const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
    if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
      const long long row = ((long long)n * OH + oh) * OW + ow;
      atomicAdd(dx + (((long long)n * C + c) * H + ih) * W + iw,
                ldf<T>(dcol, row * ldcol + ((long long)c * K + kh) * K + kw));
    }
  }
}
__global__ void maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                   int* __restrict__ argmax, int N, int C, int H, int W, int K,
                                   int stride, int OH, int OW) {
  const long long total = (long long)N * C * OH * OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int ow = r % OW; r /= OW;
    const int oh = r % OH; r /= OH;
    const long long nc = r;
    float best = -INFINITY;
    int bi = 0;
    for (int kh = 0; kh < K; ++kh)
      for (int kw = 0; kw < K; ++kw) {
        const int ih = oh * stride + kh, iw = ow * stride + kw;
        if (ih < H && iw < W) {
          const float v = x[(nc * H + ih) * W + iw];
          if (v > best) { best = v; bi = ih * W + iw; }
        }
      }
    y[i] = best;
    if (argmax) argmax[i] = bi;
  }
}
__global__ void maxpool_bwd_kernel(const float* __restrict__ dy, const int* __restrict__ argmax,
                                   float* __restrict__ dx, int N, int C, int H, int W, int OH, int OW) {
  const long long total = (long long)N * C * OH * OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long nc = i / ((long long)OH * OW);
    atomicAdd(dx + nc * H * W + argmax[i], dy[i]);
  }
}

}  // namespace cgk

using namespace cgk;

static int ew_grid(long long n, int threads = 256) {
  int dev = 0;
  cudaGetDevice(&dev);
  long long want = (n + threads - 1) / threads;
  long long cap = (long long)sm_count(dev) * 16;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}
#define ST(s) ((cudaStream_t)(s))

// Broadcasting binary op.  shape: output shape (nd <= 8); sa / sb: element strides
// of the operands per output dimension (0 = broadcast).  nd = 0 means "all three
// are contiguous with n elements".
CGK_API int cgk_binary(int op, int dtype, const void* a, const void* b, void* out, long long n, int nd,
                       const int* shape, const long long* sa, const long long* sb, void* stream) {
  CGK_REQUIRE(a && b && out, "cgk_binary: null pointer");
  CGK_REQUIRE(nd >= 0 && nd <= 8 && op >= 0 && op <= BIN_MIN, "cgk_binary: bad nd/op");
  if (n == 0) return 0;
  if (nd == 0) {
    if (dtype == 0) binary_contig_kernel<float><<<ew_grid(n), 256, 0, ST(stream)>>>((const float*)a, (const float*)b, (float*)out, n, op);
    else binary_contig_kernel<__nv_bfloat16><<<ew_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n, op);
  } else {
    BcastDims d;
    d.nd = nd;
    for (int i = 0; i < 8; ++i) { d.shape[i] = i < nd ? shape[i] : 1; d.sa[i] = i < nd ? sa[i] : 0; d.sb[i] = i < nd ? sb[i] : 0; }
    if (dtype == 0) binary_bcast_kernel<float><<<ew_grid(n), 256, 0, ST(stream)>>>((const float*)a, (const float*)b, (float*)out, n, op, d);
    else binary_bcast_kernel<__nv_bfloat16><<<ew_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n, op, d);
  }
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_unary(int op, int dtype, const void* x, void* out, long long n, float s, void* stream) {
  CGK_REQUIRE(x && out, "cgk_unary: null pointer");
  if (n == 0) return 0;
  if (dtype == 0) unary_kernel<float><<<ew_grid(n), 256, 0, ST(stream)>>>((const float*)x, (float*)out, n, op, s);
  else unary_kernel<__nv_bfloat16><<<ew_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, op, s);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_unary_backward(int op, int dtype, const void* x, const void* dy, void* dx, long long n,
                               float s, void* stream) {
  CGK_REQUIRE(x && dy && dx, "cgk_unary_backward: null pointer");
  if (n == 0) return 0;
  if (dtype == 0) unary_bwd_kernel<float><<<ew_grid(n), 256, 0, ST(stream)>>>((const float*)x, (const float*)dy, (float*)dx, n, op, s);
  else unary_bwd_kernel<__nv_bfloat16><<<ew_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, n, op, s);
  CGK_LAUNCH_CHECK();
  return 0;
}

// to_bf16 = 1: fp32 -> bf16, 0: bf16 -> fp32
CGK_API int cgk_cast(const void* x, void* out, long long n, int to_bf16, void* stream) {
  CGK_REQUIRE(x && out, "cgk_cast: null pointer");
  if (n == 0) return 0;
  if (to_bf16) cast_kernel<float, __nv_bfloat16><<<ew_grid(n), 256, 0, ST(stream)>>>((const float*)x, (__nv_bfloat16*)out, n);
  else cast_kernel<__nv_bfloat16, float><<<ew_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (float*)out, n);
  CGK_LAUNCH_CHECK();
  return 0;
}

// hi[i] = bf16(x[i]), lo[i] = bf16(x[i] - hi[i])
CGK_API int cgk_split_bf16(const float* x, void* hi, void* lo, long long n, void* stream) {
  CGK_REQUIRE(x && hi && lo, "cgk_split_bf16: null pointer");
  if (n == 0) return 0;
  split_bf16_kernel<<<ew_grid(n), 256, 0, ST(stream)>>>(x, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n);
  CGK_LAUNCH_CHECK();
  return 0;
}

// x viewed as [outer, red, inner] -> out fp32 [outer, inner].
CGK_API int cgk_reduce_axis(int op, int dtype, const void* x, float* out, long long outer, long long red,
                            long long inner, void* stream) {
  CGK_REQUIRE(x && out && red > 0, "cgk_reduce_axis: bad argument");
  if (outer * inner == 0) return 0;
  if (inner == 1) {
    int grid = (int)(outer < 4096 ? outer : 4096);
    if (dtype == 0) reduce_rows_kernel<float><<<grid, 256, 0, ST(stream)>>>((const float*)x, out, outer, red, op);
    else reduce_rows_kernel<__nv_bfloat16><<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, out, outer, red, op);
  } else {
    if (dtype == 0) reduce_strided_kernel<float><<<ew_grid(outer * inner), 256, 0, ST(stream)>>>((const float*)x, out, outer, red, inner, op);
    else reduce_strided_kernel<__nv_bfloat16><<<ew_grid(outer * inner), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, out, outer, red, inner, op);
  }
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_reduce_all_scratch_elems(long long n) { return ew_grid(n); }

// Full reduction to out[0] (fp32).  scratch: cgk_reduce_all_scratch_elems(n) floats.
CGK_API int cgk_reduce_all(int op, int dtype, const void* x, long long n, float* out, float* scratch,
                           void* stream) {
  CGK_REQUIRE(x && out && scratch && n > 0, "cgk_reduce_all: bad argument");
  int grid = ew_grid(n);
  if (dtype == 0) reduce_all_partial_kernel<float><<<grid, 256, 0, ST(stream)>>>((const float*)x, n, scratch, op);
  else reduce_all_partial_kernel<__nv_bfloat16><<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, n, scratch, op);
  CGK_LAUNCH_CHECK();
  reduce_all_final_kernel<<<1, 256, 0, ST(stream)>>>(scratch, grid, out, op, n);
  CGK_LAUNCH_CHECK();
  return 0;
}

static int colsum_parts(long long M) {
  long long p = (M + 255) / 256;
  if (p > 256) p = 256;
  if (p < 1) p = 1;
  return (int)p;
}
CGK_API long long cgk_colsum_scratch_elems(long long M, int N) { return (long long)colsum_parts(M) * N; }

// out[n] (+)= sum_m x[m, n]; x bf16 [M, N] with leading dimension ld; out fp32.
CGK_API int cgk_colsum_bf16(const void* x, long long M, int N, long long ld, float* out, float* scratch,
                            int accumulate, void* stream) {
  CGK_REQUIRE(x && out && scratch, "cgk_colsum_bf16: null pointer");
  if (N == 0) return 0;
  const int parts = colsum_parts(M);
  if (N % 8 == 0 && ld % 8 == 0 && ((uintptr_t)x & 15u) == 0) {
    dim3 grid((N + 255) / 256, parts);
    colsum_partial_vec_kernel<<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, M, N, ld, scratch);
  } else {
    dim3 grid((N + 63) / 64, parts);
    colsum_partial_kernel<<<grid, 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, M, N, ld, scratch);
  }
  CGK_LAUNCH_CHECK();
  colsum_final_kernel<<<(N + 31) / 32, 256, 0, ST(stream)>>>(scratch, parts, N, out, accumulate);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_embedding_forward(const long long* ids, const void* wte, const void* wpe, void* out,
                                  long long rows, int D, int T, long long id_offset,
                                  long long vocab_local, void* stream) {
  CGK_REQUIRE(ids && wte && out && D % 8 == 0 && T > 0, "cgk_embedding_forward: bad argument");
  if (rows == 0) return 0;
  int grid = (int)(rows < 148 * 32 ? rows : 148 * 32);
  embedding_fwd_kernel<<<grid, 128, 0, ST(stream)>>>(ids, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe,
                                                     (__nv_bfloat16*)out, rows, D, T, id_offset, vocab_local);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_embedding_backward(const long long* ids, const void* dout, float* dwte, float* dwpe,
                                   long long rows, int D, int T, long long id_offset,
                                   long long vocab_local, void* stream) {
  CGK_REQUIRE(ids && dout && T > 0, "cgk_embedding_backward: bad argument");
  if (rows == 0) return 0;
  int grid = (int)(rows < 148 * 32 ? rows : 148 * 32);
  embedding_bwd_kernel<<<grid, 256, 0, ST(stream)>>>(ids, (const __nv_bfloat16*)dout, dwte, dwpe, rows, D, T,
                                                     id_offset, vocab_local);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_dropout(int dtype, const void* x, void* out, long long n, float p,
                        unsigned long long seed, void* stream) {
  CGK_REQUIRE(x && out && p >= 0.0f && p < 1.0f, "cgk_dropout: bad argument");
  if (n == 0) return 0;
  if (dtype == 0) dropout_kernel<float><<<ew_grid(n), 256, 0, ST(stream)>>>((const float*)x, (float*)out, n, p, seed);
  else dropout_kernel<__nv_bfloat16><<<ew_grid(n), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, p, seed);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_swiglu_forward(int dtype, const void* x, void* y, long long rows, int H, void* stream) {
  CGK_REQUIRE(x && y && H > 0, "cgk_swiglu_forward: bad argument");
  if (rows == 0) return 0;
  if (dtype == 0) swiglu_fwd_kernel<float><<<ew_grid(rows * H), 256, 0, ST(stream)>>>((const float*)x, (float*)y, rows, H);
  else swiglu_fwd_kernel<__nv_bfloat16><<<ew_grid(rows * H), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, H);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_swiglu_backward(int dtype, const void* x, const void* dy, void* dx, long long rows, int H,
                                void* stream) {
  CGK_REQUIRE(x && dy && dx && H > 0, "cgk_swiglu_backward: bad argument");
  if (rows == 0) return 0;
  if (dtype == 0) swiglu_bwd_kernel<float><<<ew_grid(rows * H), 256, 0, ST(stream)>>>((const float*)x, (const float*)dy, (float*)dx, rows, H);
  else swiglu_bwd_kernel<__nv_bfloat16><<<ew_grid(rows * H), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, rows, H);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_transpose2d(int dtype, const void* x, void* y, int rows, int cols, void* stream) {
  CGK_REQUIRE(x && y, "cgk_transpose2d: null pointer");
  if (rows == 0 || cols == 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (dtype == 0) transpose_kernel<float><<<grid, block, 0, ST(stream)>>>((const float*)x, (float*)y, rows, cols);
  else transpose_kernel<__nv_bfloat16><<<grid, block, 0, ST(stream)>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_batchnorm_forward(const float* x, const float* gamma, const float* beta, float* y,
                                  float* running_mean, float* running_var, float* save_mean,
                                  float* save_rstd, int B, int F, float eps, float momentum,
                                  int training, void* stream) {
  CGK_REQUIRE(x && y && running_mean && running_var, "cgk_batchnorm_forward: null pointer");
  if (B == 0 || F == 0) return 0;
  batchnorm_fwd_kernel<<<F, 256, 0, ST(stream)>>>(x, gamma, beta, y, running_mean, running_var, save_mean,
                                                  save_rstd, B, F, eps, momentum, training);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_batchnorm_backward(const float* x, const float* dy, const float* gamma,
                                   const float* save_mean, const float* save_rstd, float* dx,
                                   float* dgamma, float* dbeta, int B, int F, void* stream) {
  CGK_REQUIRE(x && dy && save_mean && save_rstd && dx, "cgk_batchnorm_backward: null pointer");
  if (B == 0 || F == 0) return 0;
  batchnorm_bwd_kernel<<<F, 256, 0, ST(stream)>>>(x, dy, gamma, save_mean, save_rstd, dx, dgamma, dbeta, B, F);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_API int cgk_im2col(int dtype, const void* x, void* col, int N, int C, int H, int W, int K, int stride,
                       int pad, int OH, int OW, long long ldcol, void* stream) {
  CGK_REQUIRE(x && col, "cgk_im2col: null pointer");
  long long total = (long long)N * OH * OW * C * K * K;
  if (total == 0) return 0;
  if (dtype == 0) im2col_kernel<float><<<ew_grid(total), 256, 0, ST(stream)>>>((const float*)x, (float*)col, N, C, H, W, K, stride, pad, OH, OW, ldcol);
  else im2col_kernel<__nv_bfloat16><<<ew_grid(total), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)col, N, C, H, W, K, stride, pad, OH, OW, ldcol);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_col2im(int dtype, const void* dcol, float* dx, int N, int C, int H, int W, int K, int stride,
                       int pad, int OH, int OW, long long ldcol, void* stream) {
  CGK_REQUIRE(dcol && dx, "cgk_col2im: null pointer");
  long long total = (long long)N * OH * OW * C * K * K;
  if (total == 0) return 0;
  if (dtype == 0) col2im_kernel<float><<<ew_grid(total), 256, 0, ST(stream)>>>((const float*)dcol, dx, N, C, H, W, K, stride, pad, OH, OW, ldcol);
  else col2im_kernel<__nv_bfloat16><<<ew_grid(total), 256, 0, ST(stream)>>>((const __nv_bfloat16*)dcol, dx, N, C, H, W, K, stride, pad, OH, OW, ldcol);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_maxpool_forward(const float* x, float* y, int* argmax, int N, int C, int H, int W, int K,
                                int stride, int OH, int OW, void* stream) {
  CGK_REQUIRE(x && y, "cgk_maxpool_forward: null pointer");
  long long total = (long long)N * C * OH * OW;
  if (total == 0) return 0;
  maxpool_fwd_kernel<<<ew_grid(total), 256, 0, ST(stream)>>>(x, y, argmax, N, C, H, W, K, stride, OH, OW);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_maxpool_backward(const float* dy, const int* argmax, float* dx, int N, int C, int H, int W,
                                 int OH, int OW, void* stream) {
  CGK_REQUIRE(dy && argmax && dx, "cgk_maxpool_backward: null pointer");
  long long total = (long long)N * C * OH * OW;
  if (total == 0) return 0;
  maxpool_bwd_kernel<<<ew_grid(total), 256, 0, ST(stream)>>>(dy, argmax, dx, N, C, H, W, OH, OW);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_BOUNDS_READER(elementwise)
