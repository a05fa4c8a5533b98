// Rotary position embedding, rotate-half convention (element i pairs with
// i + D/2), applied in place to a strided bf16 or fp32 tensor [B, T, H, D].
// The backward pass is the same kernel with the sine negated.
//
// Reference counterparts: rope_kernel (src/cuda/flash_attn_kernels.c:216-249),
// the host backward (:656-682) and cg_rope_precompute_freqs
// (src/attention/flash_attn.c:318-362): cos/sin tables of shape [max_seq, D/2]
// with angle = pos * theta^(-2i/D).
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cgk {

__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int max_seq,
                                  int half, float theta) {
  const long long n = (long long)max_seq * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int pos = (int)(i / half), j = (int)(i % half);
    const float freq = powf(theta, -2.0f * (float)j / (float)(2 * half));
    float s, c;
    sincosf((float)pos * freq, &s, &c);
    cos_t[i] = c;
    sin_t[i] = s;
  }
}

template <typename T>
__device__ __forceinline__ float rd(const T* p);
template <> __device__ __forceinline__ float rd<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float rd<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void wr(T* p, float v);
template <> __device__ __forceinline__ void wr<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void wr<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// positions: int32 [B, T] or null (then position = pos_offset + t).
template <typename T>
__global__ void rope_apply_kernel(T* x, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ positions, int B, int Tn, int H, int D,
                                  long long bs, long long ts, long long hs, int pos_offset,
                                  int max_seq, float sign) {
  const int half = D / 2;
  const long long n = (long long)B * Tn * H * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    long long r = i / half;
    const int h = (int)(r % H); r /= H;
    const int t = (int)(r % Tn);
    const int b = (int)(r / Tn);
    int pos = positions ? positions[(long long)b * Tn + t] : pos_offset + t;
    if (pos < 0) pos = 0;
    if (pos >= max_seq) pos = max_seq - 1;
    const float c = cos_t[(long long)pos * half + j], s = sign * sin_t[(long long)pos * half + j];
    T* p = x + b * bs + t * ts + h * hs;
    const float a = rd<T>(p + j), bb = rd<T>(p + j + half);
    wr<T>(p + j, a * c - bb * s);
    wr<T>(p + j + half, bb * c + a * s);
  }
}

}  // namespace cgk

using namespace cgk;

CGK_API int cgk_rope_table(float* cos_t, float* sin_t, int max_seq, int head_dim, float theta,
                           void* stream) {
  CGK_REQUIRE(cos_t && sin_t && head_dim % 2 == 0 && max_seq > 0, "cgk_rope_table: bad argument");
  const long long n = (long long)max_seq * (head_dim / 2);
  int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  rope_table_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(cos_t, sin_t, max_seq, head_dim / 2, theta);
  CGK_LAUNCH_CHECK();
  return 0;
}

// dtype 0 = fp32, 1 = bf16.  backward != 0 applies the inverse rotation.
CGK_API int cgk_rope_apply(int dtype, void* x, const float* cos_t, const float* sin_t,
                           const int* positions, int B, int T, int H, int D, long long bs,
                           long long ts, long long hs, int pos_offset, int max_seq, int backward,
                           void* stream) {
  CGK_REQUIRE(x && cos_t && sin_t && D % 2 == 0, "cgk_rope_apply: bad argument");
  const long long n = (long long)B * T * H * (D / 2);
  if (n == 0) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  long long blocks = (n + 255) / 256, cap = (long long)sm_count(dev) * 16;
  if (blocks > cap) blocks = cap;
  const float sign = backward ? -1.0f : 1.0f;
  if (dtype == 0)
    rope_apply_kernel<float><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
        (float*)x, cos_t, sin_t, positions, B, T, H, D, bs, ts, hs, pos_offset, max_seq, sign);
  else
    rope_apply_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)x, cos_t, sin_t, positions, B, T, H, D, bs, ts, hs, pos_offset, max_seq, sign);
  CGK_LAUNCH_CHECK();
  return 0;
}
