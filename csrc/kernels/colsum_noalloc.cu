// Column sums without any allocation: see include/cogito_noalloc.h for who needs this.
//
// The partial sums that cgk_colsum_bf16 keeps in caller-provided scratch live here
// in a fixed array in device memory that is part of the library image.  Host code
// cannot use the array's name as an address (on the host the name is only a
// stand-in for the symbol), so the address is looked up once per device with
// cudaGetSymbolAddress and that pointer is what the kernels receive.
#include "../../include/cogito_noalloc.h"

#include <mutex>

#include "host_common.h"
#include "sm100.cuh"

namespace cgk {

constexpr int NA_MAX_COLS = CGK_COLSUM_NOALLOC_MAX_COLS;
constexpr int NA_MAX_PARTS = 64;

// 64 x 16384 floats = 4 MiB, resident on every GPU that loads the library.
static __device__ __align__(256) float g_colsum_scratch[NA_MAX_PARTS * NA_MAX_COLS];

// One CTA column strip of 64 columns; blockIdx.y walks the rows with stride
// gridDim.y * 4.  Every (part, column < N) slot is written, so stale contents of
// the shared array never reach the result.
__global__ void __launch_bounds__(256)
colsum_na_partial_kernel(const __nv_bfloat16* __restrict__ x, long long M, int N, long long ld,
                         float* __restrict__ partial) {
  __shared__ float sh[4][64];
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int rlane = threadIdx.x >> 6;
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

__global__ void colsum_na_final_kernel(const float* __restrict__ partial, int nparts, int N,
                                       float* __restrict__ out, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.0f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * N + c];
  out[c] = accumulate ? out[c] + s : s;
}

static std::mutex g_na_mu;
static float* g_na_ptr[64] = {nullptr};

// Device address of the scratch array on the current device (looked up on first use).
static int scratch_address(float** out) {
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  CGK_REQUIRE(dev >= 0 && dev < 64, "cgk_colsum_bf16_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_na_mu);
  if (g_na_ptr[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_colsum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("cgk_colsum_bf16_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(e));
      return CGK_E_CUDA;
    }
    g_na_ptr[dev] = p;
  }
  *out = g_na_ptr[dev];
  return 0;
}

}  // namespace cgk

using namespace cgk;

CGK_API int cgk_colsum_bf16_noalloc(const void* x, long long M, int N, long long ld, float* out,
                                    int accumulate, void* stream) {
  CGK_REQUIRE(x && out, "cgk_colsum_bf16_noalloc: null pointer");
  CGK_REQUIRE(M >= 0 && N >= 0 && ld >= N, "cgk_colsum_bf16_noalloc: bad shape M=%lld N=%d ld=%lld", M, N, ld);
  if (N > NA_MAX_COLS) {
    set_error("cgk_colsum_bf16_noalloc: N=%d exceeds the built-in scratch (at most %d columns); "
              "use cgk_colsum_bf16 with caller-provided scratch",
              N, NA_MAX_COLS);
    return CGK_E_LIMIT;
  }
  if (N == 0) return 0;
  float* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc) return rc;
  long long parts = (M + 255) / 256;
  if (parts > NA_MAX_PARTS) parts = NA_MAX_PARTS;
  if (parts < 1) parts = 1;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((N + 63) / 64, (unsigned)parts);
  colsum_na_partial_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, M, N, ld, scratch);
  CGK_LAUNCH_CHECK();
  colsum_na_final_kernel<<<(N + 255) / 256, 256, 0, st>>>(scratch, (int)parts, N, out, accumulate);
  CGK_LAUNCH_CHECK();
  return 0;
}
