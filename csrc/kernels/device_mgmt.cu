// Device management entry points of the kernel library: device discovery, memory,
// copies, streams and synchronisation.  The host runtime (libcogito.so) has no link-time
// dependency on CUDA; it opens this library at run time and reaches the CUDA runtime only
// through these functions, so that kernels and allocations share one runtime instance.
//
// Reference counterpart: the cudart branch of src/cuda/cg_cuda.c:186-376 (cudaMalloc,
// cudaMemcpy, cudaMemset, stream creation, device properties).
#include <string.h>

#include "host_common.h"

// Number of usable devices; 0 when the driver is absent or reports none (never an error).
CGK_API int cgk_dev_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// out[0..7] = {cc major, cc minor, SM count, max threads per block, warp size, reserved...};
// mem[0..2] = {total bytes, free bytes, shared memory per block (opt-in maximum)}.
CGK_API int cgk_dev_info(int device, int* out, unsigned long long* mem, char* name, int name_len) {
  CGK_REQUIRE(out && mem && name && name_len > 0, "cgk_dev_info: null pointer");
  cudaDeviceProp p;
  CGK_CUDA_CHECK(cudaGetDeviceProperties(&p, device));
  out[0] = p.major;
  out[1] = p.minor;
  out[2] = p.multiProcessorCount;
  out[3] = p.maxThreadsPerBlock;
  out[4] = p.warpSize;
  out[5] = out[6] = out[7] = 0;
  int prev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&prev));
  CGK_CUDA_CHECK(cudaSetDevice(device));
  size_t free_b = 0, total_b = 0;
  cudaError_t e = cudaMemGetInfo(&free_b, &total_b);
  cudaSetDevice(prev);
  CGK_CUDA_CHECK(e);
  mem[0] = total_b;
  mem[1] = free_b;
  mem[2] = p.sharedMemPerBlockOptin;
  strncpy(name, p.name, (size_t)name_len - 1);
  name[name_len - 1] = 0;
  return 0;
}

CGK_API int cgk_dev_set(int device) {
  CGK_CUDA_CHECK(cudaSetDevice(device));
  return 0;
}

CGK_API int cgk_dev_get(void) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  return d;
}

CGK_API int cgk_dev_malloc(void** out, unsigned long long bytes) {
  CGK_REQUIRE(out, "cgk_dev_malloc: null pointer");
  *out = nullptr;
  CGK_CUDA_CHECK(cudaMalloc(out, bytes ? bytes : 1));
  return 0;
}

CGK_API int cgk_dev_free(void* p) {
  if (p) CGK_CUDA_CHECK(cudaFree(p));
  return 0;
}

// Page-locked host memory (the source / target of asynchronous copies).
CGK_API int cgk_host_malloc(void** out, unsigned long long bytes) {
  CGK_REQUIRE(out, "cgk_host_malloc: null pointer");
  *out = nullptr;
  CGK_CUDA_CHECK(cudaMallocHost(out, bytes ? bytes : 1));
  return 0;
}

CGK_API int cgk_host_free(void* p) {
  if (p) CGK_CUDA_CHECK(cudaFreeHost(p));
  return 0;
}

// kind: 0 host->device, 1 device->host, 2 device->device.  async != 0 enqueues on `stream`
// and returns; otherwise the copy is complete on return.
CGK_API int cgk_dev_memcpy(void* dst, const void* src, unsigned long long bytes, int kind, void* stream, int async) {
  CGK_REQUIRE(kind >= 0 && kind <= 2, "cgk_dev_memcpy: kind %d", kind);
  if (bytes == 0) return 0;
  CGK_REQUIRE(dst && src, "cgk_dev_memcpy: null pointer");
  const cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  CGK_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, k, (cudaStream_t)stream));
  if (!async) CGK_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}

CGK_API int cgk_dev_memset(void* p, int value, unsigned long long bytes, void* stream) {
  if (bytes == 0) return 0;
  CGK_REQUIRE(p, "cgk_dev_memset: null pointer");
  CGK_CUDA_CHECK(cudaMemsetAsync(p, value, bytes, (cudaStream_t)stream));
  return 0;
}

CGK_API int cgk_stream_create(void** out) {
  CGK_REQUIRE(out, "cgk_stream_create: null pointer");
  cudaStream_t s = nullptr;
  CGK_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *out = (void*)s;
  return 0;
}

CGK_API int cgk_stream_destroy(void* s) {
  if (s) CGK_CUDA_CHECK(cudaStreamDestroy((cudaStream_t)s));
  return 0;
}

// stream == nullptr with whole_device != 0 waits for the whole device.
CGK_API int cgk_dev_sync(void* stream, int whole_device) {
  if (whole_device) CGK_CUDA_CHECK(cudaDeviceSynchronize());
  else CGK_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}
