// How fast can an SM stream its own contiguous slab of HBM into shared memory / registers?
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -Iinclude -Icsrc/kernels benchmarks/stream_probe.cu csrc/kernels/host_common.cu -o stream_probe
//   ./stream_probe
//
// Every CTA streams 32 steps of 8704 bytes (the step of the INT4 weight stream) through a ring of
// `stages` slots; a consumer thread frees each slot as soon as it is full.  Modes:
//   0  one thread issues 1-D bulk copies          1  `lanes` threads of one warp issue them (slot bound to lane)
//   2  one thread issues tiled 2-D TMA copies     3  `lanes` threads of one warp issue them
//   5  `lanes` warps issue tiled TMA copies (one thread each)
//   4  no ring: 512 threads load 16 bytes each, four requests in flight per thread, and discard
// The table printed gives microseconds, aggregate GB/s and GB/s per SM for grids of 1, 148 (one CTA
// per SM) and 592 CTAs; successive launches read different slabs of a 165 MB buffer, so nothing
// comes from L2.  Result on B200 (see profiles/hbm_streaming_per_sm.md): a copy-engine ring delivers
// 17-30 GB/s per SM whatever its depth and however many threads issue; plain loads reach 36 GB/s per
// SM with this little in flight.  Streaming kernels in this library therefore load with ld.global.
#include <cstdio>
#include <cstdlib>
#include <cuda.h>
#include "host_common.h"
#include "sm100.cuh"
using namespace cgk;

__device__ __forceinline__ void bulk1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(512, 1)
stream_kernel(const __grid_constant__ CUtensorMap tm, const uint8_t* base, int steps, int stages, int lanes, int mode, uint32_t step_bytes, unsigned long long* sink, int* status, int cta_off) {
  const int cta = blockIdx.x + cta_off;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = (smem_u32(smem) + 1023u) & ~1023u;
  const uint32_t bars = sb, ring = sb + 1024;
  __shared__ int dead_s;
  volatile int* dead = &dead_s;
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (32 + s); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < 32; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    dead_s = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const uint8_t* src = base + (size_t)cta * steps * step_bytes;
  if (mode == 4) {
    uint4 acc = make_uint4(0, 0, 0, 0);
    const uint4* p = reinterpret_cast<const uint4*>(src);
    const size_t n = (size_t)steps * step_bytes / 16;
    for (size_t i = threadIdx.x; i < n; i += 512 * 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = (i + u * 512 < n) ? __ldcs(p + i + u * 512) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 4; ++u) { acc.x ^= v[u].x; acc.y ^= v[u].y; acc.z ^= v[u].z; acc.w ^= v[u].w; }
    }
    if ((acc.x ^ acc.y ^ acc.z ^ acc.w) == 0x12345678u) sink[0] = 1;
    return;
  }
  if (warp == 0 && mode < 4) {
    const int L = (mode == 0 || mode == 2) ? 1 : lanes;
    if (lane < L) {
      for (int i = 0; i < steps; ++i) {
        const int r = i % stages;
        if (r % L != lane) continue;
        if (!mbar_wait_backoff(empty(r), ((i / stages) & 1) ^ 1, dead, status, 1, 50)) break;
        mbar_expect_tx(full(r), step_bytes);
        if (mode <= 1) bulk1d(ring + r * step_bytes, src + (size_t)i * step_bytes, step_bytes, full(r));
        else tma_load_2d(ring + r * step_bytes, &tm, full(r), 0, (int)((size_t)cta * steps + i) * (int)(step_bytes / 128));
      }
    }
  }
  if (mode == 5 && warp < lanes && lane == 0) {          // producer warps: warp w owns slots r % lanes == w
    for (int i = 0; i < steps; ++i) {
      const int r = i % stages;
      if (r % lanes != warp) continue;
      if (!mbar_wait_backoff(empty(r), ((i / stages) & 1) ^ 1, dead, status, 1, 50)) break;
      mbar_expect_tx(full(r), step_bytes);
      tma_load_2d(ring + r * step_bytes, &tm, full(r), 0, (int)((size_t)cta * steps + i) * (int)(step_bytes / 128));
    }
  }
  if (warp == 15 && lane == 0) {
    for (int i = 0; i < steps; ++i) {
      const int r = i % stages;
      if (!mbar_wait(full(r), (i / stages) & 1, dead, status, 2)) break;
      mbar_arrive(empty(r));
    }
  }
}

int main(int argc, char** argv) {
  const int steps = 32, ctas = 148 * 4;
  const uint32_t step_bytes = 8704;
  const size_t total = (size_t)ctas * steps * step_bytes;      // 165 MB > L2
  uint8_t* buf; cudaMalloc(&buf, total); cudaMemset(buf, 1, total);
  unsigned long long* sink; cudaMalloc(&sink, 8);
  int* status; cudaMalloc(&status, 16); cudaMemset(status, 0, 16);
  CUtensorMap tm;
  const uint64_t dims[2] = {128, total / 128}, strides[1] = {128};
  const uint32_t box[2] = {128, step_bytes / 128};
  if (encode_tmap(&tm, buf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box, Swz::None)) { printf("tmap failed: %s\n", last_error()); return 1; }
  const int smem = 1024 + 1024 + 20 * step_bytes + 1024;
  cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
  struct Cfg { int mode, stages, lanes, grid; } cfgs[] = {
    {5, 16, 1, 1}, {5, 16, 2, 1}, {5, 16, 4, 1}, {5, 16, 8, 1}, {5, 16, 1, 148}, {5, 16, 2, 148}, {5, 16, 4, 148}, {5, 16, 8, 148}, {5, 16, 8, 592},
    {0, 16, 1, 148}, {1, 16, 8, 148}, {1, 16, 16, 148}, {2, 16, 1, 148}, {3, 16, 8, 148}, {3, 16, 16, 148}, {2, 4, 1, 148}, {2, 8, 1, 148}, {4, 0, 0, 148},
    {1, 16, 16, 592}, {3, 16, 16, 592}, {2, 16, 1, 592}, {4, 0, 0, 592}, {2, 16, 1, 1}, {3, 16, 16, 1}, {1, 16, 16, 1}};
  for (auto c : cfgs) {
    float best = 1e9;
    for (int it = 0; it < 4; ++it) {
      cudaEventRecord(a);
      stream_kernel<<<c.grid, 512, smem>>>(tm, buf, steps, c.stages ? c.stages : 1, c.lanes, c.mode, step_bytes, sink, status, (it * c.grid) % ctas);
      cudaEventRecord(b); cudaEventSynchronize(b);
      float ms; cudaEventElapsedTime(&ms, a, b); if (ms < best) best = ms;
    }
    const double bytes = (double)c.grid * steps * step_bytes;
    int st[4]; cudaMemcpy(st, status, 16, cudaMemcpyDeviceToHost);
    printf("mode %d stages %2d lanes %2d grid %3d: %8.1f us  %7.1f GB/s total  %6.1f GB/s per SM-slot  status %d err %s\n", c.mode, c.stages, c.lanes, c.grid, best * 1e3,
           bytes / best / 1e6, bytes / best / 1e6 / (c.grid < 148 ? c.grid : 148), st[0], cudaGetErrorString(cudaGetLastError()));
  }
  return 0;
}
