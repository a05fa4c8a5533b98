// Device helpers of the fused compute + collective kernels: whole-CTA copies from a
// peer GPU's memory into local memory with plain 16-byte loads (many in flight per
// thread, because a load over NVLink takes a microsecond or more to come back), and
// bounded waits on flags that another GPU writes.  No bulk / TMA load ever names
// peer memory here, and none carries a cluster-broadcast qualifier.
#pragma once
#include "../kernels/sm100.cuh"

namespace cgk {

// Cross-GPU waits get a longer budget than intra-kernel ones: a peer may be a whole
// kernel behind.
#ifndef CGK_PEER_WAIT_BUDGET_NS
#define CGK_PEER_WAIT_BUDGET_NS 10000000000ull
#endif

// 16-byte load that bypasses the L1 (the line belongs to another GPU or was written by
// other CTAs of this launch).
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Depth of the software pipeline of cta_copy: loads in flight per thread.
constexpr int COPY_UNROLL = 16;

// All threads of the CTA copy `bytes` (a multiple of 16; both pointers 16-byte aligned)
// from src (possibly a peer GPU's memory) to dst (local).  Each thread keeps COPY_UNROLL
// 16-byte loads in flight before it stores: 64 KiB per 256-thread CTA, which is what it
// takes to cover the NVLink round trip.  The stores are plain generic-proxy stores; the
// caller publishes them (barrier + release).
__device__ __forceinline__ void cta_copy(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                         long long bytes) {
  const long long nvec = bytes >> 4;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  const long long step = (long long)blockDim.x * COPY_UNROLL;
  for (long long v0 = threadIdx.x; v0 < nvec; v0 += step) {
    uint4 r[COPY_UNROLL];
    if (v0 + (long long)(COPY_UNROLL - 1) * blockDim.x < nvec) {
#pragma unroll
      for (int u = 0; u < COPY_UNROLL; ++u) r[u] = ld_cg_u4(s + v0 + (long long)u * blockDim.x);
#pragma unroll
      for (int u = 0; u < COPY_UNROLL; ++u) d[v0 + (long long)u * blockDim.x] = r[u];
    } else {
#pragma unroll
      for (int u = 0; u < COPY_UNROLL; ++u) {
        const long long v = v0 + (long long)u * blockDim.x;
        if (v < nvec) r[u] = ld_cg_u4(s + v);
      }
#pragma unroll
      for (int u = 0; u < COPY_UNROLL; ++u) {
        const long long v = v0 + (long long)u * blockDim.x;
        if (v < nvec) d[v] = r[u];
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// NVSwitch multicast ("multimem") accesses.  `mc` is an address inside a multicast
// mapping that every GPU of the group has bound its copy of a symmetric buffer to.
// A store is replicated by the switch into every GPU's copy (the writer's included);
// a load-reduce returns the sum of all copies, accumulated in fp32 inside the switch.
// These are ordinary memory instructions on a multicast address: nothing here is a TMA
// or bulk copy.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void multimem_st_u4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

// All threads of the CTA broadcast `bytes` (multiple of 16) from local src to the
// multicast address mc_dst: local loads (COPY_UNROLL in flight), multicast stores.
__device__ __forceinline__ void cta_multicast(const uint8_t* __restrict__ src, uint8_t* mc_dst,
                                              long long bytes) {
  const long long nvec = bytes >> 4;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(mc_dst);
  const long long step = (long long)blockDim.x * COPY_UNROLL;
  for (long long v0 = threadIdx.x; v0 < nvec; v0 += step) {
    uint4 r[COPY_UNROLL];
#pragma unroll
    for (int u = 0; u < COPY_UNROLL; ++u) {
      const long long v = v0 + (long long)u * blockDim.x;
      if (v < nvec) r[u] = ld_cg_u4(s + v);
    }
#pragma unroll
    for (int u = 0; u < COPY_UNROLL; ++u) {
      const long long v = v0 + (long long)u * blockDim.x;
      if (v < nvec) multimem_st_u4(d + v, r[u]);
    }
  }
}

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& u) {
  float2 f;
  f = unpack_bf16x2(u.x); acc[0] += f.x; acc[1] += f.y;
  f = unpack_bf16x2(u.y); acc[2] += f.x; acc[3] += f.y;
  f = unpack_bf16x2(u.z); acc[4] += f.x; acc[5] += f.y;
  f = unpack_bf16x2(u.w); acc[6] += f.x; acc[7] += f.y;
}

}  // namespace cgk
