// Device helpers of the fused compute + collective kernels: untiled bulk copies
// (never the cluster-broadcast form), a one-thread relay that moves a byte range from
// a peer GPU into local memory through a shared-memory ring, and bounded waits on
// flags that another GPU writes.
#pragma once
#include "../kernels/sm100.cuh"

namespace cgk {

// Cross-GPU waits get a longer budget than intra-kernel ones: a peer may be a whole
// kernel behind.
#ifndef CGK_PEER_WAIT_BUDGET_NS
#define CGK_PEER_WAIT_BUDGET_NS 10000000000ull
#endif

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}

// Relay state of one thread: a ring of RELAY_STAGES pieces in shared memory.
constexpr int RELAY_STAGES = 8;
constexpr uint32_t RELAY_PIECE = 16384;

struct Relay {
  uint32_t smem;      // ring base (RELAY_STAGES * RELAY_PIECE bytes, 128-byte aligned)
  uint32_t bars;      // RELAY_STAGES mbarriers
  uint32_t count;     // pieces issued so far
};

__device__ __forceinline__ void relay_init(Relay& r, uint32_t smem, uint32_t bars) {
  r.smem = smem;
  r.bars = bars;
  r.count = 0;
  for (int s = 0; s < RELAY_STAGES; ++s) mbar_init(bars + 8u * s, 1);
  mbar_fence_init();
}

// Copies `bytes` (a multiple of 16) from src (possibly peer memory) to dst (local).
// Returns false if a wait ran out.  All copies have completed when it returns.
__device__ __forceinline__ bool relay_copy(Relay& r, const uint8_t* src, uint8_t* dst,
                                           long long bytes, volatile int* dead, int* status) {
  const long long pieces = (bytes + RELAY_PIECE - 1) / RELAY_PIECE;
  // Software pipeline: loads run up to RELAY_AHEAD pieces ahead of the stores.  Piece
  // idx reuses the stage of piece idx - RELAY_STAGES, whose store must have finished
  // reading shared memory; since at least idx - RELAY_AHEAD + 1 stores are committed
  // when piece idx is loaded, "at most RELAY_STAGES - RELAY_AHEAD stores still
  // reading" implies that.
  constexpr int RELAY_AHEAD = 6;
  long long issued = 0, stored = 0;
  const uint32_t base = r.count;
  while (stored < pieces) {
    while (issued < pieces && issued - stored < RELAY_AHEAD) {
      const uint32_t idx = base + (uint32_t)issued;
      const int s = idx % RELAY_STAGES;
      if (idx >= (uint32_t)RELAY_STAGES) tma_store_wait_read<RELAY_STAGES - RELAY_AHEAD>();
      const long long o = issued * RELAY_PIECE;
      const uint32_t n = (uint32_t)((bytes - o) < (long long)RELAY_PIECE ? (bytes - o) : RELAY_PIECE);
      mbar_expect_tx(r.bars + 8u * s, n);
      bulk_load(r.smem + s * RELAY_PIECE, src + o, n, r.bars + 8u * s);
      ++issued;
    }
    const uint32_t idx = base + (uint32_t)stored;
    const int s = idx % RELAY_STAGES;
    if (!mbar_wait(r.bars + 8u * s, (idx / RELAY_STAGES) & 1u, dead, status, 3100)) return false;
    const long long o = stored * RELAY_PIECE;
    const uint32_t n = (uint32_t)((bytes - o) < (long long)RELAY_PIECE ? (bytes - o) : RELAY_PIECE);
    bulk_store(dst + o, r.smem + s * RELAY_PIECE, n);
    tma_store_commit();
    ++stored;
  }
  r.count = base + (uint32_t)pieces;
  tma_store_wait_all<0>();
  return true;
}

}  // namespace cgk
