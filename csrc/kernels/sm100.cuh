// Blackwell (sm_100a) device primitives shared by every tensor-core kernel in
// this library: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 MMA / TMEM, and
// the shared-memory / instruction descriptor encodings.
//
// Every wait in this file is bounded.  A wait that runs out sets a CTA-local
// "dead" word and a global status word, after which all later waits return at
// once, so a protocol bug ends the kernel with an error code instead of a hang.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cgk {

// ---------------------------------------------------------------------------
// status reporting
// ---------------------------------------------------------------------------
// One int4 in global memory per library instance: {code, where, block, aux}.
// code 0 = fine.  The host reads it after a launch when asked to check.
enum : int {
  KST_OK = 0,
  KST_MBAR_TIMEOUT = 1,   // an mbarrier wait ran out
  KST_FLAG_TIMEOUT = 2,   // a wait on a global-memory flag ran out
  KST_BAD_ARG = 3,
  KST_BOUNDS = 4,         // debug build: an index outside its range (where = source line)
};

__device__ __forceinline__ void report_status(int* status, int code, int where, int aux) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = where;
    status[2] = (int)blockIdx.x;
    status[3] = aux;
    __threadfence_system();
  }
}

// ---------------------------------------------------------------------------
// Index checks of the debug build (python -m cogito_b200.build --debug-bounds, which compiles every
// kernel with -DCGK_DEBUG_BOUNDS into libcogito_kernels_dbg.so).  CGK_IDX(i, n) yields i; in the
// debug build an i outside [0, n) is recorded once per source file (code KST_BOUNDS, source line,
// index, limit) and replaced by 0, so the access that follows stays inside the array: the kernel
// never traps and the test that ran it fails on the recorded word instead
// (cgk_bounds_read_<file>, read by cogito_b200.ops._lib.assert_device_ok).
// ---------------------------------------------------------------------------
#ifdef CGK_DEBUG_BOUNDS
static __device__ int cgk_bounds_word[4];
__device__ __forceinline__ long long cgk_checked_index(long long i, long long n, int line) {
  if (i >= 0 && i < n) return i;
  if (atomicCAS(&cgk_bounds_word[0], 0, (int)KST_BOUNDS) == 0) {
    cgk_bounds_word[1] = line;
    cgk_bounds_word[2] = (int)i;
    cgk_bounds_word[3] = (int)n;
  }
  return 0;
}
#define CGK_IDX(i, n) cgk_checked_index((long long)(i), (long long)(n), __LINE__)
#define CGK_BOUNDS_READER(name)                                                               \
  extern "C" __attribute__((visibility("default"))) int cgk_bounds_read_##name(int* out, int reset) { \
    int z[4] = {0, 0, 0, 0};                                                                  \
    if (cudaMemcpyFromSymbol(out, cgk::cgk_bounds_word, sizeof(z)) != cudaSuccess) return -2; \
    if (reset && cudaMemcpyToSymbol(cgk::cgk_bounds_word, z, sizeof(z)) != cudaSuccess) return -2; \
    return 0;                                                                                 \
  }
#else
#define CGK_IDX(i, n) (i)
#define CGK_BOUNDS_READER(name)
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Budget for any single wait.  Long enough for a kernel that is queued behind a
// slow peer, short enough that a broken protocol ends well inside a test's
// limit.
#ifndef CGK_WAIT_BUDGET_NS
#define CGK_WAIT_BUDGET_NS 2000000000ull
#endif
#ifndef CGK_WAIT_MAX_ITERS
#define CGK_WAIT_MAX_ITERS (1u << 30)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One arrival per warp (the barrier counts warps, not threads): an arrival is an atomic on one
// shared-memory word, and 128 or 256 of them per tile and barrier serialise.  Every lane must have
// issued its own fences (proxy, tcgen05) before the call; the warp barrier orders the lanes'
// earlier accesses before lane 0's releasing arrival.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  __syncwarp();
  if ((threadIdx.x & 31u) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

__device__ __forceinline__ uint32_t mbar_try_wait_suspend(uint32_t bar, uint32_t parity,
                                                          uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok;
}

// Untiled bulk copy global -> shared, completing on an mbarrier.  Both addresses 16-byte aligned,
// `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Bounded wait.  `dead` is a word in shared memory that every role of the CTA
// polls; `status` is the global status word (may be null).  Returns false when
// the wait gave up (now or earlier).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* dead,
                                          int* status, int where) {
  // Plain try_wait: it already blocks for a short, hardware-chosen time.  The clock is not
  // read before 256 polls have failed: a %globaltimer read costs about as much as a short
  // pipeline step, and most waits end within a few polls.
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < CGK_WAIT_MAX_ITERS; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (*dead) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > CGK_WAIT_BUDGET_NS) break;
    }
  }
  *dead = 1;
  report_status(status, KST_MBAR_TIMEOUT, where, (int)parity);
  return false;
}

// The same wait for roles with slack (producers ahead of a deep ring, helper warps): sleeps
// `sleep_ns` after every failed poll.  A poll is a shared-memory access; a dozen threads polling
// in a tight loop take a large share of the SM's shared-memory issue slots from the warps that
// do the work (measured: a streaming kernel ran 2-3x slower per step with 20 tight pollers).
__device__ __forceinline__ bool mbar_wait_backoff(uint32_t bar, uint32_t parity, volatile int* dead,
                                                  int* status, int where, uint32_t sleep_ns) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < CGK_WAIT_MAX_ITERS; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(sleep_ns);
    if ((it & 63u) == 63u) {
      if (*dead) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > CGK_WAIT_BUDGET_NS) break;
    }
  }
  *dead = 1;
  report_status(status, KST_MBAR_TIMEOUT, where, (int)parity);
  return false;
}

// ---------------------------------------------------------------------------
// global-memory flags (same-GPU or peer), bounded
// ---------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(int* p, int v) {
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait until *flag >= want (system scope).  Returns false on timeout.
__device__ __forceinline__ bool flag_wait_ge_sys(const int* flag, int want, int* status, int where,
                                                 uint64_t budget_ns = CGK_WAIT_BUDGET_NS) {
  uint64_t t0 = 0;                                   // read lazily: see mbar_wait
  for (uint32_t it = 0; it < CGK_WAIT_MAX_ITERS; ++it) {
    if (ld_acquire_sys(flag) >= want) return true;
    if ((it & 31u) == 31u) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) break;
      __nanosleep(64);
    }
  }
  report_status(status, KST_FLAG_TIMEOUT, where, want);
  return false;
}
// The same wait for a role of a CTA whose other roles must learn that it gave up.
__device__ __forceinline__ bool flag_wait_ge_sys_cta(const int* flag, int want, volatile int* dead,
                                                     int* status, int where) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < CGK_WAIT_MAX_ITERS; ++it) {
    if (ld_acquire_sys(flag) >= want) return true;
    if ((it & 31u) == 31u) {
      if (dead && *dead) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > CGK_WAIT_BUDGET_NS) break;
      __nanosleep(32);
    }
  }
  if (dead) *dead = 1;
  report_status(status, KST_FLAG_TIMEOUT, where, want);
  return false;
}
__device__ __forceinline__ bool flag_wait_ge_gpu(const int* flag, int want, volatile int* dead,
                                                 int* status, int where) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < CGK_WAIT_MAX_ITERS; ++it) {
    if (ld_acquire_gpu(flag) >= want) return true;
    if ((it & 31u) == 31u) {
      if (dead && *dead) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > CGK_WAIT_BUDGET_NS) break;
      __nanosleep(32);
    }
  }
  if (dead) *dead = 1;
  report_status(status, KST_FLAG_TIMEOUT, where, want);
  return false;
}

// ---------------------------------------------------------------------------
// proxies and fences
// ---------------------------------------------------------------------------
// Generic-proxy writes to shared memory become visible to the async proxy
// (TMA, tcgen05.mma operand fetch).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA (tiled; every load of this library targets the issuing CTA's own shared memory)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(m), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(m), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// Bulk tensor reduction shared -> global: global[tile] += shared[tile] (element type
// and operation width come from the tensor map; out-of-range parts are clipped).
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, uint32_t src, int x, int y,
                                                  int z) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(m), "r"(src), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// TMEM
// ---------------------------------------------------------------------------
// Whole-warp call.  ncols: power of two in [32, 512].  The base address lands in
// the shared-memory word `dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate.  One thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same, with the A operand read from TMEM (used for P·V style products).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once all MMAs issued so far by this thread are done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// TMEM -> registers: each thread of the warp reads its own lane (row), N
// consecutive 32-bit columns.  The warp may only touch lanes
// 32*(warp_id % 4) .. +31, which the caller encodes in taddr[31:16].
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// registers -> TMEM, same shape as tmem_ld32.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose
// rows are 128 bytes (64 bf16) wide, stored as 8-row x 128 B atoms (1 KiB).
//   K-major operand  (rows = M/N index, 128 B of K per row):
//       stride-dim offset  = 1024 B (next group of 8 rows); leading offset unused.
//   MN-major operand (rows = K index, 128 B of M/N per row; 64-wide M/N blocks
//       placed `mn_block_bytes` apart):
//       stride-dim offset  = 1024 B (next group of 8 K rows),
//       leading-dim offset = mn_block_bytes (next block of 64 M/N elements).
// Bits: [0,14) addr>>4, [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version=1,
//       [61,64) layout (2 = 128B swizzle).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulate.
// a_mn / b_mn: 0 = K-major operand, 1 = MN-major operand.
__host__ __device__ __forceinline__ uint32_t make_idesc_bf16(int m, int n, int a_mn, int b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                      // D format: fp32
  d |= 1u << 7;                      // A format: bf16
  d |= 1u << 10;                     // B format: bf16
  d |= (uint32_t)(a_mn & 1) << 15;   // A major
  d |= (uint32_t)(b_mn & 1) << 16;   // B major
  d |= (uint32_t)(n >> 3) << 17;     // N / 8
  d |= (uint32_t)(m >> 4) << 24;     // M / 16
  return d;
}
// fp16 variant (A/B format 0).
__host__ __device__ __forceinline__ uint32_t make_idesc_f16(int m, int n, int a_mn, int b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;
  d |= (uint32_t)(a_mn & 1) << 15;
  d |= (uint32_t)(b_mn & 1) << 16;
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(m >> 4) << 24;
  return d;
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a
// 128-byte-swizzled tile with 128-byte rows (the layout TMA writes and
// tcgen05.mma reads).  `row` counts from the 1 KiB-aligned tile base.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

// ---------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------
// Hardware tanh (one MUFU instruction, relative error about 2^-11: below bf16 resolution).
// tanhf() costs tens of instructions with a divergent slow path, which made the GELU
// epilogue of a 128 x 256 tile several times longer than the tile's MMAs.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  float u = c * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanh_fast(u));
}
__device__ __forceinline__ float dgelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  float x2 = x * x;
  float u = c * (x + 0.044715f * x * x2);
  float t = tanh_fast(u);
  float du = c * (1.0f + 3.0f * 0.044715f * x2);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}
// Full-precision forms for the fp32 elementwise kernels (memory-bound: tanhf costs nothing there).
__device__ __forceinline__ float gelu_tanh_precise(float x) {
  const float c = 0.7978845608028654f;
  float u = c * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float dgelu_tanh_precise(float x) {
  const float c = 0.7978845608028654f;
  float x2 = x * x;
  float u = c * (x + 0.044715f * x * x2);
  float t = tanhf(u);
  float du = c * (1.0f + 3.0f * 0.044715f * x2);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
  float s = 1.0f / (1.0f + __expf(-x));
  return s * (1.0f + x * (1.0f - s));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Blackwell's three-input maximum and packed two-wide fp32 arithmetic: one issue slot for two
// elements.  The row loops of the attention kernels are bound by instruction issue, not by MUFU.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1)
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1,
                                      float c0, float c1) {
  asm("{\n\t.reg .b64 a, b, c, d;\n\t"
      "mov.b64 a, {%2, %3};\n\t"
      "mov.b64 b, {%4, %5};\n\t"
      "mov.b64 c, {%6, %7};\n\t"
      "fma.rn.f32x2 d, a, b, c;\n\t"
      "mov.b64 {%0, %1}, d;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t.reg .b64 a, d;\n\t"
      "mov.b64 a, {%2, %3};\n\t"
      "mov.b64 d, {%0, %1};\n\t"
      "add.rn.f32x2 d, d, a;\n\t"
      "mov.b64 {%0, %1}, d;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}
// (d0, d1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void fmul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 a, b, d;\n\t"
      "mov.b64 a, {%2, %3};\n\t"
      "mov.b64 b, {%4, %5};\n\t"
      "mul.rn.f32x2 d, a, b;\n\t"
      "mov.b64 {%0, %1}, d;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// Counter-based random bits: a hash of (seed, element index).  The dropout kernels draw their
// keep / drop decision from it, forward and backward alike, so no mask is ever stored.
__device__ __forceinline__ uint32_t mix32(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (uint32_t)(z >> 32);
}
__device__ __forceinline__ bool dropout_keep(unsigned long long seed, long long index, uint32_t thresh) {
  return mix32(seed * 0x100000001B3ull + (uint64_t)index) >= thresh;
}
// Vector reduction into global memory (16-byte aligned).
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace cgk
