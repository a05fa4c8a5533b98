// INT4 weight-only GEMM, weights on the M side of the tensor core and fed from tensor memory.
// out[M,N] = X[M,K] (bf16) . dequant(W)[K,N] (+ bias), W in the reference's format
// (src/quantize/int4.c:10-59: row-major [K,N], flat groups along N, fp32 scale per group).
//
// With few rows in X (decode: 16 .. 128) the product is bound by the weight stream, and on this
// machine the first limit a streaming kernel meets is shared-memory bandwidth (128 B per clock
// per SM): a converted bf16 tile written to shared memory and read back by the MMA costs eight
// times the bytes of the nibbles it came from.  So:
//   * the weights are the A operand (128 output features = 128 TMEM lanes) and are written by
//     the conversion warps straight into tensor memory (tcgen05.st); the MMA reads A from TMEM
//     and only the small X tile from shared memory.  Shared memory carries the raw nibbles once in
//     and once out, nothing else of the weights;
//   * the tensor core multiplies 128 features by round_up(M, 16) token columns per instruction,
//     so its time shrinks with the batch;
//   * the scale of a weight depends on (k, n / group).  With group % 128 == 0 a CTA's 128 features
//     share one scale per k, which is moved into X: x'[t,k] = x[t,k] * s[k], computed on M x 128
//     elements a step instead of 128 x 128 weights;
//   * nibbles become bf16 by bit tricks only: u = nibble ^ 8 = q + 8, and bf16 bits 0x4300 | u are
//     128 + u exactly.  The MMA therefore sums x' . (q + 136) and the epilogue subtracts
//     136 * sum_k x'[t,k], which the scaling warps accumulate in fp32 on the side.
// The tile stream is prepared once per weight (cgk_int4_wa_tile_weights): per (128 features,
// 64 k) block 4096 bytes of nibbles as [k half][feature][4 words], where nibble j of a word holds k
// element 2j and nibble j+4 element 2j+1 (the order in which the bit trick emits pairs), then the
// block's 64 scales.
//
//   warp 0      TMA: the weight stream, one 8704-byte step per copy, into a deep ring
//   warp 1      tcgen05.mma issue; accumulator [128 features x tokens] in TMEM
//   warp 2      TMEM allocation
//   warp 3      TMA: X tiles [tokens, 64 k]
//   warps 4-7   scale X in place, accumulate the row sums; epilogue
//   warps 8-23  nibbles -> bf16 pairs -> TMEM (warp w: features 32 (w % 4) .., k quarter w / 4 of the step)
// Split-K: partial sums go to an fp32 buffer with red.add; the CTA that arrives last at the
// tile's counter adds the bias, writes bf16 and leaves buffer and counter zeroed.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "host_common.h"
#include "sm100.cuh"
#include "cogito_kernels.h"

namespace {
using namespace cgk;

constexpr int WF = 128, WK = 64, WSUB = 2;                     // features per tile, k per block, blocks per step
constexpr int W_ASTAGES = 3, W_MAX_RAW = 16, W_MAX_X = 8, W_CONVERT_WARPS = 16;
constexpr int W_NIB = WF * WK / 2, W_RAW = W_NIB + WK * 4;     // 4096 + 256
constexpr int W_ACOLS = WSUB * WK / 2;                         // TMEM columns of one A stage (two bf16 per column)
constexpr int W_THREADS = 256 + 32 * W_CONVERT_WARPS;
constexpr int W_SMEM = 200 * 1024;
constexpr int W_RING_BUDGET = W_SMEM - 1024 - 2048 - 512;      // shared by the X and W rings

struct WaDev {
  const uint8_t* tiles;            // [N/128][K/64][4352]
  float* acc; int* counters;       // split-K scratch (zero between calls)
  __nv_bfloat16* out; long long ldo;
  const __nv_bfloat16* bias;
  int M, N, K;
  int splits, ksteps;              // 128-k steps per CTA
  int x_rows, x_stages, raw_stages;
  int dbg;                         // profiling build only: 1 skip the X scaling, 2 skip the conversion, 4 skip the MMAs
  int* status;
};

// Profiling build (-DCGK_WA_TIMING): CTA (0,0) sums, per role, the cycles spent in each wait and in
// the work between them; cgk_int4_wa_times copies the sums out.
#ifdef CGK_WA_TIMING
__device__ long long wa_t[32];
#define WT_DECL long long wt_[4] = {0, 0, 0, 0}; long long wt0_ = clock64();
#define WT_LAP(i) { const long long n_ = clock64(); wt_[i] += n_ - wt0_; wt0_ = n_; }
#define WT_STORE(base, n) if (blockIdx.x == 0 && blockIdx.y == 0) { for (int q_ = 0; q_ < n; ++q_) wa_t[base + q_] = wt_[q_]; }
#define WA_DBG(bit) (g.dbg & (bit))
#else
#define WA_DBG(bit) 0
#define WT_DECL
#define WT_LAP(i)
#define WT_STORE(base, n)
#endif

__global__ void __launch_bounds__(W_THREADS, 1)
int4_wa_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const WaDev g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t x_bytes = (uint32_t)g.x_rows * 128u;                                // one [tokens, 64 k] block
  const uint32_t sX = base;
  const uint32_t sRaw = sX + (uint32_t)g.x_stages * WSUB * x_bytes;                  // multiple of 2 KiB
  const uint32_t sBar = base + W_SMEM - 1024 - 2048 - 512;
  float* xsum_s = reinterpret_cast<float*>(gen + (sBar - base) + 1024);              // [128]
  volatile int* dead = reinterpret_cast<volatile int*>(gen + (sBar - base) + 960);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + (sBar - base) + 968);
  volatile int* is_last = reinterpret_cast<volatile int*>(gen + (sBar - base) + 976);
  volatile int* go_s = reinterpret_cast<volatile int*>(gen + (sBar - base) + 980);   // [2] scaling, [2] conversion: "the wait succeeded", by step parity
  auto x_full = [&](int s) { return sBar + 8u * s; };
  auto x_empty = [&](int s) { return sBar + 8u * (W_MAX_X + s); };
  auto xs_full = [&](int s) { return sBar + 8u * (2 * W_MAX_X + s); };
  auto a_full = [&](int s) { return sBar + 8u * (3 * W_MAX_X + s); };
  auto a_empty = [&](int s) { return sBar + 8u * (3 * W_MAX_X + W_ASTAGES + s); };
  auto raw_full = [&](int s) { return sBar + 8u * (3 * W_MAX_X + 2 * W_ASTAGES + s); };
  auto raw_empty = [&](int s) { return sBar + 8u * (3 * W_MAX_X + 2 * W_ASTAGES + W_MAX_RAW + s); };
  const uint32_t acc_full = sBar + 8u * (3 * W_MAX_X + 2 * W_ASTAGES + 2 * W_MAX_RAW);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = g.N / WF, k_tiles = g.K / (WSUB * WK);
  const int nt = blockIdx.x % n_tiles, split = blockIdx.x / n_tiles, mt = blockIdx.y;
  const int n0 = nt * WF, ks0 = split * g.ksteps, m0 = mt * 128;
  const int ksteps = g.ksteps, x_stages = g.x_stages, raw_stages = g.raw_stages, x_rows = g.x_rows;
  // TMEM: accumulator columns first, then W_ASTAGES operand stages
  const uint32_t acc_cols = x_rows <= 32 ? 32u : x_rows <= 64 ? 64u : 128u;
  const uint32_t tmem_cols = acc_cols + W_ASTAGES * W_ACOLS <= 256 ? 256u : 512u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W_MAX_X; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 1); mbar_init(xs_full(s), 4); }
    for (int s = 0; s < W_ASTAGES; ++s) { mbar_init(a_full(s), W_CONVERT_WARPS); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < W_MAX_RAW; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), W_CONVERT_WARPS + 4); }
    mbar_init(acc_full, 1);
    *dead = 0;
    *is_last = 0;
    mbar_fence_init();
  }
  if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot, tmem_a = tmem + acc_cols;

  if (warp == 0) {
    if (lane == 0) {
      // the tile stream seen as rows of 128 bytes: one step is 68 rows, fetched by one tiled TMA copy
      // (plain 1-D bulk copies issued by one thread ran one after the other at ~20 GB/s)
      tma_prefetch_desc(&tmW);
      const int row0 = (nt * k_tiles + ks0) * (WSUB * W_RAW / 128);
      WT_DECL
      for (int i = 0; i < ksteps; ++i) {
        const int r = i % raw_stages;
        if (!mbar_wait_backoff(raw_empty(r), ((i / raw_stages) & 1) ^ 1, dead, g.status, 320, 100)) break;
        WT_LAP(0)
        mbar_expect_tx(raw_full(r), WSUB * W_RAW);
        tma_load_2d(sRaw + r * (WSUB * W_RAW), &tmW, raw_full(r), 0, row0 + i * (WSUB * W_RAW / 128));
        WT_LAP(1)
      }
      WT_STORE(0, 2)
    }
  } else if (warp == 3) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      WT_DECL
      for (int i = 0; i < ksteps; ++i) {
        const int s = i % x_stages;
        if (!mbar_wait_backoff(x_empty(s), ((i / x_stages) & 1) ^ 1, dead, g.status, 321, 100)) break;
        WT_LAP(0)
        mbar_expect_tx(x_full(s), WSUB * x_bytes);
#pragma unroll
        for (int sub = 0; sub < WSUB; ++sub)
          tma_load_2d(sX + (s * WSUB + sub) * x_bytes, &tmX, x_full(s), ((ks0 + i) * WSUB + sub) * WK, m0);
        WT_LAP(1)
      }
      WT_STORE(2, 2)
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(WF, x_rows, 0, 0);
      bool ok = true;
      WT_DECL
      for (int i = 0; i < ksteps && ok; ++i) {
        const int sx = i % x_stages, sa = i % W_ASTAGES;
        if (!mbar_wait(xs_full(sx), (i / x_stages) & 1, dead, g.status, 322)) { ok = false; break; }
        WT_LAP(0)
        if (!mbar_wait(a_full(sa), (i / W_ASTAGES) & 1, dead, g.status, 323)) { ok = false; break; }
        WT_LAP(1)
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < WSUB * WK / 16; ++kk) {
          // 16 k per instruction: 8 TMEM columns of A, 32 bytes along a row of the X block
          const uint32_t x_addr = sX + (sx * WSUB + kk / (WK / 16)) * x_bytes + (kk % (WK / 16)) * 32;
          if (!WA_DBG(4)) umma_f16_ts(tmem, tmem_a + sa * W_ACOLS + kk * 8, make_smem_desc_sw128(x_addr, 16u, 1024u), idesc, (i | kk) != 0 ? 1u : 0u);
        }
        umma_commit(x_empty(sx));
        umma_commit(a_empty(sa));
        WT_LAP(2)
      }
      WT_STORE(4, 3)
      if (ok) umma_commit(acc_full);
    }
  } else if (warp >= 4 && warp < 8) {
    // ---- X scaling: chunk (row t, 16-byte piece ch) of both 64-k blocks of the step.  The piece a
    // thread owns is always ch = tid % 8, its rows are tid / 8 + 16 j.
    const int tid = threadIdx.x - 128, ch = tid & 7, trow = tid >> 3, slots = x_rows >> 4;
    float xs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[j] = 0.0f;
    bool ok = true;
    WT_DECL
    for (int i = 0; i < ksteps && ok; ++i) {
      const int r = i % raw_stages, s = i % x_stages;
      // one thread polls for the four warps (every poll is a shared-memory access), a hardware
      // barrier releases the others; a wait that gave up has set *dead
      if (tid == 0)
        go_s[i & 1] = mbar_wait_backoff(raw_full(r), (i / raw_stages) & 1, dead, g.status, 324, 40) &&
                      mbar_wait_backoff(x_full(s), (i / x_stages) & 1, dead, g.status, 325, 40);
      WT_LAP(0)
      asm volatile("bar.sync 1, 128;" ::: "memory");
      WT_LAP(1)
      if (!go_s[i & 1]) { ok = false; break; }      // the same word for all 128 threads: they leave together
#pragma unroll
      for (int sub = 0; sub < WSUB; ++sub) {
        if (WA_DBG(1)) break;
        const float4* sc4 = reinterpret_cast<const float4*>(gen + (sRaw - base) + (r * WSUB + sub) * W_RAW + W_NIB) + ch * 2;
        const float4 s0 = sc4[0], s1 = sc4[1];
        uint8_t* xt = gen + (sX - base) + (s * WSUB + sub) * x_bytes;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < slots) {
            const int t = trow + 16 * j;
            uint4* p = reinterpret_cast<uint4*>(xt + sw128_offset((uint32_t)t, (uint32_t)ch));
            const uint4 v = *p;
            const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
            uint4 o = make_uint4(pack_bf16x2(a.x * s0.x, a.y * s0.y), pack_bf16x2(b.x * s0.z, b.y * s0.w),
                                 pack_bf16x2(c.x * s1.x, c.y * s1.y), pack_bf16x2(d.x * s1.z, d.y * s1.w));
            const float2 ra = unpack_bf16x2(o.x), rb = unpack_bf16x2(o.y), rc = unpack_bf16x2(o.z), rd = unpack_bf16x2(o.w);
            xs[j] += ((ra.x + ra.y) + (rb.x + rb.y)) + ((rc.x + rc.y) + (rd.x + rd.y));
            *p = o;
          }
        }
      }
      WT_LAP(2)
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(xs_full(s)); mbar_arrive(raw_empty(r)); }
      WT_LAP(3)
    }
    if (threadIdx.x == 128) { WT_STORE(8, 4) }
    // row sums: the 8 threads that share a row sit in one quarter of a warp
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = xs[j];
      v += __shfl_xor_sync(0xffffffffu, v, 1); v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 4);
      if (ch == 0 && j < slots) xsum_s[trow + 16 * j] = v;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // ---- epilogue: lane = output feature, column = token
    if (ok && mbar_wait(acc_full, 0, dead, g.status, 326)) {
      tc_fence_after();
      const int f = n0 + (warp & 3) * 32 + lane;
      const float bias = (g.bias && g.splits == 1) ? __bfloat162float(g.bias[f]) : 0.0f;
#pragma unroll 1
      for (int c = 0; c < x_rows; c += 16) {
        uint32_t rr[16];
        tmem_ld16(tmem + ((uint32_t)((warp & 3) * 32) << 16) + c, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = m0 + c + j;
          if (t < g.M) {
            const float v = __uint_as_float(rr[j]) - 136.0f * xsum_s[c + j];
            if (g.splits == 1) g.out[(long long)t * g.ldo + f] = __float2bfloat16(v + bias);
            else atomicAdd(g.acc + (long long)t * g.N + f, v);
          }
        }
      }
      if (g.splits > 1) __threadfence();
    }
  } else if (warp >= 8) {
    // ---- conversion: thread = (feature, quarter of the step's k): one 16-byte unit of nibbles
    // becomes 16 bf16 pairs, stored as 16 TMEM columns of the feature's lane
    const int cw = warp - 8, quad = cw & 3, kq = cw >> 2, sub = kq >> 1, h = kq & 1, f = quad * 32 + lane;
    bool ok = true;
    WT_DECL
    for (int i = 0; i < ksteps && ok; ++i) {
      const int r = i % raw_stages, s = i % W_ASTAGES;
      if (threadIdx.x == 256)
        go_s[2 + (i & 1)] = mbar_wait_backoff(raw_full(r), (i / raw_stages) & 1, dead, g.status, 327, 40) &&
                            mbar_wait_backoff(a_empty(s), ((i / W_ASTAGES) & 1) ^ 1, dead, g.status, 328, 40);
      WT_LAP(0)
      asm volatile("bar.sync 2, 512;" ::: "memory");
      WT_LAP(1)
      if (!go_s[2 + (i & 1)]) { ok = false; break; }
      tc_fence_after();
      if (!WA_DBG(2)) {
      const uint4 raw = *reinterpret_cast<const uint4*>(gen + (sRaw - base) + (r * WSUB + sub) * W_RAW + h * (W_NIB / 2) + f * 16);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t t[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t v = w[c] ^ 0x88888888u;
        t[4 * c] = (v & 0x000F000Fu) | 0x43004300u;
        t[4 * c + 1] = ((v >> 4) & 0x000F000Fu) | 0x43004300u;
        t[4 * c + 2] = ((v >> 8) & 0x000F000Fu) | 0x43004300u;
        t[4 * c + 3] = ((v >> 12) & 0x000F000Fu) | 0x43004300u;
      }
      WT_LAP(2)
      tmem_st16(tmem_a + ((uint32_t)(quad * 32) << 16) + s * W_ACOLS + kq * 16, t);
      tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(a_full(s)); mbar_arrive(raw_empty(r)); }
      WT_LAP(3)
    }
    if (threadIdx.x == 256) { WT_STORE(12, 4) }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, tmem_cols); }
  if (g.splits > 1) {
    if (threadIdx.x == 0) *is_last = (atomicAdd(g.counters + mt * n_tiles + nt, 1) == g.splits - 1) && !*dead;
    __syncthreads();
    if (*is_last) {
      __threadfence();
      const int rows = min(128, g.M - m0);
      for (int i = threadIdx.x; i < rows * (WF / 4); i += W_THREADS) {
        const int t = i / (WF / 4), c4 = (i % (WF / 4)) * 4;
        float4* src = reinterpret_cast<float4*>(g.acc + (long long)(m0 + t) * g.N + n0 + c4);
        float4 v = __ldcg(src);
        *src = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (g.bias) {
          v.x += __bfloat162float(g.bias[n0 + c4]); v.y += __bfloat162float(g.bias[n0 + c4 + 1]);
          v.z += __bfloat162float(g.bias[n0 + c4 + 2]); v.w += __bfloat162float(g.bias[n0 + c4 + 3]);
        }
        *reinterpret_cast<uint2*>(g.out + (long long)(m0 + t) * g.ldo + n0 + c4) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
      }
      if (threadIdx.x == 0) g.counters[mt * n_tiles + nt] = 0;
    }
  }
}

// packed [K][N/2] bytes + scales (flat groups along N) -> tiles [N/128][K/64][4352]
__global__ void int4_wa_tile_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, int K, int N, int group,
                                    uint8_t* __restrict__ tiles) {
  const int k_tiles = K / WK;
  const long long blocks = (long long)(N / WF) * k_tiles;
  for (long long blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
    const int nt = (int)(blk / k_tiles), kt = (int)(blk % k_tiles);
    uint8_t* dst = tiles + blk * W_RAW;
    for (int i = threadIdx.x; i < W_NIB / 4; i += blockDim.x) {       // word i: k half i / 512, feature (i % 512) / 4, word i % 4
      const int f = nt * WF + ((i & 511) >> 2), k0 = kt * WK + (i >> 9) * 32 + (i & 3) * 8;
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint8_t byte = packed[((long long)(k0 + e) * N + f) >> 1];
        const uint32_t nib = (f & 1) ? (byte >> 4) : (byte & 0xF);
        word |= nib << (4 * ((e >> 1) + 4 * (e & 1)));
      }
      reinterpret_cast<uint32_t*>(dst)[i] = word;
    }
    for (int i = threadIdx.x; i < WK; i += blockDim.x)
      reinterpret_cast<float*>(dst + W_NIB)[i] = scales[((long long)(kt * WK + i) * N + nt * WF) / group];
  }
}
}  // namespace

#ifdef CGK_WA_TIMING
CGK_API int cgk_int4_wa_times(long long* out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, wa_t, sizeof(long long) * 32);
}
#endif
CGK_API long long cgk_int4_wa_tiles_bytes(int K, int N) { return (long long)(N / WF) * (K / WK) * W_RAW; }
// Reorders reference-format weights (packed [K, N/2] bytes, fp32 scales per flat group) into the
// stream cgk_int4_wa_gemm reads.  group: a multiple of 128 that divides N.
CGK_API int cgk_int4_wa_tile_weights(const void* packed, const float* scales, int K, int N, int group, void* tiles, void* stream) {
  CGK_REQUIRE(packed && scales && tiles, "cgk_int4_wa_tile_weights: null pointer");
  CGK_REQUIRE(N % WF == 0 && K % WK == 0, "cgk_int4_wa_tile_weights: need N %% 128 == 0 and K %% 64 == 0 (got K=%d N=%d)", K, N);
  CGK_REQUIRE(group >= 128 && group % 128 == 0 && N % group == 0, "cgk_int4_wa_tile_weights: group %d must be a multiple of 128 that divides N", group);
  CGK_REQUIRE(((uintptr_t)tiles & 15) == 0, "cgk_int4_wa_tile_weights: misaligned buffer");
  const long long blocks = (long long)(N / WF) * (K / WK);
  int4_wa_tile_kernel<<<(unsigned)(blocks < 4736 ? blocks : 4736), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, scales, K, N, group, (uint8_t*)tiles);
  CGK_LAUNCH_CHECK();
  return 0;
}

// x bf16 [M, ldx]; tiles from cgk_int4_wa_tile_weights; out bf16 [M, ldo]; bias bf16 [N] or null.
// acc (fp32 [M, N]) and counters (int32 [cgk_int4_gemm_counters(M, N)]) serve split-K: zero before
// the first call, left zero by every call.  splits 0 = chosen here.
CGK_API int cgk_int4_wa_gemm(const void* x, long long ldx, const void* tiles, float* acc, int* counters, void* out, long long ldo,
                             const void* bias, int M, int N, int K, int splits, void* stream) {
  using namespace cgk;
  CGK_REQUIRE(x && tiles && out, "cgk_int4_wa_gemm: null pointer");
  CGK_REQUIRE(M > 0 && N > 0 && K > 0 && N % WF == 0 && K % (WSUB * WK) == 0, "cgk_int4_wa_gemm: need N %% 128 == 0 and K %% 128 == 0 (got M=%d N=%d K=%d)", M, N, K);
  CGK_REQUIRE(ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)tiles & 15) == 0 && ldo % 4 == 0 && ((uintptr_t)out & 7) == 0 && ((uintptr_t)acc & 15) == 0,
              "cgk_int4_wa_gemm: misaligned operand");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const int sms = sm_count(dev), n_tiles = N / WF, m_tiles = (M + 127) / 128, ksteps = K / (WSUB * WK);
  if (splits <= 0) {
    splits = 1;
    const int max_s = (acc && counters) ? 16 : 1;
    for (int s = 2; s <= max_s && ksteps % s == 0 && ksteps / s >= 2 && n_tiles * m_tiles * s <= sms; s *= 2) splits = s;
  }
  CGK_REQUIRE(ksteps % splits == 0, "cgk_int4_wa_gemm: K/128 = %d is not divisible by splits = %d", ksteps, splits);
  CGK_REQUIRE(splits == 1 || (acc && counters), "cgk_int4_wa_gemm: split-K needs the acc and counters buffers");
  const int x_rows = m_tiles > 1 ? 128 : (M + 15) / 16 * 16;
  int x_stages = (W_RING_BUDGET / 3) / (WSUB * x_rows * 128);
  if (x_stages < 2) x_stages = 2;
  if (x_stages > W_MAX_X) x_stages = W_MAX_X;
  int raw_stages = (W_RING_BUDGET - x_stages * WSUB * x_rows * 128) / (WSUB * W_RAW);
  if (raw_stages > W_MAX_RAW) raw_stages = W_MAX_RAW;
  CUtensorMap tmX;
  int rc = encode_tmap_bf16_2d(&tmX, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)x_rows, WK);
  if (rc) return rc;
  CUtensorMap tmW;
  {
    const uint64_t dims[2] = {128, (uint64_t)cgk_int4_wa_tiles_bytes(K, N) / 128}, strides[1] = {128};
    const uint32_t box[2] = {128, WSUB * W_RAW / 128};
    rc = encode_tmap(&tmW, tiles, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box, Swz::None);
    if (rc) return rc;
  }
  static bool attr_set[64] = {};
  if (dev < 64 && !attr_set[dev]) {
    CGK_CUDA_CHECK(cudaFuncSetAttribute(int4_wa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM));
    attr_set[dev] = true;
  }
  WaDev g{(const uint8_t*)tiles, acc, counters, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, M, N, K,
          splits, ksteps / splits, x_rows, x_stages, raw_stages, getenv("CGK_WA_DEBUG") ? atoi(getenv("CGK_WA_DEBUG")) : 0, device_status(dev)};
  int4_wa_kernel<<<dim3(n_tiles * splits, m_tiles), W_THREADS, W_SMEM, (cudaStream_t)stream>>>(tmX, tmW, g);
  CGK_LAUNCH_CHECK();
  return 0;
}
