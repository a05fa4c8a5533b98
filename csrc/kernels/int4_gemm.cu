// INT4 weight-only GEMM for serving: out[M,N] = X[M,K] (bf16) . dequant(W)[K,N] (+ bias).
//
// W holds the reference's quantised values (src/quantize/int4.c:10-59, 90-114: row-major [K,N],
// 4-bit two's complement, even column in the low nibble, one fp32 scale per flat group of
// `group` elements), reordered tile-major without re-quantising: for n-tile nt (128 columns)
// and k-step ks (64 rows) one contiguous 4608-byte block holds the tile's 64 rows of 64 bytes
// followed by the tile's scales as fp32 [64 rows][2 column halves].  A CTA's slab is then one
// sequential stream, which is what keeps HBM efficient (64-byte pieces of the row-major
// layout are not); cgk_int4_tile_weights does the reordering.
//
// The shape is weight-bandwidth bound (M <= 128 rows against megabytes of weights):
//   warp 0    bulk copies of W blocks into a 12-deep ring (bytes in flight cover HBM latency)
//   warp 3    TMA: X tiles [rows, 64 k] into their own ring of up to 12 stages; only
//             round_up(M, 8) rows are fetched — the tensor core still multiplies 128 rows, the
//             others hold whatever shared memory held and only feed output rows nobody stores
//   warps 4-11 nibbles -> bf16: exact integer (magic-number trick), one multiply by the scale,
//             stored in the 128-byte-swizzled MN-major operand layout tcgen05 reads.  Columns
//             stay in the pair order the extraction yields (0,4,1,5,2,6,3,7 within each group
//             of 8); the epilogue undoes the permutation when it addresses the output.
//   warp 1    tcgen05.mma, accumulator in TMEM (128 lanes x 128 columns)
//   warps 4-7 epilogue.  One split: TMEM -> bias -> bf16 -> global.  Split-K: vector red.add
//             into a zeroed fp32 buffer; the CTA that arrives last at the tile's counter adds
//             the bias, writes bf16 and leaves buffer and counter zeroed for the next call.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "host_common.h"
#include "sm100.cuh"
#include "cogito_kernels.h"

namespace {
using namespace cgk;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int ISSUE_LANES = 8;                                // threads of a producer warp that issue copies
constexpr int SUB = 2;                                        // 64-row sub-tiles per pipeline step (a step covers 128 k)
constexpr int B_STAGES = 3, MAX_RAW_STAGES = 16, MAX_A_STAGES = 8, CONVERT_WARPS = 16;
constexpr int B_BYTES = BK * BN * 2;
constexpr int NIB_BYTES = BK * BN / 2, SCALE_BYTES = BK * 2 * 4, RAW_BYTES = NIB_BYTES + SCALE_BYTES;   // 4096 + 512
constexpr int THREADS = 128 + 32 * CONVERT_WARPS;
constexpr int SMEM_BYTES = 226 * 1024;                       // alignment slack | X ring | B ring | W ring | barriers
constexpr int RING_BUDGET = SMEM_BYTES - 1024 - B_STAGES * SUB * B_BYTES - 2048;   // shared by the X and W rings

struct Int4Dev {
  const uint8_t* w_tiles;          // [N/128][K/64][4608]
  float* acc;                      // fp32 [M, N], zero between calls (split-K only)
  int* counters;                   // int32 [m_tiles * n_tiles], zero between calls (split-K only)
  __nv_bfloat16* out; long long ldo;
  const __nv_bfloat16* bias;
  int M, N, K;
  int splits, ksteps;              // k-steps per CTA
  int a_rows, a_stages;            // rows fetched per X tile (multiple of 8), depth of the X ring
  int raw_stages;                  // depth of the W ring
  int skip_convert;                // profiling aid: leave the operand tile unwritten (results are then meaningless)
  int* status;
};



__global__ void __launch_bounds__(THREADS, 1)
int4_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const Int4Dev g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base;                                         // a_stages x (a_rows * 128 B); reads of 128 rows may run into sB
  const uint32_t sB = sA + (uint32_t)g.a_stages * SUB * (uint32_t)g.a_rows * 128u;   // B_STAGES x SUB x 16 KiB
  const uint32_t sRaw = sB + B_STAGES * SUB * B_BYTES;              // raw_stages x SUB x 4608 B
  const uint32_t sBar = base + SMEM_BYTES - 2048;
  const uint8_t* raw_s = gen + (sRaw - base);
  volatile int* dead = reinterpret_cast<volatile int*>(gen + (sBar - base) + 960);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + (sBar - base) + 968);
  volatile int* is_last = reinterpret_cast<volatile int*>(gen + (sBar - base) + 976);
  auto a_full = [&](int s) { return sBar + 8u * s; };
  auto a_empty = [&](int s) { return sBar + 8u * (MAX_A_STAGES + s); };
  auto b_full = [&](int s) { return sBar + 8u * (2 * MAX_A_STAGES + s); };
  auto b_empty = [&](int s) { return sBar + 8u * (2 * MAX_A_STAGES + B_STAGES + s); };
  auto raw_full = [&](int s) { return sBar + 8u * (2 * MAX_A_STAGES + 2 * B_STAGES + s); };
  auto raw_empty = [&](int s) { return sBar + 8u * (2 * MAX_A_STAGES + 2 * B_STAGES + MAX_RAW_STAGES + s); };
  const uint32_t acc_full = sBar + 8u * (2 * MAX_A_STAGES + 2 * B_STAGES + 2 * MAX_RAW_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = g.N / BN, k_tiles = g.K / (SUB * BK);
  const int nt = blockIdx.x % n_tiles, split = blockIdx.x / n_tiles, mt = blockIdx.y;
  const int n0 = nt * BN, ks0 = split * g.ksteps, m0 = mt * BM;     // ks0, ksteps count 128-row steps
  const int ksteps = g.ksteps, a_stages = g.a_stages, RAW_STAGES = g.raw_stages;
  const uint32_t a_bytes = (uint32_t)g.a_rows * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_A_STAGES; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < B_STAGES; ++s) { mbar_init(b_full(s), CONVERT_WARPS); mbar_init(b_empty(s), 1); }
    for (int s = 0; s < MAX_RAW_STAGES; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), CONVERT_WARPS); }
    mbar_init(acc_full, 1);
    *dead = 0;
    *is_last = 0;
    mbar_fence_init();
  }
  if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // A thread's bulk copies run one after the other (measured: ~0.43 us each, whatever the ring
    // depth), so several lanes issue, each with its own copies in flight.  A ring slot always
    // belongs to the same lane: its uses are then waited for in order, which the one-bit phase
    // parity of an mbarrier requires.
    if (lane < ISSUE_LANES) {
      const uint8_t* src = g.w_tiles + ((long long)nt * k_tiles + ks0) * (SUB * RAW_BYTES);
      for (int i = 0; i < ksteps; ++i) {
        const int r = i % RAW_STAGES;
        if (r % ISSUE_LANES != lane) continue;
        if (!mbar_wait(raw_empty(r), ((i / RAW_STAGES) & 1) ^ 1, dead, g.status, 300)) break;
        mbar_expect_tx(raw_full(r), SUB * RAW_BYTES);
        bulk_load_1d(sRaw + r * (SUB * RAW_BYTES), src + (long long)i * (SUB * RAW_BYTES), SUB * RAW_BYTES, raw_full(r));
      }
    }
  } else if (warp == 3) {
    if (lane < ISSUE_LANES) {
      if (lane == 0) tma_prefetch_desc(&tmX);
      for (int i = 0; i < ksteps; ++i) {
        const int s = i % a_stages;
        if (s % ISSUE_LANES != lane) continue;
        if (!mbar_wait(a_empty(s), ((i / a_stages) & 1) ^ 1, dead, g.status, 301)) break;
        mbar_expect_tx(a_full(s), SUB * a_bytes);
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub)
          tma_load_2d(sA + (s * SUB + sub) * a_bytes, &tmX, a_full(s), ((ks0 + i) * SUB + sub) * BK, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, 0, 1);
      bool ok = true;
      for (int i = 0; i < ksteps && ok; ++i) {
        const int sa = i % a_stages, sb = i % B_STAGES;
        if (!mbar_wait(a_full(sa), (i / a_stages) & 1, dead, g.status, 302) ||
            !mbar_wait(b_full(sb), (i / B_STAGES) & 1, dead, g.status, 303)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          const uint32_t a_addr = sA + (sa * SUB + sub) * a_bytes, b_addr = sB + (sb * SUB + sub) * B_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            if (!(g.skip_convert & 2)) umma_f16(tmem, make_smem_desc_sw128(a_addr + kk * 32, 16u, 1024u), make_smem_desc_sw128(b_addr + kk * 2048, 8192u, 1024u), idesc,
                     (i | sub | kk) != 0 ? 1u : 0u);
        }
        umma_commit(a_empty(sa));
        umma_commit(b_empty(sb));
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (warp >= 4) {
    const int tid = threadIdx.x - 128;                 // 0 .. 32*CONVERT_WARPS-1
    constexpr int WORDS_PER_THREAD = (SUB * BK * BN / 8) / (32 * CONVERT_WARPS);
    bool ok = true;
    for (int i = 0; i < ksteps && ok; ++i) {
      const int r = i % RAW_STAGES, s = i % B_STAGES;
      // one lane polls for the warp (256+ threads hammering one barrier word cost ~150 cycles a wait)
      int got = 1;
      if (lane == 0) got = mbar_wait(raw_full(r), (i / RAW_STAGES) & 1, dead, g.status, 304) &&
                           mbar_wait(b_empty(s), ((i / B_STAGES) & 1) ^ 1, dead, g.status, 305);
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { ok = false; break; }
      if (!(g.skip_convert & 1)) {
#pragma unroll
        for (int it = 0; it < WORDS_PER_THREAD; ++it) {
          // word of the step: sub-tile, then row k = w / 16 (16 words = 128 columns), 8 columns per word
          const int wi = it * (32 * CONVERT_WARPS) + tid, sub = wi >> 10, w = wi & 1023, k = w >> 4, jw = w & 15;
          const uint8_t* tile = raw_s + (r * SUB + sub) * RAW_BYTES;
          const uint32_t* raw = reinterpret_cast<const uint32_t*>(tile);
          const float* scale = reinterpret_cast<const float*>(tile + NIB_BYTES);
          const uint32_t b_addr = sB + (s * SUB + sub) * B_BYTES;
          const uint32_t v = raw[w] ^ 0x88888888u;         // two's complement -> q + 8
          const __nv_bfloat162 off = __float2bfloat162_rn(136.0f), sc = __float2bfloat162_rn(scale[2 * k + (jw >> 3)]);
          uint32_t t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t u = ((v >> (4 * j)) & 0x000F000Fu) | 0x43004300u;      // bf16 (128 + q + 8) for columns j and j + 4
            __nv_bfloat162 h = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&u), off), sc);
            t[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          // positions 0..7 of the chunk hold columns 0,4,1,5,2,6,3,7
          const uint32_t dst = b_addr + (jw >> 3) * 8192u + sw128_offset((uint32_t)k, (uint32_t)(jw & 7));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(t[0]), "r"(t[1]), "r"(t[2]), "r"(t[3]) : "memory");
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(b_full(s)); mbar_arrive(raw_empty(r)); }
    }
    // ---- epilogue (first four conversion warps): lane = output row inside the 128-row tile.
    // Accumulator positions j..j+7 of a group of 8 are columns j + {0,4,1,5,2,6,3,7}.
    if (warp < 8 && ok && mbar_wait(acc_full, 0, dead, g.status, 306)) {
      tc_fence_after();
      const int row = m0 + (warp & 3) * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t rr[32];
        tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + c, rr);
        tmem_ld_wait();
        if (row >= g.M) continue;
        if (g.splits == 1) {
          __nv_bfloat16* dstp = g.out + (long long)row * g.ldo + n0 + c;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float v[8] = {__uint_as_float(rr[j]), __uint_as_float(rr[j + 2]), __uint_as_float(rr[j + 4]), __uint_as_float(rr[j + 6]),
                          __uint_as_float(rr[j + 1]), __uint_as_float(rr[j + 3]), __uint_as_float(rr[j + 5]), __uint_as_float(rr[j + 7])};
            if (g.bias) {
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] += __bfloat162float(g.bias[n0 + c + j + e]);
            }
            uint4 pk = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
            *reinterpret_cast<uint4*>(dstp + j) = pk;
          }
        } else {
          float* dstp = g.acc + (long long)row * g.N + n0 + c;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            red_add_f32x4(dstp + j, __uint_as_float(rr[j]), __uint_as_float(rr[j + 2]), __uint_as_float(rr[j + 4]), __uint_as_float(rr[j + 6]));
            red_add_f32x4(dstp + j + 4, __uint_as_float(rr[j + 1]), __uint_as_float(rr[j + 3]), __uint_as_float(rr[j + 5]), __uint_as_float(rr[j + 7]));
          }
        }
      }
      if (g.splits > 1) __threadfence();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, BN); }
  if (g.splits > 1) {
    // the split that arrives last at the tile's counter turns the fp32 sums into the output
    if (threadIdx.x == 0) *is_last = (atomicAdd(g.counters + mt * n_tiles + nt, 1) == g.splits - 1) && !*dead;
    __syncthreads();
    if (*is_last) {
      __threadfence();
      const int rows = min(BM, g.M - m0);
      for (int i = threadIdx.x; i < rows * (BN / 4); i += THREADS) {
        const int r = i / (BN / 4), c4 = (i % (BN / 4)) * 4;
        float4* src = reinterpret_cast<float4*>(g.acc + (long long)(m0 + r) * g.N + n0 + c4);
        float4 v = __ldcg(src);
        *src = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (g.bias) {
          v.x += __bfloat162float(g.bias[n0 + c4]); v.y += __bfloat162float(g.bias[n0 + c4 + 1]);
          v.z += __bfloat162float(g.bias[n0 + c4 + 2]); v.w += __bfloat162float(g.bias[n0 + c4 + 3]);
        }
        *reinterpret_cast<uint2*>(g.out + (long long)(m0 + r) * g.ldo + n0 + c4) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
      }
      if (threadIdx.x == 0) g.counters[mt * n_tiles + nt] = 0;
    }
  }
}

// packed [K][N/2] bytes + scales (flat groups) -> tiles [N/128][K/64][4608]
__global__ void int4_tile_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, int K, int N, int group,
                                 uint8_t* __restrict__ tiles) {
  const int k_tiles = K / BK;
  const long long blocks = (long long)(N / BN) * k_tiles;
  for (long long blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
    const int nt = (int)(blk / k_tiles), ks = (int)(blk % k_tiles);
    uint8_t* dst = tiles + blk * RAW_BYTES;
    for (int i = threadIdx.x; i < NIB_BYTES / 4; i += blockDim.x) {
      const int k = i >> 4, wj = i & 15;
      reinterpret_cast<uint32_t*>(dst)[i] = *reinterpret_cast<const uint32_t*>(packed + ((long long)(ks * BK + k) * N + nt * BN) / 2 + wj * 4);
    }
    for (int i = threadIdx.x; i < BK * 2; i += blockDim.x) {
      const int k = i >> 1, half = i & 1;
      reinterpret_cast<float*>(dst + NIB_BYTES)[i] = scales[((long long)(ks * BK + k) * N + nt * BN + half * 64) / group];
    }
  }
}
}  // namespace

CGK_API long long cgk_int4_tiles_bytes(int K, int N) { return (long long)(N / BN) * (K / BK) * RAW_BYTES; }
// Reorders reference-format weights (packed [K, N/2] bytes, fp32 scales per flat group) into the
// tile-major stream the GEMM reads.  group: a multiple of 64 with N % group == 0.
CGK_API int cgk_int4_tile_weights(const void* packed, const float* scales, int K, int N, int group, void* tiles, void* stream) {
  CGK_REQUIRE(packed && scales && tiles, "cgk_int4_tile_weights: null pointer");
  CGK_REQUIRE(N % BN == 0 && K % BK == 0, "cgk_int4_tile_weights: need N %% 128 == 0 and K %% 64 == 0 (got K=%d N=%d)", K, N);
  CGK_REQUIRE(group >= 64 && group % 64 == 0 && N % group == 0, "cgk_int4_tile_weights: group %d must be a multiple of 64 that divides N", group);
  CGK_REQUIRE(((uintptr_t)packed & 3) == 0 && ((uintptr_t)tiles & 15) == 0, "cgk_int4_tile_weights: misaligned buffer");
  const long long blocks = (long long)(N / BN) * (K / BK);
  int4_tile_kernel<<<(unsigned)(blocks < 4736 ? blocks : 4736), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, scales, K, N, group, (uint8_t*)tiles);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API long long cgk_int4_gemm_counters(int M, int N) { return (long long)((M + BM - 1) / BM) * (N / BN); }

// x bf16 [M, ldx]; w_tiles from cgk_int4_tile_weights; out bf16 [M, ldo]; bias bf16 [N] or null.
// acc (fp32 [M, N]) and counters (int32 [cgk_int4_gemm_counters]) serve split-K: both must be
// zero before the first call and are left zero by every call.  splits 0 = chosen here.
CGK_API int cgk_int4_gemm(const void* x, long long ldx, const void* w_tiles, float* acc, int* counters, void* out, long long ldo,
                          const void* bias, int M, int N, int K, int splits, void* stream) {
  using namespace cgk;
  CGK_REQUIRE(x && w_tiles && out, "cgk_int4_gemm: null pointer");
  CGK_REQUIRE(M > 0 && N > 0 && K > 0 && N % BN == 0 && K % (SUB * BK) == 0, "cgk_int4_gemm: need N %% 128 == 0 and K %% 128 == 0 (got M=%d N=%d K=%d)", M, N, K);
  CGK_REQUIRE(ldx % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w_tiles & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)acc & 15) == 0,
              "cgk_int4_gemm: operands must be 16-byte aligned with leading dimensions that are multiples of 8");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const int sms = sm_count(dev), n_tiles = N / BN, m_tiles = (M + BM - 1) / BM, ksteps = K / (SUB * BK);
  if (splits <= 0) {
    // one wave: the largest power-of-two split whose CTAs all fit on the SMs at once (a second,
    // partly filled wave measured slower than fewer, longer CTAs), at least 2 steps per CTA
    splits = 1;
    const int max_s = (acc && counters) ? 16 : 1;
    for (int s = 2; s <= max_s && ksteps % s == 0 && ksteps / s >= 2 && n_tiles * m_tiles * s <= sms; s *= 2) splits = s;
  }
  CGK_REQUIRE(ksteps % splits == 0, "cgk_int4_gemm: K/128 = %d is not divisible by splits = %d", ksteps, splits);
  CGK_REQUIRE(splits == 1 || (acc && counters), "cgk_int4_gemm: split-K needs the acc and counters buffers");
  const int a_rows = m_tiles > 1 ? BM : (M + 7) / 8 * 8;
  // the X ring gets up to a quarter of the ring budget (at least 2 stages), the W ring the rest
  int a_stages = (RING_BUDGET / 4) / (SUB * a_rows * 128);
  if (a_stages < 2) a_stages = 2;
  if (a_stages > MAX_A_STAGES) a_stages = MAX_A_STAGES;
  int raw_stages = (RING_BUDGET - a_stages * SUB * a_rows * 128) / (SUB * RAW_BYTES);
  if (raw_stages > MAX_RAW_STAGES) raw_stages = MAX_RAW_STAGES;
  static const int raw_cap = getenv("CGK_INT4_RAW_STAGES") ? atoi(getenv("CGK_INT4_RAW_STAGES")) : 0;
  if (raw_cap > 0 && raw_cap < raw_stages) raw_stages = raw_cap;
  CUtensorMap tmX;
  int rc = encode_tmap_bf16_2d(&tmX, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)a_rows, BK);
  if (rc) return rc;
  static bool attr_set[64] = {};
  if (dev < 64 && !attr_set[dev]) {
    CGK_CUDA_CHECK(cudaFuncSetAttribute(int4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set[dev] = true;
  }
  static const int skip_convert = getenv("CGK_INT4_SKIP_CONVERT") ? atoi(getenv("CGK_INT4_SKIP_CONVERT")) : 0;
  Int4Dev g{(const uint8_t*)w_tiles, acc, counters, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, M, N, K,
            splits, ksteps / splits, a_rows, a_stages, raw_stages, skip_convert, device_status(dev)};
  int4_gemm_kernel<<<dim3(n_tiles * splits, m_tiles), THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tmX, g);
  CGK_LAUNCH_CHECK();
  return 0;
}
