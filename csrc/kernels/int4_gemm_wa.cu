// INT4 weight-only GEMM, weights on the M side of the tensor core and fed from tensor memory.
// out[M,N] = X[M,K] (bf16) . dequant(W)[K,N] (+ bias), W in the reference's format
// (src/quantize/int4.c:10-59: row-major [K,N], flat groups along N, fp32 scale per group).
//
// With few rows in X (decode: 16 .. 128) the product is bound by the weight stream.  What was
// measured on the way to this design:
//   * a shared-memory ring filled by TMA or bulk copies streams from HBM at 17-30 GB/s per SM
//     however deep the ring is or how many threads issue; plain 16-byte loads with a few requests
//     in flight per thread reach the memory's bandwidth.  Nibbles, scales and X therefore go
//     global -> registers, software-prefetched, never through a copy engine;
//   * a converted bf16 tile written to shared memory and read back by the MMA costs eight times
//     the bytes of its nibbles, and the SM's 128 B/clk of shared-memory bandwidth becomes the
//     limit.  The weights are therefore the A operand (128 output features = 128 TMEM lanes),
//     written straight into tensor memory (tcgen05.st); the MMA reads A from TMEM and only the
//     small X tile from shared memory;
//   * a warp-specialised pipeline of five roles chained by mbarriers spent ~1000 cycles per
//     128-k step on the hand-offs alone.  Here every thread does the same work per step and two
//     block barriers order it; two CTAs per SM overlap one CTA's barriers with the other's loads;
//   * the tensor core multiplies 128 features by round_up(M, 16) token columns per instruction,
//     so its time shrinks with the batch;
//   * the scale of a weight depends on (k, n / group).  With group % 128 == 0 a CTA's 128 features
//     share one scale per k, which is moved into X: x'[t,k] = x[t,k] * s[k], computed on M x 128
//     elements a step instead of 128 x 128 weights;
//   * nibbles become bf16 by bit tricks only: u = nibble ^ 8 = q + 8, and bf16 bits 0x4300 | u are
//     128 + u exactly.  The MMA therefore sums x' . (q + 136) and the epilogue subtracts
//     136 * sum_k x'[t,k], accumulated in fp32 on the side.
// The tile stream is prepared once per weight (cgk_int4_wa_tile_weights): per (128 features,
// 64 k) block 4096 bytes of nibbles as [k half][feature][4 words], where nibble j of a word holds k
// element 2j and nibble j+4 element 2j+1 (the order in which the bit trick emits pairs), then the
// block's 64 scales.
//
// One step = 128 k.  Thread (warp w, lane l): feature 32 (w % 4) + l, 64-k block w / 4 of the step:
// two 16-byte units of nibbles -> 32 TMEM columns; and the X chunks (token row, 8 k) number
// tid, tid + 256, ... of the step.  Split-K: partial sums go to an fp32 buffer with red.add; the CTA
// that arrives last at the tile's counter adds the bias, writes bf16 and leaves buffer and counter
// zeroed.
#include <cuda_bf16.h>

#include "host_common.h"
#include "sm100.cuh"
#include "cogito_kernels.h"

namespace {
using namespace cgk;

constexpr int WF = 128, WK = 64, WSUB = 2;                     // features per tile, k per block, blocks per step
constexpr int W_NIB = WF * WK / 2, W_RAW = W_NIB + WK * 4;     // 4096 + 256
constexpr int W_STEP = WSUB * W_RAW;                           // bytes of the stream per 128-k step
constexpr int W_ACOLS = WSUB * WK / 2;                         // TMEM columns of one A stage (two bf16 per column)
constexpr int W_PREFETCH = 4;                                  // steps of nibbles held in registers
constexpr int W_CONV_THREADS = 256, W_THREADS = W_CONV_THREADS + 32;   // conversion warps + the MMA warp
constexpr int W_STAGES = 3;                                    // operand stages (TMEM columns of A, shared-memory tiles of X')
constexpr int W_MAXCH = 8;                                     // X chunks per thread and step: 128 tokens x 16 chunks / 256

struct WaDev {
  const uint8_t* tiles;            // [N/128][K/64][4352]
  const __nv_bfloat16* x; long long ldx;
  float* acc; int* counters;       // split-K scratch (zero between calls)
  __nv_bfloat16* out; long long ldo;
  const __nv_bfloat16* bias;
  int M, N, K;
  int splits, ksteps;              // 128-k steps per CTA
  int x_rows;                      // token columns of the MMA: round_up(min(M, 128), 16)
  int* status;
};


__device__ __forceinline__ uint4 ldg_stream_16(const void* p) {     // read once: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int NCH>                   // X chunks per thread and step (x_rows * 16 / 256, rounded up)
__global__ void __launch_bounds__(W_THREADS, NCH <= 2 ? 2 : 1)
int4_wa_kernel(const WaDev g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const int x_rows = g.x_rows;
  const uint32_t x_bytes = (uint32_t)x_rows * 128u;                  // one [tokens, 64 k] block, 128-byte swizzle
  const uint32_t sX = base;                                          // W_STAGES stages x WSUB blocks
  uint8_t* misc = gen + W_STAGES * WSUB * x_bytes;
  const uint32_t sBar = base + W_STAGES * WSUB * x_bytes;            // a_full[], a_empty[], acc_full
  float* xsum_s = reinterpret_cast<float*>(misc + 128);              // [128]
  volatile int* dead = reinterpret_cast<volatile int*>(misc + 64);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 68);
  volatile int* is_last = reinterpret_cast<volatile int*>(misc + 72);
  volatile int* go_s = reinterpret_cast<volatile int*>(misc + 76);   // [2], by step parity
  auto a_full = [&](int s) { return sBar + 8u * s; };
  auto a_empty = [&](int s) { return sBar + 8u * (W_STAGES + s); };
  const uint32_t acc_full = sBar + 8u * 2 * W_STAGES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = g.N / WF, k_tiles = g.K / (WSUB * WK);
  const int nt = blockIdx.x % n_tiles, split = blockIdx.x / n_tiles, mt = blockIdx.y;
  const int n0 = nt * WF, ks0 = split * g.ksteps, m0 = mt * 128, ksteps = g.ksteps;
  const uint8_t* stream = g.tiles + ((long long)nt * k_tiles + ks0) * W_STEP;        // this CTA's slab, W_STEP bytes a step
  const uint32_t acc_cols = x_rows <= 32 ? 32u : x_rows <= 64 ? 64u : 128u;
  const uint32_t tmem_cols = acc_cols + W_STAGES * W_ACOLS <= 256 ? 256u : 512u;     // accumulator, then the operand stages

  if (tid == 0) {
    for (int s = 0; s < W_STAGES; ++s) { mbar_init(a_full(s), W_CONV_THREADS / 32); mbar_init(a_empty(s), 1); }
    mbar_init(acc_full, 1);
    *dead = 0;
    *is_last = 0;
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot, tmem_a = tmem + acc_cols;
  // X chunk c = tid + 256 j: block (c / 8) / x_rows, token row (c / 8) % x_rows, piece c % 8 (k = 8 (c % 8) ..)
  const int ch = tid & 7;
  const int chunks = WSUB * x_rows * 8;                              // per step
  float xs[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) xs[j] = 0.0f;
  bool ok = true;

  if (warp == W_CONV_THREADS / 32) {
    // ---- MMA warp: one thread issues; a stage is free again when its MMAs have completed
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(WF, x_rows, 0, 0);
      for (int i = 0; i < ksteps; ++i) {
        const int s = i % W_STAGES;
        if (!mbar_wait(a_full(s), (i / W_STAGES) & 1, dead, g.status, 332)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < WSUB * WK / 16; ++kk) {
          // 16 k per instruction: 8 TMEM columns of A, 32 bytes along a row of the X' block
          const uint32_t x_addr = sX + (s * WSUB + kk / (WK / 16)) * x_bytes + (kk % (WK / 16)) * 32;
          umma_f16_ts(tmem, tmem_a + s * W_ACOLS + kk * 8, make_smem_desc_sw128(x_addr, 16u, 1024u), idesc, (i | kk) != 0 ? 1u : 0u);
        }
        umma_commit(a_empty(s));
        if (i + 1 == ksteps) umma_commit(acc_full);
      }
    }
  } else {
    // ---- conversion warps: this thread's share of a step
    const int quad = warp & 3, sub = warp >> 2, f = quad * 32 + lane;
    const uint8_t* wsrc = stream + sub * W_RAW + f * 16;             // k half 0; half 1 is W_NIB / 2 further
    constexpr int NB = NCH == 1 ? 1 : WSUB;                          // scale blocks a thread needs (one chunk: one block)
    // Everything that does not change from step to step is worked out once: where each of this thread's
    // X chunks comes from (advances by 128 elements a step) and where it goes inside a stage's X' tile.
    const __nv_bfloat16* xsrc[NCH];                                   // null: padding row or no chunk
    uint32_t xdst[NCH];
    int xblk[NCH];
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = tid + j * W_CONV_THREADS, rowb = c >> 3, blk = rowb / x_rows, t = rowb - blk * x_rows;
      xblk[j] = c < chunks ? blk : -1;
      xdst[j] = (uint32_t)blk * x_bytes + sw128_offset((uint32_t)t, (uint32_t)ch);
      xsrc[j] = (c < chunks && m0 + t < g.M) ? g.x + (long long)(m0 + t) * g.ldx + ((long long)ks0 * WSUB + blk) * WK + ch * 8 : nullptr;
    }
    const uint8_t* ssrc = stream + (NCH == 1 ? (tid >> 3) / x_rows : 0) * W_RAW + W_NIB + ch * 32;
    uint4 raw[W_PREFETCH][2];
    uint4 xr[2][NCH];                                                // X chunks and scales of the next two steps, by step parity
    float4 sc[2][NB][2];
    auto load_w = [&](int d, int step) {
      const uint8_t* p = wsrc + (long long)step * W_STEP;
      raw[d][0] = ldg_stream_16(p);
      raw[d][1] = ldg_stream_16(p + W_NIB / 2);
    };
    auto load_x = [&](int p, int step) {
#pragma unroll
      for (int j = 0; j < NCH; ++j)
        xr[p][j] = xsrc[j] ? __ldg(reinterpret_cast<const uint4*>(xsrc[j] + step * (WSUB * WK))) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float4* sp = reinterpret_cast<const float4*>(ssrc + (long long)step * W_STEP + b * W_RAW);
        sc[p][b][0] = __ldg(sp); sc[p][b][1] = __ldg(sp + 1);
      }
    };
#pragma unroll
    for (int d = 0; d < W_PREFETCH; ++d) { raw[d][0] = raw[d][1] = make_uint4(0, 0, 0, 0); if (d < ksteps) load_w(d, d); }
    load_x(0, 0);
    if (ksteps > 1) load_x(1, 1);
    const uint32_t t_st = tmem_a + ((uint32_t)(quad * 32) << 16) + sub * 32;      // + stage * W_ACOLS + half * 16
    int s = 0;                                                       // stage of the step, and the parity its a_empty wait needs
    uint32_t par = 1;
    for (int i0 = 0; i0 < ksteps && ok; i0 += W_PREFETCH) {
#pragma unroll
      for (int d = 0; d < W_PREFETCH; ++d) {
        const int i = i0 + d;
        if (i >= ksteps || !ok) break;
        // stage s (TMEM operand columns and the X' tile) was last read by the MMAs of step i - W_STAGES;
        // one thread polls, a hardware barrier releases the rest
        if (tid == 0) go_s[d & 1] = (int)mbar_wait(a_empty(s), par, dead, g.status, 330);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (!go_s[d & 1]) { ok = false; break; }
        tc_fence_after();
        // nibbles -> bf16 pairs -> 32 TMEM columns of this feature's lane
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const uint32_t w[4] = {raw[d][hh].x, raw[d][hh].y, raw[d][hh].z, raw[d][hh].w};
          uint32_t t[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t v = w[c] ^ 0x88888888u;
            t[4 * c] = (v & 0x000F000Fu) | 0x43004300u;
            t[4 * c + 1] = ((v >> 4) & 0x000F000Fu) | 0x43004300u;
            t[4 * c + 2] = ((v >> 8) & 0x000F000Fu) | 0x43004300u;
            t[4 * c + 3] = ((v >> 12) & 0x000F000Fu) | 0x43004300u;
          }
          tmem_st16(t_st + s * W_ACOLS + hh * 16, t);
        }
        if (i + W_PREFETCH < ksteps) load_w(d, i + W_PREFETCH);
        // X chunks: times the scale of their k, rounded to bf16, summed for the offset correction, stored swizzled
        uint8_t* xstage = gen + s * (WSUB * x_bytes);
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          if (xblk[j] >= 0) {
            const int bi = NCH == 1 ? 0 : xblk[j];
            const float4 s0 = bi ? sc[d & 1][NB - 1][0] : sc[d & 1][0][0], s1 = bi ? sc[d & 1][NB - 1][1] : sc[d & 1][0][1];
            const uint4 xv = xr[d & 1][j];
            const float2 a = unpack_bf16x2(xv.x), b = unpack_bf16x2(xv.y), cc = unpack_bf16x2(xv.z), e = unpack_bf16x2(xv.w);
            const uint4 o = make_uint4(pack_bf16x2(a.x * s0.x, a.y * s0.y), pack_bf16x2(b.x * s0.z, b.y * s0.w),
                                       pack_bf16x2(cc.x * s1.x, cc.y * s1.y), pack_bf16x2(e.x * s1.z, e.y * s1.w));
            const float2 ra = unpack_bf16x2(o.x), rb = unpack_bf16x2(o.y), rc = unpack_bf16x2(o.z), rd = unpack_bf16x2(o.w);
            xs[j] += ((ra.x + ra.y) + (rb.x + rb.y)) + ((rc.x + rc.y) + (rd.x + rd.y));
            *reinterpret_cast<uint4*>(xstage + xdst[j]) = o;
          }
        }
        if (i + 2 < ksteps) load_x(d & 1, i + 2);
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(s));
        if (++s == W_STAGES) { s = 0; par ^= 1; }
      }
    }
  }
  // ---- row sums of x': a chunk's row is fixed per (thread, j); sum the 8 pieces of a row, then over the blocks
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    float v = xs[j];
    v += __shfl_xor_sync(0xffffffffu, v, 1); v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 4);
    xs[j] = v;
  }
  for (int i = tid; i < 128; i += W_THREADS) xsum_s[i] = 0.0f;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = tid + j * W_CONV_THREADS, rowb = c >> 3, blk = rowb / x_rows, t = rowb - blk * x_rows;
    if (ch == 0 && c < chunks && tid < W_CONV_THREADS) atomicAdd(xsum_s + t, xs[j]);         // two blocks per row: two adds per row
  }
  __syncthreads();
  // ---- epilogue (warps 0-3): lane = output feature, column = token
  if (warp < 4 && ok) {
    if (tid == 0) go_s[0] = (int)mbar_wait(acc_full, 0, dead, g.status, 331);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (go_s[0]) {
      tc_fence_after();
      const int fo = n0 + warp * 32 + lane;
      const float bias = (g.bias && g.splits == 1) ? __bfloat162float(g.bias[fo]) : 0.0f;
#pragma unroll 1
      for (int c = 0; c < x_rows; c += 16) {
        uint32_t rr[16];
        tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = m0 + c + j;
          if (t < g.M) {
            const float v = __uint_as_float(rr[j]) - 136.0f * xsum_s[c + j];
            if (g.splits == 1) g.out[(long long)t * g.ldo + fo] = __float2bfloat16(v + bias);
            else atomicAdd(g.acc + (long long)t * g.N + fo, v);
          }
        }
      }
      if (g.splits > 1) __threadfence();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, tmem_cols); }
  if (g.splits > 1) {
    if (tid == 0) *is_last = (atomicAdd(g.counters + mt * n_tiles + nt, 1) == g.splits - 1) && !*dead;
    __syncthreads();
    if (*is_last) {
      __threadfence();
      const int rows = min(128, g.M - m0);
      for (int i = tid; i < rows * (WF / 4); i += W_THREADS) {
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
      if (tid == 0) g.counters[mt * n_tiles + nt] = 0;
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

template <int NCH>
int launch_wa(const WaDev& g, dim3 grid, int smem, cudaStream_t st) {
  CGK_CUDA_CHECK(cudaFuncSetAttribute(int4_wa_kernel<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int4_wa_kernel<NCH><<<grid, W_THREADS, smem, st>>>(g);
  CGK_LAUNCH_CHECK();
  return 0;
}
}  // namespace

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
  CGK_REQUIRE(ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)tiles & 15) == 0 && ((uintptr_t)acc & 15) == 0 && ldo % 4 == 0 && ((uintptr_t)out & 7) == 0,
              "cgk_int4_wa_gemm: misaligned operand");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const int sms = sm_count(dev), n_tiles = N / WF, m_tiles = (M + 127) / 128, ksteps = K / (WSUB * WK);
  const int x_rows = m_tiles > 1 ? 128 : (M + 15) / 16 * 16;
  const int nch = (WSUB * x_rows * 8 + W_CONV_THREADS - 1) / W_CONV_THREADS;
  const int per_sm = nch <= 2 ? 2 : 1;                     // resident CTAs per SM (registers, TMEM columns)
  if (splits <= 0) {
    splits = 1;
    const int max_s = (acc && counters) ? 16 : 1;
    for (int s = 2; s <= max_s && ksteps % s == 0 && ksteps / s >= 4 && n_tiles * m_tiles * s <= sms * per_sm; s *= 2) splits = s;
  }
  CGK_REQUIRE(ksteps % splits == 0, "cgk_int4_wa_gemm: K/128 = %d is not divisible by splits = %d", ksteps, splits);
  CGK_REQUIRE(splits == 1 || (acc && counters), "cgk_int4_wa_gemm: split-K needs the acc and counters buffers");
  const int smem = 1024 + W_STAGES * WSUB * x_rows * 128 + 128 + 512 + 1024;
  WaDev g{(const uint8_t*)tiles, (const __nv_bfloat16*)x, ldx, acc, counters, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, M, N, K,
          splits, ksteps / splits, x_rows, device_status(dev)};
  const dim3 grid(n_tiles * splits, m_tiles);
  cudaStream_t st = (cudaStream_t)stream;
  switch (nch) {
    case 1: return launch_wa<1>(g, grid, smem, st);
    case 2: return launch_wa<2>(g, grid, smem, st);
    case 3: return launch_wa<3>(g, grid, smem, st);
    case 4: return launch_wa<4>(g, grid, smem, st);
    case 5: return launch_wa<5>(g, grid, smem, st);
    case 6: return launch_wa<6>(g, grid, smem, st);
    case 7: return launch_wa<7>(g, grid, smem, st);
    default: return launch_wa<W_MAXCH>(g, grid, smem, st);
  }
}
