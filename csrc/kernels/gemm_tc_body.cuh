// Device body of the tcgen05 bf16 GEMM, shared by the plain GEMM kernel and by the
// fused compute + collective kernels (all-gather -> GEMM, GEMM -> reduce-scatter).
// See gemm_tcgen05.cu for the description of the pipeline.
#pragma once
#include "../../include/cogito_kernels.h"
#include "sm100.cuh"

namespace cgk {

constexpr int GEMM_MAX_RANKS = 8;

struct GemmDev {
  int M, N, K, batch;
  int tiles_m, tiles_n;
  int a_mn, b_mn;
  void* out;
  long long ldc, strideC;
  int out_fp32, accumulate;
  // 1: the bf16 output (and the pre-activation output, if any) leaves through bulk tensor stores
  // from the epilogue's staging tiles; the launcher sets it when the output's layout allows a
  // tensor map (16-byte aligned base, leading dimension a multiple of 8) and nothing is accumulated
  int tma_store;
  // 1: aux_in (2: residual) is fetched by bulk tensor loads into the epilogue's staging tiles
  // (set together with tma_store when that operand's layout allows a tensor map and no
  // pre-activation output needs the second half of the staging tile)
  int tma_in;
  float alpha;
  const void* bias;
  int bias_fp32;
  int act;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* aux_out;
  long long ldaux;
  const __nv_bfloat16* aux_in;
  long long ldauxin;
  int dact;
  int* status;
  // Rotary embedding applied to output columns [0, rope_cols) (see cgk_gemm_args)
  const float* rope_cos; const float* rope_sin;
  int rope_cols, rope_D, rope_T, rope_pos0, rope_inverse;
  // Split-K: every output tile is computed by split_k work units, each over kb_per_split
  // k-blocks, that add their part into the fp32 output with vector reductions (only with
  // out_fp32 && accumulate and no other epilogue term).  For weight gradients: a small
  // output with a very long reduction dimension gives too few tiles for the SMs otherwise.
  int split_k, kb_per_split;
  // ---- hooks used by the fused kernels (all off when zero / null) ----
  // A-operand readiness: before loading rows [m0, m0+128) of A the producer waits
  // until a_ready[m0 / a_ready_rows] >= a_ready_target (flags set by the copy CTAs
  // of the same kernel, or by the GPU that multicast the rows: system scope).
  const int* a_ready;
  int a_ready_rows;
  int a_ready_target;
  // m-tile rotation: tile index tm is processed as (tm + m_rot) % tiles_m, so each
  // rank starts with the rows that are available / needed first.
  int m_rot;
  // m-tile interleave: with m_inter = P the i-th row of tiles walked is block i / P of
  // shard (i % P + m_src0) % P, so that the shards of all ranks are consumed (all-gather
  // by multicast) or filled (reduce-scatter) at the same pace.
  int m_inter, m_src0;
  // Reduce-scatter epilogue: rows [o*rs_rows, (o+1)*rs_rows) of the result belong to
  // rank o and are stored (bf16) at rs_dst[o] + (row - o*rs_rows)*ldc + col; after a
  // tile is stored, rs_flag[o][(row - o*rs_rows) / 128] is incremented (system scope).
  int rs_ranks;
  int rs_rows;
  __nv_bfloat16* rs_dst[GEMM_MAX_RANKS];
  int* rs_flag[GEMM_MAX_RANKS];
};

__device__ __forceinline__ float apply_act(int act, float v) {
  switch (act) {
    case CGK_ACT_GELU: return gelu_tanh(v);
    case CGK_ACT_RELU: return fmaxf(v, 0.0f);
    case CGK_ACT_SILU: return silu_f(v);
    case CGK_ACT_SIGMOID: return 1.0f / (1.0f + __expf(-v));
    case CGK_ACT_TANH: return tanhf(v);
    default: return v;
  }
}
__device__ __forceinline__ float apply_dact(int act, float x) {
  switch (act) {
    case CGK_ACT_GELU: return dgelu_tanh(x);
    case CGK_ACT_RELU: return x > 0.0f ? 1.0f : 0.0f;
    case CGK_ACT_SILU: return dsilu_f(x);
    case CGK_ACT_SIGMOID: { float s = 1.0f / (1.0f + __expf(-x)); return s * (1.0f - s); }
    case CGK_ACT_TANH: { float t = tanhf(x); return 1.0f - t * t; }
    default: return 1.0f;
  }
}

// Where element (b, m, n) of the result goes.
__device__ __forceinline__ void* out_address(const GemmDev& g, int b, int m, int n, bool& fp32) {
  if (g.rs_ranks > 0) {
    const int o = m / g.rs_rows;
    fp32 = false;
    return g.rs_dst[o] + (long long)(m - o * g.rs_rows) * g.ldc + n;
  }
  fp32 = g.out_fp32 != 0;
  m = (int)CGK_IDX(m, g.M);
  n = (int)CGK_IDX(n, g.N);
  const long long off = (long long)b * g.strideC + (long long)m * g.ldc + n;
  return fp32 ? (void*)(reinterpret_cast<float*>(g.out) + off)
              : (void*)(reinterpret_cast<__nv_bfloat16*>(g.out) + off);
}

// Epilogue for one element; shared by the tensor-core kernel's ragged path and
// the CUDA-core fallback.
__device__ __forceinline__ void epilogue_scalar(const GemmDev& g, int b, int m, int n, float acc) {
  float v = g.alpha * acc;
  if (g.bias) {
    v += g.bias_fp32 ? reinterpret_cast<const float*>(g.bias)[n]
                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g.bias)[n]);
  }
  if (g.aux_out) g.aux_out[(long long)m * g.ldaux + n] = __float2bfloat16(v);
  v = apply_act(g.act, v);
  if (g.aux_in) v *= apply_dact(g.dact, __bfloat162float(g.aux_in[(long long)m * g.ldauxin + n]));
  if (g.residual) v += __bfloat162float(g.residual[(long long)m * g.ldr + n]);
  bool fp32;
  void* dst = out_address(g, b, m, n, fp32);
  if (fp32) {
    float* p = reinterpret_cast<float*>(dst);
    *p = g.accumulate ? (*p + v) : v;
  } else {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(dst);
    *p = __float2bfloat16(g.accumulate ? (__bfloat162float(*p) + v) : v);
  }
}

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GROUP_M = 8;
constexpr int GEMM_THREADS = 384;       // TMA warp, MMA warp, TMEM warp, one spare, eight epilogue warps
constexpr int RS_SIGNAL_BATCH = 4;      // reduce-scatter tiles published per system-scope fence

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // per-warp staging tiles of the epilogue (8 warps x 4 KiB = 32 rows x 128 bytes each, 128-byte
  // swizzle, 1024-byte aligned): outputs are transposed through them so that they leave as whole
  // lines (bulk tensor stores, or 128-byte row segments on the reduce-scatter path)
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + 8 * 4096;
  static constexpr int NUM_BARS = 2 * STAGES + 6 + 8;    // + one per epilogue warp for its input tile
  // the tile's bias slice, two tiles deep: fp32 for tiles of up to 128 columns, bf16 for 256
  // (an fp32 bias with the widest tile is read from global memory instead)
  static constexpr int SBIAS_OFFSET = (BAR_OFFSET + NUM_BARS * 8 + 16 + 127) / 128 * 128;
  static constexpr int TOTAL = SBIAS_OFFSET + 1024 + 1024;  // + alignment slack
  static_assert(TOTAL <= 227 * 1024, "GEMM: shared memory budget of one CTA exceeded");
};

__device__ __forceinline__ void tile_coords(const GemmDev& g, int t, int& b, int& tm, int& tn) {
  const int per_batch = g.tiles_m * g.tiles_n;
  b = t / per_batch;
  int r = t - b * per_batch;
  if (g.rs_ranks > 0 || g.a_ready) {
    // fused kernels walk the result one row of tiles after the other, so that rows
    // complete (or become available) in a known order
    tm = r / g.tiles_n;
    tn = r - tm * g.tiles_n;
  } else {
    const int group_sz = GROUP_M * g.tiles_n;
    const int gidx = r / group_sz;
    const int first_m = gidx * GROUP_M;
    const int rows_in_group = min(GROUP_M, g.tiles_m - first_m);
    const int rr = r - gidx * group_sz;
    tm = first_m + rr % rows_in_group;
    tn = rr / rows_in_group;
  }
  if (g.m_inter > 1) tm = ((tm % g.m_inter + g.m_src0) % g.m_inter) * (g.tiles_m / g.m_inter) + tm / g.m_inter;
  if (g.m_rot) tm = (tm + g.m_rot) % g.tiles_m;
}

// cta / nctas: index and count of the CTAs that run this body (the fused kernels
// give some CTAs of the grid other roles).  GEMM_THREADS threads.
template <int BN, int STAGES>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& tmA, const CUtensorMap& tmB,
                                             const CUtensorMap* tmC, const CUtensorMap* tmAux,
                                             const CUtensorMap* tmIn,
                                             const GemmDev& g, int cta, int nctas,
                                             uint8_t* smem_raw) {
  using L = GemmSmem<BN, STAGES>;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  // meeting points of the 256 epilogue threads, alternating by tile parity (bounded waits,
  // unlike a named barrier)
  auto epi_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 4 + a); };
  auto in_bar = [&](int w) { return bar_base + 8u * (2 * STAGES + 6 + w); };   // epilogue warp w's input tile has landed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::BAR_OFFSET + L::NUM_BARS * 8);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);     // one arrival per epilogue warp
      mbar_init(epi_bar(a), 8);
    }
    for (int w = 0; w < 8; ++w) mbar_init(in_bar(w), 1);
    *dead = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int out_tiles = g.batch * g.tiles_m * g.tiles_n;
  const int total_tiles = out_tiles * g.split_k;       // work units: unit u = (split u / out_tiles, tile u % out_tiles)
  const int kblocks_all = (g.K + BK - 1) / BK;
  auto k_range = [&](int u, int& kb0, int& kb1) {
    if (g.split_k > 1) {
      kb0 = (u / out_tiles) * g.kb_per_split;
      kb1 = min(kblocks_all, kb0 + g.kb_per_split);
    } else {
      kb0 = 0;
      kb1 = kblocks_all;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t kit = 0;
      bool ok = true;
      int last_ready_chunk = -1;
      for (int t = cta; t < total_tiles && ok; t += nctas) {
        int b, tm, tn, kb0, kb1;
        tile_coords(g, t % out_tiles, b, tm, tn);
        k_range(t, kb0, kb1);
        const int m0 = tm * BM, n0 = tn * BN;
        if (g.a_ready) {
          // rows of this tile may span two chunks when a_ready_rows < 128: wait for the last one
          const int last_row = min(m0 + BM, g.M) - 1;
          for (int ch = m0 / g.a_ready_rows; ch <= last_row / g.a_ready_rows && ok; ++ch) {
            if (ch == last_ready_chunk) continue;
            if (!flag_wait_ge_sys_cta(g.a_ready + ch, g.a_ready_target, dead, g.status, 110)) ok = false;
            last_ready_chunk = ch;
          }
          if (!ok) break;
          // the rows were written through the generic proxy by other CTAs
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb, ++kit) {
          const int s = kit % STAGES;
          const uint32_t ph = (kit / STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, dead, g.status, 100)) { ok = false; break; }
          const uint32_t sA = smem_base + s * L::STAGE_BYTES;
          const uint32_t sB = sA + L::A_BYTES;
          mbar_expect_tx(full_bar(s), L::STAGE_BYTES);
          if (!g.a_mn) {
            tma_load_3d(sA, &tmA, full_bar(s), kb * BK, m0, b);
          } else {
#pragma unroll
            for (int blk = 0; blk < BM / 64; ++blk)
              tma_load_3d(sA + blk * 8192, &tmA, full_bar(s), m0 + blk * 64, kb * BK, b);
          }
          if (!g.b_mn) {
            tma_load_3d(sB, &tmB, full_bar(s), kb * BK, n0, b);
          } else {
#pragma unroll
            for (int blk = 0; blk < BN / 64; ++blk)
              tma_load_3d(sB + blk * 8192, &tmB, full_bar(s), n0 + blk * 64, kb * BK, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, g.a_mn, g.b_mn);
      const uint32_t a_lbo = g.a_mn ? 8192u : 16u;
      const uint32_t b_lbo = g.b_mn ? 8192u : 16u;
      // Shared-memory descriptors: the high word (1024-byte stride between 8-row groups, 128-byte
      // swizzle) is the same for every operand; the low word is address / 16 | leading offset / 16
      // << 16, so a stage or a 16-element K step adds a constant to it.  The single issuing
      // thread has about a hundred cycles per MMA: nothing but two additions belongs in the loop.
      const uint64_t desc_hi = (uint64_t)((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
      const uint32_t a_k16 = (g.a_mn ? 2048u : 32u) >> 4;  // 16 K elements, in 16-byte units
      const uint32_t b_k16 = (g.b_mn ? 2048u : 32u) >> 4;
      const uint32_t a_lo0 = ((smem_base & 0x3FFFFu) >> 4) | ((a_lbo >> 4) << 16);
      const uint32_t b_lo0 = (((smem_base + L::A_BYTES) & 0x3FFFFu) >> 4) | ((b_lbo >> 4) << 16);
      uint32_t kit = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += nctas, ++it) {
        const int acc = it & 1;
        const uint32_t aph = (it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u, dead, g.status, 200)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int kb0, kb1;
        k_range(t, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++kit) {
          const int s = kit % STAGES;
          const uint32_t ph = (kit / STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, dead, g.status, 201)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)s * (L::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)s * (L::STAGE_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            umma_f16(d_tmem, desc_hi | (uint64_t)(a_lo + kk * a_k16), desc_hi | (uint64_t)(b_lo + kk * b_k16), idesc,
                     (kb != kb0 || kk != 0) ? 1u : 0u);
          umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp >= 4) {
#include "gemm_tc_epilogue.inc"
  }

  // A role that gave up leaves copies in flight; give them time to land before
  // the shared memory and TMEM are released.
  if (*dead) __nanosleep(100000);
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace cgk
