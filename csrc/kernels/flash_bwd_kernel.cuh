// Device code of the Flash-Attention-2 backward pass (see flash_bwd.cu for the
// description and the host side).
#pragma once
#include "sm100.cuh"

namespace cgk {


struct FlashBwdDev {
  int B, Hq, Hk, Tq, Tk;
  float scale, scale_log2;
  int causal, window;
  const float* alibi;
  const float* lse;     // [B, Hq, Tq]
  const float* delta;   // [B, Hq, Tq]
  float* dq_accum;      // [B, Tq, Hq, D] fp32
  __nv_bfloat16* dK;
  long long dk_bs, dk_ts, dk_hs;
  __nv_bfloat16* dV;
  long long dv_bs, dv_ts, dv_hs;
  int* status;
};

template <int D>
struct BwdCfg {
  static constexpr int BM = 128;  // query rows per step
  static constexpr int BN = 128;  // keys per CTA
  static constexpr int DB = D / 64;
  static constexpr int TILE_BYTES = 128 * D * 2;   // K, V, Q, dO tiles
  static constexpr int PS_BYTES = BM * BN * 2;     // P and dS tiles
  static constexpr int STAGES = (D == 64) ? 3 : 1;   // Q / dO slots: a slot is held from a step's S / dP until its dK / dV
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_QDO = OFF_V + TILE_BYTES;            // [STAGES][Q, dO]
  static constexpr int OFF_P = OFF_QDO + STAGES * 2 * TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + PS_BYTES;
  // fp32 staging of the dQ tile for the bulk reduction: [D/32][128 rows][32 floats].
  // head_dim 128 has no shared memory left and reuses the P / dS tiles, which are
  // idle between the end of a step's MMAs and the next step's P / dS.
  static constexpr int DQS_BYTES = 128 * D * 4;
  static constexpr bool DQS_ALIAS = (D == 128);
  static constexpr int OFF_DQS = DQS_ALIAS ? OFF_P : OFF_DS + PS_BYTES;
  static constexpr int OFF_BAR = OFF_DS + PS_BYTES + (DQS_ALIAS ? 0 : DQS_BYTES);
  // kv_full, full[STAGES], empty[STAGES], sdp_full, pds_ready, dq_full, dq_drained, sdp_consumed, pds_free
  static constexpr int NUM_BARS = 1 + 2 * STAGES + 6;
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
  static constexpr int TMEM_S = 0;
  static constexpr int TMEM_DP = 128;
  static constexpr int TMEM_DV = 256;
  static constexpr int TMEM_DK = 256 + D;
  // head_dim 64 leaves room for a dQ tile of its own, so the next step's S / dP
  // MMAs overlap the draining of dQ; head_dim 128 fills TMEM and dQ reuses the
  // columns of S.
  static constexpr bool DQ_ALIAS = (256 + 3 * D > 512);
  static constexpr int TMEM_DQ = DQ_ALIAS ? TMEM_S : 256 + 2 * D;
  static constexpr int TMEM_COLS = 512;
  static_assert(TOTAL <= 227 * 1024, "flash backward: shared memory budget of one CTA exceeded");
};

// Rewrites one thread's 64 S columns at s_tmem as final scores in the log2 domain: product * scale
// + ALiBi bias where the key is visible, -inf elsewhere.  Column i is visible iff
// (unsigned)(rel0 + i) <= span and the row sees any key at all.  Out of line: only tiles on a mask
// edge or with a bias come here, and the hot row loop stays short.
__device__ __noinline__ void flash_bwd_mask_scores(uint32_t s_tmem, float scale_log2, float slope,
                                                   float bias0, int rel0, unsigned span, bool none) {
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
    __syncwarp();
    tmem_ld32(s_tmem + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int idx = c * 32 + i;
      const float sc = fmaf(__uint_as_float(r[i]), scale_log2, fmaf(slope, (float)idx, bias0));
      const bool vis = ((unsigned)(rel0 + idx) <= span) && !none;
      r[i] = __float_as_uint(vis ? sc : -INFINITY);
    }
    tmem_st32(s_tmem + c * 32, r);
  }
  tmem_st_wait();
}

// Warp roles (512 threads): warp 0 TMA producer, warps 1 and 3 MMA issuers, warp 2 TMEM allocator,
// warps 4..11 compute P / dS (thread = query row x half of the keys), warps 12..15 drain the
// dQ tile into the fp32 accumulator with bulk tensor reductions.  With 512 threads every thread
// has 128 registers, which each role fits; no register reallocation is needed.
template <int D>
__global__ void __launch_bounds__(512, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQ, const FlashBwdDev p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  const uint32_t kv_full = bar0;
  auto full_bar = [&](int s) { return bar0 + 8u * (1 + s); };
  auto empty_bar = [&](int s) { return bar0 + 8u * (1 + C::STAGES + s); };
  const uint32_t sdp_full = bar0 + 8u * (1 + 2 * C::STAGES);
  const uint32_t pds_ready = sdp_full + 8;
  const uint32_t dq_full = sdp_full + 16;
  const uint32_t dq_drained = sdp_full + 24;
  const uint32_t sdp_consumed = sdp_full + 32;
  const uint32_t pds_free = sdp_full + 40;     // the MMAs that read this step's P / dS tiles are done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::NUM_BARS * 8);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int k0 = kt * C::BN;
  const int off = p.Tk - p.Tq;
  const int group = p.Hq / p.Hk;
  const int nq = (p.Tq + C::BM - 1) / C::BM;
  // query tiles [i_lo, i_hi) that can see keys [k0, k0 + BN)
  int i_lo = 0, i_hi = nq;
  if (p.causal) {
    int first_q = k0 - off;  // smallest q with q + off >= k0
    i_lo = first_q > 0 ? first_q / C::BM : 0;
  } else if (p.window >= 0) {
    int first_q = k0 - off - p.window;
    i_lo = first_q > 0 ? first_q / C::BM : 0;
  }
  if (p.window >= 0) {
    long long last_q = (long long)k0 + C::BN - 1 - off + p.window;  // largest q with q + off - w <= key
    if (last_q < 0) i_hi = 0;
    else if (last_q / C::BM + 1 < i_hi) i_hi = (int)(last_q / C::BM) + 1;
  }
  if (i_lo > i_hi) i_lo = i_hi;
  const int steps_per_head = i_hi - i_lo;
  const int total_steps = steps_per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 8);          // one arrival per warp
    mbar_init(dq_full, 1);
    mbar_init(pds_free, 2);           // the dV / dK issuer and the dQ issuer
    mbar_init(dq_drained, 4);
    mbar_init(sdp_consumed, 8);
    *dead = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_holder), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
    if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0 && total_steps > 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        mbar_expect_tx(kv_full, 2 * C::TILE_BYTES);
#pragma unroll
        for (int db = 0; db < C::DB; ++db) {
          tma_load_4d(sbase + C::OFF_K + db * (C::BN * 128), &tmK, kv_full, db * 64, hk, k0, b);
          tma_load_4d(sbase + C::OFF_V + db * (C::BN * 128), &tmV, kv_full, db * 64, hk, k0, b);
        }
        for (int n = 0; n < total_steps; ++n) {
          const int g = n / steps_per_head, i = i_lo + n % steps_per_head;
          const int h = hk * group + g;
          const int s = n % C::STAGES;
          const uint32_t ph = (n / C::STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, dead, p.status, 2100)) break;
          mbar_expect_tx(full_bar(s), 2 * C::TILE_BYTES);
          const uint32_t qa = sbase + C::OFF_QDO + s * 2 * C::TILE_BYTES;
#pragma unroll
          for (int db = 0; db < C::DB; ++db) {
            tma_load_4d(qa + db * (C::BM * 128), &tmQ, full_bar(s), db * 64, h, i * C::BM, b);
            tma_load_4d(qa + C::TILE_BYTES + db * (C::BM * 128), &tmDO, full_bar(s), db * 64, h,
                        i * C::BM, b);
          }
        }
      }
    } else {
      // ------------------------------- MMA issuers -------------------------------
      // Three issuing threads: warp 1 issues S = Q K^T and dP = dO V^T of every step, warp 3 the
      // two products over the query rows (dV = P^T dO, dK = dS^T Q), warp 2 dQ = dS K.  One thread
      // issuing all 32 to 40 MMAs of a step was the kernel's critical path (some seventy cycles
      // per MMA, hundreds per barrier wait), and the P / dS tiles cannot be rewritten before the
      // last of the three products has read them.
      if (lane == 0 && total_steps > 0) {
        const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S, dP: both K-major
        const uint32_t idesc_kv = make_idesc_bf16(128, D, 1, 1);    // dV, dK: A and B MN-major
        const uint32_t idesc_q = make_idesc_bf16(128, D, 0, 1);     // dQ: A K-major, B MN-major
        // shared-memory descriptors: one high word for all operands (1024-byte stride between
        // 8-row groups, 128-byte swizzle); the low word = address / 16 | leading offset / 16 << 16
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t LBO_K = (16u >> 4) << 16;               // K-major
        constexpr uint32_t LBO_MN = ((128u * 128u) >> 4) << 16;    // MN-major: 64-wide blocks 128 rows x 128 B apart
        auto desc = [&](uint32_t lo32) -> uint64_t { return ((uint64_t)DESC_HI << 32) | (uint64_t)lo32; };
        auto lo16 = [&](uint32_t off) -> uint32_t { return ((sbase + off) & 0x3FFFFu) >> 4; };
        const uint32_t k_lo = lo16(C::OFF_K), v_lo = lo16(C::OFF_V), p_lo = lo16(C::OFF_P), ds_lo = lo16(C::OFF_DS);
        const uint32_t qdo_lo = lo16(C::OFF_QDO);
        bool ok = mbar_wait(kv_full, 0, dead, p.status, 2200);
        if (warp == 1) {
          for (int n = 0; n < total_steps && ok; ++n) {
            const int s = n % C::STAGES;
            if (!mbar_wait(full_bar(s), (n / C::STAGES) & 1u, dead, p.status, 2204)) { ok = false; break; }
            if (n > 0) {
              if (C::DQ_ALIAS) {
                // the S columns hold dQ of step n - 1 until the drain warps have read it
                if (!mbar_wait(dq_drained, (n - 1) & 1u, dead, p.status, 2205)) { ok = false; break; }
              } else {
                // S / dP of step n - 1 only have to be in registers
                if (!mbar_wait(sdp_consumed, (n - 1) & 1u, dead, p.status, 2206)) { ok = false; break; }
              }
            }
            tc_fence_after();
            const uint32_t q_lo = (qdo_lo + s * (2 * C::TILE_BYTES >> 4)) | LBO_K;
            const uint32_t do_lo = q_lo + (C::TILE_BYTES >> 4);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t o16 = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4;
              umma_f16(tmem_base + C::TMEM_S, desc(q_lo + o16), desc((k_lo | LBO_K) + o16), idesc_s, kk != 0 ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t o16 = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4;
              umma_f16(tmem_base + C::TMEM_DP, desc(do_lo + o16), desc((v_lo | LBO_K) + o16), idesc_s, kk != 0 ? 1u : 0u);
            }
            umma_commit(sdp_full);
          }
        } else if (warp == 3) {
          for (int n = 0; n < total_steps && ok; ++n) {
            const int s = n % C::STAGES;
            // this thread's own wait on the slot: its MMAs read Q and dO
            if (!mbar_wait(full_bar(s), (n / C::STAGES) & 1u, dead, p.status, 2201)) { ok = false; break; }
            if (!mbar_wait(pds_ready, n & 1u, dead, p.status, 2203)) { ok = false; break; }
            tc_fence_after();
            const uint32_t q_lo = (qdo_lo + s * (2 * C::TILE_BYTES >> 4)) | LBO_MN;
            const uint32_t do_lo = q_lo + (C::TILE_BYTES >> 4);
            // reduction dimension = the 128 query rows, 16 per MMA: 16 rows x 128 B = 2048 B
#pragma unroll
            for (int kk = 0; kk < C::BM / 16; ++kk)
              umma_f16(tmem_base + C::TMEM_DV, desc((p_lo | LBO_MN) + kk * 128u), desc(do_lo + kk * 128u), idesc_kv,
                       (n > 0 || kk != 0) ? 1u : 0u);
#pragma unroll
            for (int kk = 0; kk < C::BM / 16; ++kk)
              umma_f16(tmem_base + C::TMEM_DK, desc((ds_lo | LBO_MN) + kk * 128u), desc(q_lo + kk * 128u), idesc_kv,
                       (n > 0 || kk != 0) ? 1u : 0u);
            umma_commit(empty_bar(s));
            umma_commit(pds_free);
          }
        } else {
          for (int n = 0; n < total_steps && ok; ++n) {
            if (!mbar_wait(pds_ready, n & 1u, dead, p.status, 2207)) { ok = false; break; }
            if (!C::DQ_ALIAS && n > 0 &&
                !mbar_wait(dq_drained, (n - 1) & 1u, dead, p.status, 2202)) { ok = false; break; }
            tc_fence_after();
            // dQ = dS K: reduction over the 128 keys; A = dS K-major, B = K MN-major
#pragma unroll
            for (int kk = 0; kk < C::BN / 16; ++kk) {
              const uint32_t ao16 = (uint32_t)((kk >> 2) * (128 * 128) + (kk & 3) * 32) >> 4;
              umma_f16(tmem_base + C::TMEM_DQ, desc((ds_lo | LBO_K) + ao16), desc((k_lo | LBO_MN) + kk * 128u), idesc_q,
                       kk != 0 ? 1u : 0u);
            }
            umma_commit(dq_full);
            umma_commit(pds_free);
          }
        }
      }
    }
  } else if (warp < 12) {
#include "flash_bwd_compute.inc"
  } else {
    // ------------------------------- dQ drain -------------------------------
    // TMEM -> registers -> swizzled fp32 staging tile -> one bulk tensor reduction
    // (add) per 32 columns into the fp32 accumulator.  Rows past the end of the
    // sequence are clipped by the tensor map.
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const bool leader = (threadIdx.x == 384);
    bool ok = true;
    for (int n = 0; n < total_steps && ok; ++n) {
      const int g = n / steps_per_head, i = i_lo + n % steps_per_head;
      const int h = hk * group + g;
      if (!mbar_wait(dq_full, n & 1u, dead, p.status, 2301)) { ok = false; break; }
      // where the staging tile overlays the P / dS tiles, dV and dK must have read them too
      if (C::DQS_ALIAS && !mbar_wait(pds_free, n & 1u, dead, p.status, 2304)) { ok = false; break; }
      tc_fence_after();
      if (!C::DQS_ALIAS && n > 0) {
        // the previous step's reduction must have read the staging tile; it had a whole step for it
        if (leader) tma_store_wait_read<0>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_base + C::TMEM_DQ + c * 32 + lane_sel, r);
        tmem_ld_wait();
        uint8_t* tile = smem + C::OFF_DQS + c * (128 * 128);
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4)
          *reinterpret_cast<uint4*>(tile + sw128_offset(row, q4)) =
              make_uint4(r[4 * q4], r[4 * q4 + 1], r[4 * q4 + 2], r[4 * q4 + 3]);
      }
      tc_fence_before();
      if (!C::DQS_ALIAS) mbar_arrive_warp(dq_drained);   // the TMEM tile is free again
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (leader) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c)
          tma_reduce_add_3d(&tmDQ, sbase + C::OFF_DQS + c * (128 * 128), h * D + c * 32, i * C::BM, b);
        tma_store_commit();
        if (C::DQS_ALIAS) tma_store_wait_read<0>();
      }
      if (C::DQS_ALIAS) {
        // the staging tile overlays the P / dS tiles: they are free once the reduction has read it
        asm volatile("bar.sync 1, 128;" ::: "memory");
        mbar_arrive_warp(dq_drained);
      }
    }
    if (leader) tma_store_wait_all<0>();
  }

  if (*dead) __nanosleep(100000);
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace cgk
