// Flash-Attention-2 forward on tcgen05 tensor cores.
//
// One CTA owns 256 query rows (two 128-row tiles) of one (batch, head) and walks
// the key/value sequence in tiles of 128.  Per tile and per query tile:
//     S = Q K^T            tcgen05.mma, fp32 accumulator in TMEM (128 columns)
//     P = exp2(S*c - m)    softmax warpgroup: tcgen05.ld, online max / sum,
//                          bf16 P written to 128B-swizzled shared memory
//     O += P V             tcgen05.mma, O accumulator stays in TMEM for the
//                          whole key loop; it is rescaled in place only when a
//                          row maximum grows by more than 2^8 (the final 1/l
//                          normalisation makes a stale maximum exact)
// Warp roles: 0 = TMA producer, 1 and 3 = MMA issuers of query tile 0 and 1, 2 = TMEM allocator,
// 4..7 = softmax warpgroup of query tile 0, 8..11 = of query tile 1.  The two
// query tiles share every K/V tile, which halves the L2 -> shared traffic.
// A softmax thread owns one row: it takes the 128 scores of a key tile into
// registers and frees the S accumulator at once, so that Q K^T of the next key
// tile runs on the tensor cores while this tile's exponentials are computed.
// Masked / biased tiles (the diagonal of a causal mask, a window edge, ALiBi)
// first rewrite S in TMEM with the final scores in a separate, rarely entered
// function; every tile then takes the one short row loop (three-input maxima,
// packed two-wide fp32 multiply-adds and sums), which keeps the hot code small.
//
// Supports causal masking (bottom-right aligned when Tq != Tk), a sliding window
// |k - q| <= w, ALiBi slopes, GQA/MQA (kv head = h * Hk / Hq), head_dim 64 / 128.
// Layout [batch, seq, heads, head_dim] with arbitrary (16-byte aligned) strides,
// LSE [batch, heads, seq] as in the reference (include/cg_flash_attn.h:54-57,81).
//
// Reference counterparts: flash_attn_fwd_kernel (src/cuda/flash_attn_kernels.c:39-211),
// its host simulation (:261-396) and cg_flash_attention_forward_cpu
// (src/attention/flash_attn.c:17-152).
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cgk {


struct FlashFwdDev {
  int B, Hq, Hk, Tq, Tk;
  float scale_log2;        // softmax scale * log2(e)
  int causal;
  int window;              // < 0: none
  const float* alibi;      // [Hq] slopes or null
  __nv_bfloat16* O;
  long long o_bs, o_ts, o_hs;  // element strides of O: batch, token, head
  float* lse;              // [B, Hq, Tq] or null
  int* status;
};

template <int D>
struct FwdCfg {
  static constexpr int BM = 128;          // rows per query tile
  static constexpr int BN = 128;          // keys per tile
  static constexpr int DB = D / 64;       // 64-column blocks per row
  static constexpr int Q_TILE_BYTES = BM * D * 2;
  static constexpr int KV_TILE_BYTES = BN * D * 2;
  static constexpr int P_TILE_BYTES = BM * BN * 2;
  static constexpr int RING = (D == 64) ? 4 : 3;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + 2 * Q_TILE_BYTES;
  static constexpr int OFF_P = OFF_KV + RING * KV_TILE_BYTES;
  static constexpr int OFF_BAR = OFF_P + 2 * P_TILE_BYTES;
  // barriers: q_full, full[RING], empty[RING], s_full[2], p_ready[2], o_done[2], s_free[2], exp_done[2]
  static constexpr int NUM_BARS = 1 + 2 * RING + 10;
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
  static constexpr int TMEM_S0 = 0;
  static constexpr int TMEM_O0 = 256;
  static constexpr int TMEM_COLS = 512;
};

// Rewrites one thread's S row (128 fp32 columns at s_tmem) as final scores in the log2 domain:
// product * scale + ALiBi bias where the key is visible, -inf elsewhere.  Column i is visible iff
// (unsigned)(rel0 + i) <= span and the row sees any key at all.  Kept out of line: only tiles on
// a mask edge or with a bias come here, and the hot row loop stays short.
__device__ __noinline__ void flash_mask_scores(uint32_t s_tmem, float scale_log2, float slope, float bias0,
                                               int rel0, unsigned span, bool none) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
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

template <int D>
__global__ void __launch_bounds__(384, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashFwdDev p) {
  using C = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  const uint32_t q_full = bar0;
  auto full_bar = [&](int s) { return bar0 + 8u * (1 + s); };
  auto empty_bar = [&](int s) { return bar0 + 8u * (1 + C::RING + s); };
  auto s_full = [&](int t) { return bar0 + 8u * (1 + 2 * C::RING + t); };
  auto p_ready = [&](int t) { return bar0 + 8u * (1 + 2 * C::RING + 2 + t); };
  auto o_done = [&](int t) { return bar0 + 8u * (1 + 2 * C::RING + 4 + t); };
  auto s_free = [&](int t) { return bar0 + 8u * (1 + 2 * C::RING + 6 + t); };
  auto exp_done = [&](int t) { return bar0 + 8u * (1 + 2 * C::RING + 8 + t); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::NUM_BARS * 8);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = (int)(((long long)h * p.Hk) / p.Hq);
  const int q0 = qblk * 2 * C::BM;
  const int off = p.Tk - p.Tq;  // causal alignment: key k visible to query q iff k <= q + off

  // key-tile range [lo, hi_t) per query tile
  const int nkv = (p.Tk + C::BN - 1) / C::BN;
  int lo = 0;
  if (p.window >= 0) {
    int first = q0 + off - p.window;
    lo = first > 0 ? first / C::BN : 0;
  }
  int hi_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q_begin = q0 + t * C::BM;
    int q_end = q_begin + C::BM;
    if (q_end > p.Tq) q_end = p.Tq;
    int hi = nkv;
    if (q_begin >= p.Tq) {
      hi = lo;  // tile entirely beyond the sequence
    } else {
      long long last_key = (long long)p.Tk - 1;
      if (p.causal) last_key = min(last_key, (long long)q_end - 1 + off);
      if (p.window >= 0 && !p.causal) last_key = min(last_key, (long long)q_end - 1 + off + p.window);
      hi = last_key < 0 ? 0 : (int)(last_key / C::BN) + 1;
      if (hi > nkv) hi = nkv;
      if (hi < lo) hi = lo;
    }
    hi_t[t] = hi;
  }
  const int hi = max(hi_t[0], hi_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::RING; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 2); }   // two issuers release a slot
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1); mbar_init(p_ready(t), 4); mbar_init(o_done(t), 1); mbar_init(s_free(t), 4);   // one arrival per softmax warp
      mbar_init(exp_done(t), 4);
    }
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

  // The softmax warpgroups hold a whole S row in registers; the producer / MMA /
  // allocator warpgroup gives its share of the register file to them.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
   if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && hi > lo) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * C::Q_TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int db = 0; db < C::DB; ++db)
          tma_load_4d(sbase + C::OFF_Q + t * C::Q_TILE_BYTES + db * (C::BM * 128), &tmQ, q_full,
                      db * 64, h, q0 + t * C::BM, b);
      uint32_t n = 0;  // ring counter
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* tm, int j) {
        const int s = n % C::RING;
        const uint32_t ph = (n / C::RING) & 1u;
        if (!mbar_wait(empty_bar(s), ph ^ 1u, dead, p.status, 1100)) { ok = false; return; }
        mbar_expect_tx(full_bar(s), C::KV_TILE_BYTES);
#pragma unroll
        for (int db = 0; db < C::DB; ++db)
          tma_load_4d(sbase + C::OFF_KV + s * C::KV_TILE_BYTES + db * (C::BN * 128), tm,
                      full_bar(s), db * 64, hk, j * C::BN, b);
        ++n;
      };
      // order must match the consumer's release order: K_lo, then (K_{j+1}, V_j) per j
      load_tile(&tmK, lo);
      for (int j = lo; j < hi && ok; ++j) {
        if (j + 1 < hi) load_tile(&tmK, j + 1);
        if (ok) load_tile(&tmV, j);
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------- MMA issuers -------------------------------
    // One issuing thread per query tile (warp 1: tile 0, warp 3: tile 1).  A single thread
    // issuing for both tiles was the kernel's critical path: every MMA costs it some tens of
    // cycles and every barrier wait a few hundred, against 32 to 64 tensor cycles per MMA.
    // Both walk the K/V ring in the producer's order; a slot is free again when both have
    // released it (after their MMAs on it, or at once when their tile does not use it).
    if (lane == 0 && hi > lo) {
      const int t = warp == 1 ? 0 : 1;
      const uint32_t idesc_s = make_idesc_bf16(C::BM, C::BN, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(C::BM, D, 0, 1);
      // shared-memory descriptors: the high word is the same for every operand of this kernel
      // (1024-byte stride between 8-row groups, 128-byte swizzle); the low word holds the
      // address / 16 and the leading-dimension offset / 16, so stepping along a tile adds a
      // compile-time constant to it
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t LBO_K = (16u >> 4) << 16;                  // K-major operands
      constexpr uint32_t LBO_V = ((uint32_t)(C::BN * 128) >> 4) << 16;   // V: MN-major, 64-wide head_dim blocks
      auto desc = [&](uint32_t lo32) -> uint64_t {
        return ((uint64_t)DESC_HI << 32) | (uint64_t)lo32;
      };
      const uint32_t q_lo = (((sbase + C::OFF_Q + t * C::Q_TILE_BYTES) & 0x3FFFFu) >> 4) | LBO_K;
      const uint32_t p_lo = (((sbase + C::OFF_P + t * C::P_TILE_BYTES) & 0x3FFFFu) >> 4) | LBO_K;
      const uint32_t kv_lo = ((sbase + C::OFF_KV) & 0x3FFFFu) >> 4;
      const uint32_t s_tm = tmem_base + C::TMEM_S0 + t * 128;
      const uint32_t o_tm = tmem_base + C::TMEM_O0 + t * D;
      const int my_hi = hi_t[t];
      bool ok = true;
      uint32_t n = 0;            // ring counter (consumption order)
      auto issue_s = [&](uint32_t slot) {
        const uint32_t k_lo = (kv_lo + slot * (C::KV_TILE_BYTES >> 4)) | LBO_K;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o16 = (uint32_t)((kk >> 2) * (C::BM * 128) + (kk & 3) * 32) >> 4;
          umma_f16(s_tm, desc(q_lo + o16), desc(k_lo + o16), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full(t));
      };
      auto issue_pv = [&](uint32_t slot, bool acc) {
        const uint32_t v_lo = (kv_lo + slot * (C::KV_TILE_BYTES >> 4)) | LBO_V;
#pragma unroll
        for (int kk = 0; kk < C::BN / 16; ++kk) {
          // A = P: K-major, 64-key blocks of [128 rows x 128 B]; B = V: 16 key rows per step
          const uint32_t ao16 = (uint32_t)((kk >> 2) * (C::BM * 128) + (kk & 3) * 32) >> 4;
          const uint32_t bo16 = (uint32_t)(kk * 2048) >> 4;
          umma_f16(o_tm, desc(p_lo + ao16), desc(v_lo + bo16), idesc_o, (acc || kk != 0) ? 1u : 0u);
        }
        umma_commit(o_done(t));
      };
      // ring order (the producer's): K_lo, then (K_{j+1}, V_j) per key tile j
      auto take_slot = [&](int where) -> uint32_t {
        const int s = n % C::RING;
        if (!mbar_wait(full_bar(s), (n / C::RING) & 1u, dead, p.status, where)) { ok = false; return 0u; }
        tc_fence_after();
        ++n;
        return (uint32_t)s;
      };
      auto release = [&](uint32_t slot, bool used) {
        if (used) umma_commit(empty_bar(slot));   // once the MMAs that read it are done
        else mbar_arrive(empty_bar(slot));
      };
      if (!mbar_wait(q_full, 0, dead, p.status, 1200)) ok = false;
      if (ok) {
        const uint32_t s = take_slot(1201);
        if (ok) {
          if (lo < my_hi) issue_s(s);
          release(s, lo < my_hi);
        }
      }
      uint32_t fcount = 0, pcount = 0;
      for (int j = lo; j < hi && ok; ++j) {
        // S of the next key tile as soon as the softmax warps hold this tile's scores in registers
        if (j + 1 < hi) {
          const uint32_t ks = take_slot(1220);
          if (!ok) break;
          const bool use = j + 1 < my_hi;
          if (use) {
            if (!mbar_wait(s_free(t), fcount & 1u, dead, p.status, 1240 + t)) { ok = false; break; }
            ++fcount;
            tc_fence_after();
            issue_s(ks);
          }
          release(ks, use);
        }
        // O += P V of this key tile once P is in shared memory
        const uint32_t vs = take_slot(1230);
        if (!ok) break;
        const bool use = j < my_hi;
        if (use) {
          if (!mbar_wait(p_ready(t), pcount & 1u, dead, p.status, 1210 + t)) { ok = false; break; }
          ++pcount;
          tc_fence_after();
          issue_pv(vs, j > lo);
        }
        release(vs, use);
      }
    }
   }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // --------------------------- softmax warpgroups ---------------------------
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;          // row inside the query tile == TMEM lane
    const int qpos = q0 + t * C::BM + row;
    const int my_hi = hi_t[t];
    const int n_other = hi_t[1 - t] - lo;      // steps of the other warpgroup
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_tmem = tmem_base + C::TMEM_S0 + t * 128 + lane_sel;
    const uint32_t o_tmem = tmem_base + C::TMEM_O0 + t * D + lane_sel;
    uint8_t* p_smem = smem + C::OFF_P + t * C::P_TILE_BYTES;
    const float slope = p.alibi ? p.alibi[h] * 1.4426950408889634f : 0.0f;
    const int qk = qpos + off;                 // last visible key under the causal mask
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    uint32_t it = 0;
    for (int j = lo; j < my_hi && ok; ++j, ++it) {
      if (!mbar_wait(s_full(t), it & 1u, dead, p.status, 1300 + t)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * C::BN;
      // does any element of this tile need masking?  (warp-uniform)
      const int tile_q_lo = q0 + t * C::BM + off, tile_q_hi = tile_q_lo + C::BM - 1;
      bool need_mask = (k0 + C::BN > p.Tk);
      if (p.causal) need_mask |= (k0 + C::BN - 1 > tile_q_lo);
      if (p.window >= 0) need_mask |= (k0 < tile_q_hi - p.window) || (!p.causal && k0 + C::BN - 1 > tile_q_lo + p.window);
      // Interior tiles (no mask, no bias) use the raw products; the others are first rewritten in
      // TMEM as final log2-domain scores (-inf where masked), after which the multiplier is 1.
      const bool fast = !need_mask && !p.alibi && p.scale_log2 > 0.0f;
      if (!fast) {
        // Row-wise visible key range [klo, khi] (empty when khi < klo).  The ALiBi bias of
        // column i of the tile is bias0 + slope * i.
        int klo = 0, khi = p.Tk - 1;
        if (p.causal) khi = min(khi, qk);
        if (p.window >= 0) { klo = max(klo, qk - p.window); khi = min(khi, qk + p.window); }
        const unsigned span = khi >= klo ? (unsigned)(khi - klo) : 0u;
        const float bias0 = p.alibi ? slope * (float)(k0 - qk) : 0.0f;
        flash_mask_scores(s_tmem, p.scale_log2, slope, bias0, k0 - klo, span, khi < klo);
      }
      const float mul = fast ? p.scale_log2 : 1.0f;
      // The whole S row (128 fp32) comes into registers with four loads in flight and one wait;
      // the accumulator is then free for Q K^T of the next key tile.
      uint32_t r[4][32];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(s_free(t));
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        m0 = fmax3(m0, __uint_as_float(r[0][i]), __uint_as_float(r[0][i + 1]));
        m1 = fmax3(m1, __uint_as_float(r[1][i]), __uint_as_float(r[1][i + 1]));
        m2 = fmax3(m2, __uint_as_float(r[2][i]), __uint_as_float(r[2][i + 1]));
        m3 = fmax3(m3, __uint_as_float(r[3][i]), __uint_as_float(r[3][i + 1]));
      }
      const float mx = fmaxf(m, fmax3(m0, m1, fmaxf(m2, m3)) * mul);   // mul > 0
      // keep a stale maximum unless it grew by more than 2^8
      float m_use = (mx > m + 8.0f) ? mx : m;
      if (m == -INFINITY) m_use = mx;
      const float alpha = (m == -INFINITY) ? 0.0f : fast_exp2(m - m_use);
      const bool changed = (m_use != m);
      // PV of the previous key tile must be done before O is rescaled and before
      // P is overwritten
      if (j > lo) {
        if (!mbar_wait(o_done(t), (it - 1) & 1u, dead, p.status, 1310 + t)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, changed)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t ro[32];
            __syncwarp();
            tmem_ld32(o_tmem + c * 32, ro);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
            tmem_st32(o_tmem + c * 32, ro);
          }
          tmem_st_wait();
        }
      }
      l *= alpha;
      m = m_use;
      const float neg_m = (m == -INFINITY) ? 0.0f : -m;
      // The SM computes 16 exponentials per clock, 1024 clocks for a 128 x 128 tile, which is the
      // longest stretch of a softmax step.  The two warpgroups therefore take turns at it (tile 0's
      // step i, tile 1's step i, tile 0's step i + 1, ...): one exponentiates while the other
      // loads scores, finds maxima and waits for the tensor core, instead of both halving each
      // other's rate and then idling together.  A warpgroup that has run out of steps is not
      // waited for.
      if (t == 0) {
        if (it > 0 && (int)it - 1 < n_other &&
            !mbar_wait(exp_done(1), (it - 1) & 1u, dead, p.status, 1330)) { ok = false; break; }
      } else {
        if ((int)it < n_other && !mbar_wait(exp_done(0), it & 1u, dead, p.status, 1331)) { ok = false; break; }
      }
      // P = exp2(score * mul - m), bf16, into the swizzled operand tile
      float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          ffma2(x0, x1, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]), mul, mul, neg_m, neg_m);
          e[i] = fast_exp2(x0);
          e[i + 1] = fast_exp2(x1);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) { fadd2(s0, s1, e[i], e[i + 1]); fadd2(s2, s3, e[i + 2], e[i + 3]); }
        uint8_t* blk = p_smem + (c >> 1) * (C::BM * 128);
        const uint32_t chunk0 = (c & 1) * 4;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v = make_uint4(pack_bf16x2(e[8 * q4], e[8 * q4 + 1]), pack_bf16x2(e[8 * q4 + 2], e[8 * q4 + 3]),
                               pack_bf16x2(e[8 * q4 + 4], e[8 * q4 + 5]), pack_bf16x2(e[8 * q4 + 6], e[8 * q4 + 7]));
          *reinterpret_cast<uint4*>(blk + sw128_offset(row, chunk0 + q4)) = v;
        }
      }
      l += (s0 + s1) + (s2 + s3);
      mbar_arrive_warp(exp_done(t));
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive_warp(p_ready(t));
    }
    // epilogue: O / l -> global, LSE
    const bool have = my_hi > lo;
    if (have && ok) {
      if (!mbar_wait(o_done(t), (it - 1) & 1u, dead, p.status, 1320 + t)) ok = false;
      tc_fence_after();
    }
    const float inv_l = (l > 0.0f) ? 1.0f / l : 0.0f;
    const bool row_ok = qpos < p.Tq;
    __nv_bfloat16* orow = p.O + (long long)b * p.o_bs + (long long)qpos * p.o_ts + (long long)h * p.o_hs;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      if (have && ok) {
        __syncwarp();
        tmem_ld32(o_tmem + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * q4]) * inv_l, __uint_as_float(r[8 * q4 + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(r[8 * q4 + 2]) * inv_l, __uint_as_float(r[8 * q4 + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(r[8 * q4 + 4]) * inv_l, __uint_as_float(r[8 * q4 + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(r[8 * q4 + 6]) * inv_l, __uint_as_float(r[8 * q4 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = v;
        }
      }
    }
    if (row_ok && p.lse) {
      const float lse = (l > 0.0f) ? (m * 0.6931471805599453f + __logf(l)) : INFINITY;
      p.lse[((long long)b * p.Hq + h) * p.Tq + CGK_IDX(qpos, p.Tq)] = lse;
    }
  }

  if (*dead) __nanosleep(100000);
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// 4-D tensor map over [B, T, H, D] (element strides bs, ts, hs; D contiguous),
// box = 64 x 1 x rows x 1.
static int make_qkv_tmap(CUtensorMap* tm, const void* base, int B, int T, int H, int D,
                         long long bs, long long ts, long long hs, int rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)hs * 2, (uint64_t)ts * 2, (uint64_t)bs * 2};
  uint32_t box[4] = {64, 1, (uint32_t)rows, 1};
  return encode_tmap(tm, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, Swz::B128);
}

template <int D>
static int launch_fwd(const cgk_flash_args& a, const FlashFwdDev& p, cudaStream_t st) {
  using C = FwdCfg<D>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_qkv_tmap(&tq, a.q, a.B, a.Tq, a.Hq, D, a.q_bs, a.q_ts, a.q_hs, C::BM))) return rc;
  if ((rc = make_qkv_tmap(&tk, a.k, a.B, a.Tk, a.Hk, D, a.k_bs, a.k_ts, a.k_hs, C::BN))) return rc;
  if ((rc = make_qkv_tmap(&tv, a.v, a.B, a.Tk, a.Hk, D, a.v_bs, a.v_ts, a.v_hs, C::BN))) return rc;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      C::TOTAL));
  dim3 grid((a.Tq + 2 * C::BM - 1) / (2 * C::BM), a.Hq, a.B);
  flash_fwd_kernel<D><<<grid, 384, C::TOTAL, st>>>(tq, tk, tv, p);
  CGK_LAUNCH_CHECK();
  return 0;
}

}  // namespace cgk

using namespace cgk;


CGK_API int cgk_flash_forward(const cgk_flash_args* pa, void* stream) {
  CGK_REQUIRE(pa, "cgk_flash_forward: null args");
  const cgk_flash_args& a = *pa;
  CGK_REQUIRE(a.q && a.k && a.v && a.o, "cgk_flash_forward: null tensor");
  CGK_REQUIRE(a.D == 64 || a.D == 128, "cgk_flash_forward: head_dim %d not supported (64 or 128)", a.D);
  CGK_REQUIRE(a.Hq % a.Hk == 0, "cgk_flash_forward: Hq must be a multiple of Hk");
  CGK_REQUIRE(a.o_hs % 8 == 0 && a.o_ts % 8 == 0 && a.o_bs % 8 == 0 && ((uintptr_t)a.o & 15) == 0,
              "cgk_flash_forward: output strides must be multiples of 8 elements");
  if (a.B == 0 || a.Tq == 0 || a.Hq == 0) return 0;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  FlashFwdDev p;
  p.B = a.B; p.Hq = a.Hq; p.Hk = a.Hk; p.Tq = a.Tq; p.Tk = a.Tk;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.causal = a.causal; p.window = a.window;
  p.alibi = a.alibi_slopes;
  p.O = (__nv_bfloat16*)a.o; p.o_bs = a.o_bs; p.o_ts = a.o_ts; p.o_hs = a.o_hs;
  p.lse = a.lse;
  p.status = device_status(dev);
  if (a.D == 64) return launch_fwd<64>(a, p, (cudaStream_t)stream);
  return launch_fwd<128>(a, p, (cudaStream_t)stream);
}

CGK_BOUNDS_READER(flash_fwd)
