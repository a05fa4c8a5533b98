// Flash-Attention-2 backward on tcgen05 tensor cores.
//
// One CTA owns one tile of 128 keys of one (batch, kv head).  K and V stay in
// shared memory; dK and dV accumulate in TMEM over every query tile that sees
// these keys and over every query head of the GQA group, so they need no
// atomics.  Per query tile (128 rows):
//     S  = Q K^T, dP = dO V^T            two MMAs into TMEM
//     P  = exp2(S*c - LSE), dS = P*(dP - delta)*scale      (thread = query row)
//          both written once, bf16, to a 128B-swizzled [rows][keys] tile that
//          serves as a K-major operand (dQ = dS K) and, read the other way, as
//          an MN-major operand (dV += P^T dO, dK += dS^T Q)
//     dQ tile -> TMEM (over the columns S used) -> red.global.add.v4.f32 into an
//          fp32 accumulator that a last kernel casts to bf16
// delta = rowsum(dO * O) comes from a pre-pass.  Fully masked tiles are skipped.
//
// Reference counterparts: flash_attn_bwd_sim (src/cuda/flash_attn_kernels.c:401-525,
// materialises the full N_q x N_k matrices on the host) and
// cg_flash_attention_backward_cpu (src/attention/flash_attn.c), whose split-K
// variant is inexact.
#include "../../include/cogito_kernels.h"
#include "host_common.h"
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
  static constexpr int STAGES = (D == 64) ? 2 : 1;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_QDO = OFF_V + TILE_BYTES;            // [STAGES][Q, dO]
  static constexpr int OFF_P = OFF_QDO + STAGES * 2 * TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + PS_BYTES;
  static constexpr int OFF_BAR = OFF_DS + PS_BYTES;
  // kv_full, full[STAGES], empty[STAGES], sdp_full, pds_ready, dq_full, dq_drained
  static constexpr int NUM_BARS = 1 + 2 * STAGES + 4;
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
  static constexpr int TMEM_S = 0;      // S, later dQ
  static constexpr int TMEM_DP = 128;
  static constexpr int TMEM_DV = 256;
  static constexpr int TMEM_DK = 256 + D;
  static constexpr int TMEM_COLS = 512;
};

template <int D>
__global__ void __launch_bounds__(256, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FlashBwdDev p) {
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
    mbar_init(pds_ready, 128);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 128);
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
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && total_steps > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S, dP: both K-major
      const uint32_t idesc_kv = make_idesc_bf16(128, D, 1, 1);    // dV, dK: A and B MN-major
      const uint32_t idesc_q = make_idesc_bf16(128, D, 0, 1);     // dQ: A K-major, B MN-major
      const uint32_t sK = sbase + C::OFF_K, sV = sbase + C::OFF_V;
      const uint32_t sP = sbase + C::OFF_P, sDS = sbase + C::OFF_DS;
      bool ok = mbar_wait(kv_full, 0, dead, p.status, 2200);
      for (int n = 0; n < total_steps && ok; ++n) {
        const int s = n % C::STAGES;
        const uint32_t ph = (n / C::STAGES) & 1u;
        const uint32_t sQ = sbase + C::OFF_QDO + s * 2 * C::TILE_BYTES;
        const uint32_t sDO = sQ + C::TILE_BYTES;
        if (!mbar_wait(full_bar(s), ph, dead, p.status, 2201)) { ok = false; break; }
        // the S columns double as the dQ tile of the previous step
        if (n > 0 && !mbar_wait(dq_drained, (n - 1) & 1u, dead, p.status, 2202)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          umma_f16(tmem_base + C::TMEM_S, make_smem_desc_sw128(sQ + o, 16, 1024),
                   make_smem_desc_sw128(sK + o, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          umma_f16(tmem_base + C::TMEM_DP, make_smem_desc_sw128(sDO + o, 16, 1024),
                   make_smem_desc_sw128(sV + o, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(pds_ready, n & 1u, dead, p.status, 2203)) { ok = false; break; }
        tc_fence_after();
        // reduction dimension = the 128 query rows, 16 per MMA: 16 rows x 128 B = 2048 B;
        // 64-wide blocks of the M/N dimension are 128 rows x 128 B apart
#pragma unroll
        for (int kk = 0; kk < C::BM / 16; ++kk) {
          umma_f16(tmem_base + C::TMEM_DV, make_smem_desc_sw128(sP + kk * 2048, 128 * 128, 1024),
                   make_smem_desc_sw128(sDO + kk * 2048, 128 * 128, 1024), idesc_kv,
                   (n > 0 || kk != 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < C::BM / 16; ++kk) {
          umma_f16(tmem_base + C::TMEM_DK, make_smem_desc_sw128(sDS + kk * 2048, 128 * 128, 1024),
                   make_smem_desc_sw128(sQ + kk * 2048, 128 * 128, 1024), idesc_kv,
                   (n > 0 || kk != 0) ? 1u : 0u);
        }
        // dQ = dS K: reduction over the 128 keys; A = dS K-major, B = K MN-major
#pragma unroll
        for (int kk = 0; kk < C::BN / 16; ++kk) {
          const uint32_t ao = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          umma_f16(tmem_base + C::TMEM_S, make_smem_desc_sw128(sDS + ao, 16, 1024),
                   make_smem_desc_sw128(sK + kk * 2048, 128 * 128, 1024), idesc_q,
                   kk != 0 ? 1u : 0u);
        }
        umma_commit(empty_bar(s));
        umma_commit(dq_full);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ compute warps ------------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    for (int n = 0; n < total_steps && ok; ++n) {
      const int g = n / steps_per_head, i = i_lo + n % steps_per_head;
      const int h = hk * group + g;
      const int qpos = i * C::BM + row;
      const int qk = qpos + off;
      const bool q_ok = qpos < p.Tq;
      const long long stat = ((long long)b * p.Hq + h) * p.Tq + qpos;
      const float lse2 = q_ok ? p.lse[stat] * LOG2E : INFINITY;
      const float dlt = q_ok ? p.delta[stat] : 0.0f;
      const float slope = p.alibi ? p.alibi[h] * LOG2E : 0.0f;
      if (!mbar_wait(sdp_full, n & 1u, dead, p.status, 2300)) { ok = false; break; }
      tc_fence_after();
      const int tile_q_lo = i * C::BM + off, tile_q_hi = tile_q_lo + C::BM - 1;
      bool need_mask = (k0 + C::BN > p.Tk);
      if (p.causal) need_mask |= (k0 + C::BN - 1 > tile_q_lo);
      if (p.window >= 0) need_mask |= (k0 < tile_q_hi - p.window) || (!p.causal && k0 + C::BN - 1 > tile_q_lo + p.window);
#pragma unroll 1
      for (int c = 0; c < C::BN / 32; ++c) {
        uint32_t rs[32], rp[32];
        __syncwarp();
        tmem_ld32(tmem_base + C::TMEM_S + c * 32 + lane_sel, rs);
        tmem_ld32(tmem_base + C::TMEM_DP + c * 32 + lane_sel, rp);
        tmem_ld_wait();
        uint32_t pp[16], ds[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int k = k0 + c * 32 + e + u;
            float sc = __uint_as_float(rs[e + u]) * p.scale_log2;
            if (p.alibi) sc += slope * (float)(k - qk);
            float pr = fast_exp2(sc - lse2);
            if (need_mask) {
              bool vis = k < p.Tk;
              if (p.causal) vis &= (k <= qk);
              if (p.window >= 0) vis &= (k >= qk - p.window) && (k <= qk + p.window);
              if (!vis) pr = 0.0f;
            }
            pv[u] = pr;
            dv[u] = pr * (__uint_as_float(rp[e + u]) - dlt) * p.scale;
          }
          pp[e >> 1] = pack_bf16x2(pv[0], pv[1]);
          ds[e >> 1] = pack_bf16x2(dv[0], dv[1]);
        }
        const uint32_t blk = (c >> 1) * (128 * 128);
        const uint32_t chunk0 = (c & 1) * 4;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t o = blk + sw128_offset(row, chunk0 + q4);
          *reinterpret_cast<uint4*>(smem + C::OFF_P + o) =
              make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(smem + C::OFF_DS + o) =
              make_uint4(ds[4 * q4], ds[4 * q4 + 1], ds[4 * q4 + 2], ds[4 * q4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_ready);
      // drain dQ
      if (!mbar_wait(dq_full, n & 1u, dead, p.status, 2301)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = p.dq_accum + (((long long)b * p.Tq + qpos) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_base + C::TMEM_S + c * 32 + lane_sel, r);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            red_add_f32x4(dq_row + c * 32 + e, __uint_as_float(r[e]), __uint_as_float(r[e + 1]),
                          __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
        }
      }
      tc_fence_before();
      mbar_arrive(dq_drained);
    }
    // dK, dV of this key tile (thread = key row)
    const int kpos = k0 + row;
    const bool k_ok = kpos < p.Tk;
    __nv_bfloat16* dk_row = p.dK + (long long)b * p.dk_bs + (long long)kpos * p.dk_ts + (long long)hk * p.dk_hs;
    __nv_bfloat16* dv_row = p.dV + (long long)b * p.dv_bs + (long long)kpos * p.dv_ts + (long long)hk * p.dv_hs;
    const bool have = total_steps > 0 && ok;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = which ? dk_row : dv_row;
      const uint32_t src = tmem_base + (which ? C::TMEM_DK : C::TMEM_DV) + lane_sel;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (have) {
          __syncwarp();
          tmem_ld32(src + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        if (k_ok) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * q4]), __uint_as_float(r[8 * q4 + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = v;
          }
        }
      }
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

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]; one warp per row.
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                   float* __restrict__ delta, int B, int H, int T, int D,
                                   long long o_bs, long long o_ts, long long o_hs, long long do_bs,
                                   long long do_ts, long long do_hs) {
  const long long total = (long long)B * H * T;
  const int lane = threadIdx.x & 31;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total;
       w += ((long long)gridDim.x * blockDim.x) >> 5) {
    const int t = (int)(w % T);
    const int h = (int)((w / T) % H);
    const int b = (int)(w / ((long long)T * H));
    const __nv_bfloat16* o = O + b * o_bs + t * o_ts + h * o_hs;
    const __nv_bfloat16* d = dO + b * do_bs + t * do_ts + h * do_hs;
    float s = 0.0f;
    for (int c = lane * 2; c < D; c += 64) {
      float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o + c));
      float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(d + c));
      s += a.x * g.x + a.y * g.y;
    }
    s = warp_sum(s);
    if (lane == 0) delta[((long long)b * H + h) * T + t] = s;
  }
}

// dq[b, t, h, :] = bf16(accum[b, t, h, :])
__global__ void flash_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B,
                                     int T, int H, int D, long long bs, long long ts, long long hs) {
  const long long total = (long long)B * T * H * (D / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % (D / 4)) * 4;
    long long r = i / (D / 4);
    const int h = (int)(r % H); r /= H;
    const int t = (int)(r % T);
    const int b = (int)(r / T);
    const float4 v = *reinterpret_cast<const float4*>(acc + (((long long)b * T + t) * H + h) * D + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + b * bs + t * ts + h * hs + c) = o;
  }
}

static int make_tmap4(CUtensorMap* tm, const void* base, int B, int T, int H, int D, long long bs,
                      long long ts, long long hs) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)hs * 2, (uint64_t)ts * 2, (uint64_t)bs * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap(tm, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, Swz::B128);
}

template <int D>
static int launch_bwd(const cgk_flash_args& a, const FlashBwdDev& p, cudaStream_t st) {
  using C = BwdCfg<D>;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tmap4(&tq, a.q, a.B, a.Tq, a.Hq, D, a.q_bs, a.q_ts, a.q_hs))) return rc;
  if ((rc = make_tmap4(&tk, a.k, a.B, a.Tk, a.Hk, D, a.k_bs, a.k_ts, a.k_hs))) return rc;
  if ((rc = make_tmap4(&tv, a.v, a.B, a.Tk, a.Hk, D, a.v_bs, a.v_ts, a.v_hs))) return rc;
  if ((rc = make_tmap4(&tdo, a.d_o, a.B, a.Tq, a.Hq, D, a.o_bs, a.o_ts, a.o_hs))) return rc;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      C::TOTAL));
  dim3 grid((a.Tk + C::BN - 1) / C::BN, a.Hk, a.B);
  flash_bwd_kernel<D><<<grid, 256, C::TOTAL, st>>>(tq, tk, tv, tdo, p);
  CGK_LAUNCH_CHECK();
  return 0;
}

}  // namespace cgk

using namespace cgk;

// Needs args->delta (fp32 [B,Hq,Tq]) and args->dq_accum (fp32 [B,Tq,Hq,D]) as
// scratch; dq_accum is zeroed here.  d_o must have the strides of o.
CGK_API int cgk_flash_backward(const cgk_flash_args* pa, void* stream) {
  CGK_REQUIRE(pa, "cgk_flash_backward: null args");
  const cgk_flash_args& a = *pa;
  CGK_REQUIRE(a.q && a.k && a.v && a.o && a.d_o && a.lse && a.dq && a.dk && a.dv && a.delta && a.dq_accum,
              "cgk_flash_backward: null tensor");
  CGK_REQUIRE(a.D == 64 || a.D == 128, "cgk_flash_backward: head_dim %d not supported (64 or 128)", a.D);
  CGK_REQUIRE(a.Hq % a.Hk == 0, "cgk_flash_backward: Hq must be a multiple of Hk");
  CGK_REQUIRE((a.dq_hs | a.dq_ts | a.dq_bs | a.dk_hs | a.dk_ts | a.dk_bs | a.dv_hs | a.dv_ts | a.dv_bs) % 8 == 0,
              "cgk_flash_backward: gradient strides must be multiples of 8 elements");
  if (a.B == 0 || a.Tq == 0 || a.Hq == 0 || a.Tk == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const long long rows = (long long)a.B * a.Hq * a.Tq;
  {
    long long blocks = (rows * 32 + 255) / 256;
    long long cap = (long long)sm_count(dev) * 16;
    if (blocks > cap) blocks = cap;
    flash_delta_kernel<<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)a.o, (const __nv_bfloat16*)a.d_o,
                                                    a.delta, a.B, a.Hq, a.Tq, a.D, a.o_bs, a.o_ts, a.o_hs,
                                                    a.o_bs, a.o_ts, a.o_hs);
    CGK_LAUNCH_CHECK();
  }
  CGK_CUDA_CHECK(cudaMemsetAsync(a.dq_accum, 0, (size_t)rows * a.D * sizeof(float), st));
  FlashBwdDev p;
  p.B = a.B; p.Hq = a.Hq; p.Hk = a.Hk; p.Tq = a.Tq; p.Tk = a.Tk;
  p.scale = a.scale; p.scale_log2 = a.scale * 1.4426950408889634f;
  p.causal = a.causal; p.window = a.window; p.alibi = a.alibi_slopes;
  p.lse = a.lse; p.delta = a.delta; p.dq_accum = a.dq_accum;
  p.dK = (__nv_bfloat16*)a.dk; p.dk_bs = a.dk_bs; p.dk_ts = a.dk_ts; p.dk_hs = a.dk_hs;
  p.dV = (__nv_bfloat16*)a.dv; p.dv_bs = a.dv_bs; p.dv_ts = a.dv_ts; p.dv_hs = a.dv_hs;
  p.status = device_status(dev);
  int rc = (a.D == 64) ? launch_bwd<64>(a, p, st) : launch_bwd<128>(a, p, st);
  if (rc) return rc;
  {
    long long n = rows * (a.D / 4);
    long long blocks = (n + 255) / 256;
    long long cap = (long long)sm_count(dev) * 16;
    if (blocks > cap) blocks = cap;
    flash_dq_cast_kernel<<<(int)blocks, 256, 0, st>>>(a.dq_accum, (__nv_bfloat16*)a.dq, a.B, a.Tq, a.Hq,
                                                      a.D, a.dq_bs, a.dq_ts, a.dq_hs);
    CGK_LAUNCH_CHECK();
  }
  return 0;
}
