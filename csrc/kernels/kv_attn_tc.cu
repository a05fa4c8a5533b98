// Attention over the paged INT4 KV cache on the tcgen05 tensor cores (head_dim 128).
// Reference counterpart: cg_attention_int4_kv (include/cg_quantize.h, declared only).
//
// One CTA per (key split, kv head, sequence) handles up to NP query rows (the Tq new tokens of
// every query head that shares the kv head) against its slice of the history, 128 keys at a time:
//   1. all threads turn the block's K and V nibbles into bf16 operand tiles in shared memory
//      (128-byte swizzle; the same image serves K as a K-major A operand and V as an MN-major one),
//   2. S^T[128 keys, NP] = K . Q^T           (tcgen05.mma, accumulator in TMEM, keys on the lanes),
//   3. every thread owns one key: scale, mask; row maxima through a row-major copy in shared memory,
//      p = 2^(s - m) written as the K-major B operand P[NP, 128 keys],
//   4. O^T[128 d, NP] = V^T . P^T            (tcgen05.mma), read back and folded into the
//      running, rescaled accumulator in registers.
// The raw bytes of the next block are fetched into registers before the MMAs of the current one are
// waited for.  The nibble -> bf16 conversion leaves the eight elements of every 32-bit word in the
// order 0,4,1,5,2,6,3,7; Q is stored with the same order (the contraction over d does not care) and
// the rows of O^T are mapped back when the partial result is written.
#include <cuda_bf16.h>

#include "host_common.h"
#include "sm100.cuh"
#include "kv_dev.cuh"

namespace cgk {
namespace {

constexpr int KVT_THREADS = 256, KVT_KB = 128, KVT_D = 128;
constexpr uint32_t KVT_TILE = KVT_KB * KVT_D * 2;          // one converted K or V tile: 32 KiB
constexpr uint32_t KVT_HALF = KVT_KB * 128;                // one 64-wide block of a tile: 16 KiB

template <int NP>
struct KvtSmem {
  static constexpr uint32_t Q_BYTES = NP * KVT_D * 2, P_BYTES = NP * KVT_KB * 2;
  static constexpr uint32_t OFF_K = 0, OFF_V = KVT_TILE, OFF_Q = 2 * KVT_TILE, OFF_P = OFF_Q + Q_BYTES;
  static constexpr uint32_t T_STRIDE = KVT_KB + 4;                      // floats per row of the transposed score tile (padded)
  static constexpr uint32_t OFF_T = OFF_P + P_BYTES;                    // float [NP][T_STRIDE]: scores, row-major, for the row maxima
  static constexpr uint32_t OFF_WMAX = OFF_T + NP * T_STRIDE * 4;       // float [3][NP]: new maximum, rescale factor, running maximum per row
  static constexpr uint32_t OFF_LRED = OFF_WMAX + 4 * NP * 4;           // float [4][NP]
  static constexpr uint32_t OFF_BAR = OFF_LRED + 4 * NP * 4;            // two mbarriers
  static constexpr uint32_t OFF_MISC = OFF_BAR + 16;                    // tmem slot, dead flag
  static constexpr uint32_t TOTAL = OFF_MISC + 16 + 1024;               // + slack for the 1 KiB alignment
};

// position p (0..7) of a converted word holds element (p & 1) * 4 + (p >> 1)
__device__ __forceinline__ int kvt_perm(int p) { return ((p & 1) << 2) | (p >> 1); }

// eight nibbles -> eight bf16 (order 0,4,1,5,2,6,3,7), times the group scale
__device__ __forceinline__ uint4 kvt_convert(uint32_t w, __nv_bfloat162 s2) {
  const uint32_t v = w ^ 0x88888888u;
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t x = ((v >> (4 * j)) & 0x000F000Fu) | 0x43004300u;          // 128 + (nibble ^ 8) in both halves
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&x);
    const uint32_t c136 = 0x43084308u;
    h = __hmul2(__hsub2(h, *reinterpret_cast<const __nv_bfloat162*>(&c136)), s2);
    o[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}


template <int N>
__device__ __forceinline__ void kvt_tmem_ld(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 16) tmem_ld16(taddr, r); else tmem_ld32(taddr, r);
}

template <int NP>
__global__ void __launch_bounds__(KVT_THREADS, NP == 32 ? 2 : 1)
kv_attention_tc_kernel(KvDev c, const __nv_bfloat16* __restrict__ q, int Tq, int Hq, float scale_log2, int splits,
                       float* __restrict__ part_acc, float* __restrict__ part_ml, int* status) {
  using S = KvtSmem<NP>;
  constexpr int D = KVT_D, CPT = NP / 2;                   // accumulator columns (query rows) per thread
  constexpr uint32_t TMEM_COLS = 2 * NP;                   // S^T then O^T
  extern __shared__ uint8_t kvt_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(kvt_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(sm);
  float* tsc = reinterpret_cast<float*>(sm + S::OFF_T);
  float* rowstat = reinterpret_cast<float*>(sm + S::OFF_WMAX);      // [0] new maximum, [NP] rescale factor, [2 NP] running maximum
  constexpr int TS = (int)S::T_STRIDE;
  float* lred = reinterpret_cast<float*>(sm + S::OFF_LRED);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + S::OFF_MISC);
  volatile int* dead = reinterpret_cast<volatile int*>(sm + S::OFF_MISC + 4);
  volatile int* go = reinterpret_cast<volatile int*>(sm + S::OFF_MISC + 8);      // [2] "the wait succeeded"
  const uint32_t bar_s = sb + S::OFF_BAR, bar_o = bar_s + 8;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, quad = warp & 3, half = warp >> 2;
  const int split = blockIdx.x % splits, pass = blockIdx.x / splits, hk = blockIdx.y, b = blockIdx.z;
  const int rep = Hq / c.heads, R = Tq * rep, r0 = pass * NP, rows = min(NP, R - r0);
  const int len = c.lengths[b] + Tq;                        // the Tq new tokens were appended before the call
  const int per = ((len + splits - 1) / splits + KVT_KB - 1) / KVT_KB * KVT_KB;
  const int k_begin = split * per, k_end = min(len, k_begin + per);
  const int G = D / c.group;

  if (warp == 0) tmem_alloc(sb + S::OFF_MISC, TMEM_COLS);
  if (tid == 0) { mbar_init(bar_s, 1); mbar_init(bar_o, 1); *dead = 0; mbar_fence_init(); }
  // Q rows -> K-major operand tile [NP][128], two 64-wide blocks, word order 0,4,1,5,2,6,3,7
  for (int i = tid; i < NP * 16; i += KVT_THREADS) {
    const int r = i >> 4, ch = i & 15;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      const int rr = r0 + r, t = rr / rep, h = hk * rep + rr % rep;
      const uint4 w = *reinterpret_cast<const uint4*>(q + (((long long)b * Tq + t) * Hq + h) * D + ch * 8);
      o = make_uint4(__byte_perm(w.x, w.z, 0x5410), __byte_perm(w.x, w.z, 0x7632), __byte_perm(w.y, w.w, 0x5410), __byte_perm(w.y, w.w, 0x7632));
    }
    *reinterpret_cast<uint4*>(sm + S::OFF_Q + (ch >> 3) * (NP * 128) + sw128_offset(r, ch & 7)) = o;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s = tmem + ((uint32_t)(quad * 32) << 16) + half * CPT, t_o = t_s + NP;

  // raw bytes of one block: two 16-byte units of K and of V per thread (unit = 32 elements of one key)
  uint4 kraw[2], vraw[2];
  float ksc[2], vsc[2];
  auto fetch = [&](int kb) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int u = tid + i * KVT_THREADS, key = kb + (u >> 2), qu = u & 3;
      kraw[i] = vraw[i] = make_uint4(0, 0, 0, 0);
      ksc[i] = vsc[i] = 0.0f;
      if (key < k_end) {
        const int page = c.page_table[b * c.max_pages + key / c.page_size];
        const long long tok = ((long long)page * c.page_size + key % c.page_size) * c.heads + hk;
        kraw[i] = *reinterpret_cast<const uint4*>(c.k_pages + tok * (D / 2) + qu * 16);
        vraw[i] = *reinterpret_cast<const uint4*>(c.v_pages + tok * (D / 2) + qu * 16);
        ksc[i] = c.k_scales[tok * G + qu * 32 / c.group];
        vsc[i] = c.v_scales[tok * G + qu * 32 / c.group];
      }
    }
  };
  auto convert = [&]() {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int u = tid + i * KVT_THREADS, row = u >> 2, qu = u & 3;
      const __nv_bfloat162 ks2 = __float2bfloat162_rn(ksc[i]), vs2 = __float2bfloat162_rn(vsc[i]);
      const uint32_t base = (qu >> 1) * KVT_HALF;
      const uint32_t kw[4] = {kraw[i].x, kraw[i].y, kraw[i].z, kraw[i].w}, vw[4] = {vraw[i].x, vraw[i].y, vraw[i].z, vraw[i].w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t off = base + sw128_offset(row, (qu & 1) * 4 + w);
        *reinterpret_cast<uint4*>(sm + S::OFF_K + off) = kvt_convert(kw[w], ks2);
        *reinterpret_cast<uint4*>(sm + S::OFF_V + off) = kvt_convert(vw[w], vs2);
      }
    }
  };

  float acc[CPT], l_part[CPT];
#pragma unroll
  for (int j = 0; j < CPT; ++j) { acc[j] = 0.0f; l_part[j] = 0.0f; }
  if (tid < NP) rowstat[2 * NP + tid] = -INFINITY;                   // ordered before its first use by the barriers of the first block
  const uint32_t idesc_s = make_idesc_bf16(128, NP, 0, 0), idesc_o = make_idesc_bf16(128, NP, 1, 0);
  uint32_t phase = 0;
  bool ok = true;
  if (k_begin < k_end) fetch(k_begin);
  for (int kb = k_begin; kb < k_end && ok; kb += KVT_KB) {
    convert();
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        umma_f16(tmem, make_smem_desc_sw128(sb + S::OFF_K + (kk >> 2) * KVT_HALF + (kk & 3) * 32, 16, 1024),
                 make_smem_desc_sw128(sb + S::OFF_Q + (kk >> 2) * (NP * 128) + (kk & 3) * 32, 16, 1024), idesc_s, kk != 0);
      umma_commit(bar_s);
    }
    if (kb + KVT_KB < k_end) fetch(kb + KVT_KB);
    // one thread polls (a poll is a shared-memory access; 256 pollers would crowd out the work), a
    // block barrier releases the rest, who read that thread's verdict
    if (tid == 0) go[0] = mbar_wait(bar_s, phase, dead, status, 610);
    __syncthreads();
    ok = go[0] != 0;
    if (!ok) break;
    tc_fence_after();
    uint32_t sr[CPT];
    kvt_tmem_ld<CPT>(t_s, sr);
    tmem_ld_wait();
    const int key = kb + quad * 32 + lane, kin = quad * 32 + lane;
    float s[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const int t = (r0 + half * CPT + j) / rep;
      s[j] = (key >= k_end || key > len - Tq + t) ? -INFINITY : __uint_as_float(sr[j]) * scale_log2;   // causal among the new tokens
      tsc[(half * CPT + j) * TS + kin] = s[j];                      // row-major copy: the keys of a row lie on the lanes here
    }
    __syncthreads();
    {
      // row maximum over the block's 128 keys by TPR threads (a warp-wide redux per row and thread cost
      // ~100 cycles each), then ONE thread per row folds it into the running maximum and works out the
      // rescale factor, instead of every thread repeating the exponential
      constexpr int TPR = KVT_THREADS / NP, F4 = KVT_KB / 4 / TPR;
      const int r = tid / TPR, seg = tid % TPR;
      const float4* row4 = reinterpret_cast<const float4*>(tsc + r * TS);
      float mb = -INFINITY;
#pragma unroll
      for (int i = 0; i < F4; ++i) { const float4 v = row4[i * TPR + seg]; mb = fmaxf(fmaxf(mb, fmaxf(v.x, v.y)), fmaxf(v.z, v.w)); }
#pragma unroll
      for (int o = 1; o < TPR; o <<= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
      if (seg == 0) {
        const float mo = rowstat[2 * NP + r], mn = fmaxf(mo, mb);
        rowstat[r] = mn;
        rowstat[NP + r] = mo > -INFINITY ? fast_exp2(mo - mn) : 1.0f;
        rowstat[2 * NP + r] = mn;
      }
    }
    __syncthreads();
    float corr[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const int r = half * CPT + j;
      const float mn = rowstat[r];
      corr[j] = rowstat[NP + r];
      const float p = s[j] > -INFINITY ? fast_exp2(s[j] - mn) : 0.0f;
      const __nv_bfloat16 pb = __float2bfloat16(p);
      l_part[j] = l_part[j] * corr[j] + __bfloat162float(pb);
      *reinterpret_cast<__nv_bfloat16*>(sm + S::OFF_P + (kin >> 6) * (NP * 128) + sw128_offset(r, (kin & 63) >> 3) + (kin & 7) * 2) = pb;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < KVT_KB / 16; ++kk)
        umma_f16(tmem + NP, make_smem_desc_sw128(sb + S::OFF_V + kk * 2048, KVT_HALF, 1024),
                 make_smem_desc_sw128(sb + S::OFF_P + (kk >> 2) * (NP * 128) + (kk & 3) * 32, 16, 1024), idesc_o, kk != 0);
      umma_commit(bar_o);
    }
    if (tid == 0) go[1] = mbar_wait(bar_o, phase, dead, status, 611);
    __syncthreads();
    ok = go[1] != 0;
    if (!ok) break;
    tc_fence_after();
    uint32_t orr[CPT];
    kvt_tmem_ld<CPT>(t_o, orr);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < CPT; ++j) acc[j] = acc[j] * corr[j] + __uint_as_float(orr[j]);
    phase ^= 1;
  }
  // row sums across the 128 keys of every block, then this split's partial
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const float v = warp_sum(l_part[j]);
    if (lane == 0) lred[quad * NP + half * CPT + j] = v;
  }
  tc_fence_before();
  __syncthreads();
  if (ok) {
    const int L = quad * 32 + lane, d = (L & ~7) | kvt_perm(L & 7);
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const int r = half * CPT + j;
      if (r < rows) {
        const long long row = ((long long)(b * c.heads + hk) * R + r0 + r) * splits + split;
        part_acc[row * D + d] = acc[j];
        if (L == 0) {
          part_ml[row * 2] = rowstat[2 * NP + r] * 0.69314718056f;         // the combine step works with natural logarithms
          part_ml[row * 2 + 1] = lred[r] + lred[NP + r] + lred[2 * NP + r] + lred[3 * NP + r];
        }
      }
    }
  }
  if (warp == 0) { tmem_relinquish(); tmem_dealloc(tmem, TMEM_COLS); }
}

template <int NP>
cudaError_t launch_np(const KvDev& c, const __nv_bfloat16* q, int Tq, int Hq, float scale, int splits, int passes,
                      float* part_acc, float* part_ml, int* status, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kv_attention_tc_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)KvtSmem<NP>::TOTAL);
  if (e != cudaSuccess) return e;
  const dim3 grid(splits * passes, c.heads, c.batch);
  kv_attention_tc_kernel<NP><<<grid, KVT_THREADS, KvtSmem<NP>::TOTAL, stream>>>(c, q, Tq, Hq, scale * 1.44269504089f, splits, part_acc, part_ml, status);
  return cudaGetLastError();
}
}  // namespace

cudaError_t launch_kv_attention_tc(const KvDev& c, const __nv_bfloat16* q, int Tq, int Hq, float scale, int splits,
                                   float* part_acc, float* part_ml, int* status, cudaStream_t stream) {
  const int R = Tq * (Hq / c.heads);
  if (R <= 32) return launch_np<32>(c, q, Tq, Hq, scale, splits, 1, part_acc, part_ml, status, stream);
  return launch_np<64>(c, q, Tq, Hq, scale, splits, (R + 63) / 64, part_acc, part_ml, status, stream);
}
}  // namespace cgk
