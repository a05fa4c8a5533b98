// Serving kernels: INT4 quantise / dequantise, paged INT4 KV cache (append + attention over
// it), batched temperature / top-k / top-p sampling, speculative accept / correct / commit,
// tree-attention masks.
// Reference counterparts: src/quantize/int4.c (cg_quantize_int4, cg_dequantize,
// cg_kv_cache_int4_append/get), src/inference/speculative.c (samplers, cg_acceptance_prob,
// cg_sample_corrected, cg_tree_attention_mask); cg_attention_int4_kv is declared only
// (include/cg_quantize.h).  The host restatement of each is in csrc/capi and is the oracle.
#include <cuda_bf16.h>

#include "host_common.h"
#include "sm100.cuh"
#include "kv_dev.cuh"
#include "cogito_kernels.h"

namespace {
using namespace cgk;

// ------------------------------------------------------------------ Philox4x32-10
struct Philox { uint32_t c[4]; };
__device__ __forceinline__ Philox philox(uint64_t seed, uint64_t stream, uint64_t offset) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = (uint32_t)stream, c3 = (uint32_t)(stream >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return Philox{{c0, c1, c2, c3}};
}
__device__ __forceinline__ float u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }

// -------------------------------------------------------------- quantise (Q1)
// One warp per group.  scale = absmax / 7 (1 when < 1e-10); q = clamp(round(x / scale), -8, 7);
// even index in the low nibble.  Bit-exact with cg_quantize_int4.
__global__ void int4_quantize_kernel(const float* __restrict__ x, long long n, int group, uint8_t* __restrict__ packed, float* __restrict__ scales) {
  const long long gidx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long long lo = gidx * group;
  if (lo >= n) return;
  const int cnt = (int)(n - lo < group ? n - lo : group);
  float m = 0.0f;
  for (int i = lane; i < cnt; i += 32) m = fmaxf(m, fabsf(x[lo + i]));
  m = warp_max(m);
  const float s = m < 1e-10f ? 1.0f : m / 7.0f;
  if (lane == 0) scales[gidx] = s;
  for (int i = lane * 2; i < cnt; i += 64) {            // lo is even whenever group is even
    int q0 = (int)roundf(x[lo + i] / s), q1 = i + 1 < cnt ? (int)roundf(x[lo + i + 1] / s) : 0;
    q0 = max(-8, min(7, q0)); q1 = max(-8, min(7, q1));
    packed[(lo + i) >> 1] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
  }
}
__global__ void int4_dequantize_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, long long n, int group,
                                       float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
  for (long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x; b < (n + 1) / 2; b += (long long)gridDim.x * blockDim.x) {
    const uint8_t v = packed[b];
    const int q0 = (v & 0xF) >= 8 ? (v & 0xF) - 16 : (v & 0xF), q1 = (v >> 4) >= 8 ? (v >> 4) - 16 : (v >> 4);
    const long long e = b * 2;
    const float a = q0 * scales[e / group], c = e + 1 < n ? q1 * scales[(e + 1) / group] : 0.0f;
    if (out_f32) { out_f32[e] = a; if (e + 1 < n) out_f32[e + 1] = c; }
    if (out_bf16) { out_bf16[e] = __float2bfloat16(a); if (e + 1 < n) out_bf16[e + 1] = __float2bfloat16(c); }
  }
}

// ------------------------------------------------------------ KV cache (A3)
// The pool layout and the KvDev view are in kv_dev.cuh.
// k_new / v_new: bf16 [batch, T, heads, D]; token t of sequence b lands at position lengths[b] + t.
// One warp per (b, t, head).
__global__ void kv_append_kernel(KvDev c, const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new, int T, int* status) {
  const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wid >= c.batch * T * c.heads) return;
  const int h = wid % c.heads, t = (wid / c.heads) % T, b = wid / (c.heads * T);
  const int pos = c.lengths[b] + t, lp = pos / c.page_size;
  if (lp >= c.max_pages) { if (lane == 0) report_status(status, KST_BAD_ARG, 400, pos); return; }
  const int page = c.page_table[CGK_IDX(b * c.max_pages + lp, c.batch * c.max_pages)];
  const long long tok = ((long long)page * c.page_size + pos % c.page_size) * c.heads + h;
  const int G = c.D / c.group;
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* src = (which ? v_new : k_new) + (((long long)b * T + t) * c.heads + h) * c.D;
    uint8_t* dst = (which ? c.v_pages : c.k_pages) + tok * (c.D / 2);
    float* sc = (which ? c.v_scales : c.k_scales) + tok * G;
    for (int g = 0; g < G; ++g) {
      float m = 0.0f;
      for (int i = lane; i < c.group; i += 32) m = fmaxf(m, fabsf(__bfloat162float(src[g * c.group + i])));
      m = warp_max(m);
      const float s = m < 1e-10f ? 1.0f : m / 7.0f;
      if (lane == 0) sc[g] = s;
      for (int i = lane * 2; i < c.group; i += 64) {
        int q0 = (int)roundf(__bfloat162float(src[g * c.group + i]) / s), q1 = (int)roundf(__bfloat162float(src[g * c.group + i + 1]) / s);
        q0 = max(-8, min(7, q0)); q1 = max(-8, min(7, q1));
        dst[(g * c.group + i) >> 1] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
      }
    }
  }
}

// Attention of R = Tq * (Hq / Hk) query rows per (sequence, kv head) over the quantised
// history, split along the keys.  Each lane scores one key (its bytes are read once and
// dequantised in registers), the warp keeps an online softmax per row, then the lanes switch
// to owning a slice of D for P.V through a warp-private shared tile.  Partials (m, l, acc) of
// every split are merged by kv_combine_kernel.
constexpr int KV_MAXR = 24;
template <int D>
__global__ void __launch_bounds__(128)
kv_attention_kernel(KvDev c, const __nv_bfloat16* __restrict__ q, int Tq, int Hq, float scale, int splits,
                    float* __restrict__ part_acc, float* __restrict__ part_ml) {
  constexpr int MAXR = KV_MAXR, DPL = D / 32, KH = 64;  // rows per pass; D elements per lane in P.V; key elements held at once
  constexpr unsigned FULL = 0xffffffffu;
  extern __shared__ float smem[];
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, rep = Hq / c.heads, R = Tq * rep;
  const int len = c.lengths[b] + Tq;                   // the Tq new tokens were appended before the call
  float* q_s = smem;                                   // [MAXR][D] pre-scaled queries
  constexpr int VS = D + 1;                              // padded row: conflict-free writes (lane = key) and reads (lane = d)
  float* v_s = q_s + MAXR * D + warp * (32 * VS);      // [32 keys][VS], per warp
  float* p_s = smem + MAXR * D + 4 * 32 * VS + warp * (MAXR * 32);   // [MAXR][32 keys], per warp
  float* red_s = smem + MAXR * D + 4 * 32 * VS + 4 * MAXR * 32;       // cross-warp merge: 4 x MAXR x (2 + D)
  const int G = D / c.group;
  const int per = ((len + splits - 1) / splits + 31) / 32 * 32;      // keys per split, whole 32-key blocks
  const int k_begin = split * per, k_end = min(len, k_begin + per);
  for (int r0 = 0; r0 < R; r0 += MAXR) {
    const int rows = min(MAXR, R - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < rows * D; i += blockDim.x) {
      const int r = r0 + i / D, d = i % D, t = r / rep, h = hk * rep + r % rep;
      q_s[i] = __bfloat162float(q[(((long long)b * Tq + t) * Hq + h) * D + d]) * scale;
    }
    __syncthreads();
    float m_own = -INFINITY, l_own = 0.0f;              // lane r keeps the running max / sum of row r
    float acc[MAXR][DPL];
#pragma unroll
    for (int r = 0; r < MAXR; ++r)
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[r][j] = 0.0f;
    for (int kb = k_begin + warp * 32; kb < k_end; kb += 4 * 32) {
      const int key = kb + lane;
      const bool valid = key < k_end;
      long long tok = 0;
      if (valid) {
        const int page = c.page_table[b * c.max_pages + key / c.page_size];
        tok = ((long long)page * c.page_size + key % c.page_size) * c.heads + hk;
      }
      float s_acc[MAXR];
#pragma unroll
      for (int r = 0; r < MAXR; ++r) s_acc[r] = 0.0f;
#pragma unroll
      for (int half = 0; half < D / KH; ++half) {
        float kf[KH];                                   // this lane's key, dequantised
        if (valid) {
          const uint32_t* kw = reinterpret_cast<const uint32_t*>(c.k_pages + tok * (D / 2)) + half * (KH / 8);
          const uint32_t* vw = reinterpret_cast<const uint32_t*>(c.v_pages + tok * (D / 2)) + half * (KH / 8);
#pragma unroll
          for (int w = 0; w < KH / 8; ++w) {
            const uint32_t kv = kw[w], vv = vw[w];
            const int e0 = half * KH + w * 8;
            const float ks = c.k_scales[tok * G + e0 / c.group], vs = c.v_scales[tok * G + e0 / c.group];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int kq = (int)((kv >> (4 * j)) & 0xF), vq = (int)((vv >> (4 * j)) & 0xF);
              kf[w * 8 + j] = (float)(kq >= 8 ? kq - 16 : kq) * ks;
              v_s[lane * VS + e0 + j] = (float)(vq >= 8 ? vq - 16 : vq) * vs;
            }
          }
        } else {
#pragma unroll
          for (int d = 0; d < KH; ++d) { kf[d] = 0.0f; v_s[lane * VS + half * KH + d] = 0.0f; }
        }
#pragma unroll
        for (int r = 0; r < MAXR; ++r) {
          if (r < rows) {
            const float4* qr = reinterpret_cast<const float4*>(q_s + r * D + half * KH);
            float s = 0.0f;
#pragma unroll
            for (int d4 = 0; d4 < KH / 4; ++d4) { const float4 qq = qr[d4]; s += qq.x * kf[d4 * 4] + qq.y * kf[d4 * 4 + 1] + qq.z * kf[d4 * 4 + 2] + qq.w * kf[d4 * 4 + 3]; }
            s_acc[r] += s;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        if (r < rows) {
          const int t = (r0 + r) / rep;
          const float s = (!valid || key > len - Tq + t) ? -INFINITY : s_acc[r];   // causal among the new tokens
          const float mb = warp_max(s);
          const float m_old = __shfl_sync(FULL, m_own, r);
          const float mn = fmaxf(m_old, mb);
          const float corr = m_old > -INFINITY ? __expf(m_old - mn) : 1.0f;
          const float p = s > -INFINITY ? __expf(s - mn) : 0.0f;
          const float ps = warp_sum(p);
          if (lane == r) { l_own = l_own * corr + ps; m_own = mn; }
          p_s[r * 32 + lane] = p;
#pragma unroll
          for (int j = 0; j < DPL; ++j) acc[r][j] *= corr;
        }
      }
      __syncwarp();
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        if (r < rows) {
#pragma unroll 8
          for (int kk = 0; kk < 32; ++kk) {
            const float p = p_s[r * 32 + kk];
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[r][j] += p * v_s[kk * VS + j * 32 + lane];
          }
        }
      }
      __syncwarp();
    }
    // merge the four warps through shared memory, then write this split's partial
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      if (r < rows) {
        float* slot = red_s + (warp * MAXR + r) * (2 + D);
        if (lane == r) { slot[0] = m_own; slot[1] = l_own; }
#pragma unroll
        for (int j = 0; j < DPL; ++j) slot[2 + j * 32 + lane] = acc[r][j];
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows * D; i += blockDim.x) {
      const int r = i / D, d = i % D;
      float m = -INFINITY;
      for (int w = 0; w < 4; ++w) m = fmaxf(m, red_s[(w * MAXR + r) * (2 + D)]);
      float l = 0.0f, a = 0.0f;
      for (int w = 0; w < 4; ++w) {
        const float* slot = red_s + (w * MAXR + r) * (2 + D);
        const float f = slot[0] > -INFINITY ? __expf(slot[0] - m) : 0.0f;
        l += slot[1] * f; a += slot[2 + d] * f;
      }
      const long long row = ((long long)(b * c.heads + hk) * R + r0 + r) * splits + split;
      part_acc[row * D + d] = a;
      if (d == 0) { part_ml[row * 2] = m; part_ml[row * 2 + 1] = l; }
    }
  }
}
template <int D>
__global__ void kv_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int splits, int batch, int Hk, int Tq, int Hq,
                                  __nv_bfloat16* __restrict__ out) {
  const int rep = Hq / Hk, R = Tq * rep;
  const long long rows = (long long)batch * Hk * R;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < rows * D; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / D; const int d = (int)(i % D);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(row * splits + s) * 2]);
    float l = 0.0f, a = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(row * splits + s) * 2];
      const float f = ms > -INFINITY ? __expf(ms - m) : 0.0f;
      l += part_ml[(row * splits + s) * 2 + 1] * f; a += part_acc[(row * splits + s) * D + d] * f;
    }
    const int r = (int)(row % R), hk = (int)((row / R) % Hk), b = (int)(row / ((long long)R * Hk));
    const int t = r / rep, h = hk * rep + r % rep;
    out[(((long long)b * Tq + t) * Hq + h) * D + d] = __float2bfloat16(l > 0.0f ? a / l : 0.0f);
  }
}

// ------------------------------------------------------------- sampling (S1)
// One CTA per row: logits / temperature -> keep the top_k largest -> keep the smallest prefix of
// those whose probability mass reaches top_p -> renormalise -> sample.  temperature <= 0 is
// argmax.  top_k is clamped to [1, 1024] (0 = 1024).  probs_out (optional, fp32 [rows, V])
// receives the final distribution (zeros outside the kept set).
__device__ __forceinline__ uint32_t float_key(float f) { const uint32_t u = __float_as_uint(f); return (u & 0x80000000u) ? ~u : u | 0x80000000u; }
__device__ __forceinline__ float key_float(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? k ^ 0x80000000u : ~k); }
constexpr int SAMPLE_THREADS = 1024, MAX_TOPK = 1024;
constexpr int SAMPLE_REGS = 32;       // rows of up to 32 * 1024 logits are read once and kept as sort keys in registers

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const void* __restrict__ logits, int logits_bf16, long long ld, int V, float temperature, int top_k, float top_p,
              unsigned long long seed, const long long* __restrict__ step, int* __restrict__ tokens, float* __restrict__ probs_out) {
  __shared__ uint32_t s_count;
  __shared__ float s_red[32];
  __shared__ float cand_v[MAX_TOPK];
  __shared__ int cand_i[MAX_TOPK];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto load = [&](int i) -> float {
    const float v = logits_bf16 ? __bfloat162float(((const __nv_bfloat16*)logits)[row * ld + i]) : ((const float*)logits)[row * ld + i];
    return temperature > 0.0f ? v / temperature : v;
  };
  auto block_sum = [&](float v) { v = warp_sum(v); if (lane == 0) s_red[warp] = v; __syncthreads(); v = s_red[lane]; v = warp_sum(v); __syncthreads(); return v; };
  const int k = temperature > 0.0f ? (top_k <= 0 || top_k > MAX_TOPK ? MAX_TOPK : top_k) : 1;
  const int kk = k < V ? k : V;
  // The 32 selection rounds and the two gathering passes below each look at every logit: from registers
  // when the row fits (key 0 stands for "no element": it is below the key of any float), else from memory.
  const bool in_regs = V <= SAMPLE_REGS * SAMPLE_THREADS;
  uint32_t key[SAMPLE_REGS];
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < SAMPLE_REGS; ++j) { const int i = tid + j * SAMPLE_THREADS; key[j] = i < V ? float_key(load(i)) : 0u; }
  }
  // radix bisection (32 rounds) for the key of the kk-th largest value
  uint32_t prefix = 0;
  for (int bit = 31; bit >= 0; --bit) {
    if (tid == 0) s_count = 0;
    __syncthreads();
    const uint32_t want = prefix | (1u << bit);
    uint32_t mine = 0;
    if (in_regs) {
#pragma unroll
      for (int j = 0; j < SAMPLE_REGS; ++j) mine += (key[j] >> bit) >= (want >> bit);
    } else {
      for (int i = tid; i < V; i += SAMPLE_THREADS) mine += (float_key(load(i)) >> bit) >= (want >> bit);
    }
    mine = (uint32_t)__reduce_add_sync(0xffffffffu, mine);
    if (lane == 0 && mine) atomicAdd(&s_count, mine);
    __syncthreads();
    if (s_count >= (uint32_t)kk) prefix = want;        // at least kk values have this bit pattern or larger
    __syncthreads();
  }
  // gather the candidates: everything above the threshold, then ties until kk slots are used
  if (tid == 0) s_count = 0;
  __syncthreads();
  auto take = [&](uint32_t kv, int i) { const uint32_t slot = atomicAdd(&s_count, 1u); if (slot < (uint32_t)kk) { cand_v[slot] = key_float(kv); cand_i[slot] = i; } };
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < SAMPLE_REGS; ++j) if (key[j] > prefix) take(key[j], tid + j * SAMPLE_THREADS);
  } else {
    for (int i = tid; i < V; i += SAMPLE_THREADS) { const uint32_t kv = float_key(load(i)); if (kv > prefix) take(kv, i); }
  }
  __syncthreads();
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < SAMPLE_REGS; ++j) if (key[j] == prefix) take(key[j], tid + j * SAMPLE_THREADS);
  } else {
    for (int i = tid; i < V; i += SAMPLE_THREADS) { const uint32_t kv = float_key(load(i)); if (kv == prefix) take(kv, i); }
  }
  __syncthreads();
  const int n = (int)min(s_count, (uint32_t)kk);
  // bitonic sort, descending by (value, then smaller index first) so that the result is deterministic
  int n2 = 1; while (n2 < n) n2 <<= 1;
  for (int i = n + tid; i < n2; i += SAMPLE_THREADS) { cand_v[i] = -INFINITY; cand_i[i] = 0x7fffffff; }
  __syncthreads();
  for (int size = 2; size <= n2; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < n2; i += SAMPLE_THREADS) {
        const int j = i ^ stride;
        if (j > i) {
          const bool desc = (i & size) == 0;
          const bool i_first = cand_v[i] > cand_v[j] || (cand_v[i] == cand_v[j] && cand_i[i] < cand_i[j]);
          if (i_first != desc) { const float tv = cand_v[i]; cand_v[i] = cand_v[j]; cand_v[j] = tv; const int ti = cand_i[i]; cand_i[i] = cand_i[j]; cand_i[j] = ti; }
        }
      }
      __syncthreads();
    }
  // softmax over the candidates, nucleus cut, sample
  const float mx = cand_v[0];
  float e = tid < n ? __expf(cand_v[tid] - mx) : 0.0f;
  const float total = block_sum(e);
  if (tid < n) cand_v[tid] = e / total;
  __syncthreads();
  if (probs_out) for (int i = tid; i < V; i += SAMPLE_THREADS) probs_out[(long long)row * V + i] = 0.0f;
  __syncthreads();
  if (tid == 0) {
    int keep = n;
    if (top_p > 0.0f && top_p < 1.0f) { float acc = 0.0f; keep = 0; while (keep < n) { acc += cand_v[keep++]; if (acc >= top_p) break; } }
    float mass = 0.0f;
    for (int i = 0; i < keep; ++i) mass += cand_v[i];
    const Philox rnd = philox(seed, (uint64_t)row, step ? (uint64_t)*step : 0ull);
    const float u = u01(rnd.c[0]) * mass;
    float acc = 0.0f; int pick = keep - 1;
    for (int i = 0; i < keep; ++i) { acc += cand_v[i]; if (u < acc) { pick = i; break; } }
    tokens[row] = cand_i[CGK_IDX(pick, keep)];
    if (probs_out) for (int i = 0; i < keep; ++i) probs_out[(long long)row * V + cand_i[i]] = cand_v[i] / mass;
  }
}

// ------------------------------------------------- accept / correct / commit (S2)
// One CTA per sequence.  draft_tokens [B, gamma]; q = draft distributions [B, gamma, V];
// p = target distributions [B, gamma + 1, V] (row i scores draft token i, row gamma the bonus).
// Writes n_accepted[b], out_tokens[b, 0 .. n] (accepted drafts then the corrected or bonus
// token), and advances lengths[b] by n + 1 — the cache positions of rejected drafts fall
// beyond the new length, which is the rollback.
__global__ void __launch_bounds__(256)
spec_accept_kernel(const int* __restrict__ draft_tokens, const float* __restrict__ q, const float* __restrict__ p, int gamma, int V,
                   unsigned long long seed, const long long* __restrict__ step, int* __restrict__ n_accepted, int* __restrict__ out_tokens,
                   int* __restrict__ lengths, int* __restrict__ stats) {
  __shared__ int s_n;
  __shared__ float s_part[256];
  __shared__ float s_target;
  __shared__ int s_owner;
  const int b = blockIdx.x, tid = threadIdx.x;
  const Philox rnd = philox(seed, 0x5bd1e995ull + (uint64_t)b, step ? (uint64_t)*step : 0ull);
  if (tid == 0) {
    int n = 0;
    for (; n < gamma; ++n) {
      const int tok = (int)CGK_IDX(draft_tokens[b * gamma + n], V);
      const float pd = q[((long long)b * gamma + n) * V + tok], pt = p[((long long)b * (gamma + 1) + n) * V + tok];
      const Philox r2 = philox(seed, 0x9747b28cull + (uint64_t)b, (step ? (uint64_t)*step : 0ull) * 64 + n);
      const float ratio = pd > 0.0f ? fminf(1.0f, pt / pd) : 1.0f;
      if (!(u01(r2.c[0]) < ratio)) break;
      out_tokens[b * (gamma + 1) + n] = tok;
    }
    s_n = n;
  }
  __syncthreads();
  const int n = s_n;
  const float* pt = p + ((long long)b * (gamma + 1) + n) * V;
  const float* pd = n < gamma ? q + ((long long)b * gamma + n) * V : nullptr;
  // residual max(0, p - q) at the first rejected position; the plain target row for the bonus token
  const int chunk = (V + 255) / 256, lo = tid * chunk, hi = min(V, lo + chunk);
  float mine = 0.0f;
  for (int i = lo; i < hi; ++i) mine += pd ? fmaxf(0.0f, pt[i] - pd[i]) : pt[i];
  s_part[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int i = 0; i < 256; ++i) total += s_part[i];
    bool fallback = !(total > 1e-12f);
    if (fallback) total = 1.0f;                          // degenerate residual: sample the target row itself
    float target = u01(rnd.c[1]) * total, acc = 0.0f;
    int owner = 255;
    if (!fallback) for (int i = 0; i < 256; ++i) { if (target < acc + s_part[i]) { owner = i; break; } acc += s_part[i]; }
    s_owner = fallback ? -1 : owner;
    s_target = fallback ? target : target - acc;
  }
  __syncthreads();
  int pick = -1;
  if (s_owner == -1) {
    if (tid == 0) { float acc = 0.0f; pick = V - 1; for (int i = 0; i < V; ++i) { acc += pt[i]; if (s_target < acc) { pick = i; break; } } }
  } else if (tid == s_owner) {
    float acc = 0.0f; pick = hi - 1;
    for (int i = lo; i < hi; ++i) { const float r = pd ? fmaxf(0.0f, pt[i] - pd[i]) : pt[i]; acc += r; if (s_target < acc && r > 0.0f) { pick = i; break; } }
  }
  if (pick >= 0) {
    out_tokens[b * (gamma + 1) + n] = pick;
    n_accepted[b] = n;
    if (lengths) lengths[b] += n + 1;
    if (stats) { atomicAdd(&stats[0], gamma); atomicAdd(&stats[1], n); }
  }
}

// ------------------------------------------------------------ tree mask (S3)
// mask [L + n, L + n] additive (0 or -1e9): causal prefix; tree node i sees the prefix, its
// ancestors and itself.
__global__ void tree_mask_kernel(const int* __restrict__ parents, int n, int L, float* __restrict__ mask_f32, __nv_bfloat16* __restrict__ mask_bf16) {
  const int T = L + n;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < (long long)T * T; idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx / T), j = (int)(idx % T);
    bool vis;
    if (i < L) vis = j <= i;
    else if (j < L) vis = true;
    else { vis = false; int a = i - L; for (int hop = 0; hop <= n && a >= 0; ++hop) { if (a == j - L) { vis = true; break; } a = parents[CGK_IDX(a, n)]; if (a >= 0) (void)CGK_IDX(a, n); } }
    const float v = vis ? 0.0f : -1e9f;
    if (mask_f32) mask_f32[idx] = v;
    if (mask_bf16) mask_bf16[idx] = __float2bfloat16(v);
  }
}
}  // namespace

// ================================================================== entry points
CGK_API int cgk_int4_quantize(const float* x, long long n, int group, void* packed, float* scales, void* stream) {
  CGK_REQUIRE(x && packed && scales && n > 0 && group > 0 && group % 2 == 0, "cgk_int4_quantize: bad argument");
  const long long groups = (n + group - 1) / group;
  int4_quantize_kernel<<<(unsigned)((groups + 7) / 8), 256, 0, (cudaStream_t)stream>>>(x, n, group, (uint8_t*)packed, scales);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_int4_dequantize(const void* packed, const float* scales, long long n, int group, float* out_f32, void* out_bf16, void* stream) {
  CGK_REQUIRE(packed && scales && n > 0 && group > 0 && (out_f32 || out_bf16), "cgk_int4_dequantize: bad argument");
  const long long bytes = (n + 1) / 2;
  const int blocks = (int)((bytes + 255) / 256 < 2368 ? (bytes + 255) / 256 : 2368);
  int4_dequantize_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, scales, n, group, out_f32, (__nv_bfloat16*)out_bf16);
  CGK_LAUNCH_CHECK();
  return 0;
}
static int check_kv(const cgk_kv_args* a, const char* who) {
  CGK_REQUIRE(a && a->k_pages && a->v_pages && a->k_scales && a->v_scales && a->page_table && a->lengths, "%s: null pointer", who);
  CGK_REQUIRE(a->batch > 0 && a->heads > 0 && (a->D == 64 || a->D == 128) && a->group >= 8 && a->group % 8 == 0 && a->D % a->group == 0 && a->page_size > 0 && a->max_pages > 0,
              "%s: need D in {64,128}, group a multiple of 8 dividing D", who);
  return 0;
}
static KvDev kv_dev(const cgk_kv_args* a) {
  return KvDev{(uint8_t*)a->k_pages, (uint8_t*)a->v_pages, a->k_scales, a->v_scales, a->page_table, a->lengths, a->batch, a->heads, a->D, a->group, a->page_size, a->max_pages};
}
CGK_API int cgk_kv_int4_append(const cgk_kv_args* a, const void* k_new, const void* v_new, int T, void* stream) {
  if (int rc = check_kv(a, "cgk_kv_int4_append")) return rc;
  CGK_REQUIRE(k_new && v_new && T > 0, "cgk_kv_int4_append: bad argument");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const int warps = a->batch * T * a->heads;
  kv_append_kernel<<<(warps + 7) / 8, 256, 0, (cudaStream_t)stream>>>(kv_dev(a), (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, T, device_status(dev));
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API long long cgk_kv_int4_attention_scratch_floats(int batch, int Hq, int Tq, int D, int splits) {
  return (long long)batch * Hq * Tq * splits * (D + 2);
}
// q, out: bf16 [batch, Tq, Hq, D]; the Tq newest tokens must already be in the cache (positions
// lengths[b] .. lengths[b] + Tq - 1).  scratch: cgk_kv_int4_attention_scratch_floats floats.
CGK_API int cgk_kv_int4_attention(const cgk_kv_args* a, const void* q, void* out, int Tq, int Hq, float scale, int splits, float* scratch, void* stream) {
  if (int rc = check_kv(a, "cgk_kv_int4_attention")) return rc;
  CGK_REQUIRE(q && out && scratch && Tq > 0 && Hq % a->heads == 0 && splits > 0 && splits <= 256, "cgk_kv_int4_attention: bad argument");
  const int D = a->D;
  const size_t smem = sizeof(float) * ((size_t)KV_MAXR * D + 4 * 32 * (D + 1) + 4 * KV_MAXR * 32 + 4 * KV_MAXR * (2 + D));
  float* part_acc = scratch;
  float* part_ml = scratch + (long long)a->batch * Hq * Tq * splits * D;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(splits, a->heads, a->batch);
  const long long rows = (long long)a->batch * Hq * Tq;
  const int cblocks = (int)((rows * D + 255) / 256 < 1184 ? (rows * D + 255) / 256 : 1184);
  if (D == 128 && a->group % 32 == 0) {
    // tensor-core path (kv_attn_tc.cu); the CUDA-core kernel below covers the other shapes
    int dev = 0;
    CGK_CUDA_CHECK(cudaGetDevice(&dev));
    CGK_CUDA_CHECK(launch_kv_attention_tc(kv_dev(a), (const __nv_bfloat16*)q, Tq, Hq, scale, splits, part_acc, part_ml, device_status(dev), st));
    kv_combine_kernel<128><<<cblocks, 256, 0, st>>>(part_acc, part_ml, splits, a->batch, a->heads, Tq, Hq, (__nv_bfloat16*)out);
  } else if (D == 128) {
    CGK_CUDA_CHECK(cudaFuncSetAttribute(kv_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kv_attention_kernel<128><<<grid, 128, smem, st>>>(kv_dev(a), (const __nv_bfloat16*)q, Tq, Hq, scale, splits, part_acc, part_ml);
    CGK_LAUNCH_CHECK();
    kv_combine_kernel<128><<<cblocks, 256, 0, st>>>(part_acc, part_ml, splits, a->batch, a->heads, Tq, Hq, (__nv_bfloat16*)out);
  } else {
    CGK_CUDA_CHECK(cudaFuncSetAttribute(kv_attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kv_attention_kernel<64><<<grid, 128, smem, st>>>(kv_dev(a), (const __nv_bfloat16*)q, Tq, Hq, scale, splits, part_acc, part_ml);
    CGK_LAUNCH_CHECK();
    kv_combine_kernel<64><<<cblocks, 256, 0, st>>>(part_acc, part_ml, splits, a->batch, a->heads, Tq, Hq, (__nv_bfloat16*)out);
  }
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_sample(const void* logits, int logits_bf16, long long ld, int rows, int V, float temperature, int top_k, float top_p,
                       unsigned long long seed, const long long* step, int* tokens, float* probs_out, void* stream) {
  CGK_REQUIRE(logits && tokens && rows > 0 && V > 0 && ld >= V, "cgk_sample: bad argument");
  sample_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, logits_bf16, ld, V, temperature, top_k, top_p, seed, step, tokens, probs_out);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_spec_accept(const int* draft_tokens, const float* q, const float* p, int batch, int gamma, int V, unsigned long long seed,
                            const long long* step, int* n_accepted, int* out_tokens, int* lengths, int* stats, void* stream) {
  CGK_REQUIRE(draft_tokens && q && p && n_accepted && out_tokens && batch > 0 && gamma > 0 && gamma < 64 && V > 0, "cgk_spec_accept: bad argument");
  spec_accept_kernel<<<batch, 256, 0, (cudaStream_t)stream>>>(draft_tokens, q, p, gamma, V, seed, step, n_accepted, out_tokens, lengths, stats);
  CGK_LAUNCH_CHECK();
  return 0;
}
CGK_API int cgk_tree_mask(const int* parents, int n, int L, float* mask_f32, void* mask_bf16, void* stream) {
  CGK_REQUIRE(parents && n > 0 && L >= 0 && (mask_f32 || mask_bf16), "cgk_tree_mask: bad argument");
  const long long total = (long long)(L + n) * (L + n);
  const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
  tree_mask_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(parents, n, L, mask_f32, (__nv_bfloat16*)mask_bf16);
  CGK_LAUNCH_CHECK();
  return 0;
}

CGK_BOUNDS_READER(serving)
