// Flash-Attention-2 backward on tcgen05 tensor cores.
//
// One CTA owns one tile of 128 keys of one (batch, kv head).  K and V stay in
// shared memory; dK and dV accumulate in TMEM over every query tile that sees
// these keys and over every query head of the GQA group, so they need no
// atomics.  Per query tile (128 rows):
//     S  = Q K^T, dP = dO V^T            two MMAs into TMEM
//     P  = exp2(S*c - LSE), dS = P*(dP - delta)*scale      (two warpgroups, thread = query row
//          x 64 keys, packed two-wide fp32 arithmetic)
//          both written once, bf16, to a 128B-swizzled [rows][keys] tile that
//          serves as a K-major operand (dQ = dS K) and, read the other way, as
//          an MN-major operand (dV += P^T dO, dK += dS^T Q)
//     dQ tile -> TMEM -> a separate warpgroup drains it with
//          red.global.add.v4.f32 into an fp32 accumulator that a last kernel
//          casts to bf16; with head_dim 64 the next step's S / dP MMAs and the
//          P / dS computation overlap that drain
// delta = rowsum(dO * O) comes from a pre-pass.  Fully masked tiles are skipped.
//
// Reference counterparts: flash_attn_bwd_sim (src/cuda/flash_attn_kernels.c:401-525,
// materialises the full N_q x N_k matrices on the host) and
// cg_flash_attention_backward_cpu (src/attention/flash_attn.c), whose split-K
// variant is inexact.
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "flash_bwd_kernel.cuh"

namespace cgk {

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d].  A row of D elements is shared by D / 8
// lanes (one 16-byte load of each tensor per lane); every thread works on four rows at a time so
// that eight loads are in flight, which is what a streaming kernel needs to approach HBM rate.
template <int D>
__global__ void __launch_bounds__(256)
flash_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                   float* __restrict__ delta, int B, int H, int T,
                   long long o_bs, long long o_ts, long long o_hs, long long do_bs,
                   long long do_ts, long long do_hs) {
  constexpr int LPR = D / 8;                 // lanes per row
  constexpr int U = 4;
  const long long rows = (long long)B * T * H;            // row r = (b * T + t) * H + h
  const long long groups = (long long)gridDim.x * blockDim.x / LPR;
  const long long g0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
  const int c = ((int)threadIdx.x % LPR) * 8;
  for (long long r0 = g0; r0 < rows; r0 += groups * U) {
    uint4 a[U], g[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + u * groups;
      if (r < rows) {
        const int h = (int)(r % H);
        const long long bt = r / H;
        const int t = (int)(bt % T);
        const long long b = bt / T;
        a[u] = __ldg(reinterpret_cast<const uint4*>(O + b * o_bs + t * o_ts + h * o_hs + c));
        g[u] = __ldg(reinterpret_cast<const uint4*>(dO + b * do_bs + t * do_ts + h * do_hs + c));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + u * groups;
      float s = 0.0f;
      if (r < rows) {
        float2 x, y;
        x = unpack_bf16x2(a[u].x); y = unpack_bf16x2(g[u].x); s += x.x * y.x + x.y * y.y;
        x = unpack_bf16x2(a[u].y); y = unpack_bf16x2(g[u].y); s += x.x * y.x + x.y * y.y;
        x = unpack_bf16x2(a[u].z); y = unpack_bf16x2(g[u].z); s += x.x * y.x + x.y * y.y;
        x = unpack_bf16x2(a[u].w); y = unpack_bf16x2(g[u].w); s += x.x * y.x + x.y * y.y;
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (r < rows && (threadIdx.x % LPR) == 0) {
        const int h = (int)(r % H);
        const long long bt = r / H;
        delta[CGK_IDX(((bt / T) * H + h) * T + (bt % T), rows)] = s;
      }
    }
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
  CUtensorMap tq, tk, tv, tdo, tdq;
  int rc;
  {
    // fp32 accumulator [B, Tq, Hq*D]; box = 32 floats x 128 rows, 128-byte swizzle
    uint64_t dims[3] = {(uint64_t)a.Hq * D, (uint64_t)a.Tq, (uint64_t)a.B};
    uint64_t strides[2] = {(uint64_t)a.Hq * D * 4, (uint64_t)a.Tq * a.Hq * D * 4};
    uint32_t box[3] = {32, 128, 1};
    if ((rc = encode_tmap(&tdq, a.dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dims, strides, box,
                          Swz::B128)))
      return rc;
  }
  if ((rc = make_tmap4(&tq, a.q, a.B, a.Tq, a.Hq, D, a.q_bs, a.q_ts, a.q_hs))) return rc;
  if ((rc = make_tmap4(&tk, a.k, a.B, a.Tk, a.Hk, D, a.k_bs, a.k_ts, a.k_hs))) return rc;
  if ((rc = make_tmap4(&tv, a.v, a.B, a.Tk, a.Hk, D, a.v_bs, a.v_ts, a.v_hs))) return rc;
  if ((rc = make_tmap4(&tdo, a.d_o, a.B, a.Tq, a.Hq, D, a.o_bs, a.o_ts, a.o_hs))) return rc;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      C::TOTAL));
  dim3 grid((a.Tk + C::BN - 1) / C::BN, a.Hk, a.B);
  flash_bwd_kernel<D><<<grid, 512, C::TOTAL, st>>>(tq, tk, tv, tdo, tdq, p);
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
  CGK_REQUIRE((a.o_hs | a.o_ts | a.o_bs) % 8 == 0 && (((uintptr_t)a.o | (uintptr_t)a.d_o) & 15) == 0,
              "cgk_flash_backward: O and dO must be 16-byte aligned with strides that are multiples of 8 elements");
  if (a.B == 0 || a.Tq == 0 || a.Hq == 0 || a.Tk == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  const long long rows = (long long)a.B * a.Hq * a.Tq;
  {
    long long blocks = (rows * (a.D / 8) + 256 * 4 - 1) / (256 * 4);
    long long cap = (long long)sm_count(dev) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (a.D == 64)
      flash_delta_kernel<64><<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)a.o, (const __nv_bfloat16*)a.d_o,
                                                          a.delta, a.B, a.Hq, a.Tq, a.o_bs, a.o_ts, a.o_hs,
                                                          a.o_bs, a.o_ts, a.o_hs);
    else
      flash_delta_kernel<128><<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)a.o, (const __nv_bfloat16*)a.d_o,
                                                           a.delta, a.B, a.Hq, a.Tq, a.o_bs, a.o_ts, a.o_hs,
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

CGK_BOUNDS_READER(flash_bwd)
