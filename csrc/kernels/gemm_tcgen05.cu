// bf16 GEMM on the 5th-generation tensor cores: TMA -> 128B-swizzled shared
// memory -> tcgen05.mma (fp32 accumulators in TMEM) -> tcgen05.ld epilogue.
//
// One persistent CTA per SM, 256 threads, warp-specialised:
//   warp 0      TMA producer (one lane)
//   warp 1      MMA issuer   (one lane)
//   warp 2      TMEM allocator / deallocator
//   warps 4..7  epilogue: each warp drains its 32-lane quadrant of TMEM
// Tile = 128 x BN x 64 with a STAGES-deep shared-memory ring and two TMEM
// accumulators, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Counterpart in the reference: cg_tensor_matmul (src/core/tensor_ops.c:175),
// the cublasSgemm call (src/cuda/tensor_kernels.c:523-546), cg_bf16_matmul
// (src/core/bf16.c:233) and the matmul-epilogue fusion patterns
// (src/jit/fusion.c:230-277), which there only exist as text.
#include "../../include/cogito_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cgk {

struct GemmDev {
  int M, N, K, batch;
  int tiles_m, tiles_n;
  int a_mn, b_mn;
  void* out;
  long long ldc, strideC;
  int out_fp32, accumulate;
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
  long long o = (long long)b * g.strideC + (long long)m * g.ldc + n;
  if (g.out_fp32) {
    float* p = reinterpret_cast<float*>(g.out) + o;
    *p = g.accumulate ? (*p + v) : v;
  } else {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(g.out) + o;
    *p = __float2bfloat16(g.accumulate ? (__bfloat162float(*p) + v) : v);
  }
}

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GROUP_M = 8;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;  // + alignment slack
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& b, int& tm,
                                            int& tn) {
  const int per_batch = tiles_m * tiles_n;
  b = t / per_batch;
  int r = t - b * per_batch;
  const int group_sz = GROUP_M * tiles_n;
  const int gidx = r / group_sz;
  const int first_m = gidx * GROUP_M;
  const int rows_in_group = min(GROUP_M, tiles_m - first_m);
  const int rr = r - gidx * group_sz;
  tm = first_m + rr % rows_in_group;
  tn = rr / rows_in_group;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(256, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmDev g) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
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
      mbar_init(tempty_bar(a), 128);
    }
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

  const int total_tiles = g.batch * g.tiles_m * g.tiles_n;
  const int kblocks = (g.K + BK - 1) / BK;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t kit = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, tm, tn;
        tile_coords(t, g.tiles_m, g.tiles_n, b, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++kit) {
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
      const uint32_t a_kstep = g.a_mn ? 2048u : 32u;  // bytes per 16 K elements
      const uint32_t b_kstep = g.b_mn ? 2048u : 32u;
      uint32_t kit = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t aph = (it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u, dead, g.status, 200)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++kit) {
          const int s = kit % STAGES;
          const uint32_t ph = (kit / STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, dead, g.status, 201)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + s * L::STAGE_BYTES;
          const uint32_t sB = sA + L::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t ad = make_smem_desc_sw128(sA + kk * a_kstep, a_lbo, 1024u);
            const uint64_t bd = make_smem_desc_sw128(sB + kk * b_kstep, b_lbo, 1024u);
            umma_f16(d_tmem, ad, bd, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp >= 4) {
    const int q = warp - 4;  // == warp % 4: the TMEM lane quadrant this warp may read
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
      int b, tm, tn;
      tile_coords(t, g.tiles_m, g.tiles_n, b, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int acc = it & 1;
      const uint32_t aph = (it >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), aph, dead, g.status, 300)) { ok = false; break; }
      tc_fence_after();
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < g.M;
      const bool vec_ok = ((g.ldc & 7) == 0) && (!g.residual || (g.ldr & 7) == 0) &&
                          (!g.aux_out || (g.ldaux & 7) == 0) &&
                          (!g.aux_in || (g.ldauxin & 7) == 0) && ((g.strideC & 7) == 0) &&
                          ((reinterpret_cast<uintptr_t>(g.out) & 15) == 0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int nc = n0 + c * 32;
        if (nc >= g.N) break;
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (!row_ok) {
          // rows beyond M: nothing to store (the warp still took part in the load)
        } else if (vec_ok && nc + 32 <= g.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = g.alpha * __uint_as_float(r[j]);
          if (g.bias) {
            if (g.bias_fp32) {
              const float4* bp = reinterpret_cast<const float4*>(
                  reinterpret_cast<const float*>(g.bias) + nc);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 bv = __ldg(bp + j);
                v[4 * j] += bv.x; v[4 * j + 1] += bv.y; v[4 * j + 2] += bv.z; v[4 * j + 3] += bv.w;
              }
            } else {
              const uint4* bp = reinterpret_cast<const uint4*>(
                  reinterpret_cast<const __nv_bfloat16*>(g.bias) + nc);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 bv = __ldg(bp + j);
                float2 f;
                f = unpack_bf16x2(bv.x); v[8 * j] += f.x; v[8 * j + 1] += f.y;
                f = unpack_bf16x2(bv.y); v[8 * j + 2] += f.x; v[8 * j + 3] += f.y;
                f = unpack_bf16x2(bv.z); v[8 * j + 4] += f.x; v[8 * j + 5] += f.y;
                f = unpack_bf16x2(bv.w); v[8 * j + 6] += f.x; v[8 * j + 7] += f.y;
              }
            }
          }
          if (g.aux_out) {
            uint4* ap = reinterpret_cast<uint4*>(g.aux_out + (long long)m * g.ldaux + nc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
              o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
              o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
              o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
              ap[j] = o;
            }
          }
          if (g.act != CGK_ACT_NONE) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(g.act, v[j]);
          }
          if (g.aux_in) {
            const uint4* ap =
                reinterpret_cast<const uint4*>(g.aux_in + (long long)m * g.ldauxin + nc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 a = __ldg(ap + j);
              float2 f;
              f = unpack_bf16x2(a.x); v[8 * j] *= apply_dact(g.dact, f.x); v[8 * j + 1] *= apply_dact(g.dact, f.y);
              f = unpack_bf16x2(a.y); v[8 * j + 2] *= apply_dact(g.dact, f.x); v[8 * j + 3] *= apply_dact(g.dact, f.y);
              f = unpack_bf16x2(a.z); v[8 * j + 4] *= apply_dact(g.dact, f.x); v[8 * j + 5] *= apply_dact(g.dact, f.y);
              f = unpack_bf16x2(a.w); v[8 * j + 6] *= apply_dact(g.dact, f.x); v[8 * j + 7] *= apply_dact(g.dact, f.y);
            }
          }
          if (g.residual) {
            const uint4* rp = reinterpret_cast<const uint4*>(g.residual + (long long)m * g.ldr + nc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 a = __ldg(rp + j);
              float2 f;
              f = unpack_bf16x2(a.x); v[8 * j] += f.x; v[8 * j + 1] += f.y;
              f = unpack_bf16x2(a.y); v[8 * j + 2] += f.x; v[8 * j + 3] += f.y;
              f = unpack_bf16x2(a.z); v[8 * j + 4] += f.x; v[8 * j + 5] += f.y;
              f = unpack_bf16x2(a.w); v[8 * j + 6] += f.x; v[8 * j + 7] += f.y;
            }
          }
          const long long o = (long long)b * g.strideC + (long long)m * g.ldc + nc;
          if (g.out_fp32) {
            float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(g.out) + o);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 w = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              if (g.accumulate) {
                float4 old = op[j];
                w.x += old.x; w.y += old.y; w.z += old.z; w.w += old.w;
              }
              op[j] = w;
            }
          } else {
            uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(g.out) + o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (g.accumulate) {
                uint4 old = op[j];
                float2 f;
                f = unpack_bf16x2(old.x); v[8 * j] += f.x; v[8 * j + 1] += f.y;
                f = unpack_bf16x2(old.y); v[8 * j + 2] += f.x; v[8 * j + 3] += f.y;
                f = unpack_bf16x2(old.z); v[8 * j + 4] += f.x; v[8 * j + 5] += f.y;
                f = unpack_bf16x2(old.w); v[8 * j + 6] += f.x; v[8 * j + 7] += f.y;
              }
              uint4 w;
              w.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
              w.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
              w.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
              w.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
              op[j] = w;
            }
          }
        } else {
          // ragged edge or unaligned leading dimension
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (nc + j < g.N) epilogue_scalar(g, b, m, nc + j, __uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
    }
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

// CUDA-core fallback for operands that TMA cannot address (leading dimension not a
// multiple of 8 elements, unaligned base) and for tiny problems in tests.
__global__ void gemm_bf16_simt_kernel(const __nv_bfloat16* __restrict__ A,
                                      const __nv_bfloat16* __restrict__ B, long long lda,
                                      long long ldb, long long strideA, long long strideB,
                                      const GemmDev g) {
  __shared__ float sa[32][33];
  __shared__ float sb[32][33];
  const int b = blockIdx.z;
  const int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const __nv_bfloat16* Ab = A + (long long)b * strideA;
  const __nv_bfloat16* Bb = B + (long long)b * strideB;
  float acc = 0.0f;
  for (int k0 = 0; k0 < g.K; k0 += 32) {
    {
      int m = m0 + ty, k = k0 + tx;
      float v = 0.0f;
      if (m < g.M && k < g.K) v = __bfloat162float(g.a_mn ? Ab[(long long)k * lda + m] : Ab[(long long)m * lda + k]);
      sa[ty][tx] = v;
      int n = n0 + ty;
      float w = 0.0f;
      if (n < g.N && k < g.K) w = __bfloat162float(g.b_mn ? Bb[(long long)k * ldb + n] : Bb[(long long)n * ldb + k]);
      sb[ty][tx] = w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; ++k) acc += sa[ty][k] * sb[tx][k];
    __syncthreads();
  }
  const int m = m0 + ty, n = n0 + tx;
  if (m < g.M && n < g.N) epilogue_scalar(g, b, m, n, acc);
}

template <int BN, int STAGES>
static int launch_tc(const cgk_gemm_args& a, const GemmDev& g0, int sms, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  GemmDev g = g0;
  g.tiles_m = (a.M + BM - 1) / BM;
  g.tiles_n = (a.N + BN - 1) / BN;
  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a.a_mn) {
      dims[0] = (uint64_t)a.K; dims[1] = (uint64_t)a.M;
      box[0] = BK; box[1] = BM;
    } else {
      dims[0] = (uint64_t)a.M; dims[1] = (uint64_t)a.K;
      box[0] = 64; box[1] = BK;
    }
    dims[2] = (uint64_t)a.batch;
    strides[0] = (uint64_t)a.lda * 2;
    strides[1] = (uint64_t)(a.batch > 1 ? a.strideA : (int64_t)dims[1] * a.lda) * 2;
    box[2] = 1;
    rc = encode_tmap(&tmA, a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B128);
    if (rc) return rc;
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a.b_mn) {
      dims[0] = (uint64_t)a.K; dims[1] = (uint64_t)a.N;
      box[0] = BK; box[1] = BN;
    } else {
      dims[0] = (uint64_t)a.N; dims[1] = (uint64_t)a.K;
      box[0] = 64; box[1] = BK;
    }
    dims[2] = (uint64_t)a.batch;
    strides[0] = (uint64_t)a.ldb * 2;
    strides[1] = (uint64_t)(a.batch > 1 ? a.strideB : (int64_t)dims[1] * a.ldb) * 2;
    box[2] = 1;
    rc = encode_tmap(&tmB, a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B128);
    if (rc) return rc;
  }
  CGK_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN, STAGES>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  int total = g.batch * g.tiles_m * g.tiles_n;
  int cap = a.max_ctas > 0 ? a.max_ctas : sms;
  int grid = total < cap ? total : cap;
  gemm_bf16_tc_kernel<BN, STAGES><<<grid, 256, L::TOTAL, stream>>>(tmA, tmB, g);
  CGK_LAUNCH_CHECK();
  return 0;
}

}  // namespace cgk

CGK_API int cgk_gemm_bf16(const cgk_gemm_args* pa, void* stream_) {
  using namespace cgk;
  CGK_REQUIRE(pa != nullptr, "cgk_gemm_bf16: null args");
  const cgk_gemm_args& a = *pa;
  cudaStream_t stream = (cudaStream_t)stream_;
  CGK_REQUIRE(a.A && a.B && a.out, "cgk_gemm_bf16: null operand");
  CGK_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0 && a.batch >= 1, "cgk_gemm_bf16: bad sizes");
  if (a.M == 0 || a.N == 0) return 0;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  GemmDev g;
  g.M = a.M; g.N = a.N; g.K = a.K; g.batch = a.batch;
  g.tiles_m = g.tiles_n = 0;
  g.a_mn = a.a_mn ? 1 : 0; g.b_mn = a.b_mn ? 1 : 0;
  g.out = a.out; g.ldc = a.ldc; g.strideC = a.strideC;
  g.out_fp32 = a.out_fp32; g.accumulate = a.accumulate;
  g.alpha = a.alpha;
  g.bias = a.bias; g.bias_fp32 = a.bias_fp32; g.act = a.act;
  g.residual = (const __nv_bfloat16*)a.residual; g.ldr = a.ldr;
  g.aux_out = (__nv_bfloat16*)a.aux_out; g.ldaux = a.ldaux;
  g.aux_in = (const __nv_bfloat16*)a.aux_in; g.ldauxin = a.ldauxin;
  g.dact = a.dact;
  g.status = device_status(dev);
  CGK_REQUIRE(a.batch == 1 || !(a.residual || a.aux_out || a.aux_in),
              "cgk_gemm_bf16: residual/aux epilogues are 2-D only");

  const bool tma_ok = (a.lda % 8 == 0) && (a.ldb % 8 == 0) &&
                      (((uintptr_t)a.A & 15) == 0) && (((uintptr_t)a.B & 15) == 0) &&
                      (a.batch == 1 || (a.strideA % 8 == 0 && a.strideB % 8 == 0)) && a.K > 0;
  if (a.force_simt || !tma_ok) {
    dim3 grid((a.N + 31) / 32, (a.M + 31) / 32, a.batch);
    dim3 block(32, 32, 1);
    gemm_bf16_simt_kernel<<<grid, block, 0, stream>>>(
        (const __nv_bfloat16*)a.A, (const __nv_bfloat16*)a.B, a.lda, a.ldb, a.strideA, a.strideB, g);
    CGK_LAUNCH_CHECK();
    return 0;
  }
  const int sms = sm_count(dev);
  const long long tm = (a.M + BM - 1) / BM;
  auto tiles = [&](int bn) { return (long long)a.batch * tm * ((a.N + bn - 1) / bn); };
  // Widest tile that still gives every SM work; narrow tiles for small problems.
  if (a.N > 128 && tiles(256) >= (long long)sms * 3 / 4) return launch_tc<256, 4>(a, g, sms, stream);
  if (a.N > 64 && tiles(128) >= (long long)sms / 2) return launch_tc<128, 6>(a, g, sms, stream);
  return launch_tc<64, 8>(a, g, sms, stream);
}
