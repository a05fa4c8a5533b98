// bf16 GEMM on the 5th-generation tensor cores: TMA -> 128B-swizzled shared
// memory -> tcgen05.mma (fp32 accumulators in TMEM) -> tcgen05.ld epilogue.
//
// One persistent CTA per SM, 384 threads, warp-specialised:
//   warp 0      TMA producer (one lane)
//   warp 1      MMA issuer   (one lane)
//   warp 2      TMEM allocator / deallocator
//   warps 4..11 epilogue: warp w drains TMEM lane quadrant w % 4 for one half of the columns
// Tile = 128 x BN x 64 with a STAGES-deep shared-memory ring and two TMEM
// accumulators, so the epilogue of tile i overlaps the main loop of tile i+1.
// The device code is in gemm_tc_body.cuh (shared with the fused collective kernels).
//
// Counterpart in the reference: cg_tensor_matmul (src/core/tensor_ops.c:175),
// the cublasSgemm call (src/cuda/tensor_kernels.c:523-546), cg_bf16_matmul
// (src/core/bf16.c:233) and the matmul-epilogue fusion patterns
// (src/jit/fusion.c:230-277), which there only exist as text.
#include "gemm_host.h"

namespace cgk {

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
                    const __grid_constant__ CUtensorMap tmIn, const GemmDev g) {
  extern __shared__ uint8_t smem_raw[];
  gemm_tc_body<BN, STAGES>(tmA, tmB, &tmC, &tmAux, &tmIn, g, (int)blockIdx.x, (int)gridDim.x, smem_raw);
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

int make_gemm_tmaps(const cgk_gemm_args& a, int BN, CUtensorMap* tmA, CUtensorMap* tmB) {
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
    rc = encode_tmap(tmA, a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B128);
    if (rc) return rc;
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a.b_mn) {
      dims[0] = (uint64_t)a.K; dims[1] = (uint64_t)a.N;
      box[0] = BK; box[1] = (uint32_t)BN;
    } else {
      dims[0] = (uint64_t)a.N; dims[1] = (uint64_t)a.K;
      box[0] = 64; box[1] = BK;
    }
    dims[2] = (uint64_t)a.batch;
    strides[0] = (uint64_t)a.ldb * 2;
    strides[1] = (uint64_t)(a.batch > 1 ? a.strideB : (int64_t)dims[1] * a.ldb) * 2;
    box[2] = 1;
    rc = encode_tmap(tmB, a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B128);
    if (rc) return rc;
  }
  return 0;
}

// Tensor maps of the bf16 output and of the pre-activation output for the epilogue's bulk stores
// (box: 32 columns x 32 rows, 64-byte swizzle).  *ok = 0 when the layout rules them out; the
// epilogue then stores from registers.
int make_gemm_out_tmaps(const cgk_gemm_args& a, CUtensorMap* tmC, CUtensorMap* tmAux, CUtensorMap* tmIn, int* ok,
                        int* in_kind) {
  memset(tmC, 0, sizeof(*tmC));
  memset(tmAux, 0, sizeof(*tmAux));
  memset(tmIn, 0, sizeof(*tmIn));
  *ok = 0;
  *in_kind = 0;
  if (a.out_fp32 || a.accumulate || a.rope_cos || a.force_simt) return 0;
  if ((a.ldc % 8) != 0 || (((uintptr_t)a.out) & 15) != 0 || (a.batch > 1 && (a.strideC % 8) != 0)) return 0;
  if (a.aux_out && ((a.ldaux % 8) != 0 || (((uintptr_t)a.aux_out) & 15) != 0 || a.batch > 1)) return 0;
  uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.M, (uint64_t)a.batch};
  uint32_t box[3] = {32, 32, 1};
  {
    uint64_t strides[2] = {(uint64_t)a.ldc * 2, (uint64_t)(a.batch > 1 ? a.strideC : (long long)a.M * a.ldc) * 2};
    int rc = encode_tmap(tmC, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B64);
    if (rc) return rc;
  }
  if (a.aux_out) {
    uint64_t strides[2] = {(uint64_t)a.ldaux * 2, (uint64_t)((long long)a.M * a.ldaux) * 2};
    int rc = encode_tmap(tmAux, a.aux_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B64);
    if (rc) return rc;
  }
  *ok = 1;
  // one epilogue input by bulk loads: the activation-derivative operand, else the residual
  if (!a.aux_out && a.batch == 1) {
    const void* src = nullptr;
    long long ld = 0;
    int kind = 0;
    if (a.aux_in && (a.ldauxin % 8) == 0 && (((uintptr_t)a.aux_in) & 15) == 0) { src = a.aux_in; ld = a.ldauxin; kind = 1; }
    else if (a.residual && (a.ldr % 8) == 0 && (((uintptr_t)a.residual) & 15) == 0) { src = a.residual; ld = a.ldr; kind = 2; }
    if (kind) {
      uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)((long long)a.M * ld) * 2};
      int rc = encode_tmap(tmIn, src, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, Swz::B64);
      if (rc) return rc;
      *in_kind = kind;
    }
  }
  return 0;
}

int fill_gemm_dev(const cgk_gemm_args& a, GemmDev* pg) {
  GemmDev& g = *pg;
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  g = GemmDev{};
  g.M = a.M; g.N = a.N; g.K = a.K; g.batch = a.batch;
  g.a_mn = a.a_mn ? 1 : 0; g.b_mn = a.b_mn ? 1 : 0;
  g.out = a.out; g.ldc = a.ldc; g.strideC = a.strideC;
  g.out_fp32 = a.out_fp32; g.accumulate = a.accumulate;
  g.alpha = a.alpha;
  g.bias = a.bias; g.bias_fp32 = a.bias_fp32; g.act = a.act;
  g.residual = (const __nv_bfloat16*)a.residual; g.ldr = a.ldr;
  g.aux_out = (__nv_bfloat16*)a.aux_out; g.ldaux = a.ldaux;
  g.aux_in = (const __nv_bfloat16*)a.aux_in; g.ldauxin = a.ldauxin;
  g.dact = a.dact;
  g.rope_cos = a.rope_cos; g.rope_sin = a.rope_sin;
  g.rope_cols = a.rope_cols; g.rope_D = a.rope_D; g.rope_T = a.rope_T; g.rope_pos0 = a.rope_pos0;
  g.rope_inverse = a.rope_inverse;
  g.split_k = 1;
  g.kb_per_split = 0;
  g.status = device_status(dev);
  return 0;
}

bool gemm_tma_ok(const cgk_gemm_args& a) {
  return (a.lda % 8 == 0) && (a.ldb % 8 == 0) && (((uintptr_t)a.A & 15) == 0) &&
         (((uintptr_t)a.B & 15) == 0) &&
         (a.batch == 1 || (a.strideA % 8 == 0 && a.strideB % 8 == 0)) && a.K > 0;
}

int gemm_rope_ok(const cgk_gemm_args& a) {
  CGK_REQUIRE(a.rope_sin && (a.rope_D == 64 || a.rope_D == 128) && a.rope_cols > 0 && a.rope_cols % a.rope_D == 0 &&
                  a.rope_cols <= a.N && a.rope_T > 0 && a.rope_pos0 >= 0,
              "gemm: rotary epilogue needs sin/cos tables, head_dim 64 or 128 and whole heads");
  CGK_REQUIRE(a.batch == 1 && !a.out_fp32 && !a.accumulate && a.act == 0 && !a.residual && !a.aux_out && !a.aux_in &&
                  a.N % 32 == 0 && a.ldc % 8 == 0 && (((uintptr_t)a.out) & 15) == 0 && !a.force_simt && gemm_tma_ok(a),
              "gemm: the rotary epilogue takes a plain bf16 2-D output (bias allowed), N a multiple of 32");
  return 0;
}

int pick_bn(const cgk_gemm_args& a, int ctas) {
  if (a.rope_cos) return 256;       // both halves of a tile's columns must hold whole heads of up to 128 elements
  const long long tm = (a.M + BM - 1) / BM;
  auto tiles = [&](int bn) { return (long long)a.batch * tm * ((a.N + bn - 1) / bn); };
  // Widest tile that still gives every SM work; narrow tiles for small problems.
  if (a.N > 128 && tiles(256) >= (long long)ctas * 3 / 4) return 256;
  if (a.N > 64 && tiles(128) >= (long long)ctas / 2) return 128;
  return 64;
}

template <int BN, int STAGES>
static int launch_tc(const cgk_gemm_args& a, const GemmDev& g0, int sms, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  GemmDev g = g0;
  g.tiles_m = (a.M + BM - 1) / BM;
  g.tiles_n = (a.N + BN - 1) / BN;
  CUtensorMap tmA, tmB, tmC, tmAux, tmIn;
  int rc = make_gemm_tmaps(a, BN, &tmA, &tmB);
  if (rc) return rc;
  int out_ok = 0, in_kind = 0;
  if ((rc = make_gemm_out_tmaps(a, &tmC, &tmAux, &tmIn, &out_ok, &in_kind))) return rc;
  g.tma_store = (out_ok && g.split_k == 1) ? 1 : 0;
  g.tma_in = g.tma_store ? in_kind : 0;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN, STAGES>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  int total = g.batch * g.tiles_m * g.tiles_n * g.split_k;
  int cap = a.max_ctas > 0 ? a.max_ctas : sms;
  int grid = total < cap ? total : cap;
  gemm_bf16_tc_kernel<BN, STAGES><<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmC, tmAux, tmIn, g);
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
  int rc = fill_gemm_dev(a, &g);
  if (rc) return rc;
  CGK_REQUIRE(a.batch == 1 || !(a.residual || a.aux_out || a.aux_in),
              "cgk_gemm_bf16: residual/aux epilogues are 2-D only");
  if (a.rope_cos) {
    int rc2 = gemm_rope_ok(a);
    if (rc2) return rc2;
  }
  if (a.force_simt || !gemm_tma_ok(a)) {
    dim3 grid((a.N + 31) / 32, (a.M + 31) / 32, a.batch);
    dim3 block(32, 32, 1);
    gemm_bf16_simt_kernel<<<grid, block, 0, stream>>>(
        (const __nv_bfloat16*)a.A, (const __nv_bfloat16*)a.B, a.lda, a.ldb, a.strideA, a.strideB, g);
    CGK_LAUNCH_CHECK();
    return 0;
  }
  const int sms = sm_count(dev);
  const int ctas = a.max_ctas > 0 && a.max_ctas < sms ? a.max_ctas : sms;
  // Split-K for accumulating fp32 outputs (weight gradients) whose tiles would leave SMs idle:
  // the widest tile the output allows, and as many K slices as fill the machine.
  const bool can_split = a.out_fp32 && a.accumulate && a.batch == 1 && !a.bias && a.act == 0 && !a.residual &&
                         !a.aux_out && !a.aux_in && a.split_k != 1 && (a.ldc % 4) == 0 &&
                         (((uintptr_t)a.out & 15) == 0) && (a.N % 32) == 0;
  if (can_split) {
    const int bn = a.N >= 192 ? 256 : (a.N >= 96 ? 128 : 64);
    const long long tiles = (long long)((a.M + BM - 1) / BM) * ((a.N + bn - 1) / bn);
    const int kblocks = (a.K + BK - 1) / BK;
    int S = a.split_k > 1 ? a.split_k : (int)(ctas / tiles);
    if (S > kblocks / 8) S = kblocks / 8;
    if (S >= 2 && (a.split_k > 1 || tiles * 4 < (long long)ctas * 3)) {
      g.kb_per_split = (kblocks + S - 1) / S;
      g.split_k = (kblocks + g.kb_per_split - 1) / g.kb_per_split;     // no empty slice
      switch (bn) {
        case 256: return launch_tc<256, 4>(a, g, sms, stream);
        case 128: return launch_tc<128, 6>(a, g, sms, stream);
        default: return launch_tc<64, 8>(a, g, sms, stream);
      }
    }
  }
  switch (pick_bn(a, a.max_ctas > 0 ? a.max_ctas : sms)) {
    case 256: return launch_tc<256, 4>(a, g, sms, stream);
    case 128: return launch_tc<128, 6>(a, g, sms, stream);
    default: return launch_tc<64, 8>(a, g, sms, stream);
  }
}

CGK_BOUNDS_READER(gemm_tcgen05)
