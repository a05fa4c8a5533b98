// Tensor-parallel hot paths as ONE kernel each: the collective runs over NVLink peer
// memory from inside the kernel that does the tensor-core work, tile by tile.
//
//  (a) all-gather -> GEMM  (cgk_ag_gemm):  out[M, N] = gather_r(x_r)[M, K] . W^T
//      A few "copy" CTAs pull the peers' activation shards into this GPU's gathered
//      buffer with bulk async copies (peer -> shared memory ring -> local HBM),
//      chunk by chunk in ring order starting at the own shard, and publish one
//      flag per chunk.  The remaining CTAs run the persistent tcgen05 GEMM; its
//      TMA producer waits for the chunk a tile needs and then loads it from local
//      memory, so every remote byte crosses NVLink once and the GEMM starts on
//      the rows that are already here.  The gathered buffer is an output: the
//      backward pass reuses it for dW.
//  (b) GEMM -> reduce-scatter (cgk_gemm_rs): out_r[M/P, N] = sum_p (x_p . W_p^T)[rows of r]
//      The GEMM epilogue stores each bf16 partial tile straight into its owner's
//      staging slot (a P2P store for remote owners) and bumps a per-row-block flag
//      on the owner.  "Reduce" CTAs of the same kernel wait for a row block to be
//      complete, add the P slots in rank order in fp32 (bitwise reproducible),
//      apply bias / residual and write the output shard.  Tiles are walked
//      starting after the own rank, so remote rows leave first.
//
// Handshakes use epoch-numbered words in symmetric memory (no reset pass).  Every
// wait is bounded and reports through the device status word.
//
// Reference counterparts: cg_tp_column_parallel_forward (local matmul then
// ncclAllGather, src/pipeline/tensor_parallel.c:31-75) and
// cg_tp_row_parallel_forward (local matmul then ncclAllReduce, :81-105).
#include "../kernels/gemm_host.h"
#include "comm_device.cuh"

namespace cgk {

struct AgDev {
  int rank, ranks;
  int epoch;                         // > 0, increases by one per call on this workspace
  const uint8_t* shard[GEMM_MAX_RANKS];   // peers' shard buffers (own included)
  int* sig[GEMM_MAX_RANKS];          // peers' signal words: [0..P) ready, [P..2P) done
  uint8_t* gathered;                 // local [M, K] bf16
  long long shard_bytes;             // bytes per rank
  long long chunk_bytes;             // bytes per readiness chunk
  int chunks_per_shard;
  int* chunk_flags;                  // local, [P * chunks_per_shard]
  int* done_count;                   // local, [P] scratch counters (zero between calls)
  int n_copy;
};

// ---------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(256, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmDev g, const AgDev a) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x >= a.n_copy) {
    gemm_tc_body<BN, STAGES>(tmA, tmB, g, (int)blockIdx.x - a.n_copy, (int)gridDim.x - a.n_copy, smem_raw);
    return;
  }
  // ------------------------------ copy CTAs ------------------------------
  if (threadIdx.x != 0) return;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ int dead_word;
  volatile int* dead = &dead_word;
  dead_word = 0;
  Relay relay;
  relay_init(relay, smem_u32(smem), smem_u32(smem) + RELAY_STAGES * RELAY_PIECE);
  const int P = a.ranks, me = a.rank, c = (int)blockIdx.x;
  int* my_sig = a.sig[me];
  if (c == 0) {
    // my shard is complete (stream order): tell every peer
    for (int p = 0; p < P; ++p)
      if (p != me) st_release_sys(a.sig[p] + me, a.epoch);
  }
  // the own shard is copied into the gathered buffer before the launch; only the
  // peers' shards go through the relay, nearest ring neighbour first
  const int items = (P - 1) * a.chunks_per_shard;
  bool ok = true;
  for (int it = c; it < items && ok; it += a.n_copy) {
    const int d = 1 + it / a.chunks_per_shard, j = it % a.chunks_per_shard;
    const int src = (me + d) % P;
    if (src != me) {
      if (!flag_wait_ge_sys(my_sig + src, a.epoch, g.status, 3000 + src, CGK_PEER_WAIT_BUDGET_NS)) { ok = false; break; }
    }
    const long long off = (long long)j * a.chunk_bytes;
    long long n = a.shard_bytes - off;
    if (n > a.chunk_bytes) n = a.chunk_bytes;
    if (!relay_copy(relay, a.shard[src] + off, a.gathered + (long long)src * a.shard_bytes + off, n, dead,
                    g.status)) { ok = false; break; }
    __threadfence();
    st_release_gpu(a.chunk_flags + src * a.chunks_per_shard + j, a.epoch);
    // the last chunk pulled from a peer releases that peer's shard buffer
    if (src != me && atomicAdd(a.done_count + src, 1) == a.chunks_per_shard - 1) {
      a.done_count[src] = 0;
      st_release_sys(a.sig[src] + P + me, a.epoch);
    }
  }
  if (c == 0 && ok) {
    // nobody may overwrite my shard buffer before every peer has pulled it
    for (int p = 0; p < P && ok; ++p)
      if (p != me) ok = flag_wait_ge_sys(my_sig + P + p, a.epoch, g.status, 3050 + p, CGK_PEER_WAIT_BUDGET_NS);
  }
}

// ---------------------------------------------------------------------------------
struct RsDev {
  int rank, ranks;
  int n_reduce;
  int rows;                 // rows of the output shard (M / P)
  int N;
  int target;               // flag value that marks a row block complete
  int* flags;               // local, [rows / 128]; a row block's counter is cleared once it is reduced
  int* queue;               // local work counter, grows by (blocks + CTAs) per call
  int queue_base;           // its value when this call starts
  const __nv_bfloat16* staging;   // local, [P][rows][ld]
  long long ld;             // leading dimension of a slot
  long long slot_elems;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;  // [rows][ldr] or null
  long long ldr;
  __nv_bfloat16* out;       // [rows][ldo]
  long long ldo;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(256, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmDev g, const RsDev r) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x >= r.n_reduce)
    gemm_tc_body<BN, STAGES>(tmA, tmB, g, (int)blockIdx.x - r.n_reduce, (int)gridDim.x - r.n_reduce,
                             smem_raw);
  // ------------------------------ reduce phase ------------------------------
  // A few CTAs reduce from the start; every GEMM CTA joins once it has run out of
  // tiles.  Row blocks are handed out in order through one counter.
  __shared__ int rb_word;
  const int blocks = (r.rows + 127) / 128;
  const int vec_per_row = r.N >> 3;
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) {
      int rb = atomicAdd(r.queue, 1) - r.queue_base;
      if (rb < blocks && !flag_wait_ge_sys(r.flags + rb, r.target, g.status, 3200, CGK_PEER_WAIT_BUDGET_NS))
        rb = blocks;     // give up: the status word says why
      rb_word = rb;
    }
    __syncthreads();
    const int rb = rb_word;
    if (rb >= blocks) break;
    const int row0 = rb * 128;
    const int nrows = min(128, r.rows - row0);
    // U vectors per thread per round so that about eight 16-byte loads are in flight
    const int U = r.ranks >= 8 ? 1 : (r.ranks >= 4 ? 2 : (r.ranks >= 2 ? 4 : 8));
    const int total = nrows * vec_per_row;
    for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * U) {
      uint4 ld[8];
#pragma unroll 4
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i >= total) break;
        const int row = row0 + i / vec_per_row, v = i % vec_per_row;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        // peers wrote these lines; read them past the L1.  The loads of all slots are
        // issued before the first add.
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s < r.ranks)
            ld[s] = __ldcg(reinterpret_cast<const uint4*>(r.staging + s * r.slot_elems + (long long)row * r.ld) + v);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s < r.ranks) {
            float2 f;
            f = unpack_bf16x2(ld[s].x); acc[0] += f.x; acc[1] += f.y;
            f = unpack_bf16x2(ld[s].y); acc[2] += f.x; acc[3] += f.y;
            f = unpack_bf16x2(ld[s].z); acc[4] += f.x; acc[5] += f.y;
            f = unpack_bf16x2(ld[s].w); acc[6] += f.x; acc[7] += f.y;
          }
        }
        if (r.bias) {
          const uint4 u4 = __ldg(reinterpret_cast<const uint4*>(r.bias) + v);
          float2 f;
          f = unpack_bf16x2(u4.x); acc[0] += f.x; acc[1] += f.y;
          f = unpack_bf16x2(u4.y); acc[2] += f.x; acc[3] += f.y;
          f = unpack_bf16x2(u4.z); acc[4] += f.x; acc[5] += f.y;
          f = unpack_bf16x2(u4.w); acc[6] += f.x; acc[7] += f.y;
        }
        if (r.residual) {
          const uint4 u4 = *(reinterpret_cast<const uint4*>(r.residual + (long long)row * r.ldr) + v);
          float2 f;
          f = unpack_bf16x2(u4.x); acc[0] += f.x; acc[1] += f.y;
          f = unpack_bf16x2(u4.y); acc[2] += f.x; acc[3] += f.y;
          f = unpack_bf16x2(u4.z); acc[4] += f.x; acc[5] += f.y;
          f = unpack_bf16x2(u4.w); acc[6] += f.x; acc[7] += f.y;
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *(reinterpret_cast<uint4*>(r.out + (long long)row * r.ldo) + v) = o;
      }
    }
    // every arrival of this call has been counted; the next writers of this counter
    // belong to a later call on the same buffer parity, which cannot start before
    // this kernel has ended
    if (threadIdx.x == 0) r.flags[rb] = 0;
    __syncthreads();
  }
}

template <int BN, int STAGES>
static int launch_ag(const cgk_gemm_args& ga, GemmDev g, const AgDev& a, int ctas, cudaStream_t st) {
  using L = GemmSmem<BN, STAGES>;
  static_assert(L::TOTAL >= RELAY_STAGES * (int)RELAY_PIECE + RELAY_STAGES * 8 + 1024, "relay ring does not fit");
  g.tiles_m = (ga.M + BM - 1) / BM;
  g.tiles_n = (ga.N + BN - 1) / BN;
  CUtensorMap tmA, tmB;
  int rc = make_gemm_tmaps(ga, BN, &tmA, &tmB);
  if (rc) return rc;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(ag_gemm_kernel<BN, STAGES>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  ag_gemm_kernel<BN, STAGES><<<ctas, 256, L::TOTAL, st>>>(tmA, tmB, g, a);
  CGK_LAUNCH_CHECK();
  return 0;
}

template <int BN, int STAGES>
static int launch_rs(const cgk_gemm_args& ga, GemmDev g, const RsDev& r, int ctas, cudaStream_t st) {
  using L = GemmSmem<BN, STAGES>;
  g.tiles_m = (ga.M + BM - 1) / BM;
  g.tiles_n = (ga.N + BN - 1) / BN;
  CUtensorMap tmA, tmB;
  int rc = make_gemm_tmaps(ga, BN, &tmA, &tmB);
  if (rc) return rc;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(gemm_rs_kernel<BN, STAGES>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  gemm_rs_kernel<BN, STAGES><<<ctas, 256, L::TOTAL, st>>>(tmA, tmB, g, r);
  CGK_LAUNCH_CHECK();
  return 0;
}

}  // namespace cgk

using namespace cgk;

// out = epilogue(gathered . B^T) with gathered[M, K] assembled from the P shards.
// g: the GEMM description with A = the LOCAL gathered buffer (M = P * shard rows).
// x: see cgk_ag_args in cogito_kernels.h.
CGK_API int cgk_ag_gemm(const cgk_gemm_args* pg, const cgk_ag_args* px, void* stream) {
  CGK_REQUIRE(pg && px, "cgk_ag_gemm: null args");
  const cgk_gemm_args& ga = *pg;
  const cgk_ag_args& x = *px;
  CGK_REQUIRE(x.ranks >= 1 && x.ranks <= GEMM_MAX_RANKS && x.rank >= 0 && x.rank < x.ranks, "cgk_ag_gemm: bad rank");
  CGK_REQUIRE(ga.batch == 1 && !ga.a_mn, "cgk_ag_gemm: A must be a row-major 2-D matrix");
  CGK_REQUIRE(ga.M % x.ranks == 0 && (ga.M / x.ranks) % BM == 0, "cgk_ag_gemm: rows per rank must be a multiple of 128");
  CGK_REQUIRE(ga.lda == ga.K && gemm_tma_ok(ga), "cgk_ag_gemm: gathered buffer must be dense and TMA-addressable");
  CGK_REQUIRE(x.epoch > 0 && x.chunk_rows > 0 && x.chunk_rows % BM == 0, "cgk_ag_gemm: bad epoch / chunk_rows");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  GemmDev g;
  int rc = fill_gemm_dev(ga, &g);
  if (rc) return rc;
  const int rows = ga.M / x.ranks;
  AgDev a{};
  a.rank = x.rank; a.ranks = x.ranks; a.epoch = x.epoch;
  for (int p = 0; p < x.ranks; ++p) { a.shard[p] = (const uint8_t*)x.shard_ptrs[p]; a.sig[p] = (int*)x.signal_ptrs[p]; }
  a.gathered = (uint8_t*)ga.A;
  a.shard_bytes = (long long)rows * ga.K * 2;
  a.chunk_bytes = (long long)x.chunk_rows * ga.K * 2;
  a.chunks_per_shard = (rows + x.chunk_rows - 1) / x.chunk_rows;
  a.chunk_flags = x.chunk_flags;
  a.done_count = x.done_count;
  const int sms = sm_count(dev);
  a.n_copy = x.n_copy_ctas > 0 ? x.n_copy_ctas : (x.ranks > 1 ? 20 : 1);
  if (a.n_copy > sms / 2) a.n_copy = sms / 2;
  g.a_ready = a.chunk_flags;
  g.a_ready_rows = x.chunk_rows;
  g.a_ready_target = x.epoch;
  g.m_rot = x.rank * (rows / BM);
  g.a_ready_skip_first = x.rank * a.chunks_per_shard;
  g.a_ready_skip_count = a.chunks_per_shard;
  const int gemm_ctas = sms - a.n_copy;
  switch (pick_bn(ga, gemm_ctas)) {
    case 256: return launch_ag<256, 4>(ga, g, a, sms, (cudaStream_t)stream);
    case 128: return launch_ag<128, 6>(ga, g, a, sms, (cudaStream_t)stream);
    default: return launch_ag<64, 8>(ga, g, a, sms, (cudaStream_t)stream);
  }
}

// out_shard[M/P, N] = bias + residual + sum_p partial_p[rows of this rank], where
// partial = A . B^T is this rank's [M, N] product.  See cgk_rs_args.
CGK_API int cgk_gemm_rs(const cgk_gemm_args* pg, const cgk_rs_args* px, void* stream) {
  CGK_REQUIRE(pg && px, "cgk_gemm_rs: null args");
  const cgk_gemm_args& ga = *pg;
  const cgk_rs_args& x = *px;
  CGK_REQUIRE(x.ranks >= 1 && x.ranks <= GEMM_MAX_RANKS && x.rank >= 0 && x.rank < x.ranks, "cgk_gemm_rs: bad rank");
  CGK_REQUIRE(ga.batch == 1 && gemm_tma_ok(ga), "cgk_gemm_rs: operands must be 2-D and TMA-addressable");
  CGK_REQUIRE(ga.M % x.ranks == 0 && (ga.M / x.ranks) % BM == 0, "cgk_gemm_rs: rows per rank must be a multiple of 128");
  CGK_REQUIRE(ga.N % 8 == 0 && x.ld % 8 == 0 && x.ldo % 8 == 0, "cgk_gemm_rs: N and leading dimensions must be multiples of 8");
  CGK_REQUIRE(!ga.residual && !ga.aux_out && !ga.aux_in && !ga.bias && ga.act == 0,
              "cgk_gemm_rs: epilogue terms are applied after the reduction (pass bias / residual in cgk_rs_args)");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  GemmDev g;
  int rc = fill_gemm_dev(ga, &g);
  if (rc) return rc;
  const int rows = ga.M / x.ranks;
  const int sms = sm_count(dev);
  int n_reduce = x.n_reduce_ctas > 0 ? x.n_reduce_ctas : 8;
  if (n_reduce > sms / 2) n_reduce = sms / 2;
  const int gemm_ctas = sms - n_reduce;
  const int bn = pick_bn(ga, gemm_ctas);
  g.rs_ranks = x.ranks;
  g.rs_rows = rows;
  g.ldc = x.ld;
  g.out_fp32 = 0; g.accumulate = 0;
  for (int p = 0; p < x.ranks; ++p) {
    g.rs_dst[p] = (__nv_bfloat16*)x.staging_ptrs[p] + (long long)x.rank * x.slot_elems;
    g.rs_flag[p] = (int*)x.flag_ptrs[p];
  }
  g.m_rot = ((x.rank + 1) % x.ranks) * (rows / BM);
  RsDev r{};
  r.rank = x.rank; r.ranks = x.ranks; r.n_reduce = n_reduce;
  r.rows = rows; r.N = ga.N;
  r.target = x.ranks * ((ga.N + 63) / 64);
  r.flags = (int*)x.flag_ptrs[x.rank];
  r.queue = x.queue;
  r.queue_base = x.queue_base;
  r.staging = (const __nv_bfloat16*)x.staging_ptrs[x.rank];
  r.ld = x.ld; r.slot_elems = x.slot_elems;
  r.bias = (const __nv_bfloat16*)x.bias;
  r.residual = (const __nv_bfloat16*)x.residual; r.ldr = x.ldr;
  r.out = (__nv_bfloat16*)x.out; r.ldo = x.ldo;
  switch (bn) {
    case 256: return launch_rs<256, 4>(ga, g, r, sms, (cudaStream_t)stream);
    case 128: return launch_rs<128, 6>(ga, g, r, sms, (cudaStream_t)stream);
    default: return launch_rs<64, 8>(ga, g, r, sms, (cudaStream_t)stream);
  }
}

// Every CTA of the launch takes one ticket past the last row block before it leaves.
CGK_API int cgk_gemm_rs_queue_step(int M, int ranks) {
  int dev = 0;
  cudaGetDevice(&dev);
  const int rows = M / (ranks > 0 ? ranks : 1);
  return (rows + 127) / 128 + sm_count(dev);
}
