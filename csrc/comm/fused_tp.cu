// Tensor-parallel hot paths as ONE kernel each: the collective runs over NVLink peer
// memory from inside the kernel that does the tensor-core work, tile by tile.
//
//  (a) all-gather -> GEMM  (cgk_ag_gemm):  out[M, N] = gather_r(x_r)[M, K] . W^T
//      "Copy" CTAs pull the activation shards (the own one first, then the peers' in
//      ring order) straight into this GPU's gathered buffer with plain 16-byte loads,
//      every thread of the CTA with 16 loads in flight, and publish one flag per chunk of rows.
//      The remaining CTAs run the persistent tcgen05 GEMM; its TMA producer waits for
//      the chunk a tile needs and then loads it from local memory, so every remote
//      byte crosses NVLink once and the GEMM starts on the rows that are already here.
//      The gathered buffer is an output: the backward pass reuses it for dW.
//  (b) GEMM -> reduce-scatter (cgk_gemm_rs): out_r[M/P, N] = sum_p (x_p . W_p^T)[rows of r]
//      Every rank writes its bf16 partial product into its OWN symmetric buffer (fast
//      local stores) and, tile by tile, counts it on the flag of the row block's owner.
//      All ranks walk the row blocks in the same order (block 0 of every owner, then
//      block 1 of every owner ...), so a block is complete on all ranks at about the
//      same time.  "Reduce" CTAs of the same kernel wait for a row block of the own
//      shard, pull its P partials (P - 1 of them over NVLink, many loads in flight),
//      add them in rank order in fp32 (bitwise reproducible), apply bias / residual
//      and write the output shard.  GEMM CTAs join the reduction when they run out
//      of tiles.
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
  // multicast mode (null = pull mode): multicast address of the gathered buffer, and every
  // rank's chunk-flag array as mapped here
  uint8_t* mc_gathered;
  int* peer_flags[GEMM_MAX_RANKS];
};

// ---------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
               const __grid_constant__ CUtensorMap tmIn, const GemmDev g, const AgDev a) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x >= a.n_copy) {
    gemm_tc_body<BN, STAGES>(tmA, tmB, &tmC, &tmAux, &tmIn, g, (int)blockIdx.x - a.n_copy, (int)gridDim.x - a.n_copy, smem_raw);
    return;
  }
  // ------------------------------ copy CTAs ------------------------------
  __shared__ int ok_word;
  const int P = a.ranks, me = a.rank, c = (int)blockIdx.x;
  int* my_sig = a.sig[me];
  if (a.mc_gathered != nullptr) {
    // Multicast mode: every rank broadcasts its own shard through the switch into the
    // gathered buffers of all ranks (one store instead of P - 1), chunk by chunk, and sets
    // the chunk's flag on every rank.  A multicast store lands on every GPU at once, so
    // nothing is sent before all peers have announced that their kernel of this call is
    // running (their gathered buffer of the previous use is dead by then).
    const int t = (int)threadIdx.x;
    if (c == 0 && t < P && t != me) st_release_sys(a.sig[t] + me, a.epoch);
    int ok = 1;
    if (t < P && t != me)
      ok = flag_wait_ge_sys(my_sig + t, a.epoch, g.status, 3000 + t, CGK_PEER_WAIT_BUDGET_NS) ? 1 : 0;
    if (!__syncthreads_and(ok)) return;
    for (int j = c; j < a.chunks_per_shard; j += a.n_copy) {
      const long long off = (long long)j * a.chunk_bytes;
      long long n = a.shard_bytes - off;
      if (n > a.chunk_bytes) n = a.chunk_bytes;
      cta_multicast(a.shard[me] + off, a.mc_gathered + (long long)me * a.shard_bytes + off, n);
      __syncthreads();
      if (t < P) {
        __threadfence_system();
        st_release_sys(a.peer_flags[t] + me * a.chunks_per_shard + j, a.epoch);
      }
    }
    return;
  }
  if (c == 0 && threadIdx.x == 0) {
    // my shard is complete (stream order): tell every peer
    for (int p = 0; p < P; ++p)
      if (p != me) st_release_sys(a.sig[p] + me, a.epoch);
  }
  // Items are (source, chunk) pairs: the own shard first (a local copy), then the peers
  // in ring order, nearest neighbour first, so that no two ranks start on the same source.
  const int items = P * a.chunks_per_shard;
  int ready_src = me;          // sources whose "ready" word this CTA has seen
  bool ok = true;
  for (int it = c; it < items; it += a.n_copy) {
    const int d = it / a.chunks_per_shard, j = it % a.chunks_per_shard;
    const int src = (me + d) % P;
    if (src != ready_src) {
      if (threadIdx.x == 0)
        ok_word = flag_wait_ge_sys(my_sig + src, a.epoch, g.status, 3000 + src, CGK_PEER_WAIT_BUDGET_NS) ? 1 : 0;
      __syncthreads();
      ok = ok_word != 0;
      __syncthreads();
      if (!ok) break;
      ready_src = src;
    }
    const long long off = (long long)j * a.chunk_bytes;
    long long n = a.shard_bytes - off;
    if (n > a.chunk_bytes) n = a.chunk_bytes;
    cta_copy(a.shard[src] + off, a.gathered + (long long)src * a.shard_bytes + off, n);
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      st_release_gpu(a.chunk_flags + src * a.chunks_per_shard + j, a.epoch);
      // the last chunk pulled from a peer releases that peer's shard buffer
      if (src != me && atomicAdd(a.done_count + src, 1) == a.chunks_per_shard - 1) {
        a.done_count[src] = 0;
        st_release_sys(a.sig[src] + P + me, a.epoch);
      }
    }
  }
  if (c == 0 && threadIdx.x == 0 && ok) {
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
  const __nv_bfloat16* partial[GEMM_MAX_RANKS];   // every rank's [M][ld] partial product, offset to MY rows
  const __nv_bfloat16* mc_partial;   // multicast address of the same rows (null: sum the P copies here)
  long long ld;             // leading dimension of a partial row
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;  // [rows][ldr] or null
  long long ldr;
  __nv_bfloat16* out;       // [rows][ldo]
  long long ldo;
};

// Sums the P partials of `total` 16-byte vectors starting at row0; U vectors per thread
// per round, all U * P loads issued before the first add.
template <int P, int U>
__device__ __forceinline__ void reduce_block(const RsDev& r, int row0, int total, int vec_per_row) {
  for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * U) {
    uint4 ld[U][P];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < total) {
        const long long o = (long long)(row0 + i / vec_per_row) * r.ld + (long long)(i % vec_per_row) * 8;
#pragma unroll
        for (int s = 0; s < P; ++s) ld[u][s] = ld_cg_u4(r.partial[s] + o);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i >= total) break;
      const int row = row0 + i / vec_per_row, v = i % vec_per_row;
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll
      for (int s = 0; s < P; ++s) add_bf16x8(acc, ld[u][s]);
      if (r.bias) add_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(r.bias) + v));
      if (r.residual) add_bf16x8(acc, *(reinterpret_cast<const uint4*>(r.residual + (long long)row * r.ldr) + v));
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *(reinterpret_cast<uint4*>(r.out + (long long)row * r.ldo) + v) = o;
    }
  }
}

// The same with the sum done inside the NVSwitch: one load-reduce on the multicast address
// of the partial buffers returns the fp32-accumulated sum of all ranks' copies.
template <int U>
__device__ __forceinline__ void reduce_block_mc(const RsDev& r, int row0, int total, int vec_per_row) {
  for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * U) {
    uint4 ld[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < total)
        ld[u] = multimem_ld_reduce_bf16x8(r.mc_partial + (long long)(row0 + i / vec_per_row) * r.ld +
                                          (long long)(i % vec_per_row) * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i >= total) break;
      const int row = row0 + i / vec_per_row, v = i % vec_per_row;
      uint4 o = ld[u];
      if (r.bias || r.residual) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        add_bf16x8(acc, o);
        if (r.bias) add_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(r.bias) + v));
        if (r.residual) add_bf16x8(acc, *(reinterpret_cast<const uint4*>(r.residual + (long long)row * r.ldr) + v));
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      }
      *(reinterpret_cast<uint4*>(r.out + (long long)row * r.ldo) + v) = o;
    }
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmDev g, const RsDev r) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x >= r.n_reduce)
    gemm_tc_body<BN, STAGES>(tmA, tmB, nullptr, nullptr, nullptr, g, (int)blockIdx.x - r.n_reduce, (int)gridDim.x - r.n_reduce,
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
    const int total = min(128, r.rows - row0) * vec_per_row;
    // about sixteen 16-byte loads in flight per thread
    if (r.mc_partial != nullptr) {
      reduce_block_mc<8>(r, row0, total, vec_per_row);
    } else switch (r.ranks) {
      case 1: reduce_block<1, 8>(r, row0, total, vec_per_row); break;
      case 2: reduce_block<2, 8>(r, row0, total, vec_per_row); break;
      case 3: reduce_block<3, 4>(r, row0, total, vec_per_row); break;
      case 4: reduce_block<4, 4>(r, row0, total, vec_per_row); break;
      case 5: reduce_block<5, 2>(r, row0, total, vec_per_row); break;
      case 6: reduce_block<6, 2>(r, row0, total, vec_per_row); break;
      case 7: reduce_block<7, 2>(r, row0, total, vec_per_row); break;
      default: reduce_block<8, 2>(r, row0, total, vec_per_row); break;
    }
    // every arrival of this call has been counted; the next writers of this counter
    // belong to a later call on the same buffer parity, which cannot start before
    // this kernel has ended
    if (threadIdx.x == 0) r.flags[rb] = 0;
  }
}

template <int BN, int STAGES>
static int launch_ag(const cgk_gemm_args& ga, GemmDev g, const AgDev& a, int ctas, cudaStream_t st) {
  using L = GemmSmem<BN, STAGES>;
  g.tiles_m = (ga.M + BM - 1) / BM;
  g.tiles_n = (ga.N + BN - 1) / BN;
  CUtensorMap tmA, tmB, tmC, tmAux, tmIn;
  int rc = make_gemm_tmaps(ga, BN, &tmA, &tmB);
  if (rc) return rc;
  int out_ok = 0, in_kind = 0;
  if ((rc = make_gemm_out_tmaps(ga, &tmC, &tmAux, &tmIn, &out_ok, &in_kind))) return rc;
  g.tma_store = out_ok;
  g.tma_in = out_ok ? in_kind : 0;
  CGK_CUDA_CHECK(cudaFuncSetAttribute(ag_gemm_kernel<BN, STAGES>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  ag_gemm_kernel<BN, STAGES><<<ctas, GEMM_THREADS, L::TOTAL, st>>>(tmA, tmB, tmC, tmAux, tmIn, g, a);
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
  gemm_rs_kernel<BN, STAGES><<<ctas, GEMM_THREADS, L::TOTAL, st>>>(tmA, tmB, g, r);
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
  if (ga.rope_cos) {
    int rc2 = gemm_rope_ok(ga);
    if (rc2) return rc2;
  }
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
  a.chunk_flags = (int*)x.chunk_flag_ptrs[x.rank];
  a.done_count = x.done_count;
  a.mc_gathered = x.ranks > 1 ? (uint8_t*)x.mc_gathered : nullptr;
  for (int p = 0; p < x.ranks; ++p) a.peer_flags[p] = (int*)x.chunk_flag_ptrs[p];
  CGK_REQUIRE(a.chunk_flags != nullptr, "cgk_ag_gemm: no chunk flags");
  const int sms = sm_count(dev);
  const int ctas = ga.max_ctas > 0 && ga.max_ctas < sms ? ga.max_ctas : sms;
  if (x.n_copy_ctas > 0) {
    a.n_copy = x.n_copy_ctas;
  } else if (a.mc_gathered != nullptr) {
    // Each rank only reads its own shard (local) and issues one multicast store per 16 bytes;
    // a CTA moves 15-20 GB/s that way.  Enough of them to finish in the longer of (the time
    // the other ranks' shards need to come in at NVLink rate) and (half of the GEMM's time).
    const double t_link = (double)(x.ranks - 1) * (double)a.shard_bytes / 700e9;
    const double t_gemm = 2.0 * ga.M * (double)ga.N * ga.K / 1.0e15 +
                          2.0 * ((double)ga.M * ga.N + (double)ga.M * ga.K) / 5.0e12;
    const double t = t_link > 0.5 * t_gemm ? t_link : 0.5 * t_gemm;
    a.n_copy = (int)((double)a.shard_bytes / (t * 15e9) + 0.999);
    if (a.n_copy < 4) a.n_copy = 4;
    if (a.n_copy > 24) a.n_copy = 24;
  } else if (x.ranks == 1) {
    a.n_copy = 8;
  } else {
    // Enough copy CTAs to finish the gather in the longer of (its time at NVLink rate) and
    // (a good part of the GEMM's time on the remaining SMs); one CTA pulls about 22 GB/s.
    const double remote = (double)(x.ranks - 1) * (double)a.shard_bytes;
    const double t_link = remote / 700e9;
    const double t_gemm = 2.0 * ga.M * (double)ga.N * ga.K / 1.0e15 +
                          2.0 * ((double)ga.M * ga.N + (double)ga.M * ga.K) / 5.0e12;
    const double t = t_link > 0.6 * t_gemm ? t_link : 0.6 * t_gemm;
    a.n_copy = (int)(remote / (t * 22e9) + 0.999);
    if (a.n_copy < 4) a.n_copy = 4;
    if (a.n_copy > 40) a.n_copy = 40;
  }
  if (a.n_copy > ctas / 2) a.n_copy = ctas / 2;
  if (a.n_copy < 1) a.n_copy = 1;
  g.a_ready = a.chunk_flags;
  g.a_ready_rows = x.chunk_rows;
  g.a_ready_target = x.epoch;
  if (a.mc_gathered != nullptr) {
    g.m_inter = x.ranks;               // all shards arrive at the same pace: block b of each in turn
    g.m_src0 = x.rank;
  } else {
    g.m_rot = x.rank * (rows / BM);    // start on the own rows, then follow the pull order
  }
  const int gemm_ctas = ctas - a.n_copy;
  switch (pick_bn(ga, gemm_ctas)) {
    case 256: return launch_ag<256, 4>(ga, g, a, ctas, (cudaStream_t)stream);
    case 128: return launch_ag<128, 6>(ga, g, a, ctas, (cudaStream_t)stream);
    default: return launch_ag<64, 8>(ga, g, a, ctas, (cudaStream_t)stream);
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
  CGK_REQUIRE(!ga.residual && !ga.aux_out && !ga.aux_in && !ga.bias && ga.act == 0 && !ga.rope_cos,
              "cgk_gemm_rs: epilogue terms are applied after the reduction (pass bias / residual in cgk_rs_args)");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  GemmDev g;
  int rc = fill_gemm_dev(ga, &g);
  if (rc) return rc;
  const int rows = ga.M / x.ranks;
  const int sms = sm_count(dev);
  const int ctas = ga.max_ctas > 0 && ga.max_ctas < sms ? ga.max_ctas : sms;
  // measured on 8 GPUs (131072 x 768 rows, all 148 CTAs): 8 reduce CTAs 0.373 ms, 16: 0.357, 32: 0.336,
  // 64: 0.344.  A kernel capped well below the machine (two of them run side by side in the two-stream
  // schedule, 56 CTAs each) keeps 16: its GEMM tiles would otherwise become the longer part.
  int n_reduce = x.n_reduce_ctas > 0 ? x.n_reduce_ctas : (x.ranks >= 4 && ctas >= 100 ? 32 : (x.ranks > 1 ? 16 : 4));
  if (n_reduce > ctas / 2) n_reduce = ctas / 2;
  if (n_reduce < 1) n_reduce = 1;
  const int gemm_ctas = ctas - n_reduce;
  const int bn = pick_bn(ga, gemm_ctas);
  g.rs_ranks = x.ranks;
  g.rs_rows = rows;
  g.ldc = x.ld;
  g.out_fp32 = 0; g.accumulate = 0;
  __nv_bfloat16* mine = (__nv_bfloat16*)x.partial_ptrs[x.rank];
  for (int p = 0; p < x.ranks; ++p) {
    g.rs_dst[p] = mine + (long long)p * rows * x.ld;      // rows of owner p in MY partial buffer
    g.rs_flag[p] = (int*)x.flag_ptrs[p];
  }
  g.m_inter = x.ranks;                                    // block b of every owner before block b + 1
  RsDev r{};
  r.rank = x.rank; r.ranks = x.ranks; r.n_reduce = n_reduce;
  r.rows = rows; r.N = ga.N;
  r.target = x.ranks * ((ga.N + 63) / 64);
  r.flags = (int*)x.flag_ptrs[x.rank];
  r.queue = x.queue;
  r.queue_base = x.queue_base;
  for (int p = 0; p < x.ranks; ++p)
    r.partial[p] = (const __nv_bfloat16*)x.partial_ptrs[p] + (long long)x.rank * rows * x.ld;
  r.mc_partial = (x.ranks > 1 && x.mc_partial) ? (const __nv_bfloat16*)x.mc_partial + (long long)x.rank * rows * x.ld
                                              : nullptr;
  r.ld = x.ld;
  r.bias = (const __nv_bfloat16*)x.bias;
  r.residual = (const __nv_bfloat16*)x.residual; r.ldr = x.ldr;
  r.out = (__nv_bfloat16*)x.out; r.ldo = x.ldo;
  switch (bn) {
    case 256: return launch_rs<256, 4>(ga, g, r, ctas, (cudaStream_t)stream);
    case 128: return launch_rs<128, 6>(ga, g, r, ctas, (cudaStream_t)stream);
    default: return launch_rs<64, 8>(ga, g, r, ctas, (cudaStream_t)stream);
  }
}

// Every CTA of the launch takes one ticket past the last row block before it leaves.
CGK_API int cgk_gemm_rs_queue_step(int M, int ranks, int max_ctas) {
  int dev = 0;
  cudaGetDevice(&dev);
  const int rows = M / (ranks > 0 ? ranks : 1);
  const int sms = sm_count(dev);
  return (rows + 127) / 128 + (max_ctas > 0 && max_ctas < sms ? max_ctas : sms);
}
