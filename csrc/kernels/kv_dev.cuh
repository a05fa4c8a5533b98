// Device-side view of one layer of the paged INT4 KV cache, shared by the kernels that touch it.
// Pool layout per layer: pages[num_pages][page_size][heads][D/2] bytes and
// scales[num_pages][page_size][heads][D/group] fp32; page_table[batch][max_pages] maps a
// sequence's logical page to a pool page; lengths[batch] tokens are valid.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace cgk {
struct KvDev {
  uint8_t* k_pages; uint8_t* v_pages; float* k_scales; float* v_scales;
  const int* page_table; const int* lengths;
  int batch, heads, D, group, page_size, max_pages;
};

// Tensor-core attention over the cache for head_dim 128 and a quantisation group that is a
// multiple of 32.  Writes per-split partials in the layout kv_combine_kernel reads:
// part_acc [rows][splits][128], part_ml [rows][splits][2] with rows = batch * heads * Tq * rep.
cudaError_t launch_kv_attention_tc(const KvDev& c, const __nv_bfloat16* q, int Tq, int Hq, float scale, int splits,
                                   float* part_acc, float* part_ml, int* status, cudaStream_t stream);
}  // namespace cgk
