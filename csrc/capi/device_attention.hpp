// Part of device.cpp (included at its end): attention and RoPE entry points of the cg_cuda_* API.
// Device tensors are fp32 [batch, seq, heads, d_head]; the tcgen05 flash kernels take bf16, so
// each call converts its operands into scratch, runs the kernel and converts the result back.
// Reference counterparts: src/cuda/flash_attn_kernels.c:531-629 (forward launch, wrappers,
// RoPE launch) and :401-525, :656-682 (backward passes that exist there only as host loops).
#pragma once

namespace {

struct AttnDims { int B, Tq, Tk, H, Hk, D; };
bool attn_dims(const cg_flash_attn_params* p, AttnDims* d) {
  if (!p || !p->Q || !p->K || !p->V || p->Q->ndim != 4 || p->K->ndim != 4 || p->V->ndim != 4) return false;
  d->B = p->Q->shape[0]; d->Tq = p->Q->shape[1]; d->H = p->Q->shape[2]; d->D = p->Q->shape[3];
  d->Tk = p->K->shape[1]; d->Hk = p->K->shape[2];
  return p->K->shape[0] == d->B && p->K->shape[3] == d->D && p->V->size == p->K->size && d->Hk > 0 && d->H % d->Hk == 0;
}

// fp32 device tensor -> bf16 scratch copy
void* to_bf16(cgdev::Scratch& sc, const cg_tensor* t) {
  void* p = sc.get((size_t)t->size * 2);
  if (p && !ok(S().k.cast(t->data, p, t->size, 1, stream()), "cast to bf16")) return nullptr;
  return p;
}

void set_strides(int64_t* bs, int64_t* ts, int64_t* hs, int T, int H, int D) { *hs = D; *ts = (int64_t)H * D; *bs = (int64_t)T * H * D; }

// Fills the fields shared by forward and backward.  Returns false for what the device kernels
// do not cover (arbitrary additive masks, other head sizes).
bool fill_flash(const cg_flash_attn_params* p, const AttnDims& d, cgdev::Scratch& sc, cgk_flash_args* a) {
  if (d.D != 64 && d.D != 128) { note_error("device attention needs d_head 64 or 128"); return false; }
  if (p->mask_type == CG_MASK_CUSTOM) { note_error("device attention takes causal / sliding-window masks and ALiBi, not a mask tensor"); return false; }
  std::memset(a, 0, sizeof(*a));
  a->B = d.B; a->Hq = d.H; a->Hk = d.Hk; a->Tq = d.Tq; a->Tk = d.Tk; a->D = d.D;
  set_strides(&a->q_bs, &a->q_ts, &a->q_hs, d.Tq, d.H, d.D);
  set_strides(&a->o_bs, &a->o_ts, &a->o_hs, d.Tq, d.H, d.D);
  set_strides(&a->dq_bs, &a->dq_ts, &a->dq_hs, d.Tq, d.H, d.D);
  set_strides(&a->k_bs, &a->k_ts, &a->k_hs, d.Tk, d.Hk, d.D);
  set_strides(&a->v_bs, &a->v_ts, &a->v_hs, d.Tk, d.Hk, d.D);
  set_strides(&a->dk_bs, &a->dk_ts, &a->dk_hs, d.Tk, d.Hk, d.D);
  set_strides(&a->dv_bs, &a->dv_ts, &a->dv_hs, d.Tk, d.Hk, d.D);
  a->scale = p->softmax_scale > 0 ? p->softmax_scale : 1.0f / std::sqrt((float)d.D);
  a->causal = p->mask_type == CG_MASK_CAUSAL || p->mask_type == CG_MASK_SLIDING_WINDOW;
  // the host oracle hides keys at distance >= window_size; the kernel keeps |distance| <= window
  a->window = p->mask_type == CG_MASK_SLIDING_WINDOW && p->window_size > 0 ? p->window_size - 1 : -1;
  if (p->alibi_slopes) {
    float* sl = (float*)sc.get(sizeof(float) * (size_t)d.H);
    if (!sl || !ok(S().k.dev_memcpy(sl, p->alibi_slopes, sizeof(float) * (size_t)d.H, 0, stream(), 0), "ALiBi slopes")) return false;
    a->alibi_slopes = sl;
  }
  a->q = to_bf16(sc, p->Q); a->k = to_bf16(sc, p->K); a->v = to_bf16(sc, p->V);
  return a->q && a->k && a->v;
}

// A tensor the parameter block owns (O, L, dQ, dK, dV): made on the device when missing, and
// remade there when cg_flash_attn_params_new left a host tensor in the slot.
cg_tensor* ensure_dev(cg_tensor*& slot, const int* shape, int ndim) {
  int n = 1;
  for (int i = 0; i < ndim; ++i) n *= shape[i];
  if (slot && (slot->size != n || !is_dev_ptr(slot->data))) { cg_tensor_release(slot); slot = nullptr; }
  if (!slot) slot = cg_tensor_cuda_new(const_cast<int*>(shape), ndim, false);
  return slot;
}
cg_tensor* ensure_dev_like(cg_tensor*& slot, const cg_tensor* like) { return ensure_dev(slot, like->shape, like->ndim); }

void rope_impl(float* x, int B, int T, int H, int D, float* cos_c, float* sin_c, int offset, bool backward) {
  if (!x || !cos_c || !sin_c) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (D % 2 || offset < 0) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (dev()) {
    ok(S().k.rope_apply(0, x, cos_c, sin_c, nullptr, B, T, H, D, (long long)T * H * D, (long long)H * D, D, offset, offset + T,
                        backward ? 1 : 0, stream()), "RoPE");
    return;
  }
  const int half = D / 2;
  for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) for (int h = 0; h < H; ++h) {
    float* v = x + (((size_t)b * T + t) * H + h) * D;
    const float* c = cos_c + (size_t)(t + offset) * half; const float* s = sin_c + (size_t)(t + offset) * half;
    for (int i = 0; i < half; ++i) {
      const float x0 = v[i], x1 = v[i + half], sn = backward ? -s[i] : s[i];
      v[i] = x0 * c[i] - x1 * sn; v[i + half] = x0 * sn + x1 * c[i];
    }
  }
}

}  // namespace

CG_EXPORT void cg_flash_attention_forward_cuda(cg_flash_attn_params* p) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (!dev()) { cg_flash_attention_forward_cpu(p); return; }
  AttnDims d;
  if (!attn_dims(p, &d)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (!operands_ok({p->Q, p->K, p->V})) return;
  cgdev::Scratch sc;
  cgk_flash_args a;
  if (!fill_flash(p, d, sc, &a)) return;
  const int ls[3] = {d.B, d.H, d.Tq};
  if (!ensure_dev_like(p->O, p->Q) || !ensure_dev(p->L, ls, 3)) return;
  a.o = sc.get((size_t)p->O->size * 2);
  a.lse = p->L->data;
  if (!a.o || !ok(S().k.flash_forward(&a, stream()), "flash attention forward")) return;
  ok(S().k.cast(a.o, p->O->data, p->O->size, 0, stream()), "cast to fp32");
}

CG_EXPORT void cg_flash_attention_backward_cuda(cg_flash_attn_params* p) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (!dev()) { cg_flash_attention_backward_cpu(p); return; }
  AttnDims d;
  if (!attn_dims(p, &d)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (!p->dO || !p->O || !p->L) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (!operands_ok({p->Q, p->K, p->V, p->O, p->dO, p->L})) return;
  cgdev::Scratch sc;
  cgk_flash_args a;
  if (!fill_flash(p, d, sc, &a)) return;
  if (!ensure_dev_like(p->dQ, p->Q) || !ensure_dev_like(p->dK, p->K) || !ensure_dev_like(p->dV, p->V)) return;
  a.o = to_bf16(sc, p->O);
  a.d_o = to_bf16(sc, p->dO);
  a.lse = p->L->data;
  a.dq = sc.get((size_t)p->Q->size * 2); a.dk = sc.get((size_t)p->K->size * 2); a.dv = sc.get((size_t)p->V->size * 2);
  a.delta = (float*)sc.get(sizeof(float) * (size_t)d.B * d.H * d.Tq);
  a.dq_accum = (float*)sc.get(sizeof(float) * (size_t)p->Q->size);
  if (!a.o || !a.d_o || !a.dq || !a.dk || !a.dv || !a.delta || !a.dq_accum) return;
  if (!ok(S().k.flash_backward(&a, stream()), "flash attention backward")) return;
  State& s = S();
  ok(s.k.cast(a.dq, p->dQ->data, p->Q->size, 0, stream()), "cast to fp32");
  ok(s.k.cast(a.dk, p->dK->data, p->K->size, 0, stream()), "cast to fp32");
  ok(s.k.cast(a.dv, p->dV->data, p->V->size, 0, stream()), "cast to fp32");
}

CG_EXPORT void cg_flash_attention_mqa_cuda(cg_flash_attn_params* p) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (flash_raw_block(p)) { cg_flash_attention_mqa(p); return; }                    // host mode
  if (!p || !p->K) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (p->K->ndim != 4 || p->K->shape[2] != 1) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  p->n_kv_heads = 1;
  cg_flash_attention_forward_cuda(p);
}
CG_EXPORT void cg_flash_attention_gqa_cuda(cg_flash_attn_params* p, int num_kv_groups) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (flash_raw_block(p)) { cg_flash_attention_gqa(p, num_kv_groups); return; }     // host mode
  if (!p || !p->K || !p->Q) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (num_kv_groups <= 0 || p->K->ndim != 4 || p->K->shape[2] != num_kv_groups || p->Q->shape[2] % num_kv_groups) {
    set_error(CG_ERROR_SHAPE_MISMATCH); return;
  }
  p->n_kv_heads = num_kv_groups;
  cg_flash_attention_forward_cuda(p);
}
CG_EXPORT void cg_flash_attention_sliding_window_cuda(cg_flash_attn_params* p, int window_size) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (flash_raw_block(p)) { p->mask_type = CG_MASK_SLIDING_WINDOW; p->window_size = window_size; cg_flash_attention_forward_cpu(p); return; }   // host mode
  if (!p) { set_error(CG_ERROR_NULL_POINTER); return; }
  p->mask_type = CG_MASK_SLIDING_WINDOW;
  p->window_size = window_size;
  cg_flash_attention_forward_cuda(p);
}

// Rotates x in place: element i pairs with i + d_head/2, angles from row (t + position_offset) of the caches.
CG_EXPORT void cg_rope_forward_cuda(float* x, int batch, int seqlen, int n_heads, int d_head, float* cos_cache, float* sin_cache,
                                    int position_offset) {
  rope_impl(x, batch, seqlen, n_heads, d_head, cos_cache, sin_cache, position_offset, false);
}
CG_EXPORT void cg_rope_backward_cuda(float* dx, int batch, int seqlen, int n_heads, int d_head, float* cos_cache, float* sin_cache,
                                     int position_offset) {
  rope_impl(dx, batch, seqlen, n_heads, d_head, cos_cache, sin_cache, position_offset, true);
}

// RoPE on Q and K (in place, as the reference's fused entry point leaves them), then attention.
CG_EXPORT void cg_flash_attention_forward_rope_cuda(cg_flash_attn_params* p, float* cos_cache, float* sin_cache, int position_offset) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (flash_raw_block(p)) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }         // rotary embedding and paged keys take tensor blocks
  AttnDims d;
  if (!attn_dims(p, &d)) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (!operands_ok({p->Q, p->K})) return;
  // queries are the last Tq positions of the Tk keys
  rope_impl(p->Q->data, d.B, d.Tq, d.H, d.D, cos_cache, sin_cache, position_offset + d.Tk - d.Tq, false);
  rope_impl(p->K->data, d.B, d.Tk, d.Hk, d.D, cos_cache, sin_cache, position_offset, false);
  cg_flash_attention_forward_cuda(p);
}

// Paged keys / values: p->K and p->V are block pools [num_blocks, block_size, kv_heads, d_head];
// block_tables (host, [batch, ceil(max_context_len / block_size)]) names each sequence's blocks in
// order.  The blocks are gathered into contiguous [batch, context, kv_heads, d_head] tensors (one
// device copy per block) and attended with the flash kernel; every sequence has max_context_len
// keys.  (The reference's entry point only prints "not yet implemented",
// src/cuda/flash_attn_kernels.c:601-611.)
CG_EXPORT void cg_flash_attention_paged_cuda(cg_flash_attn_params* p, int* block_tables, int block_size, int max_context_len) {
  if (dev() && flash_raw_block(p)) { note_error("raw-array parameter blocks run on the host; on a device use cg_flash_attn_params_new"); set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (flash_raw_block(p)) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (!p || !p->Q || !p->K || !p->V || !block_tables) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (p->Q->ndim != 4 || p->K->ndim != 4 || p->V->ndim != 4 || block_size <= 0 || max_context_len <= 0 ||
      p->K->shape[1] != block_size || p->V->size != p->K->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (!operands_ok({p->Q, p->K, p->V})) return;
  const int B = p->Q->shape[0], Hk = p->K->shape[2], D = p->K->shape[3], pool = p->K->shape[0];
  const int ctx = max_context_len;
  const int per_seq = (max_context_len + block_size - 1) / block_size;
  int shape[4] = {B, ctx, Hk, D};
  cg_tensor* Kc = cg_tensor_cuda_new(shape, 4, false), *Vc = cg_tensor_cuda_new(shape, 4, false);
  bool good = Kc && Vc;
  const size_t tok = (size_t)Hk * D;
  for (int b = 0; good && b < B; ++b) for (int t0 = 0; t0 < ctx; t0 += block_size) {
    const int blk = block_tables[(size_t)b * per_seq + t0 / block_size];
    if (blk < 0 || blk >= pool) { note_error("block table entry outside the pool"); good = false; break; }
    const int nt = ctx - t0 < block_size ? ctx - t0 : block_size;
    const size_t dst = ((size_t)b * ctx + t0) * tok, src = (size_t)blk * block_size * tok, bytes = sizeof(float) * nt * tok;
    cg_cuda_memcpy_async(Kc->data + dst, p->K->data + src, bytes, CG_MEMCPY_DEVICE_TO_DEVICE, nullptr);
    cg_cuda_memcpy_async(Vc->data + dst, p->V->data + src, bytes, CG_MEMCPY_DEVICE_TO_DEVICE, nullptr);
  }
  if (good) {
    cg_tensor* K0 = p->K, *V0 = p->V;
    const int sk = p->seqlen_k;
    p->K = Kc; p->V = Vc; p->seqlen_k = ctx;
    cg_flash_attention_forward_cuda(p);
    p->K = K0; p->V = V0; p->seqlen_k = sk;
  }
  cg_cuda_stream_synchronize(nullptr);
  cg_tensor_free(Kc);
  cg_tensor_free(Vc);
}

// Tile shape of the forward kernel of this library: 256 query rows per CTA (two 128-row halves,
// S and O accumulators in tensor memory) against 128-key blocks; sm_version is accepted for
// source compatibility and ignored (one architecture, sm_100a).
CG_EXPORT void cg_flash_attn_get_tile_sizes(int d_head, int sm_version, int* block_m, int* block_n) {
  (void)sm_version; (void)d_head;
  if (block_m) *block_m = 256;
  if (block_n) *block_n = 128;
}
CG_EXPORT size_t cg_flash_attn_estimate_shmem(int block_m, int block_n, int d_head) { return cg_flash_attn_shared_mem(block_m, block_n, d_head); }
CG_EXPORT bool cg_flash_attn_check_config(int block_m, int block_n, int d_head, size_t max_shmem) {
  if (block_m <= 0 || block_n <= 0 || d_head <= 0 || block_m % 64 || block_n % 16 || d_head % 16) return false;
  return cg_flash_attn_estimate_shmem(block_m, block_n, d_head) <= max_shmem;
}
