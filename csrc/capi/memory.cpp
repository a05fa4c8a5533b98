// Caching pool (power-of-two bins plus exact-size sub-bins), buddy allocator, lifetime-based
// memory planner with compaction, and the capture / replay allocation trace.
// Reference surface: include/cg_memory.h, src/memory/planner.c.
// Fixes relative to the reference: bins cover 2^5 .. 2^40 without running past the table,
// sub-bin blocks return to their own list, frees look the block up in a hash map.
#include <algorithm>
#include <map>
#include <set>
#include <unordered_map>

#include "internal.hpp"

using namespace cgi;

namespace {
constexpr int kMinShift = 5, kBins = 36;            // 32 B .. 2^40 B
constexpr size_t kSub[3] = {768, 1024, 4096};
struct Block { size_t size; int bin; };             // bin >= 0 power-of-two, -1-i sub-bin i
}  // namespace

struct PoolImpl : cg_memory_pool {
  PoolImpl() : cg_memory_pool{} {}
  std::vector<void*> free_list[kBins];
  std::vector<void*> sub_free[3];
  std::unordered_map<void*, Block> live, cached;
  cg_memory_stats st{};
  size_t sub_hits = 0;
  // the counters of the public struct (the reference's names) follow the internal ones
  void sync() {
    total_in_use = st.total_allocated; total_allocated = st.total_allocated + st.total_cached; peak_usage = st.peak_allocated;
    num_allocs = (size_t)st.num_allocs; num_frees = (size_t)st.num_frees; cache_hits = (size_t)st.cache_hits;
    cache_misses = (size_t)st.cache_misses; subbin_hits = sub_hits;
  }
};
static PoolImpl* impl(cg_memory_pool* x) { return static_cast<PoolImpl*>(x); }

static int bin_of(size_t size) {
  int b = 0; size_t cap = (size_t)1 << kMinShift;
  while (cap < size && b < kBins - 1) { cap <<= 1; ++b; }
  return cap >= size ? b : -1;
}
CG_EXPORT int cg_subbin_index(size_t size) { for (int i = 0; i < 3; ++i) if (size == kSub[i]) return i; return -1; }
CG_EXPORT cg_memory_pool* cg_memory_pool_new(void) { return new PoolImpl(); }
static void* pool_take(cg_memory_pool* p_, std::vector<void*>& list, size_t cap, int bin, size_t want) { auto* p = impl(p_);
  void* ptr;
  if (!list.empty()) {
    ptr = list.back(); list.pop_back();
    p->cached.erase(ptr); p->st.total_cached -= cap; ++p->st.cache_hits;
    if (bin < 0) ++p->sub_hits;
  } else {
    if (posix_memalign(&ptr, 256, cap) != 0) return fail(CG_ERROR_OUT_OF_MEMORY, (void*)nullptr);
    ++p->st.cache_misses;
  }
  p->live[ptr] = {cap, bin};
  p->st.total_allocated += cap; ++p->st.num_allocs;
  if (p->st.total_allocated > p->st.peak_allocated) p->st.peak_allocated = p->st.total_allocated;
  (void)want;
  p->sync();
  return ptr;
}
CG_EXPORT void* cg_pool_alloc(cg_memory_pool* p_, size_t size) { auto* p = impl(p_);
  if (!p) return fail(CG_ERROR_NULL_POINTER, (void*)nullptr);
  if (size == 0) size = 1;
  const int sb = cg_subbin_index(size);
  if (sb >= 0) return pool_take(p, p->sub_free[sb], kSub[sb], -1 - sb, size);
  const int b = bin_of(size);
  if (b < 0) return fail(CG_ERROR_INVALID_ARGUMENT, (void*)nullptr);
  return pool_take(p, p->free_list[b], (size_t)1 << (kMinShift + b), b, size);
}
CG_EXPORT void* cg_pool_alloc_subbin(cg_memory_pool* p_, size_t size) { auto* p = impl(p_);
  if (cg_subbin_index(size) < 0) return fail(CG_ERROR_INVALID_ARGUMENT, (void*)nullptr);
  return cg_pool_alloc(p, size);
}
CG_EXPORT void cg_pool_free(cg_memory_pool* p_, void* ptr) { auto* p = impl(p_);
  if (!p || !ptr) return;
  auto it = p->live.find(ptr);
  if (it == p->live.end()) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  const Block b = it->second;
  p->live.erase(it);
  (b.bin >= 0 ? p->free_list[b.bin] : p->sub_free[-1 - b.bin]).push_back(ptr);
  p->cached[ptr] = b;
  p->st.total_allocated -= b.size; p->st.total_cached += b.size; ++p->st.num_frees;
  p->sync();
}
CG_EXPORT void cg_pool_trim(cg_memory_pool* p_) { auto* p = impl(p_);
  if (!p) return;
  for (auto& kv : p->cached) std::free(kv.first);
  p->cached.clear();
  for (auto& l : p->free_list) l.clear();
  for (auto& l : p->sub_free) l.clear();
  p->st.total_cached = 0;
  p->sync();
}
CG_EXPORT void cg_memory_pool_free(cg_memory_pool* p_) { auto* p = impl(p_);
  if (!p) return;
  cg_pool_trim(p);
  for (auto& kv : p->live) std::free(kv.first);
  delete p;
}
// The host library has one address space; the arena only selects the accounting bucket on the
// GPU side (device memory vs pinned host memory).
CG_EXPORT void* cg_pool_alloc_arena(cg_memory_pool* p_, size_t size, cg_arena_type) { auto* p = impl(p_); return cg_pool_alloc(p, size); }
CG_EXPORT void cg_pool_free_arena(cg_memory_pool* p_, void* ptr, cg_arena_type) { auto* p = impl(p_); cg_pool_free(p, ptr); }
// Share of the pool's bytes that sit unused in the cache.
CG_EXPORT float cg_memory_fragmentation(cg_memory_pool* p_) { auto* p = impl(p_);
  if (!p) return 0.0f;
  const double all = (double)p->st.total_allocated + (double)p->st.total_cached;
  return all > 0 ? (float)(p->st.total_cached / all) : 0.0f;
}
CG_EXPORT bool cg_memory_needs_compact(cg_memory_pool* p_, float threshold) { auto* p = impl(p_); return cg_memory_fragmentation(p) > threshold; }

// ------------------------------------------------------------------- buddy
struct BuddyImpl : cg_buddy_allocator {
  BuddyImpl() : cg_buddy_allocator{} {}
  char* base; size_t size; int max_order;            // block of order k = kMin << k
  std::vector<std::set<size_t>> free_at;             // offsets per order
  int splits = 0, coalesces = 0;
  void sync() { base_ptr = base; total_size = size; buddy_splits = (size_t)splits; buddy_coalesces = (size_t)coalesces; }
};
static BuddyImpl* impl(cg_buddy_allocator* x) { return static_cast<BuddyImpl*>(x); }
static constexpr size_t kBuddyMin = 256;
static int order_for(size_t size) { int k = 0; size_t cap = kBuddyMin; while (cap < size) { cap <<= 1; ++k; } return k; }
CG_EXPORT cg_buddy_allocator* cg_buddy_new(void* base, size_t size) {
  if (!base || size < kBuddyMin) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_buddy_allocator*)nullptr);
  BuddyImpl* b = new BuddyImpl();
  int k = 0; while ((kBuddyMin << (k + 1)) <= size) ++k;        // largest power of two that fits
  b->base = (char*)base; b->size = kBuddyMin << k; b->max_order = k;
  b->free_at.resize(k + 1);
  b->free_at[k].insert(0);
  b->sync();
  return b;
}
CG_EXPORT void* cg_buddy_alloc(cg_buddy_allocator* b_, size_t size) { auto* b = impl(b_);
  if (!b || size == 0) return fail(CG_ERROR_INVALID_ARGUMENT, (void*)nullptr);
  const int want = order_for(size);
  int k = want;
  while (k <= b->max_order && b->free_at[k].empty()) ++k;
  if (k > b->max_order) return fail(CG_ERROR_OUT_OF_MEMORY, (void*)nullptr);
  size_t off = *b->free_at[k].begin();
  b->free_at[k].erase(b->free_at[k].begin());
  while (k > want) { --k; b->free_at[k].insert(off + (kBuddyMin << k)); ++b->splits; }
  b->allocated += kBuddyMin << want;
  b->sync();
  return b->base + off;
}
CG_EXPORT void cg_buddy_free(cg_buddy_allocator* b_, void* ptr, size_t size) { auto* b = impl(b_);
  if (!b || !ptr) return;
  size_t off = (char*)ptr - b->base;
  int k = order_for(size);
  if (off >= b->size || off % (kBuddyMin << k)) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  b->allocated -= (kBuddyMin << k) <= b->allocated ? (kBuddyMin << k) : b->allocated;
  while (k < b->max_order) {
    const size_t buddy = off ^ (kBuddyMin << k);
    auto it = b->free_at[k].find(buddy);
    if (it == b->free_at[k].end()) break;
    b->free_at[k].erase(it);
    off = off < buddy ? off : buddy;
    ++k; ++b->coalesces;
  }
  b->free_at[k].insert(off);
  b->sync();
}
CG_EXPORT void cg_buddy_destroy(cg_buddy_allocator* b_) { auto* b = impl(b_); delete b; }
CG_EXPORT int cg_buddy_splits(cg_buddy_allocator* b_) { auto* b = impl(b_); return b ? b->splits : 0; }
CG_EXPORT int cg_buddy_coalesces(cg_buddy_allocator* b_) { auto* b = impl(b_); return b ? b->coalesces : 0; }

// ----------------------------------------------------------------- planner
namespace {
struct Life { int first = -1, last = -1; size_t bytes = 0; size_t offset = 0; bool planned = false; bool pinned = false; };
struct Trace { int tensor_id; size_t size; void* ptr; };
}  // namespace
struct PlannerImpl : cg_memory_planner {
  PlannerImpl() : cg_memory_planner{} {}
  cg_memory_pool* pools[2];
  std::map<int, Life> life;                         // tensor id -> lifetime and planned offset
  size_t plan_bytes = 0; char* slab = nullptr; size_t slab_bytes = 0;
  std::map<int, void*> handed;                      // tensor id -> pointer inside the slab
  int reuse_pairs = 0;
  bool capturing = false, captured = false, replaying = false, stale = true;
  std::vector<Trace> trace; size_t cursor = 0;
};
static PlannerImpl* impl(cg_memory_planner* x) { return static_cast<PlannerImpl*>(x); }
CG_EXPORT cg_memory_planner* cg_memory_planner_new(void) {
  PlannerImpl* p = new PlannerImpl();
  p->pools[0] = cg_memory_pool_new(); p->pools[1] = cg_memory_pool_new();
  p->device_pool = p->pools[0]; p->host_pool = p->pools[1];
  p->frag_threshold = 0.5f; p->defrag_enabled = true;
  return p;
}
CG_EXPORT cg_memory_pool* cg_memory_planner_pool(cg_memory_planner* p_, cg_arena_type a) { auto* p = impl(p_); return p ? p->pools[a == CG_ARENA_HOST ? 1 : 0] : nullptr; }
CG_EXPORT void cg_memory_planner_free(cg_memory_planner* p_) { auto* p = impl(p_);
  if (!p) return;
  cg_memory_pool_free(p->pools[0]); cg_memory_pool_free(p->pools[1]);
  std::free(p->slab);
  delete p;
}
// Lifetime of every tensor of the graph: produced at its node's position, dead after its last
// reader.  Graph inputs and outputs are pinned for the whole run.
CG_EXPORT void cg_analyze_tensor_lifetimes(cg_memory_planner* p_, void* ir_graph) { auto* p = impl(p_);
  cg_ir_graph* g = (cg_ir_graph*)ir_graph;
  if (!p || !g) { set_error(CG_ERROR_NULL_POINTER); return; }
  p->life.clear();
  int pos = 0;
  for (int i = 0; i < g->num_nodes; ++i) {
    cg_ir_node* n = g->nodes[i];
    if (n->dead) continue;
    for (int k = 0; k < n->num_inputs; ++k) { Life& l = p->life[n->input_ids[k]]; if (l.first < 0) { l.first = 0; l.pinned = true; } l.last = pos; }
    Life& o = p->life[n->output_id];
    if (o.first < 0) o.first = pos;
    if (o.last < pos) o.last = pos;
    ++pos;
  }
  for (int i = 0; i < g->num_outputs; ++i) { Life& l = p->life[g->output_node_ids[i]]; l.pinned = true; l.last = pos; }
  for (auto& kv : p->life) {
    const int id = kv.first;
    size_t n = 0;
    if (id >= 0 && id < g->num_tensors && g->tensors[id]) n = (size_t)g->tensors[id]->size * sizeof(float);
    kv.second.bytes = (n + 255) / 256 * 256;
    if (kv.second.pinned) { kv.second.first = 0; kv.second.last = pos; }
  }
}
CG_EXPORT bool cg_can_reuse_memory(cg_memory_planner* p_, int a, int b) { auto* p = impl(p_);
  if (!p) return false;
  auto ia = p->life.find(a), ib = p->life.find(b);
  if (ia == p->life.end() || ib == p->life.end() || ia->second.pinned || ib->second.pinned) return false;
  return ia->second.last < ib->second.first || ib->second.last < ia->second.first;
}
// Greedy offset assignment, largest first: a tensor takes the lowest offset at which it
// overlaps no already-placed tensor whose lifetime intersects its own.
CG_EXPORT void cg_find_reuse_opportunities(cg_memory_planner* p_) { auto* p = impl(p_);
  if (!p) return;
  std::vector<int> ids;
  for (auto& kv : p->life) { kv.second.planned = false; if (kv.second.bytes) ids.push_back(kv.first); }
  std::sort(ids.begin(), ids.end(), [&](int a, int b) { const Life &x = p->life[a], &y = p->life[b]; return x.bytes > y.bytes || (x.bytes == y.bytes && a < b); });
  p->plan_bytes = 0; p->reuse_pairs = 0;
  std::vector<int> placed;
  for (int id : ids) {
    Life& l = p->life[id];
    std::vector<std::pair<size_t, size_t>> busy;
    for (int q : placed) { const Life& o = p->life[q]; if (!(o.last < l.first || l.last < o.first)) busy.push_back({o.offset, o.offset + o.bytes}); }
    std::sort(busy.begin(), busy.end());
    size_t off = 0;
    for (auto& iv : busy) { if (off + l.bytes <= iv.first) break; if (iv.second > off) off = iv.second; }
    l.offset = off; l.planned = true;
    for (int q : placed) { const Life& o = p->life[q]; if (o.offset < off + l.bytes && off < o.offset + o.bytes) ++p->reuse_pairs; }
    placed.push_back(id);
    if (off + l.bytes > p->plan_bytes) p->plan_bytes = off + l.bytes;
  }
  p->stale = true;
}
CG_EXPORT void cg_memory_plan_analyze(cg_memory_planner* p_, void* ir_graph) { auto* p = impl(p_);
  cg_analyze_tensor_lifetimes(p, ir_graph);
  cg_find_reuse_opportunities(p);
}
CG_EXPORT size_t cg_memory_plan_bytes(cg_memory_planner* p_) { auto* p = impl(p_); return p ? p->plan_bytes : 0; }
CG_EXPORT size_t cg_memory_plan_offset(cg_memory_planner* p_, int tensor_id) { auto* p = impl(p_);
  if (!p) return (size_t)-1;
  auto it = p->life.find(tensor_id);
  return it == p->life.end() || !it->second.planned ? (size_t)-1 : it->second.offset;
}
CG_EXPORT void* cg_planned_alloc(cg_memory_planner* p_, size_t size, int tensor_id) { auto* p = impl(p_);
  if (!p) return fail(CG_ERROR_NULL_POINTER, (void*)nullptr);
  if (p->replaying) {                                    // same sequence of requests -> same addresses
    if (p->cursor < p->trace.size() && p->trace[p->cursor].tensor_id == tensor_id && p->trace[p->cursor].size >= size) return p->trace[p->cursor++].ptr;
    p->stale = true; p->replaying = false;
  }
  void* ptr = nullptr;
  auto it = p->life.find(tensor_id);
  if (it != p->life.end() && it->second.planned && size <= it->second.bytes) {
    if (!p->slab || p->slab_bytes < p->plan_bytes) {
      if (!p->handed.empty()) return fail(CG_ERROR_INVALID_ARGUMENT, (void*)nullptr);   // cannot move a slab that is in use
      std::free(p->slab);
      p->slab = nullptr;
      if (posix_memalign((void**)&p->slab, 256, p->plan_bytes ? p->plan_bytes : 256) != 0) return fail(CG_ERROR_OUT_OF_MEMORY, (void*)nullptr);
      p->slab_bytes = p->plan_bytes;
    }
    ptr = p->slab + it->second.offset;
    p->handed[tensor_id] = ptr;
  } else ptr = cg_pool_alloc(p->pools[0], size);
  if (p->capturing && ptr) p->trace.push_back({tensor_id, size, ptr});
  return ptr;
}
CG_EXPORT void cg_planned_free(cg_memory_planner* p_, void* ptr, int tensor_id) { auto* p = impl(p_);
  if (!p || !ptr) return;
  auto it = p->handed.find(tensor_id);
  if (it != p->handed.end() && it->second == ptr) { p->handed.erase(it); return; }
  if (p->replaying || p->captured) { for (auto& t : p->trace) if (t.ptr == ptr) return; }   // captured blocks stay reserved
  cg_pool_free(p->pools[0], ptr);
}
// Slides the live planned tensors towards offset 0 in address order (contents move with
// them) and shrinks the plan to the bytes in use.
CG_EXPORT void cg_memory_sliding_compact(cg_memory_planner* p_) { auto* p = impl(p_);
  if (!p) return;
  cg_pool_trim(p->pools[0]); cg_pool_trim(p->pools[1]);      // blocks that wait in the caches are the pools' fragmentation
  if (!p->slab) return;
  std::vector<int> ids;
  for (auto& kv : p->handed) ids.push_back(kv.first);
  std::sort(ids.begin(), ids.end(), [&](int a, int b) { return p->life[a].offset < p->life[b].offset; });
  size_t off = 0;
  for (int id : ids) {
    Life& l = p->life[id];
    if (l.offset != off) { std::memmove(p->slab + off, p->slab + l.offset, l.bytes); l.offset = off; p->handed[id] = p->slab + off; }
    off += l.bytes;
  }
  p->stale = true;
}
CG_EXPORT void cg_memory_defrag(cg_memory_planner* p_) { auto* p = impl(p_);
  if (!p) return;
  cg_pool_trim(p->pools[0]); cg_pool_trim(p->pools[1]);
  cg_memory_sliding_compact(p);
}
CG_EXPORT void cg_memory_maybe_defrag(cg_memory_planner* p_) { auto* p = impl(p_);
  if (p && (cg_memory_needs_compact(p->pools[0], 0.5f) || cg_memory_needs_compact(p->pools[1], 0.5f))) cg_memory_defrag(p);
}
CG_EXPORT void* cg_planned_lookup(cg_memory_planner* p_, int tensor_id) { auto* p = impl(p_);
  if (!p) return nullptr;
  auto it = p->handed.find(tensor_id);
  return it == p->handed.end() ? nullptr : it->second;
}
// Allocation trace for graph capture: between begin and end every planned allocation is
// recorded; replay hands the same addresses back in the same order, which is what a captured
// CUDA graph needs.  A request that deviates from the trace marks it stale.
CG_EXPORT void cg_cuda_graph_capture_begin(cg_memory_planner* p_) { auto* p = impl(p_); if (p) { p->trace.clear(); p->capturing = true; p->captured = false; p->replaying = false; p->graph_captured = false; } }
CG_EXPORT void cg_cuda_graph_capture_end(cg_memory_planner* p_) { auto* p = impl(p_); if (p && p->capturing) { p->capturing = false; p->captured = true; p->stale = false; p->graph_captured = true; } }
CG_EXPORT void cg_cuda_graph_replay(cg_memory_planner* p_) { auto* p = impl(p_); if (p && p->captured && !p->stale) { p->replaying = true; p->cursor = 0; } }
CG_EXPORT bool cg_cuda_graph_needs_update(cg_memory_planner* p_) { auto* p = impl(p_); return !p || !p->captured || p->stale; }

CG_EXPORT cg_memory_stats cg_memory_get_stats(cg_memory_planner* p_) { auto* p = impl(p_);
  cg_memory_stats s{};
  if (!p) return s;
  for (cg_memory_pool* q_ : p->pools) {
    PoolImpl* q = impl(q_);
    s.total_allocated += q->st.total_allocated; s.total_cached += q->st.total_cached; s.peak_allocated += q->st.peak_allocated;
    s.num_allocs += q->st.num_allocs; s.num_frees += q->st.num_frees; s.cache_hits += q->st.cache_hits; s.cache_misses += q->st.cache_misses;
    for (const auto& l : q->free_list) s.num_bins_used += l.empty() ? 0 : 1;
    for (const auto& l : q->sub_free) s.num_bins_used += l.empty() ? 0 : 1;
  }
  const double all = (double)s.total_allocated + (double)s.total_cached;
  s.fragmentation = all > 0 ? (float)(s.total_cached / all) : 0.0f;
  s.total_in_use = s.total_allocated;
  s.peak_usage = s.peak_allocated;
  const long long req = (long long)s.cache_hits + s.cache_misses;
  s.cache_hit_rate = req > 0 ? (size_t)(100LL * s.cache_hits / req) : 0;
  return s;
}
CG_EXPORT void cg_memory_print_stats(cg_memory_planner* p_) { auto* p = impl(p_);
  const cg_memory_stats s = cg_memory_get_stats(p);
  std::printf("memory: allocated %zu B, cached %zu B, peak %zu B, allocs %d, frees %d, hits %d, misses %d, fragmentation %.1f%%, plan %zu B\n",
              s.total_allocated, s.total_cached, s.peak_allocated, s.num_allocs, s.num_frees, s.cache_hits, s.cache_misses,
              100.0f * s.fragmentation, p ? p->plan_bytes : (size_t)0);
}
