// Device layer of the C API (cg_cuda_*): device discovery, memory, device tensors, and fp32
// tensor operations that launch the sm_100a kernel library.
//
// libcogito.so has no link-time dependency on CUDA.  cg_cuda_init() opens libcogito_kernels.so
// (the file next to this library) with dlopen and binds its C entry points; when that fails, or
// no GPU is reported, the layer stays in host mode and every call computes with the host
// implementations on ordinary memory.  The reference has the same two faces: the cudart branch
// and the simulation branch of src/cuda/cg_cuda.c:56-376 and src/cuda/tensor_kernels.c:265-909;
// its operations ignore where a tensor lives, here device tensors are tracked and checked.
#include <dlfcn.h>

#include <mutex>
#include <string>
#include <unordered_map>

#include "internal.hpp"

using namespace cgi;

namespace {

// ---- entry points of the kernel library, bound at run time ------------------------------
struct Kern {
  void* handle = nullptr;
  int (*dev_count)() = nullptr;
  int (*dev_info)(int, int*, unsigned long long*, char*, int) = nullptr;
  int (*dev_set)(int) = nullptr;
  int (*dev_get)() = nullptr;
  int (*dev_malloc)(void**, unsigned long long) = nullptr;
  int (*dev_free)(void*) = nullptr;
  int (*host_malloc)(void**, unsigned long long) = nullptr;
  int (*host_free)(void*) = nullptr;
  int (*dev_memcpy)(void*, const void*, unsigned long long, int, void*, int) = nullptr;
  int (*dev_memset)(void*, int, unsigned long long, void*) = nullptr;
  int (*stream_create)(void**) = nullptr;
  int (*stream_destroy)(void*) = nullptr;
  int (*dev_sync)(void*, int) = nullptr;
  const char* (*last_error)() = nullptr;
  int (*binary)(int, int, const void*, const void*, void*, long long, int, const int*, const long long*, const long long*, void*) = nullptr;
  int (*unary)(int, int, const void*, void*, long long, float, void*) = nullptr;
  int (*unary_backward)(int, int, const void*, const void*, void*, long long, float, void*) = nullptr;
  int (*cast)(const void*, void*, long long, int, void*) = nullptr;
  int (*split_bf16)(const float*, void*, void*, long long, void*) = nullptr;
  int (*reduce_axis)(int, int, const void*, float*, long long, long long, long long, void*) = nullptr;
  int (*reduce_all)(int, int, const void*, long long, float*, float*, void*) = nullptr;
  int (*reduce_all_scratch)(long long) = nullptr;
  int (*transpose2d)(int, const void*, void*, int, int, void*) = nullptr;
  int (*softmax_rows)(const float*, float*, int, int, float, void*) = nullptr;
  int (*softmax_rows_backward)(const float*, const float*, float*, int, int, void*) = nullptr;
  int (*norm_forward)(const void*, const void*, const void*, const void*, void*, void*, float*, float*, int, int, float, int, void*) = nullptr;
  long long (*norm_backward_scratch)(int, int) = nullptr;
  int (*norm_backward)(const void*, const void*, const void*, const float*, const float*, const void*, void*, float*, float*,
                       float*, int, int, int, int, void*) = nullptr;
  int (*gemm)(const void*, void*) = nullptr;
  int (*flash_forward)(const void*, void*) = nullptr;
  int (*flash_backward)(const void*, void*) = nullptr;
  int (*rope_apply)(int, void*, const float*, const float*, const int*, int, int, int, int, long long, long long, long long,
                    int, int, int, void*) = nullptr;
};

struct State {
  std::mutex mu;
  bool initialized = false;
  bool device_mode = false;
  int devices = 0;
  Kern k;
  cg_cuda_context ctx{nullptr, nullptr, 0, false};
  std::unordered_map<void*, size_t> dev_allocs;     // device allocations made through this layer
  std::unordered_map<void*, size_t> pinned;         // page-locked host allocations
  std::string error;
  int matmul_products = 3;
};
State& S() { static State s; return s; }

template <class F> bool bind(void* h, const char* name, F& slot) {
  slot = reinterpret_cast<F>(dlsym(h, name));
  return slot != nullptr;
}

void note_error(const std::string& msg) { S().error = msg; set_error(CG_ERROR_INVALID_ARGUMENT); }

// rc of a kernel-library call -> recorded error
bool ok(int rc, const char* what) {
  if (rc == 0) return true;
  State& s = S();
  s.error = std::string(what) + ": " + (s.k.last_error ? s.k.last_error() : "error");
  set_error(CG_ERROR_INVALID_ARGUMENT);
  return false;
}

std::string library_dir() {
  Dl_info info;
  if (dladdr((void*)&library_dir, &info) && info.dli_fname) {
    std::string p(info.dli_fname);
    const size_t cut = p.rfind('/');
    return cut == std::string::npos ? std::string(".") : p.substr(0, cut);
  }
  return ".";
}

bool open_kernels(State& s) {
  const char* force = std::getenv("COGITO_FORCE_HOST");
  if (force && force[0] && force[0] != '0') return false;
  const char* over = std::getenv("COGITO_KERNEL_LIBRARY");
  const std::string path = over && over[0] ? std::string(over) : library_dir() + "/libcogito_kernels.so";
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) { s.error = std::string("kernel library not opened: ") + dlerror(); return false; }
  Kern& k = s.k;
  bool all = bind(h, "cgk_dev_count", k.dev_count) & bind(h, "cgk_dev_info", k.dev_info) & bind(h, "cgk_dev_set", k.dev_set) &
             bind(h, "cgk_dev_get", k.dev_get) & bind(h, "cgk_dev_malloc", k.dev_malloc) & bind(h, "cgk_dev_free", k.dev_free) &
             bind(h, "cgk_host_malloc", k.host_malloc) & bind(h, "cgk_host_free", k.host_free) &
             bind(h, "cgk_dev_memcpy", k.dev_memcpy) & bind(h, "cgk_dev_memset", k.dev_memset) &
             bind(h, "cgk_stream_create", k.stream_create) & bind(h, "cgk_stream_destroy", k.stream_destroy) &
             bind(h, "cgk_dev_sync", k.dev_sync) & bind(h, "cgk_last_error", k.last_error) & bind(h, "cgk_binary", k.binary) &
             bind(h, "cgk_unary", k.unary) & bind(h, "cgk_unary_backward", k.unary_backward) & bind(h, "cgk_cast", k.cast) &
             bind(h, "cgk_split_bf16", k.split_bf16) & bind(h, "cgk_reduce_axis", k.reduce_axis) &
             bind(h, "cgk_reduce_all", k.reduce_all) & bind(h, "cgk_reduce_all_scratch_elems", k.reduce_all_scratch) &
             bind(h, "cgk_transpose2d", k.transpose2d) & bind(h, "cgk_softmax_rows", k.softmax_rows) &
             bind(h, "cgk_softmax_rows_backward", k.softmax_rows_backward) & bind(h, "cgk_norm_forward", k.norm_forward) &
             bind(h, "cgk_norm_backward_scratch_elems", k.norm_backward_scratch) & bind(h, "cgk_norm_backward", k.norm_backward) &
             bind(h, "cgk_gemm_bf16", k.gemm) & bind(h, "cgk_flash_forward", k.flash_forward) &
             bind(h, "cgk_flash_backward", k.flash_backward) & bind(h, "cgk_rope_apply", k.rope_apply);
  if (!all) { s.error = "kernel library lacks an entry point of the device layer"; dlclose(h); s.k = Kern(); return false; }
  k.handle = h;
  return true;
}

inline bool dev() { return S().device_mode; }
inline void* stream() { return S().ctx.stream; }

}  // namespace

// Device scratch that lives for one call: freed (after a stream synchronise) by the destructor.
namespace cgdev {
struct Scratch {
  std::vector<void*> ptrs;
  void* get(size_t bytes) {
    void* p = nullptr;
    if (!ok(S().k.dev_malloc(&p, bytes), "scratch allocation")) return nullptr;
    ptrs.push_back(p);
    return p;
  }
  ~Scratch() {
    if (ptrs.empty()) return;
    S().k.dev_sync(stream(), 0);
    for (void* p : ptrs) S().k.dev_free(p);
  }
};
}  // namespace cgdev

namespace cgi {
void free_storage(void* p) {
  if (!p) return;
  State& s = S();
  if (s.device_mode) {
    std::unique_lock<std::mutex> lock(s.mu);
    auto it = s.dev_allocs.find(p);
    if (it != s.dev_allocs.end()) {
      s.dev_allocs.erase(it);
      lock.unlock();
      s.k.dev_free(p);
      return;
    }
  }
  std::free(p);
}
}  // namespace cgi

// ------------------------------------------------------------------ bring-up
CG_EXPORT bool cg_cuda_init(void) {
  State& s = S();
  std::lock_guard<std::mutex> lock(s.mu);
  if (s.initialized) return true;
  s.device_mode = false;
  s.devices = 0;
  if (open_kernels(s)) {
    s.devices = s.k.dev_count();
    if (s.devices > 0 && s.k.stream_create(&s.ctx.stream) == 0) s.device_mode = true;
    else { s.ctx.stream = nullptr; s.devices = 0; }
  }
  s.ctx.device_id = s.device_mode ? s.k.dev_get() : 0;
  s.ctx.cublas_handle = nullptr;
  s.ctx.initialized = s.initialized = true;
  return true;
}

CG_EXPORT void cg_cuda_shutdown(void) {
  State& s = S();
  std::lock_guard<std::mutex> lock(s.mu);
  if (!s.initialized) return;
  if (s.device_mode) {
    s.k.dev_sync(nullptr, 1);
    s.k.stream_destroy(s.ctx.stream);
  }
  // live device tensors keep working: allocations stay registered and the library stays open
  s.ctx.stream = nullptr;
  s.ctx.initialized = s.initialized = false;
  if (s.device_mode && s.dev_allocs.empty() && s.pinned.empty()) {
    dlclose(s.k.handle);
    s.k = Kern();
    s.device_mode = false;
  }
}

CG_EXPORT bool cg_cuda_is_available(void) { return S().initialized; }
CG_EXPORT bool cg_cuda_device_mode(void) { return S().initialized && S().device_mode; }
CG_EXPORT int cg_cuda_device_count(void) { return S().device_mode ? S().devices : 1; }

CG_EXPORT cg_cuda_device_info cg_cuda_get_device_info(int device_id) {
  cg_cuda_device_info info;
  std::memset(&info, 0, sizeof(info));
  info.device_id = device_id;
  State& s = S();
  if (s.device_mode) {
    int v[8]; unsigned long long mem[3];
    if (device_id < 0 || device_id >= s.devices || !ok(s.k.dev_info(device_id, v, mem, info.device_name, 256), "device info"))
      return info;
    info.compute_capability_major = v[0]; info.compute_capability_minor = v[1];
    info.multiprocessor_count = v[2]; info.max_threads_per_block = v[3]; info.warp_size = v[4];
    info.total_memory = mem[0]; info.free_memory = mem[1]; info.shared_memory_per_block = mem[2];
    info.is_available = true;
    return info;
  }
  // host mode: the host itself, described in the device's terms
  std::snprintf(info.device_name, sizeof(info.device_name), "host (no GPU: cg_cuda_* runs on the CPU)");
  info.multiprocessor_count = 1; info.max_threads_per_block = 1024; info.warp_size = 32;
  info.is_available = device_id == 0 && s.initialized;
  return info;
}

CG_EXPORT void cg_cuda_set_device(int device_id) {
  State& s = S();
  if (!s.device_mode) { if (device_id != 0) note_error("host mode has device 0 only"); return; }
  if (ok(s.k.dev_set(device_id), "set device")) s.ctx.device_id = device_id;
}
CG_EXPORT int cg_cuda_get_device(void) { return S().device_mode ? S().k.dev_get() : 0; }
CG_EXPORT cg_cuda_context* cg_cuda_get_context(void) { return &S().ctx; }
CG_EXPORT const char* cg_cuda_get_last_error(void) { return S().error.c_str(); }
CG_EXPORT void cg_cuda_clear_error(void) { S().error.clear(); }

// ------------------------------------------------------------------ memory
CG_EXPORT void* cg_cuda_malloc(size_t size) {
  State& s = S();
  if (!s.device_mode) return std::malloc(size ? size : 1);
  void* p = nullptr;
  if (!ok(s.k.dev_malloc(&p, size), "cg_cuda_malloc")) { set_error(CG_ERROR_OUT_OF_MEMORY); return nullptr; }
  std::lock_guard<std::mutex> lock(s.mu);
  s.dev_allocs[p] = size;
  return p;
}
CG_EXPORT void cg_cuda_free(void* ptr) { free_storage(ptr); }

CG_EXPORT void* cg_cuda_malloc_host(size_t size) {
  State& s = S();
  if (!s.device_mode) return std::malloc(size ? size : 1);
  void* p = nullptr;
  if (!ok(s.k.host_malloc(&p, size), "cg_cuda_malloc_host")) { set_error(CG_ERROR_OUT_OF_MEMORY); return nullptr; }
  std::lock_guard<std::mutex> lock(s.mu);
  s.pinned[p] = size;
  return p;
}
CG_EXPORT void cg_cuda_free_host(void* ptr) {
  if (!ptr) return;
  State& s = S();
  {
    std::unique_lock<std::mutex> lock(s.mu);
    auto it = s.pinned.find(ptr);
    if (it != s.pinned.end()) { s.pinned.erase(it); lock.unlock(); s.k.host_free(ptr); return; }
  }
  std::free(ptr);
}

CG_EXPORT void cg_cuda_memcpy_async(void* dst, const void* src, size_t size, cg_memcpy_kind kind, void* stream_) {
  if (size == 0) return;
  if (!dst || !src) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (!dev()) { std::memmove(dst, src, size); return; }
  ok(S().k.dev_memcpy(dst, src, size, (int)kind, stream_ ? stream_ : stream(), 1), "cg_cuda_memcpy_async");
}
CG_EXPORT void cg_cuda_memcpy(void* dst, const void* src, size_t size, cg_memcpy_kind kind) {
  if (size == 0) return;
  if (!dst || !src) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (!dev()) { std::memmove(dst, src, size); return; }
  ok(S().k.dev_memcpy(dst, src, size, (int)kind, stream(), 0), "cg_cuda_memcpy");
}
CG_EXPORT void cg_cuda_memset(void* ptr, int value, size_t size) {
  if (!ptr) { if (size) set_error(CG_ERROR_NULL_POINTER); return; }
  if (!dev()) { std::memset(ptr, value, size); return; }
  ok(S().k.dev_memset(ptr, value, size, stream()), "cg_cuda_memset");
}
CG_EXPORT void cg_cuda_device_synchronize(void) { if (dev()) ok(S().k.dev_sync(nullptr, 1), "device synchronize"); }
CG_EXPORT void cg_cuda_stream_synchronize(void* stream_) {
  if (dev()) ok(S().k.dev_sync(stream_ ? stream_ : stream(), 0), "stream synchronize");
}

// One thread per element up to a grid that fills the machine a few times over; the kernels
// iterate with a grid-stride loop, so the cap loses no elements (the reference caps at 65 535
// blocks without such a loop, src/cuda/cg_cuda.c:355-363).
CG_EXPORT void cg_cuda_calculate_launch_dims(int n, int* grid, int* block) {
  const int b = 256;
  long long g = ((long long)(n > 0 ? n : 1) + b - 1) / b;
  const long long cap = 148LL * 8;
  if (block) *block = b;
  if (grid) *grid = (int)(g < cap ? g : cap);
}
CG_EXPORT void cg_cuda_calculate_launch_dims_2d(int rows, int cols, int* gx, int* gy, int* bx, int* by) {
  if (bx) *bx = 32;
  if (by) *by = 8;
  if (gx) *gx = ((cols > 0 ? cols : 1) + 31) / 32;
  if (gy) *gy = ((rows > 0 ? rows : 1) + 31) / 32;
}

// ------------------------------------------------------------------ device tensors
namespace {
enum { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_DIV = 3 };
enum { UN_EXP = 0, UN_LOG = 1, UN_SQRT = 2, UN_ABS = 3, UN_RSQRT = 5, UN_RELU = 6, UN_SIGMOID = 7, UN_TANH = 8, UN_GELU = 9,
       UN_POW = 11, UN_SCALE = 12, UN_ADDS = 13, UN_SQUARE = 15 };
enum { RED_SUM = 0, RED_MEAN = 1, RED_MAX = 2, RED_MIN = 3 };

bool is_dev_ptr(const void* p) {
  State& s = S();
  std::lock_guard<std::mutex> lock(s.mu);
  return s.dev_allocs.count(const_cast<void*>(p)) != 0;
}
// In device mode every operand has to be device memory of this layer; host mode takes anything.
bool operands_ok(std::initializer_list<const cg_tensor*> ts) {
  for (const cg_tensor* t : ts) if (!t || !t->data) { set_error(CG_ERROR_NULL_POINTER); return false; }
  if (!dev()) return true;
  for (const cg_tensor* t : ts)
    if (!is_dev_ptr(t->data)) { note_error("operand is not a device tensor (use cg_tensor_to_cuda)"); return false; }
  return true;
}
bool same_size(const cg_tensor* a, const cg_tensor* b) {
  if (a->size != b->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return false; }
  return true;
}

// broadcast kinds of the second operand of a [rows, D] elementwise product
enum Bc { FULL, PER_ROW, PER_COL };
bool dbin(int op, const float* a, const float* b, Bc kind, float* out, long long rows, long long D) {
  const int shape[2] = {(int)rows, (int)D};
  const long long sa[2] = {D, 1};
  const long long sb_full[2] = {D, 1}, sb_row[2] = {1, 0}, sb_col[2] = {0, 1};
  const long long* sb = kind == FULL ? sb_full : kind == PER_ROW ? sb_row : sb_col;
  return ok(S().k.binary(op, 0, a, b, out, rows * D, 2, shape, sa, sb, stream()), "elementwise kernel");
}
bool dun(int op, const float* x, float* out, long long n, float s = 0.0f) {
  return ok(S().k.unary(op, 0, x, out, n, s, stream()), "unary kernel");
}
bool dred(int op, const float* x, float* out, long long outer, long long red, long long inner) {
  return ok(S().k.reduce_axis(op, 0, x, out, outer, red, inner, stream()), "reduction kernel");
}

void binary_op(int op, cg_tensor* a, cg_tensor* b, cg_tensor* o) {
  if (!operands_ok({a, b, o}) || !same_size(a, b) || !same_size(a, o)) return;
  if (dev()) { dbin(op, a->data, b->data, FULL, o->data, 1, a->size); return; }
  for (int i = 0; i < o->size; ++i) {
    const float x = a->data[i], y = b->data[i];
    o->data[i] = op == BIN_ADD ? x + y : op == BIN_SUB ? x - y : op == BIN_MUL ? x * y : x / y;
  }
}
float host_unary(int op, float x, float s) {
  switch (op) {
    case UN_EXP: return std::exp(x);
    case UN_LOG: return std::log(x);
    case UN_SQRT: return std::sqrt(x);
    case UN_ABS: return std::fabs(x);
    case UN_RELU: return x > 0 ? x : 0.0f;
    case UN_SIGMOID: return sigmoidf(x);
    case UN_TANH: return std::tanh(x);
    case UN_GELU: return geluf(x);
    case UN_POW: return std::pow(x, s);
    case UN_SCALE: return x * s;
    default: return x;
  }
}
void unary_op(int op, cg_tensor* a, cg_tensor* o, float s = 0.0f) {
  if (!operands_ok({a, o}) || !same_size(a, o)) return;
  if (dev()) { dun(op, a->data, o->data, a->size, s); return; }
  for (int i = 0; i < o->size; ++i) o->data[i] = host_unary(op, a->data[i], s);
}

// a viewed as [outer, red, inner] for a reduction over `axis`
bool split_axis(const cg_tensor* a, int axis, long long* outer, long long* red, long long* inner) {
  if (axis >= a->ndim) { set_error(CG_ERROR_INVALID_ARGUMENT); return false; }
  *outer = *inner = 1;
  for (int i = 0; i < axis; ++i) *outer *= a->shape[i];
  for (int i = axis + 1; i < a->ndim; ++i) *inner *= a->shape[i];
  *red = a->shape[axis];
  return *red > 0;
}
void reduce_op(int op, cg_tensor* a, int axis, cg_tensor* o) {
  if (!operands_ok({a, o})) return;
  long long outer = 1, red = a->size, inner = 1;
  if (axis >= 0 && !split_axis(a, axis, &outer, &red, &inner)) return;
  if (o->size != outer * inner || red <= 0) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  if (dev()) {
    if (axis < 0) {
      cgdev::Scratch sc;
      float* tmp = (float*)sc.get(sizeof(float) * (size_t)S().k.reduce_all_scratch(a->size));
      if (tmp) ok(S().k.reduce_all(op, 0, a->data, a->size, o->data, tmp, stream()), "reduction kernel");
    } else {
      dred(op, a->data, o->data, outer, red, inner);
    }
    return;
  }
  for (long long u = 0; u < outer; ++u) for (long long v = 0; v < inner; ++v) {
    const float* x = a->data + u * red * inner + v;
    double acc = op == RED_MAX || op == RED_MIN ? x[0] : 0.0;
    for (long long r = 0; r < red; ++r) {
      const float e = x[r * inner];
      if (op == RED_MAX) acc = e > acc ? e : acc;
      else if (op == RED_MIN) acc = e < acc ? e : acc;
      else acc += e;
    }
    o->data[u * inner + v] = (float)(op == RED_MEAN ? acc / red : acc);
  }
}
}  // namespace

CG_EXPORT cg_tensor* cg_tensor_cuda_new(int* shape, int ndim, bool requires_grad) {
  if (!S().initialized) cg_cuda_init();
  if (!dev()) return make(shape, ndim, requires_grad);
  cg_tensor* t = make_header(shape, ndim, requires_grad);
  if (!t) return nullptr;
  const size_t bytes = sizeof(float) * (size_t)(t->size > 0 ? t->size : 1);
  t->data = (float*)cg_cuda_malloc(bytes);
  if (t->data && requires_grad) {
    t->grad = (float*)cg_cuda_malloc(bytes);
    if (t->grad) cg_cuda_memset(t->grad, 0, bytes);
  }
  if (!t->data || (requires_grad && !t->grad)) { cg_tensor_free(t); return fail(CG_ERROR_OUT_OF_MEMORY, (cg_tensor*)nullptr); }
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_cuda_zeros(int* shape, int ndim, bool requires_grad) {
  cg_tensor* t = cg_tensor_cuda_new(shape, ndim, requires_grad);
  if (t && dev()) cg_cuda_memset(t->data, 0, sizeof(float) * (size_t)t->size);
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_to_cuda(cg_tensor* t) {
  if (!t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* g = cg_tensor_cuda_new(t->shape, t->ndim, t->requires_grad);
  if (!g) return nullptr;
  const size_t bytes = sizeof(float) * (size_t)t->size;
  const bool from_dev = dev() && is_dev_ptr(t->data);
  cg_cuda_memcpy(g->data, t->data, bytes, from_dev ? CG_MEMCPY_DEVICE_TO_DEVICE : CG_MEMCPY_HOST_TO_DEVICE);
  if (t->requires_grad && t->grad && g->grad)
    cg_cuda_memcpy(g->grad, t->grad, bytes, from_dev ? CG_MEMCPY_DEVICE_TO_DEVICE : CG_MEMCPY_HOST_TO_DEVICE);
  return g;
}
CG_EXPORT cg_tensor* cg_tensor_to_cpu(cg_tensor* t) {
  if (!t) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (!dev() || !is_dev_ptr(t->data)) return cg_tensor_clone(t);
  cg_tensor* h = make(t->shape, t->ndim, t->requires_grad);
  if (!h) return nullptr;
  const size_t bytes = sizeof(float) * (size_t)t->size;
  cg_cuda_memcpy(h->data, t->data, bytes, CG_MEMCPY_DEVICE_TO_HOST);
  if (t->grad && h->grad) cg_cuda_memcpy(h->grad, t->grad, bytes, CG_MEMCPY_DEVICE_TO_HOST);
  return h;
}
CG_EXPORT bool cg_tensor_is_cuda(cg_tensor* t) { return t && t->data && dev() && is_dev_ptr(t->data); }

// ------------------------------------------------------------------ elementwise, reductions
CG_EXPORT void cg_cuda_tensor_add(cg_tensor* a, cg_tensor* b, cg_tensor* o) { binary_op(BIN_ADD, a, b, o); }
CG_EXPORT void cg_cuda_tensor_sub(cg_tensor* a, cg_tensor* b, cg_tensor* o) { binary_op(BIN_SUB, a, b, o); }
CG_EXPORT void cg_cuda_tensor_mul(cg_tensor* a, cg_tensor* b, cg_tensor* o) { binary_op(BIN_MUL, a, b, o); }
CG_EXPORT void cg_cuda_tensor_div(cg_tensor* a, cg_tensor* b, cg_tensor* o) { binary_op(BIN_DIV, a, b, o); }
CG_EXPORT void cg_cuda_tensor_scale(cg_tensor* a, float s, cg_tensor* o) { unary_op(UN_SCALE, a, o, s); }
CG_EXPORT void cg_cuda_tensor_exp(cg_tensor* a, cg_tensor* o) { unary_op(UN_EXP, a, o); }
CG_EXPORT void cg_cuda_tensor_log(cg_tensor* a, cg_tensor* o) { unary_op(UN_LOG, a, o); }
CG_EXPORT void cg_cuda_tensor_pow(cg_tensor* a, float p, cg_tensor* o) { unary_op(UN_POW, a, o, p); }
CG_EXPORT void cg_cuda_tensor_sqrt(cg_tensor* a, cg_tensor* o) { unary_op(UN_SQRT, a, o); }
CG_EXPORT void cg_cuda_tensor_abs(cg_tensor* a, cg_tensor* o) { unary_op(UN_ABS, a, o); }
CG_EXPORT void cg_cuda_tensor_sum(cg_tensor* a, int axis, cg_tensor* o) { reduce_op(RED_SUM, a, axis, o); }
CG_EXPORT void cg_cuda_tensor_mean(cg_tensor* a, int axis, cg_tensor* o) { reduce_op(RED_MEAN, a, axis, o); }
CG_EXPORT void cg_cuda_tensor_max(cg_tensor* a, int axis, cg_tensor* o) { reduce_op(RED_MAX, a, axis, o); }
CG_EXPORT void cg_cuda_tensor_min(cg_tensor* a, int axis, cg_tensor* o) { reduce_op(RED_MIN, a, axis, o); }

CG_EXPORT void cg_cuda_relu_forward(cg_tensor* x, cg_tensor* y) { unary_op(UN_RELU, x, y); }
CG_EXPORT void cg_cuda_sigmoid_forward(cg_tensor* x, cg_tensor* y) { unary_op(UN_SIGMOID, x, y); }
CG_EXPORT void cg_cuda_tanh_forward(cg_tensor* x, cg_tensor* y) { unary_op(UN_TANH, x, y); }
CG_EXPORT void cg_cuda_gelu_forward(cg_tensor* x, cg_tensor* y) { unary_op(UN_GELU, x, y); }

// The rest of the layer, split by topic; each part uses the helpers above.
#include "device_math.hpp"
#include "device_norm.hpp"
#include "device_attention.hpp"
