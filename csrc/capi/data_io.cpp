// Datasets and loaders, COG1 checkpoints, the layer profiler, bf16 tensors and the
// mixed-precision helper.  Reference surface: include/cg_datasets.h + src/datasets/*.c,
// include/cg_serialization.h + src/core/serialization.c, include/cg_profiler.h +
// src/utils/profiler.c, include/cg_bf16.h + src/core/bf16.c.
#include <chrono>
#include <map>
#include <string>

#include "internal.hpp"

using namespace cgi;

// ------------------------------------------------------------------- MNIST
static bool read_be32(FILE* f, uint32_t* v) {
  unsigned char b[4];
  if (std::fread(b, 1, 4, f) != 4) return false;
  *v = ((uint32_t)b[0] << 24) | ((uint32_t)b[1] << 16) | ((uint32_t)b[2] << 8) | b[3];
  return true;
}
CG_EXPORT cg_mnist* cg_mnist_load(const char* images_path, const char* labels_path) {
  if (!images_path || !labels_path) return fail(CG_ERROR_NULL_POINTER, (cg_mnist*)nullptr);
  FILE* fi = std::fopen(images_path, "rb");
  FILE* fl = fi ? std::fopen(labels_path, "rb") : nullptr;
  if (!fi || !fl) { if (fi) std::fclose(fi); return fail(CG_ERROR_FILE_NOT_FOUND, (cg_mnist*)nullptr); }
  uint32_t magic_i, n_i, rows, cols, magic_l, n_l;
  cg_mnist* m = nullptr;
  if (read_be32(fi, &magic_i) && read_be32(fi, &n_i) && read_be32(fi, &rows) && read_be32(fi, &cols) &&
      read_be32(fl, &magic_l) && read_be32(fl, &n_l) && magic_i == 2051 && magic_l == 2049 && n_i == n_l &&
      rows > 0 && cols > 0 && rows <= 4096 && cols <= 4096) {
    const size_t px = (size_t)rows * cols;
    std::vector<unsigned char> buf(px);
    int is[2] = {(int)n_i, (int)px}, ls[1] = {(int)n_i};
    m = (cg_mnist*)std::calloc(1, sizeof(cg_mnist));
    m->images = make(is, 2, false); m->labels = make(ls, 1, false);
    m->num_samples = (int)n_i; m->rows = (int)rows; m->cols = (int)cols;
    bool ok = m->images && m->labels;
    for (uint32_t i = 0; ok && i < n_i; ++i) {
      ok = std::fread(buf.data(), 1, px, fi) == px;
      for (size_t j = 0; ok && j < px; ++j) m->images->data[i * px + j] = buf[j] * (1.0f / 255.0f);
    }
    for (uint32_t i = 0; ok && i < n_i; ++i) { unsigned char c; ok = std::fread(&c, 1, 1, fl) == 1; if (ok) m->labels->data[i] = (float)c; }
    if (!ok) { cg_mnist_free(m); m = nullptr; set_error(CG_ERROR_INVALID_FORMAT); }
  } else set_error(CG_ERROR_INVALID_FORMAT);
  std::fclose(fi); std::fclose(fl);
  return m;
}
CG_EXPORT void cg_mnist_free(cg_mnist* m) {
  if (!m) return;
  if (m->images) cg_tensor_release(m->images);
  if (m->labels) cg_tensor_release(m->labels);
  std::free(m);
}
CG_EXPORT void cg_mnist_get_batch(cg_mnist* m, int start, int bs, cg_tensor* img_out, cg_tensor* lab_out) {
  if (!m || !img_out || !lab_out) { set_error(CG_ERROR_NULL_POINTER); return; }
  const int px = m->rows * m->cols;
  if (start < 0 || bs < 0 || start + bs > m->num_samples || img_out->size < bs * px || lab_out->size < bs) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  std::memcpy(img_out->data, m->images->data + (size_t)start * px, sizeof(float) * bs * px);
  std::memcpy(lab_out->data, m->labels->data + start, sizeof(float) * bs);
}
CG_EXPORT cg_tensor* cg_tensor_onehot(cg_tensor* labels, int C) {
  if (!labels) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (C <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr);
  int s[2] = {labels->size, C};
  cg_tensor* o = make(s, 2, false);
  if (!o) return nullptr;
  for (int i = 0; i < labels->size; ++i) {
    const int c = (int)labels->data[i];
    if (c < 0 || c >= C) { cg_tensor_release(o); return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor*)nullptr); }
    o->data[(size_t)i * C + c] = 1.0f;
  }
  return o;
}
CG_EXPORT cg_tensor* cg_labels_to_onehot(cg_tensor* labels, int C) { return cg_tensor_onehot(labels, C); }
CG_EXPORT void cg_augment_gaussian_noise(cg_tensor* t, float std_, unsigned int seed) {
  if (!t) return;
  Rng r(seed);
  for (int i = 0; i < t->size; ++i) t->data[i] += std_ * r.normal();
}
CG_EXPORT void cg_augment_horizontal_flip(cg_tensor* t, float prob, unsigned int seed) {
  if (!t || t->ndim < 2) return;
  const int N = t->shape[0], px = t->size / N;
  int W = t->ndim >= 3 ? t->shape[t->ndim - 1] : (int)std::lround(std::sqrt((double)px));
  if (W <= 0 || px % W) return;
  Rng r(seed);
  for (int n = 0; n < N; ++n) {
    if (r.uniform() >= prob) continue;
    for (int row = 0; row < px / W; ++row) {
      float* p = t->data + (size_t)n * px + (size_t)row * W;
      for (int x = 0; x < W / 2; ++x) { const float tmp = p[x]; p[x] = p[W - 1 - x]; p[W - 1 - x] = tmp; }
    }
  }
}

// -------------------------------------------------------------- iterators
static void shuffle_indices(cg_data_iter* it, unsigned int seed) {
  for (int i = 0; i < it->num_samples; ++i) it->indices[i] = i;
  if (!it->shuffle) return;
  Rng r(seed);
  for (int i = it->num_samples - 1; i > 0; --i) { const int j = r.below(i + 1); const int t = it->indices[i]; it->indices[i] = it->indices[j]; it->indices[j] = t; }
}
static bool iter_init(cg_data_iter* it, cg_tensor* data, cg_tensor* labels, int bs, bool shuffle, unsigned int seed) {
  if (!data || data->ndim < 1 || bs <= 0 || (labels && (labels->ndim < 1 || labels->shape[0] != data->shape[0]))) return false;
  it->data = data; it->labels = labels; it->batch_size = bs; it->shuffle = shuffle; it->seed = seed;
  it->num_samples = data->shape[0]; it->position = 0;
  it->indices = (int*)std::malloc(sizeof(int) * (it->num_samples ? it->num_samples : 1));
  cg_tensor_retain(data); if (labels) cg_tensor_retain(labels);
  shuffle_indices(it, seed);
  return true;
}
static void iter_drop(cg_data_iter* it) {
  if (it->batch_data) cg_tensor_release(it->batch_data);
  if (it->batch_labels) cg_tensor_release(it->batch_labels);
  it->batch_data = it->batch_labels = nullptr;
}
static cg_tensor* gather_rows(cg_tensor* src, const int* idx, int n) {
  int shape[CG_MAX_DIMS];
  for (int i = 0; i < src->ndim; ++i) shape[i] = src->shape[i];
  shape[0] = n;
  cg_tensor* o = make(shape, src->ndim, false);
  const int row = src->shape[0] ? src->size / src->shape[0] : 0;
  if (o) for (int i = 0; i < n; ++i) std::memcpy(o->data + (size_t)i * row, src->data + (size_t)idx[i] * row, sizeof(float) * row);
  return o;
}
static bool iter_next(cg_data_iter* it, cg_tensor** bd, cg_tensor** bl, int* actual) {
  if (it->position >= it->num_samples) return false;
  const int n = it->num_samples - it->position < it->batch_size ? it->num_samples - it->position : it->batch_size;
  iter_drop(it);
  it->batch_data = gather_rows(it->data, it->indices + it->position, n);
  if (it->labels) it->batch_labels = gather_rows(it->labels, it->indices + it->position, n);
  it->position += n;
  if (bd) *bd = it->batch_data;
  if (bl) *bl = it->batch_labels;
  if (actual) *actual = n;
  return true;
}
static void iter_fini(cg_data_iter* it) {
  iter_drop(it);
  if (it->data) cg_tensor_release(it->data);
  if (it->labels) cg_tensor_release(it->labels);
  std::free(it->indices);
}
CG_EXPORT cg_data_iter* cg_data_iter_new(cg_tensor* data, cg_tensor* labels, int bs, bool shuffle, unsigned int seed) {
  cg_data_iter* it = (cg_data_iter*)std::calloc(1, sizeof(cg_data_iter));
  if (!iter_init(it, data, labels, bs, shuffle, seed)) { std::free(it); return fail(CG_ERROR_INVALID_ARGUMENT, (cg_data_iter*)nullptr); }
  return it;
}
// The returned batch tensors belong to the iterator and live until the next call.
CG_EXPORT bool cg_data_iter_next(cg_data_iter* it, cg_tensor** bd, cg_tensor** bl) { return it && iter_next(it, bd, bl, nullptr); }
CG_EXPORT void cg_data_iter_reset(cg_data_iter* it, unsigned int seed) { if (it) { it->position = 0; it->seed = seed; shuffle_indices(it, seed); } }
CG_EXPORT void cg_data_iter_free(cg_data_iter* it) { if (it) { iter_fini(it); std::free(it); } }
CG_EXPORT cg_dataloader* cg_dataloader_new(cg_tensor* data, cg_tensor* labels, int bs, bool shuffle, unsigned int seed) {
  cg_dataloader* l = (cg_dataloader*)std::calloc(1, sizeof(cg_dataloader));
  if (!iter_init(&l->it, data, labels, bs, shuffle, seed)) { std::free(l); return fail(CG_ERROR_INVALID_ARGUMENT, (cg_dataloader*)nullptr); }
  return l;
}
CG_EXPORT bool cg_dataloader_next(cg_dataloader* l, cg_tensor** bd, cg_tensor** bl, int* actual) { return l && iter_next(&l->it, bd, bl, actual); }
CG_EXPORT void cg_dataloader_reset(cg_dataloader* l) { if (l) { ++l->epoch; l->it.position = 0; shuffle_indices(&l->it, l->it.seed + (unsigned)l->epoch); } }
CG_EXPORT int cg_dataloader_num_batches(cg_dataloader* l) { return l ? (l->it.num_samples + l->it.batch_size - 1) / l->it.batch_size : 0; }
CG_EXPORT void cg_dataloader_free(cg_dataloader* l) { if (l) { iter_fini(&l->it); std::free(l); } }
CG_EXPORT int cg_tensor_argmax(cg_tensor* t, int sample, int C) {
  if (!t || C <= 0 || sample < 0 || (size_t)(sample + 1) * C > (size_t)t->size) return fail(CG_ERROR_INVALID_ARGUMENT, -1);
  const float* p = t->data + (size_t)sample * C;
  int best = 0;
  for (int j = 1; j < C; ++j) if (p[j] > p[best]) best = j;
  return best;
}
// labels: class indices [N] or one-hot [N, C]
CG_EXPORT float cg_compute_accuracy(cg_tensor* logits, cg_tensor* labels, int C) {
  if (!logits || !labels || C <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, 0.0f);
  const int N = logits->size / C;
  if (N == 0) return 0.0f;
  int hit = 0;
  for (int i = 0; i < N; ++i) {
    const int want = labels->size == N ? (int)labels->data[i] : cg_tensor_argmax(labels, i, C);
    hit += cg_tensor_argmax(logits, i, C) == want;
  }
  return (float)hit / N;
}

// ------------------------------------------------------------ checkpoints
// Layout: 24-byte header {magic, version, count, pad, total_size}, count 120-byte directory
// entries, then the payloads back to back (include/cg_serialization.h:11-27,
// src/core/serialization.c:9-77).
static_assert(sizeof(cg_model_header) == 24, "COG1 header layout");
static_assert(sizeof(cg_tensor_entry) == 120, "COG1 directory entry layout");
CG_EXPORT void cg_save_model(const char* filename, cg_tensor** tensors, const char** names, int count) {
  if (!filename || !tensors || !names || count < 0) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  FILE* f = std::fopen(filename, "wb");
  if (!f) { set_error(CG_ERROR_FILE_NOT_FOUND); return; }
  cg_model_header h;
  std::memset(&h, 0, sizeof(h));
  h.magic = CG_MODEL_MAGIC; h.version = 1; h.num_tensors = (uint32_t)count;
  uint64_t off = sizeof(h) + (uint64_t)count * sizeof(cg_tensor_entry);
  std::vector<cg_tensor_entry> dir(count);
  for (int i = 0; i < count; ++i) {
    cg_tensor_entry& e = dir[i];
    std::memset(&e, 0, sizeof(e));
    std::strncpy(e.name, names[i] ? names[i] : "", sizeof(e.name) - 1);
    e.ndim = tensors[i]->ndim;
    for (int d = 0; d < tensors[i]->ndim; ++d) e.shape[d] = tensors[i]->shape[d];
    e.dtype = 0; e.offset = off; e.size_bytes = (uint64_t)tensors[i]->size * sizeof(float);
    off += e.size_bytes;
  }
  h.total_size = off;
  bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1;
  ok = ok && (count == 0 || std::fwrite(dir.data(), sizeof(cg_tensor_entry), count, f) == (size_t)count);
  for (int i = 0; ok && i < count; ++i) ok = tensors[i]->size == 0 || std::fwrite(tensors[i]->data, sizeof(float), tensors[i]->size, f) == (size_t)tensors[i]->size;
  if (std::fclose(f) != 0 || !ok) set_error(CG_ERROR_INVALID_FORMAT);
}
CG_EXPORT void cg_load_model(const char* filename, cg_tensor*** out_t, char*** out_n, int* out_c) {
  if (!filename || !out_t || !out_n || !out_c) { set_error(CG_ERROR_NULL_POINTER); return; }
  *out_t = nullptr; *out_n = nullptr; *out_c = 0;
  FILE* f = std::fopen(filename, "rb");
  if (!f) { set_error(CG_ERROR_FILE_NOT_FOUND); return; }
  cg_model_header h;
  if (std::fread(&h, sizeof(h), 1, f) != 1 || h.magic != CG_MODEL_MAGIC || h.num_tensors > (1u << 24)) { std::fclose(f); set_error(CG_ERROR_INVALID_FORMAT); return; }
  const int n = (int)h.num_tensors;
  std::vector<cg_tensor_entry> dir(n);
  if (n && std::fread(dir.data(), sizeof(cg_tensor_entry), n, f) != (size_t)n) { std::fclose(f); set_error(CG_ERROR_INVALID_FORMAT); return; }
  cg_tensor** ts = (cg_tensor**)std::calloc(n ? n : 1, sizeof(cg_tensor*));
  char** ns = (char**)std::calloc(n ? n : 1, sizeof(char*));
  bool ok = true;
  // Payload types: 0 fp32, 1 bf16 (widened), 2 packed INT4 (flat groups, low nibble first, as
  // cg_quantize_int4 writes them) dequantised with the "<name>.scales" entry that follows it,
  // 16-23 exact-byte integer / bool / fp64 / fp16 payloads of the Python writer, converted to
  // fp32 values.  An entry of any other type becomes a 1-D tensor of its byte values, so that one
  // unknown entry does not make the rest of the file unreadable.
  auto read_raw = [&](const cg_tensor_entry& e, std::vector<unsigned char>& raw) {
    raw.resize((size_t)e.size_bytes);
    return std::fseek(f, (long)e.offset, SEEK_SET) == 0 && (raw.empty() || std::fread(raw.data(), 1, raw.size(), f) == raw.size());
  };
  for (int i = 0; ok && i < n; ++i) {
    cg_tensor_entry& e = dir[i];
    e.name[63] = 0;
    ok = e.ndim >= 0 && e.ndim <= CG_MAX_DIMS && e.size_bytes <= ((uint64_t)1 << 40);
    if (!ok) break;
    ns[i] = strdup(e.name);
    std::vector<unsigned char> raw;
    if (e.dtype == 0 || e.dtype == 1) {
      ts[i] = make(e.shape, e.ndim, false);
      ok = ts[i] && std::fseek(f, (long)e.offset, SEEK_SET) == 0;
      if (!ok) break;
      if (e.dtype == 0) ok = e.size_bytes == (uint64_t)ts[i]->size * 4 && (ts[i]->size == 0 || std::fread(ts[i]->data, 4, ts[i]->size, f) == (size_t)ts[i]->size);
      else {
        std::vector<uint16_t> half(ts[i]->size);
        ok = e.size_bytes == (uint64_t)ts[i]->size * 2 && (ts[i]->size == 0 || std::fread(half.data(), 2, half.size(), f) == half.size());
        for (int j = 0; ok && j < ts[i]->size; ++j) ts[i]->data[j] = cg_bf16_to_fp32(half[j]);
      }
    } else if (e.dtype == 2) {
      ts[i] = make(e.shape, e.ndim, false);
      ok = ts[i] && read_raw(e, raw) && raw.size() * 2 >= (size_t)ts[i]->size;
      if (!ok) break;
      // the scales: next entry, named "<name>.scales", fp32 or bf16
      std::vector<float> scales;
      const std::string want = std::string(e.name) + ".scales";
      if (i + 1 < n) {
        cg_tensor_entry& se = dir[i + 1];
        se.name[63] = 0;
        std::vector<unsigned char> sraw;
        if (want == se.name && (se.dtype == 0 || se.dtype == 1) && read_raw(se, sraw)) {
          const size_t cnt = sraw.size() / (se.dtype == 0 ? 4 : 2);
          scales.resize(cnt);
          for (size_t j = 0; j < cnt; ++j) {
            if (se.dtype == 0) std::memcpy(&scales[j], sraw.data() + 4 * j, 4);
            else { uint16_t h16; std::memcpy(&h16, sraw.data() + 2 * j, 2); scales[j] = cg_bf16_to_fp32(h16); }
          }
        }
      }
      const long long cnt = ts[i]->size;
      ok = !scales.empty() || cnt == 0;
      if (!ok) break;
      const long long group = cnt == 0 ? 1 : (cnt + (long long)scales.size() - 1) / (long long)scales.size();
      for (long long j = 0; j < cnt; ++j) {
        const unsigned char byte = raw[(size_t)(j >> 1)];
        int q = (j & 1) ? (byte >> 4) : (byte & 0xF);
        if (q >= 8) q -= 16;
        ts[i]->data[j] = (float)q * scales[(size_t)(j / group)];
      }
    } else if (e.dtype >= 16 && e.dtype <= 23) {
      static const int width[8] = {8, 4, 1, 1, 8, 2, 2, 1};
      const int w = width[e.dtype - 16];
      ts[i] = make(e.shape, e.ndim, false);
      ok = ts[i] && read_raw(e, raw) && raw.size() == (size_t)ts[i]->size * w;
      for (int j = 0; ok && j < ts[i]->size; ++j) {
        const unsigned char* p = raw.data() + (size_t)j * w;
        float v = 0.0f;
        switch (e.dtype) {
          case 16: { int64_t x; std::memcpy(&x, p, 8); v = (float)x; break; }
          case 17: { int32_t x; std::memcpy(&x, p, 4); v = (float)x; break; }
          case 18: v = (float)*p; break;
          case 19: v = *p ? 1.0f : 0.0f; break;
          case 20: { double x; std::memcpy(&x, p, 8); v = (float)x; break; }
          case 21: {   // IEEE half
            uint16_t h16; std::memcpy(&h16, p, 2);
            const int sgn = h16 >> 15, ex = (h16 >> 10) & 31, man = h16 & 1023;
            if (ex == 0) v = std::ldexp((float)man, -24);
            else if (ex == 31) v = man ? NAN : INFINITY;
            else v = std::ldexp((float)(man | 1024), ex - 25);
            if (sgn) v = -v;
            break;
          }
          case 22: { int16_t x; std::memcpy(&x, p, 2); v = (float)x; break; }
          default: v = (float)(signed char)*p; break;
        }
        ts[i]->data[j] = v;
      }
    } else {
      int shape1[1] = {(int)e.size_bytes};
      ts[i] = make(shape1, 1, false);
      ok = ts[i] && read_raw(e, raw);
      for (size_t j = 0; ok && j < raw.size(); ++j) ts[i]->data[j] = (float)raw[j];
    }
  }
  std::fclose(f);
  if (!ok) {
    for (int i = 0; i < n; ++i) { if (ts[i]) cg_tensor_release(ts[i]); std::free(ns[i]); }
    std::free(ts); std::free(ns);
    set_error(CG_ERROR_INVALID_FORMAT);
    return;
  }
  *out_t = ts; *out_n = ns; *out_c = n;
}

// ---------------------------------------------------------------- profiler
namespace {
struct Prof { double total_ms = 0; int count = 0; std::chrono::steady_clock::time_point start; bool open = false; };
std::map<std::string, Prof> g_prof;
std::vector<std::string> g_prof_order;
bool g_prof_on = false;
int g_prof_steps = 0;
cg_profiler g_state = {nullptr, 0, 0, false, 0};            // the public view of the tables above
void publish_profile() {
  const int n = (int)g_prof_order.size();
  if (n > g_state.capacity) {
    const int cap = n * 2 > 16 ? n * 2 : 16;
    cg_layer_stat* grown = (cg_layer_stat*)std::realloc(g_state.layers, sizeof(cg_layer_stat) * cap);
    if (!grown) return;
    g_state.layers = grown; g_state.capacity = cap;
  }
  for (int i = 0; i < n; ++i) {
    const Prof& p = g_prof[g_prof_order[i]];
    cg_layer_stat& s = g_state.layers[i];
    std::snprintf(s.name, sizeof(s.name), "%s", g_prof_order[i].c_str());
    s.start_event = s.stop_event = nullptr; s.total_ms = (float)p.total_ms; s.count = p.count;
  }
  g_state.num_layers = n; g_state.enabled = g_prof_on; g_state.current_epoch = g_prof_steps;
}
}  // namespace
CG_EXPORT cg_profiler* cg_profiler_state(void) { publish_profile(); return &g_state; }
CG_EXPORT void cg_profiler_init(void) { g_prof.clear(); g_prof_order.clear(); g_prof_steps = 0; g_prof_on = true; }
CG_EXPORT void cg_profiler_enable(bool e) { g_prof_on = e; }
CG_EXPORT void cg_profiler_begin_layer(const char* name) {
  if (!g_prof_on || !name) return;
  auto it = g_prof.find(name);
  if (it == g_prof.end()) { it = g_prof.emplace(name, Prof()).first; g_prof_order.push_back(name); }
  it->second.start = std::chrono::steady_clock::now(); it->second.open = true;
}
CG_EXPORT void cg_profiler_end_layer(const char* name) {
  if (!g_prof_on || !name) return;
  auto it = g_prof.find(name);
  if (it == g_prof.end() || !it->second.open) return;
  it->second.total_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - it->second.start).count();
  ++it->second.count; it->second.open = false;
}
CG_EXPORT void cg_profiler_step_end(void) { if (g_prof_on) ++g_prof_steps; }
CG_EXPORT void cg_profiler_report(void) {
  double all = 0;
  for (auto& kv : g_prof) all += kv.second.total_ms;
  std::printf("%-32s %8s %12s %12s %7s\n", "layer", "calls", "total ms", "mean ms", "share");
  for (auto& name : g_prof_order) {
    const Prof& p = g_prof[name];
    std::printf("%-32s %8d %12.3f %12.4f %6.1f%%\n", name.c_str(), p.count, p.total_ms, p.count ? p.total_ms / p.count : 0.0, all > 0 ? 100.0 * p.total_ms / all : 0.0);
  }
  std::printf("steps: %d, total %.3f ms\n", g_prof_steps, all);
}
CG_EXPORT void cg_profiler_reset(void) { g_prof.clear(); g_prof_order.clear(); g_prof_steps = 0; }
CG_EXPORT double cg_profiler_total_ms(const char* name) { auto it = name ? g_prof.find(name) : g_prof.end(); return it == g_prof.end() ? 0.0 : it->second.total_ms; }
CG_EXPORT int cg_profiler_count(const char* name) { auto it = name ? g_prof.find(name) : g_prof.end(); return it == g_prof.end() ? 0 : it->second.count; }

// -------------------------------------------------------------------- bf16
CG_EXPORT cg_bf16 cg_fp32_to_bf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return (cg_bf16)((u >> 16) | ((u & 0xffffu) ? 0x40u : 0u));   // inf / quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (cg_bf16)(u >> 16);
}
CG_EXPORT float cg_bf16_to_fp32(cg_bf16 h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
CG_EXPORT cg_tensor_bf16* cg_tensor_bf16_new(int* shape, int ndim, bool rg) {
  if (ndim < 0 || ndim > CG_MAX_DIMS || (ndim && !shape)) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_tensor_bf16*)nullptr);
  cg_tensor_bf16* t = (cg_tensor_bf16*)std::calloc(1, sizeof(cg_tensor_bf16));
  long n = 1;
  for (int i = 0; i < ndim; ++i) { t->shape[i] = shape[i]; n *= shape[i]; }
  t->ndim = ndim; t->size = (int)n; t->requires_grad = rg;
  t->data = (cg_bf16*)std::calloc(n ? n : 1, sizeof(cg_bf16));
  if (rg) {
    t->master = (float*)std::calloc(n ? n : 1, sizeof(float)); t->grad_fp32 = (float*)std::calloc(n ? n : 1, sizeof(float));
    t->grad = (cg_bf16*)std::calloc(n ? n : 1, sizeof(cg_bf16));
    t->has_master_copy = true;
  }
  return t;
}
CG_EXPORT cg_tensor_bf16* cg_tensor_bf16_from_fp32(cg_tensor* s) {
  if (!s) return fail(CG_ERROR_NULL_POINTER, (cg_tensor_bf16*)nullptr);
  cg_tensor_bf16* t = cg_tensor_bf16_new(s->shape, s->ndim, s->requires_grad);
  for (int i = 0; i < s->size; ++i) { t->data[i] = cg_fp32_to_bf16(s->data[i]); if (t->master) t->master[i] = s->data[i]; }
  return t;
}
CG_EXPORT cg_tensor* cg_tensor_bf16_to_fp32(cg_tensor_bf16* s) {
  if (!s) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  cg_tensor* t = make(s->shape, s->ndim, s->requires_grad);
  if (t) for (int i = 0; i < s->size; ++i) t->data[i] = cg_bf16_to_fp32(s->data[i]);
  return t;
}
CG_EXPORT void cg_tensor_bf16_free(cg_tensor_bf16* t) {
  if (t) { std::free(t->data); std::free(t->master); std::free(t->grad); std::free(t->grad_fp32); std::free(t); }
}

#define BF(x) cg_bf16_to_fp32(x)
CG_EXPORT void cg_bf16_add(cg_tensor_bf16* a, cg_tensor_bf16* b, cg_tensor_bf16* o) {
  if (!a || !b || !o || a->size != b->size || a->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  for (int i = 0; i < o->size; ++i) o->data[i] = cg_fp32_to_bf16(BF(a->data[i]) + BF(b->data[i]));
}
CG_EXPORT void cg_bf16_mul(cg_tensor_bf16* a, cg_tensor_bf16* b, cg_tensor_bf16* o) {
  if (!a || !b || !o || a->size != b->size || a->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  for (int i = 0; i < o->size; ++i) o->data[i] = cg_fp32_to_bf16(BF(a->data[i]) * BF(b->data[i]));
}
// a [M,K] x b [K,N] with fp32 accumulation
CG_EXPORT void cg_bf16_matmul(cg_tensor_bf16* a, cg_tensor_bf16* b, cg_tensor_bf16* o) {
  if (!a || !b || !o || a->ndim != 2 || b->ndim != 2 || a->shape[1] != b->shape[0] || o->size != a->shape[0] * b->shape[1]) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int M = a->shape[0], K = a->shape[1], N = b->shape[1];
  std::vector<float> fa(a->size), fb(b->size), fc((size_t)M * N);
  for (int i = 0; i < a->size; ++i) fa[i] = BF(a->data[i]);
  for (int i = 0; i < b->size; ++i) fb[i] = BF(b->data[i]);
  gemm(fa.data(), fb.data(), fc.data(), M, N, K, false, false, false);
  for (int i = 0; i < M * N; ++i) o->data[i] = cg_fp32_to_bf16(fc[i]);
}
CG_EXPORT void cg_bf16_gelu(cg_tensor_bf16* a, cg_tensor_bf16* o) {
  if (!a || !o || a->size != o->size) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  for (int i = 0; i < o->size; ++i) o->data[i] = cg_fp32_to_bf16(geluf(BF(a->data[i])));
}
CG_EXPORT void cg_bf16_layernorm(cg_tensor_bf16* x, cg_tensor_bf16* gamma, cg_tensor_bf16* beta, float eps, cg_tensor_bf16* o) {
  if (!x || !o || x->size != o->size || x->ndim < 1) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int C = x->shape[x->ndim - 1], R = x->size / C;
  for (int r = 0; r < R; ++r) {
    double m = 0, v = 0;
    for (int j = 0; j < C; ++j) m += BF(x->data[(size_t)r * C + j]);
    m /= C;
    for (int j = 0; j < C; ++j) { const double d = BF(x->data[(size_t)r * C + j]) - m; v += d * d; }
    const float inv = 1.0f / std::sqrt((float)(v / C) + eps);
    for (int j = 0; j < C; ++j) {
      float y = (BF(x->data[(size_t)r * C + j]) - (float)m) * inv;
      if (gamma) y *= BF(gamma->data[j]);
      if (beta) y += BF(beta->data[j]);
      o->data[(size_t)r * C + j] = cg_fp32_to_bf16(y);
    }
  }
}

// --------------------------------------------------------- mixed precision
// fp32 masters in `params`, bf16 working copies in `model_params`; dynamic loss scale
// 65536 in [1, 65536], x2 after 2000 clean steps, /2 and skip on overflow
// (src/core/bf16.c:88-94,115-198).
CG_EXPORT cg_mixed_precision* cg_mixed_precision_new(cg_tensor** params, int n) {
  if (!params || n <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_mixed_precision*)nullptr);
  cg_mixed_precision* mp = (cg_mixed_precision*)std::calloc(1, sizeof(cg_mixed_precision));
  mp->params = (cg_tensor**)std::malloc(sizeof(cg_tensor*) * n);
  mp->model_params = (cg_tensor_bf16**)std::malloc(sizeof(cg_tensor_bf16*) * n);
  for (int i = 0; i < n; ++i) { mp->params[i] = params[i]; cg_tensor_retain(params[i]); mp->model_params[i] = cg_tensor_bf16_from_fp32(params[i]); }
  mp->num_params = n;
  mp->loss_scale = 65536.0f; mp->min_loss_scale = 1.0f; mp->max_loss_scale = 65536.0f; mp->scale_factor = 2.0f; mp->scale_window = 2000;
  mp->max_grad_norm = 1.0f; mp->learning_rate = 1e-3f;
  return mp;
}
CG_EXPORT cg_tensor_bf16* cg_mp_forward(cg_mixed_precision* mp, cg_tensor_bf16* (*model_fn)(void*, cg_tensor_bf16*), void* model, cg_tensor_bf16* input) {
  if (!mp || !model_fn) return fail(CG_ERROR_NULL_POINTER, (cg_tensor_bf16*)nullptr);
  return model_fn(model, input);
}
CG_EXPORT bool cg_mp_check_overflow(cg_mixed_precision* mp) {
  if (!mp) return false;
  mp->found_overflow = false;
  for (int i = 0; i < mp->num_params && !mp->found_overflow; ++i) {
    cg_tensor* p = mp->params[i];
    if (p->grad) for (int j = 0; j < p->size; ++j) if (!std::isfinite(p->grad[j])) { mp->found_overflow = true; break; }
  }
  return mp->found_overflow;
}
// Seeds the loss gradient with the loss scale; the caller's backward pass then fills
// params[i]->grad.  Returns false (and halves the scale) when those gradients overflowed.
CG_EXPORT bool cg_mp_backward(cg_mixed_precision* mp, cg_tensor_bf16* loss) {
  if (!mp) return fail(CG_ERROR_NULL_POINTER, false);
  if (loss && loss->grad) for (int i = 0; i < loss->size; ++i) loss->grad[i] = mp->loss_scale;
  if (cg_mp_check_overflow(mp)) {
    mp->loss_scale = mp->loss_scale / mp->scale_factor < mp->min_loss_scale ? mp->min_loss_scale : mp->loss_scale / mp->scale_factor;
    mp->steps_since_overflow = 0; ++mp->num_skipped;
    std::printf("MP: Overflow detected, scale -> %g\n", mp->loss_scale);
    return false;
  }
  return true;
}
CG_EXPORT void cg_mp_step(cg_mixed_precision* mp) {
  if (!mp) return;
  if (mp->found_overflow) { mp->found_overflow = false; for (int i = 0; i < mp->num_params; ++i) cg_tensor_zero_grad(mp->params[i]); return; }
  const float inv = 1.0f / mp->loss_scale;
  double ss = 0;
  for (int i = 0; i < mp->num_params; ++i) { cg_tensor* p = mp->params[i]; if (p->grad) for (int j = 0; j < p->size; ++j) { const double g = (double)p->grad[j] * inv; ss += g * g; } }
  const float norm = (float)std::sqrt(ss);
  const float clip = mp->max_grad_norm > 0 && norm > mp->max_grad_norm ? mp->max_grad_norm / (norm + 1e-6f) : 1.0f;
  for (int i = 0; i < mp->num_params; ++i) {
    cg_tensor* p = mp->params[i];
    if (!p->grad) continue;
    for (int j = 0; j < p->size; ++j) {
      p->data[j] -= mp->learning_rate * p->grad[j] * inv * clip;
      mp->model_params[i]->data[j] = cg_fp32_to_bf16(p->data[j]);
      p->grad[j] = 0.0f;
    }
  }
  ++mp->num_steps;
  if (++mp->steps_since_overflow >= mp->scale_window) {
    mp->loss_scale = mp->loss_scale * mp->scale_factor > mp->max_loss_scale ? mp->max_loss_scale : mp->loss_scale * mp->scale_factor;
    mp->steps_since_overflow = 0;
  }
}
CG_EXPORT void cg_mixed_precision_free(cg_mixed_precision* mp) {
  if (!mp) return;
  for (int i = 0; i < mp->num_params; ++i) { cg_tensor_release(mp->params[i]); cg_tensor_bf16_free(mp->model_params[i]); }
  std::free(mp->params); std::free(mp->model_params); std::free(mp);
}
