#include "host_common.h"

#include <stdarg.h>
#include <string.h>

#include <mutex>

namespace cgk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

static std::mutex g_mu;
static int* g_status[64] = {nullptr};
static int g_sms[64] = {0};

int* device_status(int device) {
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[device] == nullptr) {
    int* p = nullptr;
    if (cudaMalloc(&p, 4 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 4 * sizeof(int));
    g_status[device] = p;
  }
  return g_status[device];
}

int sm_count(int device) {
  if (device < 0 || device >= 64) return 148;
  if (g_sms[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = 148;
    g_sms[device] = n;
  }
  return g_sms[device];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int encode_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int rank,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, Swz swz) {
  // A thread that has made no runtime call yet (an autograd worker thread, say)
  // has no current driver context, and the driver-API encoder then fails with
  // CUDA_ERROR_INVALID_CONTEXT; a no-op runtime call binds the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  EncodeTiledFn fn = get_encode();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return CGK_E_CUDA;
  }
  if (((uintptr_t)base & 15u) != 0) {
    set_error("tensor map base %p is not 16-byte aligned", base);
    return CGK_E_ARG;
  }
  cuuint64_t gd[5];
  cuuint64_t gs[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      gs[i] = strides_bytes[i];
      if (gs[i] % 16 != 0) {
        set_error("tensor map stride %d = %llu bytes is not a multiple of 16", i,
                  (unsigned long long)gs[i]);
        return CGK_E_ARG;
      }
    }
  }
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swz == Swz::B32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swz == Swz::B64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swz == Swz::B128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (rank %d, dims %llu x %llu, box %u x %u)",
              (int)r, rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 1),
              box[0], rank > 1 ? box[1] : 1);
    return CGK_E_CUDA;
  }
  return 0;
}

int encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld * 2};
  uint32_t box[2] = {box_cols, box_rows};
  return encode_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, strides, box, Swz::B128);
}

}  // namespace cgk

CGK_API const char* cgk_last_error() { return cgk::last_error(); }

// Reads and clears the device status word of the current device.
// out[0..3] = {code, where, block, aux}.  Synchronises the given stream first.
CGK_API int cgk_read_status(int* out, void* stream) {
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  int* st = cgk::device_status(dev);
  if (!st) {
    cgk::set_error("no status word for device %d", dev);
    return CGK_E_CUDA;
  }
  CGK_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
  CGK_CUDA_CHECK(cudaMemcpy(out, st, 4 * sizeof(int), cudaMemcpyDeviceToHost));
  if (out[0] != 0) CGK_CUDA_CHECK(cudaMemset(st, 0, 4 * sizeof(int)));
  return 0;
}

CGK_API int cgk_version() { return 100; }
