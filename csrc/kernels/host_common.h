// Host-side helpers shared by the kernel launchers: tensor-map encoding through
// the driver entry point (no link-time dependency on libcuda), the per-device
// status word, and the error convention of the exported C functions.
//
// Every exported launcher returns 0 on success or a negative CGK_E_* code and
// leaves a message retrievable with cgk_last_error().
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define CGK_API extern "C" __attribute__((visibility("default")))

enum {
  CGK_E_ARG = -1,      // bad argument (shape, alignment, null pointer)
  CGK_E_CUDA = -2,     // a CUDA runtime / driver call failed
  CGK_E_LIMIT = -3,    // size beyond a stated maximum
  CGK_E_DEVICE = -4,   // the kernel reported a device-side status
};

namespace cgk {

void set_error(const char* fmt, ...);
const char* last_error();

// Device status words: int[4] per device, allocated once (lazily) per device.
int* device_status(int device);

// Encode a tiled bf16/fp32/u8 tensor map.  dims[0] is the innermost (contiguous)
// dimension.  strides_bytes[i] is the stride of dims[i+1].  Returns 0 or CGK_E_*.
enum class Swz { None = 0, B32 = 1, B64 = 2, B128 = 3 };
int encode_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int rank,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, Swz swz);

// Shorthand for a row-major 2-D bf16 matrix [rows, cols] with leading dimension
// ld (elements), box = box_rows x box_cols, 128-byte swizzle.
int encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols);

int sm_count(int device);

#define CGK_CUDA_CHECK(expr)                                                         \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess) {                                                         \
      ::cgk::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                       __LINE__);                                                    \
      return CGK_E_CUDA;                                                             \
    }                                                                                \
  } while (0)

#define CGK_LAUNCH_CHECK()                                                           \
  do {                                                                               \
    cudaError_t _e = cudaGetLastError();                                             \
    if (_e != cudaSuccess) {                                                         \
      ::cgk::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e),   \
                       __FILE__, __LINE__);                                          \
      return CGK_E_CUDA;                                                             \
    }                                                                                \
  } while (0)

#define CGK_REQUIRE(cond, ...)              \
  do {                                      \
    if (!(cond)) {                          \
      ::cgk::set_error(__VA_ARGS__);        \
      return CGK_E_ARG;                     \
    }                                       \
  } while (0)

}  // namespace cgk
