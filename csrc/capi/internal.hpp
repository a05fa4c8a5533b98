// Shared internals of the host runtime (libcogito.so).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <initializer_list>
#include <vector>

#include "cogito.h"

#define CG_EXPORT extern "C" __attribute__((visibility("default")))

namespace cgi {

void set_error(cg_error e);
// Returns v after recording the error; for `return fail(CG_ERROR_…, nullptr);`
template <class T> inline T fail(cg_error e, T v) { set_error(e); return v; }

// ---- tensors
cg_tensor* make(const int* shape, int ndim, bool requires_grad);          // zero-filled
cg_tensor* make_like(const cg_tensor* t, bool requires_grad);
cg_tensor* make_header(const int* shape, int ndim, bool requires_grad);  // counted, data / grad left null
void ensure_grad(cg_tensor* t);
// Frees tensor storage: std::free, or the device layer's free when p is device memory.
void free_storage(void* p);
inline bool wants_grad(const cg_tensor* t) { return t && t->requires_grad; }
inline int rows_of(const cg_tensor* t) { return t->ndim ? t->size / t->shape[t->ndim - 1] : 1; }
inline int cols_of(const cg_tensor* t) { return t->ndim ? t->shape[t->ndim - 1] : 1; }

// ---- tape: the closure runs with self->grad holding the upstream gradient and adds
// into the parents' ->grad.
using BackFn = std::function<void(cg_tensor* self)>;
struct BackCtx { BackFn fn; bool ran = false; };
// True once the node's backward closure has run since it was recorded (lets the per-layer
// backward entry points be no-ops after cg_backward has already walked the tape).
inline bool tape_ran(const cg_tensor* t) { return t && t->backward_ctx && ((const BackCtx*)t->backward_ctx)->ran; }
void attach(cg_tensor* out, std::initializer_list<cg_tensor*> parents, BackFn fn);
void attach_n(cg_tensor* out, cg_tensor* const* parents, int n, BackFn fn);   // n may exceed CG_MAX_PARENTS

// ---- dense kernels (row-major fp32).  C[M,N] (+)= op(A) op(B)
//   ta = false: A is [M,K];  ta = true: A is [K,M]
//   tb = false: B is [K,N];  tb = true: B is [N,K]
void gemm(const float* A, const float* B, float* C, int M, int N, int K, bool ta, bool tb, bool accumulate);
// attention.cpp: true when a flash-attention parameter block holds raw fp32 arrays (filled the reference's way) rather than tensors
bool flash_raw_block(const cg_flash_attn_params* p);
// host_simd.cpp (built with -O3, AVX2 + FMA copies picked at load time)
void gemm_rows(const float* A, const float* B, float* C, int M, int N, int K, bool ta);       // C += op(A) B, B [K,N]
void gemm_dots(const float* A, const float* B, float* C, int M, int N, int K);                // C += A B^T, B [N,K], few rows
void adam_update(float* w, float* m, float* v, const float* g, int n, float b1, float b2, float lr, float eps,
                 float bc1, float bc2, float decay);

// ---- random streams
struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull) {}
  uint64_t next() { uint64_t z = (s += 0x9E3779B97F4A7C15ull); z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
                    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); }
  float uniform() { return (float)((next() >> 40) * (1.0 / 16777216.0)); }          // [0,1)
  float normal() { float u1 = uniform(), u2 = uniform(); if (u1 < 1e-7f) u1 = 1e-7f;
                   return std::sqrt(-2.0f * std::log(u1)) * std::cos(6.28318530718f * u2); }
  int below(int n) { return (int)(next() % (uint64_t)n); }
};
uint64_t next_layer_seed();      // global seed mixed with a per-layer counter

inline float sigmoidf(float x) { return 1.0f / (1.0f + std::exp(-x)); }
inline float siluf(float x) { return x * sigmoidf(x); }
inline float geluf(float x) { return 0.5f * x * (1.0f + std::tanh(0.7978845608f * (x + 0.044715f * x * x * x))); }

}  // namespace cgi
