// Shared helpers for the fpq_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cstdlib>

#include "../../include/fpq_b200.h"

namespace fpq {

// Thread-local text of the last failure, returned by fpq_last_error().
void set_error(const char* fmt, ...);
const char* get_error();

// Number of SMs of the current device (cached per device).
int sm_count();

#define FPQ_CHECK_ARG(cond, ...)                         \
  do {                                                   \
    if (!(cond)) {                                       \
      ::fpq::set_error(__VA_ARGS__);                     \
      return FPQ_ERR_INVALID_ARGUMENT;                   \
    }                                                    \
  } while (0)

#define FPQ_CHECK_CUDA(expr)                                                        \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess) {                                                        \
      ::fpq::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),      \
                       __FILE__, __LINE__);                                         \
      return FPQ_ERR_CUDA;                                                          \
    }                                                                               \
  } while (0)

#define FPQ_CHECK_LAUNCH()  FPQ_CHECK_CUDA(cudaGetLastError())

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------- E2M1 rounding rule
// Index (0..7) of the E2M1 magnitude nearest to |v|, ties to the even code:
// <=0.25 -> 0, (0.25,0.75) -> 0.5, [0.75,1.25] -> 1, (1.25,1.75) -> 1.5,
// [1.75,2.5] -> 2, (2.5,3.5) -> 3, [3.5,5] -> 4, >5 -> 6.
__device__ __forceinline__ uint32_t e2m1_index(float a /* |v| */) {
  uint32_t i = 0;
  i += (a > 0.25f);
  i += (a >= 0.75f);
  i += (a > 1.25f);
  i += (a >= 1.75f);
  i += (a > 2.5f);
  i += (a >= 3.5f);
  i += (a > 5.0f);
  return i;
}

// 4-bit code of v: magnitude index | sign << 3, and every zero (either sign) as 0x8.
__device__ __forceinline__ uint32_t e2m1_code(float v) {
  uint32_t i = e2m1_index(fabsf(v));
  uint32_t neg = (v < 0.0f) | (i == 0);
  return i | (neg << 3);
}

__device__ __forceinline__ float e2m1_magnitude(uint32_t idx) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6
  return idx < 4 ? 0.5f * (float)idx : (idx == 4 ? 2.0f : (idx == 5 ? 3.0f : (idx == 6 ? 4.0f : 6.0f)));
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  float m = e2m1_magnitude(code & 7u);
  return (code & 8u) ? -m : m;
}

// In a word of eight 4-bit codes, turn every nibble whose low three bits are zero into 0x8.
__device__ __forceinline__ uint32_t patch_zero_codes(uint32_t w) {
  uint32_t t = w | (w >> 1) | (w >> 2);
  uint32_t z = ~t & 0x11111111u;
  return w | (z << 3);
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may
// start while the previous kernel of the stream is still finishing; it calls grid_dependency_wait() before it
// touches anything that kernel (or an earlier one) wrote.  launch_dependents() lets the NEXT kernel's blocks be
// scheduled as soon as resources free up.  Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Whether launches carry the attribute (environment FPQ_PDL=0 switches it off).
inline bool use_dependent_launch() {
  static const bool on = [] {
    const char* e = getenv("FPQ_PDL");
    return e ? atoi(e) != 0 : true;
  }();
  return on;
}

}  // namespace fpq
