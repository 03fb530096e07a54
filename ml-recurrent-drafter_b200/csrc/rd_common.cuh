// Shared device/host helpers for the ReDrafter B200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/redrafter_b200.h"

#define RD_LOG_0 (-50000.0f)

// Launch-time check: returns a negative code for an invalid argument found on the host.
#define RD_REQUIRE(cond, code) \
  do {                         \
    if (!(cond)) return (code); \
  } while (0)

// Returns RD_ERR_LAUNCH when the launch itself was rejected (bad configuration).
#define RD_CHECK_LAUNCH()                                   \
  do {                                                      \
    cudaError_t e__ = cudaPeekAtLastError();                \
    if (e__ != cudaSuccess) {                               \
      rd_set_last_cuda_error((int)e__);                     \
      return RD_ERR_LAUNCH;                                 \
    }                                                       \
  } while (0)

void rd_set_last_cuda_error(int e);

namespace rd {

template <typename T>
struct Num;
template <>
struct Num<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// fast form for rounded (bf16) outputs: approximate exp and division, ~2 ulp
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
// expf with full fp32 accuracy (used where parity with a CPU fp32 path matters)
__device__ __forceinline__ float silu_exact(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Order-preserving map float -> uint32 (larger float <=> larger key).
__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Effective row count: min(*m_dev, m_max) when a device-side count is given.
__device__ __forceinline__ int live_rows(const int* m_dev, int m_max) {
  if (m_dev == nullptr) return m_max;
  int m = *m_dev;
  return m < m_max ? (m < 0 ? 0 : m) : m_max;
}

}  // namespace rd
