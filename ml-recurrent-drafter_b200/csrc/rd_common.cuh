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

// The same for a cudaError_t already in hand (rd::launch_chained() returns one).
#define RD_CHECK_CHAINED(err)                               \
  do {                                                      \
    if ((err) != cudaSuccess) {                             \
      rd_set_last_cuda_error((int)(err));                   \
      return RD_ERR_LAUNCH;                                 \
    }                                                       \
  } while (0)

void rd_set_last_cuda_error(int e);
// 1 unless the environment variable RD_PDL is "0" (read once): launch the kernels of the decode
// chain with programmatic stream serialisation so that a kernel's launch and prologue overlap the
// tail of its predecessor.
int rd_pdl_enabled();

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

// Programmatic dependent launch.  A kernel launched with rd::launch_chained() may begin before the
// previous kernel of the stream has finished: it must execute pdl_wait() before its first access to
// global memory (reads of the predecessor's results and writes to anything the predecessor may still
// read), and it lets its own successor start early with pdl_launch_dependents().  Both are no-ops
// in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, int cluster_x,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (rd_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace rd
