// C = epilogue(A * W^T) on CUDA cores with fp32 accumulation, for fp32 models (exact-fp32 parity
// with a CPU run is only possible without tensor cores) and as the cross-check of the tcgen05
// path.  64x64 tile, K step 16, 256 threads, 4x4 outputs per thread.
#include "rd_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename OutT>
__device__ __forceinline__ void store_out(OutT* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) {
  *p = v;
}
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

template <typename T, typename OutT, int EPI>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                                                        int64_t ldw, OutT* C, int64_t ldc, const T* __restrict__ bias,
                                                        const OutT* R, int64_t ldr, int m_max,
                                                        const int32_t* __restrict__ m_dev, int N, int K) {
  const int M = rd::live_rows(m_dev, m_max);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (m0 >= M) return;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + lk + e;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + e][lr] = (am < M && kk < K) ? rd::Num<T>::to_f(A[(int64_t)am * lda + kk]) : 0.f;
      Ws[lk + e][lr] = (wn < N && kk < K) ? rd::Num<T>::to_f(W[(int64_t)wn * ldw + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    if (EPI == RD_EPI_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 < N) store_out<OutT>(C + (int64_t)m * ldc + (n >> 1), rd::silu_exact(acc[i][j]) * acc[i][j + 1]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n >= N) continue;
        float v = acc[i][j];
        if (EPI == RD_EPI_BIAS || EPI == RD_EPI_BIAS_SILU || EPI == RD_EPI_BIAS_SILU_RES) v += rd::Num<T>::to_f(bias[n]);
        if (EPI == RD_EPI_BIAS_SILU || EPI == RD_EPI_BIAS_SILU_RES) v = rd::silu_exact(v);
        if (EPI == RD_EPI_BIAS_SILU_RES || EPI == RD_EPI_RES) v += rd::Num<OutT>::to_f(R[(int64_t)m * ldr + n]);
        store_out<OutT>(C + (int64_t)m * ldc + n, v);
      }
    }
  }
}

template <typename T, typename OutT>
int launch(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, const void* bias, const void* R,
           int64_t ldr, int m_max, const int32_t* m_dev, int N, int K, int epilogue, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (m_max + BM - 1) / BM);
#define RD_LAUNCH_EPI(E)                                                                                              \
  case E:                                                                                                             \
    gemm_simt_kernel<T, OutT, E><<<grid, 256, 0, s>>>((const T*)A, lda, (const T*)W, ldw, (OutT*)C, ldc, (const T*)bias, \
                                                      (const OutT*)R, ldr, m_max, m_dev, N, K);                       \
    break;
  switch (epilogue) {
    RD_LAUNCH_EPI(RD_EPI_NONE)
    RD_LAUNCH_EPI(RD_EPI_BIAS)
    RD_LAUNCH_EPI(RD_EPI_BIAS_SILU)
    RD_LAUNCH_EPI(RD_EPI_BIAS_SILU_RES)
    RD_LAUNCH_EPI(RD_EPI_RES)
    RD_LAUNCH_EPI(RD_EPI_SWIGLU)
    default:
      return RD_ERR_ARG;
  }
#undef RD_LAUNCH_EPI
  RD_CHECK_LAUNCH();
  return RD_OK;
}

}  // namespace

extern "C" int rd_gemm(int dtype, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, void* C,
                       int64_t ldc, const void* bias, const void* R, int64_t ldr, int m_max, const int32_t* m_dev, int N,
                       int K, int epilogue, void* stream) {
  RD_REQUIRE(A && W && C, RD_ERR_ARG);
  RD_REQUIRE(m_max >= 1 && N >= 1 && K >= 1 && lda >= K && ldw >= K, RD_ERR_SIZE);
  const bool need_bias = epilogue == RD_EPI_BIAS || epilogue == RD_EPI_BIAS_SILU || epilogue == RD_EPI_BIAS_SILU_RES;
  const bool need_res = epilogue == RD_EPI_BIAS_SILU_RES || epilogue == RD_EPI_RES;
  RD_REQUIRE(!need_bias || bias, RD_ERR_ARG);
  RD_REQUIRE(!need_res || R, RD_ERR_ARG);
  RD_REQUIRE(epilogue != RD_EPI_SWIGLU || N % 2 == 0, RD_ERR_SIZE);
  RD_REQUIRE(ldc >= (epilogue == RD_EPI_SWIGLU ? N / 2 : N), RD_ERR_SIZE);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == RD_F32 && out_dtype == RD_F32)
    return launch<float, float>(A, lda, W, ldw, C, ldc, bias, R, ldr, m_max, m_dev, N, K, epilogue, s);
  if (dtype == RD_BF16 && out_dtype == RD_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, C, ldc, bias, R, ldr, m_max, m_dev, N, K, epilogue, s);
  if (dtype == RD_BF16 && out_dtype == RD_F32)
    return launch<__nv_bfloat16, float>(A, lda, W, ldw, C, ldc, bias, R, ldr, m_max, m_dev, N, K, epilogue, s);
  return RD_ERR_DTYPE;
}
