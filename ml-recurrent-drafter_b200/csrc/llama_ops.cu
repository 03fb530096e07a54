// Element-wise and reduction kernels of the Llama verify forward: embedding gather, RMSNorm,
// rotary embedding + KV-cache append, row argmax, and the small data-movement helpers of the
// decode loop.
#include "rd_common.cuh"

namespace {

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids, T* __restrict__ out,
                                    int m_max, const int32_t* __restrict__ m_dev, int H, int vec) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int t = blockIdx.x;
  if (t >= rd::live_rows(m_dev, m_max)) return;
  const T* src = table + ids[t] * (int64_t)H;
  T* dst = out + (int64_t)t * H;
  constexpr int VEC = 16 / sizeof(T);
  if (vec) {
    for (int d = threadIdx.x; d < H / VEC; d += blockDim.x) reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(src)[d];
    return;
  }
  for (int d = threadIdx.x; d < H; d += blockDim.x) dst[d] = src[d];
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                                      int m_max, const int32_t* __restrict__ m_dev, int H, float eps,
                                                      int vectorised) {
  constexpr int VEC = 16 / sizeof(T);
  const int t = blockIdx.x;
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  if (t >= rd::live_rows(m_dev, m_max)) return;
  const T* xr = x + (int64_t)t * H;
  T* yr = y + (int64_t)t * H;
  float ss = 0.f;
  if (vectorised) {
    for (int v = threadIdx.x; v < H / VEC; v += 256) {
      T e[VEC];
      *reinterpret_cast<uint4*>(e) = reinterpret_cast<const uint4*>(xr)[v];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float f = rd::Num<T>::to_f(e[i]);
        ss += f * f;
      }
    }
  } else {
    for (int d = threadIdx.x; d < H; d += 256) {
      float v = rd::Num<T>::to_f(xr[d]);
      ss += v * v;
    }
  }
  __shared__ float red[8];
  ss = rd::warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rs = 1.0f / sqrtf(tot / (float)H + eps);
  // normalise in fp32, round to the model dtype, then scale by the weight (as the reference does)
  if (vectorised) {
    for (int v = threadIdx.x; v < H / VEC; v += 256) {
      T e[VEC], g[VEC], o[VEC];
      *reinterpret_cast<uint4*>(e) = reinterpret_cast<const uint4*>(xr)[v];
      *reinterpret_cast<uint4*>(g) = reinterpret_cast<const uint4*>(w)[v];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const T n = rd::Num<T>::from_f(rd::Num<T>::to_f(e[i]) * rs);
        o[i] = rd::Num<T>::from_f(rd::Num<T>::to_f(g[i]) * rd::Num<T>::to_f(n));
      }
      reinterpret_cast<uint4*>(yr)[v] = *reinterpret_cast<const uint4*>(o);
    }
  } else {
    for (int d = threadIdx.x; d < H; d += 256) {
      T n = rd::Num<T>::from_f(rd::Num<T>::to_f(xr[d]) * rs);
      yr[d] = rd::Num<T>::from_f(rd::Num<T>::to_f(w[d]) * rd::Num<T>::to_f(n));
    }
  }
}

// One block per token.  A work item is a pair of 16-byte chunks (d .. d+VEC) and (d+hd/2 .. ) of one
// q or k head - the two halves that the NeoX rotation mixes - or one 16-byte chunk of a v head.
constexpr int kRopeThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kRopeThreads) rope_kv_write_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const int32_t* __restrict__ tok_row, const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ tok_slot,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_pos, int m_max,
    const int32_t* __restrict__ m_dev, int nh, int nkv, int hd, int max_len) {
  constexpr int VEC = 16 / sizeof(T);
  const int t = blockIdx.x;
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  if (t >= rd::live_rows(m_dev, m_max)) return;
  const int b = tok_row[t], slot = tok_slot[t];
  int pos = tok_pos[t];
  pos = pos < 0 ? 0 : (pos >= n_pos ? n_pos - 1 : pos);
  const int half = hd / 2;
  const int width = (nh + 2 * nkv) * hd;
  const T* src = qkv + (int64_t)t * width;
  const float* c = cos_t + (int64_t)pos * hd;
  const float* s = sin_t + (int64_t)pos * hd;
  const int pairs_per_head = half / VEC;
  const int n_rot = (nh + nkv) * pairs_per_head;
  const int n_v = nkv * (hd / VEC);
  // 16-byte loads of the fp32 tables need aligned rows
  const bool vec_tables = (VEC % 4 == 0) && (hd % 4 == 0) && ((((uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0);
#pragma unroll 2
  for (int w = threadIdx.x; w < n_rot + n_v; w += kRopeThreads) {
    if (w < n_rot) {
      const int head = w / pairs_per_head, d = (w % pairs_per_head) * VEC;
      T lo[VEC], hi[VEC], olo[VEC], ohi[VEC];
      float cl[VEC], ch[VEC], sl[VEC], sh[VEC];
      *reinterpret_cast<uint4*>(lo) = *reinterpret_cast<const uint4*>(src + head * hd + d);
      *reinterpret_cast<uint4*>(hi) = *reinterpret_cast<const uint4*>(src + head * hd + d + half);
      if (vec_tables) {
#pragma unroll
        for (int e = 0; e < VEC; e += 4) {
          *reinterpret_cast<float4*>(cl + e) = *reinterpret_cast<const float4*>(c + d + e);
          *reinterpret_cast<float4*>(ch + e) = *reinterpret_cast<const float4*>(c + d + half + e);
          *reinterpret_cast<float4*>(sl + e) = *reinterpret_cast<const float4*>(s + d + e);
          *reinterpret_cast<float4*>(sh + e) = *reinterpret_cast<const float4*>(s + d + half + e);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          cl[e] = c[d + e];
          ch[e] = c[d + half + e];
          sl[e] = s[d + e];
          sh[e] = s[d + half + e];
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float x1 = rd::Num<T>::to_f(lo[e]), x2 = rd::Num<T>::to_f(hi[e]);
        // q*cos + rotate_half(q)*sin with two rounded products and one rounded sum
        olo[e] = rd::Num<T>::from_f(__fadd_rn(__fmul_rn(x1, cl[e]), __fmul_rn(-x2, sl[e])));
        ohi[e] = rd::Num<T>::from_f(__fadd_rn(__fmul_rn(x2, ch[e]), __fmul_rn(x1, sh[e])));
      }
      T* dst = head < nh ? q_out + (int64_t)t * nh * hd + head * hd
                         : k_cache + (((int64_t)b * nkv + (head - nh)) * max_len + slot) * hd;
      *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(olo);
      *reinterpret_cast<uint4*>(dst + d + half) = *reinterpret_cast<const uint4*>(ohi);
    } else {
      const int wv = w - n_rot;
      const int head = wv / (hd / VEC), d = (wv % (hd / VEC)) * VEC;
      const uint4 v = *reinterpret_cast<const uint4*>(src + (nh + nkv + head) * hd + d);
      *reinterpret_cast<uint4*>(v_cache + (((int64_t)b * nkv + head) * max_len + slot) * hd + d) = v;
    }
  }
}

__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ logits, int64_t ld, int m_max,
                                                          const int32_t* __restrict__ m_dev, int V,
                                                          int32_t* __restrict__ out32, int64_t* __restrict__ out64) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int t = blockIdx.x;
  if (t >= rd::live_rows(m_dev, m_max)) return;
  const float* row = logits + (int64_t)t * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += 256) {
    const float f = row[v];
    if (f > best || (f == best && v < bi)) {
      best = f;
      bi = v;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
    }
  }
  __shared__ float sb[8];
  __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) {
    sb[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i)
      if (sb[i] > best || (sb[i] == best && si[i] < bi)) {
        best = sb[i];
        bi = si[i];
      }
    if (bi == 0x7fffffff) bi = 0;
    if (out32) out32[t] = bi;
    if (out64) out64[t] = bi;
  }
}

__global__ void emit_tokens_kernel(const int64_t* __restrict__ token_buf, int max_len, const int32_t* __restrict__ kv_begin,
                                   const int32_t* __restrict__ kv_len, const int64_t* __restrict__ next_tokens,
                                   int64_t pad_id, int out_len, int64_t* __restrict__ out) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int b = blockIdx.x;
  const int len = kv_len[b], begin = kv_begin[b];
  const int lead = out_len - 1 - len;  // pad ids on the left
  for (int c = threadIdx.x; c < out_len; c += blockDim.x) {
    int64_t v;
    if (c == out_len - 1)
      v = next_tokens[b];
    else if (c < lead)
      v = pad_id;
    else
      v = token_buf[(int64_t)b * max_len + begin + (c - lead)];
    out[(int64_t)b * out_len + c] = v;
  }
}

__global__ void commit_reference_slots_kernel(int W, int Lb, const int32_t* __restrict__ unpacker,
                                              const int32_t* __restrict__ n_accepted,
                                              const int32_t* __restrict__ seq_in_beam, int S, int S2,
                                              int64_t* __restrict__ out) {
  const int b = blockIdx.x, j = threadIdx.x;
  if (j >= Lb) return;
  const int A = n_accepted[b], seq = seq_in_beam[b];
  int64_t* o = out + ((int64_t)b * Lb + j) * 3;
  if (j <= A) {
    o[0] = S + unpacker[((int64_t)b * W + seq) * Lb + j];
    o[1] = S + seq * Lb + j;
    o[2] = S2 - (A + 1) + j;
  } else {
    o[0] = o[1] = o[2] = -1;
  }
}

// Cache.unpack of the reference layout: gather into scratch, then write back.
template <typename T>
__global__ void cache_unpack_gather_kernel(const T* __restrict__ cache, int B, int nkv, int max_len, int hd, int S,
                                           const int64_t* __restrict__ unpacker, int n_flat, T* __restrict__ scratch) {
  // grid (n_flat, B*nkv, NL*2)
  const int f = blockIdx.x, bh = blockIdx.y, lk = blockIdx.z;
  const int b = bh / nkv;
  const int64_t src_slot = S + unpacker[(int64_t)b * n_flat + f];
  const T* src = cache + (((int64_t)lk * B * nkv + bh) * max_len + src_slot) * hd;
  T* dst = scratch + (((int64_t)lk * B * nkv + bh) * n_flat + f) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) dst[d] = src[d];
}
template <typename T>
__global__ void cache_unpack_scatter_kernel(T* __restrict__ cache, int B, int nkv, int max_len, int hd, int S, int n_flat,
                                            const T* __restrict__ scratch) {
  const int f = blockIdx.x, bh = blockIdx.y, lk = blockIdx.z;
  const T* src = scratch + (((int64_t)lk * B * nkv + bh) * n_flat + f) * hd;
  T* dst = cache + (((int64_t)lk * B * nkv + bh) * max_len + S + f) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) dst[d] = src[d];
}

// Staging array of rd_cache_unpack_static.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel may be given.
__device__ __align__(256) unsigned char g_static_unpack_scratch[RD_STATIC_SCRATCH_BYTES];

}  // namespace

#define RD_DISPATCH_T(dtype, ...)                  \
  if ((dtype) == RD_F32) {                         \
    using T = float;                               \
    __VA_ARGS__;                                   \
  } else if ((dtype) == RD_BF16) {                 \
    using T = __nv_bfloat16;                       \
    __VA_ARGS__;                                   \
  } else {                                         \
    return RD_ERR_DTYPE;                           \
  }

extern "C" int rd_embed_gather(int dtype, const void* table, const int64_t* ids, void* out, int m_max,
                               const int32_t* m_dev, int H, void* stream) {
  RD_REQUIRE(table && ids && out, RD_ERR_ARG);
  RD_REQUIRE(m_max >= 1 && H >= 1, RD_ERR_SIZE);
  cudaStream_t s = (cudaStream_t)stream;
  const int esz = dtype == RD_F32 ? 4 : 2;
  const int vec = ((H * esz) % 16 == 0) && ((((uintptr_t)table | (uintptr_t)out) & 15) == 0);
  cudaError_t err = cudaSuccess;
  RD_DISPATCH_T(dtype, (err = rd::launch_chained(embed_gather_kernel<T>, dim3(m_max), dim3(256), 0, s, 1, (const T*)table, ids, (T*)out,
                                                 m_max, m_dev, H, vec)));
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_rmsnorm(int dtype, const void* x, const void* weight, void* y, int m_max, const int32_t* m_dev, int H,
                          float eps, void* stream) {
  RD_REQUIRE(x && weight && y, RD_ERR_ARG);
  RD_REQUIRE(m_max >= 1 && H >= 1, RD_ERR_SIZE);
  cudaStream_t s = (cudaStream_t)stream;
  const int vec = dtype == RD_F32 ? 4 : 8;
  const int vectorised = (H % vec == 0) && (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)y) % 16 == 0);
  cudaError_t err = cudaSuccess;
  RD_DISPATCH_T(dtype, (err = rd::launch_chained(rmsnorm_kernel<T>, dim3(m_max), dim3(256), 0, s, 1, (const T*)x, (const T*)weight,
                                                 (T*)y, m_max, m_dev, H, eps, vectorised)));
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_rope_kv_write(int dtype, const void* qkv, void* q_out, void* k_cache, void* v_cache,
                                const int32_t* tok_row, const int32_t* tok_pos, const int32_t* tok_slot,
                                const float* cos_table, const float* sin_table, int n_pos, int m_max,
                                const int32_t* m_dev, int nh, int nkv, int hd, int max_len, void* stream) {
  RD_REQUIRE(qkv && q_out && k_cache && v_cache && tok_row && tok_pos && tok_slot && cos_table && sin_table, RD_ERR_ARG);
  RD_REQUIRE(m_max >= 1 && nh >= 1 && nkv >= 1 && hd >= 2 && hd % 2 == 0 && max_len >= 1 && n_pos >= 1, RD_ERR_SIZE);
  {
    // 16-byte vector accesses: half a head must be a whole number of vectors and every base aligned
    const int vec = dtype == RD_F32 ? 4 : 8;
    RD_REQUIRE((hd / 2) % vec == 0, RD_ERR_ALIGN);
    RD_REQUIRE(((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0, RD_ERR_ALIGN);
  }
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t err = cudaSuccess;
  RD_DISPATCH_T(dtype, (err = rd::launch_chained(rope_kv_write_kernel<T>, dim3(m_max), dim3(kRopeThreads), 0, s, 1, (const T*)qkv, (T*)q_out,
                                                 (T*)k_cache, (T*)v_cache, tok_row, tok_pos, tok_slot, cos_table, sin_table,
                                                 n_pos, m_max, m_dev, nh, nkv, hd, max_len)));
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_argmax_rows(const float* logits, int64_t ld, int m_max, const int32_t* m_dev, int V, int32_t* out32,
                              int64_t* out64, void* stream) {
  RD_REQUIRE(logits && (out32 || out64), RD_ERR_ARG);
  RD_REQUIRE(m_max >= 1 && V >= 1 && ld >= V, RD_ERR_SIZE);
  cudaError_t err = rd::launch_chained(argmax_rows_kernel, dim3(m_max), dim3(256), 0, (cudaStream_t)stream, 1, logits, ld, m_max, m_dev, V,
                                       out32, out64);
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_emit_tokens(const int64_t* token_buf, int max_len, const int32_t* kv_begin, const int32_t* kv_len,
                              const int64_t* next_tokens, int64_t pad_id, int B, int out_len, int64_t* out,
                              void* stream) {
  RD_REQUIRE(token_buf && kv_begin && kv_len && next_tokens && out, RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && out_len >= 1 && max_len >= 1, RD_ERR_SIZE);
  cudaError_t err = rd::launch_chained(emit_tokens_kernel, dim3(B), dim3(256), 0, (cudaStream_t)stream, 1, token_buf, max_len, kv_begin,
                                       kv_len, next_tokens, pad_id, out_len, out);
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_commit_reference_slots(int B, int W, int Lb, const int32_t* unpacker, const int32_t* n_accepted,
                                         const int32_t* seq_in_beam, int S, int S2, int64_t* out, void* stream) {
  RD_REQUIRE(unpacker && n_accepted && seq_in_beam && out, RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && W >= 1 && Lb >= 1 && Lb <= RD_MAX_BEAM_LENGTH, RD_ERR_SIZE);
  commit_reference_slots_kernel<<<B, 32, 0, (cudaStream_t)stream>>>(W, Lb, unpacker, n_accepted, seq_in_beam, S, S2, out);
  RD_CHECK_LAUNCH();
  return RD_OK;
}

extern "C" int rd_cache_unpack(int dtype, void* cache, int NL, int B, int nkv, int max_len, int hd, int S,
                               const int64_t* unpacker, int n_flat, void* scratch, void* stream) {
  RD_REQUIRE(cache && unpacker && scratch, RD_ERR_ARG);
  RD_REQUIRE(NL >= 1 && B >= 1 && nkv >= 1 && hd >= 1 && S >= 0 && n_flat >= 1 && S + n_flat <= max_len &&
                 (int64_t)B * nkv <= 65535 && NL * 2 <= 65535,
             RD_ERR_SIZE);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_flat, B * nkv, NL * 2);
  RD_DISPATCH_T(dtype, {
    cache_unpack_gather_kernel<T><<<grid, 64, 0, s>>>((const T*)cache, B, nkv, max_len, hd, S, unpacker, n_flat, (T*)scratch);
    cache_unpack_scatter_kernel<T><<<grid, 64, 0, s>>>((T*)cache, B, nkv, max_len, hd, S, n_flat, (const T*)scratch);
  });
  RD_CHECK_LAUNCH();
  return RD_OK;
}

// Device address of g_static_unpack_scratch per device ordinal, looked up on the first call made
// with that device current.  Looking it up twice from two host threads yields the same value.
static void* g_static_scratch_addr[64] = {};

extern "C" int rd_cache_unpack_static(int dtype, void* cache, int NL, int B, int nkv, int max_len, int hd, int S,
                                      const int64_t* unpacker, int n_flat, void* stream) {
  RD_REQUIRE(cache && unpacker, RD_ERR_ARG);
  RD_REQUIRE(dtype == RD_F32 || dtype == RD_BF16, RD_ERR_DTYPE);
  RD_REQUIRE(NL >= 1 && B >= 1 && nkv >= 1 && hd >= 1 && S >= 0 && n_flat >= 1 && S + n_flat <= max_len &&
                 (int64_t)B * nkv <= 65535 && NL * 2 <= 65535,
             RD_ERR_SIZE);
  {
    // bytes gathered = NL*2 * B*nkv * n_flat * hd * element size; the product is formed factor by factor
    // and refused as soon as it passes the capacity, so it cannot wrap around
    const unsigned long long cap = (unsigned long long)RD_STATIC_SCRATCH_BYTES;
    unsigned long long need = dtype == RD_F32 ? 4ull : 2ull;
    const unsigned long long factors[4] = {(unsigned long long)NL * 2ull, (unsigned long long)B * (unsigned long long)nkv,
                                           (unsigned long long)n_flat, (unsigned long long)hd};
    for (int i = 0; i < 4; ++i) {
      RD_REQUIRE(factors[i] <= cap, RD_ERR_CAPACITY);
      need *= factors[i];  // both operands <= 2^24 here: no overflow
      RD_REQUIRE(need <= cap, RD_ERR_CAPACITY);
    }
  }
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0) {
    rd_set_last_cuda_error((int)err);
    return RD_ERR_LAUNCH;
  }
  RD_REQUIRE(dev < 64, RD_ERR_UNSUPPORTED);  // the address table below holds 64 device ordinals
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_static_unpack_scratch);
    if (err != cudaSuccess || p == nullptr) {
      rd_set_last_cuda_error((int)err);
      return RD_ERR_LAUNCH;
    }
    g_static_scratch_addr[dev] = p;
  }
  void* scratch = g_static_scratch_addr[dev];
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_flat, B * nkv, NL * 2);
  RD_DISPATCH_T(dtype, {
    cache_unpack_gather_kernel<T><<<grid, 64, 0, s>>>((const T*)cache, B, nkv, max_len, hd, S, unpacker, n_flat, (T*)scratch);
    cache_unpack_scatter_kernel<T><<<grid, 64, 0, s>>>((T*)cache, B, nkv, max_len, hd, S, n_flat, (const T*)scratch);
  });
  RD_CHECK_LAUNCH();
  return RD_OK;
}
