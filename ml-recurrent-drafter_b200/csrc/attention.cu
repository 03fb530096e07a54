// Attention of newly appended tokens over a per-row KV cache: a fully visible cached prefix
// followed by the new tokens themselves, which see each other causally (prefill, autoregressive
// step) or through the prefix-tree bitmask (verification of packed draft beams).
//
// Exact-fp32 path: one warp per (query, head); scores are staged in shared memory, so the softmax
// is the plain two-pass one.  Used for fp32 models and as the numerical cross-check of the
// tensor-core path.
#include "attention_tc.cuh"
#include "rd_common.cuh"

namespace {

constexpr int kQPB = 8;  // queries (warps) per block

template <typename T>
__global__ void __launch_bounds__(kQPB * 32) attention_rowwise_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
    const int32_t* __restrict__ row_start, const int32_t* __restrict__ kv_begin, const int32_t* __restrict__ base_len,
    int nh, int nkv, int hd, int max_len, int max_kv, int mode, const uint32_t* __restrict__ tree_mask, int mask_words,
    const uint8_t* __restrict__ dense_mask, int64_t dense_ld_q, int64_t dense_ld_b, float scale) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rs = row_start[b];
  const int n_new = row_start[b + 1] - rs;
  const int i = blockIdx.x * kQPB + warp;  // query index within the row
  if (i >= n_new) return;
  extern __shared__ float smem[];
  float* sc = smem + (size_t)warp * (max_kv + hd);  // [max_kv] scores
  float* qs = sc + max_kv;                          // [hd] the query in fp32
  const int base = base_len[b];
  int kv = base + n_new;
  if (kv > max_kv) kv = max_kv;  // host bound violated: stay inside shared memory
  const int t = rs + i;
  const int hk = h / (nh / nkv);
  const T* qrow = q + ((int64_t)t * nh + h) * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = rd::Num<T>::to_f(qrow[d]);
  __syncwarp();
  const T* kbase = k_cache + (((int64_t)b * nkv + hk) * max_len + kv_begin[b]) * hd;
  const T* vbase = v_cache + (((int64_t)b * nkv + hk) * max_len + kv_begin[b]) * hd;
  const uint32_t* mrow = tree_mask ? tree_mask + (int64_t)t * mask_words : nullptr;
  const uint8_t* drow = dense_mask ? dense_mask + (int64_t)b * dense_ld_b + (int64_t)i * dense_ld_q : nullptr;

  // scores: lanes over keys
  float mx = -INFINITY;
  for (int j = lane; j < kv; j += 32) {
    bool vis;
    if (mode == RD_ATTN_DENSE)
      vis = drow[j] != 0;
    else if (j < base)
      vis = true;
    else {
      const int jn = j - base;
      vis = (mode == RD_ATTN_CAUSAL) ? (jn <= i) : ((mrow[jn >> 5] >> (jn & 31)) & 1u);
    }
    float s = -INFINITY;
    if (vis) {
      const T* kr = kbase + (int64_t)j * hd;
      float acc = 0.f;
      for (int d = 0; d < hd; ++d) acc = fmaf(qs[d], rd::Num<T>::to_f(kr[d]), acc);
      s = acc * scale;
    }
    sc[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = rd::warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < kv; j += 32) {
    const float p = sc[j] == -INFINITY ? 0.f : expf(sc[j] - mx);
    sc[j] = p;
    sum += p;
  }
  sum = rd::warp_sum(sum);
  __syncwarp();
  const float inv = sum > 0.f ? 1.0f / sum : 0.f;
  // output: lanes over head_dim
  T* orow = out + ((int64_t)t * nh + h) * hd;
  for (int d = lane; d < hd; d += 32) {
    float acc = 0.f;
    for (int j = 0; j < kv; ++j) {
      const float p = sc[j];
      if (p != 0.f) acc = fmaf(p, rd::Num<T>::to_f(vbase[(int64_t)j * hd + d]), acc);
    }
    orow[d] = rd::Num<T>::from_f(acc * inv);
  }
}

}  // namespace

extern "C" int rd_attention(int dtype, const void* q, const void* k_cache, const void* v_cache, void* out,
                            const int32_t* row_start, const int32_t* kv_begin, const int32_t* base_len, int B, int nh,
                            int nkv, int hd, int max_len, int max_new, int max_kv, int mode, const uint32_t* tree_mask,
                            int mask_words, const uint8_t* dense_mask, int64_t dense_ld_q, int64_t dense_ld_b,
                            void* stream) {
  RD_REQUIRE(q && k_cache && v_cache && out && row_start && kv_begin && base_len, RD_ERR_ARG);
  RD_REQUIRE(mode == RD_ATTN_CAUSAL || (mode == RD_ATTN_TREE && tree_mask && mask_words >= 1) ||
                 (mode == RD_ATTN_DENSE && dense_mask),
             RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && B <= 65535 && nh >= 1 && nh <= 65535 && nkv >= 1 && nh % nkv == 0 && hd >= 1 && max_len >= 1 &&
                 max_new >= 1 && max_kv >= 1,
             RD_ERR_SIZE);
  cudaStream_t s = (cudaStream_t)stream;
  // bf16 with the common head sizes runs on the tensor cores; everything else (fp32 models, the
  // reference's explicit dense mask) on the exact row-wise kernel
  if (dtype == RD_BF16 && mode != RD_ATTN_DENSE && (hd == 128 || hd == 64)) {
    if (hd == 128)
      rd_attn::launch<128>(q, k_cache, v_cache, out, row_start, kv_begin, base_len, B, nh, nkv, max_len, max_new, mode,
                           tree_mask, mask_words, s);
    else
      rd_attn::launch<64>(q, k_cache, v_cache, out, row_start, kv_begin, base_len, B, nh, nkv, max_len, max_new, mode,
                          tree_mask, mask_words, s);
    RD_CHECK_LAUNCH();
    return RD_OK;
  }
  const size_t smem = (size_t)kQPB * (max_kv + hd) * sizeof(float);
  RD_REQUIRE(smem <= 220 * 1024, RD_ERR_SIZE);
  const float scale = 1.0f / sqrtf((float)hd);
  dim3 grid((max_new + kQPB - 1) / kQPB, nh, B);
  if (dtype == RD_F32) {
    auto kern = attention_rowwise_kernel<float>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, kQPB * 32, smem, s>>>((const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out,
                                       row_start, kv_begin, base_len, nh, nkv, hd, max_len, max_kv, mode, tree_mask,
                                       mask_words, dense_mask, dense_ld_q, dense_ld_b, scale);
  } else if (dtype == RD_BF16) {
    auto kern = attention_rowwise_kernel<__nv_bfloat16>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, kQPB * 32, smem, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                                       (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, row_start, kv_begin, base_len,
                                       nh, nkv, hd, max_len, max_kv, mode, tree_mask, mask_words, dense_mask, dense_ld_q,
                                       dense_ld_b, scale);
  } else {
    return RD_ERR_DTYPE;
  }
  RD_CHECK_LAUNCH();
  return RD_OK;
}
