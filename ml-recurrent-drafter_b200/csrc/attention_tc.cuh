// bf16 flash attention of new tokens over a per-row KV cache (cached prefix + causal or
// prefix-tree visibility among the new tokens), tensor-core path.
//
// One CTA = 8 warps = 128 queries of one (batch row, head) - normally all the packed tree tokens
// of the row, so that K/V are read once per (row, head); each warp owns 16 queries.  K/V tiles of
// 64 keys stream through a three-stage cp.async pipeline in XOR-swizzled shared memory; S = Q K^T
// and O += P V run on mma.sync m16n8k16 (bf16 in, fp32 accumulate) with ldmatrix-fed fragments;
// the softmax is the online (running max / running sum) form in the exp2 domain.  Tiles that lie
// wholly inside the cached prefix skip the mask; tiles overlapping the new tokens read the tree
// bitmask rows staged in shared memory.
#pragma once
#include "rd_common.cuh"

namespace rd_attn {

constexpr int kBM = 128;  // queries per CTA
constexpr int kBN = 64;  // keys per tile
constexpr int kThreads = 256;
constexpr int kStages = 3;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0 zero-fills the 16 destination bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `c` of row `r` in a tile whose rows hold HD bf16 values.
template <int HD>
__device__ __forceinline__ int swz(int r, int c) {
  return r * (HD * 2) + ((c ^ (r & 7)) << 4);
}

template <int HD>
struct Smem {
  static constexpr int kTile = kBN * HD * 2;           // one K or V tile
  static constexpr int kQ = kBM * HD * 2;              // the Q tile
  static constexpr int kBytes = kQ + 2 * kStages * kTile;  // Q + stages x (K, V)
};

template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const __nv_bfloat16* src_base, int row0, int row_end, int tid) {
  // 64 rows x (HD/8) chunks of 16 bytes
  constexpr int kChunks = HD / 8;
#pragma unroll
  for (int i = 0; i < (kBN * kChunks) / kThreads; ++i) {
    const int idx = i * kThreads + tid;
    const int r = idx / kChunks, c = idx % kChunks;
    const bool valid = row0 + r < row_end;
    const __nv_bfloat16* src = src_base + (int64_t)(valid ? row0 + r : row0) * HD + c * 8;
    cp_async16(dst + swz<HD>(r, c), src, valid);
  }
}

template <int HD>
__global__ void __launch_bounds__(kThreads) attention_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
    __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ row_start, const int32_t* __restrict__ kv_begin,
    const int32_t* __restrict__ base_len, int nh, int nkv, int max_len, int mode, const uint32_t* __restrict__ tree_mask,
    int mask_words, float scale_log2) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int rs = row_start[b];
  const int n_new = row_start[b + 1] - rs;
  const int q0 = blockIdx.x * kBM;
  if (q0 >= n_new) return;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + Smem<HD>::kQ;  // stage s: K at sKV + s*2*kTile, V right after it
  uint32_t* sMask = reinterpret_cast<uint32_t*>(smem + Smem<HD>::kBytes);  // [kBM][mask_words]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int base = base_len[b];
  const int hk = h / (nh / nkv);
  const int kv_end = (mode == RD_ATTN_CAUSAL) ? base + min(n_new, q0 + kBM) : base + n_new;
  const int n_tiles = (kv_end + kBN - 1) / kBN;
  const __nv_bfloat16* kbase = k_cache + (((int64_t)b * nkv + hk) * max_len + kv_begin[b]) * HD;
  const __nv_bfloat16* vbase = v_cache + (((int64_t)b * nkv + hk) * max_len + kv_begin[b]) * HD;

  // Q tile (rows beyond n_new zero-filled) and the tile's mask rows
  {
    constexpr int kChunks = HD / 8;
#pragma unroll
    for (int i = 0; i < (kBM * kChunks) / kThreads; ++i) {
      const int idx = i * kThreads + tid;
      const int r = idx / kChunks, c = idx % kChunks;
      const bool valid = q0 + r < n_new;
      const __nv_bfloat16* src = q + ((int64_t)(rs + (valid ? q0 + r : 0)) * nh + h) * HD + c * 8;
      cp_async16(sQ + swz<HD>(r, c), src, valid);
    }
    if (mode == RD_ATTN_TREE) {
      for (int i = tid; i < kBM * mask_words; i += kThreads) {
        const int r = i / mask_words, w = i % mask_words;
        sMask[i] = (q0 + r < n_new) ? tree_mask[(int64_t)(rs + q0 + r) * mask_words + w] : 0u;
      }
    }
  }
  // prologue: tiles 0 and 1 in flight (every iteration commits exactly one group, empty or not,
  // so that "all but the newest group" always means "tile `it` has landed")
  load_tile<HD>(sKV, kbase, 0, kv_end, tid);
  load_tile<HD>(sKV + Smem<HD>::kTile, vbase, 0, kv_end, tid);
  cp_async_commit();
  if (n_tiles > 1) {
    load_tile<HD>(sKV + 2 * Smem<HD>::kTile, kbase, kBN, kv_end, tid);
    load_tile<HD>(sKV + 3 * Smem<HD>::kTile, vbase, kBN, kv_end, tid);
  }
  cp_async_commit();

  uint32_t qf[HD / 16][4];
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int qi0 = q0 + warp * 16 + g;  // this thread's query rows: qi0 and qi0 + 8

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % kStages;
    cp_async_wait<1>();
    __syncthreads();  // tile `it` visible to all; everyone is done with tile it-1, whose stage is refilled next
    if (it + 2 < n_tiles) {
      uint8_t* dst = sKV + ((it + 2) % kStages) * 2 * Smem<HD>::kTile;
      load_tile<HD>(dst, kbase, (it + 2) * kBN, kv_end, tid);
      load_tile<HD>(dst + Smem<HD>::kTile, vbase, (it + 2) * kBN, kv_end, tid);
    }
    cp_async_commit();
    if (it == 0) {
      // Q fragments stay in registers for the whole kernel
#pragma unroll
      for (int kd = 0; kd < HD / 16; ++kd) {
        const int r = warp * 16 + (lane & 15);
        const int c = kd * 2 + (lane >> 4);
        ldmatrix_x4(qf[kd][0], qf[kd][1], qf[kd][2], qf[kd][3], smem_addr(sQ + swz<HD>(r, c)));
      }
    }
    const uint8_t* sK = sKV + stage * 2 * Smem<HD>::kTile;
    const uint8_t* sV = sK + Smem<HD>::kTile;

    // S = Q K^T for 16 queries x 64 keys
    float s[kBN / 8][4];
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int kd = 0; kd < HD / 16; ++kd) {
#pragma unroll
      for (int nb = 0; nb < kBN / 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        const int r = nb * 8 + ((lane >> 4) << 3) + (lane & 7);
        const int c = kd * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b0, b1, b2, b3, smem_addr(sK + swz<HD>(r, c)));
        mma_bf16(s[nb], qf[kd], b0, b1);
        mma_bf16(s[nb + 1], qf[kd], b2, b3);
      }
    }

    // scale, mask, online softmax
    const int j0 = it * kBN;
    const bool need_mask = (j0 + kBN > base) || (j0 + kBN > kv_end);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nb][e] * scale_log2;
        if (need_mask) {
          const int j = j0 + nb * 8 + t4 * 2 + (e & 1);
          const int half = e >> 1;
          const int qi = qi0 + half * 8;
          bool vis;
          if (j >= kv_end)
            vis = false;
          else if (j < base)
            vis = true;
          else {
            const int jn = j - base;
            if (mode == RD_ATTN_CAUSAL)
              vis = jn <= qi;
            else
              vis = (sMask[(warp * 16 + g + half * 8) * mask_words + (jn >> 5)] >> (jn & 31)) & 1u;
          }
          if (!vis) v = -INFINITY;
        }
        s[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], m_new[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
      m_new[hh] = fmaxf(m_run[hh], mx[hh]);
      const float m_use = (m_new[hh] == -INFINITY) ? 0.f : m_new[hh];
      alpha[hh] = (m_run[hh] == -INFINITY) ? 0.f : exp2f(m_run[hh] - m_use);
      m_run[hh] = m_new[hh];
      m_new[hh] = m_use;
    }
    float rowsum[2] = {0.f, 0.f};
    uint32_t pf[kBN / 16][4];
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb) {
      const float p0 = exp2f(s[nb][0] - m_new[0]);
      const float p1 = exp2f(s[nb][1] - m_new[0]);
      const float p2 = exp2f(s[nb][2] - m_new[1]);
      const float p3 = exp2f(s[nb][3] - m_new[1]);
      rowsum[0] += p0 + p1;
      rowsum[1] += p2 + p3;
      const int kb = nb >> 1;
      if ((nb & 1) == 0) {
        pf[kb][0] = pack_bf16(p0, p1);
        pf[kb][1] = pack_bf16(p2, p3);
      } else {
        pf[kb][2] = pack_bf16(p0, p1);
        pf[kb][3] = pack_bf16(p2, p3);
      }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) l_run[hh] = l_run[hh] * alpha[hh] + rowsum[hh];
#pragma unroll
    for (int db = 0; db < HD / 8; ++db) {
      o[db][0] *= alpha[0];
      o[db][1] *= alpha[0];
      o[db][2] *= alpha[1];
      o[db][3] *= alpha[1];
    }

    // O += P V
#pragma unroll
    for (int kb = 0; kb < kBN / 16; ++kb) {
#pragma unroll
      for (int db = 0; db < HD / 8; db += 2) {
        uint32_t b0, b1, b2, b3;
        const int r = kb * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
        const int c = db + (lane >> 4);
        ldmatrix_x4_trans(b0, b1, b2, b3, smem_addr(sV + swz<HD>(r, c)));
        mma_bf16(o[db], pf[kb], b0, b1);
        mma_bf16(o[db + 1], pf[kb], b2, b3);
      }
    }
  }
  cp_async_wait<0>();

  // finalise: divide by the row sums (summed over the quad) and store bf16
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int qi = qi0 + hh * 8;
    if (qi < n_new) {
      const float inv = l_run[hh] > 0.f ? 1.0f / l_run[hh] : 0.f;
      __nv_bfloat16* dst = out + ((int64_t)(rs + qi) * nh + h) * HD;
#pragma unroll
      for (int db = 0; db < HD / 8; ++db) {
        *reinterpret_cast<uint32_t*>(dst + db * 8 + t4 * 2) = pack_bf16(o[db][hh * 2] * inv, o[db][hh * 2 + 1] * inv);
      }
    }
  }
}

template <int HD>
inline int launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* row_start,
                  const int32_t* kv_begin, const int32_t* base_len, int B, int nh, int nkv, int max_len, int max_new, int mode,
                  const uint32_t* tree_mask, int mask_words, cudaStream_t s) {
  const size_t smem = Smem<HD>::kBytes + (size_t)kBM * (mask_words > 0 ? mask_words : 1) * sizeof(uint32_t);
  auto kern = attention_tc_kernel<HD>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((max_new + kBM - 1) / kBM, nh, B);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
  kern<<<grid, kThreads, smem, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                    (__nv_bfloat16*)out, row_start, kv_begin, base_len, nh, nkv, max_len, mode, tree_mask,
                                    mask_words, scale_log2);
  return 0;
}

}  // namespace rd_attn
