// Prefix-tree pack of draft beams: dedup of shared prefixes, unpacker, flat packed token list,
// positions, cache slots and the compact tree-attention bitmask.  Integer work only.
//
// One warp owns one batch row.  Lane l holds beams l and l+32, so W <= 64.  The canonical id of
// the depth-j prefix of beam i is the smallest beam index sharing that prefix; two beams share a
// depth-j prefix iff they share the depth-(j-1) id and token j, which turns the dedup into one
// warp-wide match per depth.
#include "rd_common.cuh"

namespace {

constexpr int kMaxLb = RD_MAX_BEAM_LENGTH;

struct PackArgs {
  const int64_t* beams;
  int B, W, Lb;
  const int32_t* kv_begin;
  const int32_t* kv_len;
  int32_t* prefix_tree;
  int32_t* unpacker;
  int32_t* n_selected;
  int32_t* row_start;
  int64_t* flat_tokens;
  int32_t* flat_index;
  int32_t* tok_row;
  int32_t* tok_pos;
  int32_t* tok_slot;
  uint32_t* tree_mask;
  int mask_words;
  int32_t* base_len;
};

// Phase A for one batch row, executed by one warp: prefix ids, unpacker, n_selected.
__device__ void pack_row_ids(const PackArgs& a, int b, int lane, int32_t* seg_start /*[64] smem of this warp*/) {
  const int W = a.W, Lb = a.Lb;
  const int64_t* bm = a.beams + (int64_t)b * W * Lb;
  const int i0 = lane, i1 = lane + 32;
  const bool act0 = i0 < W, act1 = i1 < W;
  const uint32_t m0 = __ballot_sync(0xffffffffu, act0);
  const uint32_t m1 = __ballot_sync(0xffffffffu, act1);
  int pid0[kMaxLb], pid1[kMaxLb];
  int prev0 = 0, prev1 = 0;
#pragma unroll
  for (int j = 0; j < kMaxLb; ++j) {
    if (j < Lb) {
      // inactive lanes carry a token no live lane can hold together with a live prefix id
      unsigned long long t0 = act0 ? (unsigned long long)bm[i0 * Lb + j] : 0ull;
      unsigned long long t1 = act1 ? (unsigned long long)bm[i1 * Lb + j] : 0ull;
      // beams 0..31 among themselves
      uint32_t e0 = __match_any_sync(0xffffffffu, t0) & __match_any_sync(0xffffffffu, prev0) & m0;
      int p0 = act0 ? (__ffs(e0) - 1) : 0;
      // beams 32..63: first against beams 0..31, then among themselves
      int p1 = -1;
      for (int l = 0; l < 32; ++l) {
        unsigned long long tl = __shfl_sync(0xffffffffu, t0, l);
        int pl = __shfl_sync(0xffffffffu, prev0, l);
        if (p1 < 0 && l < W && tl == t1 && pl == prev1) p1 = l;
      }
      uint32_t e1 = __match_any_sync(0xffffffffu, t1) & __match_any_sync(0xffffffffu, prev1) & m1;
      if (p1 < 0) p1 = 32 + __ffs(e1) - 1;
      if (!act1) p1 = 0;
      pid0[j] = p0;
      pid1[j] = p1;
      prev0 = p0;
      prev1 = p1;
    }
  }
  // nodes owned by each beam and the exclusive scan over beams (segment starts)
  int own0 = 0, own1 = 0;
#pragma unroll
  for (int j = 0; j < kMaxLb; ++j)
    if (j < Lb) {
      own0 += (act0 && pid0[j] == i0);
      own1 += (act1 && pid1[j] == i1);
    }
  int s0 = own0, s1 = own1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int v0 = __shfl_up_sync(0xffffffffu, s0, o);
    int v1 = __shfl_up_sync(0xffffffffu, s1, o);
    if (lane >= o) {
      s0 += v0;
      s1 += v1;
    }
  }
  const int tot0 = __shfl_sync(0xffffffffu, s0, 31);
  const int tot1 = __shfl_sync(0xffffffffu, s1, 31);
  seg_start[i0] = s0 - own0;
  seg_start[i1] = tot0 + s1 - own1;
  __syncwarp();
  if (lane == 0) a.n_selected[b] = tot0 + tot1;
  // unpacker = segment start of the owning beam + earlier tokens of this beam in the same segment
#pragma unroll
  for (int j = 0; j < kMaxLb; ++j)
    if (j < Lb) {
      if (act0) {
        int off = 0;
        for (int jj = 0; jj < j; ++jj) off += (pid0[jj] == pid0[j]);
        a.unpacker[((int64_t)b * W + i0) * Lb + j] = seg_start[pid0[j]] + off;
        a.prefix_tree[((int64_t)b * W + i0) * Lb + j] = pid0[j];
      }
      if (act1) {
        int off = 0;
        for (int jj = 0; jj < j; ++jj) off += (pid1[jj] == pid1[j]);
        a.unpacker[((int64_t)b * W + i1) * Lb + j] = seg_start[pid1[j]] + off;
        a.prefix_tree[((int64_t)b * W + i1) * Lb + j] = pid1[j];
      }
    }
  __syncwarp();
}

// Phase B for one batch row: flat arrays and the bitmask, from the ids written by phase A.
__device__ void pack_row_emit(const PackArgs& a, int b, int lane, int rs) {
  const int W = a.W, Lb = a.Lb;
  const int begin = a.kv_begin ? a.kv_begin[b] : 0;
  const int len = a.kv_len ? a.kv_len[b] : 0;
  if (lane == 0 && a.base_len) a.base_len[b] = len;
  for (int i = lane; i < W; i += 32) {
    const int64_t base = ((int64_t)b * W + i) * Lb;
    int u[kMaxLb];
#pragma unroll
    for (int j = 0; j < kMaxLb; ++j) u[j] = (j < Lb) ? a.unpacker[base + j] : 0;
#pragma unroll
    for (int j = 0; j < kMaxLb; ++j) {
      if (j < Lb && a.prefix_tree[base + j] == i) {
        const int t = rs + u[j];
        a.flat_tokens[t] = a.beams[base + j];
        a.flat_index[t] = i * Lb + j;
        a.tok_row[t] = b;
        a.tok_pos[t] = len + j;
        a.tok_slot[t] = begin + len + u[j];
        for (int w = 0; w < a.mask_words; ++w) {
          uint32_t bits = 0;
#pragma unroll
          for (int jj = 0; jj < kMaxLb; ++jj)
            if (jj <= j && (u[jj] >> 5) == w) bits |= 1u << (u[jj] & 31);
          a.tree_mask[(int64_t)t * a.mask_words + w] = bits;
        }
      }
    }
  }
}

constexpr int kRowsPerCta = 4;  // one warp per batch row

// Phase A: prefix ids, unpacker and n_selected of every row (rows are independent).
__global__ void __launch_bounds__(kRowsPerCta * 32) tree_pack_ids_kernel(PackArgs a) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  __shared__ int32_t seg[kRowsPerCta][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kRowsPerCta + warp;
  if (b < a.B) pack_row_ids(a, b, lane, seg[warp]);
}

// Phase B: each warp sums the counts of the rows before its own (the batch is small), publishes
// row_start and writes its row's slice of the flat arrays and the bitmask.
__global__ void __launch_bounds__(kRowsPerCta * 32) tree_pack_emit_kernel(PackArgs a) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kRowsPerCta + warp;
  if (b >= a.B) return;
  int before = 0;
  for (int r = lane; r < b; r += 32) before += a.n_selected[r];
  before = rd::warp_sum_i(before);
  if (lane == 0) {
    a.row_start[b] = before;
    if (b == a.B - 1) a.row_start[a.B] = before + a.n_selected[b];
  }
  pack_row_emit(a, b, lane, before);
}

struct RefArgs {
  int B, W, Lb, N, S;
  const int32_t* unpacker;
  const int32_t* n_selected;
  const int32_t* row_start;
  const int64_t* flat_tokens;
  const int32_t* flat_index;
  const int64_t* padding_mask;
  int64_t* packed_beams;
  int64_t* packed_token_indices;
  int64_t* position_offsets;
  uint8_t* causal_mask;
  int64_t* unpacker64;
};

// grid (N, B): one block per (packed position p, batch row b)
__global__ void tree_pack_reference_kernel(RefArgs a) {
  const int p = blockIdx.x, b = blockIdx.y;
  const int total = a.row_start[a.B];
  int read = a.row_start[b] + p;
  if (read > total - 1) read = total - 1;
  const int idx = a.flat_index[read];
  const int m = idx / a.Lb, k = idx % a.Lb;
  if (threadIdx.x == 0) {
    a.packed_beams[(int64_t)b * a.N + p] = a.flat_tokens[read];
    a.packed_token_indices[(int64_t)b * a.N + p] = idx;
    a.position_offsets[(int64_t)b * a.N + p] = k;
  }
  if (p == 0 && a.unpacker64) {
    for (int e = threadIdx.x; e < a.W * a.Lb; e += blockDim.x)
      a.unpacker64[(int64_t)b * a.W * a.Lb + e] = a.unpacker[(int64_t)b * a.W * a.Lb + e];
  }
  __shared__ int u[kMaxLb];
  if (threadIdx.x < a.Lb) u[threadIdx.x] = a.unpacker[((int64_t)b * a.W + m) * a.Lb + threadIdx.x];
  __syncthreads();
  uint8_t* row = a.causal_mask + ((int64_t)b * a.N + p) * (a.S + a.N);
  for (int c = threadIdx.x; c < a.S + a.N; c += blockDim.x) {
    uint8_t v;
    if (c < a.S) {
      v = a.padding_mask[(int64_t)b * a.S + c] != 0;
    } else {
      const int q = c - a.S;
      v = 0;
      for (int j = 0; j <= k; ++j) v |= (u[j] == q);
    }
    row[c] = v;
  }
}

}  // namespace

extern "C" int rd_tree_pack(const int64_t* beams, int B, int W, int Lb, const int32_t* kv_begin, const int32_t* kv_len,
                            int32_t* prefix_tree, int32_t* unpacker, int32_t* n_selected, int32_t* row_start,
                            int64_t* flat_tokens, int32_t* flat_index, int32_t* tok_row, int32_t* tok_pos,
                            int32_t* tok_slot, uint32_t* tree_mask, int mask_words, int32_t* base_len, void* stream) {
  RD_REQUIRE(beams && prefix_tree && unpacker && n_selected && row_start && flat_tokens && flat_index && tok_row &&
                 tok_pos && tok_slot && tree_mask,
             RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && B <= 4096 && W >= 1 && W <= RD_MAX_BEAM_WIDTH && Lb >= 1 && Lb <= RD_MAX_BEAM_LENGTH,
             RD_ERR_SIZE);
  RD_REQUIRE(mask_words * 32 >= W * Lb, RD_ERR_SIZE);
  PackArgs a{beams,      B,          W,       Lb,      kv_begin, kv_len,    prefix_tree, unpacker,  n_selected,
             row_start,  flat_tokens, flat_index, tok_row, tok_pos,  tok_slot,  tree_mask,   mask_words, base_len};
  const int grid = (B + kRowsPerCta - 1) / kRowsPerCta;
  cudaError_t err = rd::launch_chained(tree_pack_ids_kernel, dim3(grid), dim3(kRowsPerCta * 32), 0, (cudaStream_t)stream, 1, a);
  if (err == cudaSuccess)
    err = rd::launch_chained(tree_pack_emit_kernel, dim3(grid), dim3(kRowsPerCta * 32), 0, (cudaStream_t)stream, 1, a);
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_tree_pack_reference_layout(int B, int W, int Lb, const int32_t* unpacker, const int32_t* n_selected,
                                             const int32_t* row_start, const int64_t* flat_tokens,
                                             const int32_t* flat_index, int N, const int64_t* padding_mask, int S,
                                             int64_t* packed_beams, int64_t* packed_token_indices,
                                             int64_t* position_offsets, uint8_t* causal_mask, int64_t* unpacker64,
                                             void* stream) {
  RD_REQUIRE(unpacker && n_selected && row_start && flat_tokens && flat_index && packed_beams &&
                 packed_token_indices && position_offsets && causal_mask,
             RD_ERR_ARG);
  RD_REQUIRE(S == 0 || padding_mask, RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && B <= 65535 && W >= 1 && W <= RD_MAX_BEAM_WIDTH && Lb >= 1 && Lb <= RD_MAX_BEAM_LENGTH &&
                 N >= 1 && N <= W * Lb && S >= 0,
             RD_ERR_SIZE);
  RefArgs a{B,          W,           Lb,          N,           S,           unpacker,
            n_selected, row_start,   flat_tokens, flat_index,  padding_mask, packed_beams,
            packed_token_indices, position_offsets, causal_mask, unpacker64};
  tree_pack_reference_kernel<<<dim3(N, B), 128, 0, (cudaStream_t)stream>>>(a);
  RD_CHECK_LAUNCH();
  return RD_OK;
}
