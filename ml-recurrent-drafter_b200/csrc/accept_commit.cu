// Acceptance of draft tokens (greedy match or speculative sampling) fused with the commit of the
// accepted path: next-step inputs, token buffer and the move of the accepted tokens' K/V rows from
// their packed-tree slots to the tail of the row's sequence.
//
// Grid: (NL*2 + 1, B).  Every block re-derives the (cheap) acceptance decision of its batch row;
// block x = 0 writes the row's outputs, block x = 1 + layer*2 + kv moves the K/V rows of that plane.
// With NL = 0 the launch only decides (no cache is touched).
// Rows never move inside the cache: row b lives at slots [kv_begin[b], kv_begin[b]+kv_len[b]).
#include "rd_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kKept = RD_TOPK_MAX_KEPT;
constexpr int kMaxLb = RD_MAX_BEAM_LENGTH;
constexpr int kMaxW = RD_MAX_BEAM_WIDTH;

struct SparseRows {
  const float* val;
  const int32_t* idx;
  const int32_t* cnt;
  const float* masked;
};
struct SparseIter {
  const float* val[kMaxLb];
  const int32_t* idx[kMaxLb];
  const int32_t* cnt[kMaxLb];
  const float* masked[kMaxLb];
};

__device__ __forceinline__ float sparse_lookup(const float* val, const int32_t* idx, int cnt, float masked, int64_t row,
                                               int token) {
  const int32_t* ir = idx + row * kKept;
  for (int o = 0; o < cnt; ++o)
    if (ir[o] == token) return val[row * kKept + o];
  return masked;
}

struct CommitArgs {
  const int64_t* beams;
  int B, W, Lb, V;
  const int32_t* unpacker;
  const int32_t* row_start;
  const int32_t* llm_tokens;  // greedy
  SparseRows p;               // sampling: verify log-probs per flat token
  SparseIter q;               // sampling: drafter log-probs per iteration
  const int32_t* anc;
  const float* uniforms;
  const float* uniforms_next;
  const void* hidden;
  int H;
  void* cache;
  int NL, nkv, max_len, hd;
  const int32_t* kv_begin;
  const int32_t* base_len;
  int32_t* kv_len;
  int64_t* token_buf;
  int32_t* n_accepted;
  int32_t* seq_in_beam;
  int64_t* next_tokens;
  void* next_ctx;
  float* probs_dense;
};

template <typename T, bool SAMPLE>
__global__ void __launch_bounds__(kThreads) accept_commit_kernel(CommitArgs a) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int plane = (int)blockIdx.x - 1;  // layer*2 + kv; -1 = the block that writes the row outputs
  const int b = blockIdx.y;
  const int W = a.W, Lb = a.Lb;
  __shared__ int n_of_beam[kMaxW];
  __shared__ int s_n, s_seq;
  __shared__ int s_u[kMaxLb];
  const int tid = threadIdx.x;
  const int rs = a.row_start[b];

  // 1. accepted prefix length of every beam
  if (tid < W) {
    const int64_t* beam = a.beams + ((int64_t)b * W + tid) * Lb;
    const int32_t* u = a.unpacker + ((int64_t)b * W + tid) * Lb;
    int n = 0;
    for (int k = 0; k < Lb - 1; ++k) {
      const int64_t row = rs + u[k];
      const int tok = (int)beam[k + 1];
      bool ok;
      if (!SAMPLE) {
        ok = a.llm_tokens[row] == tok;
      } else {
        const float lp = sparse_lookup(a.p.val, a.p.idx, a.p.cnt[row], a.p.masked[row], row, tok);
        const int64_t qrow = (int64_t)b * W + a.anc[((int64_t)b * W + tid) * (Lb - 1) + k];
        const float lq = sparse_lookup(a.q.val[k], a.q.idx[k], a.q.cnt[k][qrow], a.q.masked[k][qrow], qrow, tok);
        ok = a.uniforms[((int64_t)b * W + tid) * (Lb - 1) + k] < expf(lp - lq);
      }
      if (!ok) break;
      ++n;
    }
    n_of_beam[tid] = n;
  }
  __syncthreads();
  // 2. longest accepted prefix, first beam among equals
  if (tid == 0) {
    int best = -1, bi = 0;
    for (int i = 0; i < W; ++i)
      if (n_of_beam[i] > best) {
        best = n_of_beam[i];
        bi = i;
      }
    s_n = best;
    s_seq = bi;
  }
  __syncthreads();
  const int A = s_n, seq = s_seq;
  if (tid < Lb) s_u[tid] = a.unpacker[((int64_t)b * W + seq) * Lb + tid];
  __syncthreads();
  const int base = a.base_len ? a.base_len[b] : 0;
  const int begin = a.kv_begin ? a.kv_begin[b] : 0;

  // 3. move the accepted path's K/V rows of this plane: packed slot u[j] -> position j.
  //    Sources and destinations overlap between different j, so everything is read first.
  if (plane >= 0) {
    const int row_bytes = a.hd * (int)sizeof(T);
    const int vec_per_row = row_bytes / 16;
    const int n_vec = a.nkv * (A + 1) * vec_per_row;
    T* plane_base = (T*)a.cache + ((int64_t)plane * a.B + b) * a.nkv * (int64_t)a.max_len * a.hd;
    constexpr int kMaxVecPerThread = 16;
    uint4 regs[kMaxVecPerThread];
    for (int chunk0 = 0; chunk0 < n_vec; chunk0 += kThreads * kMaxVecPerThread) {
      // a pass covers whole heads only when nkv*(A+1)*vec_per_row fits; otherwise split by head
      // ranges, which never overlap each other
#pragma unroll
      for (int r = 0; r < kMaxVecPerThread; ++r) {
        const int v = chunk0 + r * kThreads + tid;
        if (v < n_vec) {
          const int head = v / ((A + 1) * vec_per_row);
          const int rem = v % ((A + 1) * vec_per_row);
          const int j = rem / vec_per_row, c = rem % vec_per_row;
          const uint4* src =
              reinterpret_cast<const uint4*>(plane_base + ((int64_t)head * a.max_len + begin + base + s_u[j]) * a.hd);
          regs[r] = src[c];
        }
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kMaxVecPerThread; ++r) {
        const int v = chunk0 + r * kThreads + tid;
        if (v < n_vec) {
          const int head = v / ((A + 1) * vec_per_row);
          const int rem = v % ((A + 1) * vec_per_row);
          const int j = rem / vec_per_row, c = rem % vec_per_row;
          uint4* dst = reinterpret_cast<uint4*>(plane_base + ((int64_t)head * a.max_len + begin + base + j) * a.hd);
          dst[c] = regs[r];
        }
      }
      __syncthreads();
    }
  }
  if (plane >= 0) return;

  // 4. row outputs
  __shared__ int s_next;
  if (!SAMPLE) {
    if (tid == 0) s_next = a.llm_tokens[rs + s_u[A]];
  } else {
    // residual distribution over the verify row's kept list, in ascending token order
    __shared__ float pr[kKept];
    __shared__ int pid[kKept];
    const bool all_accepted = (A == Lb - 1);
    const int64_t prow = rs + s_u[A];
    const int pcnt = a.p.cnt[prow];
    const int kq = all_accepted ? 0 : A;
    const int64_t qrow = (int64_t)b * W + (all_accepted ? 0 : a.anc[((int64_t)b * W + seq) * (Lb - 1) + kq]);
    if (tid < pcnt) {
      const int tok = a.p.idx[prow * kKept + tid];
      int rank = 0;
      for (int o = 0; o < pcnt; ++o) rank += a.p.idx[prow * kKept + o] < tok;
      float pv = expf(a.p.val[prow * kKept + tid]);
      if (!all_accepted) {
        const float lq = sparse_lookup(a.q.val[kq], a.q.idx[kq], a.q.cnt[kq][qrow], a.q.masked[kq][qrow], qrow, tok);
        pv = fmaxf(pv - expf(lq), 0.f);
      }
      pr[rank] = pv;
      pid[rank] = tok;
    }
    __syncthreads();
    if (a.probs_dense) {
      float* dst = a.probs_dense + (int64_t)b * a.V;
      for (int v = tid; v < a.V; v += kThreads) dst[v] = 0.f;
      __syncthreads();
      if (tid < pcnt) dst[pid[tid]] = pr[tid];
    }
    if (tid == 0) {
      float total = 0.f;
      for (int o = 0; o < pcnt; ++o)
        if (pr[o] > 0.f) total += pr[o];
      const float target = a.uniforms_next[b] * total;
      float c = 0.f;
      int pick = -1, last = -1;
      for (int o = 0; o < pcnt; ++o)
        if (pr[o] > 0.f) {
          c += pr[o];
          last = o;
          if (pick < 0 && c > target) pick = o;
        }
      if (pick < 0) pick = last;
      // an all-zero residual (P <= Q everywhere on P's support) has no defined draw: take P's mode
      s_next = pick >= 0 ? pid[pick] : a.p.idx[prow * kKept];
    }
  }
  __syncthreads();
  if (tid == 0) {
    a.n_accepted[b] = A;
    a.seq_in_beam[b] = seq;
    a.next_tokens[b] = s_next;
    if (a.kv_len) a.kv_len[b] = base + A + 1;
  }
  if (a.token_buf && tid <= A)
    a.token_buf[(int64_t)b * a.max_len + begin + base + tid] = a.beams[((int64_t)b * W + seq) * Lb + tid];
  if (a.H > 0) {
    const T* hsrc = (const T*)a.hidden + (int64_t)(rs + s_u[A]) * a.H;
    T* hdst = (T*)a.next_ctx + (int64_t)b * a.H;
    for (int d = tid; d < a.H; d += kThreads) hdst[d] = hsrc[d];
  }
}

int check_common(const CommitArgs& a) {
  RD_REQUIRE(a.beams && a.unpacker && a.row_start && a.n_accepted && a.seq_in_beam && a.next_tokens, RD_ERR_ARG);
  RD_REQUIRE(a.NL == 0 || (a.cache && a.kv_begin && a.base_len), RD_ERR_ARG);
  RD_REQUIRE(a.H == 0 || (a.hidden && a.next_ctx), RD_ERR_ARG);
  RD_REQUIRE(a.token_buf == nullptr || (a.kv_begin && a.base_len), RD_ERR_ARG);
  RD_REQUIRE(a.kv_len == nullptr || a.base_len, RD_ERR_ARG);
  RD_REQUIRE(a.B >= 1 && a.B <= 65535 && a.W >= 1 && a.W <= kMaxW && a.Lb >= 2 && a.Lb <= kMaxLb && a.H >= 0 &&
                 a.NL >= 0 && (a.NL == 0 || (a.nkv >= 1 && a.max_len >= 1 && a.hd >= 1)),
             RD_ERR_SIZE);
  return RD_OK;
}

template <bool SAMPLE>
int launch(int dtype, const CommitArgs& a, cudaStream_t s) {
  dim3 grid(a.NL * 2 + 1, a.B);
  cudaError_t err = cudaSuccess;
  if (dtype == RD_F32) {
    RD_REQUIRE(a.NL == 0 || (a.hd * 4) % 16 == 0, RD_ERR_ALIGN);
    err = rd::launch_chained(accept_commit_kernel<float, SAMPLE>, grid, dim3(kThreads), 0, s, 1, a);
  } else if (dtype == RD_BF16) {
    RD_REQUIRE(a.NL == 0 || (a.hd * 2) % 16 == 0, RD_ERR_ALIGN);
    err = rd::launch_chained(accept_commit_kernel<__nv_bfloat16, SAMPLE>, grid, dim3(kThreads), 0, s, 1, a);
  } else {
    return RD_ERR_DTYPE;
  }
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

}  // namespace

extern "C" int rd_accept_commit_greedy(int dtype, const int64_t* beams, int B, int W, int Lb, const int32_t* unpacker,
                                       const int32_t* row_start, const int32_t* llm_tokens, const void* hidden, int H,
                                       void* cache, int NL, int nkv, int max_len, int hd, const int32_t* kv_begin,
                                       const int32_t* base_len, int32_t* kv_len, int64_t* token_buf,
                                       int32_t* n_accepted, int32_t* seq_in_beam, int64_t* next_tokens, void* next_ctx,
                                       void* stream) {
  CommitArgs a{};
  a.beams = beams; a.B = B; a.W = W; a.Lb = Lb; a.V = 0;
  a.unpacker = unpacker; a.row_start = row_start; a.llm_tokens = llm_tokens;
  a.hidden = hidden; a.H = H; a.cache = cache; a.NL = NL; a.nkv = nkv; a.max_len = max_len; a.hd = hd;
  a.kv_begin = kv_begin; a.base_len = base_len; a.kv_len = kv_len; a.token_buf = token_buf;
  a.n_accepted = n_accepted; a.seq_in_beam = seq_in_beam; a.next_tokens = next_tokens; a.next_ctx = next_ctx;
  RD_REQUIRE(llm_tokens, RD_ERR_ARG);
  int rc = check_common(a);
  if (rc != RD_OK) return rc;
  return launch<false>(dtype, a, (cudaStream_t)stream);
}

extern "C" int rd_accept_commit_sample(int dtype, const int64_t* beams, int B, int W, int Lb, int V,
                                       const int32_t* unpacker, const int32_t* row_start, const float* p_val,
                                       const int32_t* p_idx, const int32_t* p_cnt, const float* p_masked,
                                       const float* const* q_val_host, const int32_t* const* q_idx_host,
                                       const int32_t* const* q_cnt_host, const float* const* q_masked_host,
                                       const int32_t* anc, const float* uniforms, const float* uniforms_next,
                                       const void* hidden, int H, void* cache, int NL, int nkv, int max_len, int hd,
                                       const int32_t* kv_begin, const int32_t* base_len, int32_t* kv_len,
                                       int64_t* token_buf, int32_t* n_accepted, int32_t* seq_in_beam,
                                       int64_t* next_tokens, void* next_ctx, float* probs_dense, void* stream) {
  CommitArgs a{};
  a.beams = beams; a.B = B; a.W = W; a.Lb = Lb; a.V = V;
  a.unpacker = unpacker; a.row_start = row_start;
  a.p = SparseRows{p_val, p_idx, p_cnt, p_masked};
  RD_REQUIRE(p_val && p_idx && p_cnt && p_masked && q_val_host && q_idx_host && q_cnt_host && q_masked_host && anc &&
                 uniforms && uniforms_next,
             RD_ERR_ARG);
  RD_REQUIRE(Lb >= 2 && Lb <= kMaxLb && V >= 1, RD_ERR_SIZE);
  for (int j = 0; j < Lb - 1; ++j) {
    a.q.val[j] = q_val_host[j]; a.q.idx[j] = q_idx_host[j]; a.q.cnt[j] = q_cnt_host[j]; a.q.masked[j] = q_masked_host[j];
    RD_REQUIRE(a.q.val[j] && a.q.idx[j] && a.q.cnt[j] && a.q.masked[j], RD_ERR_ARG);
  }
  a.anc = anc; a.uniforms = uniforms; a.uniforms_next = uniforms_next;
  a.hidden = hidden; a.H = H; a.cache = cache; a.NL = NL; a.nkv = nkv; a.max_len = max_len; a.hd = hd;
  a.kv_begin = kv_begin; a.base_len = base_len; a.kv_len = kv_len; a.token_buf = token_buf;
  a.n_accepted = n_accepted; a.seq_in_beam = seq_in_beam; a.next_tokens = next_tokens; a.next_ctx = next_ctx;
  a.probs_dense = probs_dense;
  int rc = check_common(a);
  if (rc != RD_OK) return rc;
  return launch<true>(dtype, a, (cudaStream_t)stream);
}
