// Drafter beam-search kernels other than the GEMMs: operand staging for the recurrent update,
// vocabulary-wide top-k warp + log-softmax with sparse output, cross-beam top-W and beam reorder,
// categorical draws from sparse distributions.
#include "rd_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------
// rd_drafter_prepare
template <typename T>
__global__ void drafter_prepare_kernel(const T* __restrict__ embed, const int64_t* __restrict__ beams,
                                       const int32_t* __restrict__ parent, const T* __restrict__ ctx, T* __restrict__ a,
                                       T* __restrict__ x, int W, int Lb, int H, int k, int vec, int additive) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int r = blockIdx.x;
  const int b = r / W;
  const int64_t tok = beams[(int64_t)r * Lb + k];
  const T* e = embed + tok * (int64_t)H;
  T* arow = a + (int64_t)r * 2 * H;
  T* xrow = x + (int64_t)r * 2 * H;
  const T* c = ctx + (int64_t)b * H;
  const T* s = (k == 0) ? nullptr : x + ((int64_t)b * W + parent[r]) * 2 * H + H;
  constexpr int VEC = 16 / sizeof(T);
  if (vec) {
    // 16-byte copies: a = [embedding(token), parent state or zeros]; x[:H] = context (first iteration only)
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int d = threadIdx.x; d < H / VEC; d += blockDim.x) {
      const uint4 ev = reinterpret_cast<const uint4*>(e)[d];
      uint4 sv = s ? reinterpret_cast<const uint4*>(s)[d] : zero;
      if (additive) {
        // drafter without the recurrent projections: new state = embedding + parent state
        const T* ep = reinterpret_cast<const T*>(&ev);
        T* sp = reinterpret_cast<T*>(&sv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) sp[i] = rd::Num<T>::from_f(rd::Num<T>::to_f(ep[i]) + rd::Num<T>::to_f(sp[i]));
      }
      reinterpret_cast<uint4*>(arow)[d] = ev;
      reinterpret_cast<uint4*>(arow + H)[d] = sv;
      if (k == 0) reinterpret_cast<uint4*>(xrow)[d] = reinterpret_cast<const uint4*>(c)[d];
    }
    return;
  }
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    arow[d] = e[d];
    const float sv = s ? rd::Num<T>::to_f(s[d]) : 0.f;
    arow[H + d] = rd::Num<T>::from_f(additive ? rd::Num<T>::to_f(e[d]) + sv : sv);
    if (k == 0) xrow[d] = c[d];
  }
}

// ---------------------------------------------------------------------------------------------
// rd_vocab_topk: one block per row, the row is streamed twice from global memory (the second pass
// hits L2) and never staged in shared memory.
//
//   1. every thread takes the maximum of its strided share of the row; the top_k-th largest of these
//      512 thread maxima is a LOWER bound T0 of the row's top_k-th largest value (the thread maxima
//      are distinct elements of the row), and their largest is the row maximum;
//   2. second pass: the elements >= T0 (typically one or two hundred) are collected;
//   3. the exact top_k threshold, the ties at it and the (value descending, id ascending) order come
//      from ranking the candidates against each other;
//   4. log-softmax over the warped row from the kept entries alone (masked entries share one value).
// A row with more than kCandCap elements >= T0 (massive ties) takes the radix-select path, which
// reads the row a few more times.
constexpr int kTopkThreads = 512;
constexpr int kKept = RD_TOPK_MAX_KEPT;
constexpr int kCandCap = 2048;

template <typename T>
struct RowReader {
  const T* src;
  int V;
  bool vec;  // 16-byte loads allowed
  // Optional per-slice maxima of this row (slice = 32 consecutive ids), element s at smax[s * smax_ld], written
  // by the GEMM that produced the row: with them the row is read only where it can hold values >= a bound.
  const float* smax;
  int64_t smax_ld;
  static constexpr int VEC = 16 / sizeof(T);
  // calls f(slice maximum) for this thread's share of the slices
  template <typename F>
  __device__ __forceinline__ void for_each_slice_max(int tid, F f) const {
    const int n_slices = V >> 5;
    for (int sl = tid; sl < n_slices; sl += kTopkThreads) f(smax[(int64_t)sl * smax_ld]);
  }
  // calls f(value, index) for the elements of the slices whose maximum is >= bound
  template <typename F>
  __device__ __forceinline__ void for_each_in_slices_at_least(int tid, float bound, F f) const {
    const int n_slices = V >> 5;
    for (int sl = tid; sl < n_slices; sl += kTopkThreads) {
      if (!(smax[(int64_t)sl * smax_ld] >= bound)) continue;
#pragma unroll
      for (int c = 0; c < 32 / VEC; ++c) {
        T e[VEC];
        *reinterpret_cast<uint4*>(e) = reinterpret_cast<const uint4*>(src + sl * 32)[c];
#pragma unroll
        for (int j = 0; j < VEC; ++j) f(rd::Num<T>::to_f(e[j]), sl * 32 + c * VEC + j);
      }
    }
  }
  // calls f(value, index) for this thread's share of the row
  template <typename F>
  __device__ __forceinline__ void for_each(int tid, F f) const {
    if (vec) {
      const int nvec = V / VEC;
      for (int i = tid; i < nvec; i += kTopkThreads) {
        T e[VEC];
        *reinterpret_cast<uint4*>(e) = reinterpret_cast<const uint4*>(src)[i];
#pragma unroll
        for (int j = 0; j < VEC; ++j) f(rd::Num<T>::to_f(e[j]), i * VEC + j);
      }
      for (int v = nvec * VEC + tid; v < V; v += kTopkThreads) f(rd::Num<T>::to_f(src[v]), v);
    } else {
      for (int v = tid; v < V; v += kTopkThreads) f(rd::Num<T>::to_f(src[v]), v);
    }
  }
};

struct TopkShared {
  float lmax[kTopkThreads];
  float cval[kCandCap];
  int cidx[kCandCap];
  int hist[256];
  int scan[kTopkThreads];
  float sv[kKept];
  int si[kKept];
  float t0, mx, thr;
  int ccount, gt, ties, n_gt_fallback;
  uint32_t sel_prefix;
  int sel_remaining;
};

// Radix-select path for rows whose candidate set does not fit: exact threshold by 8-bit digits over
// the whole row (read from global memory), then entries above it and ties in index order.
template <typename T>
__device__ void topk_radix_path(const RowReader<T>& row, TopkShared& sh, int top_k, int tid, int lane) {
  const int V = row.V;
  if (tid == 0) {
    sh.sel_prefix = 0;
    sh.sel_remaining = top_k < V ? top_k : V;
  }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const uint32_t hi_mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < 256; i += kTopkThreads) sh.hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = sh.sel_prefix;
    for (int v0 = 0; v0 < V; v0 += kTopkThreads) {
      const int v = v0 + tid;
      uint32_t key = 0;
      bool in = false;
      if (v < V) {
        key = rd::float_key(rd::Num<T>::to_f(row.src[v]));
        in = (key & hi_mask) == prefix;
      }
      const uint32_t digit = in ? ((key >> shift) & 255u) : 256u;
      const uint32_t peers = __match_any_sync(0xffffffffu, digit);
      if (in && lane == (__ffs(peers) - 1)) atomicAdd(&sh.hist[digit], __popc(peers));
    }
    __syncthreads();
    if (tid == 0) {
      int rem = sh.sel_remaining, d = 255;
      for (; d > 0; --d) {
        if (sh.hist[d] >= rem) break;
        rem -= sh.hist[d];
      }
      sh.sel_prefix = prefix | ((uint32_t)d << shift);
      sh.sel_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t thr_key = sh.sel_prefix;
  if (tid == 0) sh.n_gt_fallback = 0;
  __syncthreads();
  // entries strictly above the threshold (fewer than top_k), any order, into cval/cidx
  for (int v = tid; v < V; v += kTopkThreads) {
    const float f = rd::Num<T>::to_f(row.src[v]);
    if (rd::float_key(f) > thr_key) {
      const int s = atomicAdd(&sh.n_gt_fallback, 1);
      if (s < kKept) {
        sh.cval[s] = f;
        sh.cidx[s] = v;
      }
    }
  }
  // ties in ascending index order while capacity lasts (blocked assignment + scan)
  const int chunk = (V + kTopkThreads - 1) / kTopkThreads;
  const int v0 = tid * chunk, v1 = min(V, v0 + chunk);
  int my_ties = 0;
  float thr_val = 0.f;
  for (int v = v0; v < v1; ++v) {
    const float f = rd::Num<T>::to_f(row.src[v]);
    if (rd::float_key(f) == thr_key) {
      ++my_ties;
      thr_val = f;
    }
  }
  sh.scan[tid] = my_ties;
  __syncthreads();
  for (int o = 1; o < kTopkThreads; o <<= 1) {
    const int add = tid >= o ? sh.scan[tid - o] : 0;
    __syncthreads();
    sh.scan[tid] += add;
    __syncthreads();
  }
  const int gt = min(sh.n_gt_fallback, kKept);
  int pos = gt + sh.scan[tid] - my_ties;
  for (int v = v0; v < v1; ++v) {
    const float f = rd::Num<T>::to_f(row.src[v]);
    if (rd::float_key(f) == thr_key) {
      if (pos < kKept) {
        sh.cval[pos] = f;
        sh.cidx[pos] = v;
      }
      ++pos;
    }
  }
  if (my_ties > 0) sh.thr = thr_val;
  if (tid == kTopkThreads - 1) {
    sh.gt = gt;
    sh.ties = sh.scan[tid];
    sh.ccount = min(kKept, gt + sh.scan[tid]);
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads) vocab_topk_kernel(
    const T* __restrict__ logits, int64_t ld, int rows_max, const int32_t* __restrict__ rows_dev, int V, int top_k,
    float mask_value, int subtract_max, float temperature, int vec_ok, const float* __restrict__ slice_max, int64_t slice_ld,
    float* __restrict__ kept_val, int32_t* __restrict__ kept_idx, int32_t* __restrict__ kept_cnt,
    float* __restrict__ masked_logp) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int row_id = blockIdx.x;
  if (row_id >= rd::live_rows(rows_dev, rows_max)) return;
  __shared__ TopkShared sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool sliced = slice_max != nullptr;
  RowReader<T> row{logits + (int64_t)row_id * ld, V, vec_ok != 0, sliced ? slice_max + row_id : nullptr, slice_ld};
  const int K = top_k < V ? top_k : V;

  // 1. thread maxima -> lower bound T0 of the K-th largest value, and the row maximum.  With slice maxima
  //    the thread maxima come from them (each is an element of the row, distinct slices hold distinct
  //    elements), so this pass reads V/32 floats instead of the row.
  float lm = -INFINITY;
  if (sliced)
    row.for_each_slice_max(tid, [&](float f) { lm = fmaxf(lm, f); });
  else
    row.for_each(tid, [&](float f, int) { lm = fmaxf(lm, f); });
  if (tid == 0) {
    sh.ccount = 0;
    sh.gt = 0;
    sh.ties = 0;
    sh.t0 = -INFINITY;
  }
  // Each warp publishes its four largest thread maxima: kTopkThreads / 8 = 64 distinct elements of
  // the row, so the K-th largest of them (K <= 64) cannot exceed the K-th largest of the row.
  {
    float v = lm;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float m = rd::warp_max(v);
      const uint32_t eq = __ballot_sync(0xffffffffu, v == m);
      if (lane == 0) sh.lmax[warp * 4 + r] = m;
      if (lane == __ffs(eq) - 1) v = -INFINITY;  // retire one holder of the maximum
    }
  }
  __syncthreads();
  if (warp == 0) {
    constexpr int kVals = kTopkThreads / 8;  // 64
    float best = -INFINITY;
#pragma unroll
    for (int h = 0; h < kVals / 32; ++h) {
      const int me = h * 32 + lane;
      const float mv = sh.lmax[me];
      best = fmaxf(best, mv);
      int rank = 0;
      for (int o = 0; o < kVals; ++o) {
        const float ov = sh.lmax[o];
        rank += (ov > mv) || (ov == mv && o < me);
      }
      if (rank == K - 1 && mv > -INFINITY) sh.t0 = mv;  // stays -inf when fewer than K values exist
    }
    best = rd::warp_max(best);
    if (lane == 0) sh.mx = best;
  }
  __syncthreads();
  const float t0 = sh.t0, mx = sh.mx;

  // 2. candidates (every element >= T0 lies in a slice whose maximum is >= T0)
  auto take = [&](float f, int v) {
    if (f >= t0) {
      const int s = atomicAdd(&sh.ccount, 1);
      if (s < kCandCap) {
        sh.cval[s] = f;
        sh.cidx[s] = v;
      }
    }
  };
  if (sliced)
    row.for_each_in_slices_at_least(tid, t0, take);
  else
    row.for_each(tid, take);
  __syncthreads();
  const int n_cand = sh.ccount;
  int cnt;
  if (n_cand > kCandCap) {
    __syncthreads();
    topk_radix_path(row, sh, K, tid, lane);
    cnt = sh.ccount;
    // order the (at most kKept) survivors
    if (tid < cnt) {
      const float mv = sh.cval[tid];
      const int mi = sh.cidx[tid];
      int rank = 0;
      for (int o = 0; o < cnt; ++o) rank += (sh.cval[o] > mv) || (sh.cval[o] == mv && sh.cidx[o] < mi);
      sh.sv[rank] = mv;
      sh.si[rank] = mi;
    }
    __syncthreads();
  } else {
    // 3. rank the candidates: unique ranks in (value descending, id ascending) order
    int my_rank[kCandCap / kTopkThreads];
#pragma unroll
    for (int c = 0; c < kCandCap / kTopkThreads; ++c) {
      const int i = c * kTopkThreads + tid;
      my_rank[c] = -1;
      if (i < n_cand) {
        const float mv = sh.cval[i];
        const int mi = sh.cidx[i];
        int rank = 0;
        for (int o = 0; o < n_cand; ++o) {
          const float ov = sh.cval[o];
          rank += (ov > mv) || (ov == mv && sh.cidx[o] < mi);
        }
        my_rank[c] = rank;
        if (rank == K - 1) sh.thr = mv;
      }
    }
    __syncthreads();
    const float thr = sh.thr;
#pragma unroll
    for (int c = 0; c < kCandCap / kTopkThreads; ++c) {
      const int i = c * kTopkThreads + tid;
      if (i < n_cand) {
        const float mv = sh.cval[i];
        if (mv > thr) atomicAdd(&sh.gt, 1);
        if (mv == thr) atomicAdd(&sh.ties, 1);
      }
    }
    __syncthreads();
    cnt = min(kKept, sh.gt + sh.ties);
#pragma unroll
    for (int c = 0; c < kCandCap / kTopkThreads; ++c) {
      const int i = c * kTopkThreads + tid;
      if (i < n_cand && my_rank[c] >= 0 && my_rank[c] < cnt) {
        sh.sv[my_rank[c]] = sh.cval[i];
        sh.si[my_rank[c]] = sh.cidx[i];
      }
    }
    __syncthreads();
  }

  // 4. log-softmax over the warped row: kept entries, ties that did not fit, and masked entries
  if (warp == 0) {
    const int gt = sh.gt, ties = sh.ties;
    const float shift = subtract_max ? mx : 0.f;
    const float top = (sh.sv[0] - shift) / temperature;
    const float masked_s = mask_value / temperature;
    const float m = fmaxf(top, masked_s);
    float acc = 0.f;
    for (int o = lane; o < cnt; o += 32) acc += expf((sh.sv[o] - shift) / temperature - m);
    acc = rd::warp_sum(acc);
    const float thr_val = sh.sv[cnt - 1] - shift;
    const int dropped = gt + ties - cnt;
    const int n_masked = V - gt - ties;
    acc += (float)dropped * expf(thr_val / temperature - m);
    acc += (float)n_masked * expf(masked_s - m);
    const float lse = m + logf(acc);
    for (int o = lane; o < kKept; o += 32) {
      const bool live = o < cnt;
      kept_val[(int64_t)row_id * kKept + o] = live ? ((sh.sv[o] - shift) / temperature - lse) : -INFINITY;
      kept_idx[(int64_t)row_id * kKept + o] = live ? sh.si[o] : -1;
    }
    if (lane == 0) {
      kept_cnt[row_id] = cnt;
      masked_logp[row_id] = masked_s - lse;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// rd_beam_select: kSelSplit blocks per batch row (each holds all lists, ranks a share of the candidates).
//
// Every row's kept list is sorted by (log-prob descending, id ascending), so adding the row's beam
// score keeps it non-increasing.  The candidates' total order is (score descending, beam index
// ascending, position in the beam's list ascending) - for distinct scores that is torch.topk's
// order, for equal scores it is the flat-index order w*V+token whenever the tie is exact in the
// log-probs as well.  A candidate's rank is its own position plus, for every other beam, the number
// of entries that precede it, found by binary search; ranks below W are the new beams.
constexpr int kSelThreads = 256;
constexpr int kSelSplit = 8;  // CTAs per batch row: each ranks its share of the candidates against all lists

__global__ void __launch_bounds__(kSelThreads) beam_select_kernel(
    int W, int Lb, int k, int V, const float* __restrict__ kept_val, const int32_t* __restrict__ kept_idx,
    const int32_t* __restrict__ kept_cnt, const float* __restrict__ score_in, float* __restrict__ score_out,
    const int64_t* __restrict__ beams_in, int64_t* __restrict__ beams_out, const int32_t* __restrict__ anc_in,
    int32_t* __restrict__ anc_out, int32_t* __restrict__ parent_out) {
  rd::pdl_launch_dependents();
  rd::pdl_wait();
  const int b = blockIdx.x;
  extern __shared__ unsigned char raw[];
  float* cs = reinterpret_cast<float*>(raw);  // [W][W] candidate scores, row w = beam w's list
  int* len = reinterpret_cast<int*>(cs + W * W);  // [W] usable length of each list
  for (int w = threadIdx.x; w < W; w += kSelThreads) {
    const int cnt = kept_cnt[b * W + w];
    len[w] = min(min(cnt, W), kKept);
  }
  __syncthreads();
  const int ncand = W * W;
  for (int c = threadIdx.x; c < ncand; c += kSelThreads) {
    const int w = c / W, i = c % W;
    const int r = b * W + w;
    const float base = (k == 0) ? (w == 0 ? 0.f : RD_LOG_0) : score_in[r];
    cs[c] = (i < len[w]) ? kept_val[(int64_t)r * kKept + i] + base : -INFINITY;
  }
  __syncthreads();
  for (int c = blockIdx.y * kSelThreads + threadIdx.x; c < ncand; c += kSelThreads * gridDim.y) {
    const int w = c / W, i = c % W;
    if (i >= len[w]) continue;
    const float s = cs[c];
    int rank = i;
    for (int o = 0; o < W && rank < W; ++o) {
      if (o == w) continue;
      // entries of list o that precede (s, w): score > s, or score == s when o < w
      const float* lo_list = cs + o * W;
      int lo = 0, hi = len[o];
      // the lists are sorted: most of them contribute nothing (head does not precede) or everything
      if (hi == 0) continue;
      {
        const float head = lo_list[0], tail = lo_list[hi - 1];
        if (!((o < w) ? (head >= s) : (head > s))) continue;
        if ((o < w) ? (tail >= s) : (tail > s)) {
          rank += hi;
          continue;
        }
        lo = 1;
        hi = hi - 1;
      }
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        const float v = lo_list[mid];
        const bool before = (o < w) ? (v >= s) : (v > s);
        if (before)
          lo = mid + 1;
        else
          hi = mid;
      }
      rank += lo;
    }
    if (rank < W) {
      const int dst = b * W + rank;
      const int r = b * W + w;
      score_out[dst] = s;
      parent_out[dst] = w;
      const int64_t* src_beam = beams_in + (int64_t)r * Lb;
      int64_t* dst_beam = beams_out + (int64_t)dst * Lb;
      for (int j = 0; j <= k; ++j) dst_beam[j] = src_beam[j];
      dst_beam[k + 1] = (int64_t)kept_idx[(int64_t)r * kKept + i];
      const int32_t* src_anc = anc_in + (int64_t)r * (Lb - 1);
      int32_t* dst_anc = anc_out + (int64_t)dst * (Lb - 1);
      for (int j = 0; j < k; ++j) dst_anc[j] = src_anc[j];
      dst_anc[k] = w;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// rd_drafter_dense_log_probs
struct SparseLists {
  const float* val[RD_MAX_BEAM_LENGTH];
  const int32_t* idx[RD_MAX_BEAM_LENGTH];
  const int32_t* cnt[RD_MAX_BEAM_LENGTH];
  const float* masked[RD_MAX_BEAM_LENGTH];
};

__global__ void dense_log_probs_kernel(int W, int Lb, int V, SparseLists s, const int32_t* __restrict__ anc,
                                       float* __restrict__ out) {
  // block = (b*W + w)*(Lb-1) + j
  const int j = blockIdx.x % (Lb - 1);
  const int bw = blockIdx.x / (Lb - 1);
  const int b = bw / W;
  const int r = b * W + anc[(int64_t)bw * (Lb - 1) + j];
  float* dst = out + (int64_t)blockIdx.x * V;
  const float m = s.masked[j][r];
  for (int v = threadIdx.x; v < V; v += blockDim.x) dst[v] = m;
  __syncthreads();
  const int cnt = s.cnt[j][r];
  for (int o = threadIdx.x; o < cnt; o += blockDim.x) dst[s.idx[j][(int64_t)r * kKept + o]] = s.val[j][(int64_t)r * kKept + o];
}

// ---------------------------------------------------------------------------------------------
// rd_sample_from_sparse: one warp per row.
__global__ void sample_sparse_kernel(const float* __restrict__ kept_val, const int32_t* __restrict__ kept_idx,
                                     const int32_t* __restrict__ kept_cnt, int rows, const float* __restrict__ uniforms,
                                     int64_t* __restrict__ out) {
  const int row = blockIdx.x;
  __shared__ float p[kKept];
  __shared__ int id[kKept];
  const int cnt = kept_cnt[row];
  const int t = threadIdx.x;
  if (t < cnt) {
    const int mi = kept_idx[(int64_t)row * kKept + t];
    int rank = 0;
    for (int o = 0; o < cnt; ++o) rank += kept_idx[(int64_t)row * kKept + o] < mi;
    p[rank] = expf(kept_val[(int64_t)row * kKept + t]);
    id[rank] = mi;
  }
  __syncthreads();
  if (t == 0) {
    float total = 0.f;
    for (int o = 0; o < cnt; ++o) total += p[o];
    const float target = uniforms[row] * total;
    float c = 0.f;
    int pick = -1, last = -1;
    for (int o = 0; o < cnt; ++o) {
      if (p[o] > 0.f) {
        c += p[o];
        last = o;
        if (pick < 0 && c > target) pick = o;
      }
    }
    if (pick < 0) pick = last >= 0 ? last : 0;
    out[row] = id[pick];
  }
}

}  // namespace

extern "C" int rd_drafter_prepare(int dtype, const void* embed, const int64_t* beams, const int32_t* parent,
                                  const void* ctx, void* a, void* x, int B, int W, int Lb, int H, int k, int additive,
                                  void* stream) {
  RD_REQUIRE(embed && beams && ctx && a && x, RD_ERR_ARG);
  RD_REQUIRE(k == 0 || parent, RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && W >= 1 && W <= RD_MAX_BEAM_WIDTH && Lb >= 2 && Lb <= RD_MAX_BEAM_LENGTH && H >= 1 && k >= 0 &&
                 k < Lb - 1,
             RD_ERR_SIZE);
  cudaStream_t s = (cudaStream_t)stream;
  const int esz = dtype == RD_F32 ? 4 : 2;
  const int vec = ((H * esz) % 16 == 0) && ((((uintptr_t)embed | (uintptr_t)ctx | (uintptr_t)a | (uintptr_t)x) & 15) == 0);
  cudaError_t err = cudaSuccess;
  if (dtype == RD_F32)
    err = rd::launch_chained(drafter_prepare_kernel<float>, dim3(B * W), dim3(256), 0, s, 1, (const float*)embed, beams, parent,
                             (const float*)ctx, (float*)a, (float*)x, W, Lb, H, k, vec, additive);
  else if (dtype == RD_BF16)
    err = rd::launch_chained(drafter_prepare_kernel<__nv_bfloat16>, dim3(B * W), dim3(256), 0, s, 1, (const __nv_bfloat16*)embed,
                             beams, parent, (const __nv_bfloat16*)ctx, (__nv_bfloat16*)a, (__nv_bfloat16*)x, W, Lb, H, k, vec, additive);
  else
    return RD_ERR_DTYPE;
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

static int vocab_topk_launch(int logits_dtype, const void* logits, int64_t ld, int rows_max, const int32_t* rows_dev, int V,
                             int top_k, float mask_value, int subtract_max, float temperature, const float* slice_max,
                             int64_t slice_ld, float* kept_val, int32_t* kept_idx, int32_t* kept_cnt, float* masked_logp,
                             void* stream) {
  RD_REQUIRE(logits && kept_val && kept_idx && kept_cnt && masked_logp, RD_ERR_ARG);
  RD_REQUIRE(rows_max >= 1 && V >= 1 && top_k >= 1 && top_k <= RD_TOPK_MAX_KEPT && ld >= V, RD_ERR_SIZE);
  RD_REQUIRE(temperature > 0.f, RD_ERR_ARG);
  if (slice_max) {
    // whole slices of 32 ids, read with 16-byte loads
    RD_REQUIRE(V % 32 == 0 && slice_ld >= rows_max, RD_ERR_SIZE);
    RD_REQUIRE((uintptr_t)logits % 16 == 0 && (ld * (logits_dtype == RD_F32 ? 4 : 2)) % 16 == 0, RD_ERR_ALIGN);
  }
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t err = cudaSuccess;
  if (logits_dtype == RD_F32) {
    const int vec_ok = ((uintptr_t)logits % 16 == 0) && ((ld * 4) % 16 == 0);
    err = rd::launch_chained(vocab_topk_kernel<float>, dim3(rows_max), dim3(kTopkThreads), 0, s, 1, (const float*)logits, ld, rows_max,
                             rows_dev, V, top_k, mask_value, subtract_max, temperature, vec_ok, slice_max, slice_ld, kept_val, kept_idx,
                             kept_cnt, masked_logp);
  } else if (logits_dtype == RD_BF16) {
    const int vec_ok = ((uintptr_t)logits % 16 == 0) && ((ld * 2) % 16 == 0);
    err = rd::launch_chained(vocab_topk_kernel<__nv_bfloat16>, dim3(rows_max), dim3(kTopkThreads), 0, s, 1,
                             (const __nv_bfloat16*)logits, ld, rows_max, rows_dev, V, top_k, mask_value, subtract_max, temperature,
                             vec_ok, slice_max, slice_ld, kept_val, kept_idx, kept_cnt, masked_logp);
  } else {
    return RD_ERR_DTYPE;
  }
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_vocab_topk(int logits_dtype, const void* logits, int64_t ld, int rows_max, const int32_t* rows_dev,
                             int V, int top_k, float mask_value, int subtract_max, float temperature, float* kept_val,
                             int32_t* kept_idx, int32_t* kept_cnt, float* masked_logp, void* stream) {
  return vocab_topk_launch(logits_dtype, logits, ld, rows_max, rows_dev, V, top_k, mask_value, subtract_max, temperature, nullptr, 0,
                           kept_val, kept_idx, kept_cnt, masked_logp, stream);
}

extern "C" int rd_vocab_topk_sliced(int logits_dtype, const void* logits, int64_t ld, int rows_max, const int32_t* rows_dev,
                                    int V, int top_k, float mask_value, int subtract_max, float temperature,
                                    const float* slice_max, int64_t slice_ld, float* kept_val, int32_t* kept_idx,
                                    int32_t* kept_cnt, float* masked_logp, void* stream) {
  RD_REQUIRE(slice_max, RD_ERR_ARG);
  return vocab_topk_launch(logits_dtype, logits, ld, rows_max, rows_dev, V, top_k, mask_value, subtract_max, temperature, slice_max,
                           slice_ld, kept_val, kept_idx, kept_cnt, masked_logp, stream);
}

extern "C" int rd_beam_select(int B, int W, int Lb, int k, int V, const float* kept_val, const int32_t* kept_idx,
                              const int32_t* kept_cnt, const float* score_in, float* score_out,
                              const int64_t* beams_in, int64_t* beams_out, const int32_t* anc_in, int32_t* anc_out,
                              int32_t* parent_out, void* stream) {
  RD_REQUIRE(kept_val && kept_idx && kept_cnt && score_out && beams_in && beams_out && anc_in && anc_out && parent_out,
             RD_ERR_ARG);
  RD_REQUIRE(k == 0 || score_in, RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && W >= 1 && W <= RD_MAX_BEAM_WIDTH && Lb >= 2 && Lb <= RD_MAX_BEAM_LENGTH && k >= 0 && k < Lb - 1,
             RD_ERR_SIZE);
  RD_REQUIRE((int64_t)W * V < (int64_t)INT32_MAX, RD_ERR_SIZE);
  const size_t smem = (size_t)W * W * sizeof(float) + (size_t)W * sizeof(int);
  cudaError_t err = rd::launch_chained(beam_select_kernel, dim3(B, kSelSplit), dim3(kSelThreads), smem, (cudaStream_t)stream, 1, W, Lb, k, V,
                                       kept_val, kept_idx, kept_cnt, score_in, score_out, beams_in, beams_out, anc_in, anc_out,
                                       parent_out);
  RD_CHECK_CHAINED(err);
  return RD_OK;
}

extern "C" int rd_drafter_dense_log_probs(int B, int W, int Lb, int V, const float* const* kept_val_host,
                                          const int32_t* const* kept_idx_host, const int32_t* const* kept_cnt_host,
                                          const float* const* masked_logp_host, const int32_t* anc, float* out,
                                          void* stream) {
  RD_REQUIRE(kept_val_host && kept_idx_host && kept_cnt_host && masked_logp_host && anc && out, RD_ERR_ARG);
  RD_REQUIRE(B >= 1 && W >= 1 && Lb >= 2 && Lb <= RD_MAX_BEAM_LENGTH && V >= 1, RD_ERR_SIZE);
  SparseLists s{};
  for (int j = 0; j < Lb - 1; ++j) {
    s.val[j] = kept_val_host[j];
    s.idx[j] = kept_idx_host[j];
    s.cnt[j] = kept_cnt_host[j];
    s.masked[j] = masked_logp_host[j];
    RD_REQUIRE(s.val[j] && s.idx[j] && s.cnt[j] && s.masked[j], RD_ERR_ARG);
  }
  dense_log_probs_kernel<<<B * W * (Lb - 1), 256, 0, (cudaStream_t)stream>>>(W, Lb, V, s, anc, out);
  RD_CHECK_LAUNCH();
  return RD_OK;
}

extern "C" int rd_sample_from_sparse(const float* kept_val, const int32_t* kept_idx, const int32_t* kept_cnt, int rows,
                                     const float* uniforms, int64_t* out, void* stream) {
  RD_REQUIRE(kept_val && kept_idx && kept_cnt && uniforms && out, RD_ERR_ARG);
  RD_REQUIRE(rows >= 1, RD_ERR_SIZE);
  sample_sparse_kernel<<<rows, kKept, 0, (cudaStream_t)stream>>>(kept_val, kept_idx, kept_cnt, rows, uniforms, out);
  RD_CHECK_LAUNCH();
  return RD_OK;
}
