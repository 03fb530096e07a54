/*
 * C ABI of libredrafter_b200.so: the ReDrafter speculative-decoding step on B200 (sm_100a).
 *
 * The reference (apple/ml-recurrent-drafter) has no FFI: its hot path is Python calling PyTorch
 * operators.  Each entry point below replaces the group of PyTorch calls named in its comment
 * (file:line inside the reference project).  All pointers are DEVICE pointers unless marked
 * "host"; the caller owns every buffer; `stream` is a cudaStream_t passed as void*.  The library
 * never allocates or frees device memory, except where an entry point's comment says otherwise.
 *
 * Return value: 0 on success; negative = invalid argument found on the host before any launch.
 * No C++ exception crosses this boundary.  rd_strerror() names a code.
 *
 * Dynamic row counts: wherever an entry point takes (m_max, m_dev), buffers hold m_max rows and
 * only the first min(*m_dev, m_max) rows are computed; m_dev == NULL means all m_max rows.  This
 * lets a whole decode step be enqueued (or captured in a CUDA graph) without reading the packed
 * tree size back to the host.
 */
#ifndef REDRAFTER_B200_H_
#define REDRAFTER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RD_API __attribute__((visibility("default")))
#else
#define RD_API
#endif

#define RD_OK 0
#define RD_ERR_ARG (-1)         /* null pointer / negative size */
#define RD_ERR_DTYPE (-2)       /* unsupported dtype for this entry point */
#define RD_ERR_SIZE (-3)        /* size outside the supported range */
#define RD_ERR_LAUNCH (-4)      /* the CUDA launch was rejected; see rd_last_cuda_error() */
#define RD_ERR_ALIGN (-5)       /* pointer or leading dimension not aligned as required */
#define RD_ERR_UNSUPPORTED (-6) /* combination not implemented */
#define RD_ERR_CAPACITY (-7)    /* request larger than the fixed capacity of an entry point that cannot allocate */

#define RD_F32 0
#define RD_BF16 1

/* GEMM epilogues (C = epilogue(A * W^T)). */
#define RD_EPI_NONE 0          /* C = acc */
#define RD_EPI_BIAS 1          /* C = acc + bias[n] */
#define RD_EPI_BIAS_SILU 2     /* C = silu(acc + bias[n]) */
#define RD_EPI_BIAS_SILU_RES 3 /* C = R[m,n] + silu(acc + bias[n]) */
#define RD_EPI_RES 4           /* C = R[m,n] + acc (R may alias C) */
#define RD_EPI_SWIGLU 5        /* C[m,i] = silu(acc[m,2i]) * acc[m,2i+1]; C has N/2 columns */

/* Attention visibility of the new tokens among themselves. */
#define RD_ATTN_CAUSAL 0 /* new token i sees new tokens 0..i */
#define RD_ATTN_TREE 1   /* new token i sees new token j iff bit j of its tree-mask row is set */
#define RD_ATTN_DENSE 2  /* query i of row b sees key slot j iff dense_mask[b, i, j] != 0 (any j) */

#define RD_TOPK_MAX_KEPT 64 /* capacity of one row's kept list in rd_vocab_topk */
#define RD_MAX_BEAM_WIDTH 64
#define RD_MAX_BEAM_LENGTH 8

RD_API const char* rd_strerror(int code);
RD_API int rd_last_cuda_error(void); /* cudaError_t of the last rejected launch on this thread */
RD_API int rd_abi_version(void);

/* ---------------------------------------------------------------------------------------------
 * Prefix-tree pack.  Replaces tree_attention._dedup_prefix/_get_unpacker/_pack_beams and the
 * tree block of _get_causal_mask_of_packed_beams (recurrent_drafting/tree_attention.py:14-38,
 * 125-188, 41-122, 191-250) and the position arithmetic of _verify_candidates
 * (recurrent_drafting/recurrent_drafting.py:449-458).
 *
 * Rows are packed back to back ("flat" layout, no per-row padding): row b owns flat entries
 * [row_start[b], row_start[b+1]); row_start[B] is the total and can be passed as m_dev to the
 * other entry points.  Outputs (all required unless noted):
 *   prefix_tree [B,W,Lb] (optional), unpacker [B,W,Lb], n_selected [B], row_start [B+1],
 *   flat_tokens [cap] token ids, flat_index [cap] flat beam index i*Lb+j of each packed token,
 *   tok_row [cap] batch row, tok_pos [cap] = kv_len[b] + flat_index % Lb (RoPE position),
 *   tok_slot [cap] = kv_begin[b] + kv_len[b] + p (cache slot of packed token p of row b),
 *   tree_mask [cap, mask_words] bit q of row t set iff token t attends packed token q of its row,
 *   base_len [B] (optional) copy of kv_len taken before anything else in the step changes it.
 * cap = B*W*Lb.  kv_begin / kv_len may be NULL (treated as zeros).  Limits: W <= 64, Lb <= 8,
 * mask_words >= ceil(W*Lb/32).
 */
RD_API int rd_tree_pack(const int64_t* beams, int B, int W, int Lb, const int32_t* kv_begin, const int32_t* kv_len,
                 int32_t* prefix_tree, int32_t* unpacker, int32_t* n_selected, int32_t* row_start,
                 int64_t* flat_tokens, int32_t* flat_index, int32_t* tok_row, int32_t* tok_pos, int32_t* tok_slot,
                 uint32_t* tree_mask, int mask_words, int32_t* base_len, void* stream);

/* The reference's padded (B,N) layout of the same pack, bit for bit, including the tail of short
 * rows, which the reference fills from the FOLLOWING rows' selections
 * (recurrent_drafting/tree_attention.py:95-120) and masks through the row's own unpacker
 * (:237-249), and the dense bool mask (B,N,S+N) of tree_attention.pack (:301-338) with the
 * causal+padding block of attention.causal_mask (recurrent_drafting/attention.py:12-55).
 * N = max_b n_selected[b] is passed by the host.  padding_mask [B,S] int64, nonzero = real token.
 * unpacker64 (optional) receives the unpacker widened to int64. */
RD_API int rd_tree_pack_reference_layout(int B, int W, int Lb, const int32_t* unpacker, const int32_t* n_selected,
                                  const int32_t* row_start, const int64_t* flat_tokens, const int32_t* flat_index,
                                  int N, const int64_t* padding_mask, int S, int64_t* packed_beams,
                                  int64_t* packed_token_indices, int64_t* position_offsets, uint8_t* causal_mask,
                                  int64_t* unpacker64, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Drafter beam search (recurrent_drafting/modeling_drafter.py:133-232).
 *
 * rd_drafter_prepare builds the input of the recurrent update for iteration k
 * (modeling_drafter.py:193-197): a[r, 0:H] = embed[beams[b,w,k]], a[r, H:2H] = state of the
 * parent beam (x[b*W+parent[b,w], H:2H]; zeros when k == 0), and, when k == 0, x[r, 0:H] = ctx[b]
 * (the constant context half of the LM-head input, :174).  r = b*W + w; a, x are [B*W, 2H].
 * additive != 0 serves drafters built with rnn = false, whose state update has no projections
 * (state = embedding + state, modeling_drafter.py:196): a[r, H:2H] then holds the new state itself
 * (embedding + parent state, rounded once to the model type) and the caller copies it into x[r, H:2H]. */
RD_API int rd_drafter_prepare(int dtype, const void* embed, const int64_t* beams, const int32_t* parent, const void* ctx,
                       void* a, void* x, int B, int W, int Lb, int H, int k, int additive, void* stream);

/* Per-row top-k warp + log-softmax of a (rows, V) logits matrix, sparse output.  Replaces
 * maintain_logits, warp_logits and log_softmax (modeling_drafter.py:63-99, 201-203) and, for the
 * verify logits, warp_logits + (logits/T).log_softmax (recurrent_drafting.py:460, :86).
 *
 * For every live row: z = logits (- row max when subtract_max); every z >= the top_k-th largest
 * is kept (ties kept), the rest is set to mask_value; s = z / temperature; log-softmax over
 * the whole row.  kept_val / kept_idx [rows, RD_TOPK_MAX_KEPT] receive the kept entries' log-probs
 * and vocabulary ids ordered by (value descending, id ascending), kept_cnt [rows] their number
 * (clamped to the capacity; ties beyond it are dropped from the list but still counted in the
 * normaliser), masked_logp [rows] the log-prob shared by every entry that is not kept.
 * logits_dtype: RD_F32 or RD_BF16.  ld = leading dimension in elements. */
RD_API int rd_vocab_topk(int logits_dtype, const void* logits, int64_t ld, int rows_max, const int32_t* rows_dev, int V,
                  int top_k, float mask_value, int subtract_max, float temperature, float* kept_val,
                  int32_t* kept_idx, int32_t* kept_cnt, float* masked_logp, void* stream);

/* Cross-beam top-W of iteration k and beam reorder (modeling_drafter.py:206-230).  Candidates
 * are the kept entries of the W rows of batch row b with score kept_val + score_in[b,w]
 * (k == 0: beam 0 scores 0, the others LOG_0, :170-172); the W best by (score descending, flat
 * index w*V+token ascending) become the new beams.  beams_in/out [B,W,Lb]: columns 0..k are
 * gathered from the parent, column k+1 is the new token.  anc_in/out [B,W,Lb-1]: row index
 * (within the batch row) that produced the log-probs of position j of every surviving beam.
 * Requires W <= RD_TOPK_MAX_KEPT candidates per row to be exact (see kept_cnt). */
/* rd_vocab_topk for logits produced by rd_gemm_bf16_tc_slicemax: the threshold comes from the slice
 * maxima and only the slices that can hold kept entries are read (about a tenth of the row), with the
 * same results as rd_vocab_topk, bit for bit.  V a multiple of 32, rows 16-byte aligned. */
RD_API int rd_vocab_topk_sliced(int logits_dtype, const void* logits, int64_t ld, int rows_max, const int32_t* rows_dev, int V,
                         int top_k, float mask_value, int subtract_max, float temperature, const float* slice_max,
                         int64_t slice_ld, float* kept_val, int32_t* kept_idx, int32_t* kept_cnt, float* masked_logp,
                         void* stream);

RD_API int rd_beam_select(int B, int W, int Lb, int k, int V, const float* kept_val, const int32_t* kept_idx,
                   const int32_t* kept_cnt, const float* score_in, float* score_out, const int64_t* beams_in,
                   int64_t* beams_out, const int32_t* anc_in, int32_t* anc_out, int32_t* parent_out, void* stream);

/* Dense (B,W,Lb-1,V) fp32 log-prob tensor of beam_search_candidates' second return value,
 * rebuilt from the sparse per-iteration lists (modeling_drafter.py:222-230).  kept_* and
 * masked_logp are arrays of Lb-1 device pointers passed from the host. */
RD_API int rd_drafter_dense_log_probs(int B, int W, int Lb, int V, const float* const* kept_val_host,
                               const int32_t* const* kept_idx_host, const int32_t* const* kept_cnt_host,
                               const float* const* masked_logp_host, const int32_t* anc, float* out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * GEMM C = epilogue(A * W^T): A [M,K] row-major (lda), W [N,K] row-major (ldw, an nn.Linear
 * weight), fp32 accumulation.  Replaces nn.Linear on the path (modeling_drafter.py:36-39,
 * 112-125; modeling_llama.py:84,141-143,172,272).  out_dtype may be RD_F32 with bf16 inputs
 * (LM head, modeling_llama.py:272).  bias [N] in `dtype`; R [M, ldr] in out_dtype.
 *
 * rd_gemm is the exact-fp32 / generic path (CUDA cores).  rd_gemm_bf16_tc is the tensor-core
 * path (tcgen05 + TMEM accumulators, operands staged by TMA); it needs bf16 operands, K a
 * multiple of 64, 16-byte aligned A, W and C/R rows; `tensor_maps` is a host pointer returned
 * by rd_gemm_plan_create for these exact (A, W) buffers. */
RD_API int rd_gemm(int dtype, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
            const void* bias, const void* R, int64_t ldr, int m_max, const int32_t* m_dev, int N, int K,
            int epilogue, void* stream);

/* Allocates (host memory only) and returns the two TMA descriptors of an (A, W) operand pair.
 * Free with rd_gemm_plan_destroy.  Returns NULL on failure. */
RD_API void* rd_gemm_plan_create(const void* A, int64_t lda, int m_max, const void* W, int64_t ldw, int N, int K);
RD_API void rd_gemm_plan_destroy(void* plan);
RD_API int rd_gemm_bf16_tc(const void* plan, int out_dtype, void* C, int64_t ldc, const void* bias, const void* R,
                    int64_t ldr, const int32_t* m_dev, int epilogue, int32_t* status, void* stream);

/* The QKV projection (modeling_llama.py:141-143) with apply_rotary_pos_emb (:104-110) and the cache
 * append (:157-159) done in its epilogue: `plan` holds (normed activations, packed [q;k;v] weight
 * of (nh + 2 nkv) * 128 rows); rotated Q rows go to q_out [m, nh*128], rotated K and plain V rows
 * to the caches [B, nkv, max_len, 128] at tok_slot of row tok_row, positions from tok_pos into the
 * fp32 cos/sin tables [n_pos, 128].  head_dim 128, bf16.  Same result, bit for bit, as
 * rd_gemm_bf16_tc followed by rd_rope_kv_write. */
RD_API int rd_gemm_bf16_tc_qkv_rope(const void* plan, const int32_t* m_dev, void* q_out, void* k_cache, void* v_cache,
                             const int32_t* tok_row, const int32_t* tok_pos, const int32_t* tok_slot,
                             const float* cos_table, const float* sin_table, int n_pos, int nh, int nkv, int hd,
                             int max_len, int32_t* status, void* stream);

/* LlamaRMSNorm (modeling_llama.py:21-34) folded into the two GEMMs around it, so that the norm between a residual
 * projection and the next projection needs no kernel of its own (bf16, tensor-core path).
 * rd_gemm_bf16_tc_res_norm (producer): C = A W^T + R as RD_EPI_RES; besides, C2[t, n] = bf16(C[t, n]) * gamma[n] and
 * ss_out[t * ss_ld + n / 128] = the sum over the 128 features of slice n / 128 of bf16(C[t, n])^2 (fp32, every slice
 * of every live token is written: nothing to zero, no atomics, the same bits from launch to launch).  N a multiple
 * of 128, ss_ld >= N / 128 and a multiple of 4 with a 16-byte aligned base for the consumers, 16-byte aligned rows.
 * rd_gemm_bf16_tc_swiglu_normed / rd_gemm_bf16_tc_qkv_rope_normed (consumers): as RD_EPI_SWIGLU /
 * rd_gemm_bf16_tc_qkv_rope on an A that is such a C2; the accumulator row of token t is multiplied by
 * 1 / sqrt(sum_{s < ss_slices} ss_in[t * ss_ld + s] / norm_dim + eps) first (slices added in ascending order).
 * Against the separate rd_rmsnorm the row is rounded once (x * gamma) instead of twice (x / rms, then * gamma) before
 * the projection, and scaled in fp32 afterwards: results agree within bf16 rounding, not bit for bit. */
RD_API int rd_gemm_bf16_tc_res_norm(const void* plan, void* C, int64_t ldc, const void* R, int64_t ldr, const int32_t* m_dev,
                             const void* gamma, void* C2, int64_t ldc2, float* ss_out, int64_t ss_ld, int32_t* status,
                             void* stream);
RD_API int rd_gemm_bf16_tc_swiglu_normed(const void* plan, void* C, int64_t ldc, const int32_t* m_dev, const float* ss_in,
                                  int64_t ss_ld, int ss_slices, int norm_dim, float eps, int32_t* status, void* stream);
RD_API int rd_gemm_bf16_tc_qkv_rope_normed(const void* plan, const int32_t* m_dev, void* q_out, void* k_cache, void* v_cache,
                                    const int32_t* tok_row, const int32_t* tok_pos, const int32_t* tok_slot,
                                    const float* cos_table, const float* sin_table, int n_pos, int nh, int nkv, int hd,
                                    int max_len, const float* ss_in, int64_t ss_ld, int ss_slices, int norm_dim, float eps,
                                    int32_t* status, void* stream);

/* The LM head of the greedy verify step with the arg-max over the vocabulary done in its epilogue
 * (modeling_llama.py:272 followed by recurrent_drafting.py:52): `plan` holds (final hidden states,
 * lm_head weight [V, H]); the fp32 logits are never written.  Every 32 consecutive vocabulary ids of a
 * token are reduced to (largest logit, first id holding it) in the GEMM epilogue and a second, small
 * kernel merges the V/32 partial results per token; equal logits resolve to the smaller id, as the
 * separate rd_argmax_rows does, and the logits compared are the same fp32 accumulators it would read.
 * `workspace` (device, 16-byte aligned) holds the partial results; its size comes from
 * rd_gemm_argmax_workspace_bytes(m_max of the plan, V); RD_ERR_CAPACITY if it is too small. */
RD_API int64_t rd_gemm_argmax_workspace_bytes(int m_max, int N);
RD_API int rd_gemm_bf16_tc_argmax(const void* plan, const int32_t* m_dev, void* workspace, int64_t workspace_bytes,
                           int32_t* out32, int64_t* out64, int32_t* status, void* stream);

/* rd_gemm_bf16_tc with RD_EPI_NONE that also writes, for every token and every slice of 32 consecutive
 * output features, the largest value of the slice as stored in C: slice_max[s * slice_ld + token],
 * slice_ld >= m_max.  Feeds rd_vocab_topk_sliced (the drafter's vocabulary head, modeling_drafter.py:
 * 127-131, and the LM head of the sampling verify step).  N must be a multiple of 32, C rows 16-byte
 * aligned. */
RD_API int rd_gemm_bf16_tc_slicemax(const void* plan, int out_dtype, void* C, int64_t ldc, const int32_t* m_dev,
                             float* slice_max, int64_t slice_ld, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Llama verify forward pieces (recurrent_drafting/modeling_llama.py). */

/* out[t,:] = table[ids[t],:]  (embed_tokens, modeling_llama.py:226). */
RD_API int rd_embed_gather(int dtype, const void* table, const int64_t* ids, void* out, int m_max, const int32_t* m_dev,
                    int H, void* stream);

/* y = weight * (x * rsqrt(mean(x^2) + eps)) computed in fp32 (LlamaRMSNorm, modeling_llama.py:21-32). */
RD_API int rd_rmsnorm(int dtype, const void* x, const void* weight, void* y, int m_max, const int32_t* m_dev, int H,
               float eps, void* stream);

/* Splits qkv [M, (nh+2*nkv)*hd], applies NeoX rotary embedding at tok_pos to q and k
 * (apply_rotary_pos_emb, modeling_llama.py:87-110; cos/sin [n_pos, hd] fp32 tables), writes q to
 * q_out [M, nh*hd] and k, v straight into the cache at (tok_row, head, tok_slot)
 * (View.cat, recurrent_drafting/kv_cache.py:24-31).  k_cache / v_cache: [B, nkv, max_len, hd]. */
RD_API int rd_rope_kv_write(int dtype, const void* qkv, void* q_out, void* k_cache, void* v_cache, const int32_t* tok_row,
                     const int32_t* tok_pos, const int32_t* tok_slot, const float* cos_table, const float* sin_table,
                     int n_pos, int m_max, const int32_t* m_dev, int nh, int nkv, int hd, int max_len, void* stream);

/* Attention of the new tokens of every batch row over the row's cached prefix and over the new
 * tokens themselves (scaled_dot_product_attention with the mask of tree_attention.pack or of
 * attention.causal_mask; modeling_llama.py:157-169).  Row b's queries are flat rows
 * [row_start[b], row_start[b+1]); its keys are cache slots kv_begin[b] .. kv_begin[b]+base_len[b]
 * (all visible) followed by the n_new = row_start[b+1]-row_start[b] new tokens' slots, visible
 * per `mode`.  out [M, nh*hd].  max_new = upper bound of n_new used to size the grid; max_kv = upper
 * bound of base_len[b] + n_new[b] used to size shared memory (both known to the host without a
 * read-back: they only bound, the exact values are read on the device).  Mode RD_ATTN_DENSE takes
 * the reference's bool mask (B, q, kv) as bytes: element (b,i,j) at dense_mask[b*dense_ld_b +
 * i*dense_ld_q + j], j counted from kv_begin[b]; it covers cached and new keys alike. */
RD_API int rd_attention(int dtype, const void* q, const void* k_cache, const void* v_cache, void* out,
                 const int32_t* row_start, const int32_t* kv_begin, const int32_t* base_len, int B, int nh, int nkv,
                 int hd, int max_len, int max_new, int max_kv, int mode, const uint32_t* tree_mask, int mask_words,
                 const uint8_t* dense_mask, int64_t dense_ld_q, int64_t dense_ld_b, void* stream);

/* The same attention for bf16 and head_dim 128 on the tcgen05 tensor cores (S = Q K^T and O = P V
 * as tcgen05.mma with TMEM accumulators, K/V tiles staged by TMA).  Modes RD_ATTN_CAUSAL and
 * RD_ATTN_TREE.  `plan` is a host pointer from rd_attention_plan_create, which encodes the TMA
 * descriptors of these exact buffers: q [m_max, nh*128], k_cache / v_cache [B, nkv, max_len, 128]
 * (host memory only; free with rd_attention_plan_destroy; NULL on failure).  `status` (optional,
 * device int32) receives a non-zero code if a bounded device-side wait gave up. */
RD_API void* rd_attention_plan_create(const void* q, int m_max, const void* k_cache, const void* v_cache, int B, int nh,
                                      int nkv, int hd, int max_len);
RD_API void rd_attention_plan_destroy(void* plan);
RD_API int rd_attention_tc(const void* plan, void* out, const int32_t* row_start, const int32_t* kv_begin,
                           const int32_t* base_len, int max_new, int mode, const uint32_t* tree_mask, int mask_words,
                           int32_t* status, void* stream);

/* rd_attention_tc with the key range of every (row, head) cut into n_split shares (1..RD_ATTN_MAX_SPLIT), one CTA
 * each, merged by a second kernel: for launches with fewer (row, head) pairs than the GPU has SMs and long caches
 * (batch 1-4).  workspace: rd_attention_split_workspace_bytes(m_max, nh, n_split) bytes of device memory, 16-byte
 * aligned, holding the shares' unnormalised fp32 outputs, running maxima and sums. */
#define RD_ATTN_MAX_SPLIT 16
RD_API int64_t rd_attention_split_workspace_bytes(int m_max, int nh, int n_split);
RD_API int rd_attention_tc_split(const void* plan, void* out, const int32_t* row_start, const int32_t* kv_begin,
                          const int32_t* base_len, int max_new, int mode, const uint32_t* tree_mask, int mask_words,
                          int n_split, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/* argmax_v logits[t, v], first maximal index (torch.argmax, recurrent_drafting.py:52), written
 * to out32 [M] and/or out64 [M] (either may be NULL). */
RD_API int rd_argmax_rows(const float* logits, int64_t ld, int m_max, const int32_t* m_dev, int V, int32_t* out32,
                   int64_t* out64, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Acceptance + commit, one launch after the verify forward.  Replaces
 * _greedy_choose_from_candidates / _choose_from_candidates, _update_kv_cache_and_input_ids and
 * _[greedy_]prepare_next_input (recurrent_drafting/recurrent_drafting.py:468-556, 114-232,
 * 235-343) and Cache.unpack (recurrent_drafting/kv_cache.py:58-98), which becomes unnecessary:
 * the accepted path's K/V rows are moved from their packed slots directly.
 *
 * The cache keeps every row where the prompt put it: row b occupies slots
 * [kv_begin[b], kv_begin[b]+kv_len[b]) and only grows; the verify forward wrote the packed tree
 * tokens' K/V at kv_begin[b]+base_len[b]+p.  The commit moves packed slot
 * unpacker[b,seq_b,j] to position j for j = 0..A_b and sets kv_len[b] = base_len[b]+A_b+1.
 * The reference's right-aligned slot numbering is recovered in index space by
 * rd_commit_reference_slots.
 *
 * Greedy: llm_tokens [M] holds argmax of the verify logits per flat token.
 * Outputs: n_accepted [B], seq_in_beam [B], next_tokens [B] int64, next_ctx [B,H] (hidden state
 * of the last accepted token), token_buf [B, max_len] receives the accepted tokens at their
 * cache slots. cache: [NL, 2, B, nkv, max_len, hd].  NL = 0 decides only (cache, kv_begin,
 * base_len, kv_len and token_buf may then be NULL); H = 0 skips next_ctx. */
RD_API int rd_accept_commit_greedy(int dtype, const int64_t* beams, int B, int W, int Lb, const int32_t* unpacker,
                            const int32_t* row_start, const int32_t* llm_tokens, const void* hidden, int H,
                            void* cache, int NL, int nkv, int max_len, int hd, const int32_t* kv_begin,
                            const int32_t* base_len, int32_t* kv_len, int64_t* token_buf, int32_t* n_accepted,
                            int32_t* seq_in_beam, int64_t* next_tokens, void* next_ctx, void* stream);

/* Slot indices of the commit in the reference's right-aligned cache layout
 * (recurrent_drafting.py:179-209, kv_cache.py:90-95).  out [B, Lb, 3] int64: for j <= A_b the
 * source slot after the verify forward (S + unpacker[b,seq,j]), after Cache.unpack
 * (S + seq*Lb + j) and the final slot after realignment (S2 - (A_b+1) + j); -1 for j > A_b.
 * S = the reference's padded length before the step, S2 = max_b (new row length). */
RD_API int rd_commit_reference_slots(int B, int W, int Lb, const int32_t* unpacker, const int32_t* n_accepted,
                              const int32_t* seq_in_beam, int S, int S2, int64_t* out, void* stream);

/* Speculative-sampling variant (recurrent_drafting.py:499-556, 271-343).  p_* are the sparse
 * log-prob lists of the verify logits per flat token (rd_vocab_topk with the sampling temperature);
 * q_* the drafter's lists per iteration (host arrays of Lb-1 device pointers) with the ancestor
 * table anc [B,W,Lb-1]; uniforms [B,W,Lb-1] drive acceptance (torch.rand at :545) and
 * uniforms_next [B] the categorical draw of the next token, taken by inverse CDF in ascending
 * token order over the unnormalised residual relu(P-Q) (or P's last distribution when the whole
 * beam was accepted).  probs_dense (optional) [B,V] receives that unnormalised distribution. */
RD_API int rd_accept_commit_sample(int dtype, const int64_t* beams, int B, int W, int Lb, int V, const int32_t* unpacker,
                            const int32_t* row_start, const float* p_val, const int32_t* p_idx,
                            const int32_t* p_cnt, const float* p_masked, const float* const* q_val_host,
                            const int32_t* const* q_idx_host, const int32_t* const* q_cnt_host,
                            const float* const* q_masked_host, const int32_t* anc, const float* uniforms,
                            const float* uniforms_next, const void* hidden, int H, void* cache, int NL, int nkv,
                            int max_len, int hd, const int32_t* kv_begin, const int32_t* base_len, int32_t* kv_len,
                            int64_t* token_buf, int32_t* n_accepted, int32_t* seq_in_beam, int64_t* next_tokens,
                            void* next_ctx, float* probs_dense, void* stream);

/* Inverse-CDF draw, in ascending token order, from the sparse distribution exp(kept_val) of every
 * row (entries outside the list have probability exp(masked_logp), which must underflow to 0).
 * With rd_vocab_topk on the last prompt token's logits this is the sampled first token of
 * _comprehend_prompt (recurrent_drafting.py:422-430).  uniforms [rows]. */
RD_API int rd_sample_from_sparse(const float* kept_val, const int32_t* kept_idx, const int32_t* kept_cnt, int rows,
                          const float* uniforms, int64_t* out, void* stream);

/* The (B, S'+1) left-padded token matrix the decode loop yields
 * (recurrent_drafting.py:212-226, :681): row b holds pad ids, then its kv_len[b] tokens from
 * token_buf (starting at kv_begin[b]), then next_tokens[b], right-aligned.  S' = max_b kv_len[b]
 * is passed by the host (out_len = S'+1). */
RD_API int rd_emit_tokens(const int64_t* token_buf, int max_len, const int32_t* kv_begin, const int32_t* kv_len,
                   const int64_t* next_tokens, int64_t pad_id, int B, int out_len, int64_t* out, void* stream);

/* Cache.unpack of the reference API (recurrent_drafting/kv_cache.py:58-98) for callers that use
 * the reference's per-beam cache layout: cache[..., S+f, :] = old cache[..., S+unpacker[b,f], :]
 * for f in [0, n_flat).  scratch must hold NL*2*B*nkv*n_flat*hd elements. */
RD_API int rd_cache_unpack(int dtype, void* cache, int NL, int B, int nkv, int max_len, int hd, int S,
                    const int64_t* unpacker, int n_flat, void* scratch, void* stream);

/* Same result as rd_cache_unpack, for callers that can give the library no scratch buffer.
 * This entry point has no counterpart in the reference.
 *
 * Who needs it: a host that took all of the device's memory into its own arena at start-up (a
 * later cudaMalloc from a plug-in simply fails there), or a latency-critical loop whose rules
 * forbid device allocation after initialisation because cudaMalloc/cudaFree stall the device.
 * Such a caller passes only the cache and the index; the staging copy of the gathered rows lives
 * in a fixed array inside the library, RD_STATIC_SCRATCH_BYTES large, which every GPU that loads
 * the library keeps until the process ends.
 *
 * Limits and rules:
 *   - NL*2*B*nkv*n_flat*hd*sizeof(element) must not exceed RD_STATIC_SCRATCH_BYTES, otherwise the
 *     call returns RD_ERR_CAPACITY and does nothing;
 *   - the first call on each device looks the array's device address up (with that device
 *     current) and remembers it; make that first call during set-up, before any stream capture;
 *   - nothing in the array has to start at zero (the part in use is overwritten before it is
 *     read), so it is never cleared and keeps the previous call's bytes;
 *   - every call uses the same array: two calls whose kernels can run at the same time on one
 *     GPU (different streams) race and corrupt each other - order them on one stream;
 *   - no cudaMalloc, cudaFree or other allocating routine is called. */
#define RD_STATIC_SCRATCH_BYTES (16u << 20)
RD_API int rd_cache_unpack_static(int dtype, void* cache, int NL, int B, int nkv, int max_len, int hd, int S,
                                  const int64_t* unpacker, int n_flat, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* REDRAFTER_B200_H_ */
