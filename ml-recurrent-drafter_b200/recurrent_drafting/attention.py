"""Dense attention-mask helpers of the reference API (recurrent_drafting/attention.py).

The decode loop of this package never materialises these masks: its attention kernel derives
visibility from per-row lengths and the prefix-tree bitmask.  The helpers exist for callers that
drive LlamaForCausalLM.forward with an explicit (batch, query, key) mask, as the reference does.
"""
import torch


def causal_mask(padding_mask: torch.Tensor, query_len: int, device: torch.device) -> torch.Tensor:
    """(batch, query_len, kv_len) bool: key j visible to the query at absolute position i iff
    j <= i and key j is not padding.  Same result as attention.py:12-55 without building the
    square (kv_len, kv_len) matrix."""
    assert padding_mask.dtype in (torch.int32, torch.int64, torch.bool)
    assert query_len > 0
    kv_len = padding_mask.shape[1]
    q_pos = torch.arange(kv_len - query_len, kv_len, device=device)
    k_pos = torch.arange(kv_len, device=device)
    lower = k_pos[None, :] <= q_pos[:, None]
    return lower[None, :, :] & padding_mask.to(device).ne(0)[:, None, :]


def set_sdpa_fully_masked_rows(causal_mask: torch.Tensor) -> torch.Tensor:
    """Rows with no visible key become all-visible (attention.py:58-72)."""
    assert causal_mask.dtype in (torch.int32, torch.int64, torch.bool)
    empty = causal_mask.ne(0).sum(dim=-1, keepdim=True).eq(0)
    return causal_mask.masked_fill(empty, True)


def bias(causal_mask: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """0 where visible, the dtype's most negative finite value elsewhere (attention.py:75-88)."""
    out = torch.zeros(causal_mask.shape, dtype=dtype, device=causal_mask.device)
    return out.masked_fill_(causal_mask.logical_not(), torch.finfo(dtype).min)


ATTN_MAX_SPLIT = 16


def key_range_shares(batch: int, n_heads: int, max_new: int, max_kv: int, n_sm: int = 148) -> int:
    """How many CTAs should share the key range of one (row, head) in the tcgen05 attention
    (rd_attention_tc_split).  One, unless the launch has fewer (row, head, query tile) chains than
    the GPU can hold at two CTAs per SM: then enough shares to fill it, each with at least four key
    tiles of 64."""
    chains = batch * n_heads * ((max_new + 127) // 128)
    slots = 2 * n_sm
    if chains >= slots // 2:
        return 1
    by_fill = slots // chains
    by_length = max(1, ((max_kv + 63) // 64) // 4)
    return max(1, min(ATTN_MAX_SPLIT, by_fill, by_length))
