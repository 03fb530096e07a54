"""Greedy one-token-per-step decoding over the same model, cache and kernels
(recurrent_drafting/autoregressive.py:13-53).  The comparator of the speculative loop: with greedy
search both must produce the same tokens.

As in the reference, positions are the tokens' column indices in the left-padded input (the
reference passes arange(past, cur) without subtracting the padding, autoregressive.py:37-39)."""
from typing import Generator

import torch

from . import _lib, kv_cache
from .recurrent_drafting import RecurrentDrafting, SpecialTokens, _count_left_paddings


@torch.inference_mode()
def generate(model: RecurrentDrafting, input_ids: torch.Tensor, max_length: int,
             special_tokens: SpecialTokens) -> Generator[torch.Tensor, None, None]:
    llm = model.llm
    B, Lp = input_ids.shape
    dev = input_ids.device
    cache = kv_cache.Cache(B, max_length, llm.n_layers, model.llm_n_kv_heads(), llm.head_dim, llm.dtype, dev)
    i32 = dict(dtype=torch.int32, device=dev)
    pads = _count_left_paddings(input_ids, special_tokens.pad)
    n_new = Lp - pads
    cols = torch.arange(Lp, device=dev)[None, :].expand(B, Lp)
    live = cols >= pads[:, None]
    tok_ids = input_ids[live].contiguous()
    M = tok_ids.numel()
    tok_row = torch.arange(B, device=dev)[:, None].expand(B, Lp)[live].to(torch.int32)
    tok_slot = cols[live].to(torch.int32)
    row_start = torch.zeros(B + 1, **i32)
    row_start[1:] = torch.cumsum(n_new, 0).to(torch.int32)
    kv_begin = pads.to(torch.int32)
    kv_len = torch.zeros(B, **i32)
    n_pos = max_length + 1
    ws = llm.workspace(M, B)
    hidden = llm.backbone(ws, cache._cache, M, None, tok_ids, tok_row, tok_slot, tok_slot, row_start, kv_begin, kv_len, B,
                          Lp, Lp, _lib.ATTN_CAUSAL, n_pos=n_pos)
    last_hidden = hidden[(row_start[1:] - 1).long()].contiguous()
    kv_len = n_new.to(torch.int32)
    tokens = torch.full((B, max_length), special_tokens.pad, dtype=torch.int64, device=dev)
    tokens[:, :Lp] = input_ids
    nxt = torch.empty(B, dtype=torch.int64, device=dev)
    one_row = torch.arange(B, **i32)
    step_rows = torch.arange(B + 1, **i32)
    ws1 = llm.workspace(B, B)
    length = Lp
    V = llm.config.vocab_size
    while length < max_length:
        logits = llm.lm_logits(last_hidden, ws1["logits"])
        _lib.call("rd_argmax_rows", _lib.ptr(logits), logits.stride(0), B, None, V, None, _lib.ptr(nxt), _lib.stream())
        tokens[:, length] = nxt
        length += 1
        out = tokens[:, :length].clone()
        yield out
        if special_tokens.eos is not None and bool(((out[:, Lp:] == special_tokens.eos).sum(dim=-1) > 0).sum() == B):
            break
        if length >= max_length:
            break
        slot = (kv_begin + kv_len).contiguous()
        last_hidden = llm.backbone(ws1, cache._cache, B, None, nxt, one_row, slot, slot, step_rows, kv_begin, kv_len, B, 1,
                                   length, _lib.ATTN_CAUSAL, n_pos=n_pos)
        kv_len = kv_len + 1
