"""Oracle (numpy) for candidate acceptance and the KV-cache / input_ids commit.
Test infrastructure only.

Restates the module-level helpers of recurrent_drafting/recurrent_drafting.py.
Random numbers are always injected by the caller (uniforms), never drawn here.
"""

from typing import Dict, Tuple

import numpy as np

from . import kv_cache


def count_left_paddings(tokens: np.ndarray, pad_token_id: int) -> np.ndarray:
    """Reference: recurrent_drafting.py:387-388."""
    return np.cumprod(tokens == pad_token_id, axis=-1).sum(axis=-1).astype(np.int64)


def _first_max(n: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """max over beams with the FIRST maximal index (torch.max on CPU and CUDA)."""
    idx = np.argmax(n, axis=-1)
    return np.take_along_axis(n, idx[:, None], axis=-1)[:, 0].astype(np.int64), idx.astype(np.int64)


def greedy_choose_from_candidates(beams_by_drafter: np.ndarray, beams_by_llm: np.ndarray):
    """n[b,i] = length of the run beams_by_drafter[b,i,1+k] == beams_by_llm[b,i,k]
    from k = 0; returns (max_i n, first argmax).  Reference: recurrent_drafting.py:468-496;
    golden: recurrent_drafting_test.py:34-69."""
    cmp = beams_by_drafter[:, :, 1:] == beams_by_llm[:, :, :-1]
    n = np.cumprod(cmp, axis=-1).sum(axis=-1)
    return _first_max(n)


def choose_from_candidates(beams, log_probs_by_llm, log_probs_by_drafter, uniforms):
    """Speculative-sampling acceptance: drafted token v at (b,i,k) is accepted iff
    uniforms[b,i,k] < exp(logP[b,i,k,v] - logQ[b,i,k,v]); n[b,i] is the accepted
    prefix length.  Reference: recurrent_drafting.py:499-556 (uniforms stand for
    torch.rand at :545)."""
    tok = beams[..., 1:, None]
    by_q = np.take_along_axis(log_probs_by_drafter, tok, axis=-1)[..., 0]
    by_p = np.take_along_axis(log_probs_by_llm[:, :, :-1, :], tok, axis=-1)[..., 0]
    cmp = uniforms.astype(np.float32) < np.exp((by_p - by_q).astype(np.float32))
    n = np.cumprod(cmp, axis=-1).sum(axis=-1)
    return _first_max(n)


def greedy_prepare_next_input(beams_by_llm, last_hidden_state, seq_in_beam, n_tokens_in_seq):
    """Reference: recurrent_drafting.py:235-268."""
    r = np.arange(beams_by_llm.shape[0])
    return last_hidden_state[r, seq_in_beam, n_tokens_in_seq], beams_by_llm[r, seq_in_beam, n_tokens_in_seq]


def residual_probs(log_probs_by_drafter, log_probs_by_llm, seq_in_beam, n_tokens_in_seq) -> np.ndarray:
    """Unnormalised (B,V) distribution the next token is drawn from: the LLM's
    last distribution if the whole beam was accepted, else relu(P - Q) at the
    first rejected position.  Reference: recurrent_drafting.py:271-339."""
    B = log_probs_by_llm.shape[0]
    L1 = log_probs_by_drafter.shape[-2]
    r = np.arange(B)
    last_p = np.exp(log_probs_by_llm[r, seq_in_beam, -1, :])
    idx = n_tokens_in_seq - (n_tokens_in_seq == L1)
    p = np.exp(log_probs_by_llm[r, seq_in_beam, idx, :])
    q = np.exp(log_probs_by_drafter[r, seq_in_beam, idx, :])
    res = np.maximum(p - q, 0.0)
    return np.where((n_tokens_in_seq == L1)[:, None], last_p, res).astype(np.float32)


def sample_inverse_cdf(probs: np.ndarray, u: np.ndarray) -> np.ndarray:
    """Categorical draw from unnormalised probs (B,V) with injected uniforms u (B,):
    the smallest v with cumsum(probs)[v] > u * sum(probs), among v with probs > 0.

    The reference draws with torch.distributions.Categorical (recurrent_drafting.py:340),
    whose stream differs between devices; only the distribution is shared.
    """
    out = np.zeros(probs.shape[0], dtype=np.int64)
    for b in range(probs.shape[0]):
        nz = np.nonzero(probs[b] > 0)[0]
        c = np.cumsum(probs[b, nz].astype(np.float32), dtype=np.float32)
        t = np.float32(u[b]) * c[-1]
        k = int(np.searchsorted(c, t, side="right"))
        out[b] = nz[min(k, nz.size - 1)]
    return out


def update_kv_cache_and_input_ids(input_ids, n_tokens_in_seq, seq_in_beam, beams, cache: kv_cache.Cache, pad_token_id):
    """Append the accepted tokens and their K/V, then re-right-align every row.

    On entry the cache holds, after the S processed slots, the per-beam
    (unpacked) K/V of the W*Lb candidates.  Reference: recurrent_drafting.py:114-232.
    """
    B, W, L = beams.shape
    S = input_ids.shape[1]
    pads = count_left_paddings(input_ids, pad_token_id)
    n1 = n_tokens_in_seq + 1
    seq_len = S - pads + n1
    S2 = int(seq_len.max())
    new_pads = S2 - seq_len
    c = cache._cache
    snap = c.copy()
    for b in range(B):
        src0 = S + int(seq_in_beam[b]) * L
        # :179-198 move the chosen beam's L rows to [S, S+L)
        c[:, :, b, :, S : S + L, :] = snap[:, :, b, :, src0 : src0 + L, :]
    snap = c.copy()
    for b in range(B):
        # :200-209 shift the row so that it ends at S2
        c[:, :, b, :, new_pads[b] : S2, :] = snap[:, :, b, :, pads[b] : S + n1[b], :]
    out = np.full((B, S2), pad_token_id, dtype=np.int64)
    for b in range(B):
        keep = S - pads[b]
        out[b, new_pads[b] : new_pads[b] + keep] = input_ids[b, pads[b] :]
        out[b, new_pads[b] + keep :] = beams[b, seq_in_beam[b], : n1[b]]
    for k, v in cache.sliced:
        k.length = v.length = S2
    return out


def commit_plan(input_ids, n_tokens_in_seq, seq_in_beam, unpacker, pad_token_id) -> Dict[str, np.ndarray]:
    """Reference-layout slot indices of the commit, in index space.

    For row b and j in [0, A_b]: the K/V of accepted token j is produced by the
    verify forward at packed slot S + unpacker[b,seq_b,j], sits at
    S + seq_b*Lb + j after Cache.unpack (kv_cache.py:90-95), is appended at S + j
    (recurrent_drafting.py:179-198) and ends at S' - (A_b+1) + j after the
    realignment (:200-209).  Entries with j > A_b are -1.
    """
    B, W, L = unpacker.shape
    S = input_ids.shape[1]
    pads = count_left_paddings(input_ids, pad_token_id)
    n1 = n_tokens_in_seq + 1
    seq_len = S - pads + n1
    S2 = int(seq_len.max())
    j = np.arange(L)[None, :]
    live = j < n1[:, None]
    r = np.arange(B)
    packed = S + unpacker[r, seq_in_beam, :]
    unpacked = S + seq_in_beam[:, None] * L + j
    final = S2 - n1[:, None] + j
    neg = -np.ones((B, L), dtype=np.int64)
    return {
        "new_length": np.int64(S2),
        "new_left_pads": (S2 - seq_len).astype(np.int64),
        "src_packed_slot": np.where(live, packed, neg),
        "src_unpacked_slot": np.where(live, unpacked, neg),
        "dst_slot": np.where(live, final, neg),
    }
