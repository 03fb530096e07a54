"""Oracle (numpy fp32) for the recurrent drafter head and its beam search.
Test infrastructure only.

Restates recurrent_drafting/modeling_drafter.py of the reference.  Weights are
passed as a dict with the reference's state-dict names:
  rnn_w.weight (H,H)  rnn_u.weight (H,H)  rnn_u.bias (H,)
  [input_proj.weight (E,2H)  input_proj.bias (E,)]   only when E != 2H
  lm_head.{r}.linear.weight (E,E)  lm_head.{r}.linear.bias (E,)   r < R
  lm_head.{R}.weight (V,E)
"""

from typing import Dict, Tuple

import numpy as np

LOG_0 = np.float32(-50000.0)  # modeling_drafter.py:13
LOG_1 = np.float32(0.0)


def silu(x: np.ndarray) -> np.ndarray:
    return (x / (1.0 + np.exp(-x))).astype(np.float32)


def topk_desc(values: np.ndarray, k: int) -> Tuple[np.ndarray, np.ndarray]:
    """Top-k along the last axis: values descending, ties by ascending index.

    torch.topk leaves the order of exactly tied values undefined; this rule is
    the one the CUDA kernels implement and is only distinguishable from the
    reference's when inputs hold exact ties.
    """
    order = np.argsort(-values, axis=-1, kind="stable")[..., :k]
    return np.take_along_axis(values, order, axis=-1), order


def maintain_logits(logits: np.ndarray) -> np.ndarray:
    """Subtract the row maximum.  Reference: modeling_drafter.py:63-77."""
    return logits - logits.max(axis=-1, keepdims=True)


def warp_logits(logits: np.ndarray, top_k: int = 50, mask_value: float = float(LOG_0)) -> np.ndarray:
    """Keep every value >= the top_k-th largest of its row (ties kept), set the
    rest to mask_value.  Reference: modeling_drafter.py:80-99."""
    k = min(top_k, logits.shape[-1])
    kth = -np.partition(-logits, k - 1, axis=-1)[..., k - 1 : k]
    return np.where(logits < kth, np.float32(mask_value), logits).astype(logits.dtype)


def log_softmax(x: np.ndarray) -> np.ndarray:
    m = x.max(axis=-1, keepdims=True)
    z = x - m
    return (z - np.log(np.exp(z).sum(axis=-1, keepdims=True))).astype(np.float32)


def compute_logits(w: Dict[str, np.ndarray], x: np.ndarray, num_draft_layers: int) -> np.ndarray:
    """input_proj (optional) -> R residual blocks x + silu(Ax+b) -> vocab head
    -> maintain_logits -> warp_logits.  Reference: modeling_drafter.py:33-39,127-131."""
    if "input_proj.weight" in w:
        x = x @ w["input_proj.weight"].T + w["input_proj.bias"]
    for r in range(num_draft_layers):
        x = x + silu(x @ w[f"lm_head.{r}.linear.weight"].T + w[f"lm_head.{r}.linear.bias"])
    logits = x @ w[f"lm_head.{num_draft_layers}.weight"].T
    return warp_logits(maintain_logits(logits.astype(np.float32)))


def beam_search_candidates(
    w: Dict[str, np.ndarray],
    num_draft_layers: int,
    prompt_state: np.ndarray,
    init_token: np.ndarray,
    embeddings: np.ndarray,
    beam_width: int,
    beam_length: int,
    rnn: bool = True,
) -> Tuple[np.ndarray, np.ndarray]:
    """Returns beams (B,W,Lb) int64 and log_probs (B,W,Lb-1,V) fp32.

    Reference: modeling_drafter.py:133-232.  Beam 0 starts with score 0, every
    other beam with LOG_0, so the first iteration grows beam 0 only (:170-172).
    """
    B, H = prompt_state.shape
    V = embeddings.shape[0]
    W, Lb = beam_width, beam_length
    score = np.tile(np.array([LOG_1] + [LOG_0] * (W - 1), dtype=np.float32), (B, 1))
    context = np.repeat(prompt_state[:, None, :], W, axis=1).astype(np.float32)
    beams = np.repeat(init_token[:, None, None], W, axis=1).astype(np.int64)
    state = np.zeros((B, W, H), dtype=np.float32)
    hist = np.zeros((B, W, 0, V), dtype=np.float32)
    rows = np.arange(B)[:, None]
    for _ in range(Lb - 1):
        emb = embeddings[beams[..., -1]]
        if rnn:
            state = silu(emb @ w["rnn_w.weight"].T + state @ w["rnn_u.weight"].T + w["rnn_u.bias"])
        else:
            state = emb + state
        logp = log_softmax(compute_logits(w, np.concatenate([context, state], axis=-1), num_draft_layers))
        cand = (logp + score[:, :, None]).reshape(B, W * V)
        score, flat = topk_desc(cand, W)
        tok, parent = flat % V, flat // V
        beams = np.concatenate([beams[rows, parent], tok[:, :, None]], axis=-1)
        state = state[rows, parent]
        hist = np.concatenate([hist[rows, parent], logp[rows, parent][:, :, None, :]], axis=2)
    return beams, hist
