"""Oracle (numpy fp32) of the Llama-architecture base model with the reference's
pre-allocated KV cache.  Test infrastructure only.

Restates recurrent_drafting/modeling_llama.py.  `w` is a dict keyed by the
HF state-dict names (model.embed_tokens.weight, model.layers.N.self_attn.q_proj.weight,
..., model.norm.weight, lm_head.weight); `cfg` is a dict with hidden_size,
num_attention_heads, num_key_value_heads, num_hidden_layers, intermediate_size,
vocab_size, rms_norm_eps, rope_theta.
"""

from typing import Dict, Tuple

import numpy as np

F32_MIN = np.finfo(np.float32).min


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """Reference: modeling_llama.py:21-32."""
    x = x.astype(np.float32)
    var = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
    return (weight * (x * (1.0 / np.sqrt(var + np.float32(eps))))).astype(np.float32)


def rope_tables(head_dim: int, n_pos: int, base: float) -> Tuple[np.ndarray, np.ndarray]:
    """cos/sin tables (n_pos, head_dim), both halves holding the same angles.
    Reference: modeling_llama.py:35-64."""
    inv = (1.0 / (np.float32(base) ** (np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim)))).astype(np.float32)
    t = np.arange(n_pos, dtype=np.float32)
    fr = np.outer(t, inv).astype(np.float32)
    emb = np.concatenate([fr, fr], axis=-1)
    return np.cos(emb).astype(np.float32), np.sin(emb).astype(np.float32)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, position_ids: np.ndarray) -> np.ndarray:
    """x (B,h,q,hd); NeoX rotate-half with per-token positions.
    Reference: modeling_llama.py:87-110."""
    c = cos[position_ids][:, None]
    s = sin[position_ids][:, None]
    half = x.shape[-1] // 2
    rot = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    return (x * c + rot * s).astype(np.float32)


def silu(x: np.ndarray) -> np.ndarray:
    return (x / (1.0 + np.exp(-x))).astype(np.float32)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, mask: np.ndarray) -> np.ndarray:
    """softmax(q k^T / sqrt(hd) + bias) v with bias = 0 / finfo.min from the bool
    mask (B,q,kv).  Reference: modeling_llama.py:164-169, attention.py:75-88."""
    hd = q.shape[-1]
    s = np.einsum("bhqd,bhkd->bhqk", q, k).astype(np.float32) / np.float32(np.sqrt(hd))
    s = s + np.where(mask[:, None], np.float32(0), F32_MIN)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhqk,bhkd->bhqd", p, v).astype(np.float32)


def forward(
    w: Dict[str, np.ndarray],
    cfg: Dict,
    input_ids: np.ndarray,
    attention_mask: np.ndarray,
    position_ids: np.ndarray,
    past_key_values,
) -> Tuple[np.ndarray, np.ndarray]:
    """Returns (logits fp32 (B,q,V), hidden_states (B,q,H) after the final norm).

    K/V of the q new tokens are appended to the cache views in place.
    Reference: modeling_llama.py:113-172 (attention), :175-199 (layer),
    :207-237 (model), :240-276 (LM head, fp32 logits).
    """
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg["num_key_value_heads"]
    hd = H // nh
    eps = cfg["rms_norm_eps"]
    B, q_len = input_ids.shape
    h = w["model.embed_tokens.weight"][input_ids].astype(np.float32)
    n_pos = int(max(position_ids.max() + 1, past_key_values[0][0].length + q_len, 1))
    cos, sin = rope_tables(hd, n_pos, cfg.get("rope_theta", 10000.0))
    pos = np.maximum(position_ids, 0)  # rows of pad tokens carry negative positions; their output is never read
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        qs = (x @ w[p + "self_attn.q_proj.weight"].T).reshape(B, q_len, nh, hd).transpose(0, 2, 1, 3)
        ks = (x @ w[p + "self_attn.k_proj.weight"].T).reshape(B, q_len, nkv, hd).transpose(0, 2, 1, 3)
        vs = (x @ w[p + "self_attn.v_proj.weight"].T).reshape(B, q_len, nkv, hd).transpose(0, 2, 1, 3)
        qs = apply_rope(qs, cos, sin, pos)
        ks = apply_rope(ks, cos, sin, pos)
        kview, vview = past_key_values[l]
        k_all = kview.cat(ks)
        v_all = vview.cat(vs)
        if nkv != nh:
            k_all = np.repeat(k_all, nh // nkv, axis=1)
            v_all = np.repeat(v_all, nh // nkv, axis=1)
        o = attention(qs, k_all, v_all, attention_mask)
        o = o.transpose(0, 2, 1, 3).reshape(B, q_len, H)
        h = h + o @ w[p + "self_attn.o_proj.weight"].T
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        g = silu(x @ w[p + "mlp.gate_proj.weight"].T) * (x @ w[p + "mlp.up_proj.weight"].T)
        h = h + g @ w[p + "mlp.down_proj.weight"].T
    hidden = rms_norm(h, w["model.norm.weight"], eps)
    logits = (hidden @ w["lm_head.weight"].T).astype(np.float32)
    return logits, hidden
