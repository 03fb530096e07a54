"""Deterministic random-init weights for the parity tests.

The same numpy streams feed the reference (when golden fixtures are generated),
the numpy oracle and the CUDA models, so no weight tensor has to be stored.
"""

from typing import Dict, Tuple

import numpy as np

# BASELINE config 1: tiny CPU-runnable Llama + drafter.
C1_LLAMA = dict(
    hidden_size=256,
    num_attention_heads=4,
    num_key_value_heads=4,
    num_hidden_layers=2,
    intermediate_size=688,
    vocab_size=1000,
    rms_norm_eps=1e-6,
    rope_theta=10000.0,
)
C1_DRAFTER = dict(vocab_size=1000, hidden_size=256, exit_dim=512, num_draft_layers=1, rnn=True)

# An even smaller pair for function-level fixtures.
NANO_LLAMA = dict(
    hidden_size=64,
    num_attention_heads=2,
    num_key_value_heads=2,
    num_hidden_layers=2,
    intermediate_size=176,
    vocab_size=320,
    rms_norm_eps=1e-6,
    rope_theta=10000.0,
)
NANO_DRAFTER = dict(vocab_size=320, hidden_size=64, exit_dim=128, num_draft_layers=2, rnn=True)
# the drafter variants the reference also supports: no recurrent projections (state = embedding + state) and an
# input projection (exit_dim != 2 * hidden_size)
NANO_DRAFTER_NO_RNN = dict(vocab_size=320, hidden_size=64, exit_dim=96, num_draft_layers=1, rnn=False)


def llama_weights(cfg: Dict, seed: int, std: float = 0.05) -> Dict[str, np.ndarray]:
    rs = np.random.RandomState(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh

    def n(*shape):
        return (rs.standard_normal(shape) * std).astype(np.float32)

    def g(size):
        return (1.0 + 0.1 * rs.standard_normal(size)).astype(np.float32)

    w = {"model.embed_tokens.weight": n(V, H)}
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        w[p + "self_attn.q_proj.weight"] = n(nh * hd, H)
        w[p + "self_attn.k_proj.weight"] = n(nkv * hd, H)
        w[p + "self_attn.v_proj.weight"] = n(nkv * hd, H)
        w[p + "self_attn.o_proj.weight"] = n(H, nh * hd)
        w[p + "mlp.gate_proj.weight"] = n(I, H)
        w[p + "mlp.up_proj.weight"] = n(I, H)
        w[p + "mlp.down_proj.weight"] = n(H, I)
        w[p + "input_layernorm.weight"] = g(H)
        w[p + "post_attention_layernorm.weight"] = g(H)
    w["model.norm.weight"] = g(H)
    w["lm_head.weight"] = n(V, H)
    return w


def drafter_weights(cfg: Dict, seed: int, std: float = 0.05) -> Dict[str, np.ndarray]:
    rs = np.random.RandomState(seed)
    H, E, V, R = cfg["hidden_size"], cfg["exit_dim"], cfg["vocab_size"], cfg["num_draft_layers"]

    def n(*shape):
        return (rs.standard_normal(shape) * std).astype(np.float32)

    w = {}
    if E != 2 * H:
        w["input_proj.weight"] = n(E, 2 * H)
        w["input_proj.bias"] = n(E)
    for r in range(R):
        w[f"lm_head.{r}.linear.weight"] = n(E, E)
        w[f"lm_head.{r}.linear.bias"] = n(E)
    w[f"lm_head.{R}.weight"] = n(V, E)
    if cfg.get("rnn", True):
        w["rnn_u.weight"] = n(H, H)
        w["rnn_u.bias"] = n(H)
        w["rnn_w.weight"] = n(H, H)
    return w


def prompts(batch: int, length: int, vocab: int, seed: int, left_pads=None, pad_id: int = 0) -> np.ndarray:
    """Uniform token ids in [3, vocab); left_pads[b] leading positions set to pad_id."""
    rs = np.random.RandomState(seed)
    ids = rs.randint(3, vocab, size=(batch, length)).astype(np.int64)
    if left_pads is not None:
        for b, p in enumerate(left_pads):
            ids[b, :p] = pad_id
    return ids


def zipf_beams(batch: int, width: int, length: int, vocab: int, seed: int, a: float = 1.2, branch: int = 3) -> np.ndarray:
    """Beams whose column 0 is one shared init token per row and whose further
    tokens are drawn from a prefix-conditional Zipf(a) law over a few children
    per prefix, so that a sizeable fraction of prefixes is shared."""
    rs = np.random.RandomState(seed)
    out = np.zeros((batch, width, length), dtype=np.int64)
    for b in range(batch):
        out[b, :, 0] = rs.randint(3, vocab)
        children: Dict[Tuple, np.ndarray] = {}
        for i in range(width):
            for j in range(1, length):
                key = tuple(out[b, i, :j])
                if key not in children:
                    children[key] = np.clip(rs.zipf(a, size=branch) + 2, 3, vocab - 1)
                out[b, i, j] = children[key][min(rs.zipf(a) - 1, branch - 1)]
    return out


# A model pair with PLANTED acceptance, so that decode steps accept 0 .. Lb-1 draft tokens in a known
# pattern (random-init pairs accept nothing).  The LLM's output projections of attention and MLP are zero,
# so its residual stream stays the token embedding and its LM head maps token t to f(t); the drafter maps
# token t to g(t) through its recurrent state; f is one cycle over the ids [3, V), g equals f except on the
# ids in `wrong`, where the draft is rejected.
PLANTED_LLAMA = dict(hidden_size=64, num_attention_heads=2, num_key_value_heads=2, num_hidden_layers=2, intermediate_size=96,
                     vocab_size=200, rms_norm_eps=1e-6, rope_theta=10000.0)
PLANTED_DRAFTER = dict(vocab_size=200, hidden_size=64, exit_dim=128, num_draft_layers=1, rnn=True)


def planted_models(seed: int = 5, n_wrong: int = 30):
    """Returns (llama weights, drafter weights, cycle): cycle[i+1] = f(cycle[i]); the drafter's guess
    after cycle[2*i] (i < n_wrong) is wrong."""
    lcfg, dcfg = PLANTED_LLAMA, PLANTED_DRAFTER
    rs = np.random.RandomState(seed)
    V, H = lcfg["vocab_size"], lcfg["hidden_size"]
    lw = llama_weights(lcfg, seed)
    for l in range(lcfg["num_hidden_layers"]):
        lw[f"model.layers.{l}.self_attn.o_proj.weight"][:] = 0
        lw[f"model.layers.{l}.mlp.down_proj.weight"][:] = 0
    lw["model.norm.weight"][:] = 1
    emb = rs.standard_normal((V, H)).astype(np.float32)
    lw["model.embed_tokens.weight"] = emb
    cycle = 3 + rs.permutation(V - 3)
    f = {int(cycle[i]): int(cycle[(i + 1) % len(cycle)]) for i in range(len(cycle))}
    g = dict(f)
    for i in range(n_wrong):
        tkn = int(cycle[2 * i])
        g[tkn] = int(cycle[(2 * i + 7) % len(cycle)])  # some other id than f(tkn)
    head = np.zeros((V, H), dtype=np.float32)
    for tkn, nxt in f.items():
        head[nxt] = emb[tkn]
    lw["lm_head.weight"] = head
    dw = drafter_weights(dcfg, seed + 1)
    E = dcfg["exit_dim"]
    dw["lm_head.0.linear.weight"][:] = 0
    dw["lm_head.0.linear.bias"][:] = 0
    dw["rnn_u.weight"][:] = 0
    dw["rnn_u.bias"][:] = 0
    dw["rnn_w.weight"] = (2.0 * np.eye(H)).astype(np.float32)
    x = 2.0 * emb
    state = (x / (1.0 + np.exp(-x))).astype(np.float32)  # silu(rnn_w e_t): the state after reading token t
    centred = state - state[3:].mean(axis=0, keepdims=True)
    vocab = np.zeros((V, E), dtype=np.float32)
    # several tokens may share a wrong guess; the later assignment wins, which only moves where drafts fail
    for tkn, nxt in g.items():
        vocab[nxt, H:] = centred[tkn]
    for tkn, nxt in f.items():
        if g[tkn] == nxt:
            vocab[nxt, H:] = centred[tkn]
    dw["lm_head.1.weight"] = vocab
    return lw, dw, cycle
