"""Oracle (numpy fp32) of the ReDrafter decode loop and of the autoregressive
baseline loop.  Test infrastructure only.

Restates RecurrentDrafting._generate and its helpers
(recurrent_drafting/recurrent_drafting.py:391-465, 596-705) and
autoregressive.generate (recurrent_drafting/autoregressive.py:13-53).
"""

from typing import Callable, Dict, Iterator, List, Optional

import numpy as np

from . import acceptance, drafter, kv_cache, llama, tree_attention


class UniformSource:
    """Injected randomness: uniform(shape) returns fp32 uniforms in [0,1).  The
    order of requests per step is fixed: acceptance uniforms (B,W,Lb-1), then
    the categorical uniforms (B,)."""

    def __init__(self, seed: int):
        self._rs = np.random.RandomState(seed)

    def uniform(self, shape) -> np.ndarray:
        return self._rs.random_sample(shape).astype(np.float32)


def comprehend_prompt(llm_w, cfg, input_ids, cache, greedy, temperature, pad_token_id, rng: Optional[UniformSource]):
    """Prefill.  Reference: recurrent_drafting.py:391-434."""
    B, Lp = input_ids.shape
    mask = tree_attention.padded_causal_mask(input_ids != pad_token_id, Lp)
    pads = acceptance.count_left_paddings(input_ids, pad_token_id)
    pos = np.arange(Lp, dtype=np.int64)[None, :] - pads[:, None]
    logits, hidden = llama.forward(llm_w, cfg, input_ids, mask, pos, cache.sliced)
    last = drafter.warp_logits(logits[:, -1, :])
    if greedy:
        nxt = np.argmax(last, axis=-1).astype(np.int64)
    else:
        z = last / np.float32(temperature)
        z = z - z.max(axis=-1, keepdims=True)
        p = np.exp(z)
        p /= p.sum(axis=-1, keepdims=True)
        nxt = acceptance.sample_inverse_cdf(p.astype(np.float32), rng.uniform((B,)))
    return hidden[:, -1, :], nxt


def verify_candidates(llm_w, cfg, input_ids, beams, cache, pad_token_id):
    """Pack, run the LLM over the packed tree tokens, unpack hidden states,
    logits and the KV cache into per-beam layout.  Reference: recurrent_drafting.py:437-465."""
    packed, unpacker, mask, offs = tree_attention.pack(beams, (input_ids != pad_token_id).astype(np.int64))
    pads = acceptance.count_left_paddings(input_ids, pad_token_id)
    past = cache.sliced[0][0].length - pads[:, None]
    logits, hidden = llama.forward(llm_w, cfg, packed, mask, past + offs, cache.sliced)
    logits = drafter.warp_logits(logits)
    hidden = tree_attention.unpack(hidden, unpacker)
    logits = tree_attention.unpack(logits, unpacker)
    cache.unpack(input_ids.shape[-1], unpacker)
    return hidden, logits, unpacker


def generate(
    llm_w: Dict[str, np.ndarray],
    cfg: Dict,
    drafter_w: Dict[str, np.ndarray],
    num_draft_layers: int,
    input_ids: np.ndarray,
    max_length: int,
    beam_width: int,
    beam_length: int,
    greedy: bool = True,
    temperature: float = 1.0,
    pad_token_id: int = 0,
    eos_token_id: Optional[int] = None,
    rng: Optional[UniformSource] = None,
    max_steps: Optional[int] = None,
    trace: Optional[List[Dict]] = None,
    on_phase: Optional[Callable[[str], None]] = None,
) -> Iterator[np.ndarray]:
    """Yields the (B, <=max_length) int64 token matrix after every decode step.

    Reference: recurrent_drafting.py:596-705.  `trace`, if given, receives one
    dict per step with the intermediate tensors the parity tests compare.
    """
    B, seq_len = input_ids.shape
    init_len = seq_len
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    cache = kv_cache.Cache(B, max_length + beam_length * beam_width, cfg["num_hidden_layers"], cfg["num_key_value_heads"], H // nh)
    context, init_tokens = comprehend_prompt(llm_w, cfg, input_ids, cache, greedy, temperature, pad_token_id, rng)
    emb = llm_w["model.embed_tokens.weight"]
    steps = 0
    while seq_len < max_length and (max_steps is None or steps < max_steps):
        if on_phase:
            on_phase("generate_candidates")
        beams, logq = drafter.beam_search_candidates(
            drafter_w, num_draft_layers, context, init_tokens, emb, beam_width, beam_length
        )
        if on_phase:
            on_phase("verify_candidates")
        hidden, logits, unpacker = verify_candidates(llm_w, cfg, input_ids, beams, cache, pad_token_id)
        if on_phase:
            on_phase("accept_candidate_tokens")
        if greedy:
            by_llm = np.argmax(logits, axis=-1)
            n, seq = acceptance.greedy_choose_from_candidates(beams, by_llm)
        else:
            logp = drafter.log_softmax(logits / np.float32(temperature))
            u = rng.uniform((B, beam_width, beam_length - 1))
            n, seq = acceptance.choose_from_candidates(beams, logp, logq, u)
        plan = acceptance.commit_plan(input_ids, n, seq, unpacker, pad_token_id)
        new_ids = acceptance.update_kv_cache_and_input_ids(input_ids, n, seq, beams, cache, pad_token_id)
        if greedy:
            context, init_tokens = acceptance.greedy_prepare_next_input(by_llm, hidden, seq, n)
        else:
            probs = acceptance.residual_probs(logq, logp, seq, n)
            init_tokens = acceptance.sample_inverse_cdf(probs, rng.uniform((B,)))
            context = hidden[np.arange(B), seq, n]
        if trace is not None:
            trace.append(
                {
                    "beams": beams,
                    "unpacker": unpacker,
                    "n_tokens_in_seq": n,
                    "seq_in_beam": seq,
                    "next_tokens": init_tokens,
                    "plan": plan,
                    "input_ids": new_ids,
                }
            )
        input_ids = new_ids
        out = np.concatenate([input_ids, init_tokens[:, None]], axis=-1)
        seq_len = out.shape[1]
        steps += 1
        if on_phase:
            on_phase("end_step")
        yield out[:, :max_length] if out.shape[1] > max_length else out
        if eos_token_id is not None and ((out[:, init_len:] == eos_token_id).sum(axis=-1) > 0).sum() == B:
            break


def autoregressive(llm_w, cfg, input_ids, max_length, pad_token_id=0, eos_token_id=None) -> Iterator[np.ndarray]:
    """Greedy one-token-per-step loop over the same model and cache.
    Reference: autoregressive.py:13-53."""
    B = input_ids.shape[0]
    H = cfg["hidden_size"]
    cache = kv_cache.Cache(B, max_length, cfg["num_hidden_layers"], cfg["num_key_value_heads"], H // cfg["num_attention_heads"])
    ctx_len = input_ids.shape[1]
    while input_ids.shape[1] < max_length:
        pad_mask = input_ids != pad_token_id
        cur = input_ids[:, -1:] if input_ids.shape[1] > ctx_len else input_ids
        mask = tree_attention.padded_causal_mask(pad_mask, cur.shape[1])
        past = cache.sliced[0][0].length
        pos = np.broadcast_to(np.arange(past, past + cur.shape[1], dtype=np.int64)[None, :], cur.shape)
        logits, _ = llama.forward(llm_w, cfg, cur, mask, pos, cache.sliced)
        nxt = np.argmax(logits[:, -1, :], axis=-1).astype(np.int64)
        input_ids = np.concatenate([input_ids, nxt[:, None]], axis=-1)
        yield input_ids
        if eos_token_id is not None and ((input_ids[:, ctx_len:] == eos_token_id).sum(axis=-1) > 0).sum() == B:
            break
