"""Decode loops in which draft tokens ARE accepted (random-init model pairs accept none): a model pair
with planted next-token maps, a heavily left-padded row that accepts every draft while the longest
row accepts few, run up to max_length.  The CPU part pins the construction on the oracle; the GPU part
compares the CUDA loop with the oracle step by step, including the cache rows the commit moved
(recurrent_drafting/recurrent_drafting.py:114-232, 468-496)."""
import numpy as np
import pytest

import model_builders as mb
from oracle import generate as ogen

W, LB, LP, GEN = 4, 4, 40, 24


def _prompt(cycle):
    """Row 0: no padding, its chain runs through the ids the drafter gets wrong.  Row 1: 30 pads, chain
    in a stretch the drafter gets right.  Row 2: 15 pads, chain that crosses from right to wrong."""
    V = mb.PLANTED_LLAMA["vocab_size"]
    ids = mb.prompts(3, LP, V, 9, left_pads=[0, 30, 15])
    ids[0, -1] = cycle[0]
    ids[1, -1] = cycle[80]
    ids[2, -1] = cycle[len(cycle) - 12]
    return ids


def _oracle_run():
    lw, dw, cycle = mb.planted_models()
    prompt = _prompt(cycle)
    trace = []
    outs = list(ogen.generate(lw, mb.PLANTED_LLAMA, dw, 1, prompt, LP + GEN, W, LB, greedy=True, trace=trace))
    return lw, dw, cycle, prompt, trace, outs


def test_planted_pair_accepts_in_the_planted_pattern():
    lw, dw, cycle, prompt, trace, outs = _oracle_run()
    pos = {int(tok): i for i, tok in enumerate(cycle)}
    final = outs[-1]
    # every generated token follows the LLM's map f, whatever was drafted
    for b in range(3):
        for c in range(LP, final.shape[1]):
            if final[b, c - 1] != 0:
                assert pos[int(final[b, c])] == (pos[int(final[b, c - 1])] + 1) % len(cycle)
    n = np.stack([tr["n_tokens_in_seq"] for tr in trace])
    assert (n[:, 1] == LB - 1).all(), n[:, 1]  # the padded row accepts every draft
    assert n[:, 0].max() <= 1, n[:, 0]  # the unpadded row: every other guess is wrong
    assert len(set(n[:, 2].tolist())) >= 2, n[:, 2]
    # the padded row outgrows the unpadded one's padding: the case a fixed left offset per row cannot hold
    assert 30 + (LP - 30) + int(n[:, 1].sum()) + len(trace) > LP + GEN


@pytest.mark.gpu
def test_planted_acceptance_loop_equals_oracle():
    import torch

    import recurrent_drafting as rd
    from gpu_helpers import llama_config, t

    lw, dw, cycle, prompt, trace, outs = _oracle_run()
    llm = rd.modeling_llama.LlamaForCausalLM(llama_config(mb.PLANTED_LLAMA)).to(device="cuda", dtype=torch.float32)
    llm.load_state_dict({k: torch.from_numpy(v) for k, v in lw.items()})
    dr = rd.modeling_drafter.Drafter(rd.configuration_drafter.DrafterConfig(**mb.PLANTED_DRAFTER)).to(device="cuda", dtype=torch.float32)
    dr.load_state_dict({k: torch.from_numpy(v) for k, v in dw.items()})
    model = rd.RecurrentDrafting(llm, dr)
    shape = rd.modeling_drafter.BeamShape(W, LB)
    got = []
    for step, out in enumerate(model.generate(rd.stats.Ledger(), t(prompt), LP + GEN, shape, rd.SamplingArgs(1.0, True),
                                              rd.SpecialTokens(0, None))):
        st = model.last_state
        tr = trace[step]
        assert np.array_equal(st.small_host[1].numpy(), tr["n_tokens_in_seq"]), step
        assert np.array_equal(st.seq_in_beam.cpu().numpy(), tr["seq_in_beam"]), step
        assert np.array_equal(out.cpu().numpy(), outs[step]), step
        slots = model.reference_commit_slots(shape).cpu().numpy()
        assert np.array_equal(slots[:, :, 0], tr["plan"]["src_packed_slot"]), step
        assert np.array_equal(slots[:, :, 2], tr["plan"]["dst_slot"]), step
        max_len = st.token_buf.shape[1]
        assert int((st.kv_begin + st.kv_len).max()) + W * LB <= max_len
        got.append(out)
    assert len(got) == len(outs)
    # committed K/V: in this model pair a token's K/V depend on the token and its position only (the residual
    # stream stays the embedding), so row b's live slots [0, kv_len) must equal a fresh prefill of the same tokens
    kv_len = st.kv_len.cpu().numpy()
    B = prompt.shape[0]
    longest = int(kv_len.max())
    again = np.zeros((B, longest), dtype=np.int64)
    tok = st.token_buf.cpu().numpy()
    for b in range(B):
        again[b, longest - kv_len[b] :] = tok[b, : kv_len[b]]
    committed = model.last_cache._cache.clone()
    fresh = rd.RecurrentDrafting(llm, dr)
    next(fresh.generate(rd.stats.Ledger(), t(again), longest + 8, shape, rd.SamplingArgs(1.0, True), rd.SpecialTokens(0, None)))
    prefilled = fresh.last_cache._cache
    for b in range(B):
        np.testing.assert_allclose(committed[:, :, b, :, : kv_len[b]].cpu().numpy(), prefilled[:, :, b, :, : kv_len[b]].cpu().numpy(),
                                   rtol=1e-5, atol=1e-6)
