"""Whole decode loops through the public API against the reference's own runs (fixtures generated
by importing the reference) and against the oracle's step traces."""
from unittest import mock

import numpy as np
import pytest
import torch

import model_builders as mb
from gpu_helpers import build_models, t
from oracle import generate as ogen

pytestmark = pytest.mark.gpu

CASES = [("c1", mb.C1_LLAMA, mb.C1_DRAFTER, 123), ("c1pad", mb.C1_LLAMA, mb.C1_DRAFTER, 123), ("nano", mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)]


@pytest.mark.parametrize("tag,lcfg,dcfg,seed", CASES)
def test_generate_greedy_fp32_equals_reference(g_model, tag, lcfg, dcfg, seed):
    """fp32 greedy: token stream, per-step lengths, accepted counts, chosen beams, drafted beams and
    the reference-layout commit slots equal the reference's (bit-exact integers)."""
    import recurrent_drafting as rd

    B, Lp, gen, W, L = (int(x) for x in g_model[f"gen_{tag}_shape"])
    llm, dr, lw, dw = build_models(lcfg, dcfg, seed)
    model = rd.RecurrentDrafting(llm, dr)
    prompt = g_model[f"gen_{tag}_prompt"]
    shape = rd.modeling_drafter.BeamShape(W, L)
    trace = []
    list(ogen.generate(lw, lcfg, dw, dcfg["num_draft_layers"], prompt, Lp + gen, W, L, greedy=True, trace=trace))
    ledger = rd.stats.Ledger()
    lengths, ns, seqs, beams = [], [], [], []
    final = None
    for step, out in enumerate(model.generate(ledger, t(prompt), Lp + gen, shape, rd.SamplingArgs(1.0, True), rd.SpecialTokens(0, None))):
        st = model.last_state
        lengths.append(out.shape[1])
        ns.append(st.small_host[1].numpy().copy())
        seqs.append(st.seq_in_beam.cpu().numpy().copy())
        beams.append(dr._workspace(B, W, L)["beams"][(L - 1) % 2].cpu().numpy().copy())
        slots = model.reference_commit_slots(shape).cpu().numpy()
        plan = trace[step]["plan"]
        assert np.array_equal(slots[:, :, 0], plan["src_packed_slot"]), step
        assert np.array_equal(slots[:, :, 1], plan["src_unpacked_slot"]), step
        assert np.array_equal(slots[:, :, 2], plan["dst_slot"]), step
        final = out.cpu().numpy()
    assert lengths == g_model[f"gen_{tag}_lengths"].tolist()
    assert np.array_equal(np.stack(ns), g_model[f"gen_{tag}_n"])
    assert np.array_equal(np.stack(seqs), g_model[f"gen_{tag}_seq"])
    assert np.array_equal(np.stack(beams), g_model[f"gen_{tag}_beams"])
    assert np.array_equal(final, g_model[f"gen_{tag}_final"])
    table, _ = rd.stats.summarize(ledger, B, L - 1)
    assert table.avg_token_per_step >= 1.0 and table.avg_step_time > 0


@pytest.mark.parametrize("B,W,L,Lp,gen", [(1, 1, 2, 5, 12), (1, 50, 8, 6, 20), (3, 2, 2, 9, 10), (2, 45, 5, 3, 14)])
def test_generate_edge_beam_shapes_fp32_equal_the_oracle(B, W, L, Lp, gen):
    """The smallest and the largest beam shapes the reference's sweeps use (one beam of two tokens; fifty beams of
    eight, the widest search whose first iteration has no exact ties), single-row batches and prompts shorter than a
    beam: fp32 greedy streams, accepted counts and chosen beams equal the oracle's step by step."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    model = rd.RecurrentDrafting(llm, dr)
    prompt = mb.prompts(B, Lp, mb.NANO_LLAMA["vocab_size"], 100 + W, left_pads=[0, 2, 1][:B] if Lp > 3 else None)
    trace = []
    want = list(ogen.generate(lw, mb.NANO_LLAMA, dw, mb.NANO_DRAFTER["num_draft_layers"], prompt, Lp + gen, W, L, greedy=True, trace=trace))
    got = []
    for step, out in enumerate(model.generate(rd.stats.Ledger(), t(prompt), Lp + gen, rd.modeling_drafter.BeamShape(W, L),
                                              rd.SamplingArgs(1.0, True), rd.SpecialTokens(0, None))):
        st = model.last_state
        assert np.array_equal(st.small_host[1].numpy(), trace[step]["n_tokens_in_seq"]), step
        assert np.array_equal(st.seq_in_beam.cpu().numpy(), trace[step]["seq_in_beam"]), step
        got.append(out.cpu().numpy())
    assert len(got) == len(want)
    for a, b_ in zip(got, want):
        assert np.array_equal(a, b_)


def test_autoregressive_equals_reference_and_redrafter(g_model):
    import recurrent_drafting as rd

    B, Lp, gen, W, L = (int(x) for x in g_model["gen_c1_shape"])
    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 123)
    model = rd.RecurrentDrafting(llm, dr)
    outs = list(rd.autoregressive.generate(model, t(g_model["gen_c1_prompt"]), Lp + gen, rd.SpecialTokens(0, -1)))
    final = outs[-1].cpu().numpy()
    assert np.array_equal(final, g_model["gen_c1_ar_final"])
    assert np.array_equal(final, g_model["gen_c1_final"][:, : Lp + gen])


def test_generate_sampling_with_injected_randomness(g_model):
    """Sampling loop: with the same uniforms on both sides the stream equals the reference's."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    model = rd.RecurrentDrafting(llm, dr)
    src = ogen.UniformSource(77)

    def fake_rand(*shape, device=None, **kw):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return t(src.uniform(tuple(shape)))

    lengths = []
    with mock.patch.object(rd.recurrent_drafting.torch, "rand", fake_rand):
        for out in model.generate(rd.stats.Ledger(), t(g_model["gen_samp_prompt"]), 30, rd.modeling_drafter.BeamShape(5, 4),
                                  rd.SamplingArgs(0.7, False), rd.SpecialTokens(0, None)):
            lengths.append(out.shape[1])
            final = out.cpu().numpy()
    assert lengths == g_model["gen_samp_lengths"].tolist()
    assert np.array_equal(final, g_model["gen_samp_final"])


def test_generate_bf16_runs_and_matches_own_autoregression_mostly():
    """bf16 is not token-exact against autoregression even in the reference; check the loop runs,
    keeps its invariants (lengths grow, prompt preserved) and agrees with AR on most tokens."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 123, dtype=torch.bfloat16)
    model = rd.RecurrentDrafting(llm, dr)
    prompt = t(mb.prompts(2, 32, 1000, 9))
    outs = list(model.generate(rd.stats.Ledger(), prompt, 64, rd.modeling_drafter.BeamShape(4, 3), rd.SamplingArgs(1.0, True), rd.SpecialTokens(0, None)))
    final = outs[-1]
    assert final.shape[1] == 64 and torch.equal(final[:, :32], prompt)
    ar = list(rd.autoregressive.generate(model, prompt, 64, rd.SpecialTokens(0, -1)))[-1]
    agree = (final == ar).float().mean().item()
    assert agree > 0.6, agree


def test_cpu_input_is_rejected():
    import recurrent_drafting as rd

    llm, dr, _, _ = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    model = rd.RecurrentDrafting(llm, dr)
    with pytest.raises(rd._lib.RedrafterError):
        next(model.generate(rd.stats.Ledger(), torch.zeros(1, 4, dtype=torch.long), 8, rd.modeling_drafter.BeamShape(2, 2)))


def test_generation_stops_when_every_row_has_produced_eos(g_model):
    """The whole-batch EOS test of the loop (recurrent_drafting.py:697-705): generation ends with the
    step in which the last row has emitted the EOS id, not earlier and not later; same stream as
    the oracle run with the same EOS id."""
    import recurrent_drafting as rd

    B, Lp, gen, W, L = (int(x) for x in g_model["gen_c1_shape"])
    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 123)
    model = rd.RecurrentDrafting(llm, dr)
    prompt = g_model["gen_c1_prompt"]
    final = g_model["gen_c1_final"]
    # an id that every row emits at some point of the unconstrained run, as late as possible
    tail = final[:, Lp:]
    common = set(tail[0].tolist())
    for b in range(1, B):
        common &= set(tail[b].tolist())
    assert common, "the fixture rows share no generated token"
    eos = max(common, key=lambda tok: max(int(np.argmax(tail[b] == tok)) for b in range(B)))
    want = list(ogen.generate(lw, mb.C1_LLAMA, dw, mb.C1_DRAFTER["num_draft_layers"], prompt, Lp + gen, W, L, greedy=True,
                              eos_token_id=int(eos)))
    got = [o.cpu().numpy() for o in model.generate(rd.stats.Ledger(), t(prompt), Lp + gen, rd.modeling_drafter.BeamShape(W, L),
                                                   rd.SamplingArgs(1.0, True), rd.SpecialTokens(0, int(eos)))]
    assert len(got) == len(want) and len(got) < len(g_model["gen_c1_lengths"])
    for a, b_ in zip(got, want):
        assert np.array_equal(a, b_)
