"""Drafter kernels: vocabulary top-k/log-softmax, cross-beam selection, whole beam search."""
import numpy as np
import pytest
import torch

import model_builders as mb
from gpu_helpers import bf16_round, build_models, t
from oracle import drafter as odr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,subtract,temp", [(1000, True, 1.0), (32000, True, 1.0), (32000, False, 0.7), (320, False, 1.3), (40, True, 1.0)])
def test_vocab_topk_vs_oracle(dtype, V, subtract, temp):
    import recurrent_drafting as rd

    md = rd.modeling_drafter
    rs = np.random.RandomState(V)
    rows = 9
    logits = (rs.standard_normal((rows, V)) * 3).astype(np.float32)
    logits[2, 5] = logits[2, 17] = logits[2].max() + 1.0  # tie at the top
    tl = t(logits).to(dtype)
    logits = tl.float().cpu().numpy()
    sp = md.vocab_topk(tl, md.new_sparse(rows, "cuda"), subtract_max=subtract, temperature=temp)
    z = odr.maintain_logits(logits) if subtract else logits
    want = odr.log_softmax(odr.warp_logits(z) / np.float32(temp))
    val, idx, cnt, masked = (x.cpu().numpy() for x in (sp.val, sp.idx, sp.cnt, sp.masked))
    for r in range(rows):
        kept = np.nonzero(odr.warp_logits(z)[r] > -49000)[0]
        n = min(len(kept), 64)
        assert cnt[r] == n
        order = sorted(kept, key=lambda v: (-want[r, v], v))[:n]
        assert list(idx[r, :n]) == order
        np.testing.assert_allclose(val[r, :n], want[r, order], rtol=1e-5, atol=2e-5)
        others = np.setdiff1d(np.arange(V), kept)
        if len(others):
            np.testing.assert_allclose(masked[r], want[r, others[0]], rtol=1e-6)
    assert idx[2, 0] == 5 and idx[2, 1] == 17


def test_beam_search_fp32_vs_reference_fixture(g_model):
    """Beams equal to the reference's, log-probs within fp32 noise (fixture from the reference)."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    beams, logq = dr.beam_search_candidates(t(g_model["bs_state"]), t(g_model["bs_tok"]), llm.get_input_embeddings(),
                                            rd.modeling_drafter.BeamShape(5, 4))
    assert np.array_equal(beams.cpu().numpy(), g_model["bs_beams"])
    assert logq.dtype == torch.float32 and tuple(logq.shape) == g_model["bs_logq"].shape
    np.testing.assert_allclose(logq.cpu().numpy(), g_model["bs_logq"], rtol=1e-4, atol=2e-4)


def test_beam_search_without_recurrent_projections_vs_reference_fixture(g_variants):
    """A drafter built with rnn=False (state = embedding + state) and an input projection: beams equal to the
    reference's, log-probs within fp32 noise."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER_NO_RNN, 41)
    assert not hasattr(dr, "rnn_u") and hasattr(dr, "input_proj")
    beams, logq = dr.beam_search_candidates(t(g_variants["nornn_state"]), t(g_variants["nornn_tok"]), llm.get_input_embeddings(),
                                            rd.modeling_drafter.BeamShape(6, 4))
    assert np.array_equal(beams.cpu().numpy(), g_variants["nornn_beams"])
    np.testing.assert_allclose(logq.cpu().numpy(), g_variants["nornn_logq"], rtol=1e-4, atol=2e-4)


@pytest.mark.parametrize("B,W,Lb", [(2, 4, 3), (3, 45, 5), (1, 50, 2), (2, 16, 8)])
def test_beam_search_fp32_vs_oracle(B, W, Lb):
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 123)
    rs = np.random.RandomState(B * 100 + W)
    state = rs.standard_normal((B, 256)).astype(np.float32)
    tok = rs.randint(3, 1000, size=(B,)).astype(np.int64)
    want_beams, want_logq = odr.beam_search_candidates(dw, 1, state, tok, lw["model.embed_tokens.weight"], W, Lb)
    beams, logq = dr.beam_search_candidates(t(state), t(tok), llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(W, Lb))
    assert np.array_equal(beams.cpu().numpy(), want_beams)
    np.testing.assert_allclose(logq.cpu().numpy(), want_logq, rtol=1e-4, atol=3e-4)


def test_beam_search_bf16_tolerance():
    """bf16: beams are not pinned (near-ties reorder).  With beam_length 2 the beams are the top-W
    candidates of one iteration: their set and log-probs must agree with the fp32 oracle holding
    the same bf16-rounded weights; longer searches must still share most prefixes."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 123, dtype=torch.bfloat16)
    lwr, dwr = bf16_round(lw), bf16_round(dw)
    rs = np.random.RandomState(4)
    B, W = 4, 8
    state = t(rs.standard_normal((B, 256)).astype(np.float32)).bfloat16()
    tok_np = rs.randint(3, 1000, size=(B,)).astype(np.int64)
    tok = t(tok_np)
    emb = lwr["model.embed_tokens.weight"]
    want_beams, want_logq = odr.beam_search_candidates(dwr, 1, state.float().cpu().numpy(), tok_np, emb, W, 2)
    beams, logq = dr.beam_search_candidates(state, tok, llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(W, 2))
    beams, logq = beams.cpu().numpy(), logq.cpu().numpy()
    assert np.array_equal(beams[:, :, 0], want_beams[:, :, 0])
    for b in range(B):
        common = set(beams[b, :, 1]) & set(want_beams[b, :, 1])
        assert len(common) >= W - 2, (b, beams[b, :, 1], want_beams[b, :, 1])
        for v in common:
            i, j = list(beams[b, :, 1]).index(v), list(want_beams[b, :, 1]).index(v)
            assert abs(logq[b, i, 0, v] - want_logq[b, j, 0, v]) <= 0.08
    want4, _ = odr.beam_search_candidates(dwr, 1, state.float().cpu().numpy(), tok_np, emb, W, 4)
    got4, _ = dr.beam_search_candidates(state, tok, llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(W, 4))
    got4 = got4.cpu().numpy()
    same = sum(tuple(r) in {tuple(x) for x in want4[b]} for b in range(B) for r in got4[b])
    assert same >= B * W // 2, same


def test_beam_search_bf16_vocabulary_32000_teacher_forced():
    """The drafter at the benchmark's routing (bf16 tcgen05 GEMMs, exit_dim 1024 with two residual blocks,
    vocabulary head of 32000 with slice maxima + sliced top-k, 45 beams of 5) against the fp32 oracle holding
    the same bf16-rounded weights.  bf16 beams are not pinned (near-ties reorder), so the oracle is teacher-forced
    along the GPU's own beams: a beam's tokens determine its recurrent state, hence the log-softmax row every one
    of its positions was drawn from; those rows must agree where both sides keep the entry."""
    import recurrent_drafting as rd
    from gpu_helpers import HD128_DRAFTER, HD128_LLAMA

    llm, dr, lw, dw = build_models(HD128_LLAMA, HD128_DRAFTER, 77, dtype=torch.bfloat16)
    dwr = bf16_round(dw)
    emb = bf16_round({"e": lw["model.embed_tokens.weight"]})["e"]
    H, V, R = HD128_DRAFTER["hidden_size"], HD128_DRAFTER["vocab_size"], HD128_DRAFTER["num_draft_layers"]
    B, W, Lb = 2, 45, 5
    rs = np.random.RandomState(8)
    state = t(rs.standard_normal((B, H)).astype(np.float32)).bfloat16()
    tok_np = rs.randint(3, V, size=(B,)).astype(np.int64)
    beams, logq = dr.beam_search_candidates(state, t(tok_np), llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(W, Lb))
    beams, logq = beams.cpu().numpy(), logq.cpu().numpy()
    assert np.array_equal(beams[:, :, 0], np.repeat(tok_np[:, None], W, axis=1))
    ctx = state.float().cpu().numpy()
    worst, overlap_min, drawn_rank_max = 0.0, 1.0, 0
    for b in range(B):
        for w in range(0, W, 4):  # every fourth beam keeps the oracle's share of the test short
            s = np.zeros(H, dtype=np.float32)
            for k in range(Lb - 1):
                e = emb[beams[b, w, k]]
                s = odr.silu(e @ dwr["rnn_w.weight"].T + s @ dwr["rnn_u.weight"].T + dwr["rnn_u.bias"])
                x = np.concatenate([ctx[b], s])[None, :]
                want = odr.log_softmax(odr.compute_logits(dwr, x, R))[0]
                got = logq[b, w, k]
                kept_w, kept_g = want > -40000, got > -40000
                both = kept_w & kept_g
                overlap_min = min(overlap_min, both.sum() / max(kept_w.sum(), 1))
                worst = max(worst, float(np.abs(got[both] - want[both]).max()))
                # the token the GPU drew at this position is among the oracle's best few of that row
                drawn = beams[b, w, k + 1]
                drawn_rank_max = max(drawn_rank_max, int((want > want[drawn]).sum()))
    assert worst <= 0.1, worst  # log-probs in nats; bf16 activations through three 1024-wide layers (measured 0.068)
    assert overlap_min >= 0.85, overlap_min
    assert drawn_rank_max < W + 5, drawn_rank_max


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_vocab_topk_massive_ties(dtype):
    """Rows where thousands of entries tie at the top-k threshold (the radix-select path): the list
    holds the entries above the threshold, then ties by ascending id up to the capacity; the
    normaliser still counts every tie."""
    import recurrent_drafting as rd

    md = rd.modeling_drafter
    V, rows = 6000, 3
    logits = np.zeros((rows, V), dtype=np.float32)
    logits[0, [5, 99, 4000]] = [3.0, 2.0, 1.0]
    logits[1, :] = -1.5
    logits[2, 10:3000] = 1.0
    tl = t(logits).to(dtype)
    sp = md.vocab_topk(tl, md.new_sparse(rows, "cuda"), subtract_max=True)
    val, idx, cnt, masked = (x.cpu().numpy() for x in (sp.val, sp.idx, sp.cnt, sp.masked))
    want = odr.log_softmax(odr.warp_logits(odr.maintain_logits(logits)))
    assert cnt.tolist() == [64, 64, 64]
    assert idx[0, :3].tolist() == [5, 99, 4000] and idx[0, 3:64].tolist() == [i for i in range(64) if i != 5][:61]
    assert idx[1].tolist() == list(range(64))
    assert idx[2].tolist() == list(range(10, 74))
    for r in range(rows):
        np.testing.assert_allclose(val[r], want[r, idx[r]], rtol=1e-5, atol=2e-5)
