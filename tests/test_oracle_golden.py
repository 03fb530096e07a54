"""The numpy oracle against the reference's golden tensors and against outputs
of the reference's own PyTorch code (fixtures under tests/golden/).  CPU only."""

import numpy as np
import pytest

import model_builders as mb
from oracle import acceptance, drafter, generate, kv_cache, llama, tree_attention


def test_reference_unit_goldens_tree(g_unit):
    beams = g_unit["ta_beams"]
    pt = tree_attention.dedup_prefix(beams)
    assert np.array_equal(pt, g_unit["ta_prefix_tree"])
    unp = tree_attention.get_unpacker(beams, pt)
    assert np.array_equal(unp, g_unit["ta_unpacker"])
    packed, idx = tree_attention.pack_beams(beams, pt)
    assert np.array_equal(packed, g_unit["ta_packed_beams"])
    assert np.array_equal(idx, g_unit["ta_packed_token_indices"])
    for i in range(2):
        p, u, m, o = tree_attention.pack(beams, g_unit[f"ta_pack{i}_padding_mask"])
        assert np.array_equal(p, g_unit["ta_packed_beams"])
        assert np.array_equal(u, g_unit["ta_unpacker"])
        assert np.array_equal(m, g_unit[f"ta_pack{i}_mask"].astype(bool))
        assert np.array_equal(o, g_unit[f"ta_pack{i}_position_offsets"])
        full = tree_attention.get_causal_mask(g_unit[f"ta_full{i}_padding_mask"], unp, idx)
        assert np.array_equal(full, g_unit[f"ta_full{i}_mask"].astype(bool))


def test_reference_unit_goldens_accept_and_cache(g_unit):
    n, s = acceptance.greedy_choose_from_candidates(g_unit["acc_beams_by_drafter"], g_unit["acc_beams_by_llm"])
    assert np.array_equal(n, g_unit["acc_n_tokens_in_seq"])
    assert np.array_equal(s, g_unit["acc_seq_in_beam"])
    c = kv_cache.Cache(2, 10, 3, 2, 8)
    c._cache[:] = g_unit["kv_unpack_before"]
    c.unpack(4, np.broadcast_to(g_unit["kv_unpack_index"], (2, 2, 3)))
    assert np.array_equal(c._cache, g_unit["kv_unpack_after"])
    assert c.sliced[0][0].length == 10


def test_pack_differential(g_pack):
    for name in g_pack["pk_names"]:
        beams = g_pack[f"pk_{name}_beams"]
        pt = tree_attention.dedup_prefix(beams)
        assert np.array_equal(pt, g_pack[f"pk_{name}_prefix_tree"]), name
        p, u, m, o = tree_attention.pack(beams, g_pack[f"pk_{name}_padding_mask"])
        assert np.array_equal(p, g_pack[f"pk_{name}_packed_beams"]), name
        assert np.array_equal(u, g_pack[f"pk_{name}_unpacker"]), name
        assert np.array_equal(o, g_pack[f"pk_{name}_position_offsets"]), name
        shape = tuple(g_pack[f"pk_{name}_mask_shape"])
        ref = np.unpackbits(g_pack[f"pk_{name}_mask"], axis=-1)[..., : shape[-1]].astype(bool)
        assert m.shape == shape and np.array_equal(m, ref), name
        _, idx = tree_attention.pack_beams(beams, pt)
        assert np.array_equal(idx, g_pack[f"pk_{name}_packed_token_indices"]), name


def test_acceptance_differential(g_acc):
    n, s = acceptance.greedy_choose_from_candidates(g_acc["ga_beams"], g_acc["ga_by_llm"])
    assert np.array_equal(n, g_acc["ga_n"]) and np.array_equal(s, g_acc["ga_seq"])
    assert set(n.tolist()) >= {0, 1, 2, 4}
    n2, s2 = acceptance.choose_from_candidates(g_acc["ga_beams"], g_acc["sa_logp"], g_acc["sa_logq"], g_acc["sa_u"])
    assert np.array_equal(n2, g_acc["sa_n"]) and np.array_equal(s2, g_acc["sa_seq"])
    probs = acceptance.residual_probs(g_acc["sa_logq"], g_acc["sa_logp"], s2, n2)
    np.testing.assert_allclose(probs, g_acc["sa_probs"], rtol=1e-5, atol=1e-7)
    st = g_acc["sa_hidden"][np.arange(4), s2, n2]
    np.testing.assert_array_equal(st, g_acc["sa_state"])


def test_commit_differential(g_acc):
    before = g_acc["cm_cache_before"]
    nl, _, B, nkv, ml, hd = before.shape
    c = kv_cache.Cache(B, ml, nl, nkv, hd)
    c._cache[:] = before
    ids = g_acc["cm_input_ids"]
    beams = g_acc["ga_beams"]
    S = ids.shape[1]
    for k, v in c.sliced:
        k.length = v.length = S + beams.shape[1] * beams.shape[2]
    new_ids = acceptance.update_kv_cache_and_input_ids(ids, g_acc["ga_n"], g_acc["ga_seq"], beams, c, 0)
    assert np.array_equal(new_ids, g_acc["cm_new_input_ids"])
    S2 = int(g_acc["cm_new_length"])
    assert c.sliced[0][0].length == S2
    # every slot the next step can read must agree (slots >= S2 are dead)
    pads = acceptance.count_left_paddings(new_ids, 0)
    for b in range(B):
        np.testing.assert_array_equal(c._cache[:, :, b, :, pads[b] : S2], g_acc["cm_cache_after"][:, :, b, :, pads[b] : S2])
    np.testing.assert_array_equal(c._cache[..., :S2, :], g_acc["cm_cache_after"][..., :S2, :])


def test_commit_plan_matches_movement(g_acc):
    """The index-space plan names exactly the slots the data movement uses."""
    before = g_acc["cm_cache_before"]
    after = g_acc["cm_cache_after"]
    ids, beams = g_acc["cm_input_ids"], g_acc["ga_beams"]
    n, s = g_acc["ga_n"], g_acc["ga_seq"]
    pt = tree_attention.dedup_prefix(beams)
    unp = tree_attention.get_unpacker(beams, pt)
    plan = acceptance.commit_plan(ids, n, s, unp, 0)
    assert int(plan["new_length"]) == int(g_acc["cm_new_length"])
    for b in range(ids.shape[0]):
        for j in range(int(n[b]) + 1):
            src, dst = plan["src_unpacked_slot"][b, j], plan["dst_slot"][b, j]
            np.testing.assert_array_equal(after[:, :, b, :, dst], before[:, :, b, :, src])


def test_beam_search_differential(g_model):
    lw = mb.llama_weights(mb.NANO_LLAMA, 31)
    dw = mb.drafter_weights(mb.NANO_DRAFTER, 32)
    beams, logq = drafter.beam_search_candidates(
        dw, mb.NANO_DRAFTER["num_draft_layers"], g_model["bs_state"], g_model["bs_tok"], lw["model.embed_tokens.weight"], 5, 4
    )
    assert np.array_equal(beams, g_model["bs_beams"])
    np.testing.assert_allclose(logq, g_model["bs_logq"], rtol=1e-4, atol=1e-4)


def test_beam_search_without_recurrent_projections(g_variants):
    """The rnn=False drafter with an input projection (modeling_drafter.py:112-115, 196), fixture from the reference."""
    lw = mb.llama_weights(mb.NANO_LLAMA, 41)
    cfg = mb.NANO_DRAFTER_NO_RNN
    dw = mb.drafter_weights(cfg, 42)
    assert "rnn_u.weight" not in dw and "input_proj.weight" in dw
    beams, logq = drafter.beam_search_candidates(dw, cfg["num_draft_layers"], g_variants["nornn_state"], g_variants["nornn_tok"],
                                                 lw["model.embed_tokens.weight"], 6, 4, rnn=False)
    assert np.array_equal(beams, g_variants["nornn_beams"])
    np.testing.assert_allclose(logq, g_variants["nornn_logq"], rtol=1e-4, atol=1e-4)


def test_llama_forward_differential(g_model):
    lw = mb.llama_weights(mb.NANO_LLAMA, 31)
    dw = mb.drafter_weights(mb.NANO_DRAFTER, 32)
    cfg = mb.NANO_LLAMA
    ids = g_model["fw_ids"]
    B = ids.shape[0]
    c = kv_cache.Cache(B, 64, 2, 2, cfg["hidden_size"] // 2)
    ctx, nxt = generate.comprehend_prompt(lw, cfg, ids, c, True, 1.0, 0, None)
    np.testing.assert_allclose(ctx, g_model["fw_ctx"], rtol=1e-4, atol=1e-5)
    assert np.array_equal(nxt, g_model["fw_next"])
    beams, _ = drafter.beam_search_candidates(dw, 2, ctx, nxt, lw["model.embed_tokens.weight"], 5, 4)
    assert np.array_equal(beams, g_model["fw_beams"])
    packed, unp, mask, offs = tree_attention.pack(beams, (ids != 0).astype(np.int64))
    assert np.array_equal(packed, g_model["fw_packed"])
    past = c.sliced[0][0].length - acceptance.count_left_paddings(ids, 0)[:, None]
    logits, hidden = llama.forward(lw, cfg, packed, mask, past + offs, c.sliced)
    n_sel = tree_attention.n_selected(beams)
    for b in range(B):  # tail rows hold other rows' tokens; compare all, they are deterministic too
        np.testing.assert_allclose(logits[b], g_model["fw_logits"][b], rtol=1e-3, atol=1e-4)
        np.testing.assert_allclose(hidden[b, : n_sel[b]], g_model["fw_hidden"][b, : n_sel[b]], rtol=1e-3, atol=1e-4)
    pads = acceptance.count_left_paddings(ids, 0)
    L = c.sliced[0][0].length
    for b in range(B):
        np.testing.assert_allclose(c._cache[:, :, b, :, pads[b] : L], g_model["fw_cache"][:, :, b, :, pads[b] : L], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("tag,lcfg,dcfg,seed", [("c1", mb.C1_LLAMA, mb.C1_DRAFTER, 123), ("c1pad", mb.C1_LLAMA, mb.C1_DRAFTER, 123), ("nano", mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)])
def test_generate_greedy_stream(g_model, tag, lcfg, dcfg, seed):
    """Whole decode loop: token stream, accepted lengths and chosen beams equal
    to RecurrentDrafting.generate of the reference (fp32, greedy)."""
    B, Lp, gen, W, L = (int(x) for x in g_model[f"gen_{tag}_shape"])
    lw = mb.llama_weights(lcfg, seed)
    dw = mb.drafter_weights(dcfg, seed + 1)
    trace = []
    steps = list(
        generate.generate(lw, lcfg, dw, dcfg["num_draft_layers"], g_model[f"gen_{tag}_prompt"], Lp + gen, W, L, greedy=True, trace=trace)
    )
    assert np.array_equal(steps[-1], g_model[f"gen_{tag}_final"])
    assert [s.shape[1] for s in steps] == g_model[f"gen_{tag}_lengths"].tolist()
    assert np.array_equal(np.stack([t["n_tokens_in_seq"] for t in trace]), g_model[f"gen_{tag}_n"])
    assert np.array_equal(np.stack([t["seq_in_beam"] for t in trace]), g_model[f"gen_{tag}_seq"])
    assert np.array_equal(np.stack([t["beams"] for t in trace]), g_model[f"gen_{tag}_beams"])


def test_autoregressive_stream(g_model):
    lw = mb.llama_weights(mb.C1_LLAMA, 123)
    B, Lp, gen, W, L = (int(x) for x in g_model["gen_c1_shape"])
    steps = list(generate.autoregressive(lw, mb.C1_LLAMA, g_model["gen_c1_prompt"], Lp + gen))
    assert np.array_equal(steps[-1], g_model["gen_c1_ar_final"])
    # the reference's own invariant: greedy ReDrafter == greedy autoregression
    assert np.array_equal(steps[-1][:, : Lp + gen], g_model["gen_c1_final"][:, : Lp + gen])


def test_generate_sampling_stream(g_model):
    """Sampling loop with the randomness injected on both sides."""
    lw = mb.llama_weights(mb.NANO_LLAMA, 31)
    dw = mb.drafter_weights(mb.NANO_DRAFTER, 32)
    steps = list(
        generate.generate(
            lw, mb.NANO_LLAMA, dw, 2, g_model["gen_samp_prompt"], 30, 5, 4, greedy=False, temperature=0.7, rng=generate.UniformSource(77)
        )
    )
    assert [s.shape[1] for s in steps] == g_model["gen_samp_lengths"].tolist()
    assert np.array_equal(steps[-1], g_model["gen_samp_final"])
