"""Acceptance + commit kernels against the reference goldens and the oracle: accepted lengths,
chosen beams, next tokens, moved K/V rows, token buffer and reference-layout slot indices."""
import numpy as np
import pytest
import torch

import model_builders as mb
from gpu_helpers import t
from oracle import acceptance as oacc
from oracle import drafter as odr
from oracle import kv_cache as okv
from oracle import tree_attention as ota

pytestmark = pytest.mark.gpu


def test_greedy_choose_reference_golden(g_unit, g_acc):
    import recurrent_drafting as rd

    R = rd.recurrent_drafting
    n, s = R._greedy_choose_from_candidates(t(g_unit["acc_beams_by_drafter"]), t(g_unit["acc_beams_by_llm"]))
    assert np.array_equal(n.cpu().numpy(), g_unit["acc_n_tokens_in_seq"])
    assert np.array_equal(s.cpu().numpy(), g_unit["acc_seq_in_beam"])
    n, s = R._greedy_choose_from_candidates(t(g_acc["ga_beams"]), t(g_acc["ga_by_llm"]))
    assert np.array_equal(n.cpu().numpy(), g_acc["ga_n"]) and np.array_equal(s.cpu().numpy(), g_acc["ga_seq"])


def _scenario(B, W, L, seed, nl=2, nkv=2, hd=8, H=16, V=60):
    rs = np.random.RandomState(seed)
    beams = mb.zipf_beams(B, W, L, V, seed)
    pt = ota.dedup_prefix(beams)
    unp = ota.get_unpacker(beams, pt)
    nsel = ota.n_selected(beams)
    starts = np.concatenate([[0], np.cumsum(nsel)]).astype(np.int32)
    kv_begin = rs.randint(0, 4, size=B).astype(np.int32)
    base = rs.randint(2, 9, size=B).astype(np.int32)
    max_len = int((kv_begin + base).max()) + W * L + 2
    cache = rs.standard_normal((nl, 2, B, nkv, max_len, hd)).astype(np.float32)
    hidden = rs.standard_normal((int(starts[-1]), H)).astype(np.float32)
    return dict(beams=beams, unp=unp, nsel=nsel, starts=starts, kv_begin=kv_begin, base=base, max_len=max_len,
                cache=cache, hidden=hidden, rs=rs, V=V)


def _to_reference_layout(sc, cache_np):
    """The reference's right-aligned cache after Cache.unpack, built from the native one."""
    B, W, L = sc["beams"].shape
    S = int(sc["base"].max())
    nl, _, _, nkv, _, hd = cache_np.shape
    ref = okv.Cache(B, S + W * L + 4, nl, nkv, hd)
    for b in range(B):
        pads = S - sc["base"][b]
        beg = sc["kv_begin"][b]
        ref._cache[:, :, b, :, pads:S] = cache_np[:, :, b, :, beg : beg + sc["base"][b]]
        src = beg + sc["base"][b] + sc["unp"][b].reshape(-1)
        ref._cache[:, :, b, :, S : S + W * L] = np.take(cache_np[:, :, b], src, axis=3)
    for k, v in ref.sliced:
        k.length = v.length = S + W * L
    return ref, S


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,W,L", [(4, 6, 5), (8, 45, 5), (2, 64, 8), (3, 1, 2)])
def test_greedy_accept_commit_vs_oracle(dtype, B, W, L):
    from recurrent_drafting import _lib

    sc = _scenario(B, W, L, seed=B + W + L)
    rs = sc["rs"]
    beams, unp, starts = sc["beams"], sc["unp"], sc["starts"]
    M = int(starts[-1])
    llm_tok = rs.randint(3, sc["V"], size=M).astype(np.int32)
    for b in range(B):  # plant accepted prefixes of varying length on some beam
        i = rs.randint(W)
        n = rs.randint(0, L)
        for k in range(n):
            llm_tok[starts[b] + unp[b, i, k]] = beams[b, i, k + 1]
    by_llm = np.stack([llm_tok[starts[b] + unp[b]] for b in range(B)]).astype(np.int64)
    want_n, want_seq = oacc.greedy_choose_from_candidates(beams, by_llm)
    cache_t = t(sc["cache"]).to(dtype)
    cache_before = cache_t.float().cpu().numpy()
    hidden_t = t(sc["hidden"]).to(dtype)
    H = hidden_t.shape[1]
    nl, _, _, nkv, max_len, hd = cache_before.shape
    i32 = dict(dtype=torch.int32, device="cuda")
    kv_len = torch.zeros(B, **i32)
    n_acc, seq = torch.zeros(B, **i32), torch.zeros(B, **i32)
    nxt = torch.zeros(B, dtype=torch.int64, device="cuda")
    ctx = torch.zeros(B, H, dtype=dtype, device="cuda")
    token_buf = torch.full((B, max_len), -7, dtype=torch.int64, device="cuda")
    # device copies are held in variables: a temporary would be freed (and its memory reused) before the launch
    d_beams, d_unp, d_starts, d_tok = t(beams), t(unp.astype(np.int32)), t(starts), t(llm_tok)
    d_begin, d_base = t(sc["kv_begin"]), t(sc["base"])
    _lib.call("rd_accept_commit_greedy", _lib.dtype_code(dtype), _lib.ptr(d_beams), B, W, L, _lib.ptr(d_unp),
              _lib.ptr(d_starts), _lib.ptr(d_tok), _lib.ptr(hidden_t), H, _lib.ptr(cache_t), nl, nkv, max_len, hd,
              _lib.ptr(d_begin), _lib.ptr(d_base), _lib.ptr(kv_len), _lib.ptr(token_buf), _lib.ptr(n_acc),
              _lib.ptr(seq), _lib.ptr(nxt), _lib.ptr(ctx), _lib.stream())
    n_np, seq_np = n_acc.cpu().numpy(), seq.cpu().numpy()
    assert np.array_equal(n_np, want_n) and np.array_equal(seq_np, want_seq)
    r = np.arange(B)
    assert np.array_equal(nxt.cpu().numpy(), by_llm[r, want_seq, want_n])
    assert np.array_equal(kv_len.cpu().numpy(), sc["base"] + want_n + 1)
    after = cache_t.float().cpu().numpy()
    tb = token_buf.cpu().numpy()
    hid = hidden_t.float().cpu().numpy()
    for b in range(B):
        beg, base, A, s = sc["kv_begin"][b], sc["base"][b], want_n[b], want_seq[b]
        for j in range(A + 1):
            np.testing.assert_array_equal(after[:, :, b, :, beg + base + j], cache_before[:, :, b, :, beg + base + unp[b, s, j]])
        np.testing.assert_array_equal(after[:, :, b, :, : beg + base], cache_before[:, :, b, :, : beg + base])
        assert np.array_equal(tb[b, beg + base : beg + base + A + 1], beams[b, s, : A + 1])
        assert np.all(tb[b, : beg + base] == -7) and np.all(tb[b, beg + base + A + 1 :] == -7)
        np.testing.assert_array_equal(ctx[b].float().cpu().numpy(), hid[starts[b] + unp[b, s, A]])
    # same data movement as the reference's update, expressed in its right-aligned layout
    ref, S = _to_reference_layout(sc, cache_before)
    ids = np.zeros((B, S), dtype=np.int64)
    for b in range(B):
        ids[b, S - sc["base"][b] :] = 5  # non-pad history
    new_ids = oacc.update_kv_cache_and_input_ids(ids, want_n, want_seq, beams, ref, 0)
    S2 = new_ids.shape[1]
    for b in range(B):
        new_len = sc["base"][b] + want_n[b] + 1
        np.testing.assert_array_equal(ref._cache[:, :, b, :, S2 - new_len : S2], after[:, :, b, :, sc["kv_begin"][b] : sc["kv_begin"][b] + new_len])
    # reference-layout slot indices
    plan = oacc.commit_plan(ids, want_n, want_seq, unp, 0)
    slots = torch.zeros(B, L, 3, dtype=torch.int64, device="cuda")
    _lib.call("rd_commit_reference_slots", B, W, L, _lib.ptr(d_unp), _lib.ptr(n_acc), _lib.ptr(seq), S, S2,
              _lib.ptr(slots), _lib.stream())
    sl = slots.cpu().numpy()
    assert np.array_equal(sl[:, :, 0], plan["src_packed_slot"])
    assert np.array_equal(sl[:, :, 1], plan["src_unpacked_slot"])
    assert np.array_equal(sl[:, :, 2], plan["dst_slot"])


@pytest.mark.parametrize("B,W,L,V", [(4, 6, 5, 300), (16, 16, 5, 32000)])
@pytest.mark.parametrize("temp", [1.0, 0.6])
def test_sampling_accept_vs_oracle(temp, B, W, L, V):
    """Speculative-sampling acceptance, residual resampling and commit against the oracle with the
    same injected uniforms; the second shape is the sampling benchmark's (batch 16, 16 beams of 5,
    vocabulary 32000: recurrent_drafting.py:499-556, 271-343)."""
    import recurrent_drafting as rd
    from recurrent_drafting import _lib

    md = rd.modeling_drafter
    sc = _scenario(B, W, L, seed=11, V=V)
    rs = sc["rs"]
    beams, unp, starts = sc["beams"], sc["unp"], sc["starts"]
    M = int(starts[-1])
    # verify logits per flat token; make the drafted continuation likely so that prefixes get accepted
    logits_p = (rs.standard_normal((M, V)) * 2).astype(np.float32)
    logits_q = (rs.standard_normal((L - 1, B * W, V)) * 2).astype(np.float32)
    for b in range(B):
        for i in range(W):
            for k in range(L - 1):
                logits_q[k, b * W + i, beams[b, i, k + 1]] += 5.0
    for b in range(B):  # the verifier agrees strongly, weakly or not at all with each tree node
        for slot in range(int(sc["nsel"][b])):
            i, k = np.argwhere(unp[b] == slot)[0]
            if k + 1 < L:
                logits_p[starts[b] + slot, beams[b, i, k + 1]] += rs.choice([0.0, 3.0, 7.0])
    anc = np.broadcast_to(np.arange(W, dtype=np.int32)[None, :, None], (B, W, L - 1)).copy()
    d_lp = t(logits_p)
    d_lq = [t(logits_q[k]) for k in range(L - 1)]
    p = md.vocab_topk(d_lp, md.new_sparse(M, "cuda"), subtract_max=False, temperature=temp)
    q = [md.vocab_topk(d_lq[k], md.new_sparse(B * W, "cuda"), subtract_max=True) for k in range(L - 1)]
    logp_flat = odr.log_softmax(odr.warp_logits(logits_p) / np.float32(temp))
    logp = np.stack([logp_flat[starts[b] + unp[b]] for b in range(B)])  # (B,W,L,V)
    logq = np.stack([odr.log_softmax(odr.warp_logits(odr.maintain_logits(logits_q[k]))).reshape(B, W, V) for k in range(L - 1)], axis=2)
    u = rs.random_sample((B, W, L - 1)).astype(np.float32)
    u[1] = 1.0  # row 1 accepts only where P >= Q
    u_next = rs.random_sample(B).astype(np.float32)
    want_n, want_seq = oacc.choose_from_candidates(beams, logp, logq, u)
    assert len(set(want_n.tolist())) >= 2, want_n
    want_probs = oacc.residual_probs(logq, logp, want_seq, want_n)
    want_next = oacc.sample_inverse_cdf(want_probs, u_next)
    i32 = dict(dtype=torch.int32, device="cuda")
    n_acc, seq, kv_len = torch.zeros(B, **i32), torch.zeros(B, **i32), torch.zeros(B, **i32)
    nxt = torch.zeros(B, dtype=torch.int64, device="cuda")
    probs = torch.zeros(B, V, device="cuda")
    cache_t = t(sc["cache"])
    hidden_t = t(sc["hidden"])
    H = hidden_t.shape[1]
    ctx = torch.zeros(B, H, device="cuda")
    nl, _, _, nkv, max_len, hd = sc["cache"].shape
    token_buf = torch.zeros(B, max_len, dtype=torch.int64, device="cuda")
    d_beams, d_unp, d_starts, d_anc, d_u, d_un = t(beams), t(unp.astype(np.int32)), t(starts), t(anc), t(u), t(u_next)
    d_begin, d_base = t(sc["kv_begin"]), t(sc["base"])
    _lib.call("rd_accept_commit_sample", _lib.F32, _lib.ptr(d_beams), B, W, L, V, _lib.ptr(d_unp),
              _lib.ptr(d_starts), _lib.ptr(p.val), _lib.ptr(p.idx), _lib.ptr(p.cnt), _lib.ptr(p.masked),
              _lib.ptr_array([x.val for x in q]), _lib.ptr_array([x.idx for x in q]), _lib.ptr_array([x.cnt for x in q]),
              _lib.ptr_array([x.masked for x in q]), _lib.ptr(d_anc), _lib.ptr(d_u), _lib.ptr(d_un), _lib.ptr(hidden_t), H,
              _lib.ptr(cache_t), nl, nkv, max_len, hd, _lib.ptr(d_begin), _lib.ptr(d_base), _lib.ptr(kv_len),
              _lib.ptr(token_buf), _lib.ptr(n_acc), _lib.ptr(seq), _lib.ptr(nxt), _lib.ptr(ctx), _lib.ptr(probs), _lib.stream())
    assert np.array_equal(n_acc.cpu().numpy(), want_n) and np.array_equal(seq.cpu().numpy(), want_seq)
    np.testing.assert_allclose(probs.cpu().numpy(), want_probs, rtol=2e-4, atol=1e-6)
    assert np.array_equal(nxt.cpu().numpy(), want_next)
    after = cache_t.cpu().numpy()
    for b in range(B):
        beg, base = sc["kv_begin"][b], sc["base"][b]
        for j in range(want_n[b] + 1):
            np.testing.assert_array_equal(after[:, :, b, :, beg + base + j], sc["cache"][:, :, b, :, beg + base + unp[b, want_seq[b], j]])
