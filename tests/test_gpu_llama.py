"""Llama forward pieces and the whole forward against the oracle and the reference fixtures."""
import numpy as np
import pytest
import torch

import model_builders as mb
from gpu_helpers import bf16_round, build_models, t
from oracle import acceptance as oacc
from oracle import kv_cache as okv
from oracle import llama as ollama
from oracle import tree_attention as ota

pytestmark = pytest.mark.gpu


def test_rmsnorm_and_argmax():
    from recurrent_drafting import _lib

    rs = np.random.RandomState(1)
    x = rs.standard_normal((37, 200)).astype(np.float32)
    w = (1 + 0.1 * rs.standard_normal(200)).astype(np.float32)
    y = torch.empty(37, 200, device="cuda")
    tx, tw = t(x), t(w)  # keep the device buffers alive across the call
    _lib.call("rd_rmsnorm", _lib.F32, _lib.ptr(tx), _lib.ptr(tw), _lib.ptr(y), 37, None, 200, 1e-6, _lib.stream())
    np.testing.assert_allclose(y.cpu().numpy(), ollama.rms_norm(x, w, 1e-6), rtol=1e-5, atol=1e-6)
    logits = rs.standard_normal((50, 1000)).astype(np.float32)
    logits[3, 10] = logits[3, 700] = 9.0  # tie -> first index
    o32 = torch.empty(50, dtype=torch.int32, device="cuda")
    o64 = torch.empty(50, dtype=torch.int64, device="cuda")
    tl = t(logits)
    _lib.call("rd_argmax_rows", _lib.ptr(tl), 1000, 50, None, 1000, _lib.ptr(o32), _lib.ptr(o64), _lib.stream())
    assert np.array_equal(o32.cpu().numpy(), logits.argmax(-1)) and o32[3].item() == 10
    assert np.array_equal(o64.cpu().numpy(), logits.argmax(-1))


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["causal", "tree", "dense"])
def test_attention_modes(dtype, mode, hd):
    """Ragged rows with different cache offsets and lengths, GQA, all visibility modes."""
    from recurrent_drafting import _lib

    rs = np.random.RandomState(7)
    B, nh, nkv, max_len = 3, 4, 2, 420
    W, L = 45, 5
    beams = mb.zipf_beams(B, W, L, 100, 3)
    pt = ota.dedup_prefix(beams)
    unp = ota.get_unpacker(beams, pt)
    _, idx = ota.pack_beams(beams, pt)
    tree = ota.causal_mask_of_packed_beams(unp, idx)
    n_new = ota.n_selected(beams).astype(np.int32)
    kv_begin = np.array([0, 3, 1], dtype=np.int32)
    base = np.array([10, 70, 133], dtype=np.int32)
    row_start = np.concatenate([[0], np.cumsum(n_new)]).astype(np.int32)
    M = int(row_start[-1])
    q = rs.standard_normal((M, nh, hd)).astype(np.float32)
    k = rs.standard_normal((B, nkv, max_len, hd)).astype(np.float32)
    v = rs.standard_normal((B, nkv, max_len, hd)).astype(np.float32)
    tq, tk, tv = (t(x).to(dtype) for x in (q, k, v))
    q, k, v = (x.float().cpu().numpy() for x in (tq, tk, tv))
    out = torch.zeros(M, nh * hd, dtype=dtype, device="cuda")
    words = (W * L + 31) // 32
    fp = None
    if mode == "tree":
        import recurrent_drafting as rd

        fp = rd.tree_attention.pack_flat(t(beams))
    max_kv = int((base + n_new).max())
    dense = None
    if mode == "dense":
        dense_np = np.zeros((B, int(n_new.max()), max_kv), dtype=np.uint8)
        dense_np[:] = rs.randint(0, 2, size=dense_np.shape)
        dense_np[:, :, 0] = 1
        dense = t(dense_np)
    code = {"causal": _lib.ATTN_CAUSAL, "tree": _lib.ATTN_TREE, "dense": _lib.ATTN_DENSE}[mode]
    t_rs, t_begin, t_base = t(row_start), t(kv_begin), t(base)
    _lib.call("rd_attention", _lib.dtype_code(dtype), _lib.ptr(tq), _lib.ptr(tk), _lib.ptr(tv), _lib.ptr(out), _lib.ptr(t_rs),
              _lib.ptr(t_begin), _lib.ptr(t_base), B, nh, nkv, hd, max_len, int(n_new.max()), max_kv, code,
              _lib.ptr(fp.tree_mask) if fp else None, words, _lib.ptr(dense), dense.stride(1) if dense is not None else 0,
              dense.stride(0) if dense is not None else 0, _lib.stream())
    got = out.float().cpu().numpy().reshape(M, nh, hd)
    for b in range(B):
        n, s = int(n_new[b]), int(row_start[b])
        kv = int(base[b]) + n
        ks = np.repeat(k[b, :, kv_begin[b] : kv_begin[b] + kv], nh // nkv, axis=0)[None]
        vs = np.repeat(v[b, :, kv_begin[b] : kv_begin[b] + kv], nh // nkv, axis=0)[None]
        mask = np.zeros((1, n, kv), dtype=bool)
        if mode == "dense":
            mask[0] = dense_np[b, :n, :kv] != 0
        else:
            mask[0, :, : base[b]] = True
            mask[0, :, base[b] :] = np.tril(np.ones((n, n), dtype=bool)) if mode == "causal" else tree[b, :n, :n]
        want = ollama.attention(q[s : s + n].transpose(1, 0, 2)[None], ks, vs, mask)[0].transpose(1, 0, 2)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        np.testing.assert_allclose(got[s : s + n], want, rtol=tol, atol=tol)


def test_forward_reference_call_fp32(g_model):
    """LlamaForCausalLM.forward with the reference's arguments: prefill of a left-padded prompt, then
    the packed tree tokens with the dense mask of tree_attention.pack (fixtures from the reference)."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    ids = t(g_model["fw_ids"])
    B, Lp = ids.shape
    cache = rd.kv_cache.Cache(B, 64, 2, 2, 32, torch.float32, torch.device("cuda"))
    mask = rd.attention.causal_mask(ids != 0, Lp, ids.device)
    pads = rd.recurrent_drafting._count_left_paddings(ids, 0)
    pos = torch.arange(Lp, device="cuda")[None, :] - pads[:, None]
    out = llm(ids, attention_mask=mask, position_ids=pos, past_key_values=cache.sliced)
    np.testing.assert_allclose(out.hidden_states[:, -1].cpu().numpy(), g_model["fw_ctx"], rtol=2e-3, atol=2e-4)
    assert np.array_equal(out.logits[:, -1].argmax(-1).cpu().numpy(), g_model["fw_next"])
    assert cache.sliced[0][0].length == Lp
    beams = t(g_model["fw_beams"])
    packed, unp, tmask, offs = rd.tree_attention.pack(beams, (ids != 0).long())
    assert np.array_equal(packed.cpu().numpy(), g_model["fw_packed"])
    past = cache.sliced[0][0].length - pads[:, None]
    out = llm(packed, attention_mask=tmask, position_ids=past + offs, past_key_values=cache.sliced)
    n_sel = ota.n_selected(g_model["fw_beams"])
    for b in range(B):
        np.testing.assert_allclose(out.logits[b].cpu().numpy(), g_model["fw_logits"][b], rtol=2e-3, atol=5e-4)
        np.testing.assert_allclose(out.hidden_states[b, : n_sel[b]].cpu().numpy(), g_model["fw_hidden"][b, : n_sel[b]], rtol=2e-3, atol=5e-4)
    L = cache.sliced[0][0].length
    got = cache._cache[:, :, :, :, :L].cpu().numpy()
    p = pads.cpu().numpy()
    for b in range(B):
        np.testing.assert_allclose(got[:, :, b, :, p[b] :], g_model["fw_cache"][:, :, b, :, p[b] : L], rtol=2e-3, atol=1e-4)


def test_forward_bf16_tolerance(g_model):
    """bf16 logits against the fp32 oracle holding the same bf16-rounded weights:
    max abs diff <= 2e-2 of the logit scale."""
    import recurrent_drafting as rd

    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 123, dtype=torch.bfloat16)
    lwr = bf16_round(lw)
    ids_np = mb.prompts(2, 24, 1000, 5)
    ids = t(ids_np)
    cache = rd.kv_cache.Cache(2, 64, 2, 4, 64, torch.bfloat16, torch.device("cuda"))
    mask = rd.attention.causal_mask(ids != 0, 24, ids.device)
    pos = torch.arange(24, device="cuda")[None, :].expand(2, 24)
    out = llm(ids, attention_mask=mask, position_ids=pos, past_key_values=cache.sliced)
    oc = okv.Cache(2, 64, 2, 4, 64)
    want, _ = ollama.forward(lwr, mb.C1_LLAMA, ids_np, ota.padded_causal_mask(ids_np != 0, 24), pos.cpu().numpy(), oc.sliced)
    scale = np.abs(want).max()
    err = np.abs(out.logits.cpu().numpy() - want).max()
    assert err <= 2e-2 * scale, (err, scale)


def test_state_dict_round_trip():
    llm, dr, lw, dw = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    sd = llm.reference_state_dict()
    for k, v in lw.items():
        assert np.array_equal(sd[k].cpu().numpy(), v), k
    assert set(dr.state_dict().keys()) == set(dw.keys())


@pytest.mark.parametrize("mode", ["causal", "tree"])
@pytest.mark.parametrize("W,L,bases", [(45, 5, (10, 70, 133)), (8, 3, (0, 1, 64)), (64, 7, (300, 5, 129)), (64, 8, (0, 63, 200))])
def test_attention_tcgen05(mode, W, L, bases):
    """The tcgen05 attention (TMA + TMEM) against the fp32 oracle: ragged rows, several query tiles
    (n_new > 128), prefixes that end inside, at and before a key-tile boundary, GQA."""
    from recurrent_drafting import _lib

    rs = np.random.RandomState(W * 10 + L)
    B, nh, nkv, hd, max_len = 3, 4, 2, 128, 900
    beams = mb.zipf_beams(B, W, L, 5000, 7)
    pt = ota.dedup_prefix(beams)
    unp = ota.get_unpacker(beams, pt)
    _, idx = ota.pack_beams(beams, pt)
    tree = ota.causal_mask_of_packed_beams(unp, idx)
    n_new = ota.n_selected(beams).astype(np.int32)
    kv_begin = np.array([0, 3, 1], dtype=np.int32)
    base = np.array(bases, dtype=np.int32)
    row_start = np.concatenate([[0], np.cumsum(n_new)]).astype(np.int32)
    M = int(row_start[-1])
    tq = t(rs.standard_normal((M, nh * hd)).astype(np.float32)).bfloat16()
    tk = t(rs.standard_normal((B, nkv, max_len, hd)).astype(np.float32)).bfloat16()
    tv = t(rs.standard_normal((B, nkv, max_len, hd)).astype(np.float32)).bfloat16()
    q, k, v = (x.float().cpu().numpy() for x in (tq, tk, tv))
    q = q.reshape(M, nh, hd)
    out = torch.zeros(M, nh * hd, dtype=torch.bfloat16, device="cuda")
    import recurrent_drafting as rd

    fp = rd.tree_attention.pack_flat(t(beams))
    t_rs, t_begin, t_base = t(row_start), t(kv_begin), t(base)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = _lib.load()
    plan = lib.rd_attention_plan_create(_lib.ptr(tq), M, _lib.ptr(tk), _lib.ptr(tv), B, nh, nkv, hd, max_len)
    assert plan
    code = _lib.ATTN_CAUSAL if mode == "causal" else _lib.ATTN_TREE
    _lib.call("rd_attention_tc", plan, _lib.ptr(out), _lib.ptr(t_rs), _lib.ptr(t_begin), _lib.ptr(t_base), int(n_new.max()), code,
              _lib.ptr(fp.tree_mask), fp.mask_words, _lib.ptr(status), _lib.stream())
    torch.cuda.synchronize()
    lib.rd_attention_plan_destroy(plan)
    assert int(status.item()) == 0
    got = out.float().cpu().numpy().reshape(M, nh, hd)
    for b in range(B):
        n, s = int(n_new[b]), int(row_start[b])
        kv = int(base[b]) + n
        ks = np.repeat(k[b, :, kv_begin[b] : kv_begin[b] + kv], nh // nkv, axis=0)[None]
        vs = np.repeat(v[b, :, kv_begin[b] : kv_begin[b] + kv], nh // nkv, axis=0)[None]
        mask = np.zeros((1, n, kv), dtype=bool)
        mask[0, :, : base[b]] = True
        mask[0, :, base[b] :] = np.tril(np.ones((n, n), dtype=bool)) if mode == "causal" else tree[b, :n, :n]
        want = ollama.attention(q[s : s + n].transpose(1, 0, 2)[None], ks, vs, mask)[0].transpose(1, 0, 2)
        np.testing.assert_allclose(got[s : s + n], want, rtol=2e-2, atol=2e-2)


def test_forward_bf16_folded_norms_match_oracle_and_separate_kernels(monkeypatch):
    """head_dim 128 with hidden and MLP sizes that are multiples of 64: the bf16 forward applies the
    rotary embedding in the QKV epilogue and, when asked to (RD_FUSED_NORM=1), folds the norms inside the
    stack into the GEMMs around them.  Its logits must stay within the bf16 tolerance of the fp32 oracle on the same rounded
    weights and close to the forward that runs norms and rope as separate kernels."""
    import recurrent_drafting as rd
    from gpu_helpers import llama_config

    cfg = dict(mb.C1_LLAMA, num_attention_heads=2, num_key_value_heads=2, intermediate_size=704, num_hidden_layers=3)
    lw = mb.llama_weights(cfg, 77)
    ids_np = mb.prompts(2, 24, 1000, 5)
    ids = t(ids_np)
    pos = torch.arange(24, device="cuda")[None, :].expand(2, 24)
    outs = {}
    for tag, env in (("folded", {"RD_FUSED_NORM": "1"}), ("separate", {"RD_FUSED_ROPE": "0"}), ("rope_only", {})):
        for k in ("RD_FUSED_NORM", "RD_FUSED_ROPE"):
            monkeypatch.delenv(k, raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        llm = rd.modeling_llama.LlamaForCausalLM(llama_config(cfg)).to(device="cuda", dtype=torch.bfloat16)
        llm.load_state_dict({k: torch.from_numpy(v) for k, v in lw.items()})
        cache = rd.kv_cache.Cache(2, 64, 3, 2, 128, torch.bfloat16, torch.device("cuda"))
        mask = rd.attention.causal_mask(ids != 0, 24, ids.device)
        outs[tag] = llm(ids, attention_mask=mask, position_ids=pos, past_key_values=cache.sliced).logits.float().cpu().numpy()
    oc = okv.Cache(2, 64, 3, 2, 128)
    want, _ = ollama.forward(bf16_round(lw), cfg, ids_np, ota.padded_causal_mask(ids_np != 0, 24), pos.cpu().numpy(), oc.sliced)
    scale = np.abs(want).max()
    for tag, got in outs.items():
        err = np.abs(got - want).max()
        assert err <= 2e-2 * scale, (tag, err, scale)
    assert np.array_equal(outs["rope_only"], outs["separate"]), "the fused rope epilogue must not change a bit"
    assert np.abs(outs["folded"] - outs["separate"]).max() <= 2e-2 * scale
    assert not np.array_equal(outs["folded"], outs["separate"]), "the folded-norm path did not run"
