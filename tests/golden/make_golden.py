"""Generate the golden fixtures under tests/golden/ from the reference itself.

Run once in a container that holds the reference checkout (read-only):

    python tests/golden/make_golden.py /path/to/ml-recurrent-drafter

It imports the reference's PyTorch implementation (CPU, fp32) and

  1. lifts the golden tensors out of the reference's own unit tests
     (tree_attention_test.py, recurrent_drafting_test.py, kv_cache_test.py docstring case);
  2. runs the reference functions of the decode step on seeded inputs and records
     inputs + outputs (differential fixtures);
  3. runs RecurrentDrafting.generate and autoregressive.generate end to end on the
     tiny BASELINE configuration with weights from tests/model_builders.py.

Two shims are needed, none touches arithmetic: a stub `jsonlines` module (the
reference imports it for its stats ledger; not installed here) and a
`rope_theta` attribute on LlamaConfig (moved by newer transformers releases).
"""

import os
import sys
import tempfile
import types
from unittest import mock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import model_builders as mb  # noqa: E402


def _install_shims(ref_root: str):
    stub = types.ModuleType("jsonlines")

    class Writer:
        def __init__(self, fp):
            self.fp = fp

        def write(self, d):
            import json

            self.fp.write(json.dumps(d) + "\n")

        def close(self):
            pass

    class Reader:
        def __init__(self, fp):
            self.fp = fp

        def __iter__(self):
            import json

            for line in self.fp:
                if line.strip():
                    yield json.loads(line)

        def close(self):
            pass

    stub.Writer, stub.Reader = Writer, Reader
    sys.modules["jsonlines"] = stub
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x))


def _np(x):
    return x.detach().cpu().numpy()


def build_ref_models(rd, llama_cfg, drafter_cfg, seed):
    from transformers.models.llama.configuration_llama import LlamaConfig

    cfg = LlamaConfig(
        hidden_size=llama_cfg["hidden_size"],
        num_attention_heads=llama_cfg["num_attention_heads"],
        num_key_value_heads=llama_cfg["num_key_value_heads"],
        num_hidden_layers=llama_cfg["num_hidden_layers"],
        intermediate_size=llama_cfg["intermediate_size"],
        vocab_size=llama_cfg["vocab_size"],
        rms_norm_eps=llama_cfg["rms_norm_eps"],
        hidden_act="silu",
        pad_token_id=0,
    )
    cfg.rope_theta = llama_cfg["rope_theta"]
    llm = rd.modeling_llama.LlamaForCausalLM(cfg)
    lw = mb.llama_weights(llama_cfg, seed)
    missing, unexpected = llm.load_state_dict({k: _t(v) for k, v in lw.items()}, strict=False)
    assert not unexpected and all("rotary_emb" in m for m in missing), (missing, unexpected)
    dcfg = rd.configuration_drafter.DrafterConfig(**drafter_cfg)
    dr = rd.modeling_drafter.Drafter(dcfg)
    dw = mb.drafter_weights(drafter_cfg, seed + 1)
    dr.load_state_dict({k: _t(v) for k, v in dw.items()}, strict=True)
    return llm.eval(), dr.eval()


def unit_test_goldens(rd, out):
    """Golden tensors the reference's unit tests hold for this path."""
    from recurrent_drafting import recurrent_drafting_test as rdt
    from recurrent_drafting import tree_attention_test as tat

    out["ta_beams"] = _np(tat.BEAMS)
    out["ta_prefix_tree"] = _np(tat.PREFIX_TREE)
    out["ta_packed_beams"] = _np(tat.PACKED_BEAMS)
    out["ta_packed_token_indices"] = _np(tat.PACKED_TOKEN_INDICES)
    out["ta_unpacker"] = _np(tat.UNPACKER)
    params = [m for m in tat.test_pack.pytestmark if m.name == "parametrize"][0].args[1]
    for i, p in enumerate(params):
        pad, mask, offs = p.values
        out[f"ta_pack{i}_padding_mask"] = _np(pad)
        out[f"ta_pack{i}_mask"] = _np(mask)
        out[f"ta_pack{i}_position_offsets"] = _np(offs)
    params = [m for m in tat.test_get_causal_mask.pytestmark if m.name == "parametrize"][0].args[1]
    for i, p in enumerate(params):
        pad, mask = p.values
        out[f"ta_full{i}_padding_mask"] = _np(pad)
        out[f"ta_full{i}_mask"] = _np(mask)
    params = [m for m in rdt.test_greedy_choose_from_candidates.pytestmark if m.name == "parametrize"][0].args[1]
    d, l, n, s = params[0].values
    out["acc_beams_by_drafter"] = _np(d).astype(np.int64)
    out["acc_beams_by_llm"] = _np(l).astype(np.int64)
    out["acc_n_tokens_in_seq"] = _np(n).astype(np.int64)
    out["acc_seq_in_beam"] = _np(s).astype(np.int64)

    # kv_cache_test.py:38-93 (docstring example of Cache.unpack), rebuilt with the reference class
    kvc = rd.kv_cache.Cache(2, 10, 3, 2, 8, torch.float32, torch.device("cpu"))
    for layer in range(3):
        for kv in range(2):
            vals = torch.tensor([0.1] * 4 + [(kv + 1) + j / 10.0 for j in range(4)])
            kvc.sliced[layer][kv].cat(vals[None, None, :, None].expand(2, 2, -1, 8))
    out["kv_unpack_before"] = _np(kvc._cache).copy()
    idx = torch.tensor([[[0, 1, 2], [0, 1, 3]]])
    kvc.unpack(4, idx)
    out["kv_unpack_index"] = _np(idx)
    out["kv_unpack_after"] = _np(kvc._cache).copy()


def pack_cases(rd, out):
    """Differential fixtures for tree_attention.pack on seeded beams."""
    ta = rd.tree_attention
    cases = [
        ("c1", 2, 4, 3, 1000, 11, None),
        ("c2", 8, 45, 5, 32000, 12, None),
        ("c3", 16, 16, 5, 32000, 13, None),
        ("w64l7", 3, 64, 7, 32000, 14, None),
        ("w8l3", 5, 8, 3, 32000, 15, [0, 3, 1, 0, 2]),
        ("ragged", 4, 6, 4, 50, 16, [2, 0, 5, 1]),
        ("allsame", 2, 5, 4, 50, 17, None),
        ("w1", 2, 1, 4, 50, 18, None),
    ]
    names = []
    for name, B, W, L, V, seed, pads in cases:
        beams = mb.zipf_beams(B, W, L, V, seed)
        if name == "allsame":
            beams[:] = beams[:, :1, :]
        S = 7
        pm = np.ones((B, S), dtype=np.int64)
        if pads is not None:
            for b, p in enumerate(pads):
                pm[b, :p] = 0
        tb = _t(beams)
        pt = ta._dedup_prefix(tb)
        packed, unp, mask, offs = ta.pack(tb, _t(pm))
        _, idx = ta._pack_beams(tb, pt)
        out[f"pk_{name}_beams"] = beams
        out[f"pk_{name}_padding_mask"] = pm
        out[f"pk_{name}_prefix_tree"] = _np(pt)
        out[f"pk_{name}_packed_beams"] = _np(packed)
        out[f"pk_{name}_packed_token_indices"] = _np(idx)
        out[f"pk_{name}_unpacker"] = _np(unp)
        out[f"pk_{name}_mask"] = np.packbits(_np(mask), axis=-1)
        out[f"pk_{name}_mask_shape"] = np.array(mask.shape)
        out[f"pk_{name}_position_offsets"] = _np(offs)
        names.append(name)
    out["pk_names"] = np.array(names)


def acceptance_cases(rd, out):
    """Differential fixtures for greedy / sampling acceptance and the commit."""
    R = rd.recurrent_drafting
    rs = np.random.RandomState(21)
    B, W, L, V = 4, 6, 5, 40
    beams = mb.zipf_beams(B, W, L, V, 22)
    by_llm = rs.randint(3, V, size=(B, W, L)).astype(np.int64)
    # plant matches so that accepted lengths cover 0..L-1
    by_llm[0, 2, : L - 1] = beams[0, 2, 1:]
    by_llm[1, 3, :2] = beams[1, 3, 1:3]
    by_llm[1, 5, :2] = beams[1, 5, 1:3]
    by_llm[2, 0, :1] = beams[2, 0, 1:2]
    n, s = R._greedy_choose_from_candidates(_t(beams), _t(by_llm))
    out["ga_beams"], out["ga_by_llm"] = beams, by_llm
    out["ga_n"], out["ga_seq"] = _np(n), _np(s)

    # sampling acceptance with recorded uniforms
    logits_p = rs.standard_normal((B, W, L, V)).astype(np.float32) * 2
    logits_q = rs.standard_normal((B, W, L - 1, V)).astype(np.float32) * 2
    logp = torch.log_softmax(_t(logits_p), dim=-1)
    logq = torch.log_softmax(_t(logits_q), dim=-1)
    u = rs.random_sample((B, W, L - 1)).astype(np.float32)
    u[3, 1, :] = 0.0  # whole beam accepted
    with mock.patch("torch.rand", lambda shape, device=None: _t(u)):
        n2, s2 = R._choose_from_candidates(_t(beams), logp, logq)
    out["sa_logp"], out["sa_logq"], out["sa_u"] = _np(logp), _np(logq), u
    out["sa_n"], out["sa_seq"] = _np(n2), _np(s2)
    hidden = rs.standard_normal((B, W, L, 8)).astype(np.float32)
    captured = {}

    class FakeCategorical:
        def __init__(self, probs=None):
            captured["probs"] = probs.clone()

        def sample(self):
            return torch.zeros(captured["probs"].shape[0], dtype=torch.long)

    with mock.patch.object(R.dist, "Categorical", FakeCategorical):
        state, _ = R._prepare_next_input(logq, logp, _t(hidden), s2, n2)
    out["sa_hidden"] = hidden
    out["sa_probs"] = _np(captured["probs"])
    out["sa_state"] = _np(state)

    # commit: reference layout, small cache, ragged left pads and accepted lengths
    nl, nkv, hd, S = 2, 2, 4, 6
    ids = mb.prompts(B, S, V, 23, left_pads=[0, 2, 1, 3])
    cache = rd.kv_cache.Cache(B, S + W * L + 4, nl, nkv, hd, torch.float32, torch.device("cpu"))
    cache._cache[:] = _t(rs.standard_normal(tuple(cache._cache.shape)).astype(np.float32))
    for k, v in cache.sliced:
        k.length = v.length = S + W * L  # state after Cache.unpack
    out["cm_cache_before"] = _np(cache._cache).copy()
    new_ids = R._update_kv_cache_and_input_ids(_t(ids), n, s, _t(beams), cache, 0)
    out["cm_input_ids"], out["cm_new_input_ids"] = ids, _np(new_ids)
    out["cm_cache_after"] = _np(cache._cache).copy()
    out["cm_new_length"] = np.int64(cache.sliced[0][0].length)


def model_cases(rd, out):
    """Drafter beam search, one Llama forward, and whole decode loops."""
    R = rd.recurrent_drafting
    llm, dr = build_ref_models(rd, mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    rs = np.random.RandomState(32)
    B, H, V = 3, mb.NANO_LLAMA["hidden_size"], mb.NANO_LLAMA["vocab_size"]
    state = rs.standard_normal((B, H)).astype(np.float32)
    tok = rs.randint(3, V, size=(B,)).astype(np.int64)
    with torch.inference_mode():
        beams, logq = dr.beam_search_candidates(_t(state), _t(tok), llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(5, 4))
    out["bs_state"], out["bs_tok"] = state, tok
    out["bs_beams"], out["bs_logq"] = _np(beams), _np(logq)

    # one verify-shaped forward: left-padded prompt in cache, then packed tree tokens
    ids = mb.prompts(B, 9, V, 33, left_pads=[0, 2, 4])
    cache = rd.kv_cache.Cache(B, 64, 2, 2, H // 2, torch.float32, torch.device("cpu"))
    with torch.inference_mode():
        ctx, nxt = R._comprehend_prompt(llm, _t(ids), cache, R.SamplingArgs(1.0, True), 0)
        out["fw_ids"], out["fw_ctx"], out["fw_next"] = ids, _np(ctx), _np(nxt)
        beams2, _ = dr.beam_search_candidates(ctx, nxt, llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(5, 4))
        packed, unp, mask, offs = rd.tree_attention.pack(beams2, (_t(ids) != 0).to(torch.long))
        past = cache.sliced[0][0].length - R._count_left_paddings(_t(ids), 0).unsqueeze(-1)
        o = llm(packed, attention_mask=mask, past_key_values=cache.sliced, position_ids=past + offs)
    out["fw_beams"] = _np(beams2)
    out["fw_packed"] = _np(packed)
    out["fw_logits"] = _np(o.logits)
    out["fw_hidden"] = _np(o.hidden_states)
    out["fw_cache"] = _np(cache._cache[:, :, :, :, : cache.sliced[0][0].length]).copy()

    # whole loops
    for tag, lcfg, dcfg, seed, B, Lp, gen, W, L, pads in [
        ("c1", mb.C1_LLAMA, mb.C1_DRAFTER, 123, 2, 32, 64, 4, 3, None),
        ("c1pad", mb.C1_LLAMA, mb.C1_DRAFTER, 123, 3, 12, 24, 4, 3, [0, 5, 2]),
        ("nano", mb.NANO_LLAMA, mb.NANO_DRAFTER, 31, 3, 10, 20, 5, 4, [1, 0, 3]),
    ]:
        llm, dr = build_ref_models(rd, lcfg, dcfg, seed)
        model = rd.recurrent_drafting.RecurrentDrafting(llm, dr)
        ids = mb.prompts(B, Lp, lcfg["vocab_size"], seed + 7, left_pads=pads)
        ledger = rd.stats.Ledger()
        acc = []
        real_choose = R._greedy_choose_from_candidates

        def spy(a, b, _real=real_choose, _acc=acc):
            n, s = _real(a, b)
            _acc.append((_np(n).copy(), _np(s).copy(), _np(a).copy()))
            return n, s

        with mock.patch.object(R, "_greedy_choose_from_candidates", spy):
            steps = [
                _np(t).copy()
                for t in model.generate(
                    ledger, _t(ids), Lp + gen, rd.modeling_drafter.BeamShape(W, L), R.SamplingArgs(1.0, True), R.SpecialTokens(0, None)
                )
            ]
        out[f"gen_{tag}_prompt"] = ids
        out[f"gen_{tag}_final"] = steps[-1]
        out[f"gen_{tag}_lengths"] = np.array([s.shape[1] for s in steps])
        out[f"gen_{tag}_n"] = np.stack([a[0] for a in acc])
        out[f"gen_{tag}_seq"] = np.stack([a[1] for a in acc])
        out[f"gen_{tag}_beams"] = np.stack([a[2] for a in acc])
        out[f"gen_{tag}_shape"] = np.array([B, Lp, gen, W, L])
        if pads is None:
            ar = [
                _np(t).copy()
                for t in rd.autoregressive.generate(model, _t(ids), Lp + gen, R.SpecialTokens(0, -1))
            ]
            out[f"gen_{tag}_ar_final"] = ar[-1]

    # sampling loop with randomness injected on both sides: torch.rand and
    # Categorical.sample are replaced by draws from one numpy stream + inverse CDF
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import acceptance as oacc
    from oracle.generate import UniformSource

    src = UniformSource(77)

    class InjCategorical:
        def __init__(self, probs=None):
            self.p = _np(probs).astype(np.float32)

        def sample(self):
            return _t(oacc.sample_inverse_cdf(self.p, src.uniform((self.p.shape[0],))))

    llm, dr = build_ref_models(rd, mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    model = rd.recurrent_drafting.RecurrentDrafting(llm, dr)
    ids = mb.prompts(3, 10, mb.NANO_LLAMA["vocab_size"], 41, left_pads=[1, 0, 3])
    with mock.patch("torch.rand", lambda shape, device=None: _t(src.uniform(tuple(shape)))), mock.patch.object(
        R.dist, "Categorical", InjCategorical
    ):
        steps = [
            _np(t).copy()
            for t in model.generate(
                rd.stats.Ledger(), _t(ids), 30, rd.modeling_drafter.BeamShape(5, 4), R.SamplingArgs(0.7, False), R.SpecialTokens(0, None)
            )
        ]
    out["gen_samp_prompt"] = ids
    out["gen_samp_final"] = steps[-1]
    out["gen_samp_lengths"] = np.array([s.shape[1] for s in steps])


def drafter_variants(rd, out):
    """Beam search of a drafter built with rnn=False and an input projection (modeling_drafter.py:112-115, 196)."""
    llm, dr = build_ref_models(rd, mb.NANO_LLAMA, mb.NANO_DRAFTER_NO_RNN, 41)
    rs = np.random.RandomState(42)
    B, H, V = 2, mb.NANO_LLAMA["hidden_size"], mb.NANO_LLAMA["vocab_size"]
    state = rs.standard_normal((B, H)).astype(np.float32)
    tok = rs.randint(3, V, size=(B,)).astype(np.int64)
    with torch.inference_mode():
        beams, logq = dr.beam_search_candidates(_t(state), _t(tok), llm.get_input_embeddings(), rd.modeling_drafter.BeamShape(6, 4))
    out["nornn_state"], out["nornn_tok"] = state, tok
    out["nornn_beams"], out["nornn_logq"] = _np(beams), _np(logq)


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of apple/ml-recurrent-drafter>")
    ref_root = sys.argv[1]
    _install_shims(ref_root)
    import recurrent_drafting as rd

    torch.manual_seed(0)
    torch.set_grad_enabled(False)
    for fn, name in [
        (unit_test_goldens, "reference_unit_tests"),
        (pack_cases, "pack_cases"),
        (acceptance_cases, "acceptance_cases"),
        (model_cases, "model_cases"),
        (drafter_variants, "drafter_variants"),
    ]:
        out = {}
        fn(rd, out)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, len(out), "arrays", os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
