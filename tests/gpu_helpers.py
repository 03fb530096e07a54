"""Shared helpers of the GPU parity tests: model construction from the deterministic numpy weights."""
import numpy as np
import torch
from transformers.models.llama.configuration_llama import LlamaConfig

import model_builders as mb


def llama_config(cfg: dict) -> LlamaConfig:
    c = LlamaConfig(
        hidden_size=cfg["hidden_size"],
        num_attention_heads=cfg["num_attention_heads"],
        num_key_value_heads=cfg["num_key_value_heads"],
        num_hidden_layers=cfg["num_hidden_layers"],
        intermediate_size=cfg["intermediate_size"],
        vocab_size=cfg["vocab_size"],
        rms_norm_eps=cfg["rms_norm_eps"],
        hidden_act="silu",
        pad_token_id=0,
    )
    c.rope_theta = cfg["rope_theta"]
    return c


def build_models(lcfg: dict, dcfg: dict, seed: int, dtype=torch.float32, device="cuda"):
    import recurrent_drafting as rd

    lw = mb.llama_weights(lcfg, seed)
    dw = mb.drafter_weights(dcfg, seed + 1)
    llm = rd.modeling_llama.LlamaForCausalLM(llama_config(lcfg)).to(device=device, dtype=dtype)
    llm.load_state_dict({k: torch.from_numpy(v) for k, v in lw.items()})
    dr = rd.modeling_drafter.Drafter(rd.configuration_drafter.DrafterConfig(**dcfg)).to(device=device, dtype=dtype)
    dr.load_state_dict({k: torch.from_numpy(v).to(dtype) for k, v in dw.items()})
    return llm, dr, lw, dw


def bf16_round(w: dict) -> dict:
    """The weights a bf16 model actually holds, as fp32 arrays for the oracle."""
    return {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}


def t(x, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


# A small model with the headline configuration's kernel routing: bf16, head_dim 128 (tcgen05 attention,
# QKV projection with the rotary embedding in its epilogue, CTA-pair GEMMs), vocabulary 32000.
HD128_LLAMA = dict(hidden_size=512, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=2, intermediate_size=1408,
                   vocab_size=32000, rms_norm_eps=1e-6, rope_theta=10000.0)
HD128_DRAFTER = dict(vocab_size=32000, hidden_size=512, exit_dim=1024, num_draft_layers=2, rnn=True)


def hd128_step_check(batch=8, width=45, length=5, prompt_len=70, left_pads=(0, 5, 0, 17, 0, 0, 33, 2), steps=1, seed=77):
    """Prefill plus `steps` decode steps of the bf16 head_dim-128 model through RecurrentDrafting, each
    step compared with the numpy oracle holding the same bf16-rounded weights and fed the SAME beams:
      * pack outputs (unpacker, packed ids, dense mask, position offsets): bit-exact;
      * verify logits of every live packed token: max |diff| <= 2e-2 x the oracle's logit scale;
      * accepted lengths, chosen beams and commit slots: bit-exact given the GPU's own argmax tokens.
    The oracle's cache is kept in step with the GPU's accepted path, as the reference's would be.
    Returns a dict of the figures the callers assert or print."""
    import recurrent_drafting as rd
    from oracle import acceptance as oacc
    from oracle import generate as ogen
    from oracle import kv_cache as okv
    from oracle import llama as ollama
    from oracle import tree_attention as ota

    lcfg, dcfg = HD128_LLAMA, HD128_DRAFTER
    llm, dr, lw, dw = build_models(lcfg, dcfg, seed, dtype=torch.bfloat16)
    lwr = bf16_round(lw)
    B, W, L = batch, width, length
    V, H = lcfg["vocab_size"], lcfg["hidden_size"]
    prompt = mb.prompts(B, prompt_len, V, seed + 2, left_pads=list(left_pads)[:B])
    max_length = prompt_len + steps * L + 4
    model = rd.RecurrentDrafting(llm, dr)
    shape = rd.modeling_drafter.BeamShape(W, L)
    it = model.generate(rd.stats.Ledger(), t(prompt), max_length, shape, rd.SamplingArgs(1.0, True), rd.SpecialTokens(0, None))

    nh = lcfg["num_attention_heads"]
    ocache = okv.Cache(B, max_length + W * L, lcfg["num_hidden_layers"], lcfg["num_key_value_heads"], H // nh)
    octx, otok = ogen.comprehend_prompt(lwr, lcfg, prompt, ocache, True, 1.0, 0, None)
    ids = prompt
    res = {"logit_err": 0.0, "logit_scale": 0.0, "argmax_agree": 1.0, "steps": 0, "ctx_err": 0.0}
    for step in range(steps):
        out = next(it)
        st = model.last_state
        torch.cuda.synchronize()
        beams = dr._workspace(B, W, L)["beams"][(L - 1) % 2].cpu().numpy().copy()
        fp = st.fp
        n_sel = fp.n_selected.cpu().numpy()
        row_start = fp.row_start.cpu().numpy()
        M = int(row_start[-1])
        llm_tok = st.llm_tok[:M].cpu().numpy()
        # the greedy step takes its tokens in the LM head's epilogue and writes no logits: form them here from
        # the step's final hidden states with the plain LM-head GEMM (the same accumulators)
        ws = llm.workspace(B * W * L, B * W * L)
        logits = llm.lm_logits(ws["hidden"], ws["logits"], m_dev=fp.m_dev)[:M].cpu().numpy()
        # ---- pack: bit-exact against the oracle on the same beams
        pad_mask = (ids != 0).astype(np.int64)
        o_packed, o_unp, o_mask, o_offs = ota.pack(beams, pad_mask)
        assert np.array_equal(fp.unpacker.cpu().numpy(), o_unp), "unpacker differs"
        assert np.array_equal(n_sel, ota.n_selected(beams)), "n_selected differs"
        g_packed, g_unp, g_mask, g_offs = rd.tree_attention.pack(t(beams), t(pad_mask))
        assert np.array_equal(g_packed.cpu().numpy(), o_packed) and np.array_equal(g_unp.cpu().numpy(), o_unp)
        assert np.array_equal(g_mask.cpu().numpy(), o_mask) and np.array_equal(g_offs.cpu().numpy(), o_offs)
        # ---- verify forward of the oracle over the same packed tokens
        pads = oacc.count_left_paddings(ids, 0)
        past = ocache.sliced[0][0].length - pads[:, None]
        o_logits, o_hidden = ollama.forward(lwr, lcfg, o_packed, o_mask, past + o_offs, ocache.sliced)
        scale = float(np.abs(o_logits).max())
        agree, total = 0, 0
        for b in range(B):
            n, s = int(n_sel[b]), int(row_start[b])
            err = float(np.abs(logits[s : s + n] - o_logits[b, :n]).max())
            res["logit_err"] = max(res["logit_err"], err)
            agree += int((llm_tok[s : s + n] == o_logits[b, :n].argmax(-1)).sum())
            total += n
        res["logit_scale"] = scale
        res["argmax_agree"] = min(res["argmax_agree"], agree / total)
        # the GPU's argmax kernel against its own logits (first index among equals)
        assert np.array_equal(llm_tok, logits.argmax(-1)), "row argmax differs from the logits it was taken from"
        # ---- acceptance and commit, from the GPU's own LLM tokens
        by_llm = np.zeros((B, W, L), dtype=np.int64)
        for b in range(B):
            by_llm[b] = llm_tok[row_start[b] + o_unp[b]]
        n_acc, seq = oacc.greedy_choose_from_candidates(beams, by_llm)
        assert np.array_equal(st.small_host[1].numpy(), n_acc), "accepted lengths differ"
        assert np.array_equal(st.seq_in_beam.cpu().numpy(), seq), "chosen beams differ"
        plan = oacc.commit_plan(ids, n_acc, seq, o_unp, 0)
        slots = model.reference_commit_slots(shape).cpu().numpy()
        assert np.array_equal(slots[:, :, 0], plan["src_packed_slot"])
        assert np.array_equal(slots[:, :, 1], plan["src_unpacked_slot"])
        assert np.array_equal(slots[:, :, 2], plan["dst_slot"])
        # ---- advance the oracle along the same path; the yielded matrix must equal the oracle's ids + next token
        ocache.unpack(ids.shape[1], o_unp)
        ids = oacc.update_kv_cache_and_input_ids(ids, n_acc, seq, beams, ocache, 0)
        nxt = by_llm[np.arange(B), seq, n_acc]
        want_out = np.concatenate([ids, nxt[:, None]], axis=-1)
        assert np.array_equal(out.cpu().numpy(), want_out[:, : out.shape[1]]), "yielded tokens differ"
        o_h = ota.unpack(o_hidden, o_unp)[np.arange(B), seq, n_acc]
        res["ctx_err"] = max(res["ctx_err"], float(np.abs(st.ctx.float().cpu().numpy() - o_h).max() / max(np.abs(o_h).max(), 1e-6)))
        res["steps"] += 1
    it.close()
    assert int(st.status.item()) == 0
    return res
