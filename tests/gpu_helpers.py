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
