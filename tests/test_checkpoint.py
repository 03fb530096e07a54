"""Checkpoint directories (Hugging Face layout): the lazy name -> tensor reader on the CPU, and the
round trip save_pretrained -> from_pretrained of both models on the GPU."""
import json
import os

import numpy as np
import pytest
import torch

import model_builders as mb


def test_lazy_checkpoint_reads_sharded_safetensors(tmp_path):
    from safetensors.torch import save_file

    from recurrent_drafting.checkpoint import LazyCheckpoint

    a = {"x.weight": torch.arange(6, dtype=torch.float32).reshape(2, 3), "y.weight": torch.ones(4)}
    b = {"z.bias": torch.full((5,), 2.0)}
    save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    weight_map = {k: "model-00001-of-00002.safetensors" for k in a}
    weight_map.update({k: "model-00002-of-00002.safetensors" for k in b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    ck = LazyCheckpoint(str(tmp_path))
    assert sorted(ck.keys()) == ["x.weight", "y.weight", "z.bias"] and "z.bias" in ck and len(ck) == 3
    assert torch.equal(ck.pop("x.weight"), a["x.weight"])
    assert torch.equal(ck.pop("z.bias"), b["z.bias"])
    assert list(ck) == ["y.weight"]
    # without an index the shards are scanned
    os.remove(tmp_path / "model.safetensors.index.json")
    ck = LazyCheckpoint(str(tmp_path))
    assert sorted(ck.keys()) == ["x.weight", "y.weight", "z.bias"]
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        LazyCheckpoint(str(tmp_path / "empty"))


@pytest.mark.gpu
def test_models_round_trip_through_a_checkpoint_directory(tmp_path):
    import recurrent_drafting as rd
    from gpu_helpers import build_models, t

    llm, dr, lw, dw = build_models(mb.C1_LLAMA, mb.C1_DRAFTER, 9, dtype=torch.bfloat16)
    llm.save_pretrained(str(tmp_path / "llm"))
    dr.save_pretrained(str(tmp_path / "drafter"))
    llm2 = rd.modeling_llama.LlamaForCausalLM.from_pretrained(str(tmp_path / "llm"), torch_dtype=torch.bfloat16)
    dr2 = rd.modeling_drafter.Drafter.from_pretrained(str(tmp_path / "drafter"), torch_dtype=torch.bfloat16)
    sd, sd2 = llm.reference_state_dict(), llm2.reference_state_dict()
    assert sd.keys() == sd2.keys() and all(torch.equal(sd[k], sd2[k]) for k in sd)
    assert all(torch.equal(v, dr2.state_dict()[k]) for k, v in dr.state_dict().items())
    # same decode: a few greedy steps give the same tokens
    prompt = t(mb.prompts(2, 16, 1000, 3))
    outs = []
    for a, b in ((llm, dr), (llm2, dr2)):
        model = rd.RecurrentDrafting(a, b)
        it = model.generate(rd.stats.Ledger(), prompt, 16 + 12, rd.modeling_drafter.BeamShape(4, 3), rd.SamplingArgs(1.0, True),
                            rd.SpecialTokens(0, None))
        outs.append([o.cpu().numpy() for o in it][-1])
    assert np.array_equal(outs[0], outs[1])
