"""The environment switches of the library change how kernels are launched or fused, never what
they compute: a bf16 decode loop (head_dim 128, so the tcgen05 GEMM and attention are on the path)
must emit the same tokens with programmatic dependent launches and with ordinary launches, and with
the rotary embedding fused into the QKV projection or as a kernel of its own, and with the arg-max / slice
maxima in the LM-head and vocabulary-head epilogues or as separate passes over the logits.  The switches are read
once per process, so every setting runs in a child process (run as a script, this file is that child)."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
LLAMA = dict(hidden_size=256, num_attention_heads=2, num_key_value_heads=2, num_hidden_layers=2, intermediate_size=512,
             vocab_size=1024, rms_norm_eps=1e-5, rope_theta=10000.0)  # a multiple of 32: the fused heads apply
DRAFTER = dict(vocab_size=1024, hidden_size=256, exit_dim=512, num_draft_layers=1, rnn=True)


def _child() -> None:
    sys.path[:0] = [os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), "ml-recurrent-drafter_b200"), HERE]
    import torch

    import model_builders as mb
    import recurrent_drafting as rd
    from gpu_helpers import build_models, t

    llm, dr, _, _ = build_models(LLAMA, DRAFTER, 77, dtype=torch.bfloat16)
    model = rd.RecurrentDrafting(llm, dr)
    prompt = t(mb.prompts(3, 40, 1000, 5, left_pads=[0, 7, 2]))
    outs = list(model.generate(rd.stats.Ledger(), prompt, 96, rd.modeling_drafter.BeamShape(6, 4), rd.SamplingArgs(1.0, True),
                               rd.SpecialTokens(0, None)))
    print("TOKENS " + json.dumps(outs[-1].cpu().tolist()))


def _run(env_extra):
    env = dict(os.environ)
    for k in ("RD_PDL", "RD_FUSED_ROPE", "RD_GEMM_PAIRS", "RD_FUSED_HEAD", "RD_CUDA_GRAPHS", "RD_FUSED_NORM"):
        env.pop(k, None)
    env.update(env_extra)
    r = subprocess.run([sys.executable, os.path.abspath(__file__)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("TOKENS ")][-1]
    return json.loads(line[len("TOKENS "):])


@pytest.mark.gpu
def test_launch_and_fusion_switches_do_not_change_the_tokens():
    base = _run({})
    assert len(base) == 3 and all(len(row) == 96 for row in base)
    for setting in ({"RD_PDL": "0"}, {"RD_FUSED_ROPE": "0"}, {"RD_GEMM_PAIRS": "0"}, {"RD_FUSED_HEAD": "0"},
                    {"RD_CUDA_GRAPHS": "0"}):
        assert _run(setting) == base, setting
    # the folded RMS norms (RD_FUSED_NORM=1) round differently (once instead of twice before the projection), so they
    # are compared among themselves: how the kernels are launched must not matter
    on = {"RD_FUSED_NORM": "1"}
    folded = _run(on)
    assert len(folded) == 3 and all(len(row) == 96 for row in folded)
    for setting in ({"RD_GEMM_PAIRS": "0"}, {"RD_CUDA_GRAPHS": "0"}):
        assert _run(dict(on, **setting)) == folded, setting


if __name__ == "__main__":
    _child()
