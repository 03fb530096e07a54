"""Model-level parity of the kernels the headline configuration runs on: bf16, head_dim 128, so the
QKV projection with the rotary embedding in its epilogue, the tcgen05 attention (causal in the
prefill, prefix-tree in the verify forward) and the CTA-pair GEMMs run chained through two layers,
the 32000-wide LM head and the acceptance, and are compared with the numpy oracle holding the same
bf16-rounded weights (recurrent_drafting/recurrent_drafting.py:437-465, modeling_llama.py:255-276)."""
import pytest

from gpu_helpers import hd128_step_check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,width,length,steps", [(8, 45, 5, 2), (3, 16, 5, 1)])
def test_bf16_head_dim_128_decode_steps_against_oracle(batch, width, length, steps):
    r = hd128_step_check(batch=batch, width=width, length=length, steps=steps)
    assert r["steps"] == steps
    # stated tolerance of the bf16 path: max |logit difference| <= 2e-2 of the logit scale
    assert r["logit_err"] <= 2e-2 * r["logit_scale"], r
    assert r["ctx_err"] <= 3e-2, r
    # random-init logits are closely spaced (the best and second-best differ by less than the bf16 error
    # on some rows), so some arg-max flips against the fp32 oracle are expected; most rows must agree
    assert r["argmax_agree"] >= 0.8, r


def test_bf16_head_dim_128_decode_steps_with_folded_norms(monkeypatch):
    """The same check with the RMS norms inside the stack folded into the projections around them
    (RD_FUSED_NORM=1): same tolerances against the oracle."""
    monkeypatch.setenv("RD_FUSED_NORM", "1")
    r = hd128_step_check(batch=8, width=45, length=5, steps=2)
    assert r["steps"] == 2
    assert r["logit_err"] <= 2e-2 * r["logit_scale"], r
    assert r["ctx_err"] <= 3e-2, r
    assert r["argmax_agree"] >= 0.8, r
