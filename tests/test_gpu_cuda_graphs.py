"""Replaying the phases of a decode step from CUDA graphs changes how the kernels are launched, not what they
compute: the bf16 head_dim-128 model (tensor-core GEMMs, tcgen05 attention, fused heads) must yield the same
token matrices, accepted counts and chosen beams step by step with and without graphs, left-padded rows and a
sampling run (same generator seed on both sides) included."""
import numpy as np
import pytest
import torch

import model_builders as mb
from gpu_helpers import HD128_DRAFTER, HD128_LLAMA, build_models, t

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,width,length,greedy", [(4, 45, 5, True), (1, 8, 3, True), (3, 15, 5, False)])
def test_graph_replay_equals_eager_launches(batch, width, length, greedy):
    import recurrent_drafting as rd

    llm, dr, _, _ = build_models(HD128_LLAMA, HD128_DRAFTER, 77, dtype=torch.bfloat16)
    prompt = t(mb.prompts(batch, 40, HD128_LLAMA["vocab_size"], 5, left_pads=[0, 7, 2, 19][:batch]))
    shape = rd.modeling_drafter.BeamShape(width, length)
    runs = []
    for graphs in (False, True):
        model = rd.RecurrentDrafting(llm, dr, cuda_graphs=graphs)
        torch.manual_seed(99)  # a sampling run draws its uniforms from torch's generator, outside the graphs
        sargs = rd.SamplingArgs(1.0, True) if greedy else rd.SamplingArgs(0.7, False)
        outs, acc, seqs = [], [], []
        launches0 = rd._lib.launches
        for out in model.generate(rd.stats.Ledger(), prompt, 40 + 24, shape, sargs, rd.SpecialTokens(0, None)):
            st = model.last_state
            outs.append(out.cpu().numpy())
            acc.append(st.small_host[1].numpy().copy())
            seqs.append(st.seq_in_beam.cpu().numpy().copy())
        assert int(st.status.item()) == 0
        runs.append((outs, acc, seqs, rd._lib.launches - launches0))
    (o0, a0, s0, n0), (o1, a1, s1, n1) = runs
    assert n0 == n1 and n0 > 0  # a replay is counted as the kernels captured in it
    assert len(o0) == len(o1) and len(o0) > 4  # several steps ran after the capture
    for step in range(len(o0)):
        assert np.array_equal(o0[step], o1[step]), step
        assert np.array_equal(a0[step], a1[step]) and np.array_equal(s0[step], s1[step]), step


def test_graphs_are_not_used_where_they_do_not_apply():
    """fp32 models keep the ordinary launches even when graphs are requested."""
    import recurrent_drafting as rd

    llm, dr, _, _ = build_models(mb.NANO_LLAMA, mb.NANO_DRAFTER, 31)
    model = rd.RecurrentDrafting(llm, dr, cuda_graphs=True)
    assert not model._graphs_apply(rd.SamplingArgs(1.0, True))
    llm2, dr2, _, _ = build_models(HD128_LLAMA, HD128_DRAFTER, 77, dtype=torch.bfloat16)
    model2 = rd.RecurrentDrafting(llm2, dr2, cuda_graphs=True)
    assert model2._graphs_apply(rd.SamplingArgs(1.0, True)) and model2._graphs_apply(rd.SamplingArgs(0.8, False))
    assert not rd.RecurrentDrafting(llm2, dr2, cuda_graphs=False)._graphs_apply(rd.SamplingArgs(1.0, True))
