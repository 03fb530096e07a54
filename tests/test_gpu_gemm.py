"""GEMM kernels (CUDA-core fp32/bf16 path and the tcgen05 bf16 path) against a plain fp32 matmul of
the same (rounded) operands, every epilogue, ragged sizes, device-side row counts."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

EPIS = ["none", "bias", "bias_silu", "bias_silu_res", "res", "swiglu"]


def _ref(a, w, bias, res, epi):
    acc = a.float() @ w.float().T
    if epi in ("bias", "bias_silu", "bias_silu_res"):
        acc = acc + bias.float()
    if epi in ("bias_silu", "bias_silu_res"):
        acc = torch.nn.functional.silu(acc)
    if epi in ("bias_silu_res", "res"):
        acc = acc + res.float()
    if epi == "swiglu":
        acc = torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]
    return acc


def _run(dtype, out_dtype, M, N, K, epi, m_live=None, tc=False):
    from recurrent_drafting import _lib
    from recurrent_drafting.modeling_llama import _Linear

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(dtype)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.1).to(dtype)
    bias = (torch.randn(N, generator=g, device="cuda") * 0.5).to(dtype)
    n_out = N // 2 if epi == "swiglu" else N
    res = (torch.randn(M, n_out, generator=g, device="cuda")).to(out_dtype)
    c = torch.full((M, n_out), 7.0, dtype=out_dtype, device="cuda")
    code = EPIS.index(epi)
    m_dev = None if m_live is None else torch.tensor([m_live], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lin = _Linear(w, bias if "bias" in epi else None)
    if tc:
        assert lin._tc_ok(a, a.stride(0))
    else:
        lin._tc_ok = lambda *_: False
    lin(a, c, code, residual=res if "res" in epi else None, m_dev=m_dev, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = _ref(a, w, bias, res, epi)
    live = M if m_live is None else min(m_live, M)
    got = c.float()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    if live > 0:
        scale = want[:live].abs().max().item() + 1e-6
        err = (got[:live] - want[:live]).abs().max().item()
        assert err <= tol * scale, (err, scale)
    if live < M:
        assert torch.all(got[live:] == 7.0), "rows beyond the live count were written"


@pytest.mark.parametrize("epi", EPIS)
def test_gemm_fp32_epilogues(epi):
    _run(torch.float32, torch.float32, 70, 130, 50, epi)


@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (64, 64, 16), (97, 250, 33), (360, 1000, 512)])
def test_gemm_fp32_shapes(M, N, K):
    _run(torch.float32, torch.float32, M, N, K, "none")
    _run(torch.float32, torch.float32, M, N, K, "res", m_live=max(1, M - 3))


def test_gemm_simt_bf16():
    _run(torch.bfloat16, torch.bfloat16, 70, 130, 50, "bias_silu_res")
    _run(torch.bfloat16, torch.float32, 70, 130, 50, "none")


@pytest.mark.parametrize("epi", EPIS)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tc_epilogues(epi, out_dtype):
    _run(torch.bfloat16, out_dtype, 300, 512, 256, epi, tc=True)


@pytest.mark.parametrize(
    "M,N,K,live",
    [
        (128, 128, 64, None),
        (1, 128, 64, None),
        (129, 200, 128, None),  # ragged M and N
        (360, 4096, 4096, None),  # BN=256 path, many k-blocks, several tiles per CTA
        (1800, 2048, 512, 921),  # device-side row count
        (1800, 2048, 512, 0),
        (400, 32000, 256, None),  # vocabulary-sized N
    ],
)
def test_gemm_tc_shapes(M, N, K, live):
    _run(torch.bfloat16, torch.bfloat16, M, N, K, "none", m_live=live, tc=True)
    _run(torch.bfloat16, torch.float32, M, N, K, "res", m_live=live, tc=True)


@pytest.mark.parametrize(
    "M,N,K,live,epi,out_dtype",
    [
        (1800, 22016, 1024, 761, "swiglu", torch.bfloat16),  # several tiles per CTA pair
        (1800, 22016, 4096, 1500, "swiglu", torch.bfloat16),  # the stage ring wraps many times
        (1800, 12288, 512, 900, "none", torch.bfloat16),
        (1800, 13000, 256, 1800, "bias_silu_res", torch.bfloat16),  # ragged last tile, second half of it empty
        (400, 40000, 128, None, "res", torch.float32),
        (1800, 32000, 256, 17, "bias", torch.float32),  # one short chunk
        (1800, 15360, 5120, 1100, "none", torch.bfloat16),  # 13B-architecture shapes: QKV,
        (1800, 27648, 5120, 900, "swiglu", torch.bfloat16),  # gate/up,
        (1800, 5120, 13824, 800, "res", torch.bfloat16),  # down projection
    ],
)
def test_gemm_tc_large_n(M, N, K, live, epi, out_dtype):
    """Large-N sizes: several tiles per CTA pair, ragged last weight tile, short token chunks."""
    _run(torch.bfloat16, out_dtype, M, N, K, epi, m_live=live, tc=True)


def test_gemm_tc_strided_output():
    """The drafter writes the recurrent state into the right half of a [M, 2H] buffer."""
    from recurrent_drafting import _lib
    from recurrent_drafting.modeling_llama import _Linear

    M, H = 90, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.randn(M, 2 * H, generator=g, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(H, 2 * H, generator=g, device="cuda") * 0.1).bfloat16()
    b = (torch.randn(H, generator=g, device="cuda") * 0.1).bfloat16()
    x = torch.zeros(M, 2 * H, dtype=torch.bfloat16, device="cuda")
    _Linear(w, b)(a, x[:, H:], _lib.EPI_BIAS_SILU)
    torch.cuda.synchronize()
    want = torch.nn.functional.silu(a.float() @ w.float().T + b.float())
    assert torch.all(x[:, :H] == 0)
    assert (x[:, H:].float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()


def test_qkv_projection_with_fused_rope_equals_projection_then_rope():
    """rd_gemm_bf16_tc_qkv_rope against rd_gemm_bf16_tc + rd_rope_kv_write on the same inputs: rotated
    Q rows, rotated K and plain V rows at the tokens' cache slots, bit for bit (GQA, ragged rows,
    a live count below the capacity, positions beyond the table clamped)."""
    from recurrent_drafting import _lib
    from recurrent_drafting.modeling_llama import _Linear, rope_tables

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(3)
    B, nh, nkv, hd, H, max_len, n_pos = 3, 8, 2, 128, 512, 300, 256
    m_max, live = 700, 613
    xn = (torch.randn(m_max, H, generator=g, device=dev) * 0.5).bfloat16()
    w = (torch.randn((nh + 2 * nkv) * hd, H, generator=g, device=dev) * 0.1).bfloat16()
    tok_row = torch.randint(0, B, (m_max,), generator=g, device=dev, dtype=torch.int32)
    tok_slot = torch.empty(m_max, dtype=torch.int32, device=dev)
    for b in range(B):  # distinct slots per row
        idx = (tok_row == b).nonzero().flatten()
        tok_slot[idx] = torch.randperm(max_len, generator=g, device=dev)[: idx.numel()].to(torch.int32)
    tok_pos = torch.randint(0, n_pos + 20, (m_max,), generator=g, device=dev, dtype=torch.int32)
    cos, sin = rope_tables(hd, n_pos, 10000.0, dev)
    m_dev = torch.tensor([live], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    lin = _Linear(w)
    # separate kernels
    qkv = torch.zeros(m_max, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, device=dev)
    q1 = torch.full((m_max, nh * hd), 5.0, dtype=torch.bfloat16, device=dev)
    k1 = torch.full((B, nkv, max_len, hd), 6.0, dtype=torch.bfloat16, device=dev)
    v1 = torch.full((B, nkv, max_len, hd), 7.0, dtype=torch.bfloat16, device=dev)
    lin(xn, qkv, _lib.EPI_NONE, m_dev=m_dev, status=status)
    _lib.call("rd_rope_kv_write", _lib.BF16, _lib.ptr(qkv), _lib.ptr(q1), _lib.ptr(k1), _lib.ptr(v1), _lib.ptr(tok_row),
              _lib.ptr(tok_pos), _lib.ptr(tok_slot), _lib.ptr(cos), _lib.ptr(sin), n_pos, m_max, _lib.ptr(m_dev), nh, nkv, hd,
              max_len, _lib.stream())
    # fused
    q2, k2, v2 = torch.full_like(q1, 5.0), torch.full_like(k1, 6.0), torch.full_like(v1, 7.0)
    lin.qkv_rope(xn, q2, k2, v2, tok_row, tok_pos, tok_slot, cos, sin, nh, nkv, hd, m_dev, m_max, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(q1, q2) and torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.all(q2[live:] == 5.0), "rows beyond the live count were written"
    assert (q2[:live] != 5.0).any() and (k2 != 6.0).any() and (v2 != 7.0).any()


@pytest.mark.parametrize("M,N,K,live", [(1800, 32000, 512, 761), (360, 32000, 256, None), (300, 1000, 128, None), (64, 320, 64, 5),
                                        (1800, 32000, 256, 0)])
def test_lm_head_with_argmax_in_the_epilogue(M, N, K, live):
    """rd_gemm_bf16_tc_argmax: the tokens equal the row arg-max of the fp32 logits the plain LM-head GEMM
    writes (same accumulators), ties included: duplicated weight rows give exactly equal logits, inside one
    32-id slice, across slices and across weight tiles, and the smaller id must win."""
    from recurrent_drafting import _lib
    from recurrent_drafting.modeling_llama import _Linear

    g = torch.Generator(device="cuda").manual_seed(N + K)
    a = (torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16()
    # a dominant direction shared by a few rows, so that the duplicates ARE the maxima of many tokens
    w[7] = w[7] * 6
    for dup in (9, 40, N - 3):
        w[dup] = w[7]
    w[N // 2] = w[N // 2] * 6
    w[N // 2 + 300 if N // 2 + 300 < N else N - 1] = w[N // 2]
    lin = _Linear(w)
    m_dev = None if live is None else torch.tensor([live], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    logits = torch.empty(M, N, dtype=torch.float32, device="cuda")
    lin(a, logits, m_dev=m_dev, status=status)
    need = _lib.load().rd_gemm_argmax_workspace_bytes(M, N)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    out = torch.full((M,), -7, dtype=torch.int32, device="cuda")
    lin.argmax(a, out, ws, m_dev, M, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    n_live = M if live is None else live
    want = logits[:n_live].cpu().numpy().argmax(axis=-1)  # numpy: first index among equals
    got = out.cpu().numpy()
    assert np.array_equal(got[:n_live], want)
    assert (got[n_live:] == -7).all(), "rows beyond the live count were written"
    if n_live >= 100:
        assert np.isin(want, [7, N // 2]).mean() > 0.2, "the planted ties never decided a row"
    # a workspace that is too small is refused on the host
    small = torch.empty(max(need // 2, 16), dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.RedrafterError):
        lin.argmax(a, out, small, m_dev, M, status)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K,live", [(360, 32000, 512, None), (1280, 32000, 256, 1000), (45, 1024, 128, None)])
def test_slice_maxima_and_sliced_topk_equal_the_plain_path(out_dtype, M, N, K, live):
    """rd_gemm_bf16_tc_slicemax writes the same matrix as the plain GEMM plus exact per-slice maxima, and
    rd_vocab_topk_sliced returns what rd_vocab_topk returns, bit for bit (tie rows included)."""
    import recurrent_drafting as rd
    from recurrent_drafting.modeling_llama import _Linear

    md = rd.modeling_drafter
    g = torch.Generator(device="cuda").manual_seed(N + K + M)
    a = (torch.randn(M, K, generator=g, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.1).bfloat16()
    w[100] = w[3]  # exactly tied columns
    w[N - 1] = w[3]
    lin = _Linear(w)
    m_dev = None if live is None else torch.tensor([live], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    plain = torch.zeros(M, N, dtype=out_dtype, device="cuda")
    lin(a, plain, m_dev=m_dev, status=status)
    fused = torch.zeros(M, N, dtype=out_dtype, device="cuda")
    smax = torch.full((N // 32, (M + 31) // 32 * 32), float("nan"), dtype=torch.float32, device="cuda")
    assert lin.with_slice_max(a, fused, smax, m_dev=m_dev, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    n_live = M if live is None else live
    assert torch.equal(plain, fused)
    want_max = fused[:n_live].float().reshape(n_live, N // 32, 32).max(dim=-1).values.T
    assert torch.equal(smax[:, :n_live], want_max)
    for subtract, temp in ((True, 1.0), (False, 0.7)):
        p0 = md.vocab_topk(plain, md.new_sparse(M, "cuda"), subtract_max=subtract, temperature=temp, rows_dev=m_dev)
        p1 = md.vocab_topk(fused, md.new_sparse(M, "cuda"), subtract_max=subtract, temperature=temp, rows_dev=m_dev, slice_max=smax)
        torch.cuda.synchronize()
        for x, y in ((p0.val, p1.val), (p0.idx, p1.idx), (p0.cnt, p1.cnt), (p0.masked, p1.masked)):
            assert torch.equal(x[:n_live], y[:n_live])


@pytest.mark.parametrize("M,live,H,K1,N2", [(900, 777, 512, 256, 1024), (300, 300, 4096, 128, 512), (64, 5, 256, 64, 256)])
def test_gemm_tc_folded_rms_norm(M, live, H, K1, N2):
    """The residual projection also emits the gamma-scaled rows and their sums of squares per 128-feature slice
    (rd_gemm_bf16_tc_res_norm); the next projection scales its accumulator rows by 1 / rms
    (rd_gemm_bf16_tc_swiglu_normed).  Together they must equal residual add -> LlamaRMSNorm -> SwiGLU projection on
    the same rounded values, and give the same bits from launch to launch (no atomics in the statistics)."""
    from recurrent_drafting import _lib
    from recurrent_drafting.modeling_llama import _Linear

    g = torch.Generator(device="cuda").manual_seed(11 + M)
    eps = 1e-6
    a = (torch.randn(M, K1, generator=g, device="cuda") * 0.5).bfloat16()
    w1 = (torch.randn(H, K1, generator=g, device="cuda") * 0.1).bfloat16()
    w2 = (torch.randn(N2, H, generator=g, device="cuda") * 0.1).bfloat16()
    gamma = (1.0 + 0.2 * torch.randn(H, generator=g, device="cuda")).bfloat16()
    h0 = torch.randn(M, H, generator=g, device="cuda").bfloat16()
    m_dev = torch.tensor([live], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    l1, l2 = _Linear(w1), _Linear(w2)
    runs = []
    for _ in range(2):
        h = h0.clone()
        x2 = torch.full((M, H), 3.0, dtype=torch.bfloat16, device="cuda")
        ss = torch.full((M, (H // 128 + 3) // 4 * 4 + 4), -1.0, dtype=torch.float32, device="cuda")
        out = torch.full((M, N2 // 2), 7.0, dtype=torch.bfloat16, device="cuda")
        l1.residual_with_norm(a, h, h, gamma, x2, ss, m_dev, M, status)
        l2.swiglu_normed(x2, out, ss, H, eps, m_dev, M, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        runs.append((h, x2, ss, out))
    h, x2, ss, out = runs[0]
    for x, y in zip(runs[0], runs[1]):
        assert torch.equal(x, y)
    h_ref = (a.float() @ w1.float().T + h0.float()).bfloat16()
    torch.testing.assert_close(h[:live].float(), h_ref[:live].float(), rtol=2e-2, atol=2e-2)
    hr = h[:live].float()  # the statistics are defined on the rounded residual stream the kernel wrote
    want_ss = (hr * hr).reshape(live, H // 128, 128).sum(-1)
    torch.testing.assert_close(ss[:live, : H // 128], want_ss, rtol=1e-5, atol=1e-5)
    assert torch.all(ss[live:] == -1.0) and torch.all(ss[:, H // 128:] == -1.0)
    assert torch.equal(x2[:live], (hr * gamma.float()).bfloat16())
    r = torch.rsqrt((hr * hr).mean(-1, keepdim=True) + eps)
    normed = gamma.float() * (hr * r).bfloat16().float()  # LlamaRMSNorm: weight * x_normalised.to(dtype)
    acc = normed.bfloat16().float() @ w2.float().T
    want = torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]
    scale = want.abs().max().item()
    err = (out[:live].float() - want).abs().max().item()
    assert err <= 2e-2 * scale, (err, scale)
    assert torch.all(out[live:] == 7.0) and torch.all(x2[live:] == 3.0)
