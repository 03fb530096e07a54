"""Parity of the tree-verify kernels at the sizes of the isolated kernel sweep (32 heads x head_dim
128, cache lengths up to 4096, batch up to 64): pack + bitmask against the oracle, the tcgen05
tree attention against an fp32 masked softmax of the same bf16 inputs, plus size-independent
properties (mask row popcount = depth + 1; constant V rows give that constant back)."""
import numpy as np
import pytest
import torch

import model_builders as mb
from oracle import tree_attention as ota

pytestmark = pytest.mark.gpu

NH, NKV, HD = 32, 32, 128


def _attention(beams_np, S, q, k, v):
    import recurrent_drafting as rd
    from recurrent_drafting import _lib

    B, W, L = beams_np.shape
    dev = "cuda"
    beams = torch.from_numpy(beams_np).to(dev)
    kv_begin = torch.zeros(B, dtype=torch.int32, device=dev)
    kv_len = torch.full((B,), S, dtype=torch.int32, device=dev)
    fp = rd.tree_attention.pack_flat(beams, kv_begin, kv_len)
    cap = B * W * L
    out = torch.zeros(cap, NH * HD, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    plan = lib.rd_attention_plan_create(_lib.ptr(q), cap, _lib.ptr(k), _lib.ptr(v), B, NH, NKV, HD, k.shape[2])
    assert plan
    _lib.call("rd_attention_tc", plan, _lib.ptr(out), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len), W * L,
              _lib.ATTN_TREE, _lib.ptr(fp.tree_mask), fp.mask_words, _lib.ptr(status), _lib.stream())
    torch.cuda.synchronize()
    lib.rd_attention_plan_destroy(plan)
    assert int(status.item()) == 0
    return fp, out


@pytest.mark.parametrize("B,W,L,S", [(1, 8, 3, 512), (8, 45, 5, 2048), (64, 8, 3, 4096), (2, 64, 7, 4096), (8, 64, 5, 512)])
def test_pack_and_tree_attention_at_sweep_sizes(B, W, L, S):
    dev = "cuda"
    beams_np = mb.zipf_beams(B, W, L, 32000, 11 + B)
    max_len = S + W * L
    g = torch.Generator(device=dev).manual_seed(5)
    cap = B * W * L
    q = torch.randn(cap, NH * HD, device=dev, generator=g).bfloat16()
    k = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    v = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    fp, out = _attention(beams_np, S, q, k, v)

    # integer side: bit-exact against the oracle
    pt = ota.dedup_prefix(beams_np)
    unp = ota.get_unpacker(beams_np, pt)
    _, idx = ota.pack_beams(beams_np, pt)
    tree = ota.causal_mask_of_packed_beams(unp, idx)
    n_new = ota.n_selected(beams_np)
    np.testing.assert_array_equal(fp.unpacker.cpu().numpy(), unp)
    np.testing.assert_array_equal(fp.n_selected.cpu().numpy(), n_new)
    row_start = np.concatenate([[0], np.cumsum(n_new)])
    bits = fp.tree_mask.cpu().numpy().view(np.uint32)
    pos = fp.tok_pos.cpu().numpy()
    for b in range(B):
        n, s = int(n_new[b]), int(row_start[b])
        got = ((bits[s : s + n, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(n, -1)[:, :n].astype(bool)
        np.testing.assert_array_equal(got, tree[b, :n, :n])
        # every packed token sees exactly its ancestors and itself; positions continue the cached prefix
        np.testing.assert_array_equal(got.sum(axis=1), pos[s : s + n] - S + 1)

    # floating-point side: fp32 masked softmax of the same bf16 inputs
    scale = 1.0 / np.sqrt(HD)
    for b in range(B):
        n, s = int(n_new[b]), int(row_start[b])
        kv = S + n
        qq = q[s : s + n].float().view(n, NH, HD).transpose(0, 1)  # [nh, n, hd]
        kk, vv = k[b, :, :kv].float(), v[b, :, :kv].float()
        mask = torch.ones(n, kv, dtype=torch.bool, device=dev)
        mask[:, S:] = torch.from_numpy(tree[b, :n, :n]).to(dev)
        sc = torch.matmul(qq, kk.transpose(1, 2)) * scale
        sc = sc.masked_fill(~mask[None], float("-inf"))
        want = torch.matmul(torch.softmax(sc, dim=-1), vv).transpose(0, 1).reshape(n, NH * HD)
        torch.testing.assert_close(out[s : s + n].float(), want, rtol=2e-2, atol=2e-2)


def test_constant_values_come_back_unchanged():
    """softmax weights sum to one: with every V row equal to c the output is c for every query,
    whatever the mask - checked at the largest sweep cell."""
    dev = "cuda"
    B, W, L, S = 64, 64, 7, 4096
    beams_np = mb.zipf_beams(B, W, L, 32000, 3)
    max_len = S + W * L
    cap = B * W * L
    g = torch.Generator(device=dev).manual_seed(9)
    q = torch.randn(cap, NH * HD, device=dev, generator=g).bfloat16()
    k = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    c = torch.randn(NKV, 1, HD, device=dev, generator=g).bfloat16()
    v = c[None].expand(B, NKV, max_len, HD).contiguous()
    fp, out = _attention(beams_np, S, q, k, v)
    M = int(fp.row_start[-1].item())
    want = c.view(1, NKV * HD).float().expand(M, -1)
    torch.testing.assert_close(out[:M].float(), want, rtol=1e-2, atol=1e-2)


def test_tree_attention_is_repeatable_over_many_launches():
    """The softmax warps of a CTA progress independently (one may rescale the accumulator while
    another does not); hundreds of launches at the decode shape must give the same bits and never
    run into a bounded wait."""
    import recurrent_drafting as rd
    from recurrent_drafting import _lib

    dev = "cuda"
    B, W, L, S = 8, 45, 5, 500
    beams = torch.from_numpy(mb.zipf_beams(B, W, L, 32000, 21, branch=27)).to(dev)
    max_len = 1237
    cap = B * W * L
    g = torch.Generator(device=dev).manual_seed(2)
    # scores with a wide spread so that running maxima keep moving in some rows only
    q = (torch.randn(cap, NH * HD, device=dev, generator=g) * 3).bfloat16()
    k = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    v = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    kv_begin = torch.zeros(B, dtype=torch.int32, device=dev)
    kv_len = torch.full((B,), S, dtype=torch.int32, device=dev)
    fp = rd.tree_attention.pack_flat(beams, kv_begin, kv_len)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    plan = lib.rd_attention_plan_create(_lib.ptr(q), cap, _lib.ptr(k), _lib.ptr(v), B, NH, NKV, HD, max_len)
    assert plan
    outs = [torch.zeros(cap, NH * HD, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    M = int(fp.row_start[-1].item())
    mismatches = torch.zeros((), dtype=torch.int64, device=dev)
    for i in range(400):
        o = outs[0] if i == 0 else outs[1]
        _lib.call("rd_attention_tc", plan, _lib.ptr(o), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len), W * L,
                  _lib.ATTN_TREE, _lib.ptr(fp.tree_mask), fp.mask_words, _lib.ptr(status), _lib.stream())
        if i > 0:
            mismatches += (outs[1][:M] != outs[0][:M]).sum()
    torch.cuda.synchronize()
    lib.rd_attention_plan_destroy(plan)
    assert int(status.item()) == 0
    assert int(mismatches.item()) == 0


@pytest.mark.parametrize("mode", ["tree", "causal"])
@pytest.mark.parametrize("B,W,L,S,shares", [(1, 45, 5, 2048, 8), (2, 8, 3, 700, 3), (1, 64, 7, 300, 16), (3, 45, 5, 100, 4)])
def test_attention_with_shared_key_range_matches_the_single_cta_form(B, W, L, S, shares, mode):
    """rd_attention_tc_split: several CTAs share the keys of a (row, head) and a merge kernel combines
    them; also shares that get no key tile at all (more shares than tiles).  Compared with the
    unsplit kernel (tight) - which the tests above compare with the fp32 reference."""
    import recurrent_drafting as rd
    from recurrent_drafting import _lib

    dev = "cuda"
    beams = torch.from_numpy(mb.zipf_beams(B, W, L, 32000, 5 + B, branch=9)).to(dev)
    max_len = S + W * L
    cap = B * W * L
    g = torch.Generator(device=dev).manual_seed(31)
    q = torch.randn(cap, NH * HD, device=dev, generator=g).bfloat16()
    k = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    v = torch.randn(B, NKV, max_len, HD, device=dev, generator=g).bfloat16()
    kv_begin = torch.zeros(B, dtype=torch.int32, device=dev)
    kv_len = torch.full((B,), S, dtype=torch.int32, device=dev)
    fp = rd.tree_attention.pack_flat(beams, kv_begin, kv_len)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    plan = lib.rd_attention_plan_create(_lib.ptr(q), cap, _lib.ptr(k), _lib.ptr(v), B, NH, NKV, HD, max_len)
    assert plan
    code = _lib.ATTN_TREE if mode == "tree" else _lib.ATTN_CAUSAL
    one = torch.zeros(cap, NH * HD, dtype=torch.bfloat16, device=dev)
    many = torch.zeros(cap, NH * HD, dtype=torch.bfloat16, device=dev)
    _lib.call("rd_attention_tc", plan, _lib.ptr(one), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len), W * L, code,
              _lib.ptr(fp.tree_mask), fp.mask_words, _lib.ptr(status), _lib.stream())
    need = lib.rd_attention_split_workspace_bytes(cap, NH, shares)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    _lib.call("rd_attention_tc_split", plan, _lib.ptr(many), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len), W * L,
              code, _lib.ptr(fp.tree_mask), fp.mask_words, shares, _lib.ptr(ws), need, _lib.ptr(status), _lib.stream())
    with pytest.raises(_lib.RedrafterError):  # a workspace that is too small is refused on the host
        _lib.call("rd_attention_tc_split", plan, _lib.ptr(many), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len),
                  W * L, code, _lib.ptr(fp.tree_mask), fp.mask_words, shares, _lib.ptr(ws), need - 1, _lib.ptr(status), _lib.stream())
    torch.cuda.synchronize()
    lib.rd_attention_plan_destroy(plan)
    assert int(status.item()) == 0
    M = int(fp.row_start[-1].item())
    torch.testing.assert_close(many[:M].float(), one[:M].float(), rtol=2e-2, atol=1e-2)
