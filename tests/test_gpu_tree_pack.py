"""Prefix-tree pack kernels against the reference's golden tensors, the reference-generated
differential fixtures and the numpy oracle.  Bit-exact."""
import numpy as np
import pytest
import torch

import model_builders as mb
from gpu_helpers import t
from oracle import tree_attention as ota

pytestmark = pytest.mark.gpu


def _ta():
    import recurrent_drafting as rd

    return rd.tree_attention


def test_reference_unit_goldens(g_unit):
    ta = _ta()
    beams = t(g_unit["ta_beams"])
    assert np.array_equal(ta._dedup_prefix(beams).cpu().numpy(), g_unit["ta_prefix_tree"])
    for i in range(2):
        packed, unp, mask, offs = ta.pack(beams, t(g_unit[f"ta_pack{i}_padding_mask"]))
        assert np.array_equal(packed.cpu().numpy(), g_unit["ta_packed_beams"])
        assert np.array_equal(unp.cpu().numpy(), g_unit["ta_unpacker"])
        assert np.array_equal(mask.cpu().numpy(), g_unit[f"ta_pack{i}_mask"].astype(bool))
        assert np.array_equal(offs.cpu().numpy(), g_unit[f"ta_pack{i}_position_offsets"])
        assert np.array_equal(ta.pack.last_packed_token_indices.cpu().numpy(), g_unit["ta_packed_token_indices"])


def test_pack_differential(g_pack):
    ta = _ta()
    for name in g_pack["pk_names"]:
        beams = t(g_pack[f"pk_{name}_beams"])
        packed, unp, mask, offs = ta.pack(beams, t(g_pack[f"pk_{name}_padding_mask"]))
        assert np.array_equal(ta._dedup_prefix(beams).cpu().numpy(), g_pack[f"pk_{name}_prefix_tree"]), name
        assert np.array_equal(packed.cpu().numpy(), g_pack[f"pk_{name}_packed_beams"]), name
        assert np.array_equal(unp.cpu().numpy(), g_pack[f"pk_{name}_unpacker"]), name
        assert np.array_equal(offs.cpu().numpy(), g_pack[f"pk_{name}_position_offsets"]), name
        assert np.array_equal(ta.pack.last_packed_token_indices.cpu().numpy(), g_pack[f"pk_{name}_packed_token_indices"]), name
        shape = tuple(g_pack[f"pk_{name}_mask_shape"])
        ref = np.unpackbits(g_pack[f"pk_{name}_mask"], axis=-1)[..., : shape[-1]].astype(bool)
        assert tuple(mask.shape) == shape and np.array_equal(mask.cpu().numpy(), ref), name


@pytest.mark.parametrize("B,W,L", [(1, 1, 2), (2, 4, 3), (8, 45, 5), (64, 8, 3), (3, 64, 7), (33, 33, 8), (64, 64, 5)])
def test_flat_pack_vs_oracle(B, W, L):
    """Flat layout: counts, offsets, tokens, positions, cache slots and the bitmask."""
    ta = _ta()
    beams = mb.zipf_beams(B, W, L, 32000, seed=B * 1000 + W * 10 + L)
    rs = np.random.RandomState(5)
    kv_begin = rs.randint(0, 7, size=B).astype(np.int32)
    kv_len = rs.randint(1, 50, size=B).astype(np.int32)
    fp = ta.pack_flat(t(beams), t(kv_begin), t(kv_len))
    fp2 = ta.pack_flat(t(beams), t(kv_begin), t(kv_len))
    pt = ota.dedup_prefix(beams)
    unp = ota.get_unpacker(beams, pt)
    nsel = ota.n_selected(beams)
    assert np.array_equal(fp.prefix_tree.cpu().numpy(), pt)
    assert np.array_equal(fp.unpacker.cpu().numpy(), unp)
    assert np.array_equal(fp.n_selected.cpu().numpy(), nsel)
    starts = np.concatenate([[0], np.cumsum(nsel)])
    assert np.array_equal(fp.row_start.cpu().numpy(), starts)
    assert np.array_equal(fp.base_len.cpu().numpy(), kv_len)
    packed, idx = ota.pack_beams(beams, pt)
    tree = ota.causal_mask_of_packed_beams(unp, idx)
    tok = fp.tokens.cpu().numpy()
    fi = fp.flat_index.cpu().numpy()
    words = fp.tree_mask.cpu().numpy().view(np.uint32)
    for b in range(B):
        s, n = starts[b], nsel[b]
        assert np.array_equal(tok[s : s + n], packed[b, :n])
        assert np.array_equal(fi[s : s + n], idx[b, :n])
        assert np.all(fp.tok_row.cpu().numpy()[s : s + n] == b)
        assert np.array_equal(fp.tok_pos.cpu().numpy()[s : s + n], kv_len[b] + idx[b, :n] % L)
        assert np.array_equal(fp.tok_slot.cpu().numpy()[s : s + n], kv_begin[b] + kv_len[b] + np.arange(n))
        bits = np.unpackbits(words[s : s + n].view(np.uint8), axis=-1, bitorder="little")[:, : tree.shape[2]]
        assert np.array_equal(bits[:, :n].astype(bool), tree[b, :n, :n])
        assert not bits[:, n:].any()
    # the kernel is deterministic (a race would show as a difference between two runs)
    for a, b_ in [(fp.tokens, fp2.tokens), (fp.tree_mask, fp2.tree_mask), (fp.unpacker, fp2.unpacker)]:
        m = int(starts[-1])
        assert torch.equal(a[:m], b_[:m])


def test_unpack_and_cache_unpack(g_unit):
    import recurrent_drafting as rd

    ta = _ta()
    rs = np.random.RandomState(0)
    packed = rs.standard_normal((2, 5, 8)).astype(np.float32)
    unp = np.array([[[0, 1, 2], [0, 1, 3], [0, 1, 4]], [[0, 1, 2], [0, 2, 3], [0, 2, 4]]])
    out = ta.unpack(t(packed), t(unp)).cpu().numpy()
    assert np.array_equal(out, ota.unpack(packed, unp))
    # Cache.unpack on the reference's docstring example (kv_cache_test.py:38-93)
    c = rd.kv_cache.Cache(2, 10, 3, 2, 8, torch.float32, torch.device("cuda"))
    c._cache.copy_(t(g_unit["kv_unpack_before"]))
    c.unpack(4, t(g_unit["kv_unpack_index"]))
    assert np.array_equal(c._cache.cpu().numpy(), g_unit["kv_unpack_after"])
    assert c.sliced[0][0].length == 10


def test_cache_view_api():
    """kv_cache_test.py:10-35."""
    import recurrent_drafting as rd

    c = rd.kv_cache.Cache(7, 11, 3, 5, 2, torch.float32, torch.device("cuda"))
    assert c._cache.shape == (3, 2, 7, 5, 11, 2)
    assert all(c.sliced[i][j].shape == (7, 5, 0, 2) for i in range(3) for j in range(2))
    new_kv = torch.ones([7, 5, 2, 2], device="cuda")
    assert torch.all(c.sliced[0][0].cat(new_kv) == new_kv)
    assert c.sliced[0][0].length == 2
    assert torch.all(c.sliced[0][0].cat(new_kv) == torch.cat([new_kv, new_kv], dim=2))
    assert torch.all(c.sliced[0][0].slice(2) == new_kv)


def test_invalid_arguments_are_rejected_on_the_host():
    from recurrent_drafting import _lib

    ta = _ta()
    with pytest.raises(_lib.RedrafterError):
        ta.pack_flat(torch.zeros(1, 65, 2, dtype=torch.int64, device="cuda"))
    with pytest.raises(_lib.RedrafterError):
        ta.pack_flat(torch.zeros(1, 2, 9, dtype=torch.int64, device="cuda"))
