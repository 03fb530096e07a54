"""Oracle (numpy) for the prefix-tree pack of draft beams.  Test infrastructure only.

Restates recurrent_drafting/tree_attention.py of the reference from the
definitions of its outputs rather than from its vectorised tensor tricks.
All arrays are int64 unless stated otherwise.
"""

from typing import Tuple

import numpy as np


def dedup_prefix(beams: np.ndarray) -> np.ndarray:
    """prefix_tree[b,i,j] = smallest k with beams[b,k,:j+1] == beams[b,i,:j+1].

    Reference: tree_attention.py:14-38 (_dedup_prefix; first-max argmax over the
    candidate axis gives the smallest matching candidate index).
    """
    B, W, L = beams.shape
    out = np.zeros((B, W, L), dtype=np.int64)
    for b in range(B):
        # eq[i,k,j] true iff the first j+1 tokens of beams i and k agree
        same_tok = beams[b, :, None, :] == beams[b, None, :, :]
        eq = np.logical_and.accumulate(same_tok, axis=2)
        for j in range(L):
            out[b, :, j] = np.argmax(eq[:, :, j], axis=1)  # first True
    return out


def own_node_mask(prefix_tree: np.ndarray) -> np.ndarray:
    """own[b,i,j] true iff beam i is the first beam holding prefix (i, j): the
    token is a node of the prefix tree contributed by beam i.

    Reference: tree_attention.py:72-73 and :144-145 (pack_mask).
    """
    W = prefix_tree.shape[1]
    return prefix_tree == np.arange(W, dtype=np.int64)[None, :, None]


def get_unpacker(beams: np.ndarray, prefix_tree: np.ndarray) -> np.ndarray:
    """unpacker[b,i,j] = slot of token (i,j) in the row's packed token list, so
    that packed_beams[b, unpacker[b,i,j]] == beams[b,i,j].

    The packed list holds, beam after beam, the nodes each beam owns.  A token's
    slot is the start of the owning beam's segment plus the number of earlier
    tokens of the same beam that fall in the same segment.

    Reference: tree_attention.py:125-188 (_get_unpacker).
    """
    B, W, L = beams.shape
    own = own_node_mask(prefix_tree)
    n_own = own.sum(axis=2)
    start = np.cumsum(n_own, axis=1) - n_own  # exclusive scan over beams
    out = np.zeros((B, W, L), dtype=np.int64)
    for b in range(B):
        seg = start[b][prefix_tree[b]]  # (W, L) segment start of every token
        for j in range(L):
            earlier_same = (seg[:, :j] == seg[:, j : j + 1]).sum(axis=1)
            out[b, :, j] = seg[:, j] + earlier_same
    return out


def pack_beams(beams: np.ndarray, prefix_tree: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Row-major compaction of the owned nodes of every batch row.

    Returns (packed_beams, packed_token_indices), both (B, N) with
    N = max_b n_selected[b].  A row with fewer than N nodes is filled from the
    selections of the FOLLOWING rows (the reference gathers from one flat list
    of all rows' selections) and the read index is clamped to the last
    selected element of the whole batch.

    Reference: tree_attention.py:41-122 (_pack_beams), tail behaviour :95-120;
    golden: tree_attention_test.py:26-38.
    """
    B, W, L = beams.shape
    own = own_node_mask(prefix_tree).reshape(B, W * L)
    flat = beams.reshape(B, W * L)
    sel_tok = []
    sel_idx = []
    n_sel = np.zeros(B, dtype=np.int64)
    for b in range(B):
        idx = np.nonzero(own[b])[0]
        sel_idx.append(idx)
        sel_tok.append(flat[b, idx])
        n_sel[b] = idx.size
    all_tok = np.concatenate(sel_tok)
    all_idx = np.concatenate(sel_idx).astype(np.int64)
    N = int(n_sel.max())
    starts = np.cumsum(n_sel) - n_sel
    read = np.minimum(starts[:, None] + np.arange(N, dtype=np.int64)[None, :], all_tok.size - 1)
    return all_tok[read], all_idx[read]


def causal_mask_of_packed_beams(unpacker: np.ndarray, packed_token_indices: np.ndarray) -> np.ndarray:
    """mask[b,p,q] true iff packed token p may attend packed token q.

    Packed token p stands for flat beam index t = packed_token_indices[b,p],
    i.e. beam m = t // L, position k = t % L; it attends the packed slots of
    (m, 0..k), which are unpacker[b, m, 0..k].

    Reference: tree_attention.py:191-250.
    """
    B, W, L = unpacker.shape
    N = packed_token_indices.shape[1]
    mask = np.zeros((B, N, N), dtype=bool)
    for b in range(B):
        for p in range(N):
            t = int(packed_token_indices[b, p])
            m, k = divmod(t, L)
            # the reference scatters False for positions > k as well; those
            # writes can only land on slots unpacker[b,m,k+1:], which differ
            # from unpacker[b,m,:k+1] (slots of one beam are strictly increasing)
            mask[b, p, unpacker[b, m, : k + 1]] = True
    return mask


def padded_causal_mask(padding_mask: np.ndarray, query_len: int) -> np.ndarray:
    """(B, query_len, kv_len) lower-triangular mask with padded key columns off.

    Reference: attention.py:12-55 (causal_mask).
    """
    B, kv = padding_mask.shape
    tri = np.tril(np.ones((kv, kv), dtype=bool))
    m = np.broadcast_to(tri[None], (B, kv, kv)).copy()
    m &= (padding_mask != 0)[:, None, :]
    return m[:, kv - query_len :, :]


def get_causal_mask(padding_mask: np.ndarray, unpacker: np.ndarray, packed_token_indices: np.ndarray) -> np.ndarray:
    """Full (B, S+N, S+N) mask: causal + padding over the processed sequence,
    tree mask in the lower-right block.  Reference: tree_attention.py:253-298."""
    B, N = packed_token_indices.shape
    S = padding_mask.shape[1]
    ext = np.concatenate([padding_mask != 0, np.ones((B, N), dtype=bool)], axis=1)
    m = padded_causal_mask(ext, S + N)
    m[:, S:, S:] = causal_mask_of_packed_beams(unpacker, packed_token_indices)
    return m


def pack(beams: np.ndarray, padding_mask: np.ndarray):
    """Returns (packed_beams, unpacker, causal_mask (B,N,S+N) bool, position_offsets).

    Reference: tree_attention.py:301-338 (pack).
    """
    L = beams.shape[2]
    pt = dedup_prefix(beams)
    unpacker = get_unpacker(beams, pt)
    packed, idx = pack_beams(beams, pt)
    m = get_causal_mask(padding_mask, unpacker, idx)
    return packed, unpacker, m[:, -packed.shape[1] :, :], idx % L


def n_selected(beams: np.ndarray) -> np.ndarray:
    """Number of prefix-tree nodes of every batch row (the row's own packed length)."""
    B = beams.shape[0]
    return own_node_mask(dedup_prefix(beams)).reshape(B, -1).sum(axis=1)


def unpack(packed: np.ndarray, unpacker: np.ndarray) -> np.ndarray:
    """(B,N,D) -> (B,W,L,D) by unpacker.  Reference: tree_attention.py:341-387."""
    B, W, L = unpacker.shape
    out = np.take_along_axis(packed, unpacker.reshape(B, W * L, 1), axis=1)
    return out.reshape(B, W, L, packed.shape[2])
