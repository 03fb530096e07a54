"""Prefix-tree pack of draft beams (recurrent_drafting/tree_attention.py) on the B200 kernels.

pack_flat() is what the decode loop uses: rows packed back to back, per-token cache slots and RoPE
positions, and a compact bitmask instead of the dense (batch, N, S+N) mask.  pack() and unpack()
keep the reference's signatures and return its tensors bit for bit (padded rows included)."""
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib


@dataclass
class FlatPack:
    """Outputs of rd_tree_pack.  `cap` = B*W*Lb entries are allocated; row b owns
    [row_start[b], row_start[b+1]); row_start[B] (a device scalar view `m_dev`) is the total."""

    prefix_tree: torch.Tensor  # [B,W,Lb] int32
    unpacker: torch.Tensor  # [B,W,Lb] int32
    n_selected: torch.Tensor  # [B] int32
    row_start: torch.Tensor  # [B+1] int32
    tokens: torch.Tensor  # [cap] int64
    flat_index: torch.Tensor  # [cap] int32
    tok_row: torch.Tensor  # [cap] int32
    tok_pos: torch.Tensor  # [cap] int32
    tok_slot: torch.Tensor  # [cap] int32
    tree_mask: torch.Tensor  # [cap, mask_words] uint32 (stored as int32)
    base_len: torch.Tensor  # [B] int32
    mask_words: int

    @property
    def m_dev(self) -> torch.Tensor:
        return self.row_start[-1:]


def alloc_flat(B: int, W: int, Lb: int, device) -> FlatPack:
    cap = B * W * Lb
    words = (W * Lb + 31) // 32
    i32 = dict(dtype=torch.int32, device=device)
    return FlatPack(
        torch.zeros(B, W, Lb, **i32), torch.zeros(B, W, Lb, **i32), torch.zeros(B, **i32), torch.zeros(B + 1, **i32),
        torch.zeros(cap, dtype=torch.int64, device=device), torch.zeros(cap, **i32), torch.zeros(cap, **i32),
        torch.zeros(cap, **i32), torch.zeros(cap, **i32), torch.zeros(cap, words, **i32), torch.zeros(B, **i32), words,
    )


def pack_flat(beams: torch.Tensor, kv_begin: Optional[torch.Tensor] = None, kv_len: Optional[torch.Tensor] = None,
              out: Optional[FlatPack] = None) -> FlatPack:
    assert beams.dtype == torch.int64 and beams.ndim == 3 and beams.is_contiguous()
    B, W, Lb = beams.shape
    if out is None:
        out = alloc_flat(B, W, Lb, beams.device)
    _lib.call("rd_tree_pack", _lib.ptr(beams), B, W, Lb, _lib.ptr(kv_begin), _lib.ptr(kv_len), _lib.ptr(out.prefix_tree),
              _lib.ptr(out.unpacker), _lib.ptr(out.n_selected), _lib.ptr(out.row_start), _lib.ptr(out.tokens),
              _lib.ptr(out.flat_index), _lib.ptr(out.tok_row), _lib.ptr(out.tok_pos), _lib.ptr(out.tok_slot),
              _lib.ptr(out.tree_mask), out.mask_words, _lib.ptr(out.base_len), _lib.stream())
    return out


def _dedup_prefix(beams: torch.Tensor) -> torch.Tensor:
    """prefix_tree (tree_attention.py:14-38)."""
    return pack_flat(beams.contiguous()).prefix_tree.long()


def pack(beams: torch.Tensor, padding_mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Reference signature (tree_attention.py:301-338): returns packed_beams (B,N), unpacker (B,W,Lb),
    causal_mask (B,N,S+N) bool and position_offsets (B,N).  One host read-back (N), as in the reference."""
    beams = beams.contiguous()
    B, W, Lb = beams.shape
    S = padding_mask.shape[1]
    fp = pack_flat(beams)
    N = int(fp.n_selected.max().item())
    dev = beams.device
    packed = torch.empty(B, N, dtype=torch.int64, device=dev)
    indices = torch.empty(B, N, dtype=torch.int64, device=dev)
    offsets = torch.empty(B, N, dtype=torch.int64, device=dev)
    mask = torch.empty(B, N, S + N, dtype=torch.bool, device=dev)
    unpacker64 = torch.empty(B, W, Lb, dtype=torch.int64, device=dev)
    pm = padding_mask.to(torch.int64).contiguous()
    _lib.call("rd_tree_pack_reference_layout", B, W, Lb, _lib.ptr(fp.unpacker), _lib.ptr(fp.n_selected), _lib.ptr(fp.row_start),
              _lib.ptr(fp.tokens), _lib.ptr(fp.flat_index), N, _lib.ptr(pm), S, _lib.ptr(packed), _lib.ptr(indices),
              _lib.ptr(offsets), _lib.ptr(mask), _lib.ptr(unpacker64), _lib.stream())
    pack.last_packed_token_indices = indices  # kept for tests of _pack_beams parity
    return packed, unpacker64, mask, offsets


def unpack(packed_tensor: torch.Tensor, unpacker: torch.Tensor) -> torch.Tensor:
    """(B,N,D) -> (B,W,Lb,D) (tree_attention.py:341-387).  Not used by the decode loop, whose
    acceptance kernel reads packed rows through the unpacker instead of replicating them."""
    assert packed_tensor.ndim == 3
    B, W, Lb = unpacker.shape
    idx = unpacker.reshape(B, W * Lb, 1).long().expand(-1, -1, packed_tensor.shape[2])
    return torch.gather(packed_tensor, 1, idx).reshape(B, W, Lb, -1)
