"""Pre-allocated KV cache with the reference's API (recurrent_drafting/kv_cache.py).

One tensor [n_layers, 2, batch, n_kv_heads, max_length, head_dim].  The reference keeps every row
right-aligned and shifts whole rows after each decode step; here a row stays where the prompt put
it and only grows: row b occupies slots [kv_begin[b], kv_begin[b] + kv_len[b]).  kv_begin / kv_len
are device int32 vectors owned by the decode loop; the View/Cache surface below keeps the
reference's scalar `length` semantics for callers that use the cache the reference's way.
"""
from typing import Tuple

import torch

from . import _lib


class View:
    """Key or value cache of one layer (kv_cache.py:10-35)."""

    def __init__(self, cache: torch.Tensor, layer: int, kv: int):
        self._cache = cache
        self._layer = layer
        self._kv = kv
        self.length = 0

    @property
    def shape(self) -> Tuple[int, int, int, int]:
        _, _, batch_size, n_heads, _, head_dim = self._cache.shape
        return (batch_size, n_heads, self.length, head_dim)

    @property
    def plane(self) -> torch.Tensor:
        """[batch, n_kv_heads, max_length, head_dim] storage of this view."""
        return self._cache[self._layer, self._kv]

    def cat(self, new_kv: torch.Tensor) -> torch.Tensor:
        _, _, batch_size, n_heads, max_length, head_dim = self._cache.shape
        n = new_kv.shape[2]
        assert new_kv.shape == (batch_size, n_heads, n, head_dim)
        assert self.length + n <= max_length
        self.plane[:, :, self.length : self.length + n, :] = new_kv
        self.length += n
        return self.plane[:, :, : self.length, :]

    def slice(self, prev: int) -> torch.Tensor:
        return self.plane[:, :, prev : self.length, :]


class Cache:
    """kv_cache.py:38-98."""

    def __init__(self, batch_size: int, max_length: int, n_layers: int, n_heads: int, head_dim: int,
                 dtype: torch.dtype, device: torch.device) -> None:
        self._cache = torch.zeros([n_layers, 2, batch_size, n_heads, max_length, head_dim], dtype=dtype, device=device)
        self.sliced = tuple((View(self._cache, layer, 0), View(self._cache, layer, 1)) for layer in range(n_layers))

    def unpack(self, prompt_length: int, tree_attn_index: torch.Tensor) -> None:
        """Replicates the packed-tree K/V into per-beam layout (kv_cache.py:58-98).  The decode loop
        of this package does not need it (its commit reads the packed slots directly)."""
        batch_size = tree_attn_index.shape[0]
        n_flat = tree_attn_index.shape[1] * tree_attn_index.shape[2]
        n_layers, _, cache_batch, n_heads, max_length, head_dim = self._cache.shape
        idx = tree_attn_index.reshape(batch_size, n_flat).to(torch.int64)
        if batch_size != cache_batch:
            idx = idx.expand(cache_batch, n_flat)
        idx = idx.contiguous()
        scratch = torch.empty([n_layers, 2, cache_batch, n_heads, n_flat, head_dim], dtype=self._cache.dtype,
                              device=self._cache.device)
        _lib.call("rd_cache_unpack", _lib.dtype_code(self._cache.dtype), _lib.ptr(self._cache), n_layers, cache_batch,
                  n_heads, max_length, head_dim, prompt_length, _lib.ptr(idx), n_flat, _lib.ptr(scratch), _lib.stream())
        for k, v in self.sliced:
            k.length = v.length = prompt_length + n_flat

    def unpack_static(self, prompt_length: int, tree_attn_index: torch.Tensor) -> None:
        """Cache.unpack for callers that must not allocate device memory (a host that owns all of the
        device's memory in its own arena, or a loop that forbids allocation after set-up): the staging
        copy lives in a fixed 16 MiB array inside the library instead of a fresh tensor.

        tree_attn_index must already be a contiguous int64 tensor of shape (cache batch, W, Lb) on the
        cache's device, so that this wrapper creates no tensor either.  Raises if the gathered rows
        (n_layers*2*batch*heads*W*Lb*head_dim elements) do not fit; calls that can overlap on the GPU
        share the array and must be ordered on one stream; make the first call per device at set-up.
        """
        n_layers, _, cache_batch, n_heads, max_length, head_dim = self._cache.shape
        idx = tree_attn_index
        assert idx.dtype == torch.int64 and idx.is_contiguous() and idx.shape[0] == cache_batch
        n_flat = idx.shape[1] * idx.shape[2]
        _lib.call("rd_cache_unpack_static", _lib.dtype_code(self._cache.dtype), _lib.ptr(self._cache), n_layers, cache_batch,
                  n_heads, max_length, head_dim, prompt_length, _lib.ptr(idx), n_flat, _lib.stream())
        for k, v in self.sliced:
            k.length = v.length = prompt_length + n_flat
