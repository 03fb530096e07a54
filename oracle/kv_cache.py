"""Oracle (numpy) of the reference's pre-allocated KV cache.  Test infrastructure only.

Restates recurrent_drafting/kv_cache.py: one array
[n_layers, 2, batch, n_kv_heads, max_length, head_dim]; every (layer, k|v) view
has its own current length; rows are right-aligned (left-padded) by the caller.
"""

import numpy as np


class View:
    """Reference: kv_cache.py:10-35."""

    def __init__(self, cache: np.ndarray, layer: int, kv: int):
        self._cache, self._layer, self._kv = cache, layer, kv
        self.length = 0

    @property
    def shape(self):
        _, _, B, nh, _, hd = self._cache.shape
        return (B, nh, self.length, hd)

    def cat(self, new_kv: np.ndarray) -> np.ndarray:
        _, _, B, nh, max_len, hd = self._cache.shape
        n = new_kv.shape[2]
        assert new_kv.shape == (B, nh, n, hd)
        assert self.length + n <= max_len
        self._cache[self._layer, self._kv, :, :, self.length : self.length + n, :] = new_kv
        self.length += n
        return self._cache[self._layer, self._kv, :, :, : self.length, :]

    def slice(self, prev: int) -> np.ndarray:
        return self._cache[self._layer, self._kv, :, :, prev : self.length, :]


class Cache:
    """Reference: kv_cache.py:38-98."""

    def __init__(self, batch_size, max_length, n_layers, n_heads, head_dim, dtype=np.float32):
        self._cache = np.zeros([n_layers, 2, batch_size, n_heads, max_length, head_dim], dtype=dtype)
        self.sliced = tuple((View(self._cache, l, 0), View(self._cache, l, 1)) for l in range(n_layers))

    def unpack(self, prompt_length: int, unpacker: np.ndarray) -> None:
        """cache[..., S + flat(i,j), :] <- cache[..., S + unpacker[b,i,j], :] for
        every (i,j), reading the pre-call contents.  Reference: kv_cache.py:58-98."""
        B, W, L = unpacker.shape
        n = W * L
        src = prompt_length + unpacker.reshape(B, n)
        snap = self._cache.copy()
        for b in range(B):
            self._cache[:, :, b, :, prompt_length : prompt_length + n, :] = np.take(snap[:, :, b], src[b], axis=3)
        for k, v in self.sliced:
            k.length = v.length = prompt_length + n
