"""The allocation-free variant of the cache unpack (rd_cache_unpack_static) against the regular
entry point (rd_cache_unpack).  Collected last on purpose: a failure here must not hide any other
test from a run that stops at the first failure.

The variant exists for hosts that cannot let a library allocate device memory - all memory already
sits in the host's own arena, or allocation is banned after start-up because it stalls the device.
It keeps its staging copy in a fixed array inside the library, so the checks below also cover what
that implies: the array is shared by all calls and keeps the previous call's bytes, and a request
that does not fit is refused."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, dtype, NL=3, B=2, nkv=2, max_len=40, hd=16, S=5, W=4, Lb=3):
    g = torch.Generator(device="cuda").manual_seed(seed)
    cache = torch.randn(NL, 2, B, nkv, max_len, hd, generator=g, device="cuda").to(dtype)
    n_packed = 7
    idx = torch.randint(0, n_packed, (B, W, Lb), generator=g, device="cuda", dtype=torch.int64)
    return cache, idx, (NL, B, nkv, max_len, hd, S, W * Lb)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_variant_matches_regular_entry_point_twice(dtype):
    from recurrent_drafting import _lib

    code = _lib.dtype_code(dtype)
    # two calls in a row with different contents and sizes: the second one finds the first one's
    # bytes in the shared array and must not be affected by them
    for seed, kw in [(1, {}), (2, dict(NL=2, B=3, nkv=1, hd=32, S=9, W=5, Lb=4, max_len=64))]:
        cache, idx, (NL, B, nkv, max_len, hd, S, n_flat) = _case(seed, dtype, **kw)
        want = cache.clone()
        scratch = torch.empty(NL * 2 * B * nkv * n_flat * hd, dtype=dtype, device="cuda")
        _lib.call("rd_cache_unpack", code, _lib.ptr(want), NL, B, nkv, max_len, hd, S, _lib.ptr(idx), n_flat, _lib.ptr(scratch),
                  _lib.stream())
        got = cache.clone()
        _lib.call("rd_cache_unpack_static", code, _lib.ptr(got), NL, B, nkv, max_len, hd, S, _lib.ptr(idx), n_flat, _lib.stream())
        torch.cuda.synchronize()
        assert torch.equal(got, want)  # pure data movement: bit-exact
        assert not torch.equal(got, cache)  # and it did move something


def test_static_scratch_variant_refuses_what_does_not_fit():
    from recurrent_drafting import _lib

    lib = _lib.load()
    cache = torch.zeros(1, device="cuda")
    idx = torch.zeros(1, dtype=torch.int64, device="cuda")
    # 64 layers x 2 x 8 x 32 heads x 225 tokens x 128 x 2 bytes is far beyond the fixed 16 MiB
    rc = lib.rd_cache_unpack_static(_lib.BF16, _lib.ptr(cache), 64, 8, 32, 4096, 128, 10, _lib.ptr(idx), 225, _lib.stream())
    assert rc == -7
    assert b"capacity" in lib.rd_strerror(rc)
    with pytest.raises(_lib.RedrafterError, match="capacity"):
        _lib.call("rd_cache_unpack_static", _lib.BF16, _lib.ptr(cache), 64, 8, 32, 4096, 128, 10, _lib.ptr(idx), 225, _lib.stream())


def test_cache_method_without_allocation():
    import recurrent_drafting as rd

    c = rd.kv_cache.Cache(2, 30, 2, 2, 8, torch.float32, torch.device("cuda"))
    c._cache.copy_(torch.randn(c._cache.shape, device="cuda"))
    ref = rd.kv_cache.Cache(2, 30, 2, 2, 8, torch.float32, torch.device("cuda"))
    ref._cache.copy_(c._cache)
    idx = torch.tensor([[[0, 1, 2], [0, 1, 3]], [[0, 1, 2], [0, 3, 4]]], dtype=torch.int64, device="cuda")
    ref.unpack(4, idx)
    c.unpack_static(4, idx)
    assert torch.equal(c._cache, ref._cache) and c.sliced[0][0].length == ref.sliced[0][0].length == 10
