"""The multi-GPU path (replicas + one final gather) on CPU ranks with the gloo backend, world size 2."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ml-recurrent-drafter_b200"))
    from recurrent_drafting import replicas

    lo, hi = replicas.shard_bounds(5, rank, world)
    # rank 0 decodes 3 requests to length 7, rank 1 decodes 2 requests to length 9
    length = 7 if rank == 0 else 9
    tokens = torch.arange((hi - lo) * length, dtype=torch.int64).reshape(hi - lo, length) + 100 * rank + 1
    got = replicas.gather_tokens(tokens, pad_id=0, dst=0)
    ms, gen, acc = replicas.reduce_stats(10.0 + rank, 100.0 * (rank + 1), float(rank), torch.device("cpu"))
    ok = (ms, gen, acc) == (11.0, 300.0, 1.0)
    if rank == 0:
        ok = ok and len(got) == 2 and got[0].shape == (3, 9) and got[1].shape == (2, 9)
        ok = ok and torch.equal(got[0][:, 2:], tokens) and bool((got[0][:, :2] == 0).all())
        ok = ok and torch.equal(got[1], torch.arange(18, dtype=torch.int64).reshape(2, 9) + 101)
    else:
        ok = ok and got is None and (lo, hi) == (3, 5)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as fh:
        fh.write("ok" if ok else "fail")
    dist.destroy_process_group()


class _StubModel:
    """Stands in for RecurrentDrafting: appends one deterministic token per row and step."""

    def generate(self, ledger, input_ids, max_length, beam_shape, sampling_args, special_tokens):
        ids = input_ids.clone()
        while ids.shape[1] < max_length:
            nxt = ids.sum(dim=1, keepdim=True) % 97 + 3
            ids = torch.cat([ids, nxt], dim=1)
            yield ids


class _Special:
    pad = 0
    eos = None


def _requests():
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(3, 50, (5, 6), generator=g, dtype=torch.int64)
    ids[1, :2] = 0  # left padding
    ids[4, :4] = 0
    return ids


def _sharded_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ml-recurrent-drafter_b200"))
    from recurrent_drafting import replicas

    ids = _requests()
    res = replicas.generate_sharded(_StubModel(), ids, 11, None, None, _Special(), max_steps=None)
    want = list(_StubModel().generate(None, ids, 11, None, None, _Special()))[-1]
    lo, hi = replicas.shard_bounds(5, rank, world)
    ok = res.steps_local == 5 and res.generated_local == 5 * (hi - lo)
    if rank == 0:
        ok = ok and res.tokens is not None and torch.equal(res.tokens, want)
    else:
        ok = ok and res.tokens is None
    # a bounded number of steps and the per-step host copy
    sink = torch.zeros(3, 12, dtype=torch.int64)
    res2 = replicas.generate_sharded(_StubModel(), ids, 11, None, None, _Special(), max_steps=2, host_sink=sink)
    ok = ok and res2.steps_local == 2 and res2.d2h_bytes == (hi - lo) * (7 + 8) * 8
    if rank == 0:
        ok = ok and res2.tokens.shape == (5, 8) and torch.equal(res2.tokens, want[:, :8]) and torch.equal(sink[:, :8], want[:3, :8])
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as fh:
        fh.write("ok" if ok else "fail")
    dist.destroy_process_group()


def test_generate_sharded_world_size_2(tmp_path):
    """One batch of 5 requests in, 5 rows out on rank 0, decoded by two ranks (3 + 2 rows)."""
    port = _free_port()
    mp.spawn(_sharded_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [open(tmp_path / f"rank{r}.txt").read() for r in range(2)] == ["ok", "ok"]


def test_generate_sharded_without_process_group():
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ml-recurrent-drafter_b200"))
    from recurrent_drafting import replicas

    ids = _requests()
    res = replicas.generate_sharded(_StubModel(), ids, 9, None, None, _Special())
    assert torch.equal(res.tokens, list(_StubModel().generate(None, ids, 9, None, None, _Special()))[-1])
    assert res.generated_local == 15 and res.steps_local == 3


def test_shard_bounds():
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ml-recurrent-drafter_b200"))
    from recurrent_drafting import replicas

    for n in (1, 8, 13, 64):
        for w in (1, 2, 3, 8):
            parts = [replicas.shard_bounds(n, r, w) for r in range(w)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            sizes = [hi - lo for lo, hi in parts]
            assert max(sizes) - min(sizes) <= 1


def test_gather_and_stats_world_size_2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [open(tmp_path / f"rank{r}.txt").read() for r in range(2)] == ["ok", "ok"]
