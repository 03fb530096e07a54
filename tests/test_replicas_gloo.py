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
