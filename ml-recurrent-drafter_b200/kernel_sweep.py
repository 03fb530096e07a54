"""Isolated sweep of the tree-verify kernels: prefix-tree pack + bitmask, tree-masked attention over a
KV cache, greedy acceptance (row argmax over the vocabulary + longest-matching-beam choice) and the
KV commit, over batch x beam_width x beam_length x cache length, bf16, 32 heads x head_dim 128.

Every kernel is timed alone with CUDA events on the launching stream (a trivial kernel is queued
first so the launch latency of the timed kernel is hidden), after warm-up, with a write of a buffer
larger than L2 between repetitions; the median of the repetitions is reported next to the kernel's
algorithmic bytes and the achieved GB/s.

    python ml-recurrent-drafter_b200/kernel_sweep.py [--quick] [--out table.md]

Synthetic inputs: K/V and Q ~ N(0,1) bf16; beams share one init token per row (column 0) and draw the
further tokens from a prefix-conditional Zipf(1.2) law with a few children per prefix, so a sizeable
fraction of the beam prefixes is shared (the achieved fraction is printed per cell); verify tokens
agree with the drafted token with probability 0.5 per position, so accepted lengths cover 0..Lb-1.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from typing import Dict, List

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import recurrent_drafting as rd  # noqa: E402
from recurrent_drafting import _lib  # noqa: E402

NH, NKV, HD, V = 32, 32, 128, 32000
NL_COMMIT = 32  # layers moved by the commit kernel (capped by a memory budget per cell)
CACHE_BUDGET_BYTES = 10 << 30


def shared_prefix_beams(batch: int, width: int, length: int, vocab: int, seed: int, a: float = 1.2,
                        branch: int = 3) -> np.ndarray:
    rs = np.random.RandomState(seed)
    out = np.zeros((batch, width, length), dtype=np.int64)
    for b in range(batch):
        out[b, :, 0] = rs.randint(3, vocab)
        children: Dict[tuple, np.ndarray] = {}
        for i in range(width):
            for j in range(1, length):
                key = tuple(out[b, i, :j])
                if key not in children:
                    children[key] = np.clip(rs.zipf(a, size=branch) + 2, 3, vocab - 1)
                out[b, i, j] = children[key][min(rs.zipf(a) - 1, branch - 1)]
    return out


class Timer:
    def __init__(self, reps: int):
        self.reps = reps
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        self.dummy = torch.zeros(64, dtype=torch.float32, device="cuda")

    def __call__(self, fn, prepare=None) -> float:
        """Median device time of fn() in microseconds."""
        for _ in range(2):
            if prepare:
                prepare()
            fn()
        ts: List[float] = []
        for _ in range(self.reps):
            if prepare:
                prepare()
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.dummy.add_(1.0)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)


def run_cell(B: int, W: int, Lb: int, S: int, timer: Timer, hbm_peak: float) -> dict:
    dev = "cuda"
    i32 = dict(dtype=torch.int32, device=dev)
    # children per prefix grow with the beam width so the shared fraction stays in a mid band
    beams_np = shared_prefix_beams(B, W, Lb, V, seed=B * 10007 + W * 101 + Lb, branch=max(3, 3 * W // Lb))
    beams = torch.from_numpy(beams_np).to(dev)
    max_len = S + W * Lb
    per_layer = 2 * B * NKV * max_len * HD * 2
    NL = int(max(1, min(NL_COMMIT, CACHE_BUDGET_BYTES // per_layer)))
    cache = torch.empty(NL, 2, B, NKV, max_len, HD, dtype=torch.bfloat16, device=dev)
    cache[0].normal_()
    kv_begin = torch.zeros(B, **i32)
    kv_len0 = torch.full((B,), S, **i32)
    kv_len = kv_len0.clone()

    # ---- pack + bitmask
    fp = rd.tree_attention.alloc_flat(B, W, Lb, dev)
    t_pack = timer(lambda: rd.tree_attention.pack_flat(beams, kv_begin, kv_len, out=fp))
    n_sel = fp.n_selected.cpu().numpy()
    M = int(n_sel.sum())
    cap = B * W * Lb
    shared = 1.0 - M / cap
    pack_bytes = cap * 8 + cap * (8 + 4 * 4) + cap * fp.mask_words * 4 + 2 * cap * 4

    # ---- tree attention over one layer of the cache
    q = torch.randn(cap, NH * HD, device=dev).bfloat16()
    out = torch.empty(cap, NH * HD, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, **i32)
    lib = _lib.load()
    k0, v0 = cache[0, 0], cache[0, 1]
    plan = lib.rd_attention_plan_create(_lib.ptr(q), cap, _lib.ptr(k0), _lib.ptr(v0), B, NH, NKV, HD, max_len)
    if not plan:
        raise _lib.RedrafterError("rd_attention_plan_create failed")

    shares = rd.attention.key_range_shares(B, NH, W * Lb, S + W * Lb)
    ws_bytes = lib.rd_attention_split_workspace_bytes(cap, NH, shares) if shares > 1 else 0
    split_ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

    def attn():
        if shares > 1:
            _lib.call("rd_attention_tc_split", plan, _lib.ptr(out), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len),
                      W * Lb, _lib.ATTN_TREE, _lib.ptr(fp.tree_mask), fp.mask_words, shares, _lib.ptr(split_ws), ws_bytes,
                      _lib.ptr(status), _lib.stream())
        else:
            _lib.call("rd_attention_tc", plan, _lib.ptr(out), _lib.ptr(fp.row_start), _lib.ptr(kv_begin), _lib.ptr(fp.base_len),
                      W * Lb, _lib.ATTN_TREE, _lib.ptr(fp.tree_mask), fp.mask_words, _lib.ptr(status), _lib.stream())

    t_attn = timer(attn)
    lib.rd_attention_plan_destroy(plan)
    if int(status.item()) != 0:
        raise _lib.RedrafterError(f"attention kernel status {int(status.item())}")
    attn_bytes = (2 * NKV * int((S + n_sel).sum()) * HD + 2 * M * NH * HD) * 2
    attn_flops = 4 * NH * HD * int((n_sel * (S + n_sel)).sum())
    del q, out, split_ws

    # ---- acceptance: row argmax over fp32 logits, then choice + commit
    logits = torch.randn(M, V, device=dev)
    rs = np.random.RandomState(B + W + Lb)
    unp = fp.unpacker.cpu().numpy()
    row_start = fp.row_start.cpu().numpy()
    plant_rows, plant_cols = [], []
    for b in range(B):
        agree = rs.rand(W, Lb - 1) < 0.5
        for i in range(W):
            for j in range(Lb - 1):
                if agree[i, j]:
                    plant_rows.append(row_start[b] + unp[b, i, j])
                    plant_cols.append(beams_np[b, i, j + 1])
    if plant_rows:
        logits[torch.tensor(plant_rows, device=dev), torch.tensor(plant_cols, device=dev)] = 50.0
    llm_tok = torch.empty(cap, **i32)
    t_argmax = timer(lambda: _lib.call("rd_argmax_rows", _lib.ptr(logits), logits.stride(0), M, _lib.ptr(fp.m_dev), V,
                                       _lib.ptr(llm_tok), None, _lib.stream()))
    argmax_bytes = M * V * 4
    del logits

    H = 4096
    hidden = torch.randn(cap, H, device=dev).bfloat16()
    token_buf = torch.zeros(B, max_len, dtype=torch.int64, device=dev)
    n_acc, seq = torch.zeros(B, **i32), torch.zeros(B, **i32)
    next_tok = torch.zeros(B, dtype=torch.int64, device=dev)
    next_ctx = torch.empty(B, H, dtype=torch.bfloat16, device=dev)

    def commit():
        _lib.call("rd_accept_commit_greedy", _lib.BF16, _lib.ptr(beams), B, W, Lb, _lib.ptr(fp.unpacker), _lib.ptr(fp.row_start),
                  _lib.ptr(llm_tok), _lib.ptr(hidden), H, _lib.ptr(cache), NL, NKV, max_len, HD, _lib.ptr(kv_begin),
                  _lib.ptr(fp.base_len), _lib.ptr(kv_len), _lib.ptr(token_buf), _lib.ptr(n_acc), _lib.ptr(seq),
                  _lib.ptr(next_tok), _lib.ptr(next_ctx), _lib.stream())

    t_commit = timer(commit, prepare=lambda: kv_len.copy_(kv_len0))
    acc = n_acc.cpu().numpy()
    commit_bytes = 2 * int((acc + 1).sum()) * NL * 2 * NKV * HD * 2 + B * H * 2 * 2

    def gbs(nbytes, us):
        return nbytes / (us * 1e-6) / 1e9

    return {
        "B": B, "W": W, "Lb": Lb, "S": S, "tokens": M, "shared_prefix_fraction": round(shared, 3),
        "mean_accepted": round(float(acc.mean()), 2), "commit_layers": NL,
        "pack_us": round(t_pack, 1), "pack_gbs": round(gbs(pack_bytes, t_pack), 1),
        "attn_shares": shares, "attn_us": round(t_attn, 1), "attn_gbs": round(gbs(attn_bytes, t_attn), 1),
        "attn_frac_hbm": round(gbs(attn_bytes, t_attn) / hbm_peak, 3), "attn_tflops": round(attn_flops / (t_attn * 1e-6) / 1e12, 1),
        "argmax_us": round(t_argmax, 1), "argmax_gbs": round(gbs(argmax_bytes, t_argmax), 1),
        "argmax_frac_hbm": round(gbs(argmax_bytes, t_argmax) / hbm_peak, 3),
        "commit_us": round(t_commit, 1), "commit_gbs": round(gbs(commit_bytes, t_commit), 1),
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="corner cells only")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--out", default=None, help="write the markdown table here as well")
    ap.add_argument("--cell", type=int, nargs=4, metavar=("B", "W", "LB", "S"), default=None, help="run this one cell only")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("kernel_sweep needs a CUDA device")
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    hbm_peak, src = 6650.0, "fallback"
    if os.path.exists(peaks_path):
        hbm_peak, src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    Bs, Ws, Ls, Ss = [1, 8, 64], [8, 45, 64], [3, 5, 7], [512, 2048, 4096]
    if args.quick:
        Bs, Ws, Ls, Ss = [1, 64], [8, 64], [3, 7], [512, 4096]
    if args.cell:
        Bs, Ws, Ls, Ss = [[x] for x in args.cell]
    timer = Timer(args.reps)
    cols = ["B", "W", "Lb", "S", "tokens", "shared_prefix_fraction", "mean_accepted", "pack_us", "attn_shares", "attn_us", "attn_gbs",
            "attn_frac_hbm", "attn_tflops", "argmax_us", "argmax_gbs", "argmax_frac_hbm", "commit_layers", "commit_us", "commit_gbs"]
    lines = [f"HBM peak {hbm_peak:.1f} GB/s ({src})", "", "| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    for B in Bs:
        for W in Ws:
            for Lb in Ls:
                for S in Ss:
                    r = run_cell(B, W, Lb, S, timer, hbm_peak)
                    print(json.dumps(r), flush=True)
                    lines.append("| " + " | ".join(str(r[c]) for c in cols) + " |")
                    torch.cuda.empty_cache()
    table = "\n".join(lines)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            f.write(table + "\n")
    print(table)


if __name__ == "__main__":
    main()
