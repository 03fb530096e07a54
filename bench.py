"""Benchmark of the ReDrafter decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2|c1|c3|c4]

Workload (default c2): Vicuna-7B architecture, bf16, random-init weights, recurrent drafter with 2
residual blocks, beam_width 45, beam_length 5, batch 8 per GPU, 500-token synthetic prompts, greedy.
A step is one decode step of the whole batch: drafter beam search -> prefix-tree pack -> Llama
verify forward over the packed tree -> acceptance + KV commit.  The metric is generated tokens/s.

ours:      `value` times K steps after W warm-up steps with the prompt already on the device (CUDA
           events, max over ranks).  `e2e` times a whole request through the public API from pinned
           host memory: prompt upload, prefill, K steps, every yielded token matrix copied back.
           `roofline` is measured live for the dominant kernel (the tcgen05 GEMM); `cpu_baseline`
           times the numpy oracle on the host cores on a bounded sample (rank 0, N = 1 only).
reference: the reference's algorithm on the host cores (numpy oracle port), bounded sample.

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "ml-recurrent-drafter_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

CONFIGS = {
    # name: (llama cfg, drafter layers, batch/GPU, beam width, beam length, prompt, generate, dtype, greedy, temperature)
    "c1": (dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=2, intermediate_size=688,
                vocab_size=1000), 1, 2, 4, 3, 32, 64, "fp32", True, 1.0),
    "c2": (dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, num_hidden_layers=32,
                intermediate_size=11008, vocab_size=32000), 2, 8, 45, 5, 500, 512, "bf16", True, 1.0),
    # c2 with 4 decoder layers: same kernel shapes as c2, a few GB on the device (profiler captures)
    "c2-4l": (dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, num_hidden_layers=4,
                   intermediate_size=11008, vocab_size=32000), 2, 8, 45, 5, 500, 512, "bf16", True, 1.0),
    "c3": (dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, num_hidden_layers=32,
                intermediate_size=11008, vocab_size=32000), 2, 16, 16, 5, 256, 512, "bf16", False, 1.0),
    "c4": (dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=40, num_hidden_layers=40,
                intermediate_size=13824, vocab_size=32000), 2, 8, 32, 5, 1024, 1024, "bf16", True, 1.0),
}
# dram__bytes_read.sum + dram__bytes_write.sum of the four GEMMs of one verify layer (down, QKV, o, gate/up), mean per launch
GEMM_TRAFFIC_BYTES_PER_LAUNCH = int((113.2 + 3.8 + 109.4 + 4.7 + 45.8 + 0.1 + 191.5 + 12.5) / 4 * 1e6)
METRIC = "generated tokens/sec (ReDrafter decode, 7B-arch bw45xbl5 bs8 per GPU)"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured (MEASURED_PEAKS.json, sustained bf16)"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.rows = []
        self._stop = False
        self._proc = None
        self.index = index

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index),
                 "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self._proc = None

    def _read(self):
        for line in self._proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self._proc is not None:
            self._proc.terminate()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        watts = []
        for r in self.rows:
            try:
                watts.append(float(r[6]))
            except (IndexError, ValueError):
                pass
        watts.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(mhz), "power_w": round(watts[len(watts) // 2], 1) if watts else None}


# ------------------------------------------------------------------------------------------------
def build_gpu_models(cfg_name: str, device):
    import torch
    from transformers.models.llama.configuration_llama import LlamaConfig

    import recurrent_drafting as rd

    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    cfg = LlamaConfig(rms_norm_eps=1e-6, hidden_act="silu", pad_token_id=0, **lc)
    cfg.rope_theta = 10000.0
    with torch.device(device):
        llm = rd.modeling_llama.LlamaForCausalLM(cfg).to(dtype)
        dr = rd.modeling_drafter.Drafter(rd.configuration_drafter.DrafterConfig(
            vocab_size=lc["vocab_size"], hidden_size=lc["hidden_size"], exit_dim=2 * lc["hidden_size"], num_draft_layers=R, rnn=True)).to(dtype)
    llm.init_random(0.02, seed=123)
    dr.init_random(0.02, seed=124)
    return rd.RecurrentDrafting(llm, dr)


def run_ours(args):
    import torch
    import torch.distributed as dist

    import recurrent_drafting as rd
    from recurrent_drafting import _lib
    from recurrent_drafting.modeling_llama import _Linear

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[args.config]
    K, Wm = args.steps, max(args.warmup, 3)
    model = build_gpu_models(args.config, dev)
    g = torch.Generator().manual_seed(1000 + rank)
    prompt_host = torch.randint(3, lc["vocab_size"], (B, Lp), generator=g, dtype=torch.int64).pin_memory()
    shape = rd.modeling_drafter.BeamShape(W, Lb)
    sargs = rd.SamplingArgs(temp, greedy)
    special = rd.SpecialTokens(0, None)
    max_length = Lp + max(gen, (K + Wm + 2) * Lb + 8)

    # launch counter: every C-ABI call that enqueues kernels goes through _lib.call
    counter = {"n": 0}
    real_call = _lib.call

    def counting_call(name, *a):
        counter["n"] += 1
        return real_call(name, *a)

    _lib.call = counting_call
    for m in (rd.modeling_llama, rd.modeling_drafter, rd.recurrent_drafting, rd.tree_attention, rd.kv_cache):
        m._lib.call = counting_call

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident measurement: W warm-up steps, then K timed steps
    prompt_dev = prompt_host.to(dev)
    it = model.generate(rd.stats.Ledger(), prompt_dev, max_length, shape, sargs, special)
    for _ in range(Wm):
        next(it)
    st = model.last_state
    len0 = st.small_host[0].sum().item()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    counter["n"] = 0
    # in-kernel timing of the tensor-core GEMMs during the timed steps (ns of CTA 0 after its dependency wait, FLOP)
    gemm_acc = torch.zeros(2, dtype=torch.int64, device=dev)
    real_call("rd_gemm_set_timing", _lib.ptr(gemm_acc))
    ev0.record()
    accepted = 0
    for _ in range(K):
        next(it)
        accepted += int(st.small_host[1].sum())
    ev1.record()
    barrier()
    real_call("rd_gemm_set_timing", None)
    gemm_ns, gemm_flop = (int(x) for x in gemm_acc.tolist())
    launches = counter["n"]
    clocks = sampler.stop() if rank == 0 else None
    ms = ev0.elapsed_time(ev1)
    tokens = st.small_host[0].sum().item() - len0
    kernel_status = int(st.status.item())
    it.close()
    if kernel_status != 0:
        # a bounded wait inside a tensor-core kernel gave up: the timing is meaningless
        raise SystemExit(f"bench: kernel status word {kernel_status} is not zero (a pipeline wait timed out)")

    if args.value_only:
        if world > 1:
            dist.destroy_process_group()
        return {"metric": METRIC, "value": round(tokens / (ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": Wm,
                "ms_per_step": round(ms / K, 4), "impl": "ours", "config": {"workload": args.config}, "gpu_launches": launches,
                "note": "value only (profiling run)"} if rank == 0 else None

    # ---- roofline pass: event pairs around every kernel launch (C-ABI call) of a few more steps;
    #      the tensor-core GEMM calls also record their shapes for the FLOP count
    prof = []
    all_calls = []
    real_linear_call = _Linear.__call__

    def timed_linear(self, a, c, *pa, **kw):
        m_dev = kw.get("m_dev")
        prof.append((len(all_calls), self.weight.shape[0], self.weight.shape[1], a.shape[0] if m_dev is None else None))
        real_linear_call(self, a, c, *pa, **kw)

    real_qkv_rope = _Linear.qkv_rope

    def timed_qkv_rope(self, a, *pa, **kw):
        # the QKV projection with the rotary embedding in its epilogue: a GEMM launch with a device-side row count
        prof.append((len(all_calls), self.weight.shape[0], self.weight.shape[1], None))
        real_qkv_rope(self, a, *pa, **kw)

    def timed_call(name, *a):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        counting_call(name, *a)
        e1.record()
        all_calls.append((name, e0, e1))

    it = model.generate(rd.stats.Ledger(), prompt_dev, max_length, shape, sargs, special)
    for _ in range(3):
        next(it)
    _Linear.__call__ = timed_linear
    _Linear.qkv_rope = timed_qkv_rope
    _lib.call = timed_call
    flops = 0.0
    gemm_ms = 0.0
    n_gemm = 0
    by_kernel = {}
    by_shape = {}
    n_prof_steps = 4
    for _ in range(n_prof_steps):
        prof.clear()
        all_calls.clear()
        next(it)
        m_live = int(model.last_state.fp.row_start[-1].item())
        times = [(name, e0.elapsed_time(e1)) for name, e0, e1 in all_calls]
        for name, ms_k in times:
            agg = by_kernel.setdefault(name, [0, 0.0])
            agg[0] += 1
            agg[1] += ms_k
        for idx, N, Kd, m_fixed in prof:
            if idx >= len(times) or times[idx][0] not in ("rd_gemm_bf16_tc", "rd_gemm_bf16_tc_qkv_rope"):
                continue
            m = m_live if m_fixed is None else m_fixed
            f = 2.0 * m * N * Kd
            flops += f
            gemm_ms += times[idx][1]
            n_gemm += 1
            agg = by_shape.setdefault((N, Kd, m_fixed is None), [0, 0.0, 0.0])
            agg[0] += 1
            agg[1] += times[idx][1]
            agg[2] += f
    _Linear.__call__ = real_linear_call
    _Linear.qkv_rope = real_qkv_rope
    _lib.call = counting_call
    it.close()
    peaks = _peaks()
    ach = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    step_ms_prof = sum(v[1] for v in by_kernel.values()) / n_prof_steps
    breakdown = {k: {"launches_per_step": v[0] / n_prof_steps, "ms_per_step": round(v[1] / n_prof_steps, 4),
                     "share": round(v[1] / n_prof_steps / step_ms_prof, 4)} for k, v in sorted(by_kernel.items(), key=lambda kv: -kv[1][1])}
    if args.verbose and rank == 0:
        for k, v in breakdown.items():
            print(f"[breakdown] {k:28s} {v['launches_per_step']:7.1f}/step {v['ms_per_step']:9.4f} ms {100 * v['share']:5.1f}%", file=sys.stderr)
        for (N, Kd, dyn), v in sorted(by_shape.items(), key=lambda kv: -kv[1][1]):
            print(f"[gemm] N={N:6d} K={Kd:6d} {'verify' if dyn else 'drafter'} n={v[0] // n_prof_steps:3d}/step avg {1e3 * v[1] / v[0]:7.1f} us "
                  f"{v[2] / (v[1] * 1e-3) / 1e12:7.1f} TFLOP/s", file=sys.stderr)
    roofline = {"kernel": "gemm_tc_pair_kernel / gemm_tc_kernel (tcgen05 bf16 GEMM, all verify + drafter projections)", "bound": "tensor",
                "achieved": round(ach, 2), "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": round(ach / peaks["tflops"], 4), "traffic": GEMM_TRAFFIC_BYTES_PER_LAUNCH,
                "traffic_note": "DRAM read+write per launch, mean over the verify layer's four GEMMs, from the ncu capture in "
                                "profiles/gemm_tc_pair_kernel_c2_verify.md (c2 shapes on 4 layers)",
                "launches_timed": n_gemm, "flops_per_launch_avg": flops / max(n_gemm, 1), "peak_source": peaks["source"],
                "gemm_share_of_step": round(gemm_ms / n_prof_steps / (ms / K), 4) if ms > 0 else None,
                "kernel_time_breakdown": breakdown}
    if gemm_ns > 0:
        # the same kernels inside the timed steps, launches overlapping as they do in production: each launch's duration
        # is the lifetime of its first CTA after the dependency wait, read from %globaltimer in the kernel
        in_kernel = gemm_flop / gemm_ns / 1e3
        roofline["in_kernel"] = {"achieved": round(in_kernel, 2), "frac": round(in_kernel / peaks["tflops"], 4), "unit": "TFLOP/s",
                                 "gemm_ms_per_step": round(gemm_ns / 1e6 / K, 4),
                                 "note": "timed steps, no event records between launches; excludes launch latency and tails"}

    # ---- end to end through the public API from pinned host memory
    barrier()
    sink = torch.empty(B, max_length + 1, dtype=torch.int64).pin_memory()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    p_dev = prompt_host.to(dev, non_blocking=True)
    d2h = 0
    it = model.generate(rd.stats.Ledger(), p_dev, max_length, shape, sargs, special)
    for _ in range(K):
        out = next(it)
        sink[:, : out.shape[1]].copy_(out, non_blocking=True)
        d2h += out.numel() * 8
        torch.cuda.current_stream().synchronize()
    e2e_tokens = int(model.last_state.small_host[0].sum()) - B * Lp
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    it.close()

    if world > 1:
        from recurrent_drafting import replicas

        e2e_ms, e2e_tokens, _ = replicas.reduce_stats(e2e_ms, float(e2e_tokens), 0.0, dev)
        ms, tokens, accepted = replicas.reduce_stats(ms, float(tokens), float(accepted), dev)
        # the one collective of the path: gather of the generated tokens on rank 0 (outside the timed regions)
        gathered = replicas.gather_tokens(sink[:, : Lp + K].to(dev), 0, dst=0)
        assert rank != 0 or (len(gathered) == world and all(g.shape[0] == B for g in gathered))
    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": round(tokens / (ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt,
            "data": "synthetic", "impl": "ours",
            "config": {"workload": f"{args.config}: Vicuna-7B-arch greedy decode, random-init weights" if args.config == "c2" else args.config,
                       "batch_per_gpu": B, "beam_width": W, "beam_length": Lb, "prompt_len": Lp, "layers": lc["num_hidden_layers"],
                       "hidden": lc["hidden_size"], "vocab": lc["vocab_size"], "parallelism": f"replicas x{world} (batch sharded, no data-path collective)",
                       "l2": "inputs larger than L2 (13.5 GB of weights streamed every step)"},
            "accepted_tokens_per_step": round(accepted / (K * B * world), 4),
            "e2e": {"value": round(e2e_tokens / (e2e_ms * 1e-3), 2), "unit": "tokens/s", "h2d_bytes_per_step": B * Lp * 8 // K,
                    "d2h_bytes_per_step": d2h // K, "includes": "prompt upload + prefill + K steps + per-step token read-back"},
            "gpu_launches": launches, "roofline": roofline, "clocks": clocks,
        }
    if world > 1:
        dist.destroy_process_group()
    return line


# ------------------------------------------------------------------------------------------------
def cpu_decode_sample(cfg_name: str, rows: int, steps: int, budget_s: float):
    """Times decode steps of the numpy oracle on the host cores.  Bounded: `rows` batch rows, the
    prompt's K/V taken as already cached (zeros), one decoder layer's weights shared by all layers
    (same arithmetic, bounded host memory)."""
    import numpy as np

    from oracle import acceptance, drafter, generate, kv_cache

    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    H, I, V, NL = lc["hidden_size"], lc["intermediate_size"], lc["vocab_size"], lc["num_hidden_layers"]
    nh = lc["num_attention_heads"]
    rs = np.random.default_rng(0)

    def n(*shape):
        return rs.standard_normal(shape, dtype=np.float32) * np.float32(0.02)

    layer = {k: n(*s) for k, s in {
        "self_attn.q_proj.weight": (H, H), "self_attn.k_proj.weight": (H, H), "self_attn.v_proj.weight": (H, H),
        "self_attn.o_proj.weight": (H, H), "mlp.gate_proj.weight": (I, H), "mlp.up_proj.weight": (I, H),
        "mlp.down_proj.weight": (H, I)}.items()}
    ones = np.ones(H, dtype=np.float32)
    w = {"model.embed_tokens.weight": n(V, H), "model.norm.weight": ones, "lm_head.weight": n(V, H)}
    for l in range(NL):
        for k, v in layer.items():
            w[f"model.layers.{l}.{k}"] = v
        w[f"model.layers.{l}.input_layernorm.weight"] = ones
        w[f"model.layers.{l}.post_attention_layernorm.weight"] = ones
    E = 2 * H
    dw = {"rnn_w.weight": n(H, H), "rnn_u.weight": n(H, H), "rnn_u.bias": n(H), f"lm_head.{R}.weight": n(V, E)}
    for r in range(R):
        dw[f"lm_head.{r}.linear.weight"] = n(E, E)
        dw[f"lm_head.{r}.linear.bias"] = n(E)
    cfg = dict(lc, rms_norm_eps=1e-6, rope_theta=10000.0)
    cache = kv_cache.Cache(rows, Lp + steps * Lb + W * Lb + 8, NL, lc["num_key_value_heads"], H // nh)
    for k, v in cache.sliced:
        k.length = v.length = Lp
    ids = rs.integers(3, V, size=(rows, Lp)).astype(np.int64)
    ctx = n(rows, H) * 50
    tok = rs.integers(3, V, size=(rows,)).astype(np.int64)
    times, generated = [], 0
    t_all = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        beams, _ = drafter.beam_search_candidates(dw, R, ctx, tok, w["model.embed_tokens.weight"], W, Lb)
        hidden, logits, unp = generate.verify_candidates(w, cfg, ids, beams, cache, 0)
        by_llm = np.argmax(logits, axis=-1)
        nacc, seq = acceptance.greedy_choose_from_candidates(beams, by_llm)
        new_ids = acceptance.update_kv_cache_and_input_ids(ids, nacc, seq, beams, cache, 0)
        ctx, tok = acceptance.greedy_prepare_next_input(by_llm, hidden, seq, nacc)
        generated += int((nacc + 1).sum())
        ids = new_ids
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > budget_s:
            break
    return times, generated


def run_cpu(args, as_reference_arm: bool):
    import numpy as np  # noqa: F401

    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[args.config]
    cores = os.cpu_count() or 1
    try:
        # a launcher may have exported OMP_NUM_THREADS=1 (torchrun does): give the BLAS every host core back
        from threadpoolctl import threadpool_info, threadpool_limits

        threadpool_limits(limits=cores)
        cores = max([int(i.get("num_threads", 1)) for i in threadpool_info()] or [1])
    except ImportError:
        cores = int(os.environ.get("OMP_NUM_THREADS", cores))
    rows = 1 if args.config != "c1" else B
    steps = (max(args.warmup, 1) + args.steps) if as_reference_arm else 3
    budget = 240.0 if as_reference_arm else 40.0
    times, generated = cpu_decode_sample(args.config, rows, steps, budget)
    warm = 1 if len(times) > 1 else 0
    timed = times[warm:]
    per_row_tokens = generated / len(times) / rows  # generated tokens per row per step
    value = rows * per_row_tokens / (sum(timed) / len(timed))
    sample = (f"{len(timed)} decode step(s) after {warm} warm-up of the numpy fp32 oracle on {rows} of {B} batch rows, prompt K/V taken as "
              f"cached, one layer's weights shared by all {lc['num_hidden_layers']} layers; tokens/s of that sample (CPU throughput is compute-bound "
              f"and does not grow with batch)")
    cpu = {"value": round(value, 4), "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    if not as_reference_arm:
        return cpu
    ms = 1e3 * sum(timed) / len(timed)
    return {
        "metric": METRIC, "value": cpu["value"], "unit": "tokens/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": len(timed),
        "warmup": warm, "ms_per_step": round(ms, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "reference",
        "config": {"workload": f"{args.config}: Vicuna-7B-arch greedy decode, random-init weights" if args.config == "c2" else args.config,
                   "batch_per_gpu": B, "beam_width": W, "beam_length": Lb, "prompt_len": Lp},
        "cpu_baseline": cpu, "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--value-only", action="store_true", help="skip the roofline, end-to-end and CPU passes (profiler runs)")
    ap.add_argument("--verbose", action="store_true", help="print the per-kernel and per-GEMM-shape timing breakdown to stderr")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_cpu(args, True)), flush=True)
        return
    line = run_ours(args)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and not args.value_only:
            line["cpu_baseline"] = run_cpu(args, False)
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
