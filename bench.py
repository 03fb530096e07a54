"""Benchmark of the ReDrafter decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2|c1|c3|c4]

Workload (default c2): Vicuna-7B architecture, bf16, random-init weights, recurrent drafter with 2
residual blocks, beam_width 45, beam_length 5, batch 8 per GPU, 500-token synthetic prompts, greedy.
A step is one decode step of the whole batch: drafter beam search -> prefix-tree pack -> Llama
verify forward over the packed tree -> acceptance + KV commit.  The metric is generated tokens/s.
c3 is the sampling workload (temperature 1, batch 16, 16 beams), c4 the 13B architecture with 8
requests per GPU (64 on eight GPUs), c1 the tiny fp32 configuration.

ours:      `value` times K steps after W warm-up steps with the prompt already on the device (CUDA
           events, max over ranks).  `e2e` times whole requests through the public API from pinned
           host memory: prompt upload, prefill, K steps, every yielded token matrix copied back
           (with N > 1 ranks: one batch of N x B requests split by replicas.generate_sharded and
           gathered on rank 0 inside the timed region).  `roofline` is measured live for the dominant
           kernel (the tcgen05 GEMM); `prefill` is the time to the first token; `cpu_baseline`
           times a bounded sample (prefill + 2 decode steps) of the reference itself on the host cores in a
           child process, or the numpy port when the reference cannot run (rank 0, N = 1 only).
reference: the reference's own PyTorch implementation (installed under baseline/_ref, CPU, fp32) run
           through RecurrentDrafting.generate on the host cores with the same configuration, for the
           prefill and as many decode steps as fit a time budget; the numpy port on one row is
           timed beside it as a cross-check.  Without baseline/_ref, or without the host memory
           for the fp32 weights, the port alone is timed and the line says so.

One JSON line is printed by rank 0.
"""
import argparse
import contextlib
import datetime
import json
import os
import subprocess
import sys
import threading
import time
import types
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "ml-recurrent-drafter_b200")
REF_INSTALL = os.path.join(ROOT, "baseline", "_ref")

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
    "c3-4l": (dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, num_hidden_layers=4,
                   intermediate_size=11008, vocab_size=32000), 2, 16, 16, 5, 256, 512, "bf16", False, 1.0),
    "c4": (dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=40, num_hidden_layers=40,
                intermediate_size=13824, vocab_size=32000), 2, 8, 32, 5, 1024, 1024, "bf16", True, 1.0),
}
WORKLOADS = {
    "c1": "c1: tiny fp32 greedy decode (2 layers, hidden 256), random-init weights",
    "c2": "c2: Vicuna-7B-arch greedy decode, random-init weights",
    "c2-4l": "c2-4l: c2's shapes on 4 decoder layers (profiler case)",
    "c3": "c3: Vicuna-7B-arch speculative sampling (temperature 1.0), random-init weights",
    "c3-4l": "c3-4l: c3's shapes on 4 decoder layers (profiler case)",
    "c4": "c4: Vicuna-13B-arch greedy decode, 8 requests per GPU, random-init weights",
}
# dram__bytes_read.sum + dram__bytes_write.sum of the four GEMMs of one verify layer (down, QKV, o, gate/up), mean per launch
GEMM_TRAFFIC_BYTES_PER_LAUNCH = int((113.2 + 4.7 + 108.5 + 4.4 + 45.8 + 0.1 + 191.2 + 14.6) / 4 * 1e6)


def workload_config(cfg_name: str, world: int) -> dict:
    """The `config` object of the JSON line; both arms describe the workload with the same keys and values."""
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    H, I, V, NL = lc["hidden_size"], lc["intermediate_size"], lc["vocab_size"], lc["num_hidden_layers"]
    weight_gb = (NL * (4 * H * H + 3 * H * I) + V * H) * (2 if dt == "bf16" else 4) / 1e9
    l2 = (f"inputs larger than L2 ({weight_gb:.1f} GB of weights are streamed every step)" if weight_gb > 0.2
          else f"no flush: the {weight_gb * 1e3:.0f} MB of weights fit L2 (tiny configuration, launch bound)")
    return {"workload": WORKLOADS[cfg_name], "batch_per_gpu": B, "beam_width": W, "beam_length": Lb, "prompt_len": Lp,
            "layers": lc["num_hidden_layers"], "hidden": lc["hidden_size"], "vocab": lc["vocab_size"],
            "sampling": "greedy" if greedy else f"temperature {temp}",
            "parallelism": f"replicas x{world} (batch of {B * world} requests sharded by rows, no data-path collective)",
            "l2": l2}


def metric_name(cfg_name: str) -> str:
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    arch = {4096: "7B-arch", 5120: "13B-arch"}.get(lc["hidden_size"], f"hidden{lc['hidden_size']}")
    return f"generated tokens/sec (ReDrafter decode, {arch} bw{W}xbl{Lb} bs{B} per GPU)"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured (MEASURED_PEAKS.json, sustained bf16)"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi every 50 ms.  Rows carry
    nvidia-smi's own timestamp, so stop(t0, t1) keeps exactly the samples taken inside the timed
    region however the pipe buffered them.  Reads the GPU's state only; changes no setting."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index: int):
        self.rows = []
        self._proc = None
        self.index = index

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self._proc = None

    def _read(self):
        for line in self._proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    @staticmethod
    def _when(stamp: str):
        try:
            return datetime.datetime.strptime(stamp, "%Y/%m/%d %H:%M:%S.%f")
        except ValueError:
            return None

    def stop(self, t0: datetime.datetime, t1: datetime.datetime, ms_per_step: float):
        if self._proc is not None:
            time.sleep(0.12)  # let the samples of the last interval arrive
            self._proc.terminate()
        rows = []
        for r in self.rows:
            if len(r) < 8:
                continue
            w = self._when(r[0])
            if w is not None and t0 <= w <= t1:
                rows.append(r)
        if not rows:  # a region shorter than the sampling interval: take the nearest samples
            rows = [r for r in self.rows if len(r) >= 8][-2:]
        mhz = sorted(int(r[1]) for r in rows if r[1].isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mx = [int(r[2]) for r in rows if r[2].isdigit()]
        watts = []
        for r in rows:
            try:
                watts.append(float(r[7]))
            except ValueError:
                pass
        watts.sort()
        med = mhz[len(mhz) // 2] if mhz else None
        return {"sm_mhz": med, "sm_mhz_min": mhz[0] if mhz else None, "sm_mhz_max_seen": mhz[-1] if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(mhz), "interval_ms": 50,
                "power_w": round(watts[len(watts) // 2], 1) if watts else None,
                # SM cycles one step takes at the median sampled clock: compares runs whose clocks differ
                "cycles_per_step": round(ms_per_step * med * 1e3) if med else None}


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
    for _p in (ROOT, PKG):
        if _p not in sys.path:
            sys.path.insert(0, _p)
    import torch
    import torch.distributed as dist

    import recurrent_drafting as rd
    from recurrent_drafting import _lib, replicas
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
    # one batch of world x B requests, the same on every rank; rank r decodes rows shard_bounds(.., r, world)
    g = torch.Generator().manual_seed(1000)
    prompts_all = torch.randint(3, lc["vocab_size"], (B * world, Lp), generator=g, dtype=torch.int64).pin_memory()
    lo, hi = replicas.shard_bounds(B * world, rank, world)
    prompt_host = prompts_all[lo:hi]
    shape = rd.modeling_drafter.BeamShape(W, Lb)
    sargs = rd.SamplingArgs(temp, greedy)
    special = rd.SpecialTokens(0, None)
    max_length = Lp + max(gen, (K + Wm + 2) * Lb + 8)
    torch.manual_seed(4321 + rank)  # sampling workloads draw their uniforms from torch's generator

    # launch counter: _lib.launches counts the kernels enqueued through the C ABI (a replayed CUDA graph adds the
    # kernels captured in it)
    real_call = _lib.call

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
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)  # nvidia-smi is up before the timed region begins
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = _lib.launches
    t_wall0 = datetime.datetime.now()
    ev0.record()
    accepted = 0
    for _ in range(K):
        next(it)
        accepted += int(st.small_host[1].sum())
    ev1.record()
    barrier()
    t_wall1 = datetime.datetime.now()
    launches = _lib.launches - launches0
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_wall0, t_wall1, ms / K) if rank == 0 else None
    tokens = st.small_host[0].sum().item() - len0
    kernel_status = int(st.status.item())
    it.close()
    if kernel_status != 0:
        # a bounded wait inside a tensor-core kernel gave up: the timing is meaningless
        raise SystemExit(f"bench: kernel status word {kernel_status} is not zero (a pipeline wait timed out)")

    if args.value_only:
        if world > 1:
            dist.destroy_process_group()
        return {"metric": metric_name(args.config), "value": round(tokens / (ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": world, "steps": K,
                "warmup": Wm, "ms_per_step": round(ms / K, 4), "impl": "ours", "config": workload_config(args.config, world),
                "gpu_launches": launches, "clocks": clocks, "note": "value only (profiling run)"} if rank == 0 else None

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
        real_call(name, *a)
        e1.record()
        all_calls.append((name, e0, e1))

    # this pass brackets every launch with events, so it runs the steps as ordinary launches (the timed steps above
    # replayed them from CUDA graphs; the kernels are the same)
    graphs_setting, model.cuda_graphs = model.cuda_graphs, False
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
    gemm_names = ("rd_gemm_bf16_tc", "rd_gemm_bf16_tc_qkv_rope", "rd_gemm_bf16_tc_argmax", "rd_gemm_bf16_tc_topk")
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
            if idx >= len(times) or times[idx][0] not in gemm_names:
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
    _lib.call = real_call
    it.close()
    model.cuda_graphs = graphs_setting
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
                # every FLOP of the step's GEMMs over the whole timed step (launch gaps and all other kernels included)
                "whole_step": {"achieved": round(flops / n_prof_steps / (ms / K * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                               "frac": round(flops / n_prof_steps / (ms / K * 1e-3) / 1e12 / peaks["tflops"], 4)},
                "kernel_time_breakdown": breakdown}

    # ---- end to end through the public API from pinned host memory; the prefill is timed on its own inside it
    if world > 1:
        # first use of the collective the final gather runs on (communicator set-up is not part of a request)
        replicas.gather_tokens(torch.zeros(1, 1, dtype=torch.int64, device=dev), 0)
    barrier()
    pf0, pf1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    real_prefill = model._comprehend_prompt

    def timed_prefill(*a, **kw):
        pf0.record()
        r = real_prefill(*a, **kw)
        pf1.record()
        return r

    model._comprehend_prompt = timed_prefill
    sink = torch.empty(B, max_length + 1, dtype=torch.int64).pin_memory()
    # one short untimed request first: the timed one then measures a server in steady state (allocator blocks, pinned
    # staging and descriptor sets of this call path exist), as the warm-up steps do for the device-resident figure
    replicas.generate_sharded(model, prompts_all, max_length, shape, sargs, special, device=dev, max_steps=4, host_sink=sink)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    res = replicas.generate_sharded(model, prompts_all, max_length, shape, sargs, special, device=dev, max_steps=K, host_sink=sink)
    e1.record()
    barrier()
    model._comprehend_prompt = real_prefill
    e2e_ms = e0.elapsed_time(e1)
    prefill_ms = pf0.elapsed_time(pf1)
    e2e_tokens = res.generated_local
    if rank == 0:
        assert res.tokens is not None and res.tokens.shape[0] == B * world, "the gather lost rows"

    if world > 1:
        e2e_ms, e2e_tokens, _ = replicas.reduce_stats(e2e_ms, float(e2e_tokens), 0.0, dev)
        prefill_ms, _, _ = replicas.reduce_stats(prefill_ms, 0.0, 0.0, dev)
        ms, tokens, accepted = replicas.reduce_stats(ms, float(tokens), float(accepted), dev)
    line = None
    if rank == 0:
        line = {
            "metric": metric_name(args.config), "value": round(tokens / (ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt,
            "data": "synthetic", "impl": "ours",
            "config": workload_config(args.config, world),
            "accepted_tokens_per_step": round(accepted / (K * B * world), 4),
            "e2e": {"value": round(e2e_tokens / (e2e_ms * 1e-3), 2), "unit": "tokens/s", "h2d_bytes_per_step": B * Lp * 8 // K,
                    "d2h_bytes_per_step": res.d2h_bytes // K,
                    "includes": "prompt upload + prefill + K steps + per-step token read-back" + (" + final gather on rank 0" if world > 1 else "")},
            "prefill": {"ms": round(prefill_ms, 3), "prompt_tokens_per_gpu": B * Lp, "tokens_per_s": round(B * Lp * world / (prefill_ms * 1e-3), 1),
                        "note": "time to the first token of the e2e request (max over ranks), inside the e2e figure"},
            "gpu_launches": launches, "roofline": roofline, "clocks": clocks,
        }
    if world > 1:
        dist.destroy_process_group()
    return line


# ------------------------------------------------------------------------------------------------
def cpu_decode_sample(cfg_name: str, rows: int, steps: int, budget_s: float):
    """Times decode steps of the numpy oracle on the host cores.  Bounded: `rows` batch rows, the
    prompt's K/V taken as already cached (zeros), one decoder layer's weights shared by all layers
    (same arithmetic, bounded host memory).  Greedy or sampling acceptance as the configuration says."""
    import numpy as np

    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
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
    uni = generate.UniformSource(5)
    times, generated = [], 0
    t_all = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        beams, logq = drafter.beam_search_candidates(dw, R, ctx, tok, w["model.embed_tokens.weight"], W, Lb)
        hidden, logits, unp = generate.verify_candidates(w, cfg, ids, beams, cache, 0)
        if greedy:
            by_llm = np.argmax(logits, axis=-1)
            nacc, seq = acceptance.greedy_choose_from_candidates(beams, by_llm)
        else:
            logp = drafter.log_softmax(logits / np.float32(temp))
            nacc, seq = acceptance.choose_from_candidates(beams, logp, logq, uni.uniform((rows, W, Lb - 1)))
        new_ids = acceptance.update_kv_cache_and_input_ids(ids, nacc, seq, beams, cache, 0)
        if greedy:
            ctx, tok = acceptance.greedy_prepare_next_input(by_llm, hidden, seq, nacc)
        else:
            probs = acceptance.residual_probs(logq, logp, seq, nacc)
            tok = acceptance.sample_inverse_cdf(probs, uni.uniform((rows,)))
            ctx = hidden[np.arange(rows), seq, nacc]
        generated += int((nacc + 1).sum())
        ids = new_ids
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > budget_s:
            break
    return times, generated


def _host_threads() -> int:
    import numpy  # noqa: F401  (its BLAS must be loaded before the thread pools are looked up)

    cores = os.cpu_count() or 1
    try:
        # a launcher may have exported OMP_NUM_THREADS=1 (torchrun does): give the BLAS every host core back
        from threadpoolctl import threadpool_info, threadpool_limits

        threadpool_limits(limits=cores)
        cores = max([int(i.get("num_threads", 1)) for i in threadpool_info()] or [1])
    except ImportError:
        cores = int(os.environ.get("OMP_NUM_THREADS", cores))
    return cores


def run_port(cfg_name: str, steps: int, budget_s: float):
    """The numpy port on a bounded sample; returns the cpu_baseline object."""
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    cores = _host_threads()
    rows = 1 if cfg_name != "c1" else B
    times, generated = cpu_decode_sample(cfg_name, rows, steps, budget_s)
    warm = 1 if len(times) > 1 else 0
    timed = times[warm:]
    per_row_tokens = generated / len(times) / rows  # generated tokens per row per step
    value = rows * per_row_tokens / (sum(timed) / len(timed))
    sample = (f"{len(timed)} decode step(s) after {warm} warm-up of the numpy fp32 restatement ({'greedy' if greedy else 'sampling'} acceptance) on {rows} of "
              f"{B} batch rows, prompt K/V taken as cached, one layer's weights shared by all {lc['num_hidden_layers']} layers; tokens/s of that "
              f"sample, i.e. of ONE row's work per step")
    return {"value": round(value, 4), "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
            "ms_per_step_one_row": round(1e3 * sum(timed) / len(timed), 1), "steps_timed": len(timed), "warmup": warm}


def _install_reference_shims():
    """The reference imports `jsonlines` for its stats ledger; the module is not installed here.  A
    stand-in with the two classes it uses is registered; it touches no arithmetic."""
    stub = types.ModuleType("jsonlines")

    class Writer:
        def __init__(self, fp):
            self.fp = fp

        def write(self, d):
            self.fp.write(json.dumps(d) + "\n")

        def close(self):
            pass

    class Reader:
        def __init__(self, fp):
            self.fp = fp

        def __iter__(self):
            for line in self.fp:
                if line.strip():
                    yield json.loads(line)

        def close(self):
            pass

    stub.Writer, stub.Reader = Writer, Reader
    sys.modules.setdefault("jsonlines", stub)


def reference_max_length(cfg_name: str, steps_cap: int) -> int:
    """Token budget of the reference run: the whole generation for c1, otherwise just enough for the
    steps that will be timed (the cache it allocates, and clones every step, is sized by it)."""
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    return Lp + gen if cfg_name == "c1" else Lp + (steps_cap + 2) * Lb + 8


def reference_unavailable_reason(cfg_name: str, steps_cap: int, sample: bool = False):
    """None when the installed reference can run this configuration in fp32 on this host (and, for a bounded
    sample, when its prefill is short enough for one)."""
    if not os.path.isdir(os.path.join(REF_INSTALL, "recurrent_drafting")):
        return "baseline/_ref holds no installed reference"
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    H, I, V, NL = lc["hidden_size"], lc["intermediate_size"], lc["vocab_size"], lc["num_hidden_layers"]
    params = NL * (4 * H * H + 3 * H * I) + 2 * V * H + 2 * H * H + R * 4 * H * H + 2 * H * V
    if sample:
        # about 2 TFLOP/s of fp32 on 16 host cores: keep the sample's prefill under a minute
        prefill_tflop = 2.0 * B * Lp * (NL * (4 * H * H + 3 * H * I) + V * H) / 1e12
        if prefill_tflop > 120:
            return f"the prefill alone is {prefill_tflop:.0f} TFLOP, too long for a bounded sample on the host cores"
    cache = NL * 2 * B * lc["num_key_value_heads"] * (reference_max_length(cfg_name, steps_cap) + W * Lb) * (H // lc["num_attention_heads"])
    # weights + the cache and the copies of it the reference makes every step + unpacked logits and log-probs + slack
    need = 4 * (params + 2 * cache) + B * W * Lb * V * 4 * 6 + (4 << 30)
    try:
        import psutil

        avail = psutil.virtual_memory().available
    except ImportError:
        avail = os.sysconf("SC_PHYS_PAGES") * os.sysconf("SC_PAGE_SIZE")
    if avail < need:
        return f"host memory: {avail >> 30} GiB available, the fp32 reference needs about {need >> 30} GiB"
    return None


def run_reference_impl(cfg_name: str, max_steps: int, budget_s: float):
    """RecurrentDrafting.generate of the installed reference (baseline/_ref) on the host cores, fp32,
    same architecture, prompts, beam shape and sampling arguments as the GPU arm.  Times the first
    call (prefill + first step) and every further step until max_steps or the budget is reached."""
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") not in (PKG, ROOT)]
    sys.path.insert(0, REF_INSTALL)
    _install_reference_shims()
    from unittest import mock

    import torch
    from transformers.models.llama.configuration_llama import LlamaConfig

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    import recurrent_drafting as ref

    assert os.path.abspath(ref.__file__).startswith(REF_INSTALL), ref.__file__
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[cfg_name]
    cfg = LlamaConfig(rms_norm_eps=1e-6, hidden_act="silu", pad_token_id=0, **lc)
    cfg.rope_theta = 10000.0  # newer transformers keep it in rope_parameters; the reference reads the attribute
    t_build = time.perf_counter()
    try:
        from transformers.initialization import no_init_weights
    except ImportError:
        no_init_weights = contextlib.nullcontext
    # skip the framework's random initialisation of 7e9 parameters; every weight is filled below
    with no_init_weights(), mock.patch.object(torch.nn.Linear, "reset_parameters", lambda self: None), \
            mock.patch.object(torch.nn.Embedding, "reset_parameters", lambda self: None):
        llm = ref.modeling_llama.LlamaForCausalLM(cfg)
        drafter = ref.modeling_drafter.Drafter(ref.configuration_drafter.DrafterConfig(
            vocab_size=lc["vocab_size"], hidden_size=lc["hidden_size"], exit_dim=2 * lc["hidden_size"], num_draft_layers=R, rnn=True))
    g = torch.Generator().manual_seed(123)
    L = 1 << 22
    noise = torch.randn(L, generator=g) * 0.02
    with torch.no_grad():
        for name, prm in list(llm.named_parameters()) + list(drafter.named_parameters()):
            if prm.ndim == 1 and "bias" not in name:
                prm.fill_(1.0)
                continue
            # N(0, 0.02) values from one 4M-element block, rotated by a per-parameter offset; whole blocks are
            # written by one broadcast copy (multi-threaded), which also first-touches the pages
            src = torch.roll(noise, zlib.crc32(name.encode()) % L)
            flat = prm.view(-1)
            whole = flat.numel() // L * L
            if whole:
                flat[:whole].view(-1, L).copy_(src.expand(whole // L, L))
            flat[whole:].copy_(src[: flat.numel() - whole])
    llm.eval()
    drafter.eval()
    build_s = time.perf_counter() - t_build
    model = ref.recurrent_drafting.RecurrentDrafting(llm, drafter)
    gp = torch.Generator().manual_seed(1000)
    prompts = torch.randint(3, lc["vocab_size"], (B, Lp), generator=gp, dtype=torch.int64)
    torch.manual_seed(4321)
    ledger = ref.stats.Ledger()
    steps_cap = max(max_steps, 2) if cfg_name != "c1" else gen
    max_length = reference_max_length(cfg_name, steps_cap)
    it = model.generate(ledger, prompts, max_length, ref.modeling_drafter.BeamShape(W, Lb), ref.recurrent_drafting.SamplingArgs(temp, greedy),
                        ref.recurrent_drafting.SpecialTokens(0, None))
    t_all = time.perf_counter()
    times, lengths = [], []
    for _ in range(steps_cap):
        t0 = time.perf_counter()
        try:
            out = next(it)
        except StopIteration:
            break
        times.append(time.perf_counter() - t0)
        lengths.append(int((out != 0).sum()))
        if len(times) >= 3 and time.perf_counter() - t_all > budget_s:
            break
    it.close()
    return {"times": times, "tokens_after_step": lengths, "cores": torch.get_num_threads(), "build_s": build_s, "B": B, "Lp": Lp}


def run_cpu(args, as_reference_arm: bool):
    lc, R, B, W, Lb, Lp, gen, dt, greedy, temp = CONFIGS[args.config]
    if not as_reference_arm:
        # the GPU arm's cpu_baseline: a bounded sample of the reference itself (prefill + 2 decode steps) in a child
        # process (its package has the same name as this repository's), or of the numpy port when that is not possible
        cpu = None
        if reference_unavailable_reason(args.config, 2, sample=True) is None:
            try:
                r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--sample", "--config", args.config],
                                   capture_output=True, text=True, timeout=420, env={k: v for k, v in os.environ.items()
                                                                                      if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")})
                if r.returncode == 0:
                    cpu = json.loads(r.stdout.strip().splitlines()[-1])["cpu_baseline"]
            except (subprocess.TimeoutExpired, ValueError, KeyError, IndexError):
                cpu = None
        return cpu if cpu is not None else run_port(args.config, 3, 40.0)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    want_steps = 3 if args.sample else max(args.warmup, 1) + args.steps
    why = reference_unavailable_reason(args.config, max(want_steps, 2), sample=args.sample)
    base = {"metric": metric_name(args.config), "unit": "tokens/s", "n_gpus": world, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": workload_config(args.config, world),
            "gpu_launches": 0}
    if why is not None:
        cpu = run_port(args.config, want_steps, 240.0)
        cpu["fallback_reason"] = why
        base.update({"value": cpu["value"], "steps": cpu["steps_timed"], "warmup": cpu["warmup"], "ms_per_step": cpu["ms_per_step_one_row"],
                     "cpu_baseline": cpu, "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        return base
    r = run_reference_impl(args.config, want_steps, 200.0 if args.config != "c1" else 600.0)
    times, lengths = r["times"], r["tokens_after_step"]
    # the first call holds the prefill; the steps after it are the decode steps of the metric
    step_times = times[1:] if len(times) > 1 else times
    gen_tokens = (lengths[-1] - lengths[0]) if len(lengths) > 1 else B
    value = gen_tokens / sum(step_times)
    whole = (lengths[-1] - B * Lp + B) / sum(times)  # prompt upload is nil on the CPU: prefill + all steps, first tokens included
    cpu = {"value": round(value, 4), "unit": "tokens/s", "cores": r["cores"], "kind": "reference",
           "sample": (f"the reference's RecurrentDrafting.generate (PyTorch {dt_name()} CPU, fp32) on the whole batch of {B} rows: prefill of {B}x{Lp} "
                      f"tokens ({times[0]:.1f} s with the first step), then {len(step_times)} decode step(s); weights filled in {r['build_s']:.0f} s (untimed)"),
           "first_call_s": round(times[0], 2)}
    if args.config != "c1" and not args.sample:
        port = run_port(args.config, 2, 45.0)
        cpu["port_cross_check"] = {"ms_per_step_one_row": port["ms_per_step_one_row"], "reference_ms_per_step_per_row": round(1e3 * sum(step_times) / len(step_times) / B, 1),
                                   "note": "numpy restatement on 1 row beside the reference's per-row step time"}
    base.update({"value": cpu["value"], "steps": len(step_times), "warmup": 0, "ms_per_step": round(1e3 * sum(step_times) / len(step_times), 2),
                 "cpu_baseline": cpu, "e2e": {"value": round(whole, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                                             "includes": "prefill + the timed steps"}})
    return base


def dt_name() -> str:
    import torch

    return torch.__version__


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=160)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sample", action="store_true", help="reference arm: bounded sample (prefill + 2 decode steps, no port cross-check)")
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
