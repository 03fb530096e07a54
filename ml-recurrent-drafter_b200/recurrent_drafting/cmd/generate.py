"""Command line of the decode loop, with the flags of the reference's
recurrent_drafting/cmd/generate.py (:252-270) and the statistics table its sweep scripts scrape
(benchmark/perf_wrt_candidates/make_csv.awk:8-20 reads the "Title: beamwidth..", "Average number
of tokens per step:" and "Tokens/second" lines).

    python -m recurrent_drafting.cmd.generate --hf_llm DIR --hf_drafter DIR --batch_size 8 \\
        --beam_width 45 --beam_length 5 --dtype bf16 --max_generation_length 512 --greedy_search

Differences that the missing network and datasets impose: prompts are token ids, either read from
--prompt_token_ids (a text file, one request per line, ids separated by blanks or commas) or drawn
uniformly at random (--synthetic_prompts N, the stand-in for --eval_mt_bench); --hf_llm and
--hf_drafter are checkpoint directories, or `random:NAME` (NAME in tiny, vicuna-7b, vicuna-13b) for
random-init weights of that architecture.  A tokenizer directory is optional and only used to print
text.  There is no CPU path: --use_gpu must name a CUDA device.
"""
import argparse
import sys
from typing import Generator, Iterable, List, Optional, Sequence

import torch

ARCHITECTURES = {
    "tiny": dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=2, intermediate_size=688, vocab_size=1000),
    "vicuna-7b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=32, num_hidden_layers=32, intermediate_size=11008,
                      vocab_size=32000),
    "vicuna-13b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=40, num_hidden_layers=40, intermediate_size=13824,
                       vocab_size=32000),
}


def define_flags() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hf_tokenizer", default=None, help="Tokenizer directory (optional; only to print text).")
    ap.add_argument("--hf_llm", default="random:tiny", help="Base LLM checkpoint directory, or random:NAME.")
    ap.add_argument("--hf_drafter", required=True, help="Drafter checkpoint directory, or random:LAYERS (residual blocks).")
    ap.add_argument("--eval_mt_bench", action="store_true", help="Accepted for compatibility: synthetic prompts are used.")
    ap.add_argument("--prompt_token_ids", default=None, help="Text file with one request per line (token ids).")
    ap.add_argument("--synthetic_prompts", type=int, default=0, help="Number of random prompts of --max_prompt_length tokens.")
    ap.add_argument("--max_prompt_length", type=int, default=50)
    ap.add_argument("--max_num_prompts", type=int, default=-1)
    ap.add_argument("--max_generation_length", type=int, default=60)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--beam_length", type=int, default=-1)
    ap.add_argument("--beam_width", type=int, default=10)
    ap.add_argument("--autoregression", action="store_true")
    ap.add_argument("--greedy_search", action="store_true")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--rng_seed", type=int, default=123)
    ap.add_argument("--use_gpu", type=int, default=0)
    ap.add_argument("--dtype", default="bf16", choices=["fp32", "bf16"])
    ap.add_argument("--pad_token_id", type=int, default=0)
    ap.add_argument("--eos_token_id", type=int, default=-1, help="Negative: never stop early.")
    return ap


def read_prompt_token_ids(path: str, max_length: int, max_num_prompts: int) -> Generator[List[int], None, None]:
    """Requests shorter than max_length, at most max_num_prompts of them (cmd/generate.py:90-104)."""
    n = 0
    with open(path) as fh:
        for line in fh:
            ids = [int(x) for x in line.replace(",", " ").split()]
            if 2 < len(ids) < max_length and (max_num_prompts < 0 or n < max_num_prompts):
                n += 1
                yield ids


def synthetic_prompts(n: int, length: int, vocab: int, seed: int) -> Generator[List[int], None, None]:
    g = torch.Generator().manual_seed(seed)
    for _ in range(n):
        yield torch.randint(3, vocab, (length,), generator=g).tolist()


def batch(prompts: Iterable[List[int]], batch_size: int) -> Generator[List[List[int]], None, None]:
    """Full batches only, as the reference's batch() (cmd/generate.py:107-116)."""
    b: List[List[int]] = []
    for p in prompts:
        b.append(p)
        if len(b) >= batch_size:
            yield b
            b = []


def left_pad(rows: Sequence[List[int]], pad_id: int) -> torch.Tensor:
    """(batch, longest) int64 with pad ids on the left, what a tokenizer with padding_side="left" returns."""
    longest = max(len(r) for r in rows)
    out = torch.full((len(rows), longest), pad_id, dtype=torch.int64)
    for i, r in enumerate(rows):
        out[i, longest - len(r) :] = torch.tensor(r, dtype=torch.int64)
    return out


def load_models(args, device):
    from transformers.models.llama.configuration_llama import LlamaConfig

    from .. import configuration_drafter, modeling_drafter, modeling_llama

    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}[args.dtype]
    if args.hf_llm.startswith("random:"):
        cfg = LlamaConfig(rms_norm_eps=1e-6, hidden_act="silu", pad_token_id=args.pad_token_id, **ARCHITECTURES[args.hf_llm.split(":", 1)[1]])
        cfg.rope_theta = 10000.0
        with torch.device(device):
            llm = modeling_llama.LlamaForCausalLM(cfg).to(dtype)
        llm.init_random(0.02, seed=args.rng_seed)
    else:
        llm = modeling_llama.LlamaForCausalLM.from_pretrained(args.hf_llm, torch_dtype=dtype, device=device)
    if args.hf_drafter.startswith("random:"):
        H, V = llm.config.hidden_size, llm.config.vocab_size
        dcfg = configuration_drafter.DrafterConfig(vocab_size=V, hidden_size=H, exit_dim=2 * H,
                                                   num_draft_layers=int(args.hf_drafter.split(":", 1)[1]), rnn=True)
        with torch.device(device):
            drafter = modeling_drafter.Drafter(dcfg).to(dtype)
        drafter.init_random(0.02, seed=args.rng_seed + 1)
    else:
        drafter = modeling_drafter.Drafter.from_pretrained(args.hf_drafter, torch_dtype=dtype, device=device)
    return llm, drafter


def main(argv: Optional[List[str]] = None) -> int:
    from .. import RecurrentDrafting, SamplingArgs, SpecialTokens, autoregressive, modeling_drafter, rng, stats

    args = define_flags().parse_args(argv)
    rng.seed_pytorch(args.rng_seed)
    if args.use_gpu < 0 or not torch.cuda.is_available():
        print("this implementation has no CPU path: --use_gpu must name a CUDA device", file=sys.stderr)
        return 2
    device = torch.device(f"cuda:{args.use_gpu}")
    torch.cuda.set_device(device)
    llm, drafter = load_models(args, device)
    model = RecurrentDrafting(llm, drafter)
    special = SpecialTokens(args.pad_token_id, args.eos_token_id if args.eos_token_id >= 0 else None)
    tokenizer = None
    if args.hf_tokenizer:
        import transformers

        tokenizer = transformers.AutoTokenizer.from_pretrained(args.hf_tokenizer, padding_side="left")
    if args.prompt_token_ids:
        prompts = read_prompt_token_ids(args.prompt_token_ids, args.max_prompt_length, args.max_num_prompts)
    else:
        n = args.synthetic_prompts or args.batch_size
        if args.max_num_prompts >= 0:
            n = min(n, args.max_num_prompts)
        prompts = synthetic_prompts(n, args.max_prompt_length - 1, llm.config.vocab_size, args.rng_seed)
    ledger = stats.Ledger()
    shape = modeling_drafter.BeamShape(args.beam_width, args.beam_length)
    max_length = args.max_prompt_length + args.max_generation_length
    for rows in batch(prompts, args.batch_size):
        input_ids = left_pad(rows, args.pad_token_id).to(device)
        if args.autoregression:
            outputs = autoregressive.generate(model, input_ids, max_length, special)
        else:
            outputs = model.generate(ledger, input_ids, max_length, shape, SamplingArgs(args.temperature, args.greedy_search), special)
        last = None
        for last in outputs:
            pass
        if last is not None:
            print(tokenizer.batch_decode(last) if tokenizer is not None else last.tolist())
    if not args.autoregression:
        ts, ps = stats.summarize(ledger, args.batch_size, args.beam_length)
        title = f"beamwidth{args.beam_width}_beamlen{args.beam_length}"
        stats.draw_table(title, ts)
        stats.draw_figure(title, ps, "/tmp/title.png")
    return 0


if __name__ == "__main__":
    sys.exit(main())
