"""Per-step timing ledger with the reference's API (recurrent_drafting/stats.py).

Phases are timed with CUDA events recorded on the current stream, resolved once per step after the
step's single host synchronisation, instead of a device-wide synchronise on both sides of every
phase.  The ledger file format (one JSON object per generate call) and summarize()/draw_table()
outputs are those the reference's benchmark scripts parse."""
from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import tempfile
import time
from collections import defaultdict
from typing import Any, DefaultDict, Dict, Generator, List, Tuple

import numpy as np
import torch


class TextGeneration:
    """Stats of one call to RecurrentDrafting.generate (stats.py:47-96)."""

    def __init__(self) -> None:
        self.n_steps = 0
        self.wall_times: Dict[str, List[float]] = {}
        self.stats: Dict[str, Any] = {"step": [], "wall_times": self.wall_times}

    @contextlib.contextmanager
    def step(self) -> Generator["TextGeneration.Step", None, None]:
        r = TextGeneration.Step(self)
        self.stats["step"].append(self.n_steps)
        self.n_steps += 1
        try:
            yield r
        finally:
            r.resolve()

    class Step:
        def __init__(self, gr: "TextGeneration") -> None:
            self._gr = gr
            self._pending: List[Tuple[str, Any, Any]] = []

        @contextlib.contextmanager
        def time(self, key: str) -> Generator[None, None, None]:
            with torch.profiler.record_function(key):
                if torch.cuda.is_available():
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    yield
                    end.record()
                    self._pending.append((key, start, end))
                else:
                    t0 = time.perf_counter()
                    yield
                    self._pending.append((key, t0, time.perf_counter()))

        def resolve(self) -> None:
            """Turns recorded event pairs into seconds.  Called after the step's host sync."""
            for key, a, b in self._pending:
                if isinstance(a, float):
                    elapsed = b - a
                else:
                    b.synchronize()
                    elapsed = a.elapsed_time(b) / 1e3
                self._gr.wall_times.setdefault(key, []).append(elapsed)
            self._pending.clear()

        def set(self, d: Dict[str, Any]) -> None:
            for k, v in d.items():
                self._gr.stats.setdefault(k, []).append(v)


@contextlib.contextmanager
def text_generation(ledger: "Ledger") -> Generator[TextGeneration, None, None]:
    r = TextGeneration()
    yield r
    ledger.post(r.stats)


class Ledger:
    """A list of JSON records in a temporary file (stats.py:105-136)."""

    def __init__(self, *, prefix: str = "") -> None:
        self.folder = tempfile.TemporaryDirectory(prefix=prefix)
        self.fn = os.path.join(self.folder.name, "stats.jsonl")
        self.fp = open(self.fn, "w+")
        self._locked = False

    def __del__(self) -> None:
        try:
            self.cleanup()
        except Exception:
            pass

    def lock(self) -> None:
        if not self._locked:
            self.fp.close()
            self._locked = True

    def cleanup(self) -> None:
        self.lock()
        self.fn = ""
        self.folder.cleanup()

    def post(self, d: Dict[str, Any]) -> None:
        if self._locked:
            raise RuntimeError("ledger is locked")
        self.fp.write(json.dumps(d) + "\n")

    @contextlib.contextmanager
    def reader(self) -> Generator[Any, None, None]:
        self.lock()
        with open(self.fn, "r") as fp:
            yield (json.loads(line) for line in fp if line.strip())


@dataclasses.dataclass
class PlotStats:
    sorted_steps: List[str]
    sorted_num_tokens_step: List[float]
    sorted_input_lengths: List[str]
    sorted_num_tokens_input_length: List[float]
    acceptance_rate: float


@dataclasses.dataclass
class TableStats:
    avg_token_per_step: float
    acceptance_rate: float
    avg_generate_candidates: float
    avg_verify_candidates: float
    avg_accept_candidate_tokens: float
    avg_step_time: float


def summarize(ledger: Ledger, batch_size: int, candidate_len: int) -> Tuple[TableStats, PlotStats]:
    """Tokens/step, acceptance rate and mean phase times (stats.py:158-215)."""
    by_step: DefaultDict[Any, List[float]] = defaultdict(list)
    by_len: DefaultDict[Any, List[float]] = defaultdict(list)
    phases: Dict[str, List[float]] = {"generate_candidates": [], "verify_candidates": [], "accept_candidate_tokens": []}
    with ledger.reader() as reader:
        for rec in reader:
            for step, acc in zip(rec["step"], rec["avg_num_accepted"]):
                by_step[step].append(batch_size * (float(acc) + 1))
            for length, acc in zip(rec["input_id_length"], rec["avg_num_accepted"]):
                by_len[length].append(batch_size * (float(acc) + 1))
            for k in phases:
                phases[k] += rec["wall_times"][k]
    steps = sorted(by_step)
    lens = sorted(by_len)
    total_steps = sum(len(by_step[s]) for s in steps)
    total_tokens = sum(sum(by_step[s]) for s in steps)
    per_step = total_tokens / total_steps
    acceptance = 100.0 * (per_step - batch_size) / batch_size / candidate_len
    means = {k: float(np.mean(np.array(v))) for k, v in phases.items()}
    table = TableStats(per_step / batch_size, acceptance, means["generate_candidates"], means["verify_candidates"],
                       means["accept_candidate_tokens"], sum(means.values()))
    plot = PlotStats(steps, [sum(by_step[s]) / len(by_step[s]) for s in steps], lens,
                     [sum(by_len[n]) / len(by_len[n]) for n in lens], acceptance)
    return table, plot


def draw_table(title: str, ts: TableStats) -> None:
    """Prints the table the reference's sweep scripts scrape ("Tokens/second", "Average number of
    tokens per step:"; stats.py:218-241)."""
    from tabulate import SEPARATING_LINE, tabulate

    print(os.linesep)
    print(tabulate(
        [
            ["Average number of tokens per step:", f"{ts.avg_token_per_step:.4f}"],
            ["Average draft head acceptance rate (%):", f"{ts.acceptance_rate:.4f}"],
            SEPARATING_LINE,
            ["Wall time (seconds) per step", ""],
            ["", ""],
            ["generate_candidates:", f"{ts.avg_generate_candidates:.4f}"],
            ["verify_candidates:", f"{ts.avg_verify_candidates:.4f}"],
            ["accept_candidate_tokens:", f"{ts.avg_accept_candidate_tokens:.4f}"],
            SEPARATING_LINE,
            ["Tokens/second", f"{ts.avg_token_per_step / ts.avg_step_time:.4f}"],
            SEPARATING_LINE,
        ],
        headers=[f"Title: {title}", ""],
        colalign=("left", "right"),
    ))


def draw_figure(title: str, ps: PlotStats, filename: str) -> None:
    pass
