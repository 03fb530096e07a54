"""The command line and the statistics table in the form the reference's sweep scripts scrape
(recurrent_drafting/cmd/generate.py:156-174, 252-270; stats.py:218-241;
benchmark/perf_wrt_candidates/make_csv.awk:8-20)."""
import re

import pytest
import torch


def test_draw_table_prints_the_lines_the_awk_script_matches(capsys):
    from recurrent_drafting import stats

    ts = stats.TableStats(avg_token_per_step=2.5, acceptance_rate=37.5, avg_generate_candidates=0.002, avg_verify_candidates=0.011,
                          avg_accept_candidate_tokens=0.0005, avg_step_time=0.0135)
    stats.draw_table("beamwidth45_beamlen5", ts)
    out = capsys.readouterr().out
    # make_csv.awk: /Title: beamwidth/ with beamwidth([0-9]+)_beamlen([0-9]+)
    m = re.search(r"Title: beamwidth([0-9]+)_beamlen([0-9]+)", out)
    assert m and m.groups() == ("45", "5")
    # /Average number of tokens per step:/ -> "^Average number of tokens per step: +(.*)$"
    line = [l for l in out.splitlines() if "Average number of tokens per step:" in l][0]
    assert float(re.match(r"^Average number of tokens per step: +(.*)$", line).group(1)) == 2.5
    # /Tokens\/second/ -> "^Tokens/second +(.*)$"
    line = [l for l in out.splitlines() if "Tokens/second" in l][0]
    assert abs(float(re.match(r"^Tokens/second +(.*)$", line).group(1)) - 2.5 / 0.0135) < 1e-3
    assert "Average draft head acceptance rate (%):" in out and "verify_candidates:" in out


def test_prompt_helpers(tmp_path):
    from recurrent_drafting.cmd import generate as cli

    p = tmp_path / "prompts.txt"
    p.write_text("5 6 7 8\n1 2\n9,10,11,12,13\n" + " ".join(str(i) for i in range(3, 80)) + "\n20 21 22\n")
    rows = list(cli.read_prompt_token_ids(str(p), 50, -1))
    assert rows == [[5, 6, 7, 8], [9, 10, 11, 12, 13], [20, 21, 22]]
    assert list(cli.read_prompt_token_ids(str(p), 50, 2)) == rows[:2]
    assert [len(b) for b in cli.batch(iter(rows), 2)] == [2]  # full batches only
    padded = cli.left_pad(rows[:2], 0)
    assert padded.tolist() == [[0, 5, 6, 7, 8], [9, 10, 11, 12, 13]]
    args = cli.define_flags().parse_args(["--hf_drafter", "random:1", "--beam_width", "4", "--beam_length", "3", "--greedy_search"])
    assert (args.beam_width, args.beam_length, args.greedy_search, args.dtype, args.rng_seed) == (4, 3, True, "bf16", 123)
    assert len(list(cli.synthetic_prompts(3, 7, 100, 1))) == 3


@pytest.mark.gpu
def test_cli_runs_and_prints_the_table(capsys):
    from recurrent_drafting.cmd import generate as cli

    rc = cli.main(["--hf_llm", "random:tiny", "--hf_drafter", "random:1", "--batch_size", "2", "--synthetic_prompts", "4", "--beam_width", "4",
                   "--beam_length", "3", "--dtype", "fp32", "--max_prompt_length", "16", "--max_generation_length", "12", "--greedy_search"])
    assert rc == 0
    out = capsys.readouterr().out
    assert re.search(r"^Tokens/second +[0-9.]+$", out, re.M) and "Title: beamwidth4_beamlen3" in out
    assert re.search(r"^Average number of tokens per step: +[0-9.]+$", out, re.M)


def test_cli_refuses_cpu():
    from recurrent_drafting.cmd import generate as cli

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert cli.main(["--hf_drafter", "random:1", "--use_gpu", "-1"]) == 2
