"""The command line on the GPU, from a written model folder to tokens: the two tiny workloads of the
benchmark description (three prompts of 5, 9 and 13 tokens, 8 greedy steps; four prompts of 1, 7, 31 and 64
tokens, 16 steps at temperature 0.8 with a fixed seed), each token checked against the plain implementation."""
import json
from importlib import import_module

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def _run_cli(capsys, argv):
    cli = import_module("pytorch-engine_b200.cli")
    assert cli.main(argv) == 0
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    return sorted(lines, key=lambda r: r["request"])


def _prompts(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_cli_greedy_tiny_a(pe, tmp_path, capsys, dtype):
    folder = str(tmp_path / "a")
    pe.write_random_model(folder, pe.preset("tiny_a"), 0)
    cfg, w = plain.load_folder(folder)
    prompts = _prompts(cfg["vocab_size"], (5, 9, 13), 0)
    argv = ["--model", folder, "--dtype", dtype, "--max-tokens", "8", "--temperature", "0", "--json"]
    for p in prompts:
        argv += ["--prompt-ids", ",".join(map(str, p))]
    out = _run_cli(capsys, argv)
    assert [r["request"] for r in out] == [0, 1, 2] and [r["prompt_tokens"] for r in out] == [5, 9, 13]
    for r, p in zip(out, prompts):
        assert r["completion_tokens"] == 8 and r["finish_reason"] == "length"
        if dtype == "fp32":
            assert r["token_ids"] == plain.generate_greedy(cfg, w, p, 8)
        else:
            # bfloat16: each token is the plain implementation's best or, in a near tie, its runner-up
            plain.check_drawn_tokens(cfg, w, p, r["token_ids"], seed=0, request=r["request"], margin=0.05, temperature=0.0)


def test_cli_seeded_temperature_tiny_b(pe, tmp_path, capsys):
    folder = str(tmp_path / "b")
    pe.write_random_model(folder, pe.preset("tiny_b"), 1)
    cfg, w = plain.load_folder(folder)
    prompts = _prompts(cfg["vocab_size"], (1, 7, 31, 64), 1)
    base = ["--model", folder, "--dtype", "fp32", "--max-tokens", "16", "--temperature", "0.8", "--sampling-seed", "11", "--json"]
    argv = list(base)
    for p in prompts:
        argv += ["--prompt-ids", ",".join(map(str, p))]
    out = _run_cli(capsys, argv)
    differed = 0
    for r, p in zip(out, prompts):
        assert r["completion_tokens"] == 16 and r["prompt_tokens"] == len(p)
        # the command line's defaults are the reference's: top-k 40, top-p 0.95, min-p 0.05
        differed += plain.check_drawn_tokens(cfg, w, p, r["token_ids"], seed=11, request=r["request"], margin=1e-3,
                                             temperature=0.8, top_k=40, top_p=0.95, min_p=0.05)
    assert differed <= 2
    again = _run_cli(capsys, argv)
    assert [r["token_ids"] for r in again] == [r["token_ids"] for r in out]
    seed_at = argv.index("--sampling-seed") + 1
    other = _run_cli(capsys, argv[:seed_at] + ["12"] + argv[seed_at + 1:])
    assert [r["token_ids"] for r in other] != [r["token_ids"] for r in out]
