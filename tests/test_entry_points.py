"""Command line, entry point and replay program without a GPU: options, errors, and the refusal
to run without CUDA (there is no CPU fallback)."""
import io
import json
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, TEST_CONFIGS


def test_cli_options_follow_the_reference(pe):
    from importlib import import_module
    cli = import_module("pytorch-engine_b200.cli")
    args = cli.build_parser().parse_args(["--model", "m", "--prompt-ids", "1,2,3", "--prompt-ids", "4 5"])
    # defaults of the reference's SamplingConfig and of its --ctx / --no-cuda-graph flags
    assert (args.max_tokens, args.temperature, args.top_k, args.top_p, args.min_p, args.repetition_penalty) == \
        (512, 0.7, 40, 0.95, 0.05, 1.0)
    assert args.ctx is None and args.no_cuda_graph is False and args.dtype == "bf16"
    assert [cli._ids(t) for t in args.prompt_ids] == [[1, 2, 3], [4, 5]]


def test_cli_needs_exactly_one_model_source(pe, capsys):
    from importlib import import_module
    cli = import_module("pytorch-engine_b200.cli")
    assert cli.main(["--prompt-ids", "1"]) == 2
    assert cli.main(["--model", "x", "--random", "tiny_a", "--prompt-ids", "1"]) == 2
    assert "exactly one" in capsys.readouterr().err
    assert cli.main(["--list-presets"]) == 0
    assert "qwen3_8b" in capsys.readouterr().out


def test_cli_writes_a_random_model(pe, tmp_path):
    from importlib import import_module
    cli = import_module("pytorch-engine_b200.cli")
    assert cli.main(["--random", "tiny_a", "--seed", "4", "--write-random", str(tmp_path / "m")]) == 0
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    assert pe.load_config(str(tmp_path / "m")) == pe.preset("tiny_a")


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the refusal on a machine without CUDA")
def test_no_cuda_no_engine(pe, tmp_path):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS["A"])
    pe.write_random_model(str(tmp_path), cfg, 0)
    with pytest.raises(pe.kernels.KernelError, match="no CPU path"):
        pe.Engine(str(tmp_path))
    with pytest.raises(pe.kernels.KernelError):
        pe.kernels.ops.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))


def test_trace_run_rejects_bad_arguments():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", "nowhere"],
                          capture_output=True, text=True, timeout=120)
    assert proc.returncode != 0 and "--out" in proc.stderr


def test_replayer_bookkeeping_with_a_scripted_engine(pe, tmp_path):
    """The replayer gives a slot at a request's first appearance, returns it at ``end``, writes a file
    only when something is wanted, and refuses to end what is not live."""

    class FakeEngine:
        def __init__(self):
            self.next, self.freed, self.calls = 0, [], []

        def alloc_slot(self):
            self.next += 1
            return self.next - 1

        def free_slot(self, s):
            self.freed.append(s)

        def step(self, entries):
            self.calls.append([(e.slot, list(e.tokens), tuple(e.want)) for e in entries])
            n = sum(len(e.want) for e in entries)
            return torch.arange(n * 3, dtype=torch.float32).view(n, 3)

    eng = FakeEngine()
    rp = pe.engine.TraceReplayer(eng, str(tmp_path))
    out = io.StringIO()
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}, {"id": "b", "tokens": [3], "want": []}], "end": []}),
             "", json.dumps({"step": 1, "entries": [{"id": "a", "tokens": [4], "want": []}, {"id": "b", "tokens": [5], "want": []}], "end": ["a"]}),
             json.dumps({"step": 5, "entries": [{"id": "c", "tokens": [6], "want": [0]}], "end": ["b", "c"]})]
    assert rp.run(io.StringIO("\n".join(lines) + "\n"), out) == 0
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "5"]
    assert sorted(os.listdir(tmp_path)) == ["0.f32", "5.f32"]
    assert eng.calls[0] == [(0, [1, 2], (1,)), (1, [3], ())] and eng.calls[2] == [(2, [6], (0,))]
    assert eng.freed == [0, 1, 2] and rp.slots == {}
    assert os.path.getsize(tmp_path / "0.f32") == 12
    with pytest.raises(pe.engine.replay.TraceError):
        rp.run_step({"step": 6, "entries": [], "end": ["zz"]})


def test_default_cache_size_is_capped_by_free_memory(pe):
    import torch
    CR = pe.parts.CacheRequest
    reqs = {i: CR("kv", kv_heads=8, head_dim=128) for i in range(28)}
    per_token = 28 * 2 * 8 * 128 * 2
    f = pe.Engine.default_cache_tokens
    # plenty of memory: max_batch sequences of full length, in whole pages
    assert f(4, 100, reqs, torch.bfloat16, "cpu", free_bytes=1 << 50) == 4 * 128
    # 64 sequences of 40,960 tokens would take 300 GB: four fifths of what is free instead, in whole pages
    got = f(64, 40960, reqs, torch.bfloat16, "cpu", free_bytes=100 << 30)
    assert got % 64 == 0 and got * per_token <= 0.8 * (100 << 30) < (got + 64) * per_token
    # nothing paged: no limit from memory
    assert f(2, 64, {0: CR("state", state_shapes=(("s", (4,), "float32"),))}, torch.float32, "cpu", free_bytes=1) == 128
    assert f(2, 64, reqs, torch.float32, "cpu", free_bytes=10) == 64


def test_large_products_that_fill_their_waves_badly_go_to_the_library(pe):
    import importlib
    fill = importlib.import_module("pytorch-engine_b200.parts.runtime").large_gemm_fill
    assert fill(256, 256 * 74, 148) == 1.0                      # one full wave
    assert abs(fill(1536, 4096, 148) - 96 / 148) < 1e-9         # 96 tiles need two waves of 74
    assert fill(2048, 6144, 148) > 0.8 > fill(1024, 6144, 148)
    assert fill(1, 1, 2) == 1.0


def test_cli_text_prompts_need_a_tokenizer_file(pe, tmp_path, capsys):
    from importlib import import_module
    cli = import_module("pytorch-engine_b200.cli")
    assert cli.main(["--random", "tiny_a", "--write-random", str(tmp_path / "m")]) == 0
    assert cli.load_tokenizer(str(tmp_path / "m")) is None
    assert cli.main(["--model", str(tmp_path / "m"), "--prompt", "hello there"]) == 2
    assert "tokenizer.json" in capsys.readouterr().err
    tokenizers = pytest.importorskip("tokenizers")
    vocab = {"[UNK]": 0, "hello": 1, "there": 2}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.save(str(tmp_path / "m" / "tokenizer.json"))
    loaded = cli.load_tokenizer(str(tmp_path / "m"))
    assert loaded.encode("hello there you").ids == [1, 2, 0]


def test_reference_arm_and_plain_baseline_of_the_benchmark_run(pe):
    """The two things ``bench.py`` compares the engine with, on the CPU at a tiny size: the reference arm (the
    unmodified reference from ``baseline/_ref``, skipped where that copy is absent; it imports nothing of this
    package) and the plain PyTorch model."""
    import importlib.util

    def load(name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "baseline", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    cfg = pe.preset("tiny_b").to_dict()
    plain_torch = load("plain_torch")
    m = plain_torch.PlainTorchModel(cfg, cfg["num_hidden_layers"], "cpu", dtype=torch.float32)
    m.alloc_cache(2, 40)
    ids = torch.randint(0, cfg["vocab_size"], (2, 20))
    whole = m.forward(ids, 0, last_only=False)
    m.alloc_cache(2, 40)
    head = m.forward(ids[:, :19], 0)
    last = m.forward(ids[:, 19:], 19)
    assert whole.shape == (2, 20, cfg["vocab_size"]) and float((last[:, -1] - whole[:, -1]).abs().max()) < 1e-5
    arm = load("reference_arm")
    if arm.find_reference() is None:
        pytest.skip("no copy of the reference under baseline/_ref")
    pytest.importorskip("gguf")
    out = arm.run(cfg, preset_name="tiny_b", batch=2, context=64, steps=6, warmup=2, device="cpu", log=lambda m: None)
    assert out["impl"] == "reference" and "unavailable" not in out
    assert out["e2e"]["tokens"] == 12 and out["value"] > 0 and out["config"]["layers"] == 3
    assert "pytorch-engine_b200" not in open(os.path.join(ROOT, "baseline", "reference_arm.py")).read().split('"""', 2)[2]
