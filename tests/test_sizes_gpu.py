"""The engine against the plain implementation at Qwen3's own layer sizes (random weights): the whole
0.6B shape, and two layers of the 8B shape with its full vocabulary.  ``parity_at_size.py`` runs the
same comparison for any preset and number of layers from the command line."""
import pytest

from conftest import TOL
from parity_at_size import NOISE, run

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,layers,lengths,extra", [
    ("qwen3_0_6b", None, (96, 41), {}),
    ("qwen3_8b", 2, (96, 41), {}),
    # a prompt of more than 1,024 tokens at the 8B widths: the products run on the tcgen05 pair kernel with
    # K = 4,096 and 12,288, attention on the tcgen05 prefill kernel (one layer and a small vocabulary keep the
    # plain implementation on the CPU to some seconds)
    ("qwen3_8b", 1, (1200, 41), {"vocab_size": 8192}),
    # and of more than 2,048, where the output and down projections fill enough 256 x 256 tiles to run on the pair
    # kernel as well (at 1,200 rows they go to the library); two layers
    ("qwen3_8b", 2, (2100, 41), {"vocab_size": 4096}),
])
def test_parity_at_a_qwen3_size(preset, layers, lengths, extra):
    worst = run(preset, layers, lengths=lengths, verbose=False, **extra)
    assert len(worst) == 7
    for (dtype, way), err in worst.items():
        if way == NOISE:
            continue
        assert err < TOL[dtype], f"{preset} {dtype} {way}: worst error {err:.3e} (limit {TOL[dtype]:.0e})"


@pytest.mark.parametrize("preset,layers,tokens,dtype", [("qwen3_8b", 2, 20000, "bfloat16"), ("qwen3_8b", 1, 6000, "float32"),
                                                         ("qwen3_0_6b", 2, 33000, "bfloat16")])
def test_a_long_prompt_whole_and_cut_into_steps(preset, layers, tokens, dtype):
    """Tens of thousands of tokens: the prompt in one step against the same prompt in three steps of unequal
    lengths, and four decoded tokens after either (float32: equal bit for bit; bfloat16: within the drift that
    other ways of cutting show).  No plain implementation here: at these lengths it would take minutes."""
    import torch
    import pytorch_engine_b200 as pe
    from importlib import import_module

    StepEntry = import_module("pytorch-engine_b200.engine.batch").StepEntry
    vocab = 4096
    cfg = pe.config.preset(preset, num_hidden_layers=layers, vocab_size=vocab, max_position_embeddings=40960)
    eng = pe.Engine.from_random(cfg, seed=3, dtype=dtype, max_context_len=tokens + 128, max_cache_tokens=2 * (tokens + 192),
                                max_batch=2)
    g = torch.Generator().manual_seed(tokens)
    prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
    want = [0, tokens // 3, tokens - 2, tokens - 1]

    def decode(slot):
        return [eng.step([StepEntry(slot, [7 + i], [0])]).float().cpu().clone() for i in range(4)]

    s = eng.alloc_slot()
    whole = eng.step([StepEntry(s, prompt, want)]).float().cpu().clone()
    after_whole = decode(s)
    eng.free_slot(s)
    s = eng.alloc_slot()
    a, b = int(tokens * 0.37), int(tokens * 0.81)
    parts = []
    for lo, hi in ((0, a), (a, b), (b, tokens)):
        w = [x - lo for x in want if lo <= x < hi]
        out = eng.step([StepEntry(s, prompt[lo:hi], w)])
        if w:
            parts.append(out.float().cpu().clone())
    cut = torch.cat(parts)
    after_cut = decode(s)
    eng.free_slot(s)
    assert torch.isfinite(whole).all() and not eng.cache.live_slots
    scale = float(whole.abs().max())
    worst = max([float((whole - cut).abs().max())] + [float((x - y).abs().max()) for x, y in zip(after_whole, after_cut)]) / scale
    if dtype == "float32":
        assert worst == 0.0
    else:
        assert worst < 1e-2
