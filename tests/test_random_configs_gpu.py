"""Configurations drawn at random (head sizes 16..256 in steps of 16, any number of heads and groups, widths and
vocabularies that are no power of two, one to three layers, windows on all, some or no layers, tied or untied head)
through the same comparison as the Qwen3 sizes: float32 and bfloat16; each prompt whole, with its last tokens one by
one, and in a batch of unequal lengths whose shortest request ends earlier; against the plain implementation."""
import random

import pytest

from conftest import TOL  # noqa: F401  (the limits that parity_at_size applies)
from parity_at_size import failures, run

pytestmark = pytest.mark.gpu

LENGTHS = [9, 17, 33, 63, 64, 65, 100, 127, 128, 129, 190, 257, 300, 511]


def random_config(seed: int):
    rng = random.Random(seed)
    layers = rng.choice([1, 2, 3])
    kv = rng.choice([1, 2, 3, 4])
    cfg = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=layers,
               hidden_size=rng.choice([48, 72, 80, 104, 136, 200, 264]),
               num_attention_heads=kv * rng.choice([1, 2, 3, 4, 5, 8]), num_key_value_heads=kv,
               head_dim=rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 160, 192, 256]),
               intermediate_size=rng.choice([88, 136, 200, 304]), vocab_size=rng.randrange(100, 2000),
               rope_theta=rng.choice([1e4, 5e5, 1e6]), rms_norm_eps=rng.choice([1e-6, 3e-6, 1e-5]),
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=1024)
    window = rng.choice(["none", "none", "all", "mix"])
    if window != "none":
        cfg.update(use_sliding_window=True, sliding_window=rng.randrange(8, 120))
        cfg["layer_types"] = (["sliding_attention"] * layers if window == "all" else
                              [rng.choice(["sliding_attention", "full_attention"]) for _ in range(layers)])
    lengths = tuple(rng.choice(LENGTHS) for _ in range(rng.choice([2, 3])))
    return cfg, lengths


@pytest.mark.parametrize("seed", range(16))
def test_a_configuration_drawn_at_random(pe, monkeypatch, seed):
    cfg_dict, lengths = random_config(1000 + seed)
    cfg = pe.Qwen3Config.from_dict(cfg_dict)
    monkeypatch.setattr(pe.config, "preset", lambda name, **over: cfg)
    worst = run("drawn at random", None, lengths=lengths, verbose=False, seed=seed)
    assert len(worst) == 7
    assert not failures(worst), f"{cfg_dict} with prompts of {lengths}: {failures(worst)}"
