"""Shared test set-up: the ``gpu`` marker, the package under its importable alias, and the tests'
own small configurations (they differ from each other in every size and option)."""
import importlib
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu on the GPU box")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def pe():
    return importlib.import_module("pytorch-engine_b200")


# The tests' own configurations.  A, B and C differ in every size and option: layers, width, head
# count, group size (2, 3, 1), head size (16, 32, 48: C's is no power of two), feed-forward width,
# vocabulary (C's and B's are no power of two), rope_theta, eps, tied or untied head, window.
TEST_CONFIGS = {
    "A": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=1024),
    "B": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
              num_key_value_heads=2, head_dim=32, intermediate_size=200, vocab_size=1000, rope_theta=1e6,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=768,
              use_sliding_window=True, sliding_window=40, max_window_layers=1),
    "C": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=1, hidden_size=80, num_attention_heads=5,
              num_key_value_heads=5, head_dim=48, intermediate_size=176, vocab_size=515, rope_theta=500000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=512,
              use_sliding_window=True, sliding_window=100, layer_types=["sliding_attention"], eos_token_id=[7, 9]),
    # D has a head size that the tensor-core attention kernels take (64), a group of 4 and a window
    "D": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=112, num_attention_heads=8,
              num_key_value_heads=2, head_dim=64, intermediate_size=304, vocab_size=300, rope_theta=100000.0,
              rms_norm_eps=2e-6, tie_word_embeddings=False, max_position_embeddings=1024,
              use_sliding_window=True, sliding_window=70, max_window_layers=1),
    # E has the head size of the tcgen05 prefill attention (128), a group of 4, full and windowed layers
    "E": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=144, num_attention_heads=4,
              num_key_value_heads=1, head_dim=128, intermediate_size=272, vocab_size=333, rope_theta=250000.0,
              rms_norm_eps=4e-6, tie_word_embeddings=True, max_position_embeddings=1024,
              use_sliding_window=True, sliding_window=90, layer_types=["sliding_attention", "full_attention"]),
}
TEST_SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}


def make_model_folder(pe, tmp_path_factory, key, sharpen=None):
    """Write config ``key`` with random weights into a fresh temporary folder.  ``sharpen`` scales the
    q-norm weights so that attention is peaked and single far keys matter."""
    from safetensors.torch import load_file, save_file

    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS[key])
    folder = str(tmp_path_factory.mktemp(f"model_{key}"))
    pe.write_random_model(folder, cfg, TEST_SEEDS[key])
    if sharpen:
        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        for name in list(tensors):
            if name.endswith("q_norm.weight"):
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
        save_file(tensors, path)
    return folder


# How much the q-norm weights are scaled.  Sharper attention shows a wrong key better, and it
# amplifies every rounding of a query or key by the same factor: float32 runs take 6, bfloat16 runs 3.
SHARPEN = {"float32": 6.0, "bfloat16": 3.0}


@pytest.fixture(scope="session")
def model_folders(pe, tmp_path_factory):
    """{dtype: {key: folder}} of the test models, attention sharpened (random weights alone give nearly
    uniform attention, which would hide a wrong key)."""
    return {dt: {k: make_model_folder(pe, tmp_path_factory, k, sharpen=f) for k in TEST_CONFIGS}
            for dt, f in SHARPEN.items()}


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest absolute difference relative to the largest reference magnitude."""
    return float((got.double() - ref.double()).abs().max() / ref.double().abs().max().clamp_min(1e-30))


# Tolerances, fixed before any measurement.  float32: accumulation-order effects only.
# bfloat16: about 25 roundings of relative size 2^-9 on the way to the logits.
TOL = {"float32": 3e-5, "bfloat16": 2e-2}
