"""The plain implementation against logits that binief/pytorch-engine's own model code produced on
the CPU (tests/golden/make_golden.py wrote them; the reference is not needed to run this test)."""
import glob
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain
from golden.make_golden import weights_checksum

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "*.pt")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-3] for p in GOLDEN])
def test_plain_implementation_matches_the_reference(pe, tmp_path, path):
    g = torch.load(path)
    cfg = pe.Qwen3Config.from_dict(g["config"])
    pe.write_random_model(str(tmp_path), cfg, g["seed"])
    tensors = load_file(os.path.join(str(tmp_path), "model.safetensors"))
    if weights_checksum(tensors) != g["weights_sha256"]:
        pytest.skip("this torch build draws other random weights than the one the golden logits were made with")
    mine = plain.forward_logits(g["config"], tensors, g["tokens"])
    ref = g["logits"]
    assert mine.shape == ref.shape
    # the reference computes its linears in float16: about 1e-3 of the logits' scale
    assert float((mine - ref).abs().max()) < 2e-3 * float(ref.abs().max())


def test_golden_files_exist():
    assert len(GOLDEN) >= 2
