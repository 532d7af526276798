"""The plain implementation against logits that binief/pytorch-engine's own model code produced on
the CPU (tests/golden/make_golden.py wrote them; the reference is not needed to run this test)."""
import glob
import os
import subprocess
import sys

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain
from conftest import ROOT
from golden.make_golden import weights_checksum

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "*.pt")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-3] for p in GOLDEN])
def test_plain_implementation_matches_the_reference(pe, tmp_path, path):
    g = torch.load(path)
    cfg = pe.Qwen3Config.from_dict(g["config"])
    pe.write_random_model(str(tmp_path), cfg, g["seed"])
    tensors = load_file(os.path.join(str(tmp_path), "model.safetensors"))
    if weights_checksum(tensors) != g["weights_sha256"]:
        # this torch build draws other random weights than the one the stored logits were made with: make them
        # anew from the reference's code if a copy of it is at hand, else fail (a silent skip would drop the one
        # anchor on the reference's own output)
        ref_root = next((c for c in (os.environ.get("PE_B200_REFERENCE", ""), os.path.join(ROOT, "baseline", "_ref"))
                         if c and os.path.isfile(os.path.join(c, "pygguf_engine", "model.py"))), None)
        if ref_root is None:
            pytest.fail("the stored golden logits belong to other random weights than this torch build draws, and no "
                        "copy of the reference is at hand to make them anew: set PE_B200_REFERENCE to a checkout of "
                        "binief/pytorch-engine, or run tests/golden/make_golden.py there and commit its output")
        script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_golden.py")
        out = tmp_path / "regenerated"
        out.mkdir()
        subprocess.run([sys.executable, script, ref_root, "--out", str(out)], check=True, timeout=600)
        g = torch.load(str(out / os.path.basename(path)))
        assert weights_checksum(tensors) == g["weights_sha256"]
    mine = plain.forward_logits(g["config"], tensors, g["tokens"])
    ref = g["logits"]
    assert mine.shape == ref.shape
    # the reference computes its linears in float16: about 1e-3 of the logits' scale
    assert float((mine - ref).abs().max()) < 2e-3 * float(ref.abs().max())


def test_golden_files_exist():
    assert len(GOLDEN) >= 2
