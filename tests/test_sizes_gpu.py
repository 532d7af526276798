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
