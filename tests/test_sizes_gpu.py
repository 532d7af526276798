"""The engine against the plain implementation at Qwen3's own layer sizes (random weights): the whole
0.6B shape, and two layers of the 8B shape with its full vocabulary.  ``parity_at_size.py`` runs the
same comparison for any preset and number of layers from the command line."""
import pytest

from conftest import TOL
from parity_at_size import NOISE, run

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,layers", [("qwen3_0_6b", None), ("qwen3_8b", 2)])
def test_parity_at_a_qwen3_size(preset, layers):
    worst = run(preset, layers, verbose=False)
    assert len(worst) == 7
    for (dtype, way), err in worst.items():
        if way == NOISE:
            continue
        assert err < TOL[dtype], f"{preset} {dtype} {way}: worst error {err:.3e} (limit {TOL[dtype]:.0e})"
