"""Oracle vs golden vectors produced by the reference's own NumPy dequantiser
(tests/golden/make_golden.py records how the file was generated)."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "mlxaffine_dequant_golden.npz")


def golden_cases():
    z = np.load(GOLDEN)
    names = sorted({k.rsplit(".", 1)[0] for k in z.files})
    return z, names


def test_oracle_dequant_matches_reference_tool(oracle):
    z, names = golden_cases()
    assert len(names) == 4
    for n in names:
        bits, gs = (int(v) for v in z[n + ".meta"])
        got = oracle.dequantize(z[n + ".packed"], z[n + ".scales"], z[n + ".biases"], bits, gs)
        assert np.array_equal(got.view(np.uint32), z[n + ".dequant"].view(np.uint32)), n


def test_oracle_quantizer_reproduces_golden_bytes(oracle):
    """Re-quantising the golden dequantised values gives back the golden codes
    (mlxaffine_test.go:87-112 fixed-point property; the reference asserts it for
    its 4-bit synthWeight tensor, whose groups span their full code range)."""
    z, names = golden_cases()
    for n in ("synth_b4_g64", "synth_b2_g64"):
        bits, gs = (int(v) for v in z[n + ".meta"])
        p, _, _ = oracle.quantize(z[n + ".dequant"], bits, gs)
        assert np.array_equal(p, z[n + ".packed"]), n
