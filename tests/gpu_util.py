"""Helpers shared by the GPU parity tests."""
import numpy as np


def make_weight(oracle, N, K, seed, bits=4, gs=64, sigma=0.02, variant=0):
    """N(0, sigma) weight (NumPy default_rng(seed)), bf16-representable, quantised by the oracle."""
    w = (np.random.default_rng(seed).standard_normal((N, K)) * sigma).astype(np.float32)
    w = oracle.bf16_to_f32(oracle.f32_to_bf16(w))
    return oracle.quantize(w, bits, gs, variant)


def make_x(oracle, M, K, seed):
    x = np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)
    xb = oracle.f32_to_bf16(x)
    return oracle.bf16_to_f32(xb), xb


def rel_err(got, want):
    """max |got-want| / (1+|want|): the reference's own tolerance form
    (engine/metal/quant_seam_backend_test.go:46-89)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(got - want) / (1.0 + np.abs(want))))


def rms_err(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(got - want)) / (np.sqrt(np.mean(want * want)) + 1e-30))
