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


def bf16_close(oracle, got_bits, want_f32):
    """bf16 outputs agree with the rounded oracle value to one bf16 ulp of the value
    plus the f32 accumulation noise (3e-5 of the output RMS) that can move a value
    across a rounding boundary."""
    g = oracle.bf16_to_f32(np.asarray(got_bits, dtype=np.uint16)).astype(np.float64)
    w = np.asarray(want_f32, dtype=np.float64)
    rms = np.sqrt(np.mean(w * w)) + 1e-30
    return bool(np.all(np.abs(g - w) <= np.abs(w) * 2.0 ** -7 + 3e-5 * rms))
