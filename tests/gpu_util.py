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


# 17..32 activation rows of a large matrix run on the tcgen05 streaming matvec by default: bf16
# activations and weights dequantised to bf16 (one rounding of scale*q+bias), the numeric contract
# of affine_qmm, f32 accumulation. Against the oracle of that contract the kernel is held to
# f32-accumulation noise; against the f64 reference on unrounded weights to the north-star bound.
# Everything else (and everything, with LTHN_CUDA_BATCH_F32=1) runs on the f32-grade kernels,
# held to the f32 bound.
BATCH_CONTRACT_TOL_RMS = 2e-5
BATCH_REF_TOL_RMS = 1.2e-2   # worst output over the matrix, bf16 weight rounding: measured 4.5e-3 .. 7.8e-3 of the output RMS


def check_batched(oracle, got, x_f32, p, s, b, f32_grade, f32_tol=2e-5):
    """got [M, N] f32 from affine_qmv with M >= 3 rows of f32-representable activations x_f32."""
    ref = oracle.matnt_quant_host(x_f32, p, s, b, threads=8)
    # |got-ref| <= tol*(1+|ref|), the reference's own form: 1e-2 for the f32-grade kernels; the
    # bf16-rounded weights of the tensor-core contract reach 1.1e-2 on rows of 9216 codes
    assert rel_err(got, ref) <= (1e-2 if f32_grade else 1.5e-2)
    if f32_grade:
        assert rms_err(got, ref) <= f32_tol
        return
    want = oracle.proj_bf16_contract(x_f32, p, s, b)
    assert rms_err(got, want) <= BATCH_CONTRACT_TOL_RMS
    assert rms_err(got, ref) <= BATCH_REF_TOL_RMS
