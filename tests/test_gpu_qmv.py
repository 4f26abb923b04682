"""affine_qmv parity through the C ABI against the CPU oracle.

Tolerances: the north-star bound is max relative error <= 1e-2 against an fp32
reference on the dequantised weights; the reference's own tests use
|got-want| <= 1e-2*(1+|want|) (engine/metal/quant_seam_backend_test.go:46-89) and
0.05 absolute on the bf16 fixture (enginetest/quant_parity.go:23). The kernel is
held to much tighter bounds here (f32 accumulation): 2e-5 of the output RMS."""
import numpy as np
import pytest

from gpu_util import bf16_close, check_batched, make_weight, make_x, rel_err, rms_err
from test_oracle_kat import parity_fixture

pytestmark = pytest.mark.gpu

F32_TOL_RMS = 2e-5   # f32 output vs f64 oracle, relative to output RMS
REF_TOL = 1e-2       # the reference's tolerance form


def run_qmv(lthn, x_arr, x_dtype, M, q, y_dtype):
    xb = lthn.Buf.from_array(x_arr)
    y = lthn.Buf(M * q.N * (2 if y_dtype == lthn.BF16 else 4))
    lthn.qmv(xb, x_dtype, M, q, y, y_dtype)
    lthn.sync()
    return y.download(np.uint16 if y_dtype == lthn.BF16 else np.float32, (M, q.N))


# --- enginetest.QuantParity (quant_parity.go:77-108) through MatVec ---
def test_quant_parity_fixture_matvec(oracle):
    import lthn
    x, packed, scales, biases, out_dim, in_dim, gs, bits = parity_fixture(oracle)
    got = lthn.qmv_host(x, packed, scales, biases, out_dim, in_dim, gs, bits)
    want = oracle.ref_affine_matvec(x, packed, scales, biases, out_dim, in_dim, gs, bits)
    if not np.array_equal(got, want):
        assert np.max(np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want))) <= 0.05
    # held tighter than the reference asks: at most one bf16 ulp
    assert np.max(np.abs(got.astype(np.int32) - want.astype(np.int32))) <= 1


# --- engine/metal/quant_seam_backend_test.go:46-89 shapes (qmv M=1 and M>1, ragged N, 2/8 bit) ---
@pytest.mark.parametrize("M,K,N,bits,gs", [(1, 512, 40, 4, 64), (1, 256, 24, 2, 128), (3, 512, 64, 4, 64),
                                           (5, 256, 40, 2, 128), (2, 128, 8, 8, 64)])
def test_seam_fixture_shapes(oracle, M, K, N, bits, gs):
    import lthn
    w = (((np.arange(N * K) % 17) - 8) * np.float32(0.037)).astype(np.float32).reshape(N, K)
    x = (((np.arange(M * K) % 9) - 4) * np.float32(0.05)).astype(np.float32).reshape(M, K)
    p, s, b = oracle.quantize(w, bits, gs)
    want = oracle.matnt(x, oracle.dequantize(p, s, b, bits, gs))
    q = lthn.QuantWeight.from_host(p, s, b, bits, gs)
    got = run_qmv(lthn, x, lthn.F32, M, q, lthn.F32)
    assert rel_err(got, want) <= REF_TOL
    xb = oracle.f32_to_bf16(x)
    got_b = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
    assert rms_err(got, want) <= 1e-4
    want_b = oracle.matnt(oracle.bf16_to_f32(xb), oracle.dequantize(p, s, b, bits, gs))
    assert rms_err(got_b, want_b) <= 1e-4


@pytest.fixture(params=["tcgen05", "f32"])
def batch_f32(request, monkeypatch):
    """Both kernels that serve 3..32 rows, each forced for the whole test: the tcgen05 streaming
    matvec (bf16 contract; the default for 17..32 rows of a large matrix) and the f32-grade
    bf16-split mma.sync kernel (the default otherwise; LTHN_CUDA_BATCH_F32=1 keeps it everywhere)."""
    import lthn
    if request.param == "f32":
        monkeypatch.setenv("LTHN_CUDA_BATCH_F32", "1")
        yield True
    else:
        monkeypatch.delenv("LTHN_CUDA_BATCH_F32", raising=False)
        lthn.lib().lthn_debug_qmv_force_kernel(4)
        try:
            yield False
        finally:
            lthn.lib().lthn_debug_qmv_force_kernel(0)


@pytest.mark.parametrize("N,K", [(2304, 2304), (9216, 2304), (2304, 9216)])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_decode_sweep_shapes_bf16(oracle, N, K, M, batch_f32):
    """The decode sweep shapes, bf16 activations ~ N(0,1), weights ~ N(0,0.02)."""
    import lthn
    if M <= 2 and batch_f32:
        pytest.skip("one kernel serves 1-2 rows")
    p, s, b = make_weight(oracle, N, K, seed=N + K)
    xf, xb = make_x(oracle, M, K, seed=M)
    q = lthn.QuantWeight.from_host(p, s, b)
    got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
    got16 = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.BF16)
    if M <= 2:
        want = oracle.matnt_quant_host(xf, p, s, b, threads=8)
        assert rel_err(got, want) <= REF_TOL
        assert rms_err(got, want) <= F32_TOL_RMS
        assert bf16_close(oracle, got16, want)
    else:
        check_batched(oracle, got, xf, p, s, b, batch_f32)
        assert bf16_close(oracle, got16, got)   # the bf16 output is the f32 result rounded once


@pytest.mark.parametrize("M", [1, 2, 3, 7, 16, 32])
def test_f32_activations_keep_f32_precision(oracle, M, monkeypatch):
    """On the f32-grade kernels (1-2 rows always; 3..32 rows with LTHN_CUDA_BATCH_F32=1) f32
    activations go through exact bf16 split columns; the result must match the f64 oracle on
    the unrounded f32 activations."""
    import lthn
    monkeypatch.setenv("LTHN_CUDA_BATCH_F32", "1")
    N, K = 1024, 2304
    p, s, b = make_weight(oracle, N, K, seed=5)
    x = np.random.default_rng(M).standard_normal((M, K)).astype(np.float32)
    want = oracle.matnt_quant_host(x, p, s, b, threads=8)
    q = lthn.QuantWeight.from_host(p, s, b)
    got = run_qmv(lthn, x, lthn.F32, M, q, lthn.F32)
    tol = F32_TOL_RMS if M <= 2 else 4e-5  # 3-term split up to M=2, 2-term (16 bits) above
    assert rms_err(got, want) <= tol


@pytest.mark.parametrize("N,K", [(1, 64), (7, 64), (17, 128), (1000, 2304), (33, 4096), (4095, 512)])
def test_ragged_and_tiny_shapes(oracle, N, K, batch_f32):
    import lthn
    p, s, b = make_weight(oracle, N, K, seed=N * 7 + K)
    for M in (1, 5, 32):
        xf, xb = make_x(oracle, M, K, seed=3)
        got = run_qmv(lthn, xb, lthn.BF16, M, lthn.QuantWeight.from_host(p, s, b), lthn.F32)
        if M <= 2:
            assert rms_err(got, oracle.matnt_quant_host(xf, p, s, b)) <= F32_TOL_RMS
        else:
            check_batched(oracle, got, xf, p, s, b, batch_f32)


def test_every_kernel_configuration_agrees(oracle):
    """Both kernels and all their launch configurations compute the same function."""
    import lthn
    N, K = 2304, 2304
    p, s, b = make_weight(oracle, N, K, seed=1)
    q = lthn.QuantWeight.from_host(p, s, b)
    L = lthn.lib()
    try:
        for M in (1, 2, 8, 16):
            xf, xb = make_x(oracle, M, K, seed=9)
            want = oracle.matnt_quant_host(xf, p, s, b, threads=8)
            L.lthn_debug_qmv_force_kernel(2)  # tensor-core kernel: tiles per CTA x warps
            for rt in (1, 2, 4):
                for nw in (1, 2, 4, 8):
                    L.lthn_debug_qmv_force_config(rt, nw)
                    got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
                    assert rms_err(got, want) <= F32_TOL_RMS, ("mma", M, rt, nw)
            if M <= 2:
                L.lthn_debug_qmv_force_kernel(1)  # dp4a kernel: rows per thread
                for r in (1, 2, 4):
                    L.lthn_debug_qmv_force_config(r, 0)
                    got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
                    assert rms_err(got, want) <= F32_TOL_RMS, ("dp4a", M, r)
    finally:
        L.lthn_debug_qmv_force_config(0, 0)
        L.lthn_debug_qmv_force_kernel(0)


@pytest.mark.parametrize("K,N", [(2304, 512), (9216, 300), (5376, 256), (21504, 64), (4096, 128), (2048, 1000),
                                 (128, 40), (64, 5), (1536, 77)])
@pytest.mark.parametrize("M", [1, 2])
def test_dp4a_kernel_shapes(oracle, K, N, M):
    """The batch-1/2 kernel over every K of the two benchmark decoders (2304, 9216, 5376, 21504,
    4096, 2048) and awkward small ones, f32 and bf16 activations."""
    import lthn
    p, s, b = make_weight(oracle, N, K, seed=K + N)
    q = lthn.QuantWeight.from_host(p, s, b)
    xf, xb = make_x(oracle, M, K, seed=M + K)
    want = oracle.matnt_quant_host(xf, p, s, b, threads=8)
    lthn.lib().lthn_debug_qmv_force_kernel(1)
    try:
        got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
        assert rms_err(got, want) <= F32_TOL_RMS
        x32 = np.random.default_rng(K).standard_normal((M, K)).astype(np.float32)
        x32[0, :64] *= 1e-4   # a group of tiny activations next to ordinary ones
        if K >= 128:
            x32[0, 64:128] = 0.0  # an all-zero group
        want32 = oracle.matnt_quant_host(x32, p, s, b, threads=8)
        got32 = run_qmv(lthn, x32, lthn.F32, M, q, lthn.F32)
        assert rms_err(got32, want32) <= F32_TOL_RMS
    finally:
        lthn.lib().lthn_debug_qmv_force_kernel(0)


@pytest.mark.parametrize("K,N", [(2304, 512), (2304, 4112), (9216, 304), (5376, 256), (4096, 128), (2048, 1008),
                                 (8192, 64), (3072, 96), (128, 48), (64, 16), (1536, 80), (576, 9488),
                                 (21504, 64), (21504, 5376), (10752, 2304), (9216, 2304), (14336, 4096), (4096, 5008)])
@pytest.mark.parametrize("M", [1, 2])
def test_i8_tensor_core_kernel_shapes(oracle, K, N, M):
    """The integer tensor-core batch-1/2 kernel (forced) over the K of the two benchmark decoders and
    awkward small ones, f32 and bf16 activations, both tile heights, ragged last row block."""
    import lthn
    p, s, b = make_weight(oracle, N, K, seed=K + N)
    q = lthn.QuantWeight.from_host(p, s, b)
    xf, xb = make_x(oracle, M, K, seed=M + K)
    want = oracle.matnt_quant_host(xf, p, s, b, threads=8)
    L = lthn.lib()
    L.lthn_debug_qmv_force_kernel(3)
    try:
        for rt in (0, 1, 2):
            L.lthn_debug_qmv_force_config(rt, 0)
            got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
            assert rms_err(got, want) <= F32_TOL_RMS, rt
        L.lthn_debug_qmv_force_config(0, 0)
        x32 = np.random.default_rng(K).standard_normal((M, K)).astype(np.float32)
        x32[0, :64] *= 1e-4   # a group of tiny activations next to ordinary ones
        if K >= 128:
            x32[0, 64:128] = 0.0  # an all-zero group
        want32 = oracle.matnt_quant_host(x32, p, s, b, threads=8)
        got32 = run_qmv(lthn, x32, lthn.F32, M, q, lthn.F32)
        assert rms_err(got32, want32) <= F32_TOL_RMS
        gotb = run_qmv(lthn, x32, lthn.F32, M, q, lthn.BF16)
        assert bf16_close(oracle, gotb, want32)
    finally:
        L.lthn_debug_qmv_force_config(0, 0)
        L.lthn_debug_qmv_force_kernel(0)


@pytest.mark.parametrize("M", [3, 4, 5, 6, 7, 8, 9, 11, 16, 18, 32])
@pytest.mark.parametrize("K,N", [(2304, 528), (2048, 1008), (9216, 304), (5376, 256), (4096, 128), (3072, 96), (128, 48),
                                 (64, 16)])
def test_batched_rows_default_dispatch(oracle, K, N, M, batch_f32):
    """3..32 rows (one weight pass for all rows) on both kernels that serve them, f32 and bf16
    activations, f32 and bf16 outputs, tiny and all-zero activation groups."""
    import lthn
    p, s, b = make_weight(oracle, N, K, seed=K + N)
    q = lthn.QuantWeight.from_host(p, s, b)
    xf, xb = make_x(oracle, M, K, seed=M + K)
    got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)
    check_batched(oracle, got, xf, p, s, b, batch_f32)
    x32 = np.random.default_rng(K + M).standard_normal((M, K)).astype(np.float32)
    x32[M // 2, :64] *= 1e-4   # a group of tiny activations next to ordinary ones
    if K >= 128:
        x32[0, 64:128] = 0.0   # an all-zero group
    got32 = run_qmv(lthn, x32, lthn.F32, M, q, lthn.F32)
    gotb = run_qmv(lthn, x32, lthn.F32, M, q, lthn.BF16)
    if batch_f32:
        want32 = oracle.matnt_quant_host(x32, p, s, b, threads=8)
        assert rms_err(got32, want32) <= F32_TOL_RMS
        assert bf16_close(oracle, gotb, want32)
    else:
        # f32 activations are rounded to bf16 on the way in: that rounded copy is what the contract multiplies
        x16 = oracle.bf16_to_f32(oracle.f32_to_bf16(x32))
        check_batched(oracle, got32, x16, p, s, b, False)
        assert bf16_close(oracle, gotb, got32)


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("N,K,geglu", [(4096, 2304, False), (9216, 2304, True), (65536, 2304, False), (1024, 5376, False),
                                       (512, 4096, True), (304, 9216, False), (64, 128, False)])
def test_qmv_with_fused_norm_prologue(oracle, M, N, K, geglu):
    """lthn_affine_qmv_normed against the separate steps: lthn_rmsnorm_residual (bit-exact against
    the oracle elsewhere) then the oracle matvec on its output; the stored residual stream must be
    the norm kernel's (f64 sums in another order may move a value by one ulp at most, rarely)."""
    import lthn
    L = lthn.lib()
    rng = np.random.default_rng(N + K + M)
    a = rng.standard_normal((M, K)).astype(np.float32)
    h = (rng.standard_normal((M, K)) * 5).astype(np.float32)
    w1 = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    w2 = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    p, s, b = make_weight(oracle, N, K, seed=N)
    q = lthn.QuantWeight.from_host(p, s, b)
    up = q2 = None
    if geglu:
        up = make_weight(oracle, N, K, seed=N + 1)
        q2 = lthn.QuantWeight.from_host(*up)
    ab, hb, h2b, w1b, w2b = (lthn.Buf.from_array(v) for v in (a, h, np.zeros_like(h), w1, w2))
    y = lthn.Buf(M * N * 4)
    for with_a in (True, False):
        h_want = np.stack([h[r] + oracle.rmsnorm(a[r], w1, 1e-6) for r in range(M)]).astype(np.float32) if with_a else h
        x_want = np.stack([oracle.rmsnorm(h_want[r], w2, 1e-6) for r in range(M)])
        want = oracle.matnt_quant_host(x_want, p, s, b, threads=8)
        if geglu:
            want = oracle.gelu_tanh(want) * oracle.matnt_quant_host(x_want, *up, threads=8)
        lthn.check(L.lthn_affine_qmv_normed(None, ab.ptr if with_a else None, hb.ptr, h2b.ptr if with_a else None,
                                            w1b.ptr if with_a else None, w2b.ptr, 1e-6, M, q.packed.ptr, q.scales.ptr, q.biases.ptr,
                                            q2.packed.ptr if geglu else None, q2.scales.ptr if geglu else None,
                                            q2.biases.ptr if geglu else None, N, K, y.ptr, lthn.F32))
        lthn.sync()
        got = y.download(np.float32, (M, N))
        assert rms_err(got, want) <= (1e-4 if geglu else F32_TOL_RMS), with_a
        if with_a:
            h_got = h2b.download(np.float32, (M, K))
            assert np.mean(h_got.view(np.uint32) == h_want.view(np.uint32)) >= 0.999
            assert np.max(np.abs(h_got - h_want)) <= 1e-6 * np.max(np.abs(h_want))


@pytest.mark.parametrize("M", [1, 2, 5, 8, 16, 19])
@pytest.mark.parametrize("N,K", [(9216, 2304), (1000, 2304), (21504 // 8, 5376)])
def test_fused_geglu(oracle, M, N, K, batch_f32):
    """gate/up pair with the GeGLU epilogue against gelu_tanh(gate)*up from the oracle
    (hip_gemma4_q4_layer.go:3582-3597 GELU, oracle_test.go:939-948 multiply); for 3..32 rows on
    the tcgen05 kernel the oracle multiplies the bf16-contract projections."""
    import lthn
    if M <= 2 and batch_f32:
        pytest.skip("one kernel serves 1-2 rows")
    gp = make_weight(oracle, N, K, seed=1)
    up = make_weight(oracle, N, K, seed=2)
    x = np.random.default_rng(3).standard_normal((M, K)).astype(np.float32)
    if M > 2 and not batch_f32:
        x = oracle.bf16_to_f32(oracle.f32_to_bf16(x))
        g = oracle.proj_bf16_contract(x, *gp)
        u = oracle.proj_bf16_contract(x, *up)
    else:
        g = oracle.matnt_quant_host(x, *gp, threads=8)
        u = oracle.matnt_quant_host(x, *up, threads=8)
    want = oracle.gelu_tanh(g) * u
    gq, uq = lthn.QuantWeight.from_host(*gp), lthn.QuantWeight.from_host(*up)
    y = lthn.Buf(M * N * 4)
    xd = lthn.Buf.from_array(x)
    lthn.qmv_geglu(xd, lthn.F32, M, gq, uq, y, lthn.F32)
    lthn.sync()
    got = y.download(np.float32, (M, N))
    # the product of two projections: twice the f32 accumulation noise, and tanhf against the
    # reference's tanh formula
    assert rms_err(got, want) <= 3e-4


def test_negative_scales_and_literal_variant(oracle):
    """The reference quantiser signs the scale (mlxaffine.go:150-154); the literal
    min/max rule never does. The kernel must serve both."""
    import lthn
    N, K = 512, 1024
    for variant in (0, 1):
        p, s, b = make_weight(oracle, N, K, seed=2, variant=variant)
        if variant == 0:
            assert (oracle.bf16_to_f32(s) < 0).any()
        xf, xb = make_x(oracle, 1, K, seed=4)
        want = oracle.matnt_quant_host(xf, p, s, b)
        got = run_qmv(lthn, xb, lthn.BF16, 1, lthn.QuantWeight.from_host(p, s, b), lthn.F32)
        assert rms_err(got, want) <= F32_TOL_RMS


def test_lm_head_full_size(oracle):
    """Full-size lm_head shape (262144 x 2304), weights generated on the device:
    compared row-for-row with the oracle, plus linearity as a size-independent check."""
    import lthn
    N, K = 262144, 2304
    q = lthn.QuantWeight.synth(3, 0.02, N, K)
    p, s, b = q.to_host()
    xf, xb = make_x(oracle, 2, K, seed=8)
    want = oracle.matnt_quant_host(xf, p, s, b, threads=oracle.lib().lthn_o_num_threads())
    got = run_qmv(lthn, xb, lthn.BF16, 2, q, lthn.F32)
    assert rel_err(got, want) <= REF_TOL
    assert rms_err(got, want) <= F32_TOL_RMS
    # linearity: W(x0 + x1) = W x0 + W x1 (f32 activations so the sum is representable)
    xs = (xf[0] + xf[1])[None, :].astype(np.float32)
    got_sum = run_qmv(lthn, xs, lthn.F32, 1, q, lthn.F32)
    assert rms_err(got_sum[0], got[0].astype(np.float64) + got[1]) <= 5e-5
    # the batched row counts of the decode sweep on the same matrix, against the oracle on a sample
    # of weight rows (both ends, every tile phase, a random spread)
    rows = np.unique(np.concatenate([np.arange(0, 96), np.arange(N - 96, N),
                                     np.random.default_rng(1).integers(0, N, 4096)]))
    # default dispatch: up to 16 rows stay on the f32-grade kernel, 17..32 rows of a matrix this
    # size run on the tcgen05 streaming kernel (bf16 contract)
    for M in (4, 8, 16, 24, 32):
        xf, xb = make_x(oracle, M, K, seed=40 + M)
        got = run_qmv(lthn, xb, lthn.BF16, M, q, lthn.F32)[:, rows]
        check_batched(oracle, got, xf, p[rows], s[rows], b[rows], f32_grade=M <= 16)


def test_zero_sized_and_rejected_arguments(oracle):
    import lthn
    q = lthn.QuantWeight.from_host(*make_weight(oracle, 16, 64, seed=0))
    x = lthn.Buf(64 * 2)
    y = lthn.Buf(16 * 4)
    lthn.qmv(x, lthn.BF16, 0, q, y, lthn.F32)  # M == 0: no-op
    with pytest.raises(lthn.LthnError):
        lthn.qmv(x, lthn.BF16, 33, q, y, lthn.F32)
    with pytest.raises(lthn.LthnError):
        lthn.check(lthn.lib().lthn_affine_qmv(None, x.ptr, lthn.BF16, 1, q.packed.ptr, q.scales.ptr, q.biases.ptr,
                                              16, 64, 48, 4, y.ptr, lthn.F32))
    with pytest.raises(lthn.LthnError):
        lthn.check(lthn.lib().lthn_affine_qmv(None, x.ptr, lthn.BF16, 1, q.packed.ptr, q.scales.ptr, q.biases.ptr,
                                              16, 64, 64, 3, y.ptr, lthn.F32))


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("N,K", [(4096, 2304), (9216, 2304), (2304, 9216), (5376, 21504), (1008, 128), (16, 64)])
def test_eight_bit_codes_on_the_integer_kernel(oracle, N, K, M):
    """8-bit group-64 weights (the per-module override QAT packs give their MLP projections) through
    affine_qmv with one or two rows: the integer tensor-core kernel takes the code bytes as MMA operands
    without an unpack step - whole rows for K = 2304, K slices with partial sums for K = 9216 and 21504.
    f32-grade against the f64 reference (the activations go through the same three digit planes), and
    the same numbers as the general kernel that serves the other row counts."""
    import lthn
    p, s, b = make_weight(oracle, N, K, seed=N + K, bits=8)
    q = lthn.QuantWeight.from_host(p, s, b, 8, 64)
    xf, xb = make_x(oracle, M, K, seed=3 + M)
    want = oracle.matnt_quant_host(xf, p, s, b, 64, 8, threads=8)
    for x_arr, dt in ((xb, lthn.BF16), (xf, lthn.F32)):
        got = run_qmv(lthn, x_arr, dt, M, q, lthn.F32)
        assert rel_err(got, want) <= REF_TOL
        assert rms_err(got, want) <= F32_TOL_RMS
    got_b = oracle.bf16_to_f32(run_qmv(lthn, xb, lthn.BF16, M, q, lthn.BF16))
    assert rel_err(got_b, want) <= 1e-2
    # three rows take the general kernel: rows 0 and 1 of that result are the same matvecs
    if M == 2:
        x3 = np.concatenate([xf, xf[:1]], axis=0)
        got3 = run_qmv(lthn, x3, lthn.F32, 3, q, lthn.F32)
        assert rms_err(got3[:2], want) <= F32_TOL_RMS
    assert lthn.device_status() == 0
    q.free()


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("N,K,geglu", [(9216, 2304, True), (2688, 5376, True), (512, 1024, True), (4096, 2304, False), (64, 128, True)])
def test_eight_bit_codes_with_geglu_and_fused_norm(oracle, M, N, K, geglu):
    """8-bit group-64 gate/up pairs (the MLP projections of a mixed-precision pack) with the GeGLU epilogue
    (two full row sets per block for K < 2048, the interleaved 8 + 8 row block from there), alone and behind
    the fused residual-norm prologue, against the same steps from the oracle at the bounds of the 4-bit forms."""
    import lthn
    L = lthn.lib()
    rng = np.random.default_rng(N + K + M)
    p, s, b = make_weight(oracle, N, K, seed=N, bits=8)
    q = lthn.QuantWeight.from_host(p, s, b, 8, 64)
    up = q2 = None
    if geglu:
        up = make_weight(oracle, N, K, seed=N + 1, bits=8)
        q2 = lthn.QuantWeight.from_host(*up, 8, 64)
    y = lthn.Buf(M * N * 4)
    if geglu:
        x = rng.standard_normal((M, K)).astype(np.float32)
        want = oracle.gelu_tanh(oracle.matnt_quant_host(x, p, s, b, 64, 8, threads=8)) * oracle.matnt_quant_host(x, *up, 64, 8, threads=8)
        xb = lthn.Buf.from_array(x)
        lthn.qmv_geglu(xb, lthn.F32, M, q, q2, y, lthn.F32)
        lthn.sync()
        assert rms_err(y.download(np.float32, (M, N)), want) <= 1e-4
    a = rng.standard_normal((M, K)).astype(np.float32)
    h = (rng.standard_normal((M, K)) * 5).astype(np.float32)
    w1 = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    w2 = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    ab, hb, h2b, w1b, w2b = (lthn.Buf.from_array(v) for v in (a, h, np.zeros_like(h), w1, w2))
    for with_a in (True, False):
        h_want = np.stack([h[r] + oracle.rmsnorm(a[r], w1, 1e-6) for r in range(M)]).astype(np.float32) if with_a else h
        x_want = np.stack([oracle.rmsnorm(h_want[r], w2, 1e-6) for r in range(M)])
        want = oracle.matnt_quant_host(x_want, p, s, b, 64, 8, threads=8)
        if geglu:
            want = oracle.gelu_tanh(want) * oracle.matnt_quant_host(x_want, *up, 64, 8, threads=8)
        lthn.check(L.lthn_affine_qmv_normed_bits(None, ab.ptr if with_a else None, hb.ptr, h2b.ptr if with_a else None,
                                                 w1b.ptr if with_a else None, w2b.ptr, 1e-6, M, q.packed.ptr, q.scales.ptr, q.biases.ptr,
                                                 q2.packed.ptr if geglu else None, q2.scales.ptr if geglu else None,
                                                 q2.biases.ptr if geglu else None, N, K, 8, y.ptr, lthn.F32))
        lthn.sync()
        got = y.download(np.float32, (M, N))
        assert rms_err(got, want) <= (1e-4 if geglu else F32_TOL_RMS), with_a
        if with_a:
            h_got = h2b.download(np.float32, (M, K))
            assert np.mean(h_got.view(np.uint32) == h_want.view(np.uint32)) >= 0.999
    assert lthn.device_status() == 0
    q.free()
    if q2:
        q2.free()
