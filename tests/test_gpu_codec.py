"""GPU codec parity: quantise / dequantise are bit-exact against the oracle
(mlxaffine.go:80-241) and the golden vectors of the reference's own tool."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K,bits,gs", [(8, 3840, 4, 64), (4, 256, 4, 32), (6, 512, 8, 64), (3, 128, 8, 32),
                                         (5, 640, 2, 64), (3, 64, 4, 64), (37, 2304, 4, 64), (16, 1024, 4, 128)])
@pytest.mark.parametrize("variant", [0, 1])
def test_quantize_bit_exact(oracle, N, K, bits, gs, variant):
    import lthn
    rng = np.random.default_rng(N * 131 + K + bits)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    w[0, :gs] = 0.25  # a constant group (scale floor path)
    w[-1, :gs] = np.linspace(-1, 0.25, gs)  # min-edge dominant
    want = oracle.quantize(w, bits, gs, variant)
    q = lthn.quantize(lthn.Buf.from_array(w), N, K, bits, gs, variant)
    got = q.to_host()
    for g, wnt, name in zip(got, want, ("packed", "scales", "biases")):
        assert np.array_equal(g, wnt), name


def test_dequantize_bit_exact_against_golden(oracle):
    import lthn
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "mlxaffine_dequant_golden.npz"))
    for n in sorted({k.rsplit(".", 1)[0] for k in z.files}):
        bits, gs = (int(v) for v in z[n + ".meta"])
        q = lthn.QuantWeight.from_host(z[n + ".packed"], z[n + ".scales"], z[n + ".biases"], bits, gs)
        out = lthn.Buf(q.N * q.K * 4)
        lthn.dequantize(q, out)
        got = out.download(np.float32, (q.N, q.K))
        assert np.array_equal(got.view(np.uint32), z[n + ".dequant"].view(np.uint32)), n
        out16 = lthn.Buf(q.N * q.K * 2)
        lthn.dequantize(q, out16, bf16=True)
        assert np.array_equal(out16.download(np.uint16, (q.N, q.K)), oracle.f32_to_bf16(z[n + ".dequant"])), n


def test_synth_weight_matches_oracle_generator(oracle):
    """The on-device synthetic tensor source equals the oracle's, bit for bit, and
    the fused generate+quantise equals quantising the generated tensor."""
    import lthn
    N, K = 48, 2304
    buf = lthn.Buf(N * K * 4)
    lthn.check(lthn.lib().lthn_synth_normal_fill(None, 11, 0, N * K, 0.02, buf.ptr))
    got = buf.download(np.float32, (N, K))
    want = oracle.synth_normal(11, 0, N * K, 0.02).reshape(N, K)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    q = lthn.QuantWeight.synth(11, 0.02, N, K)
    for g, wnt in zip(q.to_host(), oracle.quantize(want)):
        assert np.array_equal(g, wnt)


def test_quantize_full_size_round_trip_property(oracle):
    """The single-linear reference case (8192 x 2048): device quantise -> device dequantise stays
    inside the reference's group error bound (mlxaffine_test.go:63-64) and the codes
    of a sample of rows equal the oracle's."""
    import lthn
    N, K = 8192, 2048
    wbuf = lthn.Buf(N * K * 4)
    lthn.check(lthn.lib().lthn_synth_normal_fill(None, 0, 0, N * K, 0.02, wbuf.ptr))
    q = lthn.quantize(wbuf, N, K)
    out = lthn.Buf(N * K * 4)
    lthn.dequantize(q, out)
    w = wbuf.download(np.float32, (N, K))
    d = out.download(np.float32, (N, K))
    g = w.reshape(N, K // 64, 64)
    step = (g.max(axis=2) - g.min(axis=2)) / 15.0
    bound = 1.5 * step + 0.02 * np.abs(g).max(axis=2) + 1e-6
    assert (np.abs(d - w).reshape(N, K // 64, 64) <= bound[..., None]).all()
    rows = np.arange(0, N, 257)
    p, s, b = q.to_host()
    wp, ws, wb = oracle.quantize(w[rows])
    assert np.array_equal(p[rows], wp) and np.array_equal(s[rows], ws) and np.array_equal(b[rows], wb)
