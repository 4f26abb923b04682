"""Pins the CPU oracle to the reference's own known-answer tests and fixtures.

Each test names the reference test it re-creates (paths relative to the
reference's go/ directory). None of these needs a GPU."""
import math
from fractions import Fraction

import numpy as np
import pytest


def bf(o, v):
    return int(o.lib().lthn_o_f32_to_bf16(float(v)))


# --- enginetest/quant_reference_test.go:13-38 TestReferenceAffineMatVec_Good ---
def test_ref_matvec_hand_checkable(oracle):
    o = oracle
    packed = np.zeros(1, dtype=np.uint8)
    o.lib().lthn_o_affine_set_code(packed.ctypes.data, 0, 4, 3)
    o.lib().lthn_o_affine_set_code(packed.ctypes.data, 4, 4, 5)
    assert packed[0] == 0x53
    scales = np.array([bf(o, 2.0)], dtype=np.uint16)
    biases = np.array([bf(o, 1.0)], dtype=np.uint16)
    x = np.array([bf(o, 1.0), bf(o, 0.5)], dtype=np.uint16)
    got = o.ref_affine_matvec(x, packed, scales, biases, 1, 2, 2, 4)
    assert got[0] == bf(o, 12.5)


def parity_fixture(o):
    """enginetest/quant_parity.go:33-67 quantAffineFixture."""
    out_dim, in_dim, gs, bits = 8, 128, 64, 4
    gpr, row_packed = in_dim // gs, in_dim * bits // 8
    packed = np.zeros((out_dim, row_packed), dtype=np.uint8)
    scales = np.zeros((out_dim, gpr), dtype=np.uint16)
    biases = np.zeros((out_dim, gpr), dtype=np.uint16)
    for r in range(out_dim):
        for g in range(gpr):
            scales[r, g] = bf(o, np.float32(0.25) + np.float32(0.125) * np.float32(g + r))
            biases[r, g] = bf(o, np.float32(-1) + np.float32(0.5) * np.float32((g + r) % 3))
            for j in range(gs):
                c = g * gs + j
                o.lib().lthn_o_affine_set_code(packed[r].ctypes.data, c * bits, bits, (c * 5 + r * 3 + 1) % 16)
    x = np.array([bf(o, np.float32(0.1) * np.float32((i % 7) - 3)) for i in range(in_dim)], dtype=np.uint16)
    return x, packed, scales, biases, out_dim, in_dim, gs, bits


# --- enginetest/quant_reference_test.go:76-95 fixture <-> unpacker agreement ---
def test_parity_fixture_round_trips(oracle):
    o = oracle
    _, packed, _, _, out_dim, in_dim, _, bits = parity_fixture(o)
    for r in range(out_dim):
        for c in range(in_dim):
            assert o.lib().lthn_o_affine_extract_code(packed[r].ctypes.data, c * bits, bits) == (c * 5 + r * 3 + 1) % 16


def test_parity_fixture_exact_value(oracle):
    """The f64 reference on the parity fixture equals exact rational arithmetic
    rounded once to bf16 (all operands are short dyadic rationals)."""
    o = oracle
    x, packed, scales, biases, out_dim, in_dim, gs, bits = parity_fixture(o)
    got = o.ref_affine_matvec(x, packed, scales, biases, out_dim, in_dim, gs, bits)
    xs = [Fraction(float(v)) for v in o.bf16_to_f32(x)]
    for r in range(out_dim):
        acc = Fraction(0)
        for c in range(in_dim):
            s = Fraction(float(o.bf16_to_f32(scales[r, c // gs:c // gs + 1])[0]))
            b = Fraction(float(o.bf16_to_f32(biases[r, c // gs:c // gs + 1])[0]))
            acc += (s * ((c * 5 + r * 3 + 1) % 16) + b) * xs[c]
        assert got[r] == bf(o, np.float32(float(acc)))
    # the other two CPU references agree to the reference's own tolerance (0.05)
    words = packed.view(np.uint32)
    hip = o.hip_affine_projection(o.bf16_to_f32(x), words, scales, biases, out_dim, in_dim, gs, bits)
    mnt = o.matnt_quant_host(o.bf16_to_f32(x), words, scales, biases, gs, bits)[0]
    ref = o.bf16_to_f32(got)
    assert np.max(np.abs(hip - ref)) <= 0.05 and np.max(np.abs(mnt - ref)) <= 0.05


# --- quant_reference_test.go:43-74 validation surface and zero-size case ---
def test_ref_matvec_bad_and_ugly(oracle):
    o = oracle
    x, packed, scales, biases, out_dim, in_dim, gs, bits = parity_fixture(o)
    with pytest.raises(o.OracleError):
        o.ref_affine_matvec(x.view(np.uint8)[:-1], packed, scales, biases, out_dim, in_dim, gs, bits)
    with pytest.raises(o.OracleError):
        o.ref_affine_matvec(x, packed.reshape(-1)[:-1], scales, biases, out_dim, in_dim, gs, bits)
    with pytest.raises(o.OracleError):
        o.ref_affine_matvec(x, packed, scales, biases, out_dim, in_dim, 3, bits)
    with pytest.raises(o.OracleError):
        o.ref_affine_matvec(x, packed, scales, biases, out_dim, in_dim, gs, 0)
    with pytest.raises(o.OracleError):
        o.ref_affine_matvec(x, packed, scales, biases, out_dim, in_dim, gs, 9)
    empty = np.zeros(0, dtype=np.uint8)
    assert o.ref_affine_matvec(empty, empty, empty, empty, 0, 0, 64, 4).size == 0


# --- quant_reference_test.go:100-111 TestBF16RoundTrip_Good ---
def test_bf16_round_trip(oracle):
    o = oracle
    for v in (0, 1, -1, 12.5, 0.25, -3.75, 100, -0.03125):
        assert o.lib().lthn_o_bf16_to_f32(bf(o, v)) == v
    a = np.random.default_rng(1).standard_normal(4096).astype(np.float32)
    scalar = np.array([bf(o, v) for v in a], dtype=np.uint16)
    assert np.array_equal(o.f32_to_bf16(a), scalar)
    # ties go to even: 1 + 2^-8 is exactly between two bf16 values
    assert bf(o, 1.00390625) == 0x3F80 and bf(o, 1.01171875) == 0x3F82


# --- engine/hip/hip_projection_reference_test.go:71-85 ---
def test_hip_projection_q4_kat(oracle):
    o = oracle
    got = o.hip_affine_projection(np.ones(8), [0x76543210, 0xFEDCBA98], [0x3F80, 0x3F00], [0x0000, 0xBF80], 2, 8, 8, 4)
    assert got.tolist() == [28.0, 38.0]


def pack_values(values, cols, bits):
    """hip_projection_reference_test.go:112-135 hipPackMLXAffineValuesForTest."""
    ppr = cols * bits // 32
    rows = (len(values) + cols - 1) // cols
    out = np.zeros(rows * ppr, dtype=np.uint64)
    for index, value in enumerate(values):
        row, col = divmod(index, cols)
        bit = col * bits
        wi, shift = row * ppr + bit // 32, bit % 32
        value &= (1 << bits) - 1
        out[wi] |= (value << shift) & 0xFFFFFFFF
        if shift + bits > 32:
            out[wi + 1] |= value >> (32 - shift)
    return out.astype(np.uint32)


# --- hip_projection_reference_test.go:87-110 (6-bit crosses words; 8-bit) ---
def test_hip_projection_q6_q8_kat(oracle):
    o = oracle
    q6 = pack_values(list(range(16)) + list(range(16, 0, -1)), 16, 6)
    got = o.hip_affine_projection(np.ones(16), q6, [0x3F80, 0x3F80], [0, 0], 2, 16, 16, 6)
    assert got.tolist() == [120.0, 136.0]
    q8 = pack_values([1, 2, 3, 4, 5, 6, 7, 8], 4, 8)
    got = o.hip_affine_projection(np.ones(4), q8, [0x3F80, 0x3F80], [0, 0], 2, 4, 4, 8)
    assert got.tolist() == [10.0, 26.0]


def test_hip_projection_rejects_bad_shapes(oracle):
    o = oracle
    with pytest.raises(o.OracleError):
        o.hip_affine_projection(np.ones(7), [0x76543210, 0xFEDCBA98], [0x3F80, 0x3F00], [0, 0], 2, 8, 8, 4)
    with pytest.raises(o.OracleError):
        o.hip_affine_projection(np.ones(8), [0x76543210, 0xFEDCBA98], [0x3F80, 0x3F00], [0, 0], 2, 8, 8, 5)
    with pytest.raises(o.OracleError):
        o.hip_affine_projection(np.ones(8), [0x76543210, 0xFEDCBA98], [0x3F80, 0x3F00], [0, 0], 2, 8, 3, 4)


# --- hip_transformer_reference_test.go:31-42 q4 embedding rows ---
def test_affine_embedding_kat(oracle):
    o = oracle
    w = np.array([0x76543210, 0x11111111, 0xFEDCBA98], dtype=np.uint32)
    s = np.array([0x3F80, 0x3F80, 0x3F00], dtype=np.uint16)
    b = np.array([0, 0, 0xBF80], dtype=np.uint16)
    out = np.empty(8, dtype=np.float32)
    assert o.lib().lthn_o_affine_embedding_row(w.ctypes.data, s.ctypes.data, b.ctypes.data, 3, 8, 8, 4, 2, out.ctypes.data) == 0
    assert out.tolist() == [3, 3.5, 4, 4.5, 5, 5.5, 6, 6.5]
    assert o.lib().lthn_o_affine_embedding_row(w.ctypes.data, s.ctypes.data, b.ctypes.data, 3, 8, 8, 4, 0, out.ctypes.data) == 0
    assert out.tolist() == [0, 1, 2, 3, 4, 5, 6, 7]
    assert o.lib().lthn_o_affine_embedding_row(w.ctypes.data, s.ctypes.data, b.ctypes.data, 3, 8, 8, 4, 3, out.ctypes.data) != 0


def synth_weight(out_dim, in_dim):
    """model/quant/mlxaffine/mlxaffine_test.go:13-26 synthWeight."""
    w = np.zeros((out_dim, in_dim), dtype=np.float32)
    for r in range(out_dim):
        amp = np.float32(0.01) + np.float32(0.5) * np.float32(r + 1) / np.float32(out_dim)
        bias = np.float32(0.1) * np.float32(r % 3 - 1)
        for c in range(in_dim):
            w[r, c] = bias + amp * np.float32(math.sin(float(r * 7 + c) * 0.013))
    return w


# --- mlxaffine_test.go:32-82 round trip within the group bound ---
@pytest.mark.parametrize("bits,gs,out_dim,in_dim", [(4, 64, 8, 3840), (4, 32, 4, 256), (8, 64, 6, 512),
                                                    (8, 32, 3, 128), (2, 64, 5, 640), (4, 64, 3, 64)])
def test_quantize_round_trip_bound(oracle, bits, gs, out_dim, in_dim):
    o = oracle
    w = synth_weight(out_dim, in_dim)
    p, s, b = o.quantize(w, bits, gs)
    got = o.dequantize(p, s, b, bits, gs)
    assert np.isfinite(got).all()
    g = w.reshape(out_dim, in_dim // gs, gs)
    step = (g.max(axis=2) - g.min(axis=2)) / np.float32((1 << bits) - 1)
    bound = 1.5 * step + 0.02 * np.abs(g).max(axis=2) + 1e-6
    err = np.abs(got - w).reshape(out_dim, in_dim // gs, gs)
    assert (err <= bound[..., None]).all()
    # the independently written NumPy codec agrees byte for byte
    p2, s2, b2 = o.np_quantize(w, bits, gs)
    assert np.array_equal(p, p2) and np.array_equal(s, s2) and np.array_equal(b, b2)
    assert np.array_equal(got.view(np.uint32), o.np_dequantize(p, s, b, bits, gs).view(np.uint32))


# --- mlxaffine_test.go:87-112 codes are a fixed point of re-quantisation ---
def test_quantize_codes_fixed_point(oracle):
    o = oracle
    w = synth_weight(6, 512)
    p1, s1, b1 = o.quantize(w, 4, 64)
    d1 = o.dequantize(p1, s1, b1, 4, 64)
    p2, s2, b2 = o.quantize(d1, 4, 64)
    assert np.array_equal(p1, p2)
    d2 = o.dequantize(p2, s2, b2, 4, 64)
    assert np.max(np.abs(d2 - d1)) <= 5e-3


# --- mlxaffine_test.go:117-139 constant group ---
def test_quantize_constant_group(oracle):
    o = oracle
    w = np.full((2, 64), 0.25, dtype=np.float32)
    got = o.dequantize(*o.quantize(w, 4, 64), 4, 64)
    assert np.isfinite(got).all() and np.max(np.abs(got - 0.25)) <= 0.01


# --- mlxaffine_test.go:144-181 shape contract and rejected widths ---
def test_quantize_shapes_and_rejects(oracle):
    o = oracle
    p, s, b = o.quantize(synth_weight(8, 3840), 4, 64)
    assert p.shape == (8, 480) and s.shape == (8, 60) and b.shape == (8, 60)
    for bits in (3, 5, 6):
        with pytest.raises(o.OracleError):
            o.quantize(np.zeros((2, 64), dtype=np.float32), bits, 64)
    with pytest.raises(o.OracleError):
        o.quantize(np.zeros((2, 100), dtype=np.float32), 4, 64)
    with pytest.raises(o.OracleError):
        o.quantize(np.zeros((2, 64), dtype=np.float32), 4, 4)  # gs % (32/bits) != 0


def test_quantize_edge_anchoring(oracle):
    """mlxaffine.go:136-161: the dominant edge dequantises exactly (up to bf16
    storage) and the scale is negative when the max edge dominates."""
    o = oracle
    w = np.linspace(-0.25, 1.0, 64, dtype=np.float32)[None, :]
    p, s, b = o.quantize(w)
    assert o.bf16_to_f32(s)[0, 0] < 0 and o.bf16_to_f32(b)[0, 0] == 1.0
    w2 = -w
    p2, s2, b2 = o.quantize(w2)
    assert o.bf16_to_f32(s2)[0, 0] > 0 and o.bf16_to_f32(b2)[0, 0] == -1.0
    lit = o.quantize(w, variant=1)
    assert o.bf16_to_f32(lit[1])[0, 0] > 0 and o.bf16_to_f32(lit[2])[0, 0] == -0.25


# --- engine/metal/quant_seam_backend_test.go:46-89 host formula fixtures ---
@pytest.mark.parametrize("M,K,N,bits,gs", [(1, 512, 40, 4, 64), (1, 256, 24, 2, 128), (3, 512, 64, 4, 64),
                                           (5, 256, 40, 2, 128), (2, 128, 8, 8, 64)])
def test_matnt_quant_host_seam_fixture(oracle, M, K, N, bits, gs):
    o = oracle
    w = (((np.arange(N * K) % 17) - 8) * np.float32(0.037)).astype(np.float32).reshape(N, K)
    x = (((np.arange(M * K) % 9) - 4) * np.float32(0.05)).astype(np.float32).reshape(M, K)
    p, s, b = o.quantize(w, bits, gs)
    want = o.matnt(x, o.dequantize(p, s, b, bits, gs))
    got = o.matnt_quant_host(x, p, s, b, gs, bits)
    assert np.array_equal(got, want)  # same dequant, same f64 ascending-k sum
    got_mt = o.matnt_quant_host(x, p, s, b, gs, bits, threads=4)
    assert np.array_equal(got_mt, want)


# --- engine/hip/hip_transformer_reference_test.go:88-190 ---
def test_transformer_reference_kats(oracle):
    o = oracle
    np.testing.assert_allclose(o.rmsnorm([3, 4], [1, 0.5], 0.0), [0.8485, 0.5657], atol=1e-4)
    np.testing.assert_allclose(o.rope_interleaved([1, 0], 1, 1.0), [math.cos(1), math.sin(1)], atol=1e-4)
    np.testing.assert_allclose(o.rope_interleaved([1, 0, 1, 0], 1, 10000.0, 8),
                               [math.cos(1), math.sin(1), math.cos(0.1), math.sin(0.1)], atol=1e-4)
    np.testing.assert_allclose(o.rope_interleaved([1, 0], 1, 1.0, 2, 0.5), [math.cos(0.5), math.sin(0.5)], atol=1e-4)
    c, s = np.float32(math.cos(1)), np.float32(math.sin(1))
    np.testing.assert_allclose(o.rope_neox([1, 2, 3, 4], 1, 1.0, 4, 2), [1 * c - 3 * s, 2, 1 * s + 3 * c, 4], atol=1e-4)
    np.testing.assert_allclose(o.attention_single_head([1, 0], [[1, 0], [0, 1]], [[2, 0], [0, 4]]),
                               [1.3395, 1.3210], atol=1e-4)
    np.testing.assert_allclose(o.attention_single_head([0, 1], [[1, 0], [0, 1]], [[2, 0], [0, 4]]),
                               [0.6605, 2.6790], atol=1e-4)
    assert o.greedy_f32([-1, 0.25, 0.2]) == 1
    assert o.greedy_f32([1, 2, 2]) == 1  # ties -> lowest index
    assert o.greedy_bf16(o.f32_to_bf16(np.array([1, 2, 2], dtype=np.float32))) == 1
    for bad in ([], ):
        with pytest.raises(o.OracleError):
            o.rmsnorm(bad, bad, 0.0)
    with pytest.raises(o.OracleError):
        o.rope_neox([1, 2, 3], 0, 10000.0)
    with pytest.raises(o.OracleError):
        o.rope_neox([1, 2, 3, 4], -1, 10000.0)


def test_kv_head_map(oracle):
    """hip_gemma4_q4_oracle_test.go:1085-1101 rocmOracleKVHeadForQuery."""
    f = oracle.lib().lthn_o_kv_head_for_query
    assert [f(h, 8, 4) for h in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    assert [f(h, 4, 4) for h in range(4)] == [0, 1, 2, 3]
    assert [f(h, 4, 1) for h in range(4)] == [0, 0, 0, 0]


def test_gelu_and_norm_fold(oracle):
    o = oracle
    x = np.array([-3, -1, 0, 0.5, 2], dtype=np.float32)
    want = [0.5 * v * (1 + math.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3))) for v in x.astype(np.float64)]
    np.testing.assert_allclose(o.gelu_tanh(x), np.array(want, dtype=np.float32), rtol=0, atol=0)
    w = np.array([0.0, 0.5, -1.0], dtype=np.float32)
    out = np.empty_like(w)
    o.lib().lthn_o_fold_norm_bias_one_f32(w.ctypes.data, 3, out.ctypes.data)
    assert out.tolist() == [1.0, 1.5, 0.0]


def test_synth_normal_is_roughly_gaussian(oracle):
    v = oracle.synth_normal(7, 0, 1 << 18, 0.02)
    assert abs(float(v.mean())) < 2e-4 and abs(float(v.std()) - 0.02) < 2e-4
    assert v[5] == oracle.lib().lthn_o_synth_normal(7, 5, 0.02)
    assert np.array_equal(oracle.synth_normal(7, 100, 16, 0.02), v[100:116])


def test_decoder_sliding_window_reduces_to_known_cases(oracle):
    """The sliding/global pattern of the restated decoder against cases with a known answer: a window
    wider than the context with the local rope base equal to the global one is the plain decoder;
    pattern 1 makes every block global whatever the window; a window of 1 makes a sliding block's
    attention output the value row itself, which a tap on the attention stage shows."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from decoder_util import NORMS, ROLES, linear_shapes
    cfg = dict(layers=2, hidden=128, q_heads=2, kv_heads=1, head_dim=64, ffn=256, vocab=64)
    rng = np.random.default_rng(3)
    w = {(li, role): oracle.quantize((rng.standard_normal(shape) * 0.05).astype(np.float32))
         for li in range(cfg["layers"]) for role, shape in linear_shapes(cfg).items()}
    w["embed"] = oracle.quantize((rng.standard_normal((cfg["vocab"], cfg["hidden"])) * 0.05).astype(np.float32))
    ids = rng.integers(0, cfg["vocab"], 12).astype(np.int32)

    def run(sliding, tap=None):
        oc = oracle.DecoderConfig(layers=cfg["layers"], hidden=cfg["hidden"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                                  head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], gs=64, bits=4, max_len=32, eps=1e-6,
                                  rope_base=10000.0, attn_scale=0.125, embed_scale=1.0, kv_bf16=0, prefill_bf16=0)
        if sliding:
            oc.sliding_window, oc.sliding_pattern, oc.rope_local_base = sliding
        d = oracle.Decoder(oc)
        ones = {"h": np.ones(cfg["hidden"], dtype=np.float32), "d": np.ones(cfg["head_dim"], dtype=np.float32)}
        for li in range(cfg["layers"]):
            for role in ROLES:
                d.set_linear(li, role, *w[(li, role)])
            for role in NORMS:
                d.set_norm(li, role, ones["d"] if role in ("q_norm", "k_norm") else ones["h"])
        d.set_linear(-1, 0, *w["embed"])
        d.set_norm(-1, 0, ones["h"])
        buf = d.tap(tap, 1, len(ids), cfg["q_heads"] * cfg["head_dim"]) if tap is not None else None   # stage 1: attention output
        logits = d.forward(ids)
        return logits, buf, d

    plain, _, _ = run(None)
    wide, _, _ = run((1000, 2, 10000.0))
    assert (plain == wide).all()
    all_global, _, _ = run((3, 1, 3000.0))
    assert (plain == all_global).all()
    narrow, att, d = run((1, 2, 10000.0), tap=0)   # block 0 sliding with a window of one key
    assert not (narrow == plain).all()
    v = d.read_kv(0, 1)[:len(ids)]                  # [tokens, kv_heads*head_dim]
    for h in range(cfg["q_heads"]):
        assert np.allclose(att[:, h * 64:(h + 1) * 64], v[:, :64], rtol=0, atol=1e-6)


def test_decoder_per_linear_code_width(oracle):
    """A linear may carry its own code width (per-module overrides of a mixed-precision pack,
    model/quant_config.go:39-88). Known answer: the same 4-bit codes stored one per byte with the same scales
    and biases dequantise to the same weights, so the decoder whose MLP projections are declared 8-bit must give
    bit-identical logits and cache rows, with and without the bf16 prefill contract; real 8-bit codes of the same
    dense tensors move the logits by less than the 4-bit quantisation step does."""
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from decoder_util import NORMS, ROLES, linear_shapes
    cfg = dict(layers=2, hidden=128, q_heads=2, kv_heads=1, head_dim=64, ffn=256, vocab=64)
    rng = np.random.default_rng(5)
    dense = {(li, role): (rng.standard_normal(shape) * 0.05).astype(np.float32)
             for li in range(cfg["layers"]) for role, shape in linear_shapes(cfg).items()}
    w = {k: oracle.quantize(v) for k, v in dense.items()}
    embed = oracle.quantize((rng.standard_normal((cfg["vocab"], cfg["hidden"])) * 0.05).astype(np.float32))
    ids = rng.integers(0, cfg["vocab"], 12).astype(np.int32)

    def bytes_of_nibbles(packed):
        shifts = (np.arange(8, dtype=np.uint32) * 4).astype(np.uint32)
        codes = ((packed[..., None] >> shifts) & np.uint32(15)).reshape(packed.shape[0], -1).astype(np.uint8)
        return np.ascontiguousarray(codes).view(np.uint32)

    def run(weights, prefill_bf16):
        oc = oracle.DecoderConfig(layers=cfg["layers"], hidden=cfg["hidden"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                                  head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], gs=64, bits=4, max_len=32, eps=1e-6,
                                  rope_base=10000.0, attn_scale=0.125, embed_scale=1.0, kv_bf16=1, prefill_bf16=prefill_bf16)
        d = oracle.Decoder(oc)
        for li in range(cfg["layers"]):
            for role in ROLES:
                d.set_linear(li, role, *weights[(li, role)])
            for role in NORMS:
                d.set_norm(li, role, np.ones(cfg["head_dim"] if role in ("q_norm", "k_norm") else cfg["hidden"], dtype=np.float32))
        d.set_linear(-1, 0, *embed)
        d.set_norm(-1, 0, np.ones(cfg["hidden"], dtype=np.float32))
        logits = d.forward(ids)
        return logits, [d.read_kv(li, which)[:len(ids)].copy() for li in range(cfg["layers"]) for which in (0, 1)]

    same_codes = dict(w)
    real8 = dict(w)
    for li in range(cfg["layers"]):
        for role in ("gate", "up", "down"):
            p, s, b = w[(li, role)]
            same_codes[(li, role)] = (bytes_of_nibbles(p), s, b, 8)
            real8[(li, role)] = (*oracle.quantize(dense[(li, role)], bits=8), 8)
    for contract in (0, 1):
        base, kv0 = run(w, contract)
        got, kv1 = run(same_codes, contract)
        assert np.array_equal(base, got)
        assert all(np.array_equal(a, b) for a, b in zip(kv0, kv1))
        finer, _ = run(real8, contract)
        assert not np.array_equal(base, finer)
        assert float(np.max(np.abs(finer - base))) < 0.25 * float(np.max(np.abs(base)))
