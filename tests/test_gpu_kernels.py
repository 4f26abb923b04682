"""Parity of the fused decoder-step kernels (lthn_rmsnorm*, lthn_rmsnorm_rope,
lthn_sdpa_decode, lthn_argmax) against the CPU references they replace."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


_KEEP = []


def dev(lthn, a):
    """Uploads an array; the buffer is kept alive for the rest of the test session
    (a temporary would be freed before the asynchronous kernel reads it)."""
    b = lthn.Buf.from_array(np.ascontiguousarray(a))
    _KEEP.append(b)
    if len(_KEEP) > 64:
        lthn.sync()
        del _KEEP[:32]
    return b


@pytest.mark.parametrize("rows,width", [(1, 2304), (5, 5376), (32, 256), (3, 64)])
def test_rmsnorm_matches_reference(oracle, rows, width):
    """hipReferenceRMSNorm (hip_transformer_reference.go:171-194): f64 sum of squares,
    x / rms * w. The device kernel reproduces it bit for bit."""
    import lthn
    rng = np.random.default_rng(rows + width)
    x = rng.standard_normal((rows, width)).astype(np.float32) * 3
    w = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    out = lthn.Buf(rows * width * 4)
    lthn.check(lthn.lib().lthn_rmsnorm(None, dev(lthn, x).ptr, dev(lthn, w).ptr, out.ptr, rows, width, 1e-6))
    got = out.download(np.float32, (rows, width))
    want = np.stack([oracle.rmsnorm(x[r], w, 1e-6) for r in range(rows)])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_rmsnorm_residual_fusion(oracle):
    """h += norm(a, w_post); out = norm(h, w_next) (hip_gemma4_q4_oracle_test.go:925-951)."""
    import lthn
    rows, width = 7, 2304
    rng = np.random.default_rng(0)
    a = rng.standard_normal((rows, width)).astype(np.float32)
    h = rng.standard_normal((rows, width)).astype(np.float32) * 5
    w1 = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    w2 = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    hb, out = dev(lthn, h), lthn.Buf(rows * width * 4)
    lthn.check(lthn.lib().lthn_rmsnorm_residual(None, dev(lthn, a).ptr, hb.ptr, dev(lthn, w1).ptr, dev(lthn, w2).ptr,
                                                out.ptr, rows, width, 1e-6))
    h_want = np.stack([h[r] + oracle.rmsnorm(a[r], w1, 1e-6) * np.float32(1.0) for r in range(rows)]).astype(np.float32)
    out_want = np.stack([oracle.rmsnorm(h_want[r], w2, 1e-6) for r in range(rows)])
    assert np.array_equal(hb.download(np.float32, (rows, width)).view(np.uint32), h_want.view(np.uint32))
    assert np.array_equal(out.download(np.float32, (rows, width)).view(np.uint32), out_want.view(np.uint32))


@pytest.mark.parametrize("t,rows,width", [(2, 1, 2304), (4, 7, 5376), (8, 3, 512)])
def test_rmsnorm_gather_rank_order_sum(oracle, t, rows, width):
    """The tensor-parallel norm with its t ranks emulated as t local buffers (flags preset, nothing
    waits): partial sums added in rank order, then exactly the fused residual norms."""
    import lthn
    rng = np.random.default_rng(t)
    parts = rng.standard_normal((t, rows, width)).astype(np.float32)
    h = rng.standard_normal((rows, width)).astype(np.float32) * 5
    w1 = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    w2 = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    a = parts[0].copy()
    for r in range(1, t):
        a = (a + parts[r]).astype(np.float32)
    pb, hb, out, scratch = dev(lthn, parts), dev(lthn, h), lthn.Buf(rows * width * 4), lthn.Buf(512)
    w1b, w2b = dev(lthn, w1), dev(lthn, w2)
    lthn.check(lthn.lib().lthn_debug_rmsnorm_gather_local(None, pb.ptr, t, scratch.ptr, hb.ptr, w1b.ptr, w2b.ptr, out.ptr,
                                                         rows, width, 1e-6, 1, 0))
    h_want = np.stack([h[r] + oracle.rmsnorm(a[r], w1, 1e-6) for r in range(rows)]).astype(np.float32)
    out_want = np.stack([oracle.rmsnorm(h_want[r], w2, 1e-6) for r in range(rows)])
    assert np.array_equal(hb.download(np.float32, (rows, width)).view(np.uint32), h_want.view(np.uint32))
    assert np.array_equal(out.download(np.float32, (rows, width)).view(np.uint32), out_want.view(np.uint32))
    # a second exchange on the same scratch must see sequence number 2: flags still say 1, so it would
    # wait; instead check that the kernel advanced its counter exactly once
    ctr = scratch.download(np.uint32, (128,))
    assert ctr[64] == 1 and ctr[65] == 0


def test_bounded_device_wait_runs_out_and_is_reported(oracle):
    """A peer that never signals: the tensor-parallel norm polls its flag line a bounded number of
    times (here 1024 polls, a fraction of a millisecond), records the time-out in the device
    status word and returns by itself; the host turns that into LTHN_ERR_DEVICE_WAIT with the
    peer-wait bit (256). The context stays usable: the status reads clean afterwards and the
    same kernel, with its flags set, gives the exact result."""
    import lthn
    t, rows, width = 2, 2, 512
    rng = np.random.default_rng(9)
    parts = rng.standard_normal((t, rows, width)).astype(np.float32)
    h = rng.standard_normal((rows, width)).astype(np.float32)
    w1 = np.ones(width, dtype=np.float32)
    w2 = np.ones(width, dtype=np.float32)
    pb, out, scratch = dev(lthn, parts), lthn.Buf(rows * width * 4), lthn.Buf(512)
    w1b, w2b = dev(lthn, w1), dev(lthn, w2)
    assert lthn.device_status() == 0
    hb = dev(lthn, h)
    with pytest.raises(lthn.LthnError) as e:
        lthn.check(lthn.lib().lthn_debug_rmsnorm_gather_local(None, pb.ptr, t, scratch.ptr, hb.ptr, w1b.ptr, w2b.ptr,
                                                             out.ptr, rows, width, 1e-6, 0, 1024))
    assert e.value.code == 5 and "256" in e.value.msg
    assert lthn.device_status() == 0            # read-and-clear: the failure is reported once
    hb = dev(lthn, h)
    lthn.check(lthn.lib().lthn_debug_rmsnorm_gather_local(None, pb.ptr, t, scratch.ptr, hb.ptr, w1b.ptr, w2b.ptr,
                                                         out.ptr, rows, width, 1e-6, 1, 0))
    a = (parts[0] + parts[1]).astype(np.float32)
    h_want = np.stack([h[r] + oracle.rmsnorm(a[r], w1, 1e-6) for r in range(rows)]).astype(np.float32)
    assert np.array_equal(hb.download(np.float32, (rows, width)).view(np.uint32), h_want.view(np.uint32))
    # the asynchronous entry points report through the same word: a clean matvec leaves it clean
    from gpu_util import make_weight
    q = lthn.QuantWeight.from_host(*make_weight(oracle, 64, 128, seed=1))
    x, y = dev(lthn, np.ones((1, 128), dtype=np.float32)), lthn.Buf(64 * 4)
    lthn.qmv(x, lthn.F32, 1, q, y, lthn.F32)
    assert lthn.device_status() == 0


@pytest.mark.parametrize("heads,D,rotary", [(8, 256, 256), (4, 128, 128), (2, 512, 512), (3, 64, 32), (2, 512, 128)])
def test_rmsnorm_rope_f32(oracle, heads, D, rotary):
    """Per-head RMSNorm + NeoX RoPE vs hipOracleNormRoPEHeads (oracle_test.go:1103-1118):
    norm bit-exact, rotation to f32 rounding (device cos/sin come from f64 like the reference)."""
    import lthn
    rows = 5
    rng = np.random.default_rng(D + heads)
    x = rng.standard_normal((rows, heads * D)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    pos = np.array([0, 1, 17, 1023, 4607], dtype=np.int32)
    out = lthn.Buf(x.nbytes)
    lthn.check(lthn.lib().lthn_rmsnorm_rope(None, dev(lthn, x).ptr, dev(lthn, w).ptr, dev(lthn, pos).ptr, out.ptr, rows,
                                            heads, D, rotary, 1e-6, 10000.0, 0))
    got = out.download(np.float32, (rows, heads, D))
    for r in range(rows):
        for h in range(heads):
            n = oracle.rmsnorm(x[r, h * D:(h + 1) * D], w, 1e-6)
            want = oracle.rope_neox(n, int(pos[r]), 10000.0, D, rotary)
            np.testing.assert_allclose(got[r, h], want, rtol=0, atol=2e-6)


def test_rmsnorm_rope_bf16_seams(oracle):
    """bf16_seams=1 follows lthn_qknorm_rope_bf16.metal:75-110 (bf16(w*bf16(x*inv)), bf16 out)."""
    import lthn
    heads, D, rows = 4, 256, 3
    rng = np.random.default_rng(1)
    xb = oracle.f32_to_bf16(rng.standard_normal((rows, heads * D)).astype(np.float32))
    wb = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32))
    pos = np.array([3, 100, 2000], dtype=np.int32)
    out = lthn.Buf(rows * heads * D * 4)
    lthn.check(lthn.lib().lthn_rmsnorm_rope(None, dev(lthn, oracle.bf16_to_f32(xb)).ptr, dev(lthn, oracle.bf16_to_f32(wb)).ptr,
                                            dev(lthn, pos).ptr, out.ptr, rows, heads, D, D, 1e-6, 10000.0, 1))
    got = out.download(np.float32, (rows, heads * D))
    for r in range(rows):
        want = oracle.bf16_to_f32(oracle.qknorm_rope_bf16(xb[r], wb, heads, D, D, 1e-6, 1.0, int(pos[r]),
                                                          float(np.log2(10000.0))))
        # the shader itself is only cosine-tight against MLX (its header says so); one bf16 ulp here
        assert np.all(np.abs(got[r] - want) <= np.abs(want) * 2.0 ** -7 + 1e-3)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 4, 256), (32, 16, 128), (4, 4, 64), (8, 1, 128), (2, 1, 512), (16, 2, 64)])
@pytest.mark.parametrize("ctxs", [[1], [1280, 5, 64, 513], [4608]])
def test_sdpa_decode_matches_reference(oracle, Hq, Hkv, D, ctxs):
    """Decode attention over the seq-major bf16 cache vs
    hipReferenceSingleHeadAttentionWithScale with the GQA head map (oracle_test.go:907-924)."""
    import lthn
    rows, lanes = len(ctxs), len(ctxs)
    max_len = max(ctxs)
    KR = Hkv * D
    rng = np.random.default_rng(Hq * 1000 + D + max_len)
    kf = oracle.bf16_to_f32(oracle.f32_to_bf16(rng.standard_normal((lanes, max_len, KR)).astype(np.float32)))
    vf = oracle.bf16_to_f32(oracle.f32_to_bf16(rng.standard_normal((lanes, max_len, KR)).astype(np.float32)))
    q = rng.standard_normal((rows, Hq * D)).astype(np.float32)
    pos = np.array([c - 1 for c in ctxs], dtype=np.int32)
    lane = np.arange(rows, dtype=np.int32)
    out = lthn.Buf(q.nbytes)
    scale = float(np.float32(1.0 / np.sqrt(D)))
    lthn.check(lthn.lib().lthn_sdpa_decode(None, dev(lthn, q).ptr, dev(lthn, oracle.f32_to_bf16(kf)).ptr,
                                           dev(lthn, oracle.f32_to_bf16(vf)).ptr, dev(lthn, pos).ptr, dev(lthn, lane).ptr,
                                           out.ptr, rows, Hq, Hkv, D, max_len * KR, scale, max_len))
    lthn.sync()
    got = out.download(np.float32, (rows, Hq, D))
    for r in range(rows):
        for h in range(Hq):
            kvh = int(oracle.lib().lthn_o_kv_head_for_query(h, Hq, Hkv))
            want = oracle.attention_single_head(q[r, h * D:(h + 1) * D], kf[r, :ctxs[r], kvh * D:(kvh + 1) * D],
                                                vf[r, :ctxs[r], kvh * D:(kvh + 1) * D], scale)
            np.testing.assert_allclose(got[r, h], want, rtol=0, atol=3e-6 * max(1.0, np.abs(want).max()) + 2e-6)


@pytest.mark.parametrize("Hq,Hkv,D,rows,pos0", [(4, 2, 64, 70, 0), (8, 4, 256, 130, 0), (4, 2, 128, 64, 37), (2, 1, 128, 33, 480),
                                              (8, 4, 256, 512, 512), (4, 4, 64, 1, 5)])
def test_prefill_attention_matches_reference(oracle, Hq, Hkv, D, rows, pos0):
    """Causal attention of a prompt chunk (rows positions from pos0, keys 0..pos0+r) against
    hipReferenceSingleHeadAttentionWithScale per row and head with the GQA head map. The oracle is
    given the query rounded to bf16, which is what the kernel multiplies; the kernel also rounds
    its softmax weights to bf16 and stores bf16, which bounds the difference at a few bf16 ulps of
    the output scale (stated below), not at f32 noise."""
    import lthn
    KR = Hkv * D
    ctx = pos0 + rows
    rng = np.random.default_rng(Hq * 1000 + D + rows)
    kf = oracle.bf16_to_f32(oracle.f32_to_bf16(rng.standard_normal((ctx, KR)).astype(np.float32)))
    vf = oracle.bf16_to_f32(oracle.f32_to_bf16(rng.standard_normal((ctx, KR)).astype(np.float32)))
    q = (rng.standard_normal((rows, Hq * D)) * 2).astype(np.float32)
    qb = oracle.bf16_to_f32(oracle.f32_to_bf16(q))
    out = lthn.Buf(rows * Hq * D * 2)
    scale = float(np.float32(1.0 / np.sqrt(D)))
    lthn.prefill_attention(dev(lthn, q), dev(lthn, oracle.f32_to_bf16(kf)), dev(lthn, oracle.f32_to_bf16(vf)), out, rows, pos0,
                           Hq, Hkv, D, scale)
    lthn.sync()
    got = oracle.bf16_to_f32(out.download(np.uint16, (rows, Hq, D)))
    check_rows = sorted({r for r in [0, 1, rows // 2, rows - 1] + list(rng.integers(0, rows, 6)) if r < rows})
    for r in check_rows:
        for h in range(Hq):
            kvh = int(oracle.lib().lthn_o_kv_head_for_query(h, Hq, Hkv))
            n = pos0 + r + 1
            want = oracle.attention_single_head(qb[r, h * D:(h + 1) * D], kf[:n, kvh * D:(kvh + 1) * D],
                                                vf[:n, kvh * D:(kvh + 1) * D], scale)
            # bf16 output (2^-9 relative) + bf16 softmax weights (2^-9 each, averaged over the keys)
            np.testing.assert_allclose(got[r, h], want, rtol=2.0 ** -7, atol=2.0 ** -7 * max(np.abs(want).max(), 1e-3))


def test_argmax_lowest_index_wins_ties(oracle):
    """model.Greedy (model/sample.go:33-50): strict '>' from -inf, so ties go to the lowest index."""
    import lthn
    rows, V = 4, 262144
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((rows, V)).astype(np.float32)
    logits[1, [5000, 70000, 200000]] = 9.0   # three-way tie
    logits[2, V - 1] = 50.0                  # last element
    logits[3, :] = -1.5                      # all equal -> index 0
    out = lthn.Buf(rows * 4)
    lthn.check(lthn.lib().lthn_argmax(None, dev(lthn, logits).ptr, rows, V, out.ptr))
    got = out.download(np.int32, (rows,))
    want = [oracle.greedy_f32(logits[r]) for r in range(rows)]
    assert got.tolist() == want and got[1] == 5000 and got[2] == V - 1 and got[3] == 0
