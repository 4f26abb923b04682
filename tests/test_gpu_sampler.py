"""Sampling on the device path: the top-k selection kernel against the order the reference's
selectTopKDesc defines, and sampled decode (session and lane set) against the restatement of
model/sample.go fed the same device logits, token for token."""
import numpy as np
import pytest

from decoder_util import MID, SMALL, build_device, synth_weights
from oracle import sampler as osamp

pytestmark = pytest.mark.gpu


def _to_bf16_bits(v):
    b = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


@pytest.mark.parametrize("vocab,k,ties", [(2048, 40, False), (262144, 64, False), (262144, 256, True), (1000, 256, True),
                                          (5000, 1, False), (300, 7, True)])
def test_topk_candidates_match_stable_descending_order(lthn, vocab, k, ties):
    rng = np.random.default_rng(vocab + k)
    rows = 3
    x = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    if ties:
        x = np.round(x * 2) / 2          # a few dozen distinct values: the k-th value is shared by many entries
    x[1, :17] = 9.5                       # a run of equal maxima at the lowest indices
    d_x = lthn.Buf.from_array(x)
    d_s = lthn.Buf(rows * vocab * 2)
    d_i = lthn.Buf(rows * 256 * 4)
    d_v = lthn.Buf(rows * 256 * 2)
    lthn.topk_candidates(d_x, rows, vocab, k, d_s, d_i, d_v)
    lthn.sync()
    ids = d_i.download(np.int32, (rows, 256))[:, :k]
    vals = d_v.download(np.uint16, (rows, 256))[:, :k]
    bits = _to_bf16_bits(x)
    assert (d_s.download(np.uint16, (rows, vocab)) == bits).all()   # the row it rounded
    f = (bits.astype(np.uint32) << 16).view(np.float32)
    for r in range(rows):
        want = np.lexsort((np.arange(vocab), -f[r].astype(np.float64)))[:k]   # value descending, index ascending
        assert sorted(ids[r].tolist()) == sorted(want.tolist()), r
        assert (vals[r] == bits[r][ids[r]]).all()
    assert lthn.device_status() == 0
    for b in (d_x, d_s, d_i, d_v):
        b.free()


def test_topk_candidates_rejects_bad_k(lthn):
    d = lthn.Buf(4096)
    for k in (0, 257, 11):
        with pytest.raises(lthn.LthnError):
            lthn.topk_candidates(d, 1, 10, k, d, d, d)
    d.free()


CASES = [
    dict(temperature=0.8, top_k=40, top_p=0.9),                      # the top-k window leaves the device
    dict(temperature=1.0, top_k=256, min_p=0.02),
    dict(temperature=0.9),                                           # whole row read back
    dict(temperature=0.7, top_k=300),                                # wider than the device window
    dict(temperature=0.8, top_k=20, repeat_penalty=1.3),
    dict(temperature=1.1, top_k=50, min_tokens_before_stop=6),
    dict(suppress=(5, 17, 99), repeat_penalty=1.5),                  # greedy with a penalty and suppression
    dict(temperature=0.8, top_k=1),
]


def _reference_tokens(lthn, m, ids, kw, seed, n, stop):
    """The reference's loop, each step sampling with the restated sampler from the logits the device produced."""
    s = m.open_session()
    s.prefill(ids)
    o = osamp.Sampler(seed)

    def step(prev):
        if prev is not None:
            s.append([prev])
        return _to_bf16_bits(s.logits())
    toks = osamp.generate_sampled(step, o, osamp.SampleParams(**kw), n, stop)
    s.close()
    return toks


@pytest.mark.parametrize("ci", range(len(CASES)))
def test_session_decode_sampled_matches_reference_sampler(oracle, lthn, ci):
    kw = CASES[ci]
    cfg = SMALL
    w, norms = synth_weights(oracle, lthn, cfg, seed=40 + ci, random_norms=True)
    m = build_device(lthn, cfg, w, norms, 96)
    ids = np.random.default_rng(ci).integers(0, cfg["vocab"], 19).astype(np.int32)
    n = 24
    stop = ()
    if kw.get("min_tokens_before_stop"):
        # stop tokens = what an unconstrained run emits early, so the suppression window matters
        free = _reference_tokens(lthn, m, ids, {k: v for k, v in kw.items() if k != "min_tokens_before_stop"}, 1000 + ci, 4, ())
        stop = tuple(int(t) for t in free[:3])
    want = _reference_tokens(lthn, m, ids, kw, 1000 + ci, n, stop)
    s = m.open_session()
    s.prefill(ids)
    smp = lthn.Sampler(1000 + ci)
    got = s.decode_sampled(smp, lthn.sample_params(**kw), n, stop).tolist()
    assert got == want
    if stop:
        assert all(t not in stop for t in got[:kw["min_tokens_before_stop"]])
    assert s.pos == len(ids) + len(got) - 1       # the last token is yielded, not fed
    # the sampler advanced once per stochastic token: its next draw equals the restatement's
    o = osamp.Sampler(1000 + ci)
    stochastic = kw.get("temperature", 0) > 0 or kw.get("min_p", 0) > 0
    for _ in range(len(got) if stochastic else 0):
        o.next()
    assert smp.draw() == float(o.next())
    smp.close(); s.close(); m.close()


def _run_lanes(lthn, m, specs, n):
    """specs: (prompt, params or None, seed). Returns the tokens of each lane, in order."""
    ls = m.open_lane_set(len(specs))
    handles = [ls.prepare(p, max_new=n) if kw is None else ls.prepare_sampled(p, lthn.sample_params(**kw), seed, max_new=n)
               for (p, kw, seed) in specs]
    got = {h: [] for h in handles}
    while True:
        res = ls.step()
        if not res:
            break
        for h, tok, has, term in res:
            got[h].append(tok)
    ls.close()
    return [got[h] for h in handles]


def test_sampled_lanes_are_independent_of_their_batch(oracle, lthn, monkeypatch):
    """LaneSpec.Sampler / SampleSeed: every lane draws from its own row of the batched logits with
    its own stream. A lane's tokens therefore depend on its prompt, parameters and seed only: not on
    which row of the batch it occupies, nor on what the other lanes hold - with the batch width
    kept, so the same kernels produce the logits in every run (a row of the batched matvec does
    not depend on the other rows). The first token, drawn from the prefill's logits, and a greedy lane
    are also what a lone session gives; later sampled tokens are compared with a session in the
    single-lane test below, where both sides run the same kernels - a 4-row forward and a 1-row
    forward differ in the last bits of the logits, which moves a bf16 value across a rounding
    boundary now and then and with it a draw."""
    monkeypatch.setenv("LTHN_CUDA_PREFILL_F32", "1")
    cfg = MID
    w, norms = synth_weights(oracle, lthn, cfg, seed=9, random_norms=True)
    m = build_device(lthn, cfg, w, norms, 128, max_lanes=4)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, cfg["vocab"], k).astype(np.int32) for k in (11, 30, 5, 21, 17, 8, 26)]
    kws = [dict(temperature=0.8, top_k=40, top_p=0.9), dict(temperature=1.0), None, dict(temperature=0.7, top_k=30, repeat_penalty=1.2)]
    n = 12
    base = _run_lanes(lthn, m, [(prompts[i], kws[i], 500 + i) for i in range(4)], n)
    assert all(len(t) == n for t in base)
    # rotated rows
    rot = _run_lanes(lthn, m, [(prompts[i], kws[i], 500 + i) for i in (2, 3, 0, 1)], n)
    assert [rot[2], rot[3], rot[0], rot[1]] == base
    # lane 0 and lane 3 among other companions (different prompts, all sampled)
    other = _run_lanes(lthn, m, [(prompts[0], kws[0], 500), (prompts[4], kws[1], 7), (prompts[5], kws[0], 8), (prompts[3], kws[3], 503)], n)
    assert other[0] == base[0] and other[3] == base[3]
    assert other[1] != base[1]
    # another seed moves the stream
    reseed = _run_lanes(lthn, m, [(prompts[i], kws[i], 900 + i) for i in range(4)], n)
    assert reseed[2] == base[2] and reseed[0] != base[0]
    # against lone sessions: the greedy lane wholly, sampled lanes on their first token
    s = m.open_session()
    for i in range(4):
        s.prefill(prompts[i])
        if kws[i] is None:
            assert s.decode_greedy(n).tolist() == base[i]
        else:
            smp = lthn.Sampler(500 + i)
            solo = s.decode_sampled(smp, lthn.sample_params(**kws[i]), n).tolist()
            smp.close()
            same = next((j for j in range(n) if solo[j] != base[i][j]), n)
            print(f"lane {i}: first {same} of {n} sampled tokens equal the lone session's")
            assert same >= 1
    s.close(); m.close()


def test_single_sampled_lane_is_bit_identical_to_session(oracle, lthn):
    """One lane runs the kernels a session runs, so the sampled tokens are the same with no caveat."""
    cfg = SMALL
    w, norms = synth_weights(oracle, lthn, cfg, seed=3)
    m = build_device(lthn, cfg, w, norms, 96, max_lanes=1)
    ids = np.arange(13, dtype=np.int32) * 11 % cfg["vocab"]
    kw = dict(temperature=0.9, top_k=64, top_p=0.95, min_p=0.01, repeat_penalty=1.1)
    s = m.open_session()
    s.prefill(ids)
    smp = lthn.Sampler(2)
    want = s.decode_sampled(smp, lthn.sample_params(**kw), 30).tolist()
    smp.close(); s.close()
    ls = m.open_lane_set(1)
    h = ls.prepare_sampled(ids, lthn.sample_params(**kw), 2, max_new=30)
    got = []
    while True:
        res = ls.step()
        if not res:
            break
        got += [t for (_, t, _, _) in res]
    assert got == want
    ls.close(); m.close()
