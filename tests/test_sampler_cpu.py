"""The library's host sampler (lthn_sampler_*) against the restatement of model/sample.go in
oracle/sampler.py: every branch of Sampler.Sample - greedy, top-k = 1, top-k first, top-p, min-p,
the plain vocabulary-order draw, suppression, candidate ids - gives the same token at the same
seed, and the two random streams stay in step afterwards. No GPU is touched."""
import numpy as np
import pytest

from oracle import sampler as osamp


def _bf16_row(rng, n, spread=4.0, ties=False):
    v = (rng.standard_normal(n) * spread).astype(np.float32)
    if ties:
        v = np.round(v)   # many equal values
    return np.array([osamp.f32_to_bf16(x) for x in v], dtype=np.uint16)


def test_splitmix64_stream_known_values(lthn):
    # splitmix64 from state 0: the first outputs are the published 0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4
    s = lthn.Sampler(0)
    o = osamp.Sampler(0)
    want = [np.float32(0xE220A8397B1DCDAF >> 40) / np.float32(1 << 24), np.float32(0x6E789E6AA1B965F4 >> 40) / np.float32(1 << 24)]
    for w in want:
        a, b = s.draw(), float(o.next())
        assert a == b == float(w)
    s.close()


PARAMS = [
    dict(),                                               # greedy
    dict(temperature=0.8),                                # vocabulary-order draw
    dict(temperature=1.0, top_k=1),                       # top-1 with a burnt draw
    dict(temperature=0.7, top_k=40),                      # top-k first
    dict(temperature=0.7, top_k=40, top_p=0.9),
    dict(temperature=1.3, top_k=64, top_p=0.95, min_p=0.05),
    dict(temperature=0.9, top_p=0.8),                     # full sort, nucleus
    dict(temperature=0.9, min_p=0.1),
    dict(min_p=0.2),                                      # temperature 0 with min_p: samples at temperature 1
    dict(temperature=0.6, top_k=5000),                    # top_k >= vocab: no rank filter
    dict(temperature=0.7, top_k=20, suppress=(3, 7, 11, 500)),
    dict(suppress=(0, 1, 2)),
]


@pytest.mark.parametrize("pi", range(len(PARAMS)))
@pytest.mark.parametrize("ties", [False, True])
def test_sample_matches_reference_restatement(lthn, pi, ties):
    kw = PARAMS[pi]
    rng = np.random.default_rng(100 + pi)
    vocab = 1536
    s = lthn.Sampler(77 + pi)
    o = osamp.Sampler(77 + pi)
    lp = lthn.sample_params(**kw)
    op = osamp.SampleParams(**kw)
    for _ in range(12):
        row = _bf16_row(rng, vocab, ties=ties)
        if kw.get("suppress") and not ties:
            row[kw["suppress"][0]] = osamp.f32_to_bf16(50.0)   # the best token is a suppressed one
        assert s.sample(row, lp) == o.sample(row, op)
    assert s.draw() == float(o.next())   # the streams advanced the same number of times
    s.close()


def test_sample_candidates_uses_ids(lthn):
    rng = np.random.default_rng(5)
    s, o = lthn.Sampler(9), osamp.Sampler(9)
    kw = dict(temperature=0.8, top_k=8, top_p=0.9, suppress=(1234,))
    lp, op = lthn.sample_params(**kw), osamp.SampleParams(**kw)
    for _ in range(10):
        vals = _bf16_row(rng, 40)
        ids = rng.permutation(5000)[:40].astype(np.int32)
        ids[3] = 1234
        assert s.sample(vals, lp, ids) == o.sample(vals, op, ids)
    s.close()


def test_top_k_window_equals_full_row(lthn):
    """The claim the engine's device path rests on (argued at sample.go:165-175): sampling from only
    the top-k entries, passed with their ids in (value descending, index ascending) order or in any
    order, gives the token the full row gives, for any top_p / min_p."""
    rng = np.random.default_rng(8)
    vocab, k = 4096, 50
    for trial in range(8):
        row = _bf16_row(rng, vocab, ties=(trial % 2 == 1))
        vals = (row.astype(np.uint32) << 16).view(np.float32)
        order = sorted(range(vocab), key=lambda i: (-float(vals[i]), i))[:k]
        kw = dict(temperature=0.7 + 0.1 * trial, top_k=k, top_p=0.9, min_p=0.02)
        full, win, shuf = lthn.Sampler(trial), lthn.Sampler(trial), lthn.Sampler(trial)
        lp = lthn.sample_params(**kw)
        a = full.sample(row, lp)
        b = win.sample(row[order], lp, np.array(order, dtype=np.int32))
        # index order (what the device compaction emits): top_k == n there, so the ranked sort re-derives the order
        idx = np.array(sorted(order), dtype=np.int32)
        c = shuf.sample(row[idx], lp, idx)
        assert a == b == c
        for x in (full, win, shuf):
            x.close()


def test_all_suppressed_is_an_error(lthn):
    s = lthn.Sampler(1)
    row = _bf16_row(np.random.default_rng(0), 4)
    with pytest.raises(lthn.LthnError):
        s.sample(row, lthn.sample_params(temperature=0.5, suppress=(0, 1, 2, 3)))
    with pytest.raises(lthn.LthnError):
        s.sample(row, lthn.sample_params(suppress=(0, 1, 2, 3)))
    s.close()


def test_repeat_penalty_restatement():
    row = np.array([osamp.f32_to_bf16(x) for x in (2.0, -2.0, 0.5, 3.0)], dtype=np.uint16)
    out = osamp.apply_repeat_penalty(row, [0, 1, 1, 9], 2.0)
    got = [float(osamp.bf16_to_f32(b)) for b in out]
    assert got == [1.0, -4.0, 0.5, 3.0]
    assert (osamp.apply_repeat_penalty(row, [0], 1.0) == row).all()
