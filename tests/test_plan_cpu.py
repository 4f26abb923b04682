"""Host logic of the integer tensor-core matvec: the plan (groups per warp, warps, ring stages, K slices, shared
memory) for every shape the decoders and benchmarks use, checked without a GPU against what the kernel and its
instantiations require. Runs against the test-hook build of the library (lthn_debug_i8_plan makes no CUDA call)."""
import ctypes as C

import numpy as np
import pytest

J4 = {1, 2, 3, 4, 6, 7, 8, 9, 12, 16, 18, 21}   # instantiated groups per warp, 4-bit codes
J8 = {2, 3, 4, 6, 9, 12}                         # 8-bit codes
SMEM_MAX = 224 * 1024


def plan(lthn, N, K, M, bits=4, fuse=0, norm=0, slices=1):
    out = (C.c_int64 * 12)()
    fn = getattr(lthn.lib(), "lthn_debug_i8_plan", None)
    if fn is None:
        pytest.skip("the test-hook build of the library is not loaded")
    if not fn(N, K, M, bits, fuse, norm, slices, out):
        return None
    keys = ("J", "W", "stg", "RS", "nblocks", "threads", "bs_off", "stage_off", "ks", "Gs", "fuse", "smem")
    return dict(zip(keys, [int(v) for v in out]))


def check(p, N, K, M, bits, fuse, norm):
    G = K // 64
    assert p["J"] * p["W"] == p["Gs"] and p["Gs"] * p["ks"] == G
    assert 1 <= p["W"] <= 16 and p["threads"] == (p["W"] + 1) * 32
    assert p["J"] in (J8 if bits == 8 else J4)
    assert not (p["W"] > 8 and p["J"] > 9)               # the 544-thread class is built for J <= 9
    assert 2 <= p["stg"] <= 4 and p["smem"] <= SMEM_MAX
    rowbytes = p["Gs"] * bits * 8
    assert p["RS"] >= rowbytes and p["RS"] % 16 == 0 and rowbytes % 16 == 0   # bulk copies: 16-byte rows
    assert (p["RS"] // 4) % 32 == 8                      # rows 8 banks apart: conflict-free 8-byte fragment loads
    if fuse or norm:
        assert p["ks"] == 1                              # a GeGLU epilogue and a norm prologue need whole rows
    if fuse:
        assert p["fuse"] in (1, 2)
    out_rows = 8 if p["fuse"] == 2 else 16
    assert p["nblocks"] == (N + out_rows - 1) // out_rows
    sets = 2 if p["fuse"] == 1 else 1
    sb = (16 * p["Gs"] * 2 + 15) // 16 * 16
    stage = sets * (16 * p["RS"] + 2 * sb)
    assert p["stage_off"] % 128 == 0 and p["stage_off"] + p["stg"] * stage == p["smem"]
    assert p["bs_off"] >= 512 + 2 * p["stg"] * p["W"] * sets * 16 * M * 4   # partial-sum ring in front of the scratch


DECODER_SHAPES = [  # (N, K, fuse) of the 26-layer and 62-layer decoders, whole and per tensor-parallel shard
    (4096, 2304, 0), (2304, 2048, 0), (9216, 2304, 1), (2304, 9216, 0), (262144, 2304, 0),
    (8192, 5376, 0), (5376, 4096, 0), (21504, 5376, 1), (5376, 21504, 0), (262144, 5376, 0),
    (4096, 5376, 0), (5376, 2048, 0), (10752, 5376, 1), (5376, 10752, 0), (131072, 5376, 0),
    (2048, 5376, 0), (5376, 1024, 0), (5376, 5376, 0), (2688, 5376, 1), (5376, 2688, 0), (32768, 5376, 0),
]


@pytest.mark.parametrize("M", [1, 2])
def test_four_bit_plans_of_the_decoder_shapes(lthn, M):
    for N, K, fuse in DECODER_SHAPES:
        for norm in (0, 1):
            p = plan(lthn, N, K, M, 4, fuse, norm)
            if K > 10752:
                # rows longer than the ring holds: whole-row plan refused (the dp4a kernel serves them by default) ...
                assert p is None
                if not fuse and not norm:
                    q = plan(lthn, N, K, M, 4, 0, 0, slices=8)   # ... and sliced when the caller allows slices
                    assert q is not None and q["ks"] > 1
                    check(q, N, K, M, 4, 0, 0)
                continue
            assert p is not None, (N, K, fuse, norm)
            check(p, N, K, M, 4, fuse, norm)


@pytest.mark.parametrize("M", [1, 2])
def test_eight_bit_plans(lthn, M):
    """8-bit codes: whole rows up to K ~ 5400, K slices beyond (the slice count whose slices are nearest 24 groups),
    GeGLU pairs and norm prologues on whole rows only."""
    for N, K, fuse in [(9216, 2304, 1), (9216, 2304, 0), (21504, 5376, 1), (21504, 5376, 0), (131072, 2304, 0), (4096, 2304, 0),
                       (512, 256, 1), (1024, 512, 1), (64, 128, 1)]:
        for norm in (0, 1):
            p = plan(lthn, N, K, M, 8, fuse, norm)
            assert p is not None, (N, K, fuse, norm)
            assert p["ks"] == 1
            check(p, N, K, M, 8, fuse, norm)
            if fuse:
                assert p["fuse"] == (2 if K >= 2048 else 1)
    assert plan(lthn, 16, 64, M, 8) is None   # a single group: no 8-bit instantiation, the general kernel serves it
    for N, K, ks in [(2304, 9216, 6), (5376, 21504, 8), (512, 1024 * 8, 4)]:
        p = plan(lthn, N, K, M, 8)
        assert p is not None and p["ks"] == ks, (N, K, p)
        check(p, N, K, M, 8, 0, 0)
        assert plan(lthn, N, K, M, 8, 1, 0) is None and plan(lthn, N, K, M, 8, 0, 1) is None


def test_plans_over_a_grid_of_shapes(lthn):
    """Whatever the planner accepts satisfies the kernel's requirements; what it must refuse, it refuses."""
    rng = np.random.default_rng(0)
    seen = 0
    for _ in range(1500):
        N = int(rng.integers(1, 600)) * 16
        K = int(rng.integers(1, 340)) * 64
        M = int(rng.integers(1, 3))
        bits = int(rng.choice([4, 8]))
        fuse, norm = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        p = plan(lthn, N, K, M, bits, fuse, norm, slices=int(rng.choice([1, 8])))
        if p is not None:
            check(p, N, K, M, bits, fuse, norm)
            seen += 1
    assert seen > 150   # most random K have no (groups per warp) x (warps) factorisation among the instantiations
    for bad in [(24, 128, 1), (16, 96, 1), (16, 64, 3), (0, 64, 1)]:   # N % 16, K % 64, more than two rows, empty
        assert plan(lthn, *bad, 4) is None and plan(lthn, *bad, 8) is None
