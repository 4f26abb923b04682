"""lthn_affine_qmv_noalloc: the entry point for callers that cannot allocate device memory.

A host that fixed its HBM budget at start-up, or that runs where the CUDA allocator must not
be entered, still needs the decode matvec on f32 activations; this entry point keeps the
kernel's scratch in a fixed array inside the library instead of an arena. The test calls it
twice in a row through the C ABI (the second call reuses the array with different contents)
and compares each result with lthn_affine_qmv on the same inputs, at the tolerance the qmv
tests use. It is collected last so a run that stops at the first failure has already run
every other test, and it passes both alone in a fresh process and after the others."""
import numpy as np
import pytest

from gpu_util import make_weight, rms_err

pytestmark = pytest.mark.gpu

TOL = 2e-5  # of the output RMS, as in tests/test_gpu_qmv.py


def _run_both(lthn, oracle, q, x):
    M, K = x.shape
    xd = lthn.Buf.from_array(x)
    y_ref = lthn.Buf(M * q.N * 4)
    y_new = lthn.Buf(M * q.N * 4)
    lthn.qmv(xd, lthn.F32, M, q, y_ref, lthn.F32)
    lthn.qmv_noalloc(xd, M, q, y_new)
    lthn.sync()
    return y_new.download(np.float32, (M, q.N)), y_ref.download(np.float32, (M, q.N))


def test_noalloc_matches_existing_entry_point_twice_in_a_row(oracle):
    import lthn
    N, K = 2304, 2304
    p, s, b = make_weight(oracle, N, K, seed=12)
    q = lthn.QuantWeight.from_host(p, s, b)
    rng = np.random.default_rng(5)
    for call, M in enumerate((3, 1)):   # second call: other size, other data, same fixed scratch
        x = rng.standard_normal((M, K)).astype(np.float32) * (1.0 + call)
        got, ref = _run_both(lthn, oracle, q, x)
        assert rms_err(got, ref) <= TOL, (call, M)
        want = oracle.matnt_quant_host(x, p, s, b, threads=4)
        assert rms_err(got, want) <= (TOL if M <= 2 else 4e-5), (call, M)


def test_noalloc_allocates_no_device_memory_and_reports_its_status(oracle):
    """The property in the name: calls of the entry point leave the device's free memory untouched
    (cudaMemGetInfo before and after), for both kernel shapes (1-2 rows, 3-32 rows). One call per
    shape comes first, untimed: the CUDA runtime loads a kernel's code into device memory at its
    first launch, which is the runtime's doing and happens once per process. Its status word,
    which lives in the same fixed array, reads clean through lthn_device_status."""
    import lthn
    N, K = 1024, 2304
    q = lthn.QuantWeight.from_host(*make_weight(oracle, N, K, seed=3))
    xs = {M: lthn.Buf.from_array(np.random.default_rng(M).standard_normal((M, K)).astype(np.float32)) for M in (1, 8)}
    ys = {M: lthn.Buf(M * N * 4) for M in (1, 8)}
    for M in (1, 8):
        lthn.qmv_noalloc(xs[M], M, q, ys[M])
    lthn.sync()
    free0, _ = lthn.mem_info()
    for _ in range(2):
        for M in (1, 8):
            lthn.qmv_noalloc(xs[M], M, q, ys[M])
    assert lthn.device_status() == 0
    free1, _ = lthn.mem_info()
    assert free1 == free0, (free0, free1)


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(oracle):
    import lthn
    q = lthn.QuantWeight.from_host(*make_weight(oracle, 16, 64, seed=1))
    big_k = 16384                      # M=32 needs 32*2*16384*2 = 2 MiB of columns > 512 KiB
    x = lthn.Buf(32 * big_k * 4)
    y = lthn.Buf(32 * 16 * 4)
    with pytest.raises(lthn.LthnError) as e:
        lthn.check(lthn.lib().lthn_affine_qmv_noalloc(None, x.ptr, 32, q.packed.ptr, q.scales.ptr, q.biases.ptr, 16,
                                                      big_k, y.ptr))
    assert "exceed the fixed scratch" in str(e.value)
    with pytest.raises(lthn.LthnError):
        lthn.check(lthn.lib().lthn_affine_qmv_noalloc(None, x.ptr, 1, q.packed.ptr, q.scales.ptr, q.biases.ptr, 16, 96,
                                                      y.ptr))  # K not a multiple of 64
