"""Tensor-parallel decoder on 2, 4 and 8 GPUs (each degree is skipped where the box has fewer):
every rank holds row/column shards of the same synthetic weights, the ranks combine partial sums
over peer memory (and, second run, with NCCL all-reduce), and must produce the tokens a single
GPU produces. Two models: a small one, and one with the projection shapes of the 62-layer
5376-wide decoder (hidden 5376, 32/16 heads x 128, FFN 21504, vocabulary 262144) cut to 4
layers, whose single-GPU tokens are also held against the CPU reference decoder - that test
runs on one GPU too."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

CFG = dict(layers=3, hidden=512, q_heads=8, kv_heads=4, head_dim=64, ffn=1024, vocab=2048)
# projection shapes of the 62-layer model, 4 layers: K = 5376, 4096 and 21504 on one GPU,
# 2048 / 10752 at two ranks, 512 / 2688 at eight
CFG_WIDE = dict(layers=4, hidden=5376, q_heads=32, kv_heads=16, head_dim=128, ffn=21504, vocab=262144)
# prompts of at most 32 tokens are fed through the decode kernels (f32 activations), which is what
# makes token identity with the CPU reference a fair demand; longer prompts take the bf16 prefill path
WIDE_PROMPT, WIDE_NEW, WIDE_SEED = 30, 24, 33


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_model(lthn, cfg, seed, rank, world, comm, ids, new, want_mode=None, kv_out=None):
    mc = lthn.make_config(cfg["layers"], cfg["hidden"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"],
                          cfg["vocab"], len(ids) + new, 1, tp_rank=rank, tp_size=world)
    m = lthn.Model(mc)
    m.synthesize(seed, 0.02)
    if comm is not None:
        m.set_comm(comm)
    m.finalize()
    if want_mode is not None:
        assert m.tp_exchange == want_mode, (m.tp_exchange, want_mode)
    s = m.open_session()
    s.prefill(ids)
    if kv_out is not None:
        # rows 3..19 of the first layer's keys and values with the kv heads of every rank (one all-gather)
        kv_out["k"] = s.kv_export_range(0, 0, 3, 17, gathered=True)
        kv_out["v"] = s.kv_export_range(0, 1, 3, 17, gathered=True)
    toks = s.decode_greedy(new)
    s.close()
    m.close()
    return toks


def _worker(rank, world, port, wide, out):
    """One rank. Whatever happens, something lands on the queue, so the parent never waits for a
    rank that has already failed."""
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "go-inference_b200"))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        import lthn
        from lthn import tp
        lthn.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        try:
            comm = tp.init_comm(rank, world)
            res = {}
            if wide:
                ids = np.random.default_rng(6).integers(0, CFG_WIDE["vocab"], WIDE_PROMPT).astype(np.int32)
                res["peer"] = _run_model(lthn, CFG_WIDE, WIDE_SEED, rank, world, comm, ids, WIDE_NEW, want_mode=2).tolist()
            else:
                ids = np.random.default_rng(4).integers(0, CFG["vocab"], 31).astype(np.int32)
                kv = {}
                res["peer"] = _run_model(lthn, CFG, 21, rank, world, comm, ids, 24, want_mode=2, kv_out=kv).tolist()
                res["kv"] = kv
                os.environ["LTHN_CUDA_TP_NCCL"] = "1"
                res["nccl"] = _run_model(lthn, CFG, 21, rank, world, comm, ids, 24, want_mode=1).tolist()
                del os.environ["LTHN_CUDA_TP_NCCL"]
            if rank == 0:
                cfg, seed, new = (CFG_WIDE, WIDE_SEED, WIDE_NEW) if wide else (CFG, 21, 24)
                skv = {} if not wide else None
                res["solo"] = _run_model(lthn, cfg, seed, 0, 1, None, ids, new, want_mode=0, kv_out=skv).tolist()
                res["solo_kv"] = skv
            lthn.check(lthn.lib().lthn_tp_destroy(comm))
            out.put((rank, res, None))
        finally:
            dist.destroy_process_group()
    except BaseException as e:  # noqa: BLE001 - reported to the parent, which fails the test with it
        out.put((rank, None, f"{type(e).__name__}: {e}"))


def _run_ranks(world, wide, timeout):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, wide, out), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results, errors = {}, []
    try:
        for _ in procs:
            rank, res, err = out.get(timeout=timeout)
            if err:
                errors.append((rank, err))
                break   # the other ranks may be waiting for this one: stop them below
            results[rank] = res
    finally:
        for p in procs:
            p.join(timeout=10 if errors else 60)
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
            if p.is_alive():
                p.kill()
    assert not errors, errors
    assert len(results) == world
    return results


def _world_or_skip(world):
    import lthn
    if lthn.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_tokens_equal_single_gpu(world):
    _world_or_skip(world)
    res = _run_ranks(world, wide=False, timeout=300)
    solo = res[0]["solo"]
    for r in range(world):
        assert res[r]["peer"] == solo, r   # the peer-memory exchange reproduces the single-GPU tokens on every rank
        assert res[r]["nccl"] == solo, r   # and so does the NCCL all-reduce path
        # the gathered cache rows hold every rank's kv heads in model order: the single-GPU rows, up to rare one-ulp flips
        for which in ("k", "v"):
            got, want = res[r]["kv"][which], res[0]["solo_kv"][which]
            assert got.shape == want.shape == (17, CFG["kv_heads"] * CFG["head_dim"]), (got.shape, want.shape)
            f = lambda a: (a.astype(np.uint32) << 16).view(np.float32)
            assert float(np.mean(got != want)) < 2e-2, (r, which, float(np.mean(got != want)))
            assert np.all(np.abs(f(got) - f(want)) <= 2.0 ** -6 * np.abs(f(want)) + 5e-3 * np.max(np.abs(f(want))))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_wide_model_tokens_equal_single_gpu(world):
    """Projection shapes of the 62-layer model at every tensor-parallel degree: row-parallel K of
    4096/world and 21504/world, vocabulary shards of 262144/world with the (value, index) gather."""
    _world_or_skip(world)
    res = _run_ranks(world, wide=True, timeout=600)
    solo = res[0]["solo"]
    for r in range(world):
        assert res[r]["peer"] == solo, r


def test_wide_model_single_gpu_matches_cpu_reference(oracle):
    """The same 4-layer, 5376-wide model on one GPU against the CPU reference decoder: prompt
    logits within the decoder bound and the greedy tokens identical. This pins the tokens the
    tensor-parallel runs above are compared with."""
    import lthn
    from decoder_util import build_oracle, synth_weights_from_device
    cfg = CFG_WIDE
    ids = np.random.default_rng(6).integers(0, cfg["vocab"], WIDE_PROMPT).astype(np.int32)
    got = _run_model(lthn, cfg, WIDE_SEED, 0, 1, None, ids, WIDE_NEW, want_mode=0)
    w, norms = synth_weights_from_device(lthn, cfg, WIDE_SEED)
    od = build_oracle(oracle, cfg, w, norms, WIDE_PROMPT + WIDE_NEW)
    want_logits = od.forward(ids)
    want, margin = od.generate(want_logits, WIDE_NEW)
    first_bad = next((i for i in range(WIDE_NEW) if got[i] != want[i]), None)
    assert first_bad is None, f"diverged at step {first_bad}: reference margin {float(margin[first_bad]):.3e}"
