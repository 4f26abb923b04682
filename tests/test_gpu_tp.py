"""Tensor-parallel decoder on 2 GPUs (skipped on a single-GPU box): both ranks hold row/column
shards of the same synthetic weights, combine partial sums over peer memory (and, second run,
with NCCL all-reduce), and must produce the tokens a single GPU produces."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

CFG = dict(layers=3, hidden=512, q_heads=8, kv_heads=4, head_dim=64, ffn=1024, vocab=2048)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_model(lthn, rank, world, comm, ids, new, want_mode=None):
    mc = lthn.make_config(CFG["layers"], CFG["hidden"], CFG["q_heads"], CFG["kv_heads"], CFG["head_dim"], CFG["ffn"],
                          CFG["vocab"], len(ids) + new, 1, tp_rank=rank, tp_size=world)
    m = lthn.Model(mc)
    m.synthesize(21, 0.02)
    if comm is not None:
        m.set_comm(comm)
    m.finalize()
    if want_mode is not None:
        assert m.tp_exchange == want_mode
    s = m.open_session()
    s.prefill(ids)
    toks = s.decode_greedy(new)
    s.close()
    m.close()
    return toks


def _worker(rank, world, port, out):
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
        ids = np.random.default_rng(4).integers(0, CFG["vocab"], 45).astype(np.int32)
        toks = _run_model(lthn, rank, world, comm, ids, 24, want_mode=2)   # partial sums read from peer memory
        os.environ["LTHN_CUDA_TP_NCCL"] = "1"
        toks_nccl = _run_model(lthn, rank, world, comm, ids, 24, want_mode=1)   # NCCL all-reduce path
        del os.environ["LTHN_CUDA_TP_NCCL"]
        solo = _run_model(lthn, 0, 1, None, ids, 24, want_mode=0) if rank == 0 else None
        lthn.check(lthn.lib().lthn_tp_destroy(comm))
        out.put((rank, toks.tolist(), toks_nccl.tolist(), None if solo is None else solo.tolist()))
    finally:
        dist.destroy_process_group()


def test_tp2_tokens_equal_single_gpu():
    import lthn
    if lthn.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, t0, n0, solo), (_, t1, n1, _) = res
    assert t0 == t1 and n0 == n1   # every rank returns the same tokens
    assert t0 == solo              # the peer-memory exchange reproduces the single-GPU tokens
    assert n0 == solo              # and so does the NCCL all-reduce path
