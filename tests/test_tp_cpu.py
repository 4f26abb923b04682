"""Tensor-parallel host logic on CPU: two gloo ranks shard a decoder layer's linears the
way the engine does, compute their partial projections with the CPU oracle, exchange with
all-reduce / all-gather, and must reproduce the single-rank result."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "go-inference_b200"))
    import torch
    import torch.distributed as dist
    from lthn import tp
    from oracle import oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, F, QR, V = 256, 512, 256, 1024
        rng = np.random.default_rng(0)  # same tensors on every rank
        full = {r: o.quantize((rng.standard_normal(shape) * 0.02).astype(np.float32))
                for r, shape in (("q", (QR, H)), ("o", (H, QR)), ("gate", (F, H)), ("up", (F, H)), ("down", (H, F)),
                                 ("lm_head", (V, H)))}
        x = rng.standard_normal((3, H)).astype(np.float32)

        def proj(w, xin):
            return o.hip_affine_projection_rows(xin, *w)

        # reference: unsharded layer slice q -> o, gate/up -> GeGLU -> down, lm_head argmax
        q_ref = proj(full["q"], x)
        o_ref = proj(full["o"], q_ref)
        act_ref = o.gelu_tanh(proj(full["gate"], x)) * proj(full["up"], x)
        d_ref = proj(full["down"], act_ref)
        tok_ref = [o.greedy_f32(row) for row in proj(full["lm_head"], x)]

        sh = {r: tp.shard_linear(r, *full[r], rank, world) for r in full}
        q_loc = proj(sh["q"], x)                                   # column parallel: a slice of the outputs
        assert np.array_equal(q_loc, q_ref[:, rank * QR // world:(rank + 1) * QR // world])
        o_part = torch.from_numpy(proj(sh["o"], q_loc))            # row parallel: partial sums
        dist.all_reduce(o_part)
        act_loc = o.gelu_tanh(proj(sh["gate"], x)) * proj(sh["up"], x)
        d_part = torch.from_numpy(proj(sh["down"], act_loc))
        dist.all_reduce(d_part)
        logits_loc = proj(sh["lm_head"], x)                        # vocab shard -> (value, global index) per row
        pairs = torch.tensor([[row.max(), float(int(row.argmax()) + rank * V // world)] for row in logits_loc],
                             dtype=torch.float64)
        gathered = [torch.zeros_like(pairs) for _ in range(world)]
        dist.all_gather(gathered, pairs)
        toks = [tp.merge_argmax([g[r, 0].item() for g in gathered], [int(g[r, 1].item()) for g in gathered])
                for r in range(3)]
        ok = (np.allclose(o_part.numpy(), o_ref, rtol=0, atol=2e-5 * np.abs(o_ref).max())
              and np.allclose(d_part.numpy(), d_ref, rtol=0, atol=2e-5 * np.abs(d_ref).max()) and toks == tok_ref)
        out.put((rank, ok, toks, tok_ref))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_single_rank():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, toks, ref in res:
        assert ok, (rank, toks, ref)


def test_shard_shapes_and_rejections():
    sys.path.insert(0, os.path.join(ROOT, "go-inference_b200"))
    from lthn import tp
    packed = np.zeros((64, 32), dtype=np.uint32)   # [64, 256] 4-bit
    sc = np.zeros((64, 4), dtype=np.uint16)
    p, s, b = tp.shard_linear("gate", packed, sc, sc, 1, 4)
    assert p.shape == (16, 32) and s.shape == (16, 4)
    p, s, b = tp.shard_linear("down", packed, sc, sc, 3, 4)
    assert p.shape == (64, 8) and s.shape == (64, 1)
    with pytest.raises(ValueError):
        tp.shard_linear("down", packed, sc, sc, 0, 8)   # 256/8 = 32 columns: not a whole group
    with pytest.raises(ValueError):
        tp.shard_linear("q", packed[:63], sc[:63], sc[:63], 0, 2)
    assert tp.activation_slice("o", 256, 1, 4) == slice(64, 128)
    assert tp.merge_argmax([1.0, 3.0, 3.0], [7, 900, 20]) == 20
