"""Host-side tensor-parallel plumbing: how a Gemma-style decoder's linears are split
over `world` ranks, and how a rank joins the NCCL communicator of the library.

The split mirrors lthn_model_upload_linear (which keeps only this rank's part of the full
tensor it is given): q/k/v/gate/up by output rows, o/down by input columns in whole
64-wide groups, lm_head by vocabulary rows. The reference is single-device; this is new
functionality. torch.distributed is used only to move the 128-byte communicator id."""
from __future__ import annotations

import numpy as np

COLUMN_PARALLEL = ("q", "k", "v", "gate", "up")   # sharded by output rows
ROW_PARALLEL = ("o", "down")                      # sharded by input columns (K)


def shard_linear(role: str, packed: np.ndarray, scales: np.ndarray, biases: np.ndarray, rank: int, world: int,
                 bits: int = 4, gs: int = 64):
    """Returns this rank's (packed, scales, biases) of a full [N,K] MLX-affine tensor."""
    n = packed.shape[0]
    k = packed.shape[1] * 32 // bits
    if role in COLUMN_PARALLEL or role == "lm_head":
        if n % world:
            raise ValueError(f"{role}: {n} rows do not divide by {world}")
        r0, r1 = rank * n // world, (rank + 1) * n // world
        return packed[r0:r1], scales[r0:r1], biases[r0:r1]
    if role in ROW_PARALLEL:
        if k % (world * gs):
            raise ValueError(f"{role}: K={k} does not split into whole groups over {world} ranks")
        k0, k1 = rank * k // world, (rank + 1) * k // world
        wpe = 32 // bits
        return (np.ascontiguousarray(packed[:, k0 // wpe:k1 // wpe]), np.ascontiguousarray(scales[:, k0 // gs:k1 // gs]),
                np.ascontiguousarray(biases[:, k0 // gs:k1 // gs]))
    raise ValueError(f"unknown role {role}")


def activation_slice(role: str, width: int, rank: int, world: int) -> slice:
    """Columns of the input activation a row-parallel linear consumes on this rank."""
    if role not in ROW_PARALLEL:
        return slice(0, width)
    return slice(rank * width // world, (rank + 1) * width // world)


def merge_argmax(values: np.ndarray, indices: np.ndarray) -> int:
    """Best (value, global index) over ranks: strict '>', lowest index wins ties
    (model.Greedy, model/sample.go:33-50, applied to per-rank winners)."""
    best_v, best_i = -np.inf, np.iinfo(np.int64).max
    for v, i in zip(values, indices):
        if v > best_v or (v == best_v and i < best_i):
            best_v, best_i = v, i
    return int(best_i)


def init_comm(rank: int, world: int):
    """Builds the library's NCCL communicator; the id travels over torch.distributed."""
    import ctypes as C

    import torch
    import torch.distributed as dist

    import lthn
    buf = (C.c_char * 128)()
    if rank == 0:
        lthn.check(lthn.lib().lthn_tp_unique_id(buf))
    t = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.broadcast(t, src=0)
    raw = bytes(t.cpu().numpy().tobytes())
    idbuf = (C.c_char * 128).from_buffer_copy(raw)
    comm = C.c_void_p()
    lthn.check(lthn.lib().lthn_tp_init(rank, world, idbuf, C.byref(comm)))
    return comm
