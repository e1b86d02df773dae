"""Tensor-parallel host side: one process per GPU, each holding a shard of every layer.

The split (the 70B-class configuration): q/k/v/gate/up by output rows (whole heads / FFN columns), o/down by input
columns, the KV cache by kv head, the LM head by vocabulary slice; norms and the embedding table are replicated. The
library sums the partial products of o and down across ranks and gathers the logits slices; this module only prepares
each rank's configuration and tensors and carries the communicator id between the processes.

Also here, for the replica configurations (every other shape: one engine per GPU, no collective): request placement over
ranks and the max-over-ranks reduction a benchmark reports.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Iterable, List, Optional

import numpy as np

from . import abi
from .synth import Shape

ROW_SPLIT = (abi.T_WQ, abi.T_WK, abi.T_WV, abi.T_GATE, abi.T_UP, abi.T_LM_HEAD)  # by output rows
COL_SPLIT = (abi.T_WO, abi.T_DOWN)                                                # by input columns
NCCL_ID_BYTES = 128


def check_divides(s: Shape, t: int):
    """Raises when the shape does not split over t ranks (Q4_K rows need every K/t to stay a multiple of 256)."""
    if t < 1:
        raise ValueError("tensor-parallel size must be at least 1")
    if s.n_experts:
        raise ValueError("tensor parallel is built for dense models")
    qd = s.n_heads * s.head_dim
    for name, v, mult in (("n_heads", s.n_heads, 1), ("n_kv_heads", s.n_kv_heads, 1), ("ffn", s.ffn, 1), ("vocab", s.vocab, 1),
                          ("o-proj input (n_heads*head_dim)", qd, 256), ("down-proj input (ffn)", s.ffn, 256)):
        if v % (t * mult):
            raise ValueError(f"{name} = {v} does not split over {t} ranks" + (" in whole Q4_K super-blocks" if mult > 1 else ""))


def local_shape(s: Shape, t: int) -> Shape:
    """This rank's share of heads, kv heads and FFN columns; hidden and vocab stay whole."""
    check_divides(s, t)
    return dataclasses.replace(s, n_heads=s.n_heads // t, n_kv_heads=s.n_kv_heads // t, ffn=s.ffn // t)


def shard_tensor(which: int, kind: int, rows: int, cols: int, arr: np.ndarray, rank: int, t: int):
    """-> (rows, cols, array) of rank's shard of one tensor; replicated tensors come back unchanged.
    Q4_K arrays are the raw bytes, [rows][cols/256][144] flattened."""
    if t == 1 or (which not in ROW_SPLIT and which not in COL_SPLIT):
        return rows, cols, arr
    if which in ROW_SPLIT:
        if rows % t:
            raise ValueError(f"tensor {which}: {rows} rows do not split over {t} ranks")
        r0, r1 = rank * rows // t, (rank + 1) * rows // t
        if kind == abi.K_Q4K:
            a = np.asarray(arr, np.uint8).reshape(rows, cols // 256 * 144)
        else:
            a = np.asarray(arr).reshape(rows, cols)
        return r1 - r0, cols, np.ascontiguousarray(a[r0:r1])
    if cols % t:
        raise ValueError(f"tensor {which}: {cols} columns do not split over {t} ranks")
    c0, c1 = rank * cols // t, (rank + 1) * cols // t
    if kind == abi.K_Q4K:
        if (cols // t) % 256:
            raise ValueError(f"tensor {which}: {cols // t} columns per rank are not whole Q4_K super-blocks")
        a = np.asarray(arr, np.uint8).reshape(rows, cols // 256, 144)
        return rows, c1 - c0, np.ascontiguousarray(a[:, c0 // 256:c1 // 256]).reshape(-1)
    a = np.asarray(arr).reshape(rows, cols)
    return rows, c1 - c0, np.ascontiguousarray(a[:, c0:c1])


def exchange_id(dist, make_id) -> bytes:
    """Rank 0 calls make_id() (128 bytes); every rank gets the bytes. `dist` is torch.distributed, initialised."""
    import torch
    buf = torch.zeros(NCCL_ID_BYTES, dtype=torch.uint8)
    if dist.get_rank() == 0:
        raw = make_id()
        if len(raw) != NCCL_ID_BYTES:
            raise ValueError("a communicator id is 128 bytes")
        buf = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()
    if dist.get_backend() == "nccl":
        buf = buf.cuda()
    dist.broadcast(buf, src=0)
    return bytes(buf.cpu().numpy().tobytes())


def max_over_ranks(dist, value: float) -> float:
    """The slowest rank's time: what a multi-GPU benchmark reports."""
    import torch
    t = torch.tensor([value], dtype=torch.float64)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.cpu()[0])


def replica_of(session: int, world: int) -> int:
    """Request-level placement over independent replicas: round-robin by arrival order."""
    return session % world


def sessions_of(rank: int, world: int, n_sessions: int) -> List[int]:
    return [i for i in range(n_sessions) if replica_of(i, world) == rank]


def open_rank(dist, device: int, stream: Optional[int] = None):
    """b200_open on this rank's GPU and b200_tp_init with the id rank 0 made. -> the driver object a Resident takes."""
    from .resident import ResidentError, _B200Driver
    drv = _B200Driver(device, stream)
    rank, size = dist.get_rank(), dist.get_world_size()

    def make_id():
        raw = (C.c_uint8 * NCCL_ID_BYTES)()
        st = drv.lib.b200_tp_unique_id(drv.ctx, raw, C.c_size_t(NCCL_ID_BYTES))
        if st != abi.OK:
            raise ResidentError(st, drv.last_error())
        return bytes(raw)

    uid = exchange_id(dist, make_id)
    st = drv.lib.b200_tp_init(drv.ctx, uid, C.c_size_t(NCCL_ID_BYTES), rank, size)
    if st != abi.OK:
        raise ResidentError(st, drv.last_error())
    return drv


def build_rank(dist, s: Shape, cfg_local: abi.ModelCfg, device: int, tensors: Optional[Iterable] = None, stream: Optional[int] = None):
    """One rank's resident shard. `cfg_local` is make_cfg(local_shape(s, t), ...) with tp_rank / tp_size set here;
    `tensors` yields full (which, layer, expert, kind, rows, cols, array) host tensors that this call shards, or None
    when the caller synthesizes the local tensors on the device itself. Returns the (unfinalized when tensors is None)
    Resident."""
    from .resident import Resident
    rank, size = dist.get_rank(), dist.get_world_size()
    cfg_local.tp_rank, cfg_local.tp_size = rank, size
    drv = open_rank(dist, device, stream)
    r = Resident(cfg_local, device=device, _driver=drv)
    if tensors is not None:
        for which, layer, expert, kind, rows, cols, arr in tensors:
            lr, lc, la = shard_tensor(which, kind, rows, cols, arr, rank, size)
            r.upload(which, la, layer, expert, kind, lr, lc)
        r.finalize()
    return r
