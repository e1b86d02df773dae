"""Host side of the multi-GPU paths on CPU: tensor-parallel sharding (the shards' partial products add up to the whole
layer), and, as two gloo ranks, the communicator-id exchange, an all-reduced split layer, replica placement and the
max-over-ranks reduction."""
import os
import socket

import numpy as np
import pytest

from goinfer_b200 import abi, q4k, synth, tp


def test_local_shape_and_divisibility():
    s = synth.SHAPES["c5-70b"]
    for t in (2, 4, 8):
        l = tp.local_shape(s, t)
        assert (l.n_heads, l.n_kv_heads, l.ffn, l.vocab, l.hidden) == (64 // t, 8 // t, 28672 // t, s.vocab, s.hidden)
        assert (l.n_heads * l.head_dim) % 256 == 0 and l.ffn % 256 == 0
    with pytest.raises(ValueError):
        tp.local_shape(s, 16)                      # 8 kv heads do not split over 16 ranks
    with pytest.raises(ValueError):
        tp.local_shape(synth.SHAPES["tiny-dense"], 2)   # 256 o-proj columns would leave half a super-block per rank
    with pytest.raises(ValueError):
        tp.local_shape(synth.SHAPES["c4-moe"], 2)
    assert tp.local_shape(synth.SHAPES["tiny-tp"], 2).ffn == 512


def test_shards_add_up_to_the_layer():
    rng = np.random.default_rng(0)
    H, F, t = 512, 1024, 2
    x = rng.normal(0, 1, (3, H))
    mid = rng.normal(0, 1, (3, F))
    w_up = q4k.quantize(rng.normal(0, 0.02, (F, H)).astype(np.float32))
    w_down = q4k.quantize(rng.normal(0, 0.02, (H, F)).astype(np.float32))
    full_up = x @ q4k.dequantize(w_up, F, H).astype(np.float64).T
    full_down = mid @ q4k.dequantize(w_down, H, F).astype(np.float64).T
    ups, downs = [], 0
    for r in range(t):
        rows, cols, a = tp.shard_tensor(abi.T_UP, abi.K_Q4K, F, H, w_up, r, t)
        assert (rows, cols) == (F // t, H) and a.size == rows * cols // 256 * 144
        ups.append(x @ q4k.dequantize(a, rows, cols).astype(np.float64).T)
        rows, cols, a = tp.shard_tensor(abi.T_DOWN, abi.K_Q4K, H, F, w_down, r, t)
        assert (rows, cols) == (H, F // t)
        downs = downs + mid[:, r * F // t:(r + 1) * F // t] @ q4k.dequantize(a, rows, cols).astype(np.float64).T
    np.testing.assert_array_equal(np.concatenate(ups, axis=1), full_up)       # a row split only regroups outputs
    np.testing.assert_allclose(downs, full_down, rtol=1e-12, atol=1e-12)      # a column split regroups one sum
    # f16 head: vocabulary slices; norms are replicated
    head = rng.normal(0, 0.02, (64, H)).astype(np.float16)
    rows, cols, a = tp.shard_tensor(abi.T_LM_HEAD, abi.K_F16, 64, H, head, 1, 2)
    assert (rows, cols) == (32, H) and np.array_equal(a, head[32:])
    nrm = np.ones(H, np.float32)
    assert tp.shard_tensor(abi.T_ATTN_NORM, abi.K_F32, 1, H, nrm, 1, 2)[2] is nrm
    with pytest.raises(ValueError):
        tp.shard_tensor(abi.T_DOWN, abi.K_Q4K, H, 768, np.zeros(H * 3 * 144, np.uint8), 0, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the communicator id: made on rank 0 only, the same 128 bytes everywhere
        made = []
        def make_id():
            made.append(1)
            return bytes(range(128))
        uid = tp.exchange_id(dist, make_id)
        assert uid == bytes(range(128)) and len(made) == (1 if rank == 0 else 0)
        # a column-split projection: each rank's partial product, summed across ranks, is the whole one
        rng = np.random.default_rng(5)
        H, F = 256, 512
        mid = rng.normal(0, 1, (4, F))
        w = q4k.quantize(rng.normal(0, 0.02, (H, F)).astype(np.float32))
        rows, cols, a = tp.shard_tensor(abi.T_DOWN, abi.K_Q4K, H, F, w, rank, world)
        part = torch.from_numpy(mid[:, rank * cols:(rank + 1) * cols] @ q4k.dequantize(a, rows, cols).astype(np.float64).T)
        dist.all_reduce(part)
        np.testing.assert_allclose(part.numpy(), mid @ q4k.dequantize(w, H, F).astype(np.float64).T, rtol=1e-12, atol=1e-12)
        # a row-split head: the gathered slices are the whole logits row
        head = rng.normal(0, 0.02, (64, H)).astype(np.float16)
        x = rng.normal(0, 1, (2, H))
        rows, cols, a = tp.shard_tensor(abi.T_LM_HEAD, abi.K_F16, 64, H, head, rank, world)
        loc = torch.from_numpy(x @ a.astype(np.float64).T)
        parts = [torch.zeros_like(loc) for _ in range(world)]
        dist.all_gather(parts, loc)
        np.testing.assert_array_equal(torch.cat(parts, dim=1).numpy(), x @ head.astype(np.float64).T)
        # replicas: every session on exactly one rank; the reported time is the slowest rank's
        mine = tp.sessions_of(rank, world, 11)
        cnt = torch.zeros(11, dtype=torch.int64)
        cnt[mine] = 1
        dist.all_reduce(cnt)
        assert bool((cnt == 1).all()) and mine == list(range(rank, 11, world))
        assert tp.max_over_ranks(dist, 1.0 + rank) == float(world)
        out.put((rank, "ok"))
    except Exception as e:  # surfaces in the parent
        out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, "ok"), (1, "ok")], res
