"""The benchmark configurations other than the headline one, as runnable workloads on one GPU.

  python -m goinfer_b200.workloads decode --shape c4-moe --batch 128 --ctx-lo 256 --ctx-hi 4096 --seed 3
  python -m goinfer_b200.workloads decode --shape c1-1.1b --batch 64 --ctx-lo 32 --ctx-hi 1280 --seed 1
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m goinfer_b200.workloads decode-tp --shape c5-70b
  python -m goinfer_b200.workloads serve  --shape c1-1.1b --sessions 512 --rate 40 --max-active 64 --seed 1

`decode` pre-fills every slot's paged KV with synthetic rows at the drawn context lengths and times resident greedy
decode steps (device loop, CUDA events); `serve` runs the continuous-batching driver of goinfer_b200.serve over a Poisson
arrival trace. Weights are synthesized on the device (N(0, 0.02) quantized to Q4_K). Each prints one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import time

import numpy as np


def decode(shape: str, batch: int, ctx_lo: int, ctx_hi: int, seed: int, steps: int, warmup: int, device: int = 0,
           n_layers: int = 0, breakdown: bool = True) -> dict:
    from . import abi, synth
    from .resident import Resident

    s = synth.SHAPES[shape]
    ctx = np.random.default_rng(seed).integers(ctx_lo, ctx_hi + 1, batch).astype(np.int32)
    growth = steps + warmup + 8
    cap = int(ctx.max()) + growth
    blocks = 1 + int(np.ceil((ctx + growth) / 16).sum())
    cfg = synth.make_cfg(s, batch, cap, 16, blocks, batch, abi.CLASS_AUTO, n_layers)
    r = Resident(cfg, device=device)
    synth.load_device_weights(r, s, seed=seed, n_layers=n_layers)
    caps = r.finalize()
    for i in range(batch):
        r.SynthKV(i, int(ctx[i]), 0.5, 1000 + i)
    lib, m, bctx = r.drv.lib, r.m, r.drv.ctx
    p32 = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    slot = np.arange(batch, dtype=np.int32)
    pos = ctx.copy()
    first = np.random.default_rng(seed + 1).integers(0, s.vocab, batch).astype(np.int32)
    ms = C.c_float(0)

    def check(st):
        if st != abi.OK:
            raise RuntimeError(f"b200 status {st}: {r.drv.last_error()}")

    if warmup:
        check(lib.b200_decode_loop_device(m, batch, p32(slot), p32(pos), p32(first), warmup, 1, None, C.byref(ms)))
        pos += warmup
    l0 = lib.b200_launch_count(bctx)
    check(lib.b200_decode_loop_device(m, batch, p32(slot), p32(pos), p32(first), steps, 1, None, C.byref(ms)))
    launches = int(lib.b200_launch_count(bctx) - l0)
    dev_ms = float(ms.value)
    keys = float(np.mean([(pos + 1 + i).sum() for i in range(steps)]))
    pos += steps
    L = n_layers or s.n_layers
    out = {"workload": f"{shape}: B={batch} ragged decode, contexts U[{ctx_lo},{ctx_hi}] seed {seed}, paged fp16 KV 16-token blocks",
           "layers": L, "steps": steps, "warmup": warmup, "ms_per_step": dev_ms / steps, "tok_s": batch * steps / (dev_ms * 1e-3),
           "gpu_launches": launches, "kv_bytes_per_step": keys * 2 * s.n_kv_heads * s.head_dim * 2 * L,
           "memory": {"weights_gb": caps.weight_bytes / 1e9, "kv_gb": caps.kv_bytes / 1e9, "scratch_gb": caps.scratch_bytes / 1e9}}
    out["hbm_floor_ms"] = (out["kv_bytes_per_step"] + caps.weight_bytes) / 6540.5e9 * 1e3
    if breakdown:
        tag_ms = (C.c_double * 8)()
        tag_n = (C.c_int64 * 8)()
        lib.b200_profile(bctx, 0xFF)
        check(lib.b200_decode_loop_device(m, batch, p32(slot), p32(pos), p32(first), 2, 1, None, C.byref(ms)))
        lib.b200_profile_read(bctx, tag_ms, tag_n, 8)
        lib.b200_profile(bctx, 0)
        names = ("attn_split", "attn_combine", "q4k_matmul", "head_matmul", "norm_quant", "rope_kvstore", "swiglu_quant", "other")
        out["breakdown_ms_per_step"] = {n: round(tag_ms[i] / 2, 4) for i, n in enumerate(names) if tag_n[i]}
    r.Close()
    return out


def decode_tp(shape: str, batch: int, ctx_lo: int, ctx_hi: int, seed: int, steps: int, warmup: int, n_layers: int = 0,
              kv_budget_gb: float = 0.0) -> dict:
    """Tensor-parallel decode: run under torch.distributed.run, one process per GPU. The batch is cut to the first
    sequences whose paged KV fits the ranks' memory (the 70B-class configuration's full batch does not fit 8 GPUs);
    the cut is reported. Rank 0 returns the result, the others None. A process group the caller already initialised
    (gloo or nccl) is used as it is and left open; otherwise a gloo group is made for the length of the call."""
    import os
    import torch
    import torch.distributed as dist
    from . import abi, synth, tp

    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("gloo")
    on_gpu = dist.get_backend() == "nccl"
    rank, world, dev = dist.get_rank(), dist.get_world_size(), int(os.environ.get("LOCAL_RANK", "0"))
    s = synth.SHAPES[shape]
    sl = tp.local_shape(s, world)
    L = n_layers or s.n_layers
    ctx_all = np.random.default_rng(seed).integers(ctx_lo, ctx_hi + 1, batch).astype(np.int32)
    growth = steps + warmup + 8
    per_pos = 2 * sl.n_kv_heads * s.head_dim * 2 * L                       # this rank's KV bytes per position, all layers
    w_bytes = L * (s.hidden * (sl.n_heads + 2 * sl.n_kv_heads) * s.head_dim + s.hidden * sl.n_heads * s.head_dim
                       + 3 * s.hidden * sl.ffn) * 144 / 256 + (s.vocab + s.vocab // world) * s.hidden * 2
    budget = (kv_budget_gb * 1e9) if kv_budget_gb > 0 else (178e9 - w_bytes - 6e9)
    # what is really free on the ranks' GPUs (a parent process may hold a context): the smallest figure decides for all
    free = torch.tensor([float(torch.cuda.mem_get_info(dev)[0])], dtype=torch.float64, device=("cuda:%d" % dev) if on_gpu else "cpu")
    dist.all_reduce(free, op=dist.ReduceOp.MIN)
    if kv_budget_gb <= 0:
        budget = min(budget, float(free.cpu()[0]) - w_bytes - 6e9)
    need = np.cumsum((np.ceil((ctx_all + growth) / 16) * 16) * per_pos)
    b_fit = int(np.searchsorted(need, budget, side="right"))
    b_fit = max(2, min(batch, b_fit))
    ctx = ctx_all[:b_fit]
    cap = int(ctx.max()) + growth
    blocks = 1 + int(np.ceil((ctx + growth) / 16).sum())
    cfg = synth.make_cfg(sl, b_fit, cap, 16, blocks, b_fit, abi.CLASS_AUTO, n_layers)
    r = tp.build_rank(dist, s, cfg, dev, None)
    synth.load_device_weights(r, sl, seed=seed * 131 + rank, n_layers=n_layers, head_rows=s.vocab // world)
    caps = r.finalize()
    for i in range(b_fit):
        r.SynthKV(i, int(ctx[i]), 0.5, 1000 + i)
    lib, m, bctx = r.drv.lib, r.m, r.drv.ctx
    p32 = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    slot = np.arange(b_fit, dtype=np.int32)
    pos = ctx.copy()
    first = np.random.default_rng(seed + 1).integers(0, s.vocab, b_fit).astype(np.int32)
    ms = C.c_float(0)

    def check(st):
        if st != abi.OK:
            raise RuntimeError(f"b200 status {st}: {r.drv.last_error()}")

    dist.barrier()
    if warmup:
        check(lib.b200_decode_loop_device(m, b_fit, p32(slot), p32(pos), p32(first), warmup, 1, None, C.byref(ms)))
        pos += warmup
    dist.barrier()
    ids = np.zeros(steps * b_fit, np.int32)
    l0 = lib.b200_launch_count(bctx)
    check(lib.b200_decode_loop_device(m, b_fit, p32(slot), p32(pos), p32(first), steps, 1, p32(ids), C.byref(ms)))
    launches = int(lib.b200_launch_count(bctx) - l0)
    dev_ms = tp.max_over_ranks(dist, float(ms.value))
    # every rank drew the same ids (the logits were gathered, the draw is replicated)
    mine = torch.from_numpy(ids.copy())
    if on_gpu:
        mine = mine.cuda()
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    flag = torch.tensor([1 if bool((mine == ref).all()) else 0], device=mine.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    same = bool(flag.cpu()[0] == 1)
    keys = float(np.mean([(pos + 1 + i).sum() for i in range(steps)]))
    pos += steps
    tag_ms = (C.c_double * 8)()
    tag_n = (C.c_int64 * 8)()
    lib.b200_profile(bctx, 0xFF)
    check(lib.b200_decode_loop_device(m, b_fit, p32(slot), p32(pos), p32(first), 2, 1, None, C.byref(ms)))
    lib.b200_profile_read(bctx, tag_ms, tag_n, 8)
    lib.b200_profile(bctx, 0)
    alone_us = None
    if lib.b200_tp_fused_active(m):   # the cross-rank kernel by itself, launches back to back on every rank at once
        one, stages = C.c_float(), (C.c_float * 4)()
        dist.barrier()
        check(lib.b200_bench_tp_reduce(m, b_fit, 0, 5, 50, C.byref(one), stages))
        alone_us = {"per_launch": one.value * 1e3, "first_cta": {"push": stages[0], "wait_and_reduce": stages[1], "stores_done_or_rearm": stages[2], "wait_for_peers": stages[3]},
                    "form": "flags and fences" if os.environ.get("B200_TP_FLAGS") else "words that announce themselves"}
    names = ("attn_split", "attn_combine", "q4k_matmul", "head_matmul", "norm_quant", "rope_kvstore", "swiglu_quant", "collectives")
    out = None
    if rank == 0:
        out = {"workload": f"{shape}: tensor parallel x{world}, B={b_fit} of {batch} (the sequences whose KV fits), contexts "
                           f"U[{ctx_lo},{ctx_hi}] seed {seed}, paged fp16 KV 16-token blocks",
               "tp": world, "layers": L, "batch": b_fit, "batch_asked": batch, "steps": steps, "warmup": warmup,
               "ms_per_step": dev_ms / steps, "tok_s": b_fit * steps / (dev_ms * 1e-3), "gpu_launches_per_rank": launches,
               "ranks_drew_the_same_ids": same, "kv_bytes_per_step_per_rank": keys * per_pos,
               "cross_rank_sum_bytes_per_step": 2 * L * b_fit * s.hidden * 4,
               "memory_per_rank": {"weights_gb": caps.weight_bytes / 1e9, "kv_gb": caps.kv_bytes / 1e9, "scratch_gb": caps.scratch_bytes / 1e9},
               "hbm_floor_ms": (keys * per_pos + caps.weight_bytes) / 6540.5e9 * 1e3,
               "nvls": os.environ.get("NCCL_NVLS_ENABLE", "library default"),
               "cross_rank_sum": ("one kernel over peer memory: sum of the ranks' partial rows + residual + RMSNorm + per-32 quantizer, rows/t per rank, "
                                  "codes stored to every rank" if lib.b200_tp_fused_active(m) else "ncclAllReduce (f32) + the norm kernel on every rank"),
               "cross_rank_sum_us_alone": alone_us,
               "breakdown_ms_per_step_rank0": {n: round(tag_ms[i] / 2, 4) for i, n in enumerate(names) if tag_n[i]}}
    dist.barrier()
    r.Close()
    r.drv.close()
    if own_group:
        dist.destroy_process_group()
    return out


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    d = sub.add_parser("decode")
    d.add_argument("--shape", default="c4-moe")
    d.add_argument("--batch", type=int, default=128)
    d.add_argument("--ctx-lo", type=int, default=256)
    d.add_argument("--ctx-hi", type=int, default=4096)
    d.add_argument("--seed", type=int, default=3)
    d.add_argument("--steps", type=int, default=8)
    d.add_argument("--warmup", type=int, default=3)
    d.add_argument("--layers", type=int, default=0)
    t = sub.add_parser("decode-tp")
    t.add_argument("--shape", default="c5-70b")
    t.add_argument("--batch", type=int, default=256)
    t.add_argument("--ctx-lo", type=int, default=1024)
    t.add_argument("--ctx-hi", type=int, default=32768)
    t.add_argument("--seed", type=int, default=4)
    t.add_argument("--steps", type=int, default=4)
    t.add_argument("--warmup", type=int, default=2)
    t.add_argument("--layers", type=int, default=0)
    t.add_argument("--kv-budget-gb", type=float, default=0.0)
    v = sub.add_parser("serve")
    v.add_argument("--shape", default="c1-1.1b")
    v.add_argument("--sessions", type=int, default=512)
    v.add_argument("--rate", type=float, default=40.0)
    v.add_argument("--max-active", type=int, default=64)
    v.add_argument("--seed", type=int, default=1)
    v.add_argument("--prompt-lo", type=int, default=32)
    v.add_argument("--prompt-hi", type=int, default=1024)
    v.add_argument("--out-lo", type=int, default=16)
    v.add_argument("--out-hi", type=int, default=256)
    v.add_argument("--chunk", type=int, default=512)
    v.add_argument("--layers", type=int, default=0)
    v.add_argument("--time-scale", type=float, default=1.0, help="arrival times are divided by this (1 = real time)")
    v.add_argument("--preamble", type=int, default=0, help="leading tokens every prompt shares with one of --n-preambles runs")
    v.add_argument("--n-preambles", type=int, default=1)
    v.add_argument("--prefix-reuse", action="store_true", help="serve shared prefixes from the slots that hold them (CopyKV)")
    v.add_argument("--device-batch", type=int, default=0, help="k > 0: decode on the device batch, k steps a run (admission and retirement on the device)")
    args = ap.parse_args()
    if args.what == "decode":
        print(json.dumps(decode(args.shape, args.batch, args.ctx_lo, args.ctx_hi, args.seed, args.steps, args.warmup,
                                n_layers=args.layers)))
    elif args.what == "decode-tp":
        res = decode_tp(args.shape, args.batch, args.ctx_lo, args.ctx_hi, args.seed, args.steps, args.warmup, args.layers,
                        args.kv_budget_gb)
        if res is not None:
            print(json.dumps(res))
    else:
        from .serve import run_poisson
        print(json.dumps(run_poisson(args.shape, args.sessions, args.rate, args.max_active, args.seed, args.prompt_lo,
                                     args.prompt_hi, args.out_lo, args.out_hi, args.chunk, n_layers=args.layers,
                                     time_scale=args.time_scale, preamble=args.preamble, n_preambles=args.n_preambles,
                                     prefix_reuse=args.prefix_reuse, device_batch=args.device_batch)))


if __name__ == "__main__":
    main()
