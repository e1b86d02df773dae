#!/usr/bin/env python
"""Benchmark of the ragged batched decode step on B200.

Workload (BASELINE configuration 3, the one the headline metric is quoted on): dense 8B shape (hidden 4096, 36 layers,
32 query / 8 KV heads of 128, per-head QK RMSNorm, SwiGLU 12288, vocab 151936, RoPE theta 1e6), random-init N(0, 0.02)
weights quantized to Q4_K with per-32 int8 activations, f16 embedding and LM head; a ragged batch of 256 sequences with
prefix contexts uniform in [128, 8192] (seed 2) held in a paged fp16 KV cache of 16-token blocks (about 160 GB, so every
step streams far more than the 126 MB L2); one step = one greedy decode token for every sequence.

  python bench.py --gpus N --steps K --warmup W          this build (one replica per GPU, no collective)
  python bench.py --impl reference --steps K --warmup W  the CPU restatement of the reference path on the host cores

One JSON line on stdout (rank 0). `value` is tok/s with everything resident in HBM and the drawn ids fed back on the
device; `e2e` is the same metric through the C ABI's step call with host buffers (embedding rows in, ids out, every step).
Beside them, on one GPU: `parity` (the timed kernel class against the CPU oracle on a 256-sequence step of this shape),
`exact_class` (the same workload in the exact kernel class), `c4` and `c1` (the routed-expert and the 1.1B-shape decode
configurations), `c2_serve` (a small serve trace through the host-driven driver and the device batch), the Q4_K small-batch
matmul sweep and the CPU baseline; on N >= 2 GPUs, after the replica legs, `tp_c5`: the 70B-class shape tensor-parallel
over the N ranks.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "ragged-batch decode tok/s (Q4_K, 8B shape, B=256)"
B, CTX_LO, CTX_HI, SEED = 256, 128, 8192, 2
SAMPLE_SEQS, SAMPLE_LAYERS = 32, 2
PF_ROWS, PF_DEEP = 2048, 4096      # the workload's prefill chunk: rows, and how deep into a context its second run starts


def contexts():
    return np.random.default_rng(SEED).integers(CTX_LO, CTX_HI + 1, B).astype(np.int32)


def workload_config(n_gpus):
    return {"workload": "c3: 8B-shape Q4_K (W4A8 per-32), B=256 ragged decode, contexts U[128,8192] seed 2, paged fp16 KV "
                        "16-token blocks", "global_batch": B * n_gpus, "parallelism": f"replicas x{n_gpus} (no collective)",
            "l2": "inputs (about 160 GB of KV and 6.4 GB of weights per step) are far larger than the 126 MB L2",
            "kernel_class": "fast (tensor-core flash-decode attention, fp32 softmax and accumulate)"}


# ---------------------------------------------------------------------------------------------------------------------
def cpu_sample(steps, warmup):
    """The oracle (CPU restatement of the reference's decodeMultiStep) on a bounded sample of the workload: the first
    SAMPLE_SEQS sequences of the batch at their drawn contexts, SAMPLE_LAYERS of the 36 layers plus the full LM head.
    Layer time is scaled by 36/SAMPLE_LAYERS and the batch by B/SAMPLE_SEQS (CPU cost is linear in both)."""
    from goinfer_b200 import abi, q4k, synth
    from oracle import binding as ob
    ob.use_all_cores()   # a launcher's OMP_NUM_THREADS=1 would otherwise leave the CPU arm on one core
    s = synth.SHAPES["c3-8b"]
    ctx = contexts()[:SAMPLE_SEQS]
    cap = int(ctx.max()) + warmup + steps + 2
    cfg = synth.make_cfg(s, SAMPLE_SEQS, cap, 16, 0, SAMPLE_SEQS, abi.CLASS_EXACT, SAMPLE_LAYERS)
    o = ob.OracleResident(cfg)
    rng = np.random.default_rng(7)
    H, qd, kvd = s.hidden, s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
    tile = rng.normal(0, 0.02, (1024, H)).astype(np.float16)
    table = np.ascontiguousarray(np.tile(tile, (s.vocab // 1024 + 1, 1))[:s.vocab])
    o.upload(abi.T_EMBED, table)
    o.upload(abi.T_LM_HEAD, table)
    o.upload(abi.T_FINAL_NORM, np.ones(H, np.float32))
    for l in range(SAMPLE_LAYERS):
        o.upload(abi.T_ATTN_NORM, np.ones(H, np.float32), l)
        o.upload(abi.T_FFN_NORM, np.ones(H, np.float32), l)
        o.upload(abi.T_Q_NORM, np.ones(s.head_dim, np.float32), l)
        o.upload(abi.T_K_NORM, np.ones(s.head_dim, np.float32), l)
        for which, rows, cols in ((abi.T_WQ, qd, H), (abi.T_WK, kvd, H), (abi.T_WV, kvd, H), (abi.T_WO, H, qd),
                                  (abi.T_GATE, s.ffn, H), (abi.T_UP, s.ffn, H), (abi.T_DOWN, H, s.ffn)):
            # random valid blocks (how the reference's own tests build Q4_K tensors); values do not matter for time
            o.upload(which, q4k.random_blocks(rng, rows, cols, 1, 4), l, -1, abi.K_Q4K, rows, cols)
    o.finalize()
    kv = rng.normal(0, 0.5, (int(ctx.max()), kvd)).astype(np.float32)
    for i, n in enumerate(ctx):
        for l in range(SAMPLE_LAYERS):
            o.UploadKV(i, l, 0, kv[:n], kv[:n])
    lay, head = C.c_double(0), C.c_double(0)
    from goinfer_b200.resident import BatchDraw, BatchSeq
    toks = rng.integers(0, s.vocab, SAMPLE_SEQS).tolist()
    times = []
    for it in range(warmup + steps):
        seqs = [BatchSeq(i, int(ctx[i]) + it, None, toks[i], BatchDraw(Greedy=True)) for i in range(SAMPLE_SEQS)]
        toks = [x.ID for x in o.StepBatch(seqs)]
        ob.lib().oracle_last_timing(C.byref(lay), C.byref(head))
        if it >= warmup:
            times.append((lay.value, head.value))
    lay_s = float(np.mean([t[0] for t in times]))
    head_s = float(np.mean([t[1] for t in times]))
    full_step_s = (B / SAMPLE_SEQS) * (lay_s * s.n_layers / SAMPLE_LAYERS + head_s)
    return {"value": B / full_step_s, "unit": "tok/s", "cores": ob.threads(), "kind": "port",
            "sample": f"{SAMPLE_SEQS} of the {B} sequences at their drawn contexts, {SAMPLE_LAYERS} of 36 layers + the LM head; "
                      f"measured {lay_s:.3f} s layers + {head_s:.3f} s head per sample step, scaled by 36/{SAMPLE_LAYERS} and "
                      f"{B}/{SAMPLE_SEQS}; CPU restatement of goinfer's CPU path (its Go binary and aikit kernels cannot be built here)",
            "ms_per_step": full_step_s * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_sample(args.steps, args.warmup)
    line = {"metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x Q4_K integer dots, f32/f64 accumulate", "data": "synthetic",
            "config": workload_config(args.gpus), "impl": "reference",
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.p, self.path = gpu_index, None, f"/tmp/clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken between the two wall-clock times (the timed region)."""
        if not self.p:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        self.p.wait()
        import datetime
        sm, mx, pw, reasons = [], [], [], set()
        for ln in open(self.path):
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if t_begin is not None and not (t_begin - 0.05 <= ts <= t_end + 0.05):
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}



def parity_leg(device):
    """The kernel class the benchmark times against the CPU oracle: one StepBatch of 256 sequences of this shape (2 of the 36
    layers, the head cut to 32768 rows, contexts U[96,320] uploaded to both sides, host-built N(0,0.02) weights quantized to
    Q4_K given to both), i.e. the tcgen05 matmuls, the fused SwiGLU epilogue, the tensor-core flash-decode and the tcgen05
    head exactly as the timed step runs them."""
    from goinfer_b200 import abi, synth
    from oracle import binding as ob, parity
    ob.use_all_cores()
    m = parity.decode_step_parity(synth.SHAPES["c3-8b"], 2, B, 96, 320, abi.CLASS_AUTO, seed=SEED, vocab=32768, device=device)
    m["sample"] = ("one StepBatch of 256 sequences, 2 of 36 layers, head cut to 32768 rows, contexts U[96,320], fast class vs the "
                   "CPU oracle; bar = 2e-2 + 1e-2*|oracle| per logit; near tie = the oracle's two logits within 4e-2")
    return m


def exact_class_leg(device, stream, steps=3, warmup=1):
    """The headline workload in the exact kernel class (f64 attention in the CPU path's order, one ascending f32 chain per
    matmul output): the class whose logits stay inside the build's bar at every depth."""
    import torch
    from goinfer_b200 import abi, synth
    from goinfer_b200.resident import Resident
    s = synth.SHAPES["c3-8b"]
    ctx = contexts()
    growth = steps + warmup + 4
    cap = int(ctx.max()) + growth
    blocks = 1 + int(np.ceil((ctx + growth) / 16).sum())
    cfg = synth.make_cfg(s, B, cap, 16, blocks, B, abi.CLASS_EXACT)
    with torch.cuda.stream(stream):
        r = Resident(cfg, device=device, stream=stream.cuda_stream)
        synth.load_device_weights(r, s, seed=SEED)
        r.finalize()
        for i in range(B):
            r.SynthKV(i, int(ctx[i]), 0.5, 1000 + i)
        first = np.random.default_rng(SEED + 1).integers(0, s.vocab, B).astype(np.int32)
        pos = ctx.copy()
        if warmup:
            r.DecodeLoop(range(B), pos, first, warmup, log_ids=False)
            pos += warmup
        _, ms = r.DecodeLoop(range(B), pos, first, steps, log_ids=False)
        pos += steps
        lib, bctx = r.drv.lib, r.drv.ctx
        tag_ms, tag_n = (C.c_double * 8)(), (C.c_int64 * 8)()
        lib.b200_profile(bctx, 0xFF)
        r.DecodeLoop(range(B), pos, first, 1, log_ids=False)
        lib.b200_profile_read(bctx, tag_ms, tag_n, 8)
        lib.b200_profile(bctx, 0)
        names = ("attn_scores", "attn_softmax", "q4k_matmul", "head_matmul", "norm_quant", "rope_kvstore", "swiglu_quant", "attn_av")
        r.Close()
        r.drv.close()
    return {"ms_per_step": ms / steps, "tok_s": B * steps / (ms * 1e-3), "steps": steps, "warmup": warmup,
            "kernel_class": "exact (f64 attention, one-chain Q4_K matmuls)",
            "breakdown_ms_per_step": {n: round(tag_ms[i], 3) for i, n in enumerate(names) if tag_n[i]}}


def run_gpu(args):
    import torch
    from goinfer_b200 import abi, synth
    from goinfer_b200.resident import Resident

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()
    K, W = args.steps, max(args.warmup, 0)
    extra = {}
    if world == 1 and not args.no_cpu:
        extra["parity"] = parity_leg(local)   # small models of its own, freed before the workload's 160 GB of KV are laid out
    s = synth.SHAPES["c3-8b"]
    ctx = contexts()
    growth = 2 * (K + W) + 12                      # positions each sequence may advance over the timed loops
    cap = int(ctx.max()) + growth
    # one more slot takes the 2048-row prefill chunk (at position 0, and again 4096 rows deep into a context)
    blocks = 1 + int(np.ceil((ctx + growth) / 16).sum()) + (PF_DEEP + PF_ROWS) // 16 + 2
    cfg = synth.make_cfg(s, B + 1, cap, 16, blocks, max(B, PF_ROWS), abi.CLASS_AUTO)
    with torch.cuda.stream(stream):
        r = Resident(cfg, device=local, stream=stream.cuda_stream)
        synth.load_device_weights(r, s, seed=SEED)
        caps = r.finalize()
        for i in range(B):
            r.SynthKV(i, int(ctx[i]), 0.5, 1000 + i)
        lib, m, bctx = r.drv.lib, r.m, r.drv.ctx
        slot = np.arange(B, dtype=np.int32)
        pos = ctx.copy()
        first = np.random.default_rng(SEED + 1).integers(0, s.vocab, B).astype(np.int32)
        ms = C.c_float(0)
        p32 = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))

        def check(st):
            if st != abi.OK:
                raise RuntimeError(f"b200 status {st}: {r.drv.last_error()}")

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                import torch.distributed as dist
                dist.barrier()
            torch.cuda.synchronize()

        # ---- resident leg: `value` ----
        clocks = Clocks(local)
        clocks.start()
        if W:
            check(lib.b200_decode_loop_device(m, B, p32(slot), p32(pos), p32(first), W, 1, None, C.byref(ms)))
            pos += W
        lib.b200_profile(bctx, 1)                   # per-launch events on the attention split kernel only
        barrier()
        wall0 = time.time()
        launches0 = lib.b200_launch_count(bctx)
        check(lib.b200_decode_loop_device(m, B, p32(slot), p32(pos), p32(first), K, 1, None, C.byref(ms)))
        barrier()
        wall1 = time.time()
        launches = int(lib.b200_launch_count(bctx) - launches0)
        dev_ms = float(ms.value)
        tag_ms = (C.c_double * 8)()
        tag_n = (C.c_int64 * 8)()
        lib.b200_profile_read(bctx, tag_ms, tag_n, 8)
        lib.b200_profile(bctx, 0)
        keys_per_step = [float((pos + 1 + i).sum()) for i in range(K)]      # keys read per layer at timed step i
        pos += K
        attn_bytes_per_launch = float(np.mean(keys_per_step)) * 2 * s.n_kv_heads * s.head_dim * 2
        attn_ms_total, attn_launches = float(tag_ms[0]), int(tag_n[0])
        attn_ms_per_launch = attn_ms_total / max(1, attn_launches)

        # ---- end-to-end leg: the C ABI step call with host buffers, H2D and D2H inside the timed region ----
        embs = torch.empty((B, s.hidden), dtype=torch.float32).normal_(0, 0.02).pin_memory()
        e_np = embs.numpy()
        ones = np.ones(B, np.int32)
        draws = (abi.Draw * B)(*[abi.Draw(abi.DRAW_GREEDY, 0, 0, 0, 0)] * B)
        ids = np.zeros(B, np.int32)

        def step_host():
            check(lib.b200_step_ragged(m, B, p32(slot), p32(pos), p32(ones), None, None,
                                       e_np.ctypes.data_as(C.POINTER(C.c_float)), None, draws, None, None, 0, None, p32(ids), None))
            pos[:] += 1

        for _ in range(min(W, 3)):
            step_host()
        barrier()
        t0 = time.perf_counter()
        for _ in range(K):
            step_host()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        clk = clocks.stop(wall0, wall1)

        # ---- per-class breakdown of one more resident step (every kernel class bracketed by events; not part of `value`) ----
        lib.b200_profile(bctx, 0xFF)
        check(lib.b200_decode_loop_device(m, B, p32(slot), p32(pos), p32(first), 2, 1, None, C.byref(ms)))
        pos += 2
        lib.b200_profile_read(bctx, tag_ms, tag_n, 8)
        lib.b200_profile(bctx, 0)
        names = ("attn_split", "attn_combine", "q4k_matmul", "head_matmul", "norm_quant", "rope_kvstore", "swiglu_quant", "other")
        breakdown = {n: {"ms_per_step": tag_ms[i] / 2, "launches_per_step": int(tag_n[i] // 2)} for i, n in enumerate(names) if tag_n[i]}
        breakdown["step_ms_with_events"] = float(ms.value) / 2

        # ---- the workload's prefill chunk: PF_ROWS prompt rows of one sequence in one ragged step (device embedding gather,
        # last row's logits read back), at position 0 and PF_DEEP rows into a context; device time by events on the stream ----
        prefill = []
        pf_tok = np.random.default_rng(SEED + 2).integers(0, s.vocab, PF_ROWS).astype(np.int32)
        pf_logits = np.zeros(s.vocab, np.float32)
        one = lambda v: np.array([v], np.int32)
        for pos0 in (0, PF_DEEP):
            best = None
            for rep in range(3):
                check(lib.b200_reset_slot(m, B))
                if pos0:
                    r.SynthKV(B, pos0, 0.5, 77)
                if rep == 2:
                    lib.b200_profile(bctx, 0xFF)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                e0.record(stream)
                check(lib.b200_step_ragged(m, 1, p32(one(B)), p32(one(pos0)), p32(one(PF_ROWS)), p32(one(pos0 + PF_ROWS)),
                                           np.array([1], np.uint8).ctypes.data_as(C.POINTER(C.c_uint8)), None, p32(pf_tok), None,
                                           None, None, 0, pf_logits.ctypes.data_as(C.POINTER(C.c_float)), None, None))
                e1.record(stream)
                torch.cuda.synchronize()
                wall_ms = (time.perf_counter() - t0) * 1e3
                if rep == 2:
                    lib.b200_profile_read(bctx, tag_ms, tag_n, 8)
                    lib.b200_profile(bctx, 0)
                    pf_break = {n: {"ms": tag_ms[i], "launches": int(tag_n[i])} for i, n in enumerate(names) if tag_n[i]}
                else:
                    dms = e0.elapsed_time(e1)
                    best = (dms, wall_ms) if best is None or dms < best[0] else best
            lin_flop = 2.0 * PF_ROWS * 36 * (4096 * 6144 + 4096 * 4096 + 3 * 4096 * 12288)
            att_flop = 4.0 * (PF_ROWS * pos0 + PF_ROWS * (PF_ROWS + 1) / 2) * s.n_heads * s.head_dim * 36
            prefill.append({"rows": PF_ROWS, "pos0": pos0, "ms": best[0], "tok_s": PF_ROWS / best[0] * 1e3, "e2e_ms": best[1],
                            "linear_tflops": lin_flop / best[0] / 1e9, "attention_tflops": att_flop / best[0] / 1e9,
                            "finite_logits": bool(np.isfinite(pf_logits).all()), "breakdown_with_events": pf_break})
        r.Close()
        r.drv.close()

    if world == 1 and not args.no_extra:
        from goinfer_b200 import workloads
        extra["exact_class"] = exact_class_leg(local, stream)
        extra["c4"] = workloads.decode("c4-moe", 128, 256, 4096, 3, steps=4, warmup=2, device=local)
        extra["c1"] = workloads.decode("c1-1.1b", 64, 32, 1280, 1, steps=8, warmup=3, device=local)
        # configuration 2 in small: a serve trace (all sessions at t=0, 64 admitted at a time) through the host-driven driver
        # (a ragged step packed per step, prefill chunks riding the decode runs) and through the device batch (seats,
        # admission and retirement on the device, 8 steps a run)
        from goinfer_b200.serve import run_poisson
        keep = ("sessions", "makespan_s", "output_tokens", "output_tok_s", "total_tok_s", "steps", "runs", "mean_step_ms", "mean_run_ms",
                "ttft_ms", "inter_token_ms", "driver")
        extra["c2_serve"] = {}
        for name, db in (("host_driven", 0), ("device_batch", 8)):
            res = run_poisson("c1-1.1b", 128, 40.0, 64, 1, 32, 1024, 16, 128, chunk=512, device=local, time_scale=0.0, device_batch=db)
            extra["c2_serve"][name] = {k: res[k] for k in keep if k in res}
        extra["c2_serve"]["workload"] = "c1-1.1b shape: 128 sessions at t=0, prompts U[32,1024], outputs U[16,128], <= 64 admitted, greedy"
    if world > 1 and not args.no_extra:
        # the 70B-class shape split over these same ranks (its own communicator; the largest batch whose KV fits)
        barrier()
        tp_c5 = tp_leg(rank)
        if tp_c5 is not None:
            extra["tp_c5"] = tp_c5

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([dev_ms, e2e_s * 1e3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_s = float(t[0]), float(t[1]) / 1e3
    if rank != 0:
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = attn_bytes_per_launch / (attn_ms_per_launch * 1e-3) / 1e9 if attn_ms_per_launch > 0 else 0.0
    # DRAM bytes per launch from an ncu capture of the same kernel on a smaller case (32 rows: dram read + write = 1.015 x the
    # algorithmic bytes), scaled by the keys a full launch processes (traffic is proportional to keys).
    traffic = 1.015 * attn_bytes_per_launch
    h2d = B * s.hidden * 4 + (2 + 3 * B) * 4 + B * 4 + B * 24
    line = {
        "metric": METRIC, "value": world * B * K / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 x s8 integer dots (Q4_K x per-32 int8), fp32 accumulate; fp16 KV", "data": "synthetic",
        "config": workload_config(world),
        "e2e": {"value": world * B * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": B * 4,
                "ms_per_step": e2e_s / K * 1e3},
        "gpu_launches": launches,
        "clocks": clk,
        "roofline": {"kernel": "attn_mma_kernel<128,4> (paged tensor-core flash-decode attention)", "bound": "hbm",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": "of measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "of fallback",
                     "frac_of_8tbs_nominal": achieved / 8000.0, "traffic": traffic,
                     "algorithmic_bytes_per_launch": attn_bytes_per_launch, "ms_per_launch": attn_ms_per_launch,
                     "launches_timed": attn_launches, "share_of_step": attn_ms_total / dev_ms if dev_ms else None},
        "breakdown": breakdown,
        "prefill_chunk": prefill,
        "memory": {"weights_gb": caps.weight_bytes / 1e9, "kv_gb": caps.kv_bytes / 1e9, "scratch_gb": caps.scratch_bytes / 1e9},
    }
    line.update(extra)
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = {k: v for k, v in cpu_sample(2, 1).items() if k != "ms_per_step"}
    if world == 1 and not args.no_gemv:
        from goinfer_b200.ops import Ops
        ops = Ops(local)
        # the matrices a decode step of this shape streams: up/down (28 MB), gate|up as the step fuses them (57 MB), and the
        # vocabulary projection were it Q4_K (350 MB). `read_floor_ms` is a kernel that only reads the same bytes, launched
        # the same way: what this size allows at all (launch and drain are a fixed part of a launch this short).
        for name, N, K, copies in (("q4k_gemv_12288x4096", 12288, 4096, 8), ("q4k_gemv_24576x4096", 24576, 4096, 8),
                                   ("q4k_gemv_151936x4096", 151936, 4096, 3)):
            gb = N * K * 144 / 256 / 1e9
            floor_ms = ops.bench_read(N * K * 144 // 256, copies, 3, 20)
            rows = []
            for M in (1, 2, 4, 8, 16, 32):
                t = ops.bench_q4k_matmul(M, K, N, 0, copies, 3, 20)
                rows.append({"rows": M, "ms": t, "weight_GBps": gb / (t * 1e-3), "frac_of_measured_peak": gb / (t * 1e-3) / peak,
                             "frac_of_read_floor": floor_ms / t})
            line[name] = {"weight_mb": gb * 1e3, "read_floor_ms": floor_ms, "read_floor_frac_of_measured_peak": gb / (floor_ms * 1e-3) / peak,
                          "rows": rows}
    print(json.dumps(line), flush=True)


def tp_leg(rank: int):
    """The tensor-parallel leg: every rank starts a child process (python -m goinfer_b200.workloads decode-tp) that joins a
    process group of its own on the next port, so that a failure or a stall of that leg costs the leg and not the
    benchmark's line; rank 0 returns the child's result (or what went wrong), the others None."""
    import subprocess
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(env.get("MASTER_PORT", "29500")) + 23)
    env["NCCL_NVLS_ENABLE"] = "0"   # the leg's sums across ranks run on the library's own kernel; its few NCCL calls need no multicast
    for k in [k for k in env if k.startswith("TORCHELASTIC_")]:
        env.pop(k)
    torch_cache_clear()
    cmd = [sys.executable, "-m", "goinfer_b200.workloads", "decode-tp", "--shape", "c5-70b", "--batch", "256", "--ctx-lo", "1024",
           "--ctx-hi", "32768", "--seed", "4", "--steps", "4", "--warmup", "2"]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, env=env, cwd=ROOT, text=True)
    try:
        out, err = p.communicate(timeout=480)
    except subprocess.TimeoutExpired:
        p.kill()
        out, err = p.communicate()
        return {"error": "the tensor-parallel leg did not finish in 480 s"} if rank == 0 else None
    if rank != 0:
        return None
    for line in reversed(out.splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                break
    return {"error": f"the tensor-parallel leg exited with code {p.returncode}", "stderr_tail": err[-600:]}


def torch_cache_clear():
    import gc
    import torch
    gc.collect()
    torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-gemv", action="store_true", help="skip the Q4_K small-batch matmul sweep")
    ap.add_argument("--no-extra", action="store_true", help="skip the legs beside the headline workload (exact class, c4, c1; tp_c5 on N >= 2)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
