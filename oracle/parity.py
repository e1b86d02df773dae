"""Parity measurements of a batched decode step at the benchmark's layer shapes: the CUDA resident against the CPU oracle
on the same host-built weights and the same uploaded KV rows. Test infrastructure (used by tests/ and by bench.py's CPU leg).

The product never imports this module. Weights are drawn with torch's CPU generator (fast, seeded) and quantized to Q4_K
by the oracle's quantizer, whose bytes equal the NumPy and the device quantizers'.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, List, Optional

import numpy as np

from goinfer_b200 import abi, synth
from . import binding

ATOL, RTOL = 2e-2, 1e-2          # the build's logit bar: |gpu - oracle| <= ATOL + RTOL * |oracle|
REF_COS, REF_REL_L2 = 0.995, 0.10  # the reference's own GPU-vs-CPU bars (decoder/selftest_gpu.go:30-35)


def _randn(gen, rows, cols, sigma):
    import torch
    return (torch.randn(rows, cols, generator=gen, dtype=torch.float32) * sigma).numpy()


def fast_host_weights(s: synth.Shape, seed: int, n_layers: int, sigma: float = 0.02):
    """Yields (which, layer, expert, kind, rows, cols, array) like synth.host_weights, from a faster generator: N(0, sigma)
    matrices quantized to Q4_K, f16 embedding and head, norms 1 + N(0, 0.05), f32 router."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    H, qd, kvd = s.hidden, s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim

    def q(which, layer, rows, cols, expert=-1):
        return which, layer, expert, abi.K_Q4K, rows, cols, binding.op_q4k_quantize(_randn(gen, rows, cols, sigma))

    def norm(n):
        return (1 + _randn(gen, 1, n, 0.05)[0]).astype(np.float32)

    yield abi.T_EMBED, -1, -1, abi.K_F16, s.vocab, H, _randn(gen, s.vocab, H, sigma).astype(np.float16)
    yield abi.T_LM_HEAD, -1, -1, abi.K_F16, s.vocab, H, _randn(gen, s.vocab, H, sigma).astype(np.float16)
    yield abi.T_FINAL_NORM, -1, -1, abi.K_F32, 1, H, norm(H)
    for l in range(n_layers):
        yield abi.T_ATTN_NORM, l, -1, abi.K_F32, 1, H, norm(H)
        yield abi.T_FFN_NORM, l, -1, abi.K_F32, 1, H, norm(H)
        yield q(abi.T_WQ, l, qd, H)
        yield q(abi.T_WK, l, kvd, H)
        yield q(abi.T_WV, l, kvd, H)
        yield q(abi.T_WO, l, H, qd)
        if s.qk_norm:
            yield abi.T_Q_NORM, l, -1, abi.K_F32, 1, s.head_dim, norm(s.head_dim)
            yield abi.T_K_NORM, l, -1, abi.K_F32, 1, s.head_dim, norm(s.head_dim)
        if s.n_experts:
            yield abi.T_ROUTER, l, -1, abi.K_F32, s.n_experts, H, _randn(gen, s.n_experts, H, sigma)
            for e in range(s.n_experts):
                yield q(abi.T_EXP_GATE, l, s.moe_ffn, H, e)
                yield q(abi.T_EXP_UP, l, s.moe_ffn, H, e)
                yield q(abi.T_EXP_DOWN, l, H, s.moe_ffn, e)
        else:
            yield q(abi.T_GATE, l, s.ffn, H)
            yield q(abi.T_UP, l, s.ffn, H)
            yield q(abi.T_DOWN, l, H, s.ffn)


def logits_metrics(g: np.ndarray, o: np.ndarray, margin: float = 4e-2) -> Dict[str, float]:
    """g, o: [rows][vocab] logits of the CUDA path and of the oracle."""
    g64, o64 = g.astype(np.float64), o.astype(np.float64)
    d = np.abs(g64 - o64)
    within = d <= ATOL + RTOL * np.abs(o64)
    rel_l2 = np.linalg.norm(g64 - o64, axis=1) / np.maximum(np.linalg.norm(o64, axis=1), 1e-30)
    cos = (g64 * o64).sum(1) / np.maximum(np.linalg.norm(g64, axis=1) * np.linalg.norm(o64, axis=1), 1e-30)
    gi, oi = g.argmax(1), o.argmax(1)
    rows = np.arange(len(g))
    near_tie = np.abs(o64[rows, gi] - o64[rows, oi]) <= margin   # ids differ only at a near-tie of the oracle's logits
    return {
        "rows": int(len(g)),
        "max_abs": float(d.max()),
        "frac_within_bar": float(within.mean()),
        "rows_within_bar": float(within.all(1).mean()),
        "rel_l2_max": float(rel_l2.max()),
        "rel_l2_mean": float(rel_l2.mean()),
        "cos_min": float(cos.min()),
        "greedy_equal": float((gi == oi).mean()),
        "greedy_equal_or_near_tie": float(((gi == oi) | near_tie).mean()),
        "logit_std": float(o64.std()),
    }


def decode_step_parity(s: synth.Shape, n_layers: int, batch: int, ctx_lo: int, ctx_hi: int, klass: int, seed: int = 0,
                       vocab: Optional[int] = None, weights: Optional[List] = None, kv_sigma: float = 1.0,
                       device: int = 0) -> Dict[str, float]:
    """One StepBatch of `batch` sequences (contexts uniform in [ctx_lo, ctx_hi], filled through UploadKV with the same N(0,
    kv_sigma) rows on both sides, random token ids) on a model of `n_layers` layers of shape `s`, CUDA resident in kernel
    class `klass` against the oracle. `weights`: a list from fast_host_weights of at least n_layers layers, to share one
    draw among several depths."""
    from goinfer_b200.resident import BatchSeq, Resident
    if vocab:
        s = replace(s, vocab=vocab)
    rng = np.random.default_rng(seed)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, batch)
    cap = int(-(-(int(ctx.max()) + 1) // 16) * 16)
    mk = lambda: synth.make_cfg(s, n_slots=batch, ctx_cap=cap, max_rows=batch, kernel_class=klass, n_layers=n_layers)
    g, o = Resident(mk(), device=device), binding.OracleResident(mk())
    try:
        for which, layer, expert, kind, rows, cols, arr in (weights if weights is not None else fast_host_weights(s, seed, n_layers)):
            if layer >= n_layers:
                continue
            for r in (g, o):
                r.upload(which, arr, layer, expert, kind, rows, cols)
        g.finalize()
        o.finalize()
        kvd = s.n_kv_heads * s.head_dim
        for slot in range(batch):
            n = int(ctx[slot])
            for l in range(n_layers):
                k = rng.standard_normal((n, kvd), dtype=np.float32) * np.float32(kv_sigma)
                v = rng.standard_normal((n, kvd), dtype=np.float32) * np.float32(kv_sigma)
                for r in (g, o):
                    r.UploadKV(slot, l, 0, k, v)
        toks = rng.integers(0, s.vocab, batch)
        seqs = [BatchSeq(i, int(ctx[i]), None, int(toks[i])) for i in range(batch)]
        lg = np.stack([b.Logits for b in g.StepBatch(seqs)])
        lo = np.stack([b.Logits for b in o.StepBatch(seqs)])
        m = logits_metrics(lg, lo)
        m["tables_equal"] = float(all(np.array_equal(g.BlockTable(i), o.BlockTable(i)) for i in range(min(batch, 8))))
        m.update({"n_layers": n_layers, "batch": batch, "klass": klass})
        return m
    finally:
        g.Close()
        o.Close()
