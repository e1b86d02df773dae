"""Synthetic models for the configurations the benchmark and the parity tests name: random-init
N(0, 0.02) weights quantized to Q4_K, f32 norms, f16 embedding and LM head."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np

from . import abi, q4k


@dataclass
class Shape:
    name: str
    hidden: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    qk_norm: bool = False
    n_experts: int = 0
    top_k: int = 0
    moe_ffn: int = 0


# The five BASELINE configurations' shapes, plus small Q4_K-compatible shapes for fast parity tests.
SHAPES: Dict[str, Shape] = {
    "c1-1.1b": Shape("c1-1.1b", 2048, 22, 32, 4, 64, 5632, 32000, 1e-5, 1e4),
    "c3-8b": Shape("c3-8b", 4096, 36, 32, 8, 128, 12288, 151936, 1e-6, 1e6, qk_norm=True),
    "c4-moe": Shape("c4-moe", 2048, 48, 32, 4, 128, 0, 151936, 1e-6, 1e6, qk_norm=True, n_experts=128, top_k=8, moe_ffn=768),
    "c5-70b": Shape("c5-70b", 8192, 80, 64, 8, 128, 28672, 128256, 1e-5, 5e5),
    "tiny-dense": Shape("tiny-dense", 256, 2, 4, 2, 64, 512, 512, 1e-5, 1e4),
    "tiny-qknorm": Shape("tiny-qknorm", 512, 2, 4, 2, 128, 768, 640, 1e-6, 1e6, qk_norm=True),
    "tiny-tp": Shape("tiny-tp", 512, 2, 8, 2, 64, 1024, 512, 1e-5, 1e4),   # splits over 2 ranks in whole super-blocks
    "tiny-moe": Shape("tiny-moe", 256, 2, 4, 2, 128, 0, 512, 1e-6, 1e6, qk_norm=True, n_experts=8, top_k=2, moe_ffn=256),
}


def make_cfg(s: Shape, n_slots: int, ctx_cap: int, kv_block_rows: int = 16, kv_pool_blocks: int = 0,
             max_rows: int = 0, kernel_class: int = abi.CLASS_AUTO, n_layers: int = 0) -> abi.ModelCfg:
    blocks_per_slot = (ctx_cap + kv_block_rows - 1) // kv_block_rows
    c = abi.ModelCfg()
    c.hidden, c.n_layers, c.n_heads, c.n_kv_heads, c.head_dim = s.hidden, n_layers or s.n_layers, s.n_heads, s.n_kv_heads, s.head_dim
    c.ffn, c.vocab, c.rotary_dim, c.qk_norm = s.ffn, s.vocab, s.head_dim, int(s.qk_norm)
    c.n_experts, c.top_k, c.norm_topk, c.moe_ffn = s.n_experts, s.top_k, 1, s.moe_ffn
    c.kv_block_rows = kv_block_rows
    c.kv_pool_blocks = kv_pool_blocks or (1 + n_slots * blocks_per_slot)
    c.n_slots, c.ctx_cap = n_slots, ctx_cap
    c.max_rows = max_rows or max(n_slots, 64)
    c.tp_rank, c.tp_size = 0, 1
    c.kernel_class, c.fast_floor = kernel_class, 0
    c.rms_eps, c.rope_theta = s.rms_eps, s.rope_theta
    c.attn_scale = c.attn_softcap = c.final_softcap = 0.0
    c.embed_scale = 0.0
    return c


Q4_K_M_KINDS = {abi.T_WV: abi.K_Q6K, abi.T_DOWN: abi.K_Q6K, abi.T_LM_HEAD: abi.K_Q6K, abi.T_WK: abi.K_Q5K, abi.T_UP: abi.K_Q5K}
"""A mix like a Q4_K_M file's (its 6-bit v, down and head; Q5_K stands in for the files that use it for q|k|v): q|k|v and
gate|up become groups of unlike kinds."""


W8A8_KINDS = {abi.T_EMBED: abi.K_I8, abi.T_LM_HEAD: abi.K_I8, abi.T_WO: abi.K_I8}
"""What a q4k load of the reference looks like where a tensor has no raw K-quant bytes: int8 rows with a scale per row for the
embedding table, the head and (here) one projection."""


def host_weights(s: Shape, seed: int, n_layers: int = 0, sigma: float = 0.02, kinds=None):
    """Yields (which, layer, expert, kind, rows, cols, array) for every tensor, built on the host.
    Matrices are N(0, sigma) f32 quantized to Q4_K (or the K-quant `kinds` names for that tensor: {which: kind}, dense
    models only); norms are 1 + N(0, 0.05); embed/head are f16 unless `kinds` names the head."""
    rng = np.random.default_rng(seed)
    H, qd, kvd = s.hidden, s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
    kinds = kinds or {}

    def q(rows, cols):
        return q4k.quantize(rng.normal(0, sigma, (rows, cols)).astype(np.float32))

    def mat(which, layer, rows, cols):
        kind = kinds.get(which, abi.K_Q4K)
        w = rng.normal(0, sigma, (rows, cols)).astype(np.float32)
        if kind == abi.K_Q4K:
            return which, layer, -1, kind, rows, cols, q4k.quantize(w)
        from . import kquants
        quant = {abi.K_Q5K: kquants.q5k_quantize, abi.K_Q6K: kquants.q6k_quantize, abi.K_I8: kquants.i8_quantize}[kind]
        return which, layer, -1, kind, rows, cols, quant(w)

    def norm(n):
        return (1 + rng.normal(0, 0.05, n)).astype(np.float32)

    if abi.T_EMBED in kinds:
        yield mat(abi.T_EMBED, -1, s.vocab, H)
    else:
        yield abi.T_EMBED, -1, -1, abi.K_F16, s.vocab, H, rng.normal(0, sigma, (s.vocab, H)).astype(np.float16)
    if abi.T_LM_HEAD in kinds:
        yield mat(abi.T_LM_HEAD, -1, s.vocab, H)
    else:
        yield abi.T_LM_HEAD, -1, -1, abi.K_F16, s.vocab, H, rng.normal(0, sigma, (s.vocab, H)).astype(np.float16)
    yield abi.T_FINAL_NORM, -1, -1, abi.K_F32, 1, H, norm(H)
    for l in range(n_layers or s.n_layers):
        yield abi.T_ATTN_NORM, l, -1, abi.K_F32, 1, H, norm(H)
        yield abi.T_FFN_NORM, l, -1, abi.K_F32, 1, H, norm(H)
        yield mat(abi.T_WQ, l, qd, H)
        yield mat(abi.T_WK, l, kvd, H)
        yield mat(abi.T_WV, l, kvd, H)
        yield mat(abi.T_WO, l, H, qd)
        if s.qk_norm:
            yield abi.T_Q_NORM, l, -1, abi.K_F32, 1, s.head_dim, norm(s.head_dim)
            yield abi.T_K_NORM, l, -1, abi.K_F32, 1, s.head_dim, norm(s.head_dim)
        if s.n_experts:
            yield abi.T_ROUTER, l, -1, abi.K_F32, s.n_experts, H, rng.normal(0, sigma, (s.n_experts, H)).astype(np.float32)
            for e in range(s.n_experts):
                yield abi.T_EXP_GATE, l, e, abi.K_Q4K, s.moe_ffn, H, q(s.moe_ffn, H)
                yield abi.T_EXP_UP, l, e, abi.K_Q4K, s.moe_ffn, H, q(s.moe_ffn, H)
                yield abi.T_EXP_DOWN, l, e, abi.K_Q4K, H, s.moe_ffn, q(H, s.moe_ffn)
        else:
            yield mat(abi.T_GATE, l, s.ffn, H)
            yield mat(abi.T_UP, l, s.ffn, H)
            yield mat(abi.T_DOWN, l, H, s.ffn)


def load_host_weights(residents, s: Shape, seed: int, n_layers: int = 0, sigma: float = 0.02, kinds=None):
    """Uploads the same host-built tensors into every resident in `residents` (e.g. GPU and oracle)."""
    for which, layer, expert, kind, rows, cols, arr in host_weights(s, seed, n_layers, sigma, kinds):
        for r in residents:
            r.upload(which, arr, layer, expert, kind, rows, cols)


def tensor_plan(s: Shape, n_layers: int = 0):
    """(which, layer, expert, kind, rows, cols) of every matrix, for device-side synthesis."""
    H, qd, kvd = s.hidden, s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
    for l in range(n_layers or s.n_layers):
        yield abi.T_WQ, l, -1, abi.K_Q4K, qd, H
        yield abi.T_WK, l, -1, abi.K_Q4K, kvd, H
        yield abi.T_WV, l, -1, abi.K_Q4K, kvd, H
        yield abi.T_WO, l, -1, abi.K_Q4K, H, qd
        if s.n_experts:
            yield abi.T_ROUTER, l, -1, abi.K_F32, s.n_experts, H
            for e in range(s.n_experts):
                yield abi.T_EXP_GATE, l, e, abi.K_Q4K, s.moe_ffn, H
                yield abi.T_EXP_UP, l, e, abi.K_Q4K, s.moe_ffn, H
                yield abi.T_EXP_DOWN, l, e, abi.K_Q4K, H, s.moe_ffn
        else:
            yield abi.T_GATE, l, -1, abi.K_Q4K, s.ffn, H
            yield abi.T_UP, l, -1, abi.K_Q4K, s.ffn, H
            yield abi.T_DOWN, l, -1, abi.K_Q4K, H, s.ffn


def load_device_weights(r, s: Shape, seed: int, n_layers: int = 0, sigma: float = 0.02, head_rows: int = 0):
    """Synthesizes every tensor on the device (no host copies): seeded N(0, sigma), matrices quantized to
    Q4_K by the device quantizer, f16 embedding and head, unit norms with small seeded jitter."""
    H = s.hidden
    k = 0
    r.synth(abi.T_EMBED, abi.K_F16, s.vocab, H, sigma, seed * 1000003 + k); k += 1
    # head_rows: a tensor-parallel rank holds a vocabulary slice of the head
    r.synth(abi.T_LM_HEAD, abi.K_F16, head_rows or s.vocab, H, sigma, seed * 1000003 + k); k += 1
    rng = np.random.default_rng(seed)
    r.upload(abi.T_FINAL_NORM, (1 + rng.normal(0, 0.05, H)).astype(np.float32))
    for l in range(n_layers or s.n_layers):
        r.upload(abi.T_ATTN_NORM, (1 + rng.normal(0, 0.05, H)).astype(np.float32), l)
        r.upload(abi.T_FFN_NORM, (1 + rng.normal(0, 0.05, H)).astype(np.float32), l)
        if s.qk_norm:
            r.upload(abi.T_Q_NORM, (1 + rng.normal(0, 0.05, s.head_dim)).astype(np.float32), l)
            r.upload(abi.T_K_NORM, (1 + rng.normal(0, 0.05, s.head_dim)).astype(np.float32), l)
    for which, layer, expert, kind, rows, cols in tensor_plan(s, n_layers):
        r.synth(which, kind, rows, cols, sigma, seed * 1000003 + k, layer, expert)
        k += 1
