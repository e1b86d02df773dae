"""GGUF Q5_K and Q6_K block formats on the host (NumPy): dequantize (for tensors this library keeps as f16, such as a
quantized embedding table) and deterministic fp32 -> Q5_K / Q6_K quantizers for synthetic weights and test files.

Q5_K, 176 bytes per 256 weights: f16 d, f16 dmin, 12 bytes of eight 6-bit scales and minimums (as Q4_K), qh[32] (the
fifth bit of element l of sub-block j is bit j of qh[l]), qs[128] (low nibbles = sub-block 2p, high = 2p+1 of byte
32p+l); w = d*sc_j*code - dmin*m_j, codes 0..31.
Q6_K, 210 bytes per 256 weights: ql[128], qh[64], sixteen int8 sub-scales (one per 16 weights), f16 d;
w = d * sc_h * (code - 32), codes 0..63. Both as ggml's dequantize_row_q5_K / dequantize_row_q6_K read them, which
the reference restates in backend/cuda/kernels/ks_a1_test.go:69-114.

The reference only reads these formats; the quantizers here are defined from the formats (nearest code against the
rounded f16 block scales), not taken from any other quantizer.
"""
from __future__ import annotations

import numpy as np

from . import q4k

Q5K_BYTES, Q6K_BYTES = 176, 210


def block_bytes(kind: int) -> int:
    from . import abi
    return {abi.K_Q4K: 144, abi.K_Q5K: Q5K_BYTES, abi.K_Q6K: Q6K_BYTES}[kind]


# ---------------------------------------------------------------------------------------------------------------------
# Q5_K
# ---------------------------------------------------------------------------------------------------------------------
def q5k_dequantize(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    b = np.frombuffer(raw, np.uint8).reshape(rows, cols // 256, Q5K_BYTES)
    d = b[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float64)
    dmin = b[..., 2:4].copy().view(np.float16)[..., 0].astype(np.float64)
    sc, m = q4k.unpack_scales(b[..., 4:16])
    qh = b[..., 16:48].astype(np.int32)                                   # [.., 32]
    qs = b[..., 48:176].reshape(rows, -1, 4, 32).astype(np.int32)         # [.., pair, l]
    codes = np.empty((rows, cols // 256, 8, 32), np.int32)
    for p in range(4):
        codes[..., 2 * p, :] = (qs[..., p, :] & 15) | (((qh >> (2 * p)) & 1) << 4)
        codes[..., 2 * p + 1, :] = (qs[..., p, :] >> 4) | (((qh >> (2 * p + 1)) & 1) << 4)
    w = (d[..., None] * sc)[..., None] * codes - (dmin[..., None] * m)[..., None]
    return w.reshape(rows, cols)


def q5k_quantize(w: np.ndarray) -> np.ndarray:
    """f32 [rows, cols] -> Q5_K bytes (uint8, flat)."""
    rows, cols = w.shape
    x = np.asarray(w, np.float64).reshape(rows, cols // 256, 8, 32)
    lo = np.minimum(x.min(-1), 0.0)
    hi = x.max(-1)
    scale = (hi - lo) / 31.0
    mn = -lo
    d = (scale.max(-1) / 63.0).astype(np.float16)
    dmin = (mn.max(-1) / 63.0).astype(np.float16)
    d64, m64 = d.astype(np.float64), dmin.astype(np.float64)
    sc = np.where(d64[..., None] > 0, np.rint(scale / np.where(d64[..., None] > 0, d64[..., None], 1)), 0).clip(0, 63).astype(np.int32)
    m = np.where(m64[..., None] > 0, np.rint(mn / np.where(m64[..., None] > 0, m64[..., None], 1)), 0).clip(0, 63).astype(np.int32)
    ds = d64[..., None] * sc
    dm = m64[..., None] * m
    codes = np.where(ds[..., None] > 0, np.rint((x + dm[..., None]) / np.where(ds[..., None] > 0, ds[..., None], 1)), 0).clip(0, 31).astype(np.int32)
    out = np.zeros((rows, cols // 256, Q5K_BYTES), np.uint8)
    head = q4k.pack(d, dmin, sc, m, np.zeros((rows, cols // 256, 256), np.uint8))
    out[..., 0:16] = head[..., 0:16]
    qh = np.zeros((rows, cols // 256, 32), np.int32)
    for j in range(8):
        qh |= ((codes[..., j, :] >> 4) & 1) << j
    out[..., 16:48] = qh.astype(np.uint8)
    for p in range(4):
        out[..., 48 + 32 * p:48 + 32 * p + 32] = ((codes[..., 2 * p, :] & 15) | ((codes[..., 2 * p + 1, :] & 15) << 4)).astype(np.uint8)
    return out.reshape(-1)


# ---------------------------------------------------------------------------------------------------------------------
# Q6_K
# ---------------------------------------------------------------------------------------------------------------------
def q6k_codes(b: np.ndarray) -> np.ndarray:
    """blocks uint8 [..., 210] -> codes int32 [..., 256] in -32..31 (element order of the row)."""
    ql = b[..., 0:128].astype(np.int32).reshape(b.shape[:-1] + (2, 2, 32))    # [half, which 32 bytes, l]
    qh = b[..., 128:192].astype(np.int32).reshape(b.shape[:-1] + (2, 32))
    out = np.empty(b.shape[:-1] + (2, 4, 32), np.int32)
    out[..., 0, :] = (ql[..., 0, :] & 15) | (((qh >> 0) & 3) << 4)
    out[..., 1, :] = (ql[..., 1, :] & 15) | (((qh >> 2) & 3) << 4)
    out[..., 2, :] = (ql[..., 0, :] >> 4) | (((qh >> 4) & 3) << 4)
    out[..., 3, :] = (ql[..., 1, :] >> 4) | (((qh >> 6) & 3) << 4)
    return (out - 32).reshape(b.shape[:-1] + (256,))


def q6k_dequantize(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    b = np.frombuffer(raw, np.uint8).reshape(rows, cols // 256, Q6K_BYTES)
    d = b[..., 208:210].copy().view(np.float16)[..., 0].astype(np.float64)
    sc = b[..., 192:208].view(np.int8).astype(np.float64)                       # one per 16 weights, in element order
    codes = q6k_codes(b).reshape(rows, -1, 16, 16)
    return (d[..., None, None] * sc[..., None] * codes).reshape(rows, cols)


def q6k_quantize(w: np.ndarray) -> np.ndarray:
    rows, cols = w.shape
    x = np.asarray(w, np.float64).reshape(rows, cols // 256, 16, 16)
    amax = np.abs(x).max(-1)
    scale = amax / 31.0                                                          # per 16 weights
    d = (scale.max(-1) / 127.0).astype(np.float16)
    d64 = d.astype(np.float64)
    sc = np.where(d64[..., None] > 0, np.rint(scale / np.where(d64[..., None] > 0, d64[..., None], 1)), 0).clip(-128, 127).astype(np.int32)
    ds = d64[..., None] * sc
    codes = (np.where(ds[..., None] != 0, np.rint(x / np.where(ds[..., None] != 0, ds[..., None], 1)), 0).clip(-32, 31).astype(np.int32) + 32)
    c = codes.reshape(rows, cols // 256, 2, 4, 32)                               # [half, group, l]
    out = np.zeros((rows, cols // 256, Q6K_BYTES), np.uint8)
    ql = np.empty((rows, cols // 256, 2, 2, 32), np.int32)
    ql[..., 0, :] = (c[..., 0, :] & 15) | ((c[..., 2, :] & 15) << 4)
    ql[..., 1, :] = (c[..., 1, :] & 15) | ((c[..., 3, :] & 15) << 4)
    qh = (c[..., 0, :] >> 4) | ((c[..., 1, :] >> 4) << 2) | ((c[..., 2, :] >> 4) << 4) | ((c[..., 3, :] >> 4) << 6)
    out[..., 0:128] = ql.reshape(rows, cols // 256, 128).astype(np.uint8)
    out[..., 128:192] = qh.reshape(rows, cols // 256, 64).astype(np.uint8)
    out[..., 192:208] = sc.astype(np.int8).view(np.uint8)
    out[..., 208:210] = d[..., None].view(np.uint8)
    return out.reshape(-1)


# ---------------------------------------------------------------------------------------------------------------------
# int8 rows with one f32 scale per row (W8A8: backend/cuda/actgroup.cu:287-297,417-432); bytes: [rows][cols] int8, then rows f32
# ---------------------------------------------------------------------------------------------------------------------
def i8_quantize(w: np.ndarray) -> np.ndarray:
    w = np.asarray(w, np.float32)
    amax = np.abs(w).max(axis=1)
    scale = (amax / 127.0).astype(np.float32)
    inv = np.where(scale > 0, 1.0 / np.where(scale > 0, scale, 1), 0).astype(np.float32)
    codes = np.clip(np.rint(w * inv[:, None]), -127, 127).astype(np.int8)
    return np.concatenate([codes.reshape(-1).view(np.uint8), scale.view(np.uint8)])


def i8_dequantize(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    b = np.frombuffer(raw, np.uint8)
    codes = b[:rows * cols].view(np.int8).reshape(rows, cols).astype(np.float64)
    scale = b[rows * cols:rows * cols + rows * 4].view(np.float32).astype(np.float64)
    return codes * scale[:, None]


def dequantize(kind: int, raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Any K-quant kind -> f64/f32 [rows, cols]."""
    from . import abi
    if kind == abi.K_Q4K:
        return q4k.dequantize(raw, rows, cols)
    if kind == abi.K_Q5K:
        return q5k_dequantize(raw, rows, cols)
    if kind == abi.K_Q6K:
        return q6k_dequantize(raw, rows, cols)
    if kind == abi.K_I8:
        return i8_dequantize(raw, rows, cols)
    raise ValueError(f"kind {kind} is not a K-quant")
