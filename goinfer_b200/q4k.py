"""GGUF Q4_K block format on the host (NumPy): pack, unpack, dequantize and a deterministic fp32 -> Q4_K
quantizer for synthetic weights.

Layout (144 bytes per 256 weights): f16 d, f16 dmin, 12 bytes of eight 6-bit scales and eight 6-bit
minimums, 128 bytes of 4-bit codes; w = d*sc_j*code - dmin*m_j. It is the layout the reference reads
from GGUF files unchanged (decoder/gguf.go:1508-1537) and restates in
backend/cuda/kernels/ks_a1_test.go:62-67,117-131 and backend/cuda/actgroup.cu:64-75.

The reference has no quantizer (it only reads Q4_K); `quantize` is defined here from the format: per
32-weight sub-block scale=(max+min)/15 and min=max(0,-min w); d and dmin are the largest sub-block
scale and minimum over 63, rounded to f16; sub-block scales, minimums and codes are rounded to nearest
even against those f16 values. The device quantizer and the test oracle's produce the same bytes.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = 144
BLOCK_WEIGHTS = 256


def row_bytes(cols: int) -> int:
    if cols % BLOCK_WEIGHTS:
        raise ValueError("Q4_K rows must be a multiple of 256 weights")
    return cols // BLOCK_WEIGHTS * BLOCK_BYTES


def unpack_scales(q12: np.ndarray):
    """q12: [..., 12] uint8 -> (sc [..., 8], m [..., 8]) int32 (ggml get_scale_min_k4)."""
    q = q12.astype(np.int32)
    sc = np.empty(q.shape[:-1] + (8,), np.int32)
    m = np.empty_like(sc)
    sc[..., :4] = q[..., 0:4] & 63
    m[..., :4] = q[..., 4:8] & 63
    sc[..., 4:] = (q[..., 8:12] & 0x0F) | ((q[..., 0:4] >> 6) << 4)
    m[..., 4:] = (q[..., 8:12] >> 4) | ((q[..., 4:8] >> 6) << 4)
    return sc, m


def unpack(blocks: np.ndarray):
    """blocks: uint8 [..., 144] -> d, dmin f32 [...], sc, m int32 [..., 8], codes uint8 [..., 256]."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = b[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    dmin = b[..., 2:4].copy().view(np.float16)[..., 0].astype(np.float32)
    sc, m = unpack_scales(b[..., 4:16])
    qs = b[..., 16:144].reshape(b.shape[:-1] + (4, 32))
    codes = np.empty(b.shape[:-1] + (4, 2, 32), np.uint8)
    codes[..., 0, :] = qs & 0x0F
    codes[..., 1, :] = qs >> 4
    return d, dmin, sc, m, codes.reshape(b.shape[:-1] + (256,))


def dequantize(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """raw Q4_K bytes of a [rows, cols] matrix -> f32 [rows, cols]."""
    blocks = np.frombuffer(raw, np.uint8).reshape(rows, cols // 256, 144)
    d, dmin, sc, m, codes = unpack(blocks)
    ds = d[..., None] * sc.astype(np.float32)
    dm = dmin[..., None] * m.astype(np.float32)
    w = ds[..., None] * codes.reshape(rows, -1, 8, 32).astype(np.float32) - dm[..., None]
    return w.reshape(rows, cols).astype(np.float32)


def pack(d16: np.ndarray, dmin16: np.ndarray, sc: np.ndarray, m: np.ndarray, codes: np.ndarray) -> np.ndarray:
    """Inverse of unpack. d16/dmin16: float16 [...]; sc, m: [..., 8] in 0..63; codes [..., 256] in 0..15."""
    shape = d16.shape
    out = np.zeros(shape + (144,), np.uint8)
    out[..., 0:2] = d16.astype(np.float16)[..., None].view(np.uint8)
    out[..., 2:4] = dmin16.astype(np.float16)[..., None].view(np.uint8)
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out[..., 4:8] = (sc[..., :4] & 63) | ((sc[..., 4:] >> 4) << 6)
    out[..., 8:12] = (m[..., :4] & 63) | ((m[..., 4:] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:] & 0x0F) | ((m[..., 4:] & 0x0F) << 4)
    c = codes.astype(np.uint8).reshape(shape + (4, 2, 32))
    out[..., 16:144] = (c[..., 0, :] | (c[..., 1, :] << 4)).reshape(shape + (128,))
    return out


def quantize(w: np.ndarray) -> np.ndarray:
    """f32 [rows, cols] -> Q4_K bytes uint8 [rows * cols/256 * 144]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    x = w.reshape(rows, cols // 256, 8, 32)
    lo = x.min(-1)
    hi = x.max(-1)
    mn = np.where(lo < 0, -lo, np.float32(0)).astype(np.float32)
    scale = np.maximum((hi + mn) / np.float32(15), np.float32(0)).astype(np.float32)
    d16 = (scale.max(-1) / np.float32(63)).astype(np.float16)
    dmin16 = (mn.max(-1) / np.float32(63)).astype(np.float16)
    d = d16.astype(np.float32)[..., None]
    dmin = dmin16.astype(np.float32)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d > 0, np.clip(np.rint(scale / d), 0, 63), 0).astype(np.int32)
        m6 = np.where(dmin > 0, np.clip(np.rint(mn / dmin), 0, 63), 0).astype(np.int32)
        ds = (d * sc.astype(np.float32)).astype(np.float32)
        dm = (dmin * m6.astype(np.float32)).astype(np.float32)
        inv = np.where(ds > 0, np.float32(1) / ds, np.float32(0)).astype(np.float32)
        t = ((x + dm[..., None]) * inv[..., None]).astype(np.float32)
    codes = np.clip(np.rint(t), 0, 15).astype(np.uint8).reshape(rows, cols // 256, 256)
    return pack(d16, dmin16, sc, m6, codes).reshape(-1)


def random_blocks(rng: np.random.Generator, rows: int, cols: int, exp_lo: int = 9, exp_hi: int = 15) -> np.ndarray:
    """Random valid block bytes the way the reference's tests build Q4_K tensors: every byte uniform, d and
    dmin positive normal f16 with exponent field in [exp_lo, exp_hi] (decoder/q4k_test.go:14-31)."""
    nb = rows * cols // 256
    b = rng.integers(0, 256, size=(nb, 144), dtype=np.uint8)
    for off in (0, 2):
        e = rng.integers(exp_lo, exp_hi + 1, size=nb).astype(np.uint16)
        man = rng.integers(0, 1024, size=nb).astype(np.uint16)
        h = (e << 10) | man
        b[:, off] = (h & 0xFF).astype(np.uint8)
        b[:, off + 1] = (h >> 8).astype(np.uint8)
    return b.reshape(-1)
