"""Operator-level entry points of libgoinfer_b200.so (host arrays in, host arrays out) and the
device-resident micro-benchmarks. These run the kernels the step uses on caller data."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import abi
from .resident import ResidentError, _B200Driver


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


class Ops:
    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self.drv = _B200Driver(device, stream)
        self.lib, self.ctx = self.drv.lib, self.drv.ctx

    def _check(self, st):
        if st != abi.OK:
            raise ResidentError(st, self.drv.last_error())

    def launch_count(self) -> int:
        return int(self.lib.b200_launch_count(self.ctx))

    def quant_g32(self, x):
        x = np.ascontiguousarray(x, np.float32)
        rows, k = x.shape
        codes = np.empty((rows, k), np.int8)
        scales = np.empty((rows, 2 * (k // 32)), np.float32)
        self._check(self.lib.b200_op_quant_g32(self.ctx, _p(x, C.c_float), rows, k, _p(codes, C.c_int8), _p(scales, C.c_float)))
        return codes, scales

    def q4k_dequant(self, raw, rows, cols):
        raw = np.ascontiguousarray(raw, np.uint8)
        out = np.empty((rows, cols), np.float32)
        self._check(self.lib.b200_op_q4k_dequant(self.ctx, _p(raw, C.c_uint8), rows, cols, _p(out, C.c_float)))
        return out

    def q4k_matmul(self, raw, a, N, klass=0):
        raw = np.ascontiguousarray(raw, np.uint8)
        a = np.ascontiguousarray(a, np.float32)
        M, K = a.shape
        out = np.empty((M, N), np.float32)
        self._check(self.lib.b200_op_q4k_matmul(self.ctx, _p(raw, C.c_uint8), _p(a, C.c_float), M, K, N, klass, _p(out, C.c_float)))
        return out

    def q4k_quantize(self, w):
        w = np.ascontiguousarray(w, np.float32)
        rows, cols = w.shape
        out = np.empty(rows * cols // 256 * 144, np.uint8)
        self._check(self.lib.b200_op_q4k_quantize(self.ctx, _p(w, C.c_float), rows, cols, _p(out, C.c_uint8)))
        return out

    def rmsnorm(self, x, w, eps):
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        out = np.empty_like(x)
        self._check(self.lib.b200_op_rmsnorm(self.ctx, _p(x, C.c_float), _p(w, C.c_float), x.shape[0], x.shape[1], C.c_float(eps), _p(out, C.c_float)))
        return out

    def route(self, logits, k, norm):
        l = np.ascontiguousarray(logits, np.float32)
        rows, nE = l.shape
        idx = np.empty((rows, k), np.int32)
        wts = np.empty((rows, k), np.float32)
        self._check(self.lib.b200_op_route(self.ctx, _p(l, C.c_float), rows, nE, k, int(norm), _p(idx, C.c_int32), _p(wts, C.c_float)))
        return idx, wts

    def draw(self, logits, draws, mask_index=None, masks=None):
        l = np.ascontiguousarray(logits, np.float32)
        rows, V = l.shape
        d = (abi.Draw * rows)(*draws)
        ids = np.empty(rows, np.int32)
        mi = None if mask_index is None else np.ascontiguousarray(mask_index, np.int32)
        mk = None if masks is None else np.ascontiguousarray(masks, np.uint32)
        self._check(self.lib.b200_op_draw(self.ctx, _p(l, C.c_float), rows, V, d, _p(mi, C.c_int32), _p(mk, C.c_uint32),
                                          0 if mk is None else mk.shape[0], _p(ids, C.c_int32)))
        return ids

    def attention(self, q, k, v, n_keys, n_heads, n_kv_heads, head_dim, scale=0.0, softcap=0.0, block_rows=16, klass=0):
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        nk = np.ascontiguousarray(n_keys, np.int32)
        rows, max_keys = k.shape[0], k.shape[1]
        out = np.empty_like(q)
        self._check(self.lib.b200_op_attention(self.ctx, _p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float), _p(nk, C.c_int32),
                                               rows, max_keys, n_heads, n_kv_heads, head_dim, C.c_float(scale), C.c_float(softcap),
                                               block_rows, klass, _p(out, C.c_float)))
        return out

    def topk(self, logits, k, inv_t=1.0):
        l = np.ascontiguousarray(logits, np.float32)
        rows, V = l.shape
        ids = np.empty((rows, k), np.int32)
        vals = np.empty((rows, k), np.float32)
        z = np.empty(rows, np.float64)
        self._check(self.lib.b200_op_topk(self.ctx, _p(l, C.c_float), rows, V, k, C.c_float(inv_t), _p(ids, C.c_int32), _p(vals, C.c_float),
                                          _p(z, C.c_double)))
        return ids, vals, z

    def philox(self, ctr, key):
        c = np.ascontiguousarray(ctr, np.uint32).reshape(-1, 4)
        k = np.ascontiguousarray(key, np.uint32).reshape(-1, 2)
        out = np.empty_like(c)
        self._check(self.lib.b200_op_philox(self.ctx, _p(c, C.c_uint32), _p(k, C.c_uint32), c.shape[0], _p(out, C.c_uint32)))
        return out

    def f16_matmul(self, w, a, klass=0):
        """w f16 [N][K], a f32 [M][K] -> f32 [M][N]."""
        w = np.ascontiguousarray(w, np.float16)
        a = np.ascontiguousarray(a, np.float32)
        (N, K), M = w.shape, a.shape[0]
        out = np.empty((M, N), np.float32)
        self._check(self.lib.b200_op_f16_matmul(self.ctx, w.view(np.uint16).ctypes.data_as(C.POINTER(C.c_uint16)), _p(a, C.c_float),
                                                M, K, N, klass, _p(out, C.c_float)))
        return out

    def bench_f16_matmul(self, M, K, N, klass=0, warmup=3, iters=10) -> float:
        ms = C.c_float(0)
        self._check(self.lib.b200_bench_f16_matmul(self.ctx, M, K, N, klass, warmup, iters, C.byref(ms)))
        return ms.value

    def prefill_attention(self, q, k, v, pos0, n_heads, n_kv_heads, head_dim, scale=0.0, softcap=0.0, block_rows=16):
        """q [rows][n_heads*head_dim], k/v [pos0+rows][n_kv_heads*head_dim]; row j sees keys 0..pos0+j."""
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        rows = q.shape[0]
        assert k.shape[0] == pos0 + rows and v.shape == k.shape
        out = np.empty_like(q)
        self._check(self.lib.b200_op_prefill_attention(self.ctx, _p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float), rows, pos0,
                                                       n_heads, n_kv_heads, head_dim, C.c_float(scale), C.c_float(softcap),
                                                       block_rows, _p(out, C.c_float)))
        return out

    def bench_prefill_attention(self, rows, pos0, n_heads, n_kv_heads, head_dim, block_rows=16, warmup=3, iters=10) -> float:
        ms = C.c_float(0)
        self._check(self.lib.b200_bench_prefill_attention(self.ctx, rows, pos0, n_heads, n_kv_heads, head_dim, block_rows,
                                                          warmup, iters, C.byref(ms)))
        return ms.value

    def bench_q4k_matmul(self, M, K, N, klass=0, n_weight_copies=8, warmup=3, iters=20) -> float:
        ms = C.c_float(0)
        self._check(self.lib.b200_bench_q4k_matmul(self.ctx, M, K, N, klass, n_weight_copies, warmup, iters, C.byref(ms)))
        return ms.value

    def kq_matmul(self, kind: int, raw: np.ndarray, a: np.ndarray, N: int) -> np.ndarray:
        """Q5_K / Q6_K weights (the file's blocks) x f32 rows, quantized per 32 on the device."""
        raw = np.ascontiguousarray(raw, np.uint8)
        a = np.ascontiguousarray(a, np.float32)
        M, K = a.shape
        out = np.empty((M, N), np.float32)
        self._check(self.lib.b200_op_kq_matmul(self.ctx, kind, raw.ctypes.data_as(C.POINTER(C.c_uint8)), a.ctypes.data_as(C.POINTER(C.c_float)),
                                               M, K, N, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def gate_up_swiglu(self, raw: np.ndarray, a: np.ndarray, F: int, mode: int):
        """-> (codes int8 [M][F], scales f32 [M][2*F/32]) of silu(gate) * up; mode 0 separate kernels, 1 fused epilogue, 2 interleaved + separate."""
        raw = np.ascontiguousarray(raw, np.uint8)
        a = np.ascontiguousarray(a, np.float32)
        M, K = a.shape
        codes = np.empty((M, F), np.int8)
        scales = np.empty((M, 2 * (F // 32)), np.float32)
        self._check(self.lib.b200_op_gate_up_swiglu(self.ctx, raw.ctypes.data_as(C.POINTER(C.c_uint8)), a.ctypes.data_as(C.POINTER(C.c_float)),
                                                    M, K, F, mode, codes.ctypes.data_as(C.POINTER(C.c_int8)), scales.ctypes.data_as(C.POINTER(C.c_float))))
        return codes, scales

    def bench_kq_matmul(self, kind, M, K, N, n_weight_copies=8, warmup=3, iters=20) -> float:
        ms = C.c_float(0)
        self._check(self.lib.b200_bench_kq_matmul(self.ctx, kind, M, K, N, n_weight_copies, warmup, iters, C.byref(ms)))
        return ms.value

    def bench_read(self, nbytes, n_copies=8, warmup=3, iters=20) -> float:
        ms = C.c_float(0)
        self._check(self.lib.b200_bench_read(self.ctx, C.c_size_t(nbytes), n_copies, warmup, iters, C.byref(ms)))
        return ms.value

    def bench_attention(self, rows, ctx_lo, ctx_hi, n_heads, n_kv_heads, head_dim, block_rows=16, seed=2, warmup=3, iters=10):
        ms = C.c_float(0)
        kvb = C.c_double(0)
        self._check(self.lib.b200_bench_attention(self.ctx, rows, ctx_lo, ctx_hi, n_heads, n_kv_heads, head_dim, block_rows,
                                                  C.c_uint64(seed), warmup, iters, C.byref(ms), C.byref(kvb)))
        return ms.value, kvb.value
