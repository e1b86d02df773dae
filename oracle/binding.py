"""ctypes binding of the CPU oracle (oracle/liboracle.so). TEST INFRASTRUCTURE ONLY: imported by tests/,
the smoke check and the benchmark's CPU-baseline leg, never by the product package."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

from goinfer_b200 import abi
from goinfer_b200.resident import Resident

_DIR = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_DIR, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_DIR, "oracle.cpp")
    if force or not os.path.exists(_PATH) or os.path.getmtime(_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _DIR, "-s"])
    return _PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            build()
        _lib = C.CDLL(_PATH)
        _lib.oracle_last_error.restype = C.c_char_p
    return _lib


class _OracleDriver:
    def __init__(self):
        self.lib = lib()
        self._m = None

    def last_error(self, model=None) -> str:
        return self.lib.oracle_last_error(model).decode() if model else ""

    def model_create(self, cfg):
        m = C.c_void_p()
        return self.lib.oracle_model_create(C.byref(cfg), C.byref(m)), m

    def fn(self, name):
        if name == "model_finalize":
            def finalize(m, caps_ref):
                return abi.OK
            return finalize
        return getattr(self.lib, "oracle_" + name)

    def close(self):
        pass


class OracleResident(Resident):
    """The oracle behind the same host mirror the product uses, so a parity test drives both alike."""

    def __init__(self, cfg: abi.ModelCfg):
        super().__init__(cfg, _driver=_OracleDriver())

    def finalize(self):
        self.caps = abi.Caps(context_cap=self.cfg.ctx_cap, kv_slots=self.cfg.n_slots, batch_lo=2,
                             batch_hi=self.cfg.n_slots, batch_greedy_draw=1)
        return self.caps

    def FreeBlocks(self) -> int:
        return self.drv.lib.oracle_free_blocks(self.m)

    def LastHidden(self, n: int) -> np.ndarray:
        out = np.zeros(n, np.float32)
        self.drv.lib.oracle_last_hidden(out.ctypes.data_as(C.POINTER(C.c_float)), n)
        return out


def last_tap(which: int, n: int) -> np.ndarray:
    out = np.zeros(n, np.float32)
    lib().oracle_last_tap(which, out.ctypes.data_as(C.POINTER(C.c_float)), n)
    return out


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def op_quant_g32(x: np.ndarray):
    x = np.ascontiguousarray(x, np.float32)
    rows, k = x.shape
    codes = np.empty((rows, k), np.int8)
    scales = np.empty((rows, 2 * (k // 32)), np.float32)
    lib().oracle_op_quant_g32(_p(x, C.c_float), rows, k, _p(codes, C.c_int8), _p(scales, C.c_float))
    return codes, scales


def op_q4k_dequant(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.empty((rows, cols), np.float32)
    lib().oracle_op_q4k_dequant(_p(raw, C.c_uint8), rows, cols, _p(out, C.c_float))
    return out


def op_q4k_unpack_ints(raw: np.ndarray):
    raw = np.ascontiguousarray(raw, np.uint8)
    nb = raw.size // 144
    codes = np.empty((nb, 256), np.uint8)
    sc = np.empty((nb, 8), np.int32)
    mn = np.empty((nb, 8), np.int32)
    lib().oracle_op_q4k_unpack_ints(_p(raw, C.c_uint8), nb, _p(codes, C.c_uint8), _p(sc, C.c_int32), _p(mn, C.c_int32))
    return codes, sc, mn


def op_q4k_matmul(raw: np.ndarray, a: np.ndarray, N: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, np.uint8)
    a = np.ascontiguousarray(a, np.float32)
    M, K = a.shape
    out = np.empty((M, N), np.float32)
    lib().oracle_op_q4k_matmul(_p(raw, C.c_uint8), _p(a, C.c_float), M, K, N, _p(out, C.c_float))
    return out


def op_q4k_matmul_f64(raw: np.ndarray, a: np.ndarray, N: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, np.uint8)
    a = np.ascontiguousarray(a, np.float32)
    M, K = a.shape
    out = np.empty((M, N), np.float64)
    lib().oracle_op_q4k_matmul_f64(_p(raw, C.c_uint8), _p(a, C.c_float), M, K, N, _p(out, C.c_double))
    return out


def op_kq_dequant(kind: int, raw: np.ndarray, rows: int, cols: int, plant: int = 0) -> np.ndarray:
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.empty((rows, cols), np.float64)
    st = lib().oracle_op_kq_dequant(kind, _p(raw, C.c_uint8), rows, cols, plant, _p(out, C.c_double))
    assert st == 0
    return out


def op_kq_matmul_f64(kind: int, raw: np.ndarray, a: np.ndarray, N: int, plant: int = 0):
    """-> (dst [M][N], bar [M][N] = sum |w*a|) in f64."""
    raw = np.ascontiguousarray(raw, np.uint8)
    a = np.ascontiguousarray(a, np.float32)
    M, K = a.shape
    out = np.empty((M, N), np.float64)
    bar = np.empty((M, N), np.float64)
    st = lib().oracle_op_kq_matmul_f64(kind, _p(raw, C.c_uint8), _p(a, C.c_float), M, K, N, plant, _p(out, C.c_double), _p(bar, C.c_double))
    assert st == 0
    return out, bar


def op_q4k_quantize(w: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    out = np.empty(rows * cols // 256 * 144, np.uint8)
    lib().oracle_op_q4k_quantize(_p(w, C.c_float), rows, cols, _p(out, C.c_uint8))
    return out


def op_rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty_like(x)
    lib().oracle_op_rmsnorm(_p(x, C.c_float), _p(w, C.c_float), x.shape[0], x.shape[1], C.c_float(eps), _p(out, C.c_float))
    return out


def op_route(logits: np.ndarray, k: int, norm: bool):
    l = np.ascontiguousarray(logits, np.float32)
    rows, nE = l.shape
    idx = np.empty((rows, k), np.int32)
    wts = np.empty((rows, k), np.float32)
    lib().oracle_op_route(_p(l, C.c_float), rows, nE, k, int(norm), _p(idx, C.c_int32), _p(wts, C.c_float))
    return idx, wts


def op_draw(logits: np.ndarray, draws, mask_index=None, masks=None) -> np.ndarray:
    l = np.ascontiguousarray(logits, np.float32)
    rows, V = l.shape
    d = (abi.Draw * rows)(*draws)
    ids = np.empty(rows, np.int32)
    mi = None if mask_index is None else np.ascontiguousarray(mask_index, np.int32)
    mk = None if masks is None else np.ascontiguousarray(masks, np.uint32)
    lib().oracle_op_draw(_p(l, C.c_float), rows, V, d, _p(mi, C.c_int32), _p(mk, C.c_uint32),
                         0 if mk is None else mk.shape[0], _p(ids, C.c_int32))
    return ids


def op_topk(logits: np.ndarray, k: int, inv_t: float = 1.0):
    l = np.ascontiguousarray(logits, np.float32)
    rows, V = l.shape
    ids = np.empty((rows, k), np.int32)
    vals = np.empty((rows, k), np.float32)
    z = np.empty(rows, np.float64)
    lib().oracle_op_topk(_p(l, C.c_float), rows, V, k, C.c_float(inv_t), _p(ids, C.c_int32), _p(vals, C.c_float), _p(z, C.c_double))
    return ids, vals, z


def op_philox(ctr: np.ndarray, key: np.ndarray) -> np.ndarray:
    c = np.ascontiguousarray(ctr, np.uint32).reshape(-1, 4)
    k = np.ascontiguousarray(key, np.uint32).reshape(-1, 2)
    out = np.empty_like(c)
    lib().oracle_op_philox(_p(c, C.c_uint32), _p(k, C.c_uint32), c.shape[0], _p(out, C.c_uint32))
    return out


def op_gumbel_keys(logits_row: np.ndarray, inv_t: float, seed: int, draw: int):
    """-> (index the host draw picks or -1, every entry's key)."""
    l = np.ascontiguousarray(logits_row, np.float32)
    keys = np.empty_like(l)
    idx = lib().oracle_op_gumbel_keys(_p(l, C.c_float), l.shape[0], C.c_float(inv_t), C.c_uint64(seed), C.c_uint64(draw), _p(keys, C.c_float))
    return idx, keys


def op_minp_set(logits_row: np.ndarray, temperature: float, min_p: float):
    l = np.ascontiguousarray(logits_row, np.float32)
    V = l.shape[0]
    ids = np.empty(V, np.int32)
    probs = np.empty(V, np.float64)
    n = lib().oracle_op_minp_set(_p(l, C.c_float), V, C.c_float(temperature), C.c_float(min_p), _p(ids, C.c_int32),
                                 _p(probs, C.c_double), V)
    return ids[:n].copy(), probs[:n].copy()


def op_attention(q, k, v, n_keys, n_heads, n_kv_heads, head_dim, scale, softcap=0.0) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    nk = np.ascontiguousarray(n_keys, np.int32)
    rows, max_keys = k.shape[0], k.shape[1]
    out = np.empty_like(q)
    lib().oracle_op_attention(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float), _p(nk, C.c_int32), rows, max_keys,
                              n_heads, n_kv_heads, head_dim, C.c_float(scale), C.c_float(softcap), _p(out, C.c_float))
    return out


def threads() -> int:
    return lib().oracle_threads()


def use_all_cores() -> int:
    """Gives the oracle's parallel loops every core this process may run on (torch.distributed.run exports
    OMP_NUM_THREADS=1 to its workers) and returns the thread count in use."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(n)
    return threads()
