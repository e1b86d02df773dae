"""GGUF ingestion: read a llama / qwen2 / qwen3 checkpoint file and hand its tensors to a resident model in the
formats the engine multiplies (Q4_K, Q5_K, Q6_K blocks as they are in the file; F16 / F32 as they are; anything else,
and the embedding table, widened to f16 on the host).

The file format is GGUF v2/v3 (little endian): magic "GGUF", version, tensor and metadata counts, the metadata
key-values, the tensor infos (name, dims innermost first, ggml type, offset), then the data, aligned to
`general.alignment` (32 when absent). The reference reads the same files through its GGUF layer; what this module
mirrors of the reference is the mapping from metadata to a model configuration (decoder/gguf.go:73-202: llama, qwen2,
qwen3 keys and defaults), the tensor names (token_embd, blk.N.attn_q/k/v/output, ffn_gate/up/down, the norms, output),
the rule that llama-family files store q and k rows in interleaved-pair RoPE order, undone row-wise on load
(decoder/gguf.go:1905-1949), and that K-quant projections go to the device as the file's own blocks
(decoder/gguf.go:1508-1541, decoder/kquant_native.go:114-120).

`write` makes small files for tests and for moving synthetic models around; it is not a general exporter.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np

from . import abi, kquants

MAGIC = b"GGUF"
# ggml tensor types this reader knows: (name, block weights, block bytes, engine kind or None)
GGML_TYPES = {
    0: ("F32", 1, 4, abi.K_F32),
    1: ("F16", 1, 2, abi.K_F16),
    8: ("Q8_0", 32, 34, None),
    12: ("Q4_K", 256, 144, abi.K_Q4K),
    13: ("Q5_K", 256, 176, abi.K_Q5K),
    14: ("Q6_K", 256, 210, abi.K_Q6K),
    30: ("BF16", 1, 2, None),
}
TYPE_OF_KIND = {abi.K_F32: 0, abi.K_F16: 1, abi.K_Q4K: 12, abi.K_Q5K: 13, abi.K_Q6K: 14}

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


@dataclass
class TensorInfo:
    name: str
    dims: Tuple[int, ...]   # innermost first, as in the file: (cols, rows) for a matrix
    ggml_type: int
    offset: int             # from the start of the data section

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        _, bw, bb, _ = GGML_TYPES[self.ggml_type]
        return self.n_elements // bw * bb


class GGUFFile:
    """The parsed header of a file and a memory map of its data."""

    def __init__(self, path: str):
        self.path = path
        self.raw = np.memmap(path, dtype=np.uint8, mode="r")
        buf = self.raw
        if bytes(buf[:4]) != MAGIC:
            raise ValueError("not a GGUF file")
        self.version = struct.unpack_from("<I", buf, 4)[0]
        if self.version not in (2, 3):
            raise ValueError(f"GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = struct.unpack_from("<QQ", buf, 8)
        pos = 24
        self.meta: Dict[str, object] = {}
        for _ in range(n_kv):
            key, pos = self._string(pos)
            vt = struct.unpack_from("<I", buf, pos)[0]
            val, pos = self._value(vt, pos + 4)
            self.meta[key] = val
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name, pos = self._string(pos)
            nd = struct.unpack_from("<I", buf, pos)[0]
            dims = struct.unpack_from("<%dQ" % nd, buf, pos + 4)
            pos += 4 + 8 * nd
            gt, off = struct.unpack_from("<IQ", buf, pos)
            pos += 12
            if gt not in GGML_TYPES:
                raise ValueError(f"tensor {name}: ggml type {gt} is not supported")
            self.tensors[name] = TensorInfo(name, tuple(int(d) for d in dims), gt, off)
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = (pos + align - 1) // align * align
        for t in self.tensors.values():
            if self.data_start + t.offset + t.nbytes > len(buf):
                raise ValueError(f"tensor {t.name} runs past the end of the file")

    def _string(self, pos: int):
        n = struct.unpack_from("<Q", self.raw, pos)[0]
        return bytes(self.raw[pos + 8:pos + 8 + n]).decode("utf-8", "replace"), pos + 8 + n

    def _value(self, vt: int, pos: int):
        if vt in _SCALAR:
            f = _SCALAR[vt]
            return struct.unpack_from(f, self.raw, pos)[0], pos + struct.calcsize(f)
        if vt == _T_STRING:
            return self._string(pos)
        if vt == _T_ARRAY:
            et, n = struct.unpack_from("<IQ", self.raw, pos)
            pos += 12
            if et in _SCALAR:
                f = _SCALAR[et]
                sz = struct.calcsize(f)
                arr = np.frombuffer(self.raw[pos:pos + sz * n].tobytes(), dtype=np.dtype(f[1:]).newbyteorder("<")) if et != 7 else \
                    np.frombuffer(self.raw[pos:pos + n].tobytes(), dtype=np.bool_)
                return arr, pos + sz * n
            out = []
            for _ in range(n):
                v, pos = self._value(et, pos)
                out.append(v)
            return out, pos
        raise ValueError(f"metadata value type {vt} is not supported")

    def data(self, name: str) -> np.ndarray:
        """The tensor's bytes, as in the file (a view of the map)."""
        t = self.tensors[name]
        a = self.data_start + t.offset
        return self.raw[a:a + t.nbytes]

    # -- the metadata the model configuration is read from (decoder/gguf.go:73-202) ---------------------------------
    def uint(self, key: str, default: int = 0) -> int:
        v = self.meta.get(key)
        return int(v) if v is not None else default

    def float(self, key: str, default: float) -> float:
        v = self.meta.get(key)
        return float(v) if v is not None else default


ARCH_DEFAULT_ROPE_BASE = {"llama": 10000.0, "qwen2": 1000000.0, "qwen3": 1000000.0}   # decoder/gguf.go:93-96,160-163,194-197
QK_PERMUTED = ("llama",)                                                             # decoder/gguf.go:1905-1912


@dataclass
class GGUFModel:
    arch: str
    hidden: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    context_length: int
    rms_eps: float
    rope_base: float
    qk_norm: bool
    tied_head: bool


def describe(g: GGUFFile) -> GGUFModel:
    arch = str(g.meta.get("general.architecture", ""))
    if arch not in ARCH_DEFAULT_ROPE_BASE:
        raise ValueError(f"architecture {arch!r} is not one this loader maps (llama, qwen2, qwen3)")
    u = lambda k: g.uint(f"{arch}.{k}")
    hidden, heads = u("embedding_length"), u("attention.head_count")
    head_dim = u("attention.key_length") or (hidden // heads if heads else 0)
    emb = g.tensors.get("token_embd.weight")
    if emb is None:
        raise ValueError("token_embd.weight is missing")
    vocab = emb.dims[1]
    biased = sorted(n for n in g.tensors if n.endswith(".bias"))
    if biased:
        # the resident step has no bias add (the path's model families, llama and qwen3, have none; qwen2's q/k/v do)
        raise ValueError(f"tensors with a bias are not supported by this engine: {biased[0]} and {len(biased) - 1} more")
    return GGUFModel(arch, hidden, u("block_count"), heads, u("attention.head_count_kv") or heads, head_dim, u("feed_forward_length"), vocab,
                     u("context_length"), g.float(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5 if arch == "llama" else 1e-6),
                     g.float(f"{arch}.rope.freq_base", ARCH_DEFAULT_ROPE_BASE[arch]), "blk.0.attn_q_norm.weight" in g.tensors,
                     "output.weight" not in g.tensors)


def model_cfg(d: GGUFModel, n_slots: int, ctx_cap: int, kv_block_rows: int = 16, kv_pool_blocks: int = 0, max_rows: int = 0,
              kernel_class: int = abi.CLASS_AUTO) -> abi.ModelCfg:
    c = abi.ModelCfg()
    c.hidden, c.n_layers, c.n_heads, c.n_kv_heads, c.head_dim = d.hidden, d.n_layers, d.n_heads, d.n_kv_heads, d.head_dim
    c.ffn, c.vocab, c.rotary_dim, c.qk_norm = d.ffn, d.vocab, d.head_dim, int(d.qk_norm)
    c.n_experts = c.top_k = c.moe_ffn = 0
    c.norm_topk = 1
    c.kv_block_rows = kv_block_rows
    c.kv_pool_blocks = kv_pool_blocks or (1 + n_slots * ((ctx_cap + kv_block_rows - 1) // kv_block_rows))
    c.n_slots, c.ctx_cap = n_slots, ctx_cap
    c.max_rows = max_rows or max(n_slots, 64)
    c.tp_rank, c.tp_size = 0, 1
    c.kernel_class, c.fast_floor, c.kv_dtype = kernel_class, 0, 0
    c.rms_eps, c.rope_theta = d.rms_eps, d.rope_base
    c.attn_scale = c.attn_softcap = c.final_softcap = 0.0
    c.embed_scale = 1.0
    return c


def _unpermute_rows(raw: np.ndarray, rows: int, row_bytes: int, n_head: int) -> np.ndarray:
    """llama-family files keep q/k rows of a head in interleaved-pair order (2j+s); the engine's RoPE is split-half
    (s*half + j). Whole rows move, so quantized blocks stay intact (decoder/gguf.go:1935-1949)."""
    hd = rows // n_head
    half = hd // 2
    src = np.arange(rows).reshape(n_head, half, 2)          # [h][j][s] = h*hd + 2j + s
    order = np.transpose(src, (0, 2, 1)).reshape(-1)        # destination row h*hd + s*half + j takes source [h][j][s]
    return np.ascontiguousarray(raw.reshape(rows, row_bytes)[order]).reshape(-1)


def _unpermute_vec(v: np.ndarray) -> np.ndarray:
    half = len(v) // 2
    return np.ascontiguousarray(v.reshape(half, 2).T).reshape(-1)


def _widen(g: GGUFFile, t: TensorInfo, rows: int, cols: int) -> np.ndarray:
    """A tensor's values as f32 [rows, cols] (for norms, and for what is kept as f16)."""
    name, bw, bb, kind = GGML_TYPES[t.ggml_type]
    raw = np.asarray(g.data(t.name))
    if name == "F32":
        return raw.view(np.float32).reshape(rows, cols).astype(np.float32)
    if name == "F16":
        return raw.view(np.float16).reshape(rows, cols).astype(np.float32)
    if name == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(rows, cols)
    if name == "Q8_0":
        b = raw.reshape(rows, cols // 32, 34)
        d = b[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
        return (d[..., None] * b[..., 2:].view(np.int8).astype(np.float32)).reshape(rows, cols)
    return np.asarray(kquants.dequantize(kind, raw, rows, cols), np.float32)


LAYER_TENSORS = (("attn_q", abi.T_WQ), ("attn_k", abi.T_WK), ("attn_v", abi.T_WV), ("attn_output", abi.T_WO),
                 ("ffn_gate", abi.T_GATE), ("ffn_up", abi.T_UP), ("ffn_down", abi.T_DOWN))
LAYER_NORMS = (("attn_norm", abi.T_ATTN_NORM), ("ffn_norm", abi.T_FFN_NORM), ("attn_q_norm", abi.T_Q_NORM), ("attn_k_norm", abi.T_K_NORM))


def tensors(g: GGUFFile, d: Optional[GGUFModel] = None) -> Iterator[tuple]:
    """Yields (which, layer, expert, kind, rows, cols, array) for every tensor the engine takes, ready for
    `Resident.upload`: K-quant projections as the file's bytes, float tensors as they are, the rest widened to f16."""
    d = d or describe(g)
    permuted = d.arch in QK_PERMUTED

    def matrix(name: str, which: int, layer: int, n_head_perm: int = 0):
        t = g.tensors[name]
        cols, rows = t.dims[0], t.dims[1]
        _, bw, bb, kind = GGML_TYPES[t.ggml_type]
        raw = np.asarray(g.data(name))
        if kind is not None and which != abi.T_EMBED:
            if n_head_perm:
                raw = _unpermute_rows(raw, rows, cols // bw * bb, n_head_perm)
            arr = raw if kind in (abi.K_Q4K, abi.K_Q5K, abi.K_Q6K) else raw.view(np.float32 if kind == abi.K_F32 else np.float16).reshape(rows, cols)
            return which, layer, -1, kind, rows, cols, np.ascontiguousarray(arr)
        w = _widen(g, t, rows, cols)
        if n_head_perm:
            w = _unpermute_rows(w.view(np.uint8).reshape(-1), rows, cols * 4, n_head_perm).view(np.float32).reshape(rows, cols)
        return which, layer, -1, abi.K_F16, rows, cols, w.astype(np.float16)

    def vector(name: str, which: int, layer: int, perm: bool = False):
        t = g.tensors[name]
        v = _widen(g, t, 1, t.dims[0]).reshape(-1)
        if perm:
            v = _unpermute_vec(v)
        return which, layer, -1, abi.K_F32, 1, len(v), np.ascontiguousarray(v, np.float32)

    yield matrix("token_embd.weight", abi.T_EMBED, -1)
    yield vector("output_norm.weight", abi.T_FINAL_NORM, -1)
    if d.tied_head:
        # the head multiplies the table's own rows: a K-quant table stays in its blocks for the head (its native lane) and is
        # widened only for the gather
        yield matrix("token_embd.weight", abi.T_LM_HEAD, -1)
    else:
        yield matrix("output.weight", abi.T_LM_HEAD, -1)
    for l in range(d.n_layers):
        for nm, which in LAYER_TENSORS:
            heads = d.n_heads if nm == "attn_q" else d.n_kv_heads if nm == "attn_k" else 0
            yield matrix(f"blk.{l}.{nm}.weight", which, l, heads if permuted else 0)
        for nm, which in LAYER_NORMS:
            if f"blk.{l}.{nm}.weight" in g.tensors:
                yield vector(f"blk.{l}.{nm}.weight", which, l, perm=permuted and nm in ("attn_q_norm", "attn_k_norm"))


def load(path: str, resident_factory, n_slots: int = 4, ctx_cap: int = 0, **cfg_kw):
    """Opens the file, creates the resident with `resident_factory(cfg)`, uploads every tensor and finalizes.
    -> (resident, GGUFModel)."""
    g = GGUFFile(path)
    d = describe(g)
    cfg = model_cfg(d, n_slots, ctx_cap or min(d.context_length or 2048, 4096), **cfg_kw)
    r = resident_factory(cfg)
    for which, layer, expert, kind, rows, cols, arr in tensors(g, d):
        r.upload(which, arr, layer, expert, kind, rows, cols)
    r.finalize()
    return r, d


# ---------------------------------------------------------------------------------------------------------------------
# a small writer (tests, synthetic models)
# ---------------------------------------------------------------------------------------------------------------------
def _w_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _w_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", 7, v)
    if isinstance(v, int):
        return struct.pack("<II", 4, v) if 0 <= v < 2 ** 32 else struct.pack("<Iq", 11, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", _T_STRING) + _w_string(v)
    if isinstance(v, (list, tuple)) and all(isinstance(x, str) for x in v):
        return struct.pack("<IIQ", _T_ARRAY, _T_STRING, len(v)) + b"".join(_w_string(x) for x in v)
    raise TypeError(f"metadata value {v!r}")


def write(path: str, meta: Dict[str, object], tensor_list: List[Tuple[str, Tuple[int, ...], int, np.ndarray]], alignment: int = 32):
    """tensor_list: (name, dims innermost first, ggml type, bytes as a uint8 array)."""
    head = [MAGIC, struct.pack("<IQQ", 3, len(tensor_list), len(meta) + 1)]
    head.append(_w_string("general.alignment") + _w_value(alignment))
    for k, v in meta.items():
        head.append(_w_string(k) + _w_value(v))
    off = 0
    blobs = []
    for name, dims, gt, data in tensor_list:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        head.append(_w_string(name) + struct.pack("<I", len(dims)) + struct.pack("<%dQ" % len(dims), *dims) + struct.pack("<IQ", gt, off))
        blobs.append((off, data))
        off = (off + len(data) + alignment - 1) // alignment * alignment
    h = b"".join(head)
    start = (len(h) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(h)
        f.write(b"\0" * (start - len(h)))
        for o, data in blobs:
            f.seek(start + o)
            f.write(data.tobytes())
        f.truncate(start + off)
