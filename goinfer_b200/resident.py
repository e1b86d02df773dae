"""Host-side mirror of goinfer's resident-backend contract over the C ABI of libgoinfer_b200.so.

Names, argument meaning and error behaviour follow the reference's Go interfaces so that tests read
like its own: `ResidentForward` (Forward / Reset, decoder/resident/forward.go:5-33), the decode
subsystem's `StepBatch` / `StepRagged` / `ForwardArgmax` (decoder/resident/subsystems.go:102-117), the
wire types `BatchSeq`, `BatchDraw`, `BatchOut`, `RaggedSeq`, `RaggedPrefill`, `RaggedOut`
(decoder/resident/forward.go:35-84), `Caps` (:119-146) and `ErrKVPoolFull` (decoder/mc3_batch.go:492-498).

The CUDA library is required: importing this module never falls back to a CPU path, and constructing a
`Resident` without the built library raises.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import abi

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libgoinfer_b200.so")
_lib = None


class ResidentError(RuntimeError):
    """Any non-OK status of the library other than a full KV pool."""

    def __init__(self, status: int, text: str):
        super().__init__(f"b200 status {status}: {text}")
        self.status = status


class ErrKVPoolFull(ResidentError):
    """decoder.ErrKVPoolFull: the step mapped every row's blocks first and wrote nothing."""


class DeclinedError(ResidentError):
    """decoder.DeclineResident: the backend will not build this model resident."""


def load_library() -> C.CDLL:
    """dlopen the CUDA library and check every declared symbol resolves. No GPU is touched."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(
                f"{_LIB_PATH} is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU fallback)")
        lib = C.CDLL(_LIB_PATH)
        missing = [s for s in abi.EXPORTS + abi.BENCH_EXPORTS if not hasattr(lib, s)]
        if missing:
            raise ImportError(f"libgoinfer_b200.so lacks symbols: {missing}")
        lib.b200_last_error.restype = C.c_char_p
        lib.b200_launch_count.restype = C.c_int64
        _lib = lib
    return _lib


@dataclass
class BatchDraw:
    """resident.BatchDraw plus the draws this backend makes on the device: min-p with the host sampler's uniform, and
    temperature-only Gumbel-max over the Philox stream (Seed, DrawIndex = Sampler.NextDraw)."""
    Greedy: bool = True
    Temperature: float = 1.0
    MinP: float = 0.0
    U: float = 0.0  # the uniform the host sampler drew for this token (min-p only)
    Gumbel: bool = False
    Seed: int = 0
    DrawIndex: int = 0

    def to_c(self) -> abi.Draw:
        if self.Gumbel:
            return abi.gumbel_draw(self.Temperature, self.Seed, self.DrawIndex)
        if self.Greedy:
            return abi.Draw(abi.DRAW_GREEDY, 1.0, 0.0, 0.0, 0.0)
        return abi.Draw(abi.DRAW_MINP, self.Temperature, self.MinP, 0.0, self.U)


@dataclass
class BatchSeq:
    Slot: int
    Pos: int
    Emb: Optional[np.ndarray] = None  # [hidden] f32, the host embedResident row
    Token: Optional[int] = None       # alternative to Emb: device table gather
    Draw: Optional[BatchDraw] = None
    Mask: Optional[np.ndarray] = None  # uint32 [ceil(vocab/32)], bit set = token allowed


@dataclass
class RaggedPrefill:
    PromptLen: int
    Last: bool


@dataclass
class RaggedSeq:
    Slot: int
    Pos: int
    Embs: Optional[np.ndarray] = None       # [rows, hidden] f32
    Tokens: Optional[Sequence[int]] = None  # alternative to Embs
    Draw: Optional[BatchDraw] = None
    Prefill: Optional[RaggedPrefill] = None
    Mask: Optional[np.ndarray] = None

    def rows(self) -> int:
        return len(self.Embs) if self.Embs is not None else len(self.Tokens)


@dataclass
class BatchOut:
    Logits: Optional[np.ndarray]
    ID: int


@dataclass
class RaggedOut:
    Logits: List[Optional[np.ndarray]] = field(default_factory=list)
    ID: int = -1


class _B200Driver:
    """The C ABI as the mirror drives it. The test oracle supplies a twin with the same methods."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self.lib = load_library()
        self.ctx = C.c_void_p()
        st = self.lib.b200_open(device, C.c_void_p(stream or 0), C.byref(self.ctx))
        if st != abi.OK:
            raise ResidentError(st, "b200_open failed (is a B200 visible?)")

    def last_error(self, model=None) -> str:
        s = self.lib.b200_last_error(self.ctx)
        return s.decode() if s else ""

    def model_create(self, cfg):
        m = C.c_void_p()
        return self.lib.b200_model_create(self.ctx, C.byref(cfg), C.byref(m)), m

    def fn(self, name):
        return getattr(self.lib, "b200_" + name)

    def close(self):
        if self.ctx:
            self.lib.b200_close(self.ctx)
            self.ctx = C.c_void_p()


def _ptr(a: Optional[np.ndarray], typ):
    return a.ctypes.data_as(C.POINTER(typ)) if a is not None else None


class Resident:
    """One model built resident on one GPU: the object `ResidencyBackend.BuildResident` returns
    (decoder/residency.go:208-210), with its four subsystems flattened into methods."""

    def __init__(self, cfg: abi.ModelCfg, device: int = 0, stream: Optional[int] = None, _driver=None):
        self.cfg = cfg
        self.drv = _driver if _driver is not None else _B200Driver(device, stream)
        st, self.m = self.drv.model_create(cfg)
        self._check(st)
        self.caps: Optional[abi.Caps] = None
        self.words = (cfg.vocab + 31) // 32

    # ---- errors ----
    def _check(self, st: int):
        if st == abi.OK:
            return
        text = self.drv.last_error(getattr(self, "m", None))
        if st == abi.KV_POOL_FULL:
            raise ErrKVPoolFull(st, text or "kv pool full")
        if st == abi.DECLINED:
            raise DeclinedError(st, text)
        raise ResidentError(st, text)

    # ---- build ----
    def upload(self, which: int, arr: np.ndarray, layer: int = -1, expert: int = -1, kind: Optional[int] = None,
               rows: Optional[int] = None, cols: Optional[int] = None):
        if kind is None:
            kind = {np.dtype(np.float32): abi.K_F32, np.dtype(np.float16): abi.K_F16}[arr.dtype]
        a = np.ascontiguousarray(arr)
        if rows is None:
            rows, cols = (a.shape if a.ndim == 2 else (1, a.shape[0]))
        self._check(self.drv.fn("upload_tensor")(self.m, which, layer, expert, kind, rows, cols,
                                                 a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes)))

    def synth(self, which: int, kind: int, rows: int, cols: int, sigma: float, seed: int, layer: int = -1,
              expert: int = -1):
        self._check(self.drv.fn("synth_tensor")(self.m, which, layer, expert, kind, rows, cols,
                                                C.c_float(sigma), C.c_uint64(seed)))

    def set_rope_inv_freq(self, inv_freq: np.ndarray, layer: int = -1):
        f = np.ascontiguousarray(inv_freq, dtype=np.float64)
        self._check(self.drv.fn("set_rope_inv_freq")(self.m, layer, _ptr(f, C.c_double), len(f)))

    def finalize(self) -> abi.Caps:
        caps = abi.Caps()
        self._check(self.drv.fn("model_finalize")(self.m, C.byref(caps)))
        self.caps = caps
        return caps

    def Close(self):
        if self.m:
            self.drv.fn("model_free")(self.m)
            self.m = None

    # ---- KV subsystem ----
    def KVSlots(self) -> int:
        return self.cfg.n_slots

    def ResetSlot(self, slot: int):
        self._check(self.drv.fn("reset_slot")(self.m, slot))

    def Reset(self):
        self._check(self.drv.fn("reset")(self.m))

    def BlockTable(self, slot: int) -> np.ndarray:
        n = (self.cfg.ctx_cap + self.cfg.kv_block_rows - 1) // self.cfg.kv_block_rows
        out = np.zeros(n, np.int32)
        self._check(self.drv.fn("block_table")(self.m, slot, _ptr(out, C.c_int32), n))
        return out

    def UploadKV(self, slot: int, layer: int, base: int, keys: np.ndarray, vals: np.ndarray):
        k = np.ascontiguousarray(keys, np.float32)
        v = np.ascontiguousarray(vals, np.float32)
        self._check(self.drv.fn("upload_kv")(self.m, slot, layer, base, k.shape[0], _ptr(k, C.c_float),
                                             _ptr(v, C.c_float)))

    def CopyKV(self, dst: int, src: int, n_rows: int):
        """KVSubsystem.CopyKV: dst is reset and then holds src's first n_rows rows (whole blocks shared, copy on write)."""
        self._check(self.drv.fn("copy_kv")(self.m, dst, src, n_rows))

    def SynthKV(self, slot: int, n_pos: int, sigma: float, seed: int):
        self._check(self.drv.fn("synth_kv")(self.m, slot, n_pos, C.c_float(sigma), C.c_uint64(seed)))

    def ResidentCaps(self) -> abi.Caps:
        return self.caps

    def BatchStepRange(self):
        return (self.caps.batch_lo, self.caps.batch_hi) if self.caps else (0, 0)

    # ---- the step ----
    def StepRagged(self, seqs: Sequence[RaggedSeq]) -> List[RaggedOut]:
        n = len(seqs)
        H, V = self.cfg.hidden, self.cfg.vocab
        slot = np.array([s.Slot for s in seqs], np.int32)
        pos = np.array([s.Pos for s in seqs], np.int32)
        nrows = np.array([s.rows() for s in seqs], np.int32)
        plen = np.array([s.Prefill.PromptLen if s.Prefill else 0 for s in seqs], np.int32)
        plast = np.array([1 if (s.Prefill and s.Prefill.Last) else 0 for s in seqs], np.uint8)
        use_tokens = all(s.Embs is None for s in seqs)
        if not use_tokens and any(s.Embs is None for s in seqs):
            raise ValueError("a step carries embeddings for every sequence or token ids for every sequence")
        embs = toks = None
        if use_tokens:
            toks = np.concatenate([np.asarray(s.Tokens, np.int32) for s in seqs]).astype(np.int32)
        else:
            embs = np.ascontiguousarray(np.concatenate(
                [np.asarray(s.Embs, np.float32).reshape(-1, H) for s in seqs]), np.float32)
        draws = (abi.Draw * n)(*[(s.Draw.to_c() if s.Draw else abi.Draw(abi.DRAW_LOGITS, 0, 0, 0, 0)) for s in seqs])
        masks = [s.Mask for s in seqs if s.Mask is not None]
        midx = np.full(n, -1, np.int32)
        j = 0
        for i, s in enumerate(seqs):
            if s.Mask is not None:
                midx[i] = j
                j += 1
        mask_arr = np.ascontiguousarray(np.stack(masks).astype(np.uint32)) if masks else None
        # rows that return logits
        n_out = 0
        for s in seqs:
            if s.Prefill:
                n_out += 1 if s.Prefill.Last else 0
            else:
                n_out += s.rows() - (1 if s.Draw else 0)
        logits = np.empty((max(n_out, 1), V), np.float32)
        ids = np.full(n, -1, np.int32)
        nlr = C.c_int32(0)
        st = self.drv.fn("step_ragged")(
            self.m, n, _ptr(slot, C.c_int32), _ptr(pos, C.c_int32), _ptr(nrows, C.c_int32), _ptr(plen, C.c_int32),
            _ptr(plast, C.c_uint8), _ptr(embs, C.c_float), _ptr(toks, C.c_int32), draws, _ptr(midx, C.c_int32),
            _ptr(mask_arr, C.c_uint32), len(masks), _ptr(logits, C.c_float), _ptr(ids, C.c_int32), C.byref(nlr))
        self._check(st)
        assert nlr.value == n_out, (nlr.value, n_out)
        outs, j = [], 0
        for i, s in enumerate(seqs):
            o = RaggedOut([], int(ids[i]))
            r = s.rows()
            for k in range(r):
                returns = (s.Prefill.Last and k == r - 1) if s.Prefill else not (s.Draw and k == r - 1)
                if returns:
                    o.Logits.append(logits[j])
                    j += 1
                else:
                    o.Logits.append(None)
            outs.append(o)
        return outs

    def StepBatch(self, seqs: Sequence[BatchSeq]) -> List[BatchOut]:
        rs = [RaggedSeq(s.Slot, s.Pos, None if s.Emb is None else np.asarray(s.Emb, np.float32).reshape(1, -1),
                        None if s.Token is None else [s.Token], s.Draw, None, s.Mask) for s in seqs]
        return [BatchOut(o.Logits[0], o.ID) for o in self.StepRagged(rs)]

    def Forward(self, emb: Optional[np.ndarray], pos: int, slot: int = 0, token: Optional[int] = None) -> np.ndarray:
        return self.StepBatch([BatchSeq(slot, pos, emb, token)])[0].Logits

    def ForwardArgmax(self, emb: Optional[np.ndarray], pos: int, slot: int = 0, token: Optional[int] = None) -> int:
        return self.StepBatch([BatchSeq(slot, pos, emb, token, BatchDraw(Greedy=True))])[0].ID

    def ForwardTopK(self, emb: Optional[np.ndarray], pos: int, k: int, temperature: float = 1.0, want_z: bool = True, slot: int = 0,
                    token: Optional[int] = None):
        """DecodeSubsystem.ForwardTopK: the k best (ids, logits) of the row, ordered (logit desc, id asc), and Z."""
        ids = np.empty(k, np.int32)
        vals = np.empty(k, np.float32)
        z = C.c_double(0)
        e = None if emb is None else np.ascontiguousarray(emb, np.float32)
        inv_t = float(np.float32(1.0 / (temperature if temperature > 0 else 1.0)))
        self._check(self.drv.fn("forward_topk")(self.m, slot, _ptr(e, C.c_float), -1 if token is None else int(token), pos, k,
                                               C.c_float(inv_t), _ptr(ids, C.c_int32), _ptr(vals, C.c_float),
                                               C.byref(z) if want_z else None))
        return ids, vals, (z.value if want_z else None)

    def PrefillLast(self, embs: Optional[np.ndarray], start_pos: int, slot: int = 0,
                    tokens: Optional[Sequence[int]] = None) -> np.ndarray:
        n = len(embs) if embs is not None else len(tokens)
        o = self.StepRagged([RaggedSeq(slot, start_pos, embs, tokens, None, RaggedPrefill(start_pos + n, True))])
        return o[0].Logits[-1]

    def DecodeLoop(self, slots: Sequence[int], pos: Sequence[int], first_ids: Sequence[int], steps: int, log_ids: bool = True,
                   advance: bool = True):
        """`steps` greedy decode steps with the drawn ids fed back on the device (no host round trip between steps):
        sequence i starts by feeding first_ids[i] at position pos[i]. Returns (ids [steps][n] or None, device ms).
        Without log_ids the loop replays one captured CUDA graph from its second step on."""
        n = len(slots)
        sl = np.asarray(slots, np.int32)
        ps = np.asarray(pos, np.int32)
        fi = np.asarray(first_ids, np.int32)
        ids = np.zeros((steps, n), np.int32) if log_ids else None
        ms = C.c_float(0)
        self._check(self.drv.fn("decode_loop_device")(self.m, n, _ptr(sl, C.c_int32), _ptr(ps, C.c_int32), _ptr(fi, C.c_int32), steps,
                                                     1 if advance else 0, _ptr(ids, C.c_int32), C.byref(ms)))
        return ids, ms.value

    # ---- the device batch: seats bound to slots, admission and retirement applied on the device ----
    def BatchOpen(self, n_seats: int, first_slot: int, park_slot: int, max_steps: int = 64):
        self._check(self.drv.fn("batch_open")(self.m, n_seats, first_slot, park_slot, max_steps))
        self._batch_seats, self._batch_steps = n_seats, max_steps

    def BatchAdmit(self, seat: int, pos: int, token: int, max_new: int, eos_id: int = -1):
        """The sequence in the seat's slot continues at `pos` by feeding `token` (its slot was prefilled up to there)."""
        self._check(self.drv.fn("batch_admit")(self.m, seat, pos, token, max_new, eos_id))

    def BatchRetire(self, seat: int):
        self._check(self.drv.fn("batch_retire")(self.m, seat))

    def BatchRun(self, steps: int):
        """`steps` greedy steps for every seat. Returns the records (seat, id, pos, retired) of live seats in step order."""
        cap = steps * self._batch_seats
        ev = np.zeros((max(1, cap), 4), np.int32)
        n = C.c_int32(0)
        self._check(self.drv.fn("batch_run")(self.m, steps, _ptr(ev, C.c_int32), cap, C.byref(n)))
        return [(int(s), int(i), int(p), bool(f & 2)) for s, i, p, f in ev[: n.value]]

    def BatchClose(self):
        self._check(self.drv.fn("batch_close")(self.m))

    def Stats(self) -> abi.Stats:
        s = abi.Stats()
        self._check(self.drv.fn("stats")(self.m, C.byref(s)))
        return s
