"""What a new request may reuse of the KV rows the slots already hold: the host-side index that feeds `CopyKV`.

The reference keeps this in its KV manager (internal/runtime/kvmgr): every full block of 64 positions a finished pass
wrote is published under a chain hash, the identity of everything that decides its bytes and the bytes of every block
before it (the root: model, namespace, adapter, KV precision; the tokens; image spans; the kernel class that wrote each
row), and a request takes the longest chain of published blocks its own cold prefill would have written identically.
The hashes here are computed over the reference's canonical byte encoding (key.go:119-210), so two hosts agree on them.

The device side of a hit is `Resident.CopyKV(dst, src, rows)`: whole device blocks are shared by reference, so a hit
costs no KV bytes. This module never touches the device; the serve driver (serve.py `drive`) connects the two.

Standing: a mirror for this repository's Python serve driver and its tests, not part of the library. A Go host keeps its
own kvmgr and only calls `b200_copy_kv`; the parts of the key this backend cannot exercise (image spans, adapter ids,
windowed layers) are carried only so that hashes and the reference's own test tables agree.
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

BLOCK_ROWS = 64          # kvmgr/key.go:21: positions per logical block; a multiple of the device's 16-row blocks
MIN_LEAD_REUSE = 64      # kvmgr/key.go:94

CLASS_UNKNOWN, CLASS_EXACT, CLASS_FAST = 0, 1, 2   # kvmgr/key.go:48-58

PART_ADAPTER, PART_IMAGE, PART_CLASS, PART_PRECISION, PART_NAMESPACE = 1, 2, 4, 8, 16
ALL_PARTS = 31


@dataclass(frozen=True)
class Root:
    """What a whole chain is built under (kvmgr/key.go:28-33). Requests whose roots differ share no block."""
    Model: str = ""
    Namespace: str = ""
    Adapter: int = 0
    Precision: str = ""


@dataclass(frozen=True)
class ImageSpan:
    """One image's rows; taken whole or not at all. Hash 0 claims nothing and never matches (kvmgr/key.go:37-41)."""
    Start: int
    Len: int
    Hash: int = 0

    @property
    def end(self) -> int:
        return self.Start + self.Len


@dataclass(frozen=True)
class ClassRun:
    Start: int
    Len: int
    Class: int


@dataclass
class Request:
    Root: Root
    Tokens: Sequence[int]
    Images: Sequence[ImageSpan] = ()


# ---------------------------------------------------------------------------------------------------------------------
# the kernel-class rule of a backend (kvmgr/key.go:60-112, share.go:7-46)
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ClassMap:
    """A pass runs the fast kernels when it has at least MinRows rows and the prompt length it is judged on is at least
    Floor; Floor 0: one class at every length. For this library: Floor = the fast-prefill floor the model's capabilities
    report, MinRows = 16 (the prefill kernel's row tile), in the fast kernel class; the zero value in the exact class."""
    Floor: int = 0
    MinRows: int = 0
    Windowed: bool = False

    def Pass(self, rows: int, judged: int) -> int:
        return CLASS_FAST if self.Floor > 0 and judged >= self.Floor and rows >= self.MinRows else CLASS_EXACT

    def PassAt(self, start: int, rows: int, judged: int) -> int:
        c = self.Pass(rows, judged)
        if c == CLASS_FAST and self.Windowed and start % BLOCK_ROWS != 0:
            return CLASS_UNKNOWN
        return c

    def DeclineShortLead(self, prompt_len: int, reuse: int) -> int:
        """reuse, or 0 when it is a lead shorter than MIN_LEAD_REUSE under a prompt whose cold prefill is fast class."""
        if reuse <= 0 or reuse >= MIN_LEAD_REUSE:
            return reuse
        return reuse if self.Pass(prompt_len, prompt_len) != CLASS_FAST else 0

    def ColdClasses(self, n: int) -> List[ClassRun]:
        return [ClassRun(0, n, self.PassAt(0, n, n))] if n > 0 else []

    def CapHit(self, n: int, hit: int) -> int:
        """Shrinks a hit block by block until the pass over the rest writes the class the cold prefill writes."""
        cold = self.Pass(n, n)
        while hit > 0 and self.PassAt(hit, n - hit, n) != cold:
            hit -= BLOCK_ROWS
        return max(hit, 0)

    def CapInPlace(self, held: Sequence[ClassRun], images: Sequence[ImageSpan], n: int, reuse: int) -> int:
        cold = self.Pass(n, n)
        if reuse <= 0 or reuse >= n or self.PassAt(reuse, n - reuse, n) == cold:
            return reuse
        runs = clip_classes(held, reuse)
        if len(runs) != 1 or runs[0].Start != 0 or runs[0].Len != reuse or runs[0].Class != cold:
            return reuse
        return _off_images(images, self.CapHit(n, reuse // BLOCK_ROWS * BLOCK_ROWS) // BLOCK_ROWS) * BLOCK_ROWS


def append_class(runs: List[ClassRun], r: ClassRun) -> List[ClassRun]:
    if r.Len <= 0:
        return runs
    if runs and runs[-1].Class == r.Class and runs[-1].Start + runs[-1].Len == r.Start:
        runs[-1] = ClassRun(runs[-1].Start, runs[-1].Len + r.Len, r.Class)
        return runs
    runs.append(r)
    return runs


def clip_classes(classes: Sequence[ClassRun], n: int) -> List[ClassRun]:
    """classes restricted to rows [0, n), adjacent runs of one class merged (kvmgr/key.go:218-231)."""
    out: List[ClassRun] = []
    for r in classes:
        if r.Start >= n or r.Len <= 0:
            continue
        if r.Start + r.Len > n:
            r = ClassRun(r.Start, n - r.Start, r.Class)
        append_class(out, r)
    return out


def record_turn_classes(prior: Sequence[ClassRun], matched: int, prompt_len: int, total_len: int, pass_class: int) -> List[ClassRun]:
    """Reused rows keep their classes, the prefilled rows are `pass_class`, decode's rows exact (kvmgr/sequence.go:42-51)."""
    out = clip_classes(prior, min(matched, total_len))
    end = min(prompt_len, total_len)
    if end > matched:
        append_class(out, ClassRun(matched, end - matched, pass_class))
    if total_len > prompt_len:
        append_class(out, ClassRun(prompt_len, total_len - prompt_len, CLASS_EXACT))
    return out


def class_at(classes: Sequence[ClassRun], p: int) -> int:
    for r in classes:
        if r.Start <= p < r.Start + r.Len:
            return r.Class
    return CLASS_UNKNOWN


# ---------------------------------------------------------------------------------------------------------------------
# chain hashes (kvmgr/key.go:119-210): tagged fields, lengths on every variable field, little-endian 64-bit integers
# ---------------------------------------------------------------------------------------------------------------------
def _u64(v: int) -> bytes:
    return struct.pack("<Q", v & 0xFFFFFFFFFFFFFFFF)


def _str(s: str) -> bytes:
    b = s.encode()
    return _u64(len(b)) + b


def root_hash(r: Root, parts: int = ALL_PARTS) -> bytes:
    buf = [b"R", _u64(BLOCK_ROWS), _str(r.Model)]
    if parts & PART_NAMESPACE:
        buf += [b"n", _str(r.Namespace)]
    if parts & PART_ADAPTER:
        buf += [b"a", _u64(r.Adapter)]
    if parts & PART_PRECISION:
        buf += [b"p", _str(r.Precision)]
    return hashlib.sha256(b"".join(buf)).digest()


def block_hash(prev: bytes, i: int, tokens: Sequence[int], images: Sequence[ImageSpan], classes: Sequence[ClassRun],
               parts: int = ALL_PARTS) -> bytes:
    """Link i of a chain; block i must be full. The classes are run-length encoded inside the block, so the same row
    classes cut into different runs hash alike."""
    lo, hi = i * BLOCK_ROWS, (i + 1) * BLOCK_ROWS
    buf = [b"B", prev, struct.pack("<%dq" % BLOCK_ROWS, *[int(t) for t in tokens[lo:hi]])]
    if parts & PART_IMAGE:
        for s in images:
            if s.Start < hi and s.end > lo:
                buf += [b"i", _u64(s.Hash), _u64(s.Start - lo), _u64(s.Len)]
    if parts & PART_CLASS:
        cur, n = class_at(classes, lo), 0
        for p in range(lo, hi):
            c = class_at(classes, p)
            if c != cur:
                buf += [b"c", bytes([cur]), _u64(n)]
                cur, n = c, 0
            n += 1
        buf += [b"c", bytes([cur]), _u64(n)]
    return hashlib.sha256(b"".join(buf)).digest()


def _unclaimed(images: Sequence[ImageSpan], i: int) -> bool:
    lo, hi = i * BLOCK_ROWS, (i + 1) * BLOCK_ROWS
    return any(s.Hash == 0 and s.Start < hi and s.end > lo for s in images)


def _unknown_class(classes: Sequence[ClassRun], i: int) -> bool:
    """Any row of block i unknown: named so, or covered by no run (kvmgr/manager.go:254-272)."""
    return any(class_at(classes, p) == CLASS_UNKNOWN for p in range(i * BLOCK_ROWS, (i + 1) * BLOCK_ROWS))


def _off_images(images: Sequence[ImageSpan], blocks: int) -> int:
    """Backs a boundary of `blocks` blocks off any image span it cuts (kvmgr/share.go:70-84)."""
    moved = True
    while moved:
        moved = False
        edge = blocks * BLOCK_ROWS
        for s in images:
            if s.Start < edge < s.end:
                blocks, moved = s.Start // BLOCK_ROWS, True
                break
    return blocks


def request_chain(root: Root, tokens: Sequence[int], images: Sequence[ImageSpan], cold: Sequence[ClassRun],
                  parts: int = ALL_PARTS) -> List[bytes]:
    """The chain hash of each leading block of a request, up to the last block that leaves a token to compute; it stops
    at a block an unclaimed image touches or a row whose producer is not named (kvmgr/share.go:49-67)."""
    limit = (len(tokens) - 1) // BLOCK_ROWS if len(tokens) > 0 else 0
    out, prev = [], root_hash(root, parts)
    for i in range(limit):
        if _unclaimed(images, i) or _unknown_class(cold, i):
            break
        prev = block_hash(prev, i, tokens, images, cold, parts)
        out.append(prev)
    return out


def safe_reuse_len(matched: int, prompt_len: int, floor: int = 0, reusable: Optional[Callable[[int], int]] = None) -> int:
    """Always leaves one token to compute; nothing under the slot's floor (kvmgr/sequence.go:121-140)."""
    if matched <= 0 or prompt_len <= 1:
        return 0
    n = min(matched, prompt_len - 1)
    if n < floor:
        return 0
    if reusable is not None:
        n = reusable(n)
        if n <= 0:
            return 0
        n = min(n, prompt_len - 1)
        if n < floor:
            return 0
    return n


def score_tokens(tokens: Sequence[int], images: Sequence[ImageSpan], req: Request) -> int:
    """Leading tokens of req a stored sequence holds, image spans atomic and only when the request claims the same image
    at the same place (kvmgr/sequence.go:154-183, the attention-model branch)."""
    if len(tokens) == 0 or len(req.Tokens) == 0:
        return 0
    n = min(len(req.Tokens) - 1, len(tokens))
    i = bi = 0
    images = list(images)
    while i < n:
        while bi < len(images) and images[bi].end <= i:
            bi += 1
        if bi < len(images) and images[bi].Start == i:
            sp = images[bi]
            c = next((c for c in req.Images if c.Start == sp.Start), None)
            if c is not None and c.Len == sp.Len and sp.Hash != 0 and c.Hash == sp.Hash and sp.end <= n:
                i = sp.end
                bi += 1
                continue
            return i
        if tokens[i] != req.Tokens[i]:
            return i
        i += 1
    return i


def pick_slot_within(scores: Sequence[int], lens: Sequence[int], uses: Sequence[int], busy: Optional[Sequence[bool]],
                     allowance: int = BLOCK_ROWS, own: Optional[Callable[[int], bool]] = None) -> int:
    """The best-scoring slot when reusing it keeps at least what the new suffix overwrites and gives up fewer than
    `allowance` rows (or `own` says the request is that conversation's rollback); else an empty slot; else the least
    recently used one; busy slots never; -1 when all are busy (kvmgr/slots.go:203-233)."""
    free = lambda i: busy is None or i >= len(busy) or not busy[i]
    best = -1
    for i, s in enumerate(scores):
        if free(i) and s > 0 and (best < 0 or s > scores[best]):
            best = i
    if best >= 0:
        keep, cut = scores[best], lens[best] - scores[best]
        if (own is not None and own(best)) or (keep >= cut and cut < allowance):
            return best
    for i, l in enumerate(lens):
        if free(i) and l == 0:
            return i
    lru = -1
    for i in range(len(uses)):
        if free(i) and (lru < 0 or uses[i] < uses[lru]):
            lru = i
    return lru


# ---------------------------------------------------------------------------------------------------------------------
# the per-slot record (kvmgr/slots.go, share.go)
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Seq:
    root: Root
    root_hash: bytes
    tokens: List[int]
    images: List[ImageSpan]
    classes: List[ClassRun]
    hashes: List[bytes] = field(default_factory=list)   # the chain hash of each published block
    first: int = 0                                      # the length of the conversation's first prompt

    def Len(self) -> int:
        return len(self.tokens)

    def Published(self) -> int:
        return len(self.hashes)


@dataclass
class _Pending:
    ok: bool = False
    reuse: int = 0
    prompt_len: int = 0
    fp: int = 0
    prefix: List[ClassRun] = field(default_factory=list)
    first: int = 0


def _fingerprint(tokens: Sequence[int]) -> int:
    return hash(tuple(int(t) for t in tokens))


class SlotIndex:
    """The reference's `Slots` for a backend whose slots keep their rows until they are given away: what each slot
    holds, published block by block, and what a request may take from it. On this library's paged pool a slot's
    published blocks can also be held by other slots (CopyKV shares them), so giving a slot away frees only the blocks
    nobody else names; the index itself is per slot, as the reference's is."""

    def __init__(self, n: int, parts: int = ALL_PARTS):
        n = max(n, 1)
        self.parts = parts
        self.seqs: List[Optional[Seq]] = [None] * n
        self.uses = [0] * n
        self.pend = [_Pending() for _ in range(n)]
        self.live = [False] * n
        self.floors = [0] * n
        self.tick = 0

    def Count(self) -> int:
        return len(self.seqs)

    def Seq(self, slot: int) -> Optional[Seq]:
        return self.seqs[slot]

    def Len(self, slot: int) -> int:
        s = self.seqs[slot]
        return len(s.tokens) if s is not None else 0

    def Use(self, slot: int) -> int:
        return self.uses[slot]

    def Touch(self, slot: int):
        self.tick += 1
        self.uses[slot] = self.tick

    def Live(self, slot: int) -> bool:
        return self.live[slot]

    def SetFloor(self, slot: int, floor: int):
        self.floors[slot] = floor

    # -- what a request may reuse ------------------------------------------------------------------------------------
    def Score(self, slot: int, req: Request) -> int:
        """Tokens of req the sequence in `slot` already holds and req may skip by continuing in that slot."""
        s = self.seqs[slot]
        if s is None or not s.tokens or len(req.Tokens) == 0 or root_hash(req.Root, self.parts) != s.root_hash:
            return 0
        return safe_reuse_len(score_tokens(s.tokens, s.images, req), len(req.Tokens), self.floors[slot])

    def Hits(self, req: Request, cold: Sequence[ClassRun]) -> List[int]:
        """Per slot, how many leading rows of req its published blocks hold: whole blocks, one token left to compute,
        never ending inside an image span; nothing under another root or another class (kvmgr/share.go:89-109)."""
        out = [0] * len(self.seqs)
        chain = request_chain(req.Root, req.Tokens, req.Images, cold, self.parts)
        if not chain:
            return out
        for sl, s in enumerate(self.seqs):
            if s is None:
                continue
            k = 0
            while k < len(chain) and k < len(s.hashes) and s.hashes[k] == chain[k]:
                k += 1
            hit = _off_images(req.Images, k) * BLOCK_ROWS
            if hit >= self.floors[sl] and hit > 0:
                out[sl] = hit
        return out

    def KeepsFirst(self, slot: int, prompt: Sequence[int]) -> bool:
        s = self.seqs[slot]
        if s is None or s.first == 0 or s.first > len(s.tokens) or len(prompt) < s.first:
            return False
        return list(prompt[:s.first]) == s.tokens[:s.first]

    # -- what the generations did ------------------------------------------------------------------------------------
    def Acquired(self, slot: int, reuse: int, prompt: Sequence[int]):
        """A generation is about to skip `reuse` rows of `prompt` in slot and prefill the rest. Call before Forget."""
        p = _Pending(True, reuse, len(prompt), _fingerprint(prompt))
        s = self.seqs[slot]
        if s is not None and reuse > 0:
            p.prefix = clip_classes(s.classes, reuse)
            p.first = s.first
        self.pend[slot] = p

    def Unrecorded(self, slot: int):
        self.pend[slot] = _Pending()

    def Forget(self, slot: int):
        """The slot's rows are no longer known to be any sequence's; nothing of it is found again."""
        self.live[slot] = False
        self.seqs[slot] = None

    def _publish(self, s: Seq):
        prev = s.hashes[-1] if s.hashes else s.root_hash
        i = len(s.hashes)
        while (i + 1) * BLOCK_ROWS <= len(s.tokens):
            prev = block_hash(prev, i, s.tokens, s.images, s.classes, self.parts)
            s.hashes.append(prev)
            i += 1

    def Commit(self, slot: int, root: Root, tokens: Sequence[int], images: Sequence[ImageSpan], prompt_len: int, cm: ClassMap):
        """The slot now holds exactly `tokens`: a prompt of prompt_len tokens and what decode emitted. The prefilled rows
        get the class cm names, reused rows keep theirs, decode's are exact; without a matching Acquired every row is
        unknown and matches no other request (kvmgr/slots.go:308-340)."""
        p = self.pend[slot]
        self.pend[slot] = _Pending()
        self.Forget(slot)
        tokens = [int(t) for t in tokens]
        if not tokens:
            return
        s = Seq(root, root_hash(root, self.parts), tokens, list(images or ()), [], [], prompt_len)
        if p.ok and p.first > 0 and p.reuse >= p.first - 1:
            s.first = p.first
        if p.ok and p.prompt_len == prompt_len and prompt_len <= len(tokens) and p.reuse < prompt_len and \
                p.fp == _fingerprint(tokens[:prompt_len]):
            s.classes = record_turn_classes(p.prefix, p.reuse, prompt_len, len(tokens),
                                            cm.PassAt(p.reuse, prompt_len - p.reuse, prompt_len))
        self._publish(s)
        self.seqs[slot] = s

    def Prefilled(self, slot: int, root: Root, prompt: Sequence[int], images: Sequence[ImageSpan], cm: ClassMap):
        """The announced generation has finished prefilling: the prompt's full blocks are published now, so a request
        arriving while it decodes can take them. The slot is live until Commit or Forget (kvmgr/share.go:160-171)."""
        p = self.pend[slot]
        self.Commit(slot, root, list(prompt), list(images or ()), len(prompt), cm)
        self.pend[slot] = p
        if self.seqs[slot] is not None:
            self.live[slot] = True

    def Copied(self, src: int, dst: int, start: int, rows: int):
        """The backend copied rows [start, rows) of src into dst, whose rows below start already were that prefix: dst
        holds the prefix under the same root, images and classes, its full blocks published (kvmgr/share.go:111-140)."""
        s = self.seqs[src]
        self.Forget(dst)
        self.pend[dst] = _Pending()
        if s is None or rows <= 0:
            return
        if start == 0:
            self.floors[dst] = 0
        self.floors[dst] = max(self.floors[dst], self.floors[src])
        rows = min(rows, len(s.hashes) * BLOCK_ROWS)
        t = Seq(s.root, s.root_hash, s.tokens[:rows], [sp for sp in s.images if sp.end <= rows], clip_classes(s.classes, rows))
        self._publish(t)
        self.seqs[dst] = t
        self.Touch(src)


def plan_reuse(index: SlotIndex, req: Request, cm: ClassMap, busy: Optional[Sequence[bool]] = None) -> Tuple[int, int]:
    """-> (donor slot or -1, rows to take by CopyKV): the slot with the longest hit (ties: the lowest index; a busy slot
    may donate, its published rows are final), capped so the rest of the prompt runs the class its cold prefill runs, a
    short lead under a fast prompt declined (decoder admission order: Hits, CapHit, DeclineShortLead)."""
    n = len(req.Tokens)
    hits = index.Hits(req, cm.ColdClasses(n))
    donor, best = -1, 0
    for sl, h in enumerate(hits):
        if h > best:
            donor, best = sl, h
    if donor < 0:
        return -1, 0
    rows = cm.DeclineShortLead(n, cm.CapHit(n, best))
    return (donor, rows) if rows > 0 else (-1, 0)
