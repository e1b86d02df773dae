"""Continuous batching over a Resident: the host logic either side of the ragged step.

Mirrors, in single-threaded event-driven form (one driver loop instead of one goroutine per generation):

* `Admission` — the FIFO turn granter of internal/runtime/scheduler/admission.go:23-122: up to Capacity holders, waiters
  never reordered, a release hands the turn straight to the front waiter.
* `common_prefix`, `best_extend`, `pick_session`, `keeps_first`, `coldest_idle`, `pick_donor` — session placement,
  internal/runtime/scheduler/placement.go:6-100 (pure functions).
* `Batcher` — the token coalescer and resident batcher of decoder/mc3_batch.go:38-73,358-545: a run serves the decode
  tokens pending, in one batched step when there are at least `lo` of them and else one call each; a prefill chunk rides
  the run as the step's first ragged sequence; a step refused with ErrKVPoolFull wrote nothing and its tokens re-run
  solo. Counters follow ResidentBatchStats (:82-94). With a single driver thread every decoding generation has always
  submitted when a run starts, so the 4 ms straggler window (:31,400) never opens; `StragglerRuns` stays 0.
* `chunk_plan` — chunked prefill's pass lengths: chunks of `chunk` rows and a final pass of at least TailMinRows = 8
  (decoder/mc3_batch.go:296-300, decoder/model.go:1076-1084,1215-1219).
* `run_poisson` — the continuous-batching workload: sessions arriving as a Poisson process, prompt and output lengths
  uniform, at most `max_active` admitted, greedy decoding.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence, Tuple

import numpy as np

PREFILL_TAIL_MIN = 8
BATCH_STATS_SIZES = 17


# ---------------------------------------------------------------------------------------------------------------------
# admission (scheduler/admission.go)
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Record:
    ID: str = ""
    PromptIDs: Optional[Sequence[int]] = None  # admission never reads it
    payload: object = None


class Admission:
    """FIFO turn granter. `Enter` returns True when the turn is granted at once, else the record waits in line; `Release`
    returns the record the turn was handed to (it now holds a turn) or None when the turn was given back."""

    def __init__(self, cap: int = 1):
        self._cap = max(1, cap)
        self._held = 0
        self._waiters: Deque[Record] = deque()

    def SetCap(self, n: int):
        self._cap = max(1, n)

    def Capacity(self) -> int:
        return self._cap

    def Load(self) -> int:
        return self._held + len(self._waiters)

    def Enter(self, rec: Record) -> bool:
        if self._held < self._cap and not self._waiters:
            self._held += 1
            return True
        self._waiters.append(rec)
        return False

    def Cancel(self, rec: Record) -> bool:
        """The waiter's context ended: it leaves the line. False when it is not waiting (granted already, or never queued)."""
        try:
            self._waiters.remove(rec)
            return True
        except ValueError:
            return False

    def Position(self, id: str) -> Tuple[int, int, bool, bool]:
        if id == "":
            return 0, 0, False, False
        place, ok = 0, False
        for i, w in enumerate(self._waiters, 1):
            if w.ID == id:
                place, ok = i, True
        return place, len(self._waiters), self._held > 0, ok

    def Release(self) -> Optional[Record]:
        if self._waiters:
            return self._waiters.popleft()  # a hand-off: the held count does not change
        self._held -= 1
        return None


# ---------------------------------------------------------------------------------------------------------------------
# placement (scheduler/placement.go)
# ---------------------------------------------------------------------------------------------------------------------
def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = min(len(a), len(b))
    i = 0
    while i < n and a[i] == b[i]:
        i += 1
    return i


def best_extend(sessions: Sequence[Optional[Sequence[int]]], prompt: Sequence[int]) -> int:
    best, best_match = -1, 0
    for i, toks in enumerate(sessions):
        match = common_prefix(toks or (), prompt)
        if match == 0:
            continue
        floor = 0
        for j, other in enumerate(sessions):
            if j != i:
                floor = max(floor, common_prefix(toks or (), other or ()))
        if match > floor and match > best_match:
            best, best_match = i, match
    return best


def keeps_first(first: int, keep: int) -> bool:
    return first > 0 and keep >= first


def pick_session(sessions, firsts: Sequence[int], prompt: Sequence[int], spare: bool) -> int:
    i = best_extend(sessions, prompt)
    if i >= 0 and spare:
        keep = common_prefix(sessions[i], prompt)
        own = i < len(firsts) and keeps_first(firsts[i], keep)
        if not own and keep < len(sessions[i]) - keep:
            return -1
    return i


def coldest_idle(busy: Sequence[bool]) -> int:
    for i in range(len(busy) - 1, -1, -1):
        if not busy[i]:
            return i
    return -1


def pick_donor(hits: Sequence[int], busy: Optional[Sequence[bool]]) -> Tuple[int, int]:
    donor, hit = -1, 0
    for i, h in enumerate(hits):
        if busy is not None and i < len(busy) and busy[i]:
            continue
        if h > 0 and h >= hit:
            donor, hit = i, h
    return donor, hit


def chunk_plan(n_rows: int, chunk: int, tail_min: int = PREFILL_TAIL_MIN) -> List[int]:
    """Pass lengths of a chunked prefill of n_rows rows: `chunk` rows a pass, the final pass never shorter than tail_min
    (the pass before it gives up rows for that) unless the whole prompt is."""
    if chunk <= 0 or n_rows <= chunk:
        return [n_rows] if n_rows > 0 else []
    out = []
    left = n_rows
    while left > chunk:
        take = chunk
        if 0 < left - take < tail_min:
            take = left - tail_min
        out.append(take)
        left -= take
    out.append(left)
    return out


# ---------------------------------------------------------------------------------------------------------------------
# the batcher (decoder/mc3_batch.go)
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class ResidentBatchStats:
    Runs: int = 0
    Steps: int = 0
    StepTokens: int = 0
    SoloTokens: int = 0
    StragglerRuns: int = 0
    StepSizes: List[int] = field(default_factory=lambda: [0] * BATCH_STATS_SIZES)
    PrefillPasses: int = 0
    RunNs: int = 0
    RidePasses: int = 0
    RideRows: int = 0
    RideNs: int = 0


class Batcher:
    """One run at a time over a resident that takes ragged steps."""

    def __init__(self, resident, max_holders: int):
        from .resident import BatchDraw, BatchSeq, ErrKVPoolFull, RaggedSeq  # the CUDA library is required
        self._BatchSeq, self._RaggedSeq, self._BatchDraw, self._ErrKVPoolFull = BatchSeq, RaggedSeq, BatchDraw, ErrKVPoolFull
        self.r = resident
        lo, hi = resident.BatchStepRange()
        if hi < 2:
            raise ValueError("the resident does not batch")
        self.lo, self.hi = max(lo, 2), hi
        self.max_holders = min(max_holders, resident.KVSlots())
        self.stats = ResidentBatchStats()

    def _solo(self, q):
        """Production's own call for one token: returns (id, error)."""
        try:
            return self.r.StepBatch([q])[0], None
        except Exception as e:  # a run serves every generation in it: one token's failure is that token's error
            return None, e

    def run_tokens(self, run):
        """-> [(BatchOut or None, error or None)] for every token of the run."""
        t0 = time.perf_counter_ns()
        self.stats.Runs += 1
        out = None
        if len(run) >= self.lo:
            try:
                res = self.r.StepBatch(run)
                out = [(o, None) for o in res]
                self.stats.Steps += 1
                self.stats.StepTokens += len(run)
                self.stats.StepSizes[min(len(run), BATCH_STATS_SIZES - 1)] += 1
            except self._ErrKVPoolFull:
                out = None   # the step wrote nothing: every token re-runs on its own and only the starved one ends
            except Exception as e:
                out = [(None, e)] * len(run)
        if out is None:
            out = []
            for q in run:
                out.append(self._solo(q))
                self.stats.SoloTokens += 1
        self.stats.RunNs += time.perf_counter_ns() - t0
        return out

    def ride(self, chunk, run):
        """One ragged step of the chunk (first) and the run's decode rows.
        -> (chunk RaggedOut or None, chunk error or None, [(BatchOut or None, error or None)])."""
        from .resident import BatchOut
        t0 = time.perf_counter_ns()
        seqs = [chunk] + [self._RaggedSeq(q.Slot, q.Pos, None if q.Emb is None else np.asarray(q.Emb, np.float32).reshape(1, -1),
                                          None if q.Token is None else [q.Token], q.Draw, None, q.Mask) for q in run]
        try:
            res = self.r.StepRagged(seqs)
        except Exception as e:
            # the chunk takes the error back; the run is served as a run without it
            toks = self.run_tokens(run) if run else []
            return None, e, toks
        self.stats.Runs += 1
        self.stats.RidePasses += 1
        self.stats.RideRows += len(run)
        self.stats.PrefillPasses += 1
        outs = []
        for q, o in zip(run, res[1:]):
            outs.append((BatchOut(None if q.Draw is not None else o.Logits[0], o.ID if q.Draw is not None else -1), None))
        self.stats.RideNs += time.perf_counter_ns() - t0
        return res[0], None, outs


# ---------------------------------------------------------------------------------------------------------------------
# the Poisson workload
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class _Session:
    idx: int
    arrival: float
    prompt: np.ndarray
    out_len: int
    slot: int = -1
    passes: List[int] = field(default_factory=list)
    done_rows: int = 0
    generated: int = 0
    last_id: int = -1
    t_first: float = 0.0
    t_last: float = 0.0
    t_end: float = 0.0
    gaps: List[float] = field(default_factory=list)
    out_ids: List[int] = field(default_factory=list)
    reused: int = 0


def poisson_trace(n: int, rate: float, seed: int, prompt_lo: int, prompt_hi: int, out_lo: int, out_hi: int, vocab: int,
                  preamble: int = 0, n_preambles: int = 1):
    """preamble > 0: every prompt starts with one of n_preambles shared token runs of that length (a system prompt),
    drawn after everything else so that the lengths and arrivals equal the preamble-free trace of the same seed."""
    rng = np.random.default_rng(seed)
    arrivals = np.cumsum(rng.exponential(1.0 / rate, n))
    p_len = rng.integers(prompt_lo, prompt_hi + 1, n)
    o_len = rng.integers(out_lo, out_hi + 1, n)
    prompts = [rng.integers(0, vocab, int(k)).astype(np.int32) for k in p_len]
    if preamble > 0:
        heads = [rng.integers(0, vocab, preamble).astype(np.int32) for _ in range(max(n_preambles, 1))]
        which = rng.integers(0, len(heads), n)
        for i in range(n):
            k = min(preamble, len(prompts[i]) - 1)
            prompts[i][:k] = heads[int(which[i])][:k]
    return [_Session(i, float(arrivals[i]), prompts[i], int(o_len[i])) for i in range(n)]


def drive(r, sessions: List[_Session], max_active: int, chunk: int, time_scale: float = 1.0, clock=time.perf_counter,
          sleep=time.sleep, index=None, root=None, class_map=None) -> dict:
    """Runs the trace to completion on resident `r` (greedy decoding); returns the measurements.

    With `index` (a kvindex.SlotIndex over the same max_active slots) a finished session's rows stay in its slot, published
    block by block, until the slot is given away; a new prompt takes the longest published prefix another slot holds by
    `CopyKV` (whole device blocks shared by reference), or continues in place in the slot that already holds most of it,
    and prefills only the rest (decoder admission: Score / PickSlot, Hits / CapHit / DeclineShortLead, Copied, Prefilled,
    Commit; internal/runtime/kvmgr/slots.go, share.go)."""
    from . import kvindex
    from .resident import BatchDraw, BatchSeq, RaggedPrefill, RaggedSeq
    adm = Admission(max_active)
    bat = Batcher(r, max_active)
    free_slots = list(range(max_active - 1, -1, -1))
    busy = [False] * max_active
    cm = class_map or kvindex.ClassMap()
    reuse_stats = {"copies": 0, "in_place": 0, "rows_reused": 0, "rows_prefilled": 0}
    waiting = deque(sessions)              # by arrival time
    prefilling: Deque[_Session] = deque()  # admitted, prompt not yet in: the oldest one's next chunk rides each run
    decoding: List[_Session] = []
    finished: List[_Session] = []
    greedy = BatchDraw(Greedy=True)
    step_rows, step_ms = [], []
    t0 = clock()
    now = lambda: (clock() - t0) * time_scale if time_scale > 0 else float("inf")

    def place(s: _Session) -> int:
        """The slot for s and how many of its prompt's leading rows are already there when this returns."""
        prompt = [int(t) for t in s.prompt]
        req = kvindex.Request(root, prompt)
        n = len(prompt)
        scores = [index.Score(i, req) for i in range(max_active)]
        lens = [index.Len(i) for i in range(max_active)]
        uses = [index.Use(i) for i in range(max_active)]
        pick = kvindex.pick_slot_within(scores, lens, uses, busy)
        donor, rows = kvindex.plan_reuse(index, req, cm)
        reuse = 0
        if scores[pick] > 0 and lens[pick] > 0 and scores[pick] >= rows:
            # its own rows, kept in place at token granularity
            reuse = cm.DeclineShortLead(n, cm.CapInPlace(index.Seq(pick).classes, (), n, scores[pick]))
        if reuse > 0:
            index.Acquired(pick, reuse, prompt)
            index.Forget(pick)
            reuse_stats["in_place"] += 1
        elif donor >= 0 and donor != pick and rows > 0:
            r.CopyKV(pick, donor, rows)
            index.Copied(donor, pick, 0, rows)
            index.Acquired(pick, rows, prompt)
            index.Forget(pick)
            reuse = rows
            reuse_stats["copies"] += 1
        else:
            r.ResetSlot(pick)
            index.Acquired(pick, 0, prompt)
            index.Forget(pick)
        index.Touch(pick)
        s.slot, s.reused = pick, reuse
        return reuse

    def start(s: _Session):
        if index is None:
            s.slot = free_slots.pop()
        else:
            s.done_rows = place(s)
            busy[s.slot] = True
            reuse_stats["rows_reused"] += s.done_rows
            reuse_stats["rows_prefilled"] += len(s.prompt) - s.done_rows
        s.passes = chunk_plan(len(s.prompt) - s.done_rows, chunk)
        prefilling.append(s)

    def finish(s: _Session, t: float, failed: bool = False):
        s.t_end = t
        finished.append(s)
        if index is None:
            r.ResetSlot(s.slot)
            free_slots.append(s.slot)
        else:
            busy[s.slot] = False
            if failed:
                index.Forget(s.slot)
                r.ResetSlot(s.slot)
            else:
                # the last drawn id was never fed, so its row does not exist: the slot holds the prompt and all but that id
                index.Commit(s.slot, root, [int(x) for x in s.prompt] + s.out_ids[:-1], None, len(s.prompt), cm)
                index.Touch(s.slot)
        nxt = adm.Release()
        if nxt is not None:
            start(nxt.payload)

    while waiting or prefilling or decoding or adm.Load() > 0:
        t = now()
        while waiting and waiting[0].arrival <= t:
            s = waiting.popleft()
            if adm.Enter(Record(str(s.idx), None, s)):
                start(s)
        if not prefilling and not decoding:
            if not waiting:
                break
            gap = (waiting[0].arrival - t) / time_scale if time_scale > 0 else 0.0
            if gap > 0:
                sleep(min(gap, 0.05))
            continue
        run = [BatchSeq(s.slot, len(s.prompt) + s.generated - 1, None, s.last_id, greedy) for s in decoding[:bat.hi]]
        run_sessions = decoding[:bat.hi]
        ts = clock()
        c_sess = prefilling[0] if prefilling else None
        if c_sess is not None:
            n = c_sess.passes[0]
            lastp = len(c_sess.passes) == 1
            c = RaggedSeq(c_sess.slot, c_sess.done_rows, None, c_sess.prompt[c_sess.done_rows:c_sess.done_rows + n], None,
                          RaggedPrefill(len(c_sess.prompt), lastp))
            c_out, c_err, outs = bat.ride(c, run)
            if c_err is not None:
                raise c_err
        else:
            outs = bat.run_tokens(run)
        te = clock()
        t = (te - t0) * time_scale if time_scale > 0 else te - t0
        step_rows.append(len(run) + (c_sess.passes[0] if c_sess is not None else 0))
        step_ms.append((te - ts) * 1e3)
        for s, (o, err) in zip(run_sessions, outs):
            if err is not None:
                decoding.remove(s)
                finish(s, t, failed=True)
                continue
            s.last_id = int(o.ID)
            s.out_ids.append(s.last_id)
            s.generated += 1
            s.gaps.append(t - s.t_last)
            s.t_last = t
            if s.generated >= s.out_len:
                decoding.remove(s)
                finish(s, t)
        if c_sess is not None:
            c_sess.done_rows += c_sess.passes.pop(0)
            if not c_sess.passes:
                prefilling.popleft()
                c_sess.last_id = int(np.argmax(c_out.Logits[-1]))   # greedy: first maximal index
                c_sess.out_ids.append(c_sess.last_id)
                c_sess.generated = 1
                if index is not None:
                    index.Prefilled(c_sess.slot, root, [int(x) for x in c_sess.prompt], None, cm)
                c_sess.t_first = c_sess.t_last = t
                if c_sess.generated >= c_sess.out_len:
                    finish(c_sess, t)
                else:
                    decoding.append(c_sess)
    makespan = clock() - t0
    out_tok = sum(s.generated for s in finished)
    in_tok = sum(len(s.prompt) for s in finished)
    scale = time_scale if time_scale > 0 else 1.0
    ttft = np.array([(s.t_first - (s.arrival if time_scale > 0 else 0.0)) / scale for s in finished])
    gaps = np.concatenate([np.asarray(s.gaps) for s in finished if s.gaps]) / scale if any(s.gaps for s in finished) else np.zeros(1)
    pct = lambda a, q: float(np.percentile(a, q))
    st = bat.stats
    return {"sessions": len(finished), **({"prefix_reuse": reuse_stats} if index is not None else {}), "makespan_s": makespan, "output_tokens": out_tok, "prompt_tokens": in_tok,
            "output_tok_s": out_tok / makespan, "total_tok_s": (out_tok + in_tok) / makespan,
            "ttft_ms": {"p50": pct(ttft, 50) * 1e3, "p95": pct(ttft, 95) * 1e3, "p99": pct(ttft, 99) * 1e3},
            "inter_token_ms": {"p50": pct(gaps, 50) * 1e3, "p99": pct(gaps, 99) * 1e3},
            "steps": len(step_rows), "mean_rows_per_step": float(np.mean(step_rows)), "mean_step_ms": float(np.mean(step_ms)),
            "busy_fraction": float(np.sum(step_ms) / 1e3 / makespan),
            "batch_stats": {"Runs": st.Runs, "Steps": st.Steps, "StepTokens": st.StepTokens, "SoloTokens": st.SoloTokens,
                            "RidePasses": st.RidePasses, "RideRows": st.RideRows, "StragglerRuns": st.StragglerRuns}}


def drive_device_batch(r, sessions: List[_Session], seats: int, chunk: int, run_steps: int = 8, time_scale: float = 1.0,
                       clock=time.perf_counter, sleep=time.sleep) -> dict:
    """The same trace on the resident's DEVICE batch (BatchOpen / BatchAdmit / BatchRun): `seats` seats over slots
    0..seats-1, slot `seats` as the parking slot. Admission is the same FIFO (scheduler.Admission); an admitted session's
    prompt is prefilled in chunks through the ordinary entry point, its first id is taken from the last chunk's logits, and
    it is seated; every run decodes `run_steps` greedy steps for all seats on the device (ids fed back, positions advanced,
    a seat retired when its session's output length is reached) with nothing packed per step, and the records say which
    session drew what. Ids equal drive()'s (greedy): the steps are the same kernels on the same rows."""
    from .resident import RaggedPrefill, RaggedSeq
    adm = Admission(seats)
    free = list(range(seats - 1, -1, -1))
    seated: dict = {}
    waiting = deque(sessions)
    finished: List[_Session] = []
    r.BatchOpen(seats, 0, seats, max_steps=run_steps)
    runs, run_ms, live_rows = 0, [], []
    t0 = clock()
    now = lambda: (clock() - t0) * time_scale if time_scale > 0 else float("inf")

    def start(s: _Session):
        seat = free.pop()
        s.slot = seat
        r.ResetSlot(seat)
        done, lg = 0, None
        for n in chunk_plan(len(s.prompt), chunk):
            last = done + n == len(s.prompt)
            o = r.StepRagged([RaggedSeq(seat, done, None, s.prompt[done:done + n], None, RaggedPrefill(len(s.prompt), last))])
            if last:
                lg = o[0].Logits[-1]
            done += n
        t = now() if time_scale > 0 else clock() - t0
        s.last_id = int(np.argmax(lg))
        s.out_ids.append(s.last_id)
        s.generated = 1
        s.t_first = s.t_last = t
        if s.generated >= s.out_len:
            finish(s, t)
        else:
            r.BatchAdmit(seat, len(s.prompt), s.last_id, s.out_len - 1)
            seated[seat] = s

    def finish(s: _Session, t: float):
        s.t_end = t
        finished.append(s)
        free.append(s.slot)
        nxt = adm.Release()
        if nxt is not None:
            start(nxt.payload)

    while waiting or seated or adm.Load() > 0:
        t = now()
        while waiting and waiting[0].arrival <= t:
            s = waiting.popleft()
            if adm.Enter(Record(str(s.idx), None, s)):
                start(s)
        if not seated:
            if not waiting:
                break
            gap = (waiting[0].arrival - t) / time_scale if time_scale > 0 else 0.0
            if gap > 0:
                sleep(min(gap, 0.05))
            continue
        ts = clock()
        recs = r.BatchRun(run_steps)
        te = clock()
        t = (te - t0) * time_scale if time_scale > 0 else te - t0
        runs += 1
        run_ms.append((te - ts) * 1e3)
        live_rows.append(len(recs))
        for seat, tok, _pos, retired in recs:
            s = seated[seat]
            s.last_id = tok
            s.out_ids.append(tok)
            s.generated += 1
            s.gaps.append(t - s.t_last)   # a run's ids arrive together: the gap is the run's, as a client of this driver would see it
            s.t_last = t
            if retired:
                del seated[seat]
                finish(s, t)
    r.BatchClose()
    makespan = clock() - t0
    out_tok = sum(s.generated for s in finished)
    return {"sessions": len(finished), "makespan_s": makespan, "output_tokens": out_tok, "output_tok_s": out_tok / makespan,
            "runs": runs, "steps_per_run": run_steps, "mean_run_ms": float(np.mean(run_ms)) if run_ms else 0.0,
            "mean_live_rows_per_run": float(np.mean(live_rows)) if live_rows else 0.0}


def run_poisson(shape: str, n_sessions: int, rate: float, max_active: int, seed: int, prompt_lo: int, prompt_hi: int, out_lo: int,
                out_hi: int, chunk: int = 512, device: int = 0, n_layers: int = 0, time_scale: float = 1.0, preamble: int = 0,
                n_preambles: int = 1, prefix_reuse: bool = False, device_batch: int = 0) -> dict:
    """Builds the synthetic model, runs the trace, returns one result dict. time_scale > 1 compresses the arrival clock;
    0 makes every session arrive at once (the closed-loop capacity of the engine at `max_active`). preamble > 0 gives the
    prompts shared leading runs; prefix_reuse serves them from the slots that already hold them."""
    from . import abi, kvindex, synth
    from .resident import Resident
    s = synth.SHAPES[shape]
    cap = prompt_hi + out_hi + 1
    blocks = 1 + max_active * ((cap + 15) // 16)
    # (the device batch parks its empty seats on one more slot)
    cfg = synth.make_cfg(s, max_active + (1 if device_batch else 0), cap, 16, blocks + 1, chunk + max_active, abi.CLASS_AUTO, n_layers)
    r = Resident(cfg, device=device)
    synth.load_device_weights(r, s, seed=seed, n_layers=n_layers)
    r.finalize()
    trace = poisson_trace(n_sessions, rate, seed, prompt_lo, prompt_hi, out_lo, out_hi, s.vocab, preamble, n_preambles)
    # warm the kernels' first-launch costs outside the measurement
    r.PrefillLast(None, 0, 0, tokens=list(range(1, 65)))
    r.ResetSlot(0)
    kw = {}
    if prefix_reuse:
        caps = r.ResidentCaps()
        kw = dict(index=kvindex.SlotIndex(max_active), root=kvindex.Root(Model=f"{shape}/q4k/b200", Precision="f16"),
                  class_map=kvindex.ClassMap(Floor=caps.fast_prefill_floor, MinRows=16) if caps.has_fast_prefill else kvindex.ClassMap())
    if device_batch:
        res = drive_device_batch(r, trace, max_active, chunk, run_steps=device_batch, time_scale=time_scale)
    else:
        res = drive(r, trace, max_active, chunk, time_scale, **kw)
    res["driver"] = (f"device batch: seats and retirement on the device, {device_batch} steps a run, prompts prefilled between runs" if device_batch
                     else "host-driven: a ragged step packed per step, prefill chunks riding the decode runs")
    res["workload"] = (f"{shape}: {n_sessions} sessions, Poisson {rate}/s seed {seed}"
                       f"{'' if time_scale == 1.0 else f' (arrival clock x{time_scale})' if time_scale > 0 else ' (all at t=0)'}, "
                       f"prompts U[{prompt_lo},{prompt_hi}]{f' sharing {n_preambles} preamble(s) of {preamble}' if preamble else ''}"
                       f"{', prefix reuse on' if prefix_reuse else ''}, outputs U[{out_lo},{out_hi}], <= {max_active} admitted, greedy, "
                       f"paged fp16 KV 16-token blocks, prefill chunks of {chunk} riding the decode runs")
    r.Close()
    return res
