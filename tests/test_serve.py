"""Host logic either side of the ragged step (no GPU): admission, placement, chunk planning, the batcher's run / ride /
pool-full behaviour and the Poisson driver, against a fake resident. Cases follow the reference's own tests of these parts
(internal/runtime/scheduler/admission_test.go, placement_test.go; decoder/mc3_batch_test.go)."""
import numpy as np
import pytest

from goinfer_b200 import serve
from goinfer_b200.resident import BatchOut, ErrKVPoolFull, RaggedOut


def test_admission_is_fifo_and_hands_the_turn_over():
    a = serve.Admission()                       # the zero value admits one
    recs = [serve.Record(str(i)) for i in range(4)]
    assert a.Enter(recs[0]) and not a.Enter(recs[1]) and not a.Enter(recs[2])
    assert a.Load() == 3 and a.Capacity() == 1
    assert a.Position("2") == (2, 2, True, True)
    assert a.Position("0") == (0, 2, True, False)      # granted: no longer a waiter
    assert a.Position("") == (0, 0, False, False)
    # a release with waiters queued is a hand-off: the newcomer still queues behind them
    assert a.Release() is recs[1]
    assert not a.Enter(recs[3])
    assert a.Cancel(recs[2]) and not a.Cancel(recs[2])  # a waiter whose context ended leaves its place
    assert a.Release() is recs[3]
    assert a.Release() is None and a.Load() == 0
    assert a.Enter(recs[0])


def test_admission_capacity():
    a = serve.Admission(3)
    granted = [a.Enter(serve.Record(str(i))) for i in range(5)]
    assert granted == [True, True, True, False, False]
    a.SetCap(0)
    assert a.Capacity() == 1                    # at least one
    assert a.Release().ID == "3" and a.Release().ID == "4"
    assert a.Release() is None and a.Release() is None and a.Release() is None
    assert a.Load() == 0


def test_placement():
    s = [[1, 2, 3, 4, 5], [1, 2, 9], [7, 7]]
    assert serve.common_prefix([1, 2, 3], [1, 2, 4, 5]) == 2
    assert serve.best_extend(s, [1, 2, 3, 4, 5, 6]) == 0        # an exact continuation qualifies
    assert serve.best_extend(s, [1, 2, 8]) == -1                # the preamble two sessions share does not
    assert serve.best_extend(s, [1, 2, 9, 9]) == 1
    assert serve.best_extend(s, [5]) == -1
    assert serve.best_extend([None, [3, 4]], [3, 4, 5]) == 1    # a held session has no tokens to read
    # the room rule: with a spare slot, a request that keeps less than it overwrites starts fresh ...
    assert serve.pick_session([[1, 2, 3, 4, 5, 6, 7, 8]], [0], [1, 2, 3, 9], True) == -1
    assert serve.pick_session([[1, 2, 3, 4, 5, 6, 7, 8]], [0], [1, 2, 3, 9], False) == 0
    # ... unless it keeps the conversation's whole first prompt (a roll-back)
    assert serve.pick_session([[1, 2, 3, 4, 5, 6, 7, 8]], [3], [1, 2, 3, 9], True) == 0
    assert serve.keeps_first(0, 10) is False
    assert serve.coldest_idle([True, False, False, True]) == 2 and serve.coldest_idle([True, True]) == -1
    assert serve.pick_donor([4, 9, 9, 0], [False, True, False]) == (2, 9)
    assert serve.pick_donor([4, 4], None) == (1, 4)             # equal hits: the least recently used
    assert serve.pick_donor([0, 0], None) == (-1, 0)


@pytest.mark.parametrize("n,chunk,want", [(0, 512, []), (300, 512, [300]), (512, 512, [512]), (513, 512, [505, 8]),
                                          (1024, 512, [512, 512]), (1030, 512, [512, 510, 8]), (1100, 512, [512, 512, 76]),
                                          (40, 0, [40])])
def test_chunk_plan_keeps_the_tail(n, chunk, want):
    got = serve.chunk_plan(n, chunk)
    assert got == want and sum(got) == n
    assert all(p <= chunk for p in got) or chunk <= 0
    assert not got or len(got) == 1 or got[-1] >= serve.PREFILL_TAIL_MIN


class FakeResident:
    """Greedy id of a row = (token fed + position) % 97; records the steps it was given."""

    def __init__(self, slots=8, lo=2, fail_pool_when=None):
        self.slots, self.lo, self.steps, self.resets = slots, lo, [], []
        self.fail_pool_when = fail_pool_when

    def BatchStepRange(self):
        return (self.lo, self.slots)

    def KVSlots(self):
        return self.slots

    def ResetSlot(self, slot):
        self.resets.append(slot)

    def StepBatch(self, seqs):
        self.steps.append(("batch", [(q.Slot, q.Pos, q.Token) for q in seqs]))
        if self.fail_pool_when and self.fail_pool_when(seqs):
            raise ErrKVPoolFull(2, "pool full")
        return [BatchOut(None, (q.Token + q.Pos) % 97) for q in seqs]

    def StepRagged(self, seqs):
        self.steps.append(("ragged", [(q.Slot, q.Pos, len(q.Tokens), bool(q.Prefill and q.Prefill.Last)) for q in seqs]))
        assert seqs[0].Prefill is not None and all(q.Prefill is None for q in seqs[1:])
        outs = []
        for q in seqs:
            if q.Prefill:
                lg = None
                if q.Prefill.Last:
                    lg = np.zeros(97, np.float32)
                    lg[(int(q.Tokens[-1]) + q.Pos + len(q.Tokens) - 1) % 97] = 1.0
                outs.append(RaggedOut([None] * (len(q.Tokens) - 1) + [lg], -1))
            else:
                outs.append(RaggedOut([None], (q.Tokens[0] + q.Pos) % 97))
        return outs


def test_batcher_run_step_solo_and_pool_full():
    from goinfer_b200.resident import BatchDraw, BatchSeq
    g = BatchDraw(Greedy=True)
    r = FakeResident(slots=8, lo=3)
    b = serve.Batcher(r, 6)
    assert (b.lo, b.hi, b.max_holders) == (3, 8, 6)
    outs = b.run_tokens([BatchSeq(i, 10 + i, None, i, g) for i in range(4)])
    assert [o.ID for o, e in outs] == [(i + 10 + i) % 97 for i in range(4)] and all(e is None for _, e in outs)
    assert (b.stats.Runs, b.stats.Steps, b.stats.StepTokens, b.stats.SoloTokens, b.stats.StepSizes[4]) == (1, 1, 4, 0, 1)
    # fewer than lo tokens: each through its own call
    b.run_tokens([BatchSeq(0, 1, None, 5, g), BatchSeq(1, 2, None, 6, g)])
    assert b.stats.SoloTokens == 2 and b.stats.Steps == 1 and [k for k, _ in r.steps[-2:]] == ["batch", "batch"]
    assert all(len(s) == 1 for _, s in r.steps[-2:])
    # a step refused for a full pool wrote nothing: every token re-runs solo, only the starved row ends
    r2 = FakeResident(slots=8, lo=2, fail_pool_when=lambda seqs: any(q.Slot == 2 for q in seqs))
    b2 = serve.Batcher(r2, 8)
    outs = b2.run_tokens([BatchSeq(i, 3, None, 1, g) for i in range(4)])
    assert [e is None for _, e in outs] == [True, True, False, True]
    assert isinstance(outs[2][1], ErrKVPoolFull) and b2.stats.SoloTokens == 4 and b2.stats.Steps == 0


def test_drive_serves_a_trace_with_chunks_riding_runs():
    vocab = 97
    trace = serve.poisson_trace(12, 40.0, 1, 5, 40, 2, 9, vocab)
    assert trace == sorted(trace, key=lambda s: s.arrival)
    r = FakeResident(slots=4, lo=2)
    t = [0.0]
    clock = lambda: t[0]
    def sleep(d):
        t[0] += d
    # every step of the fake costs 1 ms of the fake clock
    orig_b, orig_r = r.StepBatch, r.StepRagged
    def sb(seqs):
        t[0] += 1e-3
        return orig_b(seqs)
    def sr(seqs):
        t[0] += 1e-3
        return orig_r(seqs)
    r.StepBatch, r.StepRagged = sb, sr
    res = serve.drive(r, trace, max_active=4, chunk=16, clock=clock, sleep=sleep)
    assert res["sessions"] == 12
    assert res["output_tokens"] == sum(s.out_len for s in trace)
    assert res["prompt_tokens"] == sum(len(s.prompt) for s in trace)
    assert sorted(r.resets) == sorted(s.slot for s in trace) and len(r.resets) == 12
    # never more than max_active sequences in a step, a chunk always first, chunks within 16 rows and tails >= 8 rows
    for kind, seqs in r.steps:
        assert len(seqs) <= 5
        if kind == "ragged":
            assert seqs[0][2] <= 16
    for s in trace:
        plan = serve.chunk_plan(len(s.prompt), 16)
        assert len(plan) == 1 or plan[-1] >= 8
    # greedy ids follow the fake's rule: each generation is a deterministic chain from its prompt
    for s in trace:
        tok = (int(s.prompt[-1]) + len(s.prompt) - 1) % vocab
        for k in range(1, s.out_len):
            tok = (tok + len(s.prompt) + k - 1) % vocab
        assert s.last_id == tok and s.generated == s.out_len
    assert res["batch_stats"]["RidePasses"] >= 12 and res["batch_stats"]["StragglerRuns"] == 0
    # all at once (closed loop): the same tokens, admission in FIFO order
    r3 = FakeResident(slots=4, lo=2)
    trace3 = serve.poisson_trace(12, 40.0, 1, 5, 40, 2, 9, vocab)
    res3 = serve.drive(r3, trace3, max_active=4, chunk=16, time_scale=0.0)
    assert res3["output_tokens"] == res["output_tokens"]
    assert [s.last_id for s in trace3] == [s.last_id for s in trace]
    first_steps = [seqs[0][0] for kind, seqs in r3.steps if kind == "ragged"][:4]
    assert first_steps[0] == trace3[0].slot


def test_drive_with_the_prefix_index_takes_shared_preambles_by_copy():
    """Prompts sharing a 200-token preamble: after the first one finishes its prefill the others take its three whole
    64-row blocks by CopyKV (or keep them in place when they inherit the slot) and prefill only the rest; the ids are the
    ones the same trace draws without reuse."""
    from goinfer_b200 import kvindex
    vocab = 97
    mk = lambda: serve.poisson_trace(10, 40.0, 3, 230, 300, 2, 6, vocab, preamble=200)
    base = mk()
    r0 = FakeResident(slots=3, lo=2)
    serve.drive(r0, base, max_active=3, chunk=64, time_scale=0.0)
    trace = mk()
    assert all(np.array_equal(a.prompt[:200], trace[0].prompt[:200]) for a in trace)
    r = FakeResident(slots=3, lo=2)
    r.copies = []
    r.CopyKV = lambda dst, src, n: r.copies.append((dst, src, n))
    # arrivals 25 ms apart on a clock where a step costs 1 ms: the second and third prompts find empty slots and a donor
    t = [0.0]
    def sleep(d):
        t[0] += d
    ob, orr = r.StepBatch, r.StepRagged
    def sb(seqs):
        t[0] += 1e-3
        return ob(seqs)
    def sr(seqs):
        t[0] += 1e-3
        return orr(seqs)
    r.StepBatch, r.StepRagged = sb, sr
    res = serve.drive(r, trace, max_active=3, chunk=64, clock=lambda: t[0], sleep=sleep, index=kvindex.SlotIndex(3),
                      root=kvindex.Root("m", Precision="f16"), class_map=kvindex.ClassMap())
    assert res["sessions"] == 10 and [s.last_id for s in trace] == [s.last_id for s in base]
    pr = res["prefix_reuse"]
    assert pr["copies"] + pr["in_place"] >= 7 and pr["copies"] == len(r.copies) >= 1
    assert all(n == 192 and dst != src for dst, src, n in r.copies)
    assert pr["rows_reused"] + pr["rows_prefilled"] == res["prompt_tokens"]
    assert pr["rows_reused"] >= 7 * 192
    # a session that took rows starts its prefill where they end
    for s in trace:
        if s.reused:
            first = next(q for k, seqs in r.steps if k == "ragged" for q in seqs[:1] if q[0] == s.slot and q[1] >= s.reused)
            assert first[1] == s.reused or first[1] > s.reused


def test_admission_gate_is_a_pure_function_of_the_facts():
    """decoder/admit.go:35-76: the order of the refusals, the name the Q4_K gate accepts, the activation-group gate."""
    from goinfer_b200 import admit
    ok = admit.admit(admit.AdmitFacts())
    assert ok.Why == "" and ok.Shape == "" and ok.Gates == []
    assert "does not implement residency" in admit.admit(admit.AdmitFacts(Residency=False, Backend="b200")).Why
    # q4k is admitted by backend name: a shim registered under another name is refused before anything else is read
    why = admit.admit(admit.AdmitFacts(Backend="b200", Shape="recurrent block")).Why
    assert why == "--quant q4k (native Q4_K) has no resident kernel on b200 yet"
    assert admit.admit(admit.AdmitFacts(Shape="recurrent block")).Why == "arch is not eligible for the resident decode runner: recurrent block"
    assert admit.admit(admit.AdmitFacts(Gates=["router wider than 512 experts", "x"])).Why == "router wider than 512 experts"
    assert admit.admit(admit.AdmitFacts(ActGroup=64)).Why == ""                    # CUDA residency honours any group
    assert "ActQuantGroup 64" in admit.admit(admit.AdmitFacts(Backend="webgpu", QuantLabel="int8", ActGroup=64)).Why
    assert admit.admit(admit.AdmitFacts(Backend="webgpu", QuantLabel="int8", ActGroup=0)).Why == ""
    assert admit.admit_act_safe(admit.AdmitFacts()) and not admit.admit_act_safe(admit.AdmitFacts(ProjsInt4=True))
    assert not admit.admit_act_safe(admit.AdmitFacts(ActGroup=0))
    assert admit.admit_act_safe(admit.AdmitFacts(Backend="metal")) and not admit.admit_act_safe(admit.AdmitFacts(Backend="metal", QuantLabel="int8"))
