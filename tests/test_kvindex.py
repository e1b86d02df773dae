"""The prefix index against the cases the reference's own tests hold for it (internal/runtime/kvmgr/key_test.go,
share_test.go, slots_test.go), plus a randomized walk against a plain record, as share_test.go's TestOracle_share does."""
import hashlib
import struct

import numpy as np
import pytest

from goinfer_b200 import kvindex as kv
from goinfer_b200.kvindex import (BLOCK_ROWS, CLASS_EXACT, CLASS_FAST, ClassMap, ClassRun, ImageSpan, MIN_LEAD_REUSE, Request,
                                  Root, SlotIndex)

CUDA = ClassMap(Floor=512, MinRows=16)
METAL = ClassMap(Floor=64, MinRows=1)
ROOT = Root(Model="m", Precision="f16")


def seq_of(n, seed):
    return [(i * 7 + seed * 13) % 101 for i in range(n)]


def commit_prompt(a, slot, root, prompt, gen, cm):
    a.Acquired(slot, 0, prompt)
    a.Forget(slot)
    a.Commit(slot, root, list(prompt) + list(gen), None, len(prompt), cm)


@pytest.mark.parametrize("rows,judged,want", [
    (1000, 1000, CLASS_FAST), (64, 1000, CLASS_FAST), (256, 256, CLASS_EXACT), (744, 1000, CLASS_FAST), (511, 511, CLASS_EXACT),
    (512, 512, CLASS_FAST), (16, 1000, CLASS_FAST), (15, 1000, CLASS_EXACT), (8, 1000, CLASS_EXACT)])
def test_class_map_arms(rows, judged, want):
    """key_test.go:10 TestClassMap_kv0Arms."""
    assert CUDA.Pass(rows, judged) == want
    assert ClassMap().Pass(4000, 4000) == CLASS_EXACT
    assert ClassMap(Floor=16).Pass(1, 40) == CLASS_FAST


@pytest.mark.parametrize("cm,prompt,reuse,want", [
    (CUDA, 941, 13, 0), (CUDA, 941, MIN_LEAD_REUSE - 1, 0), (CUDA, 941, MIN_LEAD_REUSE, MIN_LEAD_REUSE), (CUDA, 941, 900, 900),
    (CUDA, 511, 5, 5), (CUDA, 512, 5, 0), (ClassMap(), 941, 13, 13), (ClassMap(Floor=8, MinRows=16), 15, 5, 5),
    (ClassMap(Floor=8, MinRows=16), 16, 5, 0), (CUDA, 941, 0, 0)])
def test_decline_short_lead(cm, prompt, reuse, want):
    """key_test.go:39 TestDeclineShortLead."""
    assert cm.DeclineShortLead(prompt, reuse) == want


@pytest.mark.parametrize("cm,n,hit,want", [
    (CUDA, 975, 960, 896), (CUDA, 1000, 960, 960), (CUDA, 976, 960, 960), (CUDA, 300, 256, 256), (CUDA, 520, 512, 448),
    (METAL, 975, 960, 960), (ClassMap(), 975, 960, 960), (CUDA, 975, 0, 0)])
def test_cap_hit(cm, n, hit, want):
    """share_test.go:17 TestCapHit."""
    assert cm.CapHit(n, hit) == want


def test_hash_is_the_canonical_encoding():
    """The root link spelled out byte by byte (key.go:146-165): tag, block rows, length-prefixed strings, tagged parts."""
    r = Root("m", "key-a", 1, "f16")
    u = lambda v: struct.pack("<Q", v)
    want = hashlib.sha256(b"R" + u(64) + u(1) + b"m" + b"n" + u(5) + b"key-a" + b"a" + u(1) + b"p" + u(3) + b"f16").digest()
    assert kv.root_hash(r) == want
    toks = list(range(64))
    b0 = kv.block_hash(want, 0, toks, (), [ClassRun(0, 64, CLASS_FAST)])
    assert b0 == hashlib.sha256(b"B" + want + b"".join(struct.pack("<q", t) for t in toks) + b"c" + bytes([CLASS_FAST]) + u(64)).digest()


def test_block_hash_runs_do_not_matter():
    """key_test.go:66 TestBlockHash_runsDoNotMatter."""
    tokens = [i * 7 for i in range(2 * BLOCK_ROWS)]
    rh = kv.root_hash(Root(Model="m"))
    one = kv.block_hash(rh, 1, tokens, (), [ClassRun(0, 100, CLASS_FAST), ClassRun(100, 28, CLASS_EXACT)])
    two = kv.block_hash(rh, 1, tokens, (), [ClassRun(0, 64, CLASS_FAST), ClassRun(64, 36, CLASS_FAST), ClassRun(100, 10, CLASS_EXACT),
                                            ClassRun(110, 18, CLASS_EXACT)])
    assert one == two
    assert kv.block_hash(rh, 1, tokens, (), [ClassRun(0, 101, CLASS_FAST), ClassRun(101, 27, CLASS_EXACT)]) != one


@pytest.mark.parametrize("part,root,images,cold,rows", [
    ("adapter", Root("m", "key-a", 2, "f16"), None, None, 0),
    ("image", None, [ImageSpan(70, 20, 0xB0B)], None, BLOCK_ROWS),
    ("class", None, None, [ClassRun(0, 200, CLASS_FAST), ClassRun(200, 4 * BLOCK_ROWS + 1 - 200, CLASS_EXACT)], 3 * BLOCK_ROWS),
    ("precision", Root("m", "key-a", 1, "f32"), None, None, 0),
    ("namespace", Root("m", "key-b", 1, "f16"), None, None, 0)])
def test_wrong_hit(part, root, images, cold, rows):
    """key_test.go:86 TestWrongHit: a request that differs in one input of the key takes only what lies before the first
    difference; the control (the same request again) takes everything it may."""
    n = 4 * BLOCK_ROWS
    tokens = [100 + i % 9 for i in range(n + 1)]
    base = Root("m", "key-a", 1, "f16")
    img = [ImageSpan(70, 20, 0xA11CE)]
    fast = [ClassRun(0, n + 1, CLASS_FAST)]
    a = SlotIndex(2)
    a.Acquired(0, 0, tokens)
    a.Commit(0, base, tokens, img, len(tokens), ClassMap(Floor=1, MinRows=1))
    assert a.Hits(Request(base, tokens, img), fast)[0] == n
    got = a.Hits(Request(root or base, tokens, images or img), cold or fast)[0]
    assert got == rows, part


def test_hits_preamble_across_slots():
    """share_test.go:56 TestHits_preambleAcrossSlots."""
    pre = seq_of(200, 1)
    a = SlotIndex(2)
    commit_prompt(a, 0, ROOT, pre + seq_of(30, 2), seq_of(20, 3), METAL)
    b = pre + seq_of(40, 4)
    cold = METAL.ColdClasses(len(b))
    assert a.Hits(Request(ROOT, b), cold) == [192, 0]
    assert a.Hits(Request(Root("m", "key-2", 0, "f16"), b), cold)[0] == 0
    assert a.Hits(Request(ROOT, b), [ClassRun(0, len(b), CLASS_EXACT)])[0] == 0
    assert a.Hits(Request(ROOT, b, [ImageSpan(70, 10)]), cold)[0] == 64
    assert a.Hits(Request(ROOT, pre[:65]), METAL.ColdClasses(65))[0] == 64
    assert a.Hits(Request(ROOT, pre[:64]), METAL.ColdClasses(64))[0] == 0


def test_hits_image_span_boundary():
    """share_test.go:87 TestHits_imageSpanBoundary."""
    imgs = [ImageSpan(120, 20, 9)]
    prompt = seq_of(150, 5)
    a = SlotIndex(2)
    a.Acquired(0, 0, prompt)
    a.Commit(0, ROOT, prompt + seq_of(70, 6), imgs, len(prompt), METAL)
    b = prompt + seq_of(70, 6) + [1, 2, 3]
    assert a.Hits(Request(ROOT, b, imgs), METAL.ColdClasses(len(b)))[0] == 64


def test_copied():
    """share_test.go:103 TestCopied."""
    pre = seq_of(200, 1)
    a = SlotIndex(3)
    commit_prompt(a, 0, ROOT, pre + seq_of(30, 2), seq_of(20, 3), METAL)
    use0 = a.Use(0)
    a.Copied(0, 2, 0, 192)
    s = a.Seq(2)
    assert s is not None and s.Len() == 192 and s.Published() == 3 and s.tokens == pre[:192]
    assert s.classes == [ClassRun(0, 192, CLASS_FAST)]
    b = pre + seq_of(40, 4)
    assert a.Score(2, Request(ROOT, b)) == 192
    assert a.Use(0) > use0
    assert a.Hits(Request(ROOT, b), METAL.ColdClasses(len(b))) == [192, 0, 192]
    a.Forget(0)
    assert a.Hits(Request(ROOT, b), METAL.ColdClasses(len(b))) == [0, 0, 192]


def test_prefilled():
    """share_test.go:136 TestPrefilled."""
    pre = seq_of(200, 1)
    prompt_a = pre + seq_of(30, 2)
    a = SlotIndex(2)
    a.Acquired(0, 0, prompt_a)
    a.Forget(0)
    a.Prefilled(0, ROOT, prompt_a, None, METAL)
    assert a.Live(0) and a.Seq(0).Published() == 3
    b = pre + seq_of(40, 4)
    assert a.Hits(Request(ROOT, b), METAL.ColdClasses(len(b)))[0] == 192
    a.Commit(0, ROOT, prompt_a + seq_of(20, 3), None, len(prompt_a), METAL)
    assert not a.Live(0)
    c = a.Seq(0).classes
    assert len(c) == 2 and c[0] == ClassRun(0, len(prompt_a), CLASS_FAST) and c[1].Class == CLASS_EXACT
    a.Acquired(1, 0, prompt_a)
    a.Forget(1)
    a.Prefilled(1, ROOT, prompt_a, None, METAL)
    a.Forget(1)
    assert not a.Live(1) and a.Seq(1) is None


@pytest.mark.parametrize("scores,lens,uses,busy,want", [
    ([1000, 0], [1063, 0], [1, 0], None, 0), ([1000, 0], [1064, 0], [1, 0], None, 1), ([18213, 0], [20300, 0], [1, 0], None, 1),
    ([18213, 5], [20300, 900], [2, 1], None, 1), ([18213, 5], [20300, 900], [1, 2], None, 0),
    ([3, 170], [170, 172], [1, 2], None, 1), ([7, 0], [170, 0], [1, 0], None, 1), ([7, 7, 7], [200, 180, 190], [5, 2, 9], None, 1),
    ([5, 0], [10, 0], [1, 0], None, 0), ([3, 170], [170, 172], [1, 2], [False, True], 0), ([0, 0], [1, 1], [1, 2], [True, True], -1)])
def test_pick_slot(scores, lens, uses, busy, want):
    """share_test.go:169 TestPickSlot_oneBlock and slots_test.go:246 TestPickSlot."""
    assert kv.pick_slot_within(scores, lens, uses, busy) == want


def test_windowed_unaligned_fast_rows_and_unclaimed_images():
    """share_test.go:309, :326."""
    cm = ClassMap(Floor=64, MinRows=1, Windowed=True)
    toks = seq_of(320, 8)
    a = SlotIndex(2)
    commit_prompt(a, 0, ROOT, toks[:100], [], cm)
    a.Acquired(0, 100, toks[:300])
    a.Forget(0)
    a.Commit(0, ROOT, toks[:300], None, 300, cm)
    b = toks[:310]
    assert a.Hits(Request(ROOT, b), cm.ColdClasses(len(b)))[0] == 64
    toks = seq_of(260, 9)
    img = [ImageSpan(70, 10)]
    a = SlotIndex(2)
    a.Acquired(0, 0, toks[:250])
    a.Commit(0, ROOT, toks[:250], img, 250, METAL)
    assert a.Hits(Request(ROOT, toks, img), METAL.ColdClasses(len(toks)))[0] == 64
    named = [ImageSpan(70, 10, 7)]
    a.Acquired(1, 0, toks[:250])
    a.Commit(1, ROOT, toks[:250], named, 250, METAL)
    assert a.Hits(Request(ROOT, toks, named), METAL.ColdClasses(len(toks)))[1] == 192


def test_floor():
    """slots_test.go:297 TestSlots_floor, the part that needs no snapshot restore."""
    toks = list(range(1, 4 * BLOCK_ROWS + 1))
    short, long_ = Request(ROOT, toks[:BLOCK_ROWS] + [-1]), Request(ROOT, toks + [-1])
    a = SlotIndex(3)
    commit_prompt(a, 0, ROOT, toks, [], METAL)
    hit = lambda req, s: a.Hits(req, METAL.ColdClasses(len(req.Tokens)))[s]
    assert a.Score(0, short) == BLOCK_ROWS and hit(short, 0) == BLOCK_ROWS
    a.SetFloor(0, 2 * BLOCK_ROWS)
    assert a.Score(0, short) == 0 and hit(short, 0) == 0 and a.Score(0, long_) == len(toks)
    a.Commit(0, ROOT, toks, None, len(toks), METAL)
    assert a.Score(0, short) == 0
    a.Copied(0, 1, 0, len(toks))
    assert a.Score(1, short) == 0 and a.Score(1, long_) == len(toks)


@pytest.mark.parametrize("cm", [METAL, ClassMap(Floor=96, MinRows=16)])
@pytest.mark.parametrize("seed", range(1, 7))
def test_random_walk_against_a_plain_record(cm, seed):
    """Commits, prefill-end publishes, copies and forgets at random; after each, Hits equals hits computed from a plain
    record of (root, tokens, row classes) per slot by comparing rows directly (share_test.go:191 TestOracle_share)."""
    rng = np.random.default_rng(seed)
    roots = [ROOT, Root("m", "k2", 0, "f16")]
    n = int(2 + rng.integers(0, 3))
    a = SlotIndex(n)
    rec = [None] * n
    pre = [seq_of(int(rng.integers(70, 300)), 40 + i) for i in range(3)]

    def row_classes(prompt_len, total):
        c = cm.PassAt(0, prompt_len, prompt_len)
        return [c] * prompt_len + [CLASS_EXACT] * (total - prompt_len)

    def plain_hits(root, tokens):
        cold = cm.PassAt(0, len(tokens), len(tokens))
        out = []
        for r in rec:
            k = 0
            if r is not None and r[0] == root:
                limit = (len(tokens) - 1) // BLOCK_ROWS
                while k < limit and (k + 1) * BLOCK_ROWS <= len(r[1]) and \
                        r[1][k * BLOCK_ROWS:(k + 1) * BLOCK_ROWS] == list(tokens[k * BLOCK_ROWS:(k + 1) * BLOCK_ROWS]) and \
                        all(c == cold for c in r[2][k * BLOCK_ROWS:(k + 1) * BLOCK_ROWS]):
                    k += 1
            out.append(k * BLOCK_ROWS)
        return out

    for _ in range(60):
        op = int(rng.integers(0, 4))
        sl = int(rng.integers(0, n))
        root = roots[int(rng.integers(0, 2))]
        prompt = pre[int(rng.integers(0, 3))][:int(rng.integers(40, 300))] + seq_of(int(rng.integers(1, 80)), int(rng.integers(0, 50)))
        if op == 0:
            gen = seq_of(int(rng.integers(0, 90)), 7)
            commit_prompt(a, sl, root, prompt, gen, cm)
            rec[sl] = (root, prompt + gen, row_classes(len(prompt), len(prompt) + len(gen)))
        elif op == 1:
            a.Acquired(sl, 0, prompt)
            a.Forget(sl)
            a.Prefilled(sl, root, prompt, None, cm)
            rec[sl] = (root, list(prompt), row_classes(len(prompt), len(prompt)))
        elif op == 2:
            src = int(rng.integers(0, n))
            if src != sl and rec[src] is not None:
                rows = int(rng.integers(0, len(rec[src][1]) // BLOCK_ROWS + 1)) * BLOCK_ROWS
                a.Copied(src, sl, 0, rows)
                rec[sl] = (rec[src][0], rec[src][1][:rows], rec[src][2][:rows]) if rows > 0 else None
        else:
            a.Forget(sl)
            rec[sl] = None
        for r_ in roots:
            q = pre[int(rng.integers(0, 3))][:int(rng.integers(40, 300))] + seq_of(int(rng.integers(1, 80)), 3)
            assert a.Hits(Request(r_, q), cm.ColdClasses(len(q))) == plain_hits(r_, q)
        for s_ in range(n):
            want = 0 if rec[s_] is None else len(rec[s_][1])
            assert a.Len(s_) == want


def test_plan_reuse_picks_the_longest_capped_hit():
    pre = seq_of(700, 1)
    a = SlotIndex(3)
    commit_prompt(a, 0, ROOT, pre[:300] + seq_of(300, 5), [], CUDA)     # shares 300 rows of the preamble (4 blocks)
    commit_prompt(a, 1, ROOT, pre + seq_of(30, 2), seq_of(5, 3), CUDA)  # shares all 700 (10 blocks)
    req = Request(ROOT, pre + seq_of(9, 9))                             # 709 tokens: after a 640-row hit 69 rows remain: fast
    assert kv.plan_reuse(a, req, CUDA) == (1, 640)
    req = Request(ROOT, pre[:648] + [1, 2])                             # 650 tokens: 640 would leave 10 rows (exact): one block back
    assert kv.plan_reuse(a, req, CUDA) == (1, 576)
    assert kv.plan_reuse(a, Request(Root("other"), pre + [1]), CUDA) == (-1, 0)
