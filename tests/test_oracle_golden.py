"""Pins the CPU oracle against the golden vectors the reference's own tests hold for this path
(decoder/llama_tiny_test.go:22-80 over testdata/llama_tiny_text_golden.json; decoder/qwen3moe_test.go over
testdata/qwen3moe_forward_golden.json), with f32 weights and an f32 cache as the goldens were made."""
import numpy as np

from goinfer_b200.resident import BatchDraw, RaggedPrefill, RaggedSeq
from helpers import cfg_from_hf, load_golden, upload_hf


def _oracle(oracle_lib, name, **kw):
    hf, w, g = load_golden(name)
    r = oracle_lib.OracleResident(cfg_from_hf(hf, kv_dtype=1, **kw))
    upload_hf(r, hf, w)
    r.finalize()
    return r, g


def test_llama_tiny_prefill_and_greedy_continuation(oracle_lib):
    r, g = _oracle(oracle_lib, "llama_tiny")
    ids = g["prompt_ids"].tolist()
    logits = r.PrefillLast(None, 0, slot=0, tokens=ids)
    assert int(np.argmax(logits)) == int(g["argmax"])
    np.testing.assert_allclose(logits, g["last_logits"], atol=2e-5, rtol=1e-4)
    # greedy continuation: argmax of the prefill, then 5 decode steps
    out, tok, pos = [int(g["argmax"])], int(g["argmax"]), len(ids)
    for _ in range(len(g["continuation_ids"]) - 1):
        tok = r.ForwardArgmax(None, pos, slot=0, token=tok)
        out.append(tok)
        pos += 1
    assert out == g["continuation_ids"].tolist()


def test_llama_tiny_token_by_token_equals_prefill(oracle_lib):
    """Batched rows equal sequential forwards (decoder/forwardn_test.go:109 TestForwardN_matchesSequential)."""
    r, g = _oracle(oracle_lib, "llama_tiny")
    ids = g["prompt_ids"].tolist()
    a = r.PrefillLast(None, 0, slot=0, tokens=ids)
    for p, t in enumerate(ids):
        b = r.Forward(None, p, slot=1, token=t)
    assert np.array_equal(a, b)


def test_llama_tiny_ragged_rows_match_their_own_forward(oracle_lib):
    """StepRagged: a prefill chunk riding with decode rows; every row equals its own sequence's pass
    (backend/cuda/batchstep_test.go:289 TestCUDAStepRagged_rowsMatchTheirShapes)."""
    r, g = _oracle(oracle_lib, "llama_tiny", n_slots=4)
    ids = g["prompt_ids"].tolist()
    solo = r.PrefillLast(None, 0, slot=0, tokens=ids)
    r.PrefillLast(None, 0, slot=1, tokens=ids[:5])
    # decode row on slot 1 (position 5) rides with slot 3's whole prompt as a Last prefill chunk
    out = r.StepRagged([
        RaggedSeq(3, 0, None, ids, None, RaggedPrefill(len(ids), True)),
        RaggedSeq(1, 5, None, [ids[5]], BatchDraw(Greedy=True)),
    ])
    assert out[0].Logits[:-1] == [None] * (len(ids) - 1)
    assert np.array_equal(out[0].Logits[-1], solo)
    r.PrefillLast(None, 0, slot=2, tokens=ids[:5])
    assert out[1].ID == r.ForwardArgmax(None, 5, slot=2, token=ids[5])


def test_qwen3moe_tiny_forward(oracle_lib):
    r, g = _oracle(oracle_lib, "qwen3moe_tiny")
    logits = r.PrefillLast(None, 0, slot=0, tokens=g["ids"].tolist())
    assert int(np.argmax(logits)) == int(g["argmax"])
    np.testing.assert_allclose(logits[g["top_k_ids"]], g["top_k_logits"], atol=2e-5, rtol=1e-4)
    np.testing.assert_allclose(logits[g["sample_ids"]], g["sample_logits"], atol=2e-5, rtol=1e-4)
    n, s, ss, mn, mx = g["stats"]
    assert len(logits) == int(n)
    np.testing.assert_allclose([logits.sum(dtype=np.float64), (logits.astype(np.float64) ** 2).sum(), logits.min(), logits.max()],
                               [s, ss, mn, mx], atol=1e-4, rtol=1e-4)


def test_philox_known_answers_and_gumbel_draw(oracle_lib):
    """The oracle's Philox4x32-10 against the Random123 known-answer vectors the reference pins every backend to
    (internal/runtime/sampling/philox_test.go:9-23), and the host Gumbel-max draw's rules (sampler_gumbel.go:52-64,
    104-110): ties to the lowest index, the plain argmax when nothing is comparable, an exact draw from softmax(l/T)."""
    from goinfer_b200 import abi
    kats = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
            ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
            ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    got = oracle_lib.op_philox(np.array([k[0] for k in kats], np.uint32), np.array([k[1] for k in kats], np.uint32))
    assert got.tolist() == [list(k[2]) for k in kats]
    # all -inf: nothing comparable -> the plain argmax (index 0); an isolated finite entry always wins
    row = np.full(37, -np.inf, np.float32)
    assert oracle_lib.op_draw(row[None], [abi.gumbel_draw(0.8, 5, 0)])[0] == 0
    row[11] = -3.0
    assert oracle_lib.op_draw(row[None], [abi.gumbel_draw(0.8, 5, 1)])[0] == 11
    # the draw index and the seed both move the stream; the same (seed, draw) repeats
    lg = np.random.default_rng(0).normal(0, 1, (1, 1000)).astype(np.float32)
    a = [int(oracle_lib.op_draw(lg, [abi.gumbel_draw(1.0, 7, d)])[0]) for d in range(40)]
    assert a == [int(oracle_lib.op_draw(lg, [abi.gumbel_draw(1.0, 7, d)])[0]) for d in range(40)] and len(set(a)) > 10
    assert a != [int(oracle_lib.op_draw(lg, [abi.gumbel_draw(1.0, 8, d)])[0]) for d in range(40)]
    # Gumbel-max is an exact draw from softmax(l/T): frequencies over 20000 draws of an 8-entry row
    l8 = np.array([[2.0, 1.0, 0.5, 0.0, -0.5, -1.0, -2.0, 1.5]], np.float32)
    T = 0.7
    p = np.exp(l8[0].astype(np.float64) / T)
    p /= p.sum()
    n = 20000
    ids = oracle_lib.op_draw(np.repeat(l8, n, axis=0), [abi.gumbel_draw(T, 1234, d) for d in range(n)])
    freq = np.bincount(ids, minlength=8) / n
    assert np.abs(freq - p).max() < 4 * np.sqrt(p.max() * (1 - p.max()) / n) + 2e-3


def test_prefix_reuse_on_the_golden_model(oracle_lib):
    """A slot that takes another's prefix by CopyKV continues exactly like the slot that prefilled it, whole blocks are
    shared and come back only with their last reference, and a write into a shared block goes to a private copy
    (backend/cuda/kvpool.go:16-27 refcounts and copy-on-write, :436-536 the table append and copy paths)."""
    r, g = _oracle(oracle_lib, "llama_tiny", n_slots=4, kv_block_rows=4)
    ids = g["prompt_ids"].tolist()
    n = len(ids)
    solo = r.PrefillLast(None, 0, slot=0, tokens=ids)
    assert int(np.argmax(solo)) == int(g["argmax"])
    free0 = r.FreeBlocks()
    keep = n - 1                                            # all but the last row: the taker feeds that row itself
    r.CopyKV(1, 0, keep)
    whole, tail = keep // 4, keep % 4
    assert free0 - r.FreeBlocks() == (1 if tail else 0)     # shared blocks cost nothing, the copied tail one block
    t0, t1 = r.BlockTable(0), r.BlockTable(1)
    assert t1[:whole].tolist() == t0[:whole].tolist()
    if tail:
        assert t1[whole] not in (0, t0[whole])
    again = r.Forward(None, keep, slot=1, token=ids[keep])
    assert np.array_equal(again, solo)
    # the golden continuation from the shared prefix
    tok, pos, out = int(g["argmax"]), n, [int(g["argmax"])]
    for _ in range(len(g["continuation_ids"]) - 1):
        tok = r.ForwardArgmax(None, pos, slot=1, token=tok)
        out.append(tok)
        pos += 1
    assert out == g["continuation_ids"].tolist()
    # slot 2 shares a whole first block, then rewrites inside it: the source must not see the write
    r.CopyKV(2, 0, 4)
    assert r.BlockTable(2)[0] == t0[0]
    f = r.FreeBlocks()
    r.Forward(None, 2, slot=2, token=ids[0])
    assert r.BlockTable(2)[0] != t0[0] and r.FreeBlocks() == f - 1
    assert np.array_equal(r.Forward(None, n - 1, slot=0, token=ids[n - 1]), solo)
    # the source lets go first: only blocks nobody else names come back
    shared_with_1 = whole
    own0 = int((r.BlockTable(0) != 0).sum())
    f = r.FreeBlocks()
    r.ResetSlot(0)
    assert r.FreeBlocks() == f + own0 - shared_with_1
    assert np.array_equal(r.Forward(None, keep, slot=1, token=ids[keep]), solo)   # rewriting its own private row: same result
    r.ResetSlot(1)
    r.ResetSlot(2)
    assert r.FreeBlocks() == free0 + own0
