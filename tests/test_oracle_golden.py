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
