"""Q5_K / Q6_K on the host: the oracle's dequantizers against an independent NumPy restatement of the GGUF formats and a
hand-built block, the f64 matmul reference with the planted misreadings the reference's kernel test uses
(backend/cuda/kernels/kso1c_kernels_test.go:40-104,153-175), the synthetic quantizers, and the GGUF reader."""
import struct

import numpy as np
import pytest

from goinfer_b200 import abi, gguf, kquants, q4k, synth


def random_blocks(rng, kind, rows, cols):
    """Random bytes with sane f16 scales, as the reference's ksA1Blocks makes them (ks_a1_test.go:134-150)."""
    bs = kquants.block_bytes(kind)
    raw = rng.integers(0, 256, (rows * cols // 256, bs), dtype=np.uint8)
    h = lambda n: rng.uniform(0.001, 0.05, n).astype(np.float16).view(np.uint8).reshape(n, 2)
    n = raw.shape[0]
    if kind == abi.K_Q6K:
        raw[:, 208:210] = h(n)
    else:
        raw[:, 0:2] = h(n)
        raw[:, 2:4] = h(n)
    return raw.reshape(-1)


@pytest.mark.parametrize("kind", [abi.K_Q5K, abi.K_Q6K])
def test_oracle_dequant_equals_the_format(oracle_lib, kind):
    rng = np.random.default_rng(5)
    rows, cols = 7, 768
    raw = random_blocks(rng, kind, rows, cols)
    got = oracle_lib.op_kq_dequant(kind, raw, rows, cols)
    want = kquants.dequantize(kind, raw, rows, cols)
    np.testing.assert_allclose(got, want, rtol=1e-13, atol=0)


def test_hand_built_blocks(oracle_lib):
    """One block of each kind written field by field: every weight's value follows from the format by hand."""
    # Q6_K: d = 0.5, sub-scale of half-group h is h - 8, code of element e is (e * 7) % 64
    b = np.zeros(210, np.uint8)
    codes = (np.arange(256) * 7) % 64
    for n in range(2):
        for l in range(32):
            c = [codes[128 * n + 32 * g + l] for g in range(4)]
            b[64 * n + l] = (c[0] & 15) | ((c[2] & 15) << 4)
            b[64 * n + 32 + l] = (c[1] & 15) | ((c[3] & 15) << 4)
            b[128 + 32 * n + l] = (c[0] >> 4) | ((c[1] >> 4) << 2) | ((c[2] >> 4) << 4) | ((c[3] >> 4) << 6)
    b[192:208] = (np.arange(16) - 8).astype(np.int8).view(np.uint8)
    b[208:210] = np.array([0.5], np.float16).view(np.uint8)
    want = 0.5 * (np.arange(256) // 16 - 8) * (codes - 32)
    np.testing.assert_array_equal(oracle_lib.op_kq_dequant(abi.K_Q6K, b, 1, 256)[0], want)
    np.testing.assert_array_equal(kquants.q6k_dequantize(b, 1, 256)[0], want)
    # Q5_K: d = 0.25, dmin = 0.125, sub-block j has scale j + 1 and minimum 2j, code of element e is (e * 5) % 32
    sc, mn = np.arange(8) + 1, 2 * np.arange(8)
    codes = (np.arange(256) * 5) % 32
    b = np.zeros(176, np.uint8)
    b[0:16] = q4k.pack(np.array(0.25, np.float16), np.array(0.125, np.float16), sc, mn, np.zeros(256, np.uint8))[0:16]
    for l in range(32):
        b[16 + l] = sum(((codes[32 * j + l] >> 4) & 1) << j for j in range(8))
    for p in range(4):
        for l in range(32):
            b[48 + 32 * p + l] = (codes[64 * p + l] & 15) | ((codes[64 * p + 32 + l] & 15) << 4)
    want = 0.25 * sc[np.arange(256) // 32] * codes - 0.125 * mn[np.arange(256) // 32]
    np.testing.assert_array_equal(oracle_lib.op_kq_dequant(abi.K_Q5K, b, 1, 256)[0], want)
    np.testing.assert_array_equal(kquants.q5k_dequantize(b, 1, 256)[0], want)


@pytest.mark.parametrize("kind", [abi.K_Q5K, abi.K_Q6K])
def test_matmul_reference_and_plants(oracle_lib, kind):
    rng = np.random.default_rng(11)
    N, K, M = 13, 512, 3
    raw = random_blocks(rng, kind, N, K)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    a[0, 5] = 40.0   # an outlier, as the reference's test vectors have
    got, bar = oracle_lib.op_kq_matmul_f64(kind, raw, a, N)
    codes, scales = oracle_lib.op_quant_g32(a)
    act = codes.astype(np.float64) * np.repeat(scales[:, :K // 32].astype(np.float64), 32, axis=1)
    w = kquants.dequantize(kind, raw, N, K)
    np.testing.assert_allclose(got, act @ w.T, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(bar, np.abs(act)[:, None, :].__mul__(np.abs(w)[None]).sum(-1), rtol=1e-10)
    for plant in ((1, 4) if kind == abi.K_Q5K else (2, 3, 4)):
        bad, _ = oracle_lib.op_kq_matmul_f64(kind, raw, a, N, plant)
        assert np.max(np.abs(bad - got) / bar) > 1e-5, plant


@pytest.mark.parametrize("kind,levels", [(abi.K_Q5K, 31), (abi.K_Q6K, 63)])
def test_quantizers_round_trip(kind, levels):
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (5, 1024)).astype(np.float32)
    raw = kquants.q5k_quantize(w) if kind == abi.K_Q5K else kquants.q6k_quantize(w)
    assert raw.size == 5 * 4 * kquants.block_bytes(kind)
    back = kquants.dequantize(kind, raw, 5, 1024)
    # within about a code step of the sub-block's range (the 6-bit block scales add their own rounding)
    step = (np.abs(w).reshape(5, -1, 16).max(-1).repeat(16, -1).reshape(5, 1024) * 2 + 1e-9) / levels
    assert np.all(np.abs(back - w) <= 1.6 * step)
    assert np.abs(back - w).mean() < 0.35 * step.mean()


def test_oracle_model_with_mixed_kinds_runs_and_differs_from_q4k_only(oracle_lib):
    s = synth.SHAPES["tiny-dense"]
    mk = lambda: oracle_lib.OracleResident(synth.make_cfg(s, 2, 64, 16, 0, 0, abi.CLASS_EXACT, 0))
    a, b = mk(), mk()
    synth.load_host_weights([a], s, 4, kinds=synth.Q4_K_M_KINDS)
    synth.load_host_weights([b], s, 4)
    a.finalize(); b.finalize()
    toks = list(range(3, 20))
    la, lb = a.PrefillLast(None, 0, 0, toks), b.PrefillLast(None, 0, 0, toks)
    assert np.all(np.isfinite(la)) and la.shape == lb.shape == (s.vocab,)
    assert not np.array_equal(la, lb)
    # the mixed model is close to the float model its weights were quantized from: same argmax region
    assert np.corrcoef(la, lb)[0, 1] > 0.9


def test_int8_rows_oracle_and_model(oracle_lib):
    """W8A8: the oracle's product is the f64 sum of code_w * scale_row * code_a * scale_group; a model with an int8 embedding
    table, head and o projection runs and gathers code * scale rows."""
    rng = np.random.default_rng(8)
    N, K, M = 11, 96, 3
    w = rng.normal(0, 0.05, (N, K)).astype(np.float32)
    raw = kquants.i8_quantize(w)
    assert raw.size == N * K + N * 4
    back = kquants.i8_dequantize(raw, N, K)
    assert np.abs(back - w).max() <= np.abs(w).max(axis=1).max() / 127 * 0.5001
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    got, bar = oracle_lib.op_kq_matmul_f64(abi.K_I8, raw, a, N)
    codes, scales = oracle_lib.op_quant_g32(a)
    act = codes.astype(np.float64) * np.repeat(scales[:, :K // 32].astype(np.float64), 32, axis=1)
    np.testing.assert_allclose(got, act @ back.T, rtol=1e-12, atol=1e-14)
    s = synth.SHAPES["tiny-dense"]
    r = oracle_lib.OracleResident(synth.make_cfg(s, 2, 64, 16, 0, 0, abi.CLASS_EXACT, 0))
    synth.load_host_weights([r], s, 4, kinds=synth.W8A8_KINDS)
    r.finalize()
    lg = r.PrefillLast(None, 0, 0, list(range(3, 12)))
    assert np.all(np.isfinite(lg)) and lg.std() > 0


def _tiny_gguf(tmp_path, arch, kinds, seed=6, permute=False):
    """A GGUF file of the tiny-dense shape's host weights; -> (path, the tensors it was written from)."""
    s = synth.SHAPES["tiny-qknorm" if arch == "qwen3" else "tiny-dense"]
    ts = list(synth.host_weights(s, seed, kinds=kinds))
    names = {abi.T_EMBED: "token_embd.weight", abi.T_LM_HEAD: "output.weight", abi.T_FINAL_NORM: "output_norm.weight"}
    lname = {abi.T_WQ: "attn_q", abi.T_WK: "attn_k", abi.T_WV: "attn_v", abi.T_WO: "attn_output", abi.T_GATE: "ffn_gate", abi.T_UP: "ffn_up",
             abi.T_DOWN: "ffn_down", abi.T_ATTN_NORM: "attn_norm", abi.T_FFN_NORM: "ffn_norm", abi.T_Q_NORM: "attn_q_norm", abi.T_K_NORM: "attn_k_norm"}
    out = []
    for which, layer, _, kind, rows, cols, arr in ts:
        name = names[which] if which in names else f"blk.{layer}.{lname[which]}.weight"
        data = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        if permute and which in (abi.T_WQ, abi.T_WK):
            # store the rows the way llama-family files do: file row h*hd + 2j + s holds the engine's row h*hd + s*half + j
            nh = s.n_heads if which == abi.T_WQ else s.n_kv_heads
            hd, half = rows // nh, rows // nh // 2
            rb = data.size // rows
            src = np.arange(rows).reshape(nh, 2, half)                      # engine order [h][s][j]
            order = np.transpose(src, (0, 2, 1)).reshape(-1)                # file row [h][j][s] takes engine row [h][s][j]
            data = np.ascontiguousarray(data.reshape(rows, rb)[order]).reshape(-1)
        dims = (cols, rows) if rows > 1 else (cols,)
        out.append((name, dims, gguf.TYPE_OF_KIND[kind], data))
    meta = {"general.architecture": arch, f"{arch}.embedding_length": s.hidden, f"{arch}.block_count": s.n_layers,
            f"{arch}.attention.head_count": s.n_heads, f"{arch}.attention.head_count_kv": s.n_kv_heads,
            f"{arch}.feed_forward_length": s.ffn, f"{arch}.context_length": 128, f"{arch}.attention.layer_norm_rms_epsilon": float(s.rms_eps),
            f"{arch}.rope.freq_base": float(s.rope_theta), "tokenizer.ggml.tokens": ["a", "b"]}
    if arch == "qwen3":
        meta["qwen3.attention.key_length"] = s.head_dim
    path = str(tmp_path / f"{arch}.gguf")
    gguf.write(path, meta, out)
    return path, s, ts


def test_gguf_round_trip_and_unpermute(tmp_path):
    path, s, ts = _tiny_gguf(tmp_path, "llama", synth.Q4_K_M_KINDS, permute=True)
    g = gguf.GGUFFile(path)
    d = gguf.describe(g)
    assert (d.arch, d.hidden, d.n_layers, d.n_heads, d.n_kv_heads, d.head_dim, d.ffn, d.vocab) == \
        ("llama", s.hidden, s.n_layers, s.n_heads, s.n_kv_heads, s.head_dim, s.ffn, s.vocab)
    assert d.rope_base == 10000.0 and not d.qk_norm and not d.tied_head and g.meta["tokenizer.ggml.tokens"] == ["a", "b"]
    got = {(w, l): (k, r, c, a) for w, l, _, k, r, c, a in gguf.tensors(g, d)}
    assert len(got) == len(ts)
    for which, layer, _, kind, rows, cols, arr in ts:
        k, r, c, a = got[(which, layer)]
        assert (r, c) == (rows, cols), (which, layer)
        if which == abi.T_EMBED:
            assert k == abi.K_F16
        else:
            assert k == kind
        # the loader undoes the file's q/k row order: every tensor comes back byte for byte
        assert np.array_equal(np.ascontiguousarray(a).view(np.uint8).reshape(-1), np.ascontiguousarray(arr).view(np.uint8).reshape(-1)), (which, layer)
    # defaults when the file leaves them out (decoder/gguf.go:93-96,160-163)
    assert gguf.ARCH_DEFAULT_ROPE_BASE == {"llama": 10000.0, "qwen2": 1000000.0, "qwen3": 1000000.0}
    with pytest.raises(ValueError):
        bad = tmp_path / "bad.gguf"
        bad.write_bytes(b"GGML" + bytes(60))
        gguf.GGUFFile(str(bad))


def test_gguf_loaded_oracle_equals_direct_upload(oracle_lib, tmp_path):
    path, s, ts = _tiny_gguf(tmp_path, "qwen3", synth.Q4_K_M_KINDS)
    r, d = gguf.load(path, lambda cfg: oracle_lib.OracleResident(cfg), n_slots=2, ctx_cap=64, kernel_class=abi.CLASS_EXACT)
    assert d.qk_norm and d.head_dim == s.head_dim
    cfg = gguf.model_cfg(d, 2, 64, kernel_class=abi.CLASS_EXACT)
    direct = oracle_lib.OracleResident(cfg)
    for which, layer, expert, kind, rows, cols, arr in ts:
        direct.upload(which, arr, layer, expert, kind, rows, cols)
    direct.finalize()
    toks = [5, 9, 2, 30, 7, 7, 1]
    assert np.array_equal(r.PrefillLast(None, 0, 0, toks), direct.PrefillLast(None, 0, 0, toks))


def test_gguf_tied_head_and_bf16(oracle_lib, tmp_path):
    """A file without output.weight ties the head to the embedding table: a Q6_K table reaches the head in its own blocks and the
    gather as f16; BF16 tensors are widened."""
    s = synth.SHAPES["tiny-dense"]
    ts = [t for t in synth.host_weights(s, 9, kinds={abi.T_EMBED: abi.K_Q6K}) if t[0] != abi.T_LM_HEAD]
    names = {abi.T_EMBED: "token_embd.weight", abi.T_FINAL_NORM: "output_norm.weight"}
    lname = {abi.T_WQ: "attn_q", abi.T_WK: "attn_k", abi.T_WV: "attn_v", abi.T_WO: "attn_output", abi.T_GATE: "ffn_gate", abi.T_UP: "ffn_up",
             abi.T_DOWN: "ffn_down", abi.T_ATTN_NORM: "attn_norm", abi.T_FFN_NORM: "ffn_norm"}
    out = []
    for which, layer, _, kind, rows, cols, arr in ts:
        name = names[which] if which in names else f"blk.{layer}.{lname[which]}.weight"
        data, gt = np.ascontiguousarray(arr).view(np.uint8).reshape(-1), gguf.TYPE_OF_KIND[kind]
        if which in (abi.T_ATTN_NORM, abi.T_FFN_NORM, abi.T_FINAL_NORM):   # norms as BF16 (their values survive: 1 + small, rounded here)
            bf = (np.ascontiguousarray(arr, np.float32).view(np.uint32) >> 16).astype(np.uint16)
            data, gt = bf.view(np.uint8).reshape(-1), 30
        out.append((name, (cols, rows) if rows > 1 else (cols,), gt, data))
    meta = {"general.architecture": "qwen2", "qwen2.embedding_length": s.hidden, "qwen2.block_count": s.n_layers,
            "qwen2.attention.head_count": s.n_heads, "qwen2.attention.head_count_kv": s.n_kv_heads, "qwen2.feed_forward_length": s.ffn,
            "qwen2.context_length": 64, "qwen2.attention.layer_norm_rms_epsilon": float(s.rms_eps)}
    path = str(tmp_path / "tied.gguf")
    gguf.write(path, meta, out)
    g = gguf.GGUFFile(path)
    d = gguf.describe(g)
    assert d.tied_head and d.rope_base == 1000000.0 and d.head_dim == s.hidden // s.n_heads
    got = {(w, l): (k, a) for w, l, _, k, _, _, a in gguf.tensors(g, d)}
    emb = next(t for t in ts if t[0] == abi.T_EMBED)
    assert got[(abi.T_LM_HEAD, -1)][0] == abi.K_Q6K and np.array_equal(got[(abi.T_LM_HEAD, -1)][1], emb[6])
    k, a = got[(abi.T_EMBED, -1)]
    assert k == abi.K_F16
    np.testing.assert_allclose(a.astype(np.float64), kquants.q6k_dequantize(emb[6], s.vocab, s.hidden), rtol=1e-3, atol=1e-6)
    nk, na = got[(abi.T_FINAL_NORM, -1)]
    want = next(t for t in ts if t[0] == abi.T_FINAL_NORM)[6]
    assert nk == abi.K_F32 and np.abs(na - want).max() <= 2.0 ** -7
    r, _ = gguf.load(path, lambda cfg: oracle_lib.OracleResident(cfg), n_slots=2, ctx_cap=64, kernel_class=abi.CLASS_EXACT)
    assert np.all(np.isfinite(r.PrefillLast(None, 0, 0, [1, 2, 3, 4, 5])))
    # a file whose projections carry biases is refused, not loaded without them
    gguf.write(str(tmp_path / "biased.gguf"), meta, out + [("blk.0.attn_q.bias", (s.n_heads * s.head_dim,), 0, np.zeros(s.n_heads * s.head_dim, np.float32))])
    with pytest.raises(ValueError, match="bias"):
        gguf.describe(gguf.GGUFFile(str(tmp_path / "biased.gguf")))
