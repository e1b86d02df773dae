"""Shared test helpers: golden fixtures -> residents, tolerance checks."""
import json
import os

import numpy as np

from goinfer_b200 import abi

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# The logits bar of the build: |gpu - oracle| <= ATOL + RTOL * |oracle| (fp32 accumulate).
ATOL, RTOL = 2e-2, 1e-2


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = json.loads(bytes(z["config_json"]).decode())
    w = {k[2:]: z[k] for k in z.files if k.startswith("w/")}
    g = {k[7:]: z[k] for k in z.files if k.startswith("golden/")}
    return cfg, w, g


def cfg_from_hf(hf, n_slots=2, ctx_cap=64, kv_block_rows=16, kv_dtype=0, max_rows=64):
    c = abi.ModelCfg()
    c.hidden, c.n_layers = hf["hidden_size"], hf["num_hidden_layers"]
    c.n_heads, c.n_kv_heads = hf["num_attention_heads"], hf["num_key_value_heads"]
    c.head_dim = hf.get("head_dim") or c.hidden // c.n_heads
    c.vocab, c.rotary_dim = hf["vocab_size"], c.head_dim
    moe = hf.get("num_experts", 0)
    c.ffn = 0 if moe else hf["intermediate_size"]
    c.qk_norm = 1 if hf["model_type"] in ("qwen3", "qwen3_moe") else 0
    c.n_experts, c.top_k = moe, hf.get("num_experts_per_tok", 0)
    c.norm_topk, c.moe_ffn = int(hf.get("norm_topk_prob", True)), hf.get("moe_intermediate_size", 0)
    c.kv_block_rows = kv_block_rows
    c.kv_pool_blocks = 1 + n_slots * ((ctx_cap + kv_block_rows - 1) // kv_block_rows)
    c.n_slots, c.ctx_cap, c.max_rows = n_slots, ctx_cap, max_rows
    c.tp_rank, c.tp_size, c.kernel_class, c.fast_floor, c.kv_dtype = 0, 1, abi.CLASS_AUTO, 0, kv_dtype
    c.rms_eps = hf["rms_norm_eps"]
    c.rope_theta = hf["rope_parameters"]["rope_theta"]
    return c


def upload_hf(r, hf, w):
    """HF-named f32 tensors -> the resident's tensor table."""
    f = lambda a: np.ascontiguousarray(a, np.float32)
    r.upload(abi.T_EMBED, f(w["model.embed_tokens.weight"]))
    r.upload(abi.T_LM_HEAD, f(w["lm_head.weight"]))
    r.upload(abi.T_FINAL_NORM, f(w["model.norm.weight"]))
    for l in range(hf["num_hidden_layers"]):
        p = f"model.layers.{l}."
        r.upload(abi.T_ATTN_NORM, f(w[p + "input_layernorm.weight"]), l)
        r.upload(abi.T_FFN_NORM, f(w[p + "post_attention_layernorm.weight"]), l)
        for which, nm in ((abi.T_WQ, "q"), (abi.T_WK, "k"), (abi.T_WV, "v"), (abi.T_WO, "o")):
            r.upload(which, f(w[p + f"self_attn.{nm}_proj.weight"]), l)
        if p + "self_attn.q_norm.weight" in w:
            r.upload(abi.T_Q_NORM, f(w[p + "self_attn.q_norm.weight"]), l)
            r.upload(abi.T_K_NORM, f(w[p + "self_attn.k_norm.weight"]), l)
        if hf.get("num_experts", 0):
            r.upload(abi.T_ROUTER, f(w[p + "mlp.gate.weight"]), l)
            for e in range(hf["num_experts"]):
                q = p + f"mlp.experts.{e}."
                r.upload(abi.T_EXP_GATE, f(w[q + "gate_proj.weight"]), l, e)
                r.upload(abi.T_EXP_UP, f(w[q + "up_proj.weight"]), l, e)
                r.upload(abi.T_EXP_DOWN, f(w[q + "down_proj.weight"]), l, e)
        else:
            r.upload(abi.T_GATE, f(w[p + "mlp.gate_proj.weight"]), l)
            r.upload(abi.T_UP, f(w[p + "mlp.up_proj.weight"]), l)
            r.upload(abi.T_DOWN, f(w[p + "mlp.down_proj.weight"]), l)


def close_logits(a, b, atol=ATOL, rtol=RTOL):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    fin = np.isfinite(b)
    assert np.array_equal(np.isfinite(a), fin), "masked (-inf) positions differ"
    err = np.abs(a[fin] - b[fin])
    bound = atol + rtol * np.abs(b[fin])
    worst = float((err - bound).max()) if err.size else 0.0
    return worst <= 0, float(err.max() if err.size else 0.0)
