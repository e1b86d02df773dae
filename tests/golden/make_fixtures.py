"""Regenerates tests/golden/*.npz from the reference checkout's own test data.

Usage: python make_fixtures.py <path of the reference checkout>. Machines that run the tests need not have the
reference tree, which is why the outputs are committed. Each .npz holds the tiny model's f32 weights (from the reference's
committed safetensors) and the golden vectors the reference's tests compare against:
  llama_tiny   <- testdata/llama-tiny/ + testdata/llama_tiny_text_golden.json   (decoder/llama_tiny_test.go:22-80)
  qwen3moe_tiny<- testdata/qwen3moe-tiny/ + testdata/qwen3moe_forward_golden.json (decoder/qwen3moe_test.go)
Nothing but data is copied: weights, ids and logits.
"""
import json
import os
import sys

import numpy as np
from safetensors.numpy import load_file

if len(sys.argv) < 2:
    sys.exit("usage: make_fixtures.py <path of the reference checkout>")
REF = sys.argv[1]
OUT = os.path.dirname(os.path.abspath(__file__))


def dump(name, model_dir, golden_json, extra):
    td = os.path.join(REF, "testdata")
    w = load_file(os.path.join(td, model_dir, "model.safetensors"))
    cfg = json.load(open(os.path.join(td, model_dir, "config.json")))
    g = json.load(open(os.path.join(td, golden_json)))
    out = {"w/" + k: v.astype(np.float32) for k, v in w.items()}
    out["config_json"] = np.frombuffer(json.dumps(cfg).encode(), np.uint8)
    for k, v in extra(g).items():
        out["golden/" + k] = np.asarray(v)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out)
    print(name, sum(v.size for v in w.values()), "weights")


dump("llama_tiny", "llama-tiny", "llama_tiny_text_golden.json", lambda g: {
    "prompt_ids": np.array(g["prompt_ids"], np.int32), "argmax": np.int32(g["argmax"]),
    "last_logits": np.array(g["last_logits"], np.float32),
    "continuation_ids": np.array(g["continuation_ids"], np.int32)})
dump("qwen3moe_tiny", "qwen3moe-tiny", "qwen3moe_forward_golden.json", lambda g: {
    "ids": np.array(g["ids"], np.int32), "argmax": np.int32(g["argmax"]),
    "top_k_ids": np.array([t[0] for t in g["top_k"]], np.int32),
    "top_k_logits": np.array([t[1] for t in g["top_k"]], np.float32),
    "sample_ids": np.array([t[0] for t in g["sample"]], np.int32),
    "sample_logits": np.array([t[1] for t in g["sample"]], np.float32),
    "stats": np.array([g["stats"][k] for k in ("n", "sum", "sum_sq", "min", "max")], np.float64)})
