"""Device-resident micro-benchmarks of the kernels that carry the step, on synthetic data.

  python -m goinfer_b200.microbench attention --rows 256 [--ctx-lo 128 --ctx-hi 8192 --heads 32 --kv-heads 8 --head-dim 128]
  python -m goinfer_b200.microbench q4k --rows 1 2 4 8 16 32 256 [--n 12288 --k 4096]
  python -m goinfer_b200.microbench f16 --rows 256 [--n 151936 --k 4096]
  python -m goinfer_b200.microbench prefill --rows 2048 [--pos0 0 --heads 32 --kv-heads 8 --head-dim 128]
  python -m goinfer_b200.microbench gateup --rows 256 [--f 12288 --k 4096 --mode 1]   (one call through host buffers: for profilers)

Times are CUDA-event averages per launch after warm-up. Weight matrices are cycled through several copies and KV pools
are far larger than the 126 MB L2, so no launch finds its inputs cached.
"""
import argparse
import json


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    a = sub.add_parser("attention")
    a.add_argument("--rows", type=int, default=256)
    a.add_argument("--ctx-lo", type=int, default=128)
    a.add_argument("--ctx-hi", type=int, default=8192)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--block-rows", type=int, default=16)
    a.add_argument("--iters", type=int, default=10)
    a.add_argument("--warmup", type=int, default=3)
    p = sub.add_parser("prefill")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--pos0", type=int, default=0)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--block-rows", type=int, default=16)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    h = sub.add_parser("f16")
    h.add_argument("--rows", type=int, nargs="+", default=[256])
    h.add_argument("--n", type=int, default=151936)
    h.add_argument("--k", type=int, default=4096)
    h.add_argument("--klass", type=int, default=0)
    h.add_argument("--iters", type=int, default=10)
    h.add_argument("--warmup", type=int, default=3)
    g = sub.add_parser("q4k")
    g.add_argument("--rows", type=int, nargs="+", default=[1, 2, 4, 8, 16, 32, 256])
    g.add_argument("--n", type=int, default=12288)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--klass", type=int, default=0)
    g.add_argument("--iters", type=int, default=20)
    g.add_argument("--warmup", type=int, default=3)
    g.add_argument("--kind", choices=["q4k", "q5k", "q6k"], default="q4k", help="q5k / q6k: the native K-quant lanes")
    u = sub.add_parser("gateup")
    u.add_argument("--rows", type=int, default=256)
    u.add_argument("--f", type=int, default=12288)
    u.add_argument("--k", type=int, default=4096)
    u.add_argument("--mode", type=int, default=1, help="0 matmul + SwiGLU kernel, 1 SwiGLU in the matmul's epilogue, 2 interleaved rows + SwiGLU kernel")
    args = ap.parse_args()
    from .ops import Ops
    ops = Ops(0)
    if args.what == "attention":
        ms, kvb = ops.bench_attention(args.rows, args.ctx_lo, args.ctx_hi, args.heads, args.kv_heads, args.head_dim,
                                      args.block_rows, 2, args.warmup, args.iters)
        print(json.dumps({"kernel": "paged attention (split + combine)", "rows": args.rows, "ms_per_launch": ms,
                          "kv_bytes": kvb, "GBps": kvb / ms / 1e6}))
    elif args.what == "f16":
        for m in args.rows:
            ms = ops.bench_f16_matmul(m, args.k, args.n, args.klass, args.warmup, args.iters)
            wb = args.n * args.k * 2
            print(json.dumps({"kernel": "f16-weight matmul", "rows": m, "n": args.n, "k": args.k, "ms_per_launch": ms,
                              "weight_GBps": wb / ms / 1e6, "TMACps": m * args.n * args.k / ms / 1e9}))
    elif args.what == "gateup":
        import time
        import numpy as np
        rng = np.random.default_rng(0)
        nb = 2 * args.f * args.k // 256
        raw = rng.integers(0, 256, (nb, 144), dtype=np.uint8)
        raw[:, 0:2] = rng.uniform(0.001, 0.01, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)   # d
        raw[:, 2:4] = rng.uniform(0.001, 0.01, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)   # dmin
        a = rng.normal(0, 1, (args.rows, args.k)).astype(np.float32)
        t = time.perf_counter()
        codes, scales = ops.gate_up_swiglu(raw.reshape(-1), a, args.f, args.mode)
        print(json.dumps({"kernel": "gate|up matmul + SwiGLU + quantizer", "mode": args.mode, "rows": args.rows, "f": args.f, "k": args.k,
                          "wall_ms_with_copies": (time.perf_counter() - t) * 1e3, "codes_checksum": int(codes.astype(np.int64).sum())}))
    elif args.what == "prefill":
        ms = ops.bench_prefill_attention(args.rows, args.pos0, args.heads, args.kv_heads, args.head_dim, args.block_rows,
                                         args.warmup, args.iters)
        # causal: row j sees pos0 + j + 1 keys; 4 flop per (row, key, head, dim): QK^T and PV, a multiply-add each
        pairs = args.rows * args.pos0 + args.rows * (args.rows + 1) / 2
        flop = 4.0 * pairs * args.heads * args.head_dim
        print(json.dumps({"kernel": "prefill attention (causal run)", "rows": args.rows, "pos0": args.pos0, "ms_per_launch": ms,
                          "TFLOPps": flop / ms / 1e9}))
    else:
        from . import abi
        for m in args.rows:
            if args.kind == "q4k":
                ms = ops.bench_q4k_matmul(m, args.k, args.n, args.klass, 8, args.warmup, args.iters)
                wb = args.n * args.k * 144 / 256
            else:
                kind = abi.K_Q5K if args.kind == "q5k" else abi.K_Q6K
                ms = ops.bench_kq_matmul(kind, m, args.k, args.n, 8, args.warmup, args.iters)
                wb = args.n * args.k * (176 if args.kind == "q5k" else 210) / 256
            print(json.dumps({"kernel": args.kind + " matmul", "rows": m, "n": args.n, "k": args.k, "ms_per_launch": ms,
                              "weight_GBps": wb / ms / 1e6, "TMACps": m * args.n * args.k / ms / 1e9}))


if __name__ == "__main__":
    main()
