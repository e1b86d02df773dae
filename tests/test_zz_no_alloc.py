"""b200_attention_noalloc: paged decode attention for hosts that may not allocate device memory when they need it
(memory handed out once at start-up and owned by the host's pool, or a "no device allocation after init" plug-in rule).
Its split partials live in a fixed 16 MiB array inside the library instead of a cudaMalloc'd buffer.

The test drives it through the C ABI with device buffers made by torch, twice in a row with different inputs (the
second call finds the first call's leftovers in the shared array), and compares each result with the allocating entry
point b200_op_attention on the same data and with the CPU oracle's f64 attention, to the tolerance the attention tests
use. It also checks that the caller's current device is the same after a call as before it, and that requests too
large for the array, or whose table cannot hold the keys, are refused with the sizes in the error text. The file sorts last so that a run that stops at the
first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest

from goinfer_b200 import abi

pytestmark = pytest.mark.gpu


def _paged(k, v, n_keys, nKV, hd, block_rows):
    """Contiguous [rows][max_keys][nKV*hd] f32 K/V -> fp16 pools [block][kv_head][row][hd] + identity-style tables."""
    rows, max_keys = k.shape[0], k.shape[1]
    mb = (max_keys + block_rows - 1) // block_rows
    table = np.zeros((rows, mb), np.int32)
    kp = np.zeros((1 + rows * mb, nKV, block_rows, hd), np.float16)
    vp = np.zeros_like(kp)
    nxt = 1
    for r in range(rows):
        for b in range((int(n_keys[r]) + block_rows - 1) // block_rows):
            table[r, b] = nxt
            lo, hi = b * block_rows, min((b + 1) * block_rows, int(n_keys[r]))
            kp[nxt, :, :hi - lo] = k[r, lo:hi].reshape(hi - lo, nKV, hd).transpose(1, 0, 2)
            vp[nxt, :, :hi - lo] = v[r, lo:hi].reshape(hi - lo, nKV, hd).transpose(1, 0, 2)
            nxt += 1
    return kp, vp, table


def test_no_alloc_attention_matches_the_allocating_entry_point_twice(oracle_lib):
    import torch
    from goinfer_b200.ops import Ops
    stream = torch.cuda.Stream()
    ops = Ops(0, stream=stream.cuda_stream)
    lib, ctx = ops.lib, ops.ctx
    nH, nKV, hd, br = 32, 8, 128, 16
    for call, (seed, n_keys) in enumerate(((1, [1, 17, 600, 1300, 64]), (2, [1500, 3, 1024, 1025, 512]))):
        rng = np.random.default_rng(seed)
        n_keys = np.array(n_keys, np.int32)
        rows, max_keys = len(n_keys), int(n_keys.max())
        q = rng.normal(0, 1, (rows, nH * hd)).astype(np.float32)
        k = rng.normal(0, 1, (rows, max_keys, nKV * hd)).astype(np.float32)
        v = rng.normal(0, 1, (rows, max_keys, nKV * hd)).astype(np.float32)
        want = ops.attention(q, k, v, n_keys, nH, nKV, hd, 0.0, 0.0, block_rows=br)
        want64 = oracle_lib.op_attention(q, k, v, n_keys, nH, nKV, hd, 1.0 / np.sqrt(hd), 0.0)
        kp, vp, table = _paged(k, v, n_keys, nKV, hd, br)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        dq, dk, dv, dt = dev(q), dev(kp), dev(vp), dev(table)
        dslot, dpos = dev(np.arange(rows, dtype=np.int32)), dev(n_keys - 1)
        dout = torch.full((rows, nH * hd), float("nan"), device="cuda")
        torch.cuda.synchronize()
        p = lambda t: C.c_void_p(t.data_ptr())
        st = lib.b200_attention_noalloc(ctx, p(dq), nH * hd, rows, nH, nKV, hd, C.c_float(0.0), C.c_float(0.0), p(dslot), p(dpos),
                                        max_keys, p(dk), p(dv), p(dt), table.shape[1], br, p(dout))
        assert st == abi.OK, ops.drv.last_error()
        torch.cuda.synchronize()
        assert torch.cuda.current_device() == 0
        got = dout.cpu().numpy()
        np.testing.assert_allclose(got, want, atol=2e-5, rtol=1e-4, err_msg=f"call {call}")
        np.testing.assert_allclose(got, want64, atol=2e-5, rtol=1e-4, err_msg=f"call {call} against the f64 oracle")
    # a request whose partials do not fit the fixed array is refused, and says why
    # (refusals come before any launch, so the sizes named here need no buffers behind them)
    st = lib.b200_attention_noalloc(ctx, p(dq), nH * hd, 100, nH, nKV, hd, C.c_float(0.0), C.c_float(0.0), p(dslot), p(dpos),
                                    8192, p(dk), p(dv), p(dt), 8192 // br, br, p(dout))
    assert st == abi.BAD_ARGUMENT
    msg = ops.drv.last_error()
    assert "scratch" in msg and "16777216" in msg, msg
    # a table too short for the key range, a block size of zero and a misaligned q are refused too
    for kwargs in (dict(max_blocks=table.shape[1] - 1), dict(block_rows=0), dict(q_off=4)):
        st = lib.b200_attention_noalloc(ctx, C.c_void_p(dq.data_ptr() + kwargs.get("q_off", 0)), nH * hd, rows, nH, nKV, hd, C.c_float(0.0),
                                        C.c_float(0.0), p(dslot), p(dpos), max_keys, p(dk), p(dv), p(dt),
                                        kwargs.get("max_blocks", table.shape[1]), kwargs.get("block_rows", br), p(dout))
        assert st == abi.BAD_ARGUMENT, kwargs
