"""Tensor parallel on real GPUs: the two-rank run needs at least two (one process per GPU through torch.distributed.run);
the cross-rank kernel's arithmetic is also checked on one GPU with emulated ranks."""
import os
import subprocess
import sys

import numpy as np
import pytest

from goinfer_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from goinfer_b200.ops import Ops
    return Ops(0)


def test_two_ranks_match_one_gpu_and_the_oracle():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29641", os.path.join(here, "tp_worker.py")], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0 and "TP_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]


@pytest.mark.parametrize("t,T,H", [(2, 5, 256), (4, 3, 4096), (8, 232, 8192), (8, 61, 2048), (3, 300, 1024)])
def test_reduce_norm_quant_kernel_with_emulated_ranks(ops, oracle_lib, t, T, H):
    """The kernel that replaces the all-reduce, the residual add, the RMSNorm and the quantizer of a tensor-parallel layer,
    with t blocks on one GPU standing for the ranks' blocks and one launch per rank after the other (its cross-rank waits
    left out). Against the oracle's norm and quantizer applied to h + (p0 + p1 + ...) added in rank order in f32: the
    codes, scales and group sums of every row must be the oracle's bits on every rank's view, the owner's residual rows
    the sums; in the hand-to-everyone mode every rank's residual rows are the sums. Row counts below the rank count and
    not divisible by it included."""
    import ctypes as C
    rng = np.random.default_rng(t * 1000 + T)
    parts = rng.normal(0, 1, (t, T, H)).astype(np.float32)
    h = rng.normal(0, 2, (T, H)).astype(np.float32)
    w = rng.normal(1, 0.2, H).astype(np.float32)
    s = parts[0].copy()
    for k in range(1, t):
        s = s + parts[k]
    x = h + s
    nG = H // 32

    def run(mode, given=parts, n_kparts=0):
        codes = np.zeros((t, T, H), np.int8)
        scales = np.zeros((t, T, 2 * nG), np.float32)
        h_out = np.zeros((t, T, H), np.float32)
        fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
        st = ops.lib.b200_debug_tp_reduce_emulated(ops.ctx, t, T, H, fp(given), fp(h), fp(w), C.c_float(1e-6), mode, n_kparts,
                                                   codes.ctypes.data_as(C.POINTER(C.c_int8)), fp(scales), fp(h_out))
        assert st == abi.OK, ops.lib.b200_last_error(ops.ctx)
        return codes, scales, h_out

    want_codes, want_scales = oracle_lib.op_quant_g32(oracle_lib.op_rmsnorm(x, w, 1e-6))
    rows_per = -(-T // t)
    for mode in (0, 2):   # with flags and fences; with words that announce themselves
        codes, scales, h_out = run(mode)
        for k in range(t):
            assert np.array_equal(codes[k], want_codes), (mode, k)
            assert np.array_equal(scales[k].view(np.uint32), want_scales.view(np.uint32)), (mode, k)
            lo, hi = min(T, k * rows_per), min(T, (k + 1) * rows_per)
            assert np.array_equal(h_out[k, lo:hi].view(np.uint32), x[lo:hi].view(np.uint32)), (mode, k)   # the owner's rows
            rest = np.ones(T, bool)
            rest[lo:hi] = False
            assert np.array_equal(h_out[k, rest], h[rest]), (mode, k)                                     # the others are left alone
    # each rank's product given as three K-split partials, which the kernel adds in split order before anything else
    kparts = rng.normal(0, 1, (t, 3, T, H)).astype(np.float32)
    s3 = (kparts[:, 0] + kparts[:, 1]) + kparts[:, 2]
    s = s3[0].copy()
    for k in range(1, t):
        s = s + s3[k]
    want_codes, want_scales = oracle_lib.op_quant_g32(oracle_lib.op_rmsnorm(h + s, w, 1e-6))
    codes, scales, _ = run(2, kparts, 3)
    for k in range(t):
        assert np.array_equal(codes[k], want_codes) and np.array_equal(scales[k].view(np.uint32), want_scales.view(np.uint32)), k
    _, _, h_all = run(1)
    for k in range(t):
        assert np.array_equal(h_all[k].view(np.uint32), x.view(np.uint32)), k
