"""Tensor parallel on real GPUs: needs at least two; one process per GPU through torch.distributed.run."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_two_ranks_match_one_gpu_and_the_oracle():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29641", os.path.join(here, "tp_worker.py")], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0 and "TP_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]
