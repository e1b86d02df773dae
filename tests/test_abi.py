"""The C-ABI library loads and exports every symbol include/b200_resident.h declares (no GPU calls)."""
import os
import re

import pytest

from goinfer_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from goinfer_b200 import build, resident
    build.build()
    return resident.load_library()


def test_every_declared_symbol_is_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "b200_resident.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    assert declared == set(abi.EXPORTS), declared ^ set(abi.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layouts_match_the_header():
    import ctypes as C
    assert C.sizeof(abi.ModelCfg) == 23 * 4 + 6 * 4
    assert C.sizeof(abi.Draw) == 24 and abi.Draw.u.offset == 16
    assert C.sizeof(abi.Caps) == 8 * 4 + 3 * 8
    assert C.sizeof(abi.Stats) == 6 * 8 + 8


def test_open_without_a_gpu_fails_loudly(lib):
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is visible")
    ctx = C.c_void_p()
    assert lib.b200_open(0, None, C.byref(ctx)) == abi.CUDA_ERROR
    from goinfer_b200.resident import Resident, ResidentError
    with pytest.raises(ResidentError):
        Resident(abi.ModelCfg())
