"""The C-ABI library loads and exports every symbol include/b200_resident.h and include/b200_bench.h declare (no GPU calls)."""
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


@pytest.mark.parametrize("header,table", [("b200_resident.h", abi.EXPORTS), ("b200_bench.h", abi.BENCH_EXPORTS)])
def test_every_declared_symbol_is_exported(lib, header, table):
    hdr = open(os.path.join(ROOT, "include", header)).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)   # declarations only, not names mentioned in comments
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    assert declared == set(table), declared ^ set(table)
    for name in declared:
        assert hasattr(lib, name), name


def test_the_product_header_declares_only_reference_facing_entry_points():
    """Every declaration of b200_resident.h cites the reference interface it stands in for (or says that it has none);
    benchmark, synthesis and debug entry points live in b200_bench.h."""
    hdr = open(os.path.join(ROOT, "include", "b200_resident.h")).read()
    assert not re.search(r"\bb200_(bench|synth|debug|profile)_?[a-z0-9_]*\s*\(", re.sub(r"/\*.*?\*/", "", hdr, flags=re.S))


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


def test_every_programmatically_launched_kernel_waits():
    """A kernel that goes through launch_pdl may start before the kernel ahead of it has finished, so its body must
    call pdl_wait() (before its first dependent access; this checks that the call is there at all) and pdl_trigger()."""
    import glob
    import os
    import re
    src = {}
    for ext in ("*.cu", "*.cuh"):   # (a kernel may live in a header that one source includes)
        for path in glob.glob(os.path.join(os.path.dirname(__file__), "..", "goinfer_b200", "csrc", ext)):
            src[path] = open(path).read()
    names = set()
    for text in src.values():
        names |= set(re.findall(r"launch_pdl\(\s*([A-Za-z_0-9]+)", text))
    names.discard("void")   # launch_pdl's own definition
    assert len(names) >= 10
    all_text = "\n".join(src.values())
    for name in sorted(names):
        m = re.search(r"__global__[^;{]*?\b" + name + r"\s*\(", all_text)
        assert m, name
        end = all_text.find("__global__", m.end())
        body = all_text[m.end():end if end > 0 else len(all_text)]
        assert "pdl_wait()" in body and "pdl_trigger()" in body, name
        # ... and before the first dependent access: no pointer parameter is subscripted ahead of the wait. (Weights, which no
        # kernel writes, may be fetched earlier; the kernels that do so go through copy helpers or casts, not subscripts.)
        sig = body[:body.index(")")]
        params = re.findall(r"\*\s*(?:__restrict__\s+)?([A-Za-z_][A-Za-z_0-9]*)\s*(?:,|$)", sig)
        kernel_body = body[body.index("{"):]
        before = kernel_body[:kernel_body.index("pdl_wait()")]
        before = re.sub(r"//[^\n]*", "", before)
        for prm in params:
            assert not re.search(r"\b" + prm + r"\s*\[", before), (name, prm)


def test_go_shim_binds_every_product_symbol():
    """integration/b200/lib.go (source only: no Go toolchain here) registers one function per symbol of the product header,
    no more and no fewer, and checks the struct sizes this file pins."""
    import os
    import re
    from goinfer_b200 import abi
    text = open(os.path.join(os.path.dirname(__file__), "..", "integration", "b200", "lib.go")).read()
    bound = re.findall(r'\{&\w+,\s*"(b200_[a-z0-9_]+)"\}', text)
    assert len(bound) == len(set(bound))
    assert set(bound) == set(abi.EXPORTS), (sorted(set(abi.EXPORTS) - set(bound)), sorted(set(bound) - set(abi.EXPORTS)))
    for size in ("116", "24", "56"):
        assert re.search(r"unsafe\.Sizeof\(\w+\{\}\) != " + size, text), size
