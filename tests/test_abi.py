"""The C-ABI library loads on a machine without a GPU and exports every declared symbol."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def library():
    from texelator_b200.cuda.build import build
    from texelator_b200 import runtime
    return runtime.load_library(build())


def test_every_declared_symbol_is_exported(library):
    from texelator_b200 import runtime
    header = (ROOT / "include" / "texelator_b200.h").read_text()
    declared = set(re.findall(r"\b(tx_[a-z_0-9]+)\s*\(", header))
    assert declared, "header declares no entry points"
    assert declared == set(runtime.C_API), (declared ^ set(runtime.C_API))
    for name in declared:
        assert getattr(library, name) is not None


def test_header_cites_the_reference_interface():
    header = (ROOT / "include" / "texelator_b200.h").read_text()
    for needle in ("extension.cpp", "texelator_cuda.cu:1260-1327", "texelator_cuda.cu:1329-1469",
                   "texelator_cuda.cu:1471-1478", "texelator_cuda.cu:1540-1595"):
        assert needle in header


def test_calls_without_a_gpu_fail_with_a_message(library):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert library.tx_set_lookahead(0, 2) != 0
    assert b"null Texelator handle" in library.tx_last_error()
    out = ctypes.c_uint64(0)
    blocks = (ctypes.c_uint8 * 64)()
    scales = (ctypes.c_float * 1)(1.0)
    status = library.tx_pack_encoded(blocks, 64, scales, 1, None, 1, 0, ctypes.byref(out))
    assert status != 0 and library.tx_last_error()      # no device: a CUDA error, never a CPU fallback
    assert library.tx_launch_count() == 0


def test_operator_refuses_cpu_tensors():
    import torch
    from texelator_b200 import runtime
    ext = runtime.extension()
    with pytest.raises(RuntimeError, match="null Texelator handle"):
        ext.linear(1234, torch.zeros(1, 16, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="at least one texture handle"):
        runtime.TexelatorLinear([])


def test_no_product_code_imports_the_oracle():
    for path in list((ROOT / "texelator_b200").rglob("*.py")) + list((ROOT / "texelator_b200").rglob("*.cu")):
        text = path.read_text()
        assert "oracle" not in text.replace("oracle/bc4_oracle.py", ""), path
