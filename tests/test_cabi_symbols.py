"""The C-ABI library builds, loads without a GPU and exports what include/nq_fp8.h declares."""
import ctypes
import os
import re

import torch

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nq_fp8.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(built_library):
    from nano_qwen_b200 import _cabi
    names = declared_symbols()
    assert "nq_fp8_gemm_bs128" in names and "nq_act_quant_e4m3_g128" in names and len(names) >= 12
    handle = ctypes.CDLL(built_library)
    for name in names:
        assert hasattr(handle, name), f"{name} declared in include/nq_fp8.h but not exported"
    assert sorted(_cabi.SIGNATURES) == names          # the ctypes binding covers exactly the header


def test_version_and_status_strings(built_library):
    from nano_qwen_b200 import _cabi
    lib = _cabi.lib()
    assert lib.nq_version() == 100
    assert lib.nq_status_string(0) == b"ok"
    assert b"wait" in lib.nq_status_string(-5)
    assert lib.nq_fp8_gemm_workspace_bytes(16, 4096, 4096) == 0
    assert lib.nq_launch_count() >= 0


def test_no_cpu_fallback():
    """Without a CUDA device every compute entry refuses loudly instead of computing elsewhere."""
    import pytest
    from nano_qwen_b200 import _cabi, ops
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.act_quant(x)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fp8_linear(x, torch.zeros(128, 128).to(torch.float8_e4m3fn), torch.ones(1, 1))
    if not torch.cuda.is_available():
        with pytest.raises(_cabi.NqError):
            ops.init()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "nano_qwen_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
