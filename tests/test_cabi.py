"""The C-ABI library loads and exports every symbol include/oal_b200.h declares; host-only
entry points behave (no compute call is made here, so no GPU is needed)."""

import ctypes
import re
from pathlib import Path

import pytest

from oal_b200 import _lib
from oal_b200.hd_block_gemm import make_problem

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "oal_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oal_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.load()
    declared = _declared_symbols()
    assert declared, "no declarations found in include/oal_b200.h"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_version_and_workspace_queries():
    import torch

    lib = _lib.load()
    assert b"sm_100a" in lib.oal_version_string()
    geometry = (4, 14, 2, 4096, 64, 64)
    p = make_problem(geometry, groups=8, io_dtype=torch.float32, out_dtype=torch.float32,
                     precision="fp32_ieee", chunk=0, scale=0.125, floor=1e-38)
    assert _lib.workspace_bytes(p, 0) == 0
    rows = 4 * 14 * 4096
    assert _lib.workspace_bytes(p, 1) >= rows * 80 * 4
    assert _lib.workspace_bytes(p, 2) == 0


def test_contract_violations_map_to_reference_exception_types():
    import torch

    bad = make_problem((1, 3, 2, 16, 64, 64), groups=1, io_dtype=torch.float32, out_dtype=torch.float32,
                       precision="fp32_ieee", chunk=0, scale=1.0, floor=1e-38)
    with pytest.raises(ValueError, match="divisible"):
        _lib.workspace_bytes(bad, 0)
    bad = make_problem((1, 2, 2, 16, 64, 64), groups=40, io_dtype=torch.float32, out_dtype=torch.float32,
                       precision="fp32_ieee", chunk=0, scale=1.0, floor=1e-38)
    with pytest.raises(ValueError, match="groups"):
        _lib.workspace_bytes(bad, 0)
    bad = make_problem((1, 2, 2, 16, 64, 64), groups=4, io_dtype=torch.float32, out_dtype=torch.float32,
                       precision="bf16_tensorcore", chunk=128, scale=1.0, floor=1e-38)
    with pytest.raises(TypeError, match="bf16"):
        _lib.workspace_bytes(bad, 0)
    lib = _lib.load()
    rc = lib.oal_forward(ctypes.byref(bad), *([None] * 14), 0, None, None)
    assert rc < 0
