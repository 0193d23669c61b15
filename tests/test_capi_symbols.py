"""The C-ABI library must load without a GPU and export every symbol the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "strata_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(strata_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    from strata_b200 import build, _lib
    path = build.build_library()
    assert path.exists()
    lib = ctypes.CDLL(str(path))
    names = declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/strata_b200.h but not exported"
    # the ctypes binding covers every declared entry point too
    assert sorted(_lib.exported_names()) == names


def test_error_strings_and_version():
    from strata_b200 import _lib
    lib = _lib.load()
    assert lib.strata_abi_version() >= 1
    assert b"invalid argument" in lib.strata_error_string(-1)
    assert lib.strata_block_workspace_bytes(128, 64, 256) == 3 * 128 * 64 * 2 + 128 * 192 * 2 + 128 * 256 * 2


def test_ops_refuse_cpu_tensors():
    import torch
    from strata_b200 import ops, _lib
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    with pytest.raises(_lib.StrataLibraryError):
        ops.layernorm(x)
    with pytest.raises(_lib.StrataLibraryError):
        ops.linear(x, torch.zeros(64, 64, dtype=torch.bfloat16))
