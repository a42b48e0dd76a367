"""The C-ABI library builds, loads without a GPU and exports every entry point
`include/b200q.h` declares; the Python binding declares the same set."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared() -> set[str]:
    header = (ROOT / "include" / "b200q.h").read_text()
    return set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", header))


def test_library_exports_every_declared_symbol():
    from linnet_b200 import _build, _lib

    _build.build()
    lib = ctypes.CDLL(str(_lib.LIBRARY))
    names = declared()
    assert "b200q_int4_linear" in names and "b200q_quantize_int4_groups" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_binding_matches_header():
    from linnet_b200 import _lib

    assert set(_lib.PROTOTYPES) | {"b200q_last_error"} == declared()
    lib = _lib.load()
    assert lib.b200q_abi_version() == 1


def test_binding_argument_lists_match_header():
    """Every ctypes prototype has the header's argument count and the header's kinds of
    arguments (pointer / 64-bit / 32-bit / float), in order."""
    from ctypes import c_float, c_int32, c_int64, c_void_p

    from linnet_b200 import _lib

    header = (ROOT / "include" / "b200q.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    kinds = {c_void_p: "pointer", c_int64: "int64", c_int32: "int32", c_float: "float"}
    for name, argtypes in _lib.PROTOTYPES.items():
        match = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", header, flags=re.S)
        assert match, name
        text = match.group(1).strip()
        params = [] if text in ("", "void") else [p.strip() for p in text.split(",")]
        assert len(params) == len(argtypes), f"{name}: header has {len(params)} arguments, binding {len(argtypes)}"
        for position, (param, ctype) in enumerate(zip(params, argtypes)):
            want = ("pointer" if "*" in param else "int64" if param.startswith("int64_t")
                    else "int32" if param.startswith("int32_t") else "float" if param.startswith("float") else param)
            assert kinds[ctype] == want, f"{name} argument {position}: header `{param}`, binding {kinds[ctype]}"


def test_argument_errors_need_no_gpu():
    """Shape validation happens on the host, before any launch."""
    from linnet_b200 import _lib

    lib = _lib.load()
    status = lib.b200q_quantize_int4_groups(None, _lib.F32, 4, 100, 128, None, None, None,
                                            _lib.F32, None, None)
    assert status == _lib.ERROR
    assert "must be even and divide the 100 inputs" in _lib.last_error()
    status = lib.b200q_int4_gemv(None, None, None, None, None, 1, 256, 64, 128, _lib.F32, None)
    assert status == _lib.ERROR and "bf16 or f16" in _lib.last_error()
    # empty problems succeed without touching the device
    assert lib.b200q_int4_gemv(None, None, None, None, None, 0, 256, 64, 128, _lib.BF16, None) == 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch

    from linnet_b200 import kernels

    x = torch.zeros(1, 128, dtype=torch.bfloat16)
    packed = torch.zeros(16, 1, 64, dtype=torch.uint8)
    scale = torch.ones(16, 1, dtype=torch.bfloat16)
    zero = torch.zeros(16, 1, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        kernels.int4_linear(x, packed, scale, zero)
    with pytest.raises(ValueError, match="a group of 24 is not 16, 32, 64, or a multiple of 128"):
        kernels.int4_linear(torch.zeros(1, 24, dtype=torch.bfloat16),
                            torch.zeros(16, 1, 12, dtype=torch.uint8), scale, zero)
