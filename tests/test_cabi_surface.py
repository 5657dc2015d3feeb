"""The shared library loads without a GPU and exports exactly what include/*.h declares."""

import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = header.read_text()
        names += re.findall(r"DFL_API\s+[\w\s\*]+?\b(dfl_\w+)\s*\(", text)
    return names


def test_header_declares_the_documented_entry_points():
    names = declared_symbols()
    for required in ("dfl_build_position_lut", "dfl_qkv_proj", "dfl_pos_scores", "dfl_attention_fwd",
                     "dfl_gather_slots", "dfl_status_string"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from disentangled_flash_b200 import _cabi, build

    build.build()  # no-op when up to date; nvcc cross-compiles without a GPU
    lib = _cabi.load_library()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert set(declared_symbols()) == set(_cabi.EXPORTED_SYMBOLS)
    assert lib.dfl_version() >= 100


def test_status_strings_and_argument_checks_need_no_gpu():
    import ctypes

    from disentangled_flash_b200 import _cabi

    lib = _cabi.load_library()
    assert lib.dfl_status_string(0) == b"ok"
    assert b"aligned" in lib.dfl_status_string(_cabi.DFL_ERR_ALIGNMENT)
    # null params / bad sizes are rejected on the host before any CUDA call
    assert lib.dfl_attention_fwd(None, None) == _cabi.DFL_ERR_BAD_ARG
    assert lib.dfl_qkv_proj(None, None) == _cabi.DFL_ERR_BAD_ARG
    assert lib.dfl_build_position_lut(0, 256, 512, 256, 1, None, None, None, None) == _cabi.DFL_ERR_BAD_ARG
    assert b"positive" in lib.dfl_last_error()
    p = _cabi.DflAttnParams()
    p.batch, p.heads, p.seq_len, p.head_dim, p.dtype = 1, 1, 8, 48, _cabi.DFL_F16
    assert lib.dfl_attention_fwd(ctypes.byref(p), None) == _cabi.DFL_ERR_UNSUPPORTED
    p.head_dim = 64
    p.q = p.k = p.v = p.out = p.mask = 16
    p.mask_elem_size, p.scale = 1, 0.1
    p.q = 24  # misaligned
    assert lib.dfl_attention_fwd(ctypes.byref(p), None) == _cabi.DFL_ERR_ALIGNMENT
