"""The C-ABI library builds, loads without a GPU, and exports exactly what include/q4k_b200.h
declares.  Host-only entry points are exercised; nothing here launches device work."""
import ctypes as C
import re
from pathlib import Path

import pytest

from qw38_b200 import _lib as L

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "q4k_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4k_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert names, "no declarations found"
    assert sorted(L.SIGNATURES) == names


def test_library_exports_every_declared_symbol():
    lib = L.load()
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert lib.q4k_abi_version() >= 1


def test_padding_rules_match_reference_formulas():
    """decode_pad_n / decode_pad_k / decode_code_bytes / decode_scale_bytes
    (cuda/decode_mmv.hpp:148-205, Q4_K branch)."""
    lib = L.load()
    assert lib.q4k_pad_n(0) == 0 and lib.q4k_pad_n(1) == 8 and lib.q4k_pad_n(137) == 144 and lib.q4k_pad_n(17408) == 17408
    assert lib.q4k_pad_k(0) == 0 and lib.q4k_pad_k(259) == 512 and lib.q4k_pad_k(5120) == 5120
    assert lib.q4k_code_bytes(17408, 5120) == 17408 * 5120 // 2
    assert lib.q4k_scale_bytes(17408, 5120) == 17408 * 20 * 16
    assert lib.q4k_code_bytes(17408, 5120) + lib.q4k_scale_bytes(17408, 5120) == 50135040  # 144 B per super-block


def test_geometry_rejected_before_any_device_work():
    lib = L.load()
    w = L.Weight(0x1000, 0x2000, L.LAYOUT_SPLIT_TILES, L.QUANTIZER_Q4K, 137, 259, 144, 512, 144 * 512 // 2 - 1, 144 * 2 * 16)
    x = L.Q8(0x3000, 0x4000, 0x5000, 512, 16, 16, 1, 259, 512)
    st = lib.q4k_q8_project(C.byref(w), x, 0x6000, 137, None, 0, None)
    assert st == L.ERR_INVALID_ARGUMENT and b"geometry" in lib.q4k_last_error()
    w.codes_bytes += 1
    w.layout = 0x0201  # another format's id
    assert lib.q4k_q8_project(C.byref(w), x, 0x6000, 137, None, 0, None) == L.ERR_INVALID_ARGUMENT
    w.layout = L.LAYOUT_SPLIT_TILES
    x.codes_len = 1  # truncated input (tests/q4k_q8_test.cpp:134)
    assert lib.q4k_q8_project(C.byref(w), x, 0x6000, 137, None, 0, None) == L.ERR_INVALID_ARGUMENT
    offs = (C.c_uint32 * 3)(0, 2, 1)
    x.codes_len = 512
    assert lib.q4k_q8_project_ragged(C.byref(w), x, offs, 2, 0x6000, 137, None, None) == L.ERR_INVALID_ARGUMENT
    assert lib.q4k_project_workspace_bytes(16, 5120, 1) == 0
    assert lib.q4k_project_workspace_bytes(16, 5120, 4) == 256 * 1024 + 4 * 16 * 5120 * 4
    assert lib.q4k_q8_mlp_workspace_bytes(512, 5120, 17408) == 512 * (17408 + 17408 // 32 * 8 + 2 * 17408 * 4) + 4  # cuda/q4k_q8.hpp:28-30
