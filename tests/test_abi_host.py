"""Host-only checks of the C ABI: the library loads, exports every symbol that include/zck.h declares, validates
arguments before touching a device, and fails loudly (no fallback) where there is no GPU."""

import ctypes
import pathlib
import re

import pytest
import torch

from zig_cu_kernels import _lib

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "zck.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(zck_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.library()
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/zck.h but missing from {_lib.library_path()}"
    assert set(_lib.SIGNATURES) == set(names), "the ctypes table and the header disagree"
    assert b"sm_100a" in lib.zck_version()


def test_struct_mirrors_match_the_header():
    assert ctypes.sizeof(_lib.GemmSizes) == 10 * 8 + 6 * 4
    assert ctypes.sizeof(_lib.Status) == 16


def test_arguments_are_checked_before_any_device_work():
    lib = _lib.library()
    buffer = ctypes.create_string_buffer(4096)
    address = (ctypes.addressof(buffer) + 15) & ~15
    code = lib.zck_quantize_fp8_rows(address, _lib.BF16, 100, address, address, 1, 0, 4, 100, 0, None)
    assert code == -1 and b"multiple of 128" in lib.zck_last_error()
    code = lib.zck_quantize_fp8_rows(address + 2, _lib.BF16, 128, address, address, 1, 0, 4, 128, 0, None)
    assert code == -1 and b"16 bytes" in lib.zck_last_error()
    code = lib.zck_fused_add_rms_norm(address, _lib.BF16, 12, None, 0, None, 0, None, 0, None, address, _lib.BF16, 12,
                                      2, 12, 1e-6, 0, None)
    assert code == -1 and b"multiple of 8" in lib.zck_last_error()
    sizes = _lib.GemmSizes(m=4, n=12, k=128, activation=0, splits=1)
    parts, counters = ctypes.c_size_t(), ctypes.c_uint32()
    assert lib.zck_gemm_plan(ctypes.byref(sizes), 0, 0, ctypes.byref(parts), ctypes.byref(counters)) == -1
    assert b"multiple of 8" in lib.zck_last_error()
    with pytest.raises(ValueError, match="multiple of 8"):
        _lib.check(-1)
    # empty problems queue nothing and need no device
    assert lib.zck_quantize_fp8_rows(None, _lib.BF16, 0, None, None, 0, 0, 0, 128, 0, None) == 0
    assert lib.zck_fused_add_rms_norm(None, 0, 0, None, 0, None, 0, None, 0, None, None, 0, 0, 0, 64, 1e-6, 0, None) == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="this is the no-GPU behaviour")
def test_no_gpu_means_an_error_not_a_fallback():
    lib = _lib.library()
    assert lib.zck_init(0) < 0
    assert lib.zck_last_error() != b""
    with pytest.raises((_lib.ZckError, ValueError)):
        _lib.check(lib.zck_init(0))


def test_missing_library_raises(monkeypatch, tmp_path):
    monkeypatch.setenv("ZCK_LIB", str(tmp_path / "nowhere.so"))
    monkeypatch.setattr(_lib, "_library", None)
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.library()
