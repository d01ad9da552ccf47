"""The C-ABI library loads, exports every symbol the header declares and rejects bad
arguments with the documented status codes - all without touching a GPU."""

import ctypes
import re
from pathlib import Path

from tuna_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def test_every_declared_symbol_is_exported(tuna_lib):
    header = (ROOT / "include" / "tuna_b200.h").read_text()
    declared = set(re.findall(r"\b(tuna_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found"
    c_symbols = {n for n in _lib.SYMBOLS if n.startswith("tuna_")}
    assert declared == c_symbols, declared ^ c_symbols
    for name in declared:
        assert hasattr(tuna_lib, name), name


def test_reference_named_cxx_symbols_are_exported(tuna_lib):
    # the two native symbols the reference's pybind module links against (extension.cpp:22-24)
    header = (ROOT / "include" / "tuna_b200.h").read_text()
    assert re.search(r"^void wrapper\(void \*q, void \*x, void \*c, void \*s, void \*o, int m, int n, int k,", header, re.M)
    assert re.search(r"^void dequantize_wrapper\(void \*q, void \*a, void \*c, void \*o, const int m, const int k,", header, re.M)
    mangled = [n for n in _lib.SYMBOLS if n.startswith("_Z")]
    assert sorted(mangled) == ["_Z18dequantize_wrapperPvS_S_S_iiP11CUstream_st", "_Z7wrapperPvS_S_S_S_iiiP11CUstream_st"]
    for name in mangled:
        assert hasattr(tuna_lib, name), name
    # bad shape: nothing is launched, the status says why (no GPU needed)
    tuna_lib._Z7wrapperPvS_S_S_S_iiiP11CUstream_st(None, None, None, None, None, 60, 1, 64, None)
    assert tuna_lib.tuna_last_wrapper_status() == -2


def test_struct_layout_matches_header():
    header = (ROOT / "include" / "tuna_b200.h").read_text()
    body = re.search(r"typedef struct tuna_config \{(.*?)\} tuna_config;", header, re.S).group(1)
    names = re.findall(r"int32_t\s+(\w+)", body)
    assert names == [n for n, _ in _lib.TunaConfig._fields_]
    assert ctypes.sizeof(_lib.TunaConfig) == 64


def test_status_strings(tuna_lib):
    assert tuna_lib.tuna_status_string(0) == b"ok"
    for s in range(-9, 0):
        assert tuna_lib.tuna_status_string(s) not in (b"ok", b"unknown status")
    assert tuna_lib.tuna_status_string(-99) == b"unknown status"
    assert tuna_lib.tuna_abi_version() == 1


def test_argument_validation_needs_no_gpu(tuna_lib):
    buf = ctypes.create_string_buffer(4096 + 64)
    base = (ctypes.addressof(buf) + 63) & ~63
    p = ctypes.c_void_p(base)
    odd = ctypes.c_void_p(base + 2)
    mm = tuna_lib.tuna_matmul
    assert mm(None, p, p, p, p, 64, 1, 64, None, 0, None) == -1
    assert mm(p, p, p, p, None, 64, 1, 64, None, 0, None) == -1
    assert mm(p, p, p, p, p, 60, 1, 64, None, 0, None) == -2      # m % 8
    assert mm(p, p, p, p, p, 64, 1, 60, None, 0, None) == -2      # k % 8
    assert mm(p, p, p, p, p, 64, 0, 64, None, 0, None) == -2      # n < 1
    assert mm(p, p, p, p, p, -8, 1, 64, None, 0, None) == -2
    assert mm(odd, p, p, p, p, 64, 1, 64, None, 0, None) == -3    # q misaligned
    assert mm(p, p, p, p, odd, 64, 1, 64, None, 0, None) == -3    # o misaligned
    dq = tuna_lib.tuna_dequant
    assert dq(None, p, p, p, 64, 64, None) == -1
    assert dq(p, p, p, p, 64, 4, None) == -2
    assert dq(p, p, p, odd, 64, 64, None) == -3
    assert tuna_lib.tuna_lookup_config(64, 1, 64, None) == -1
    assert tuna_lib.tuna_matmul_workspace_bytes(60, 1, 64) == 0


def test_workspace_is_always_required(tuna_lib):
    # both kernels are persistent and finish tiles cut across CTAs through the workspace
    need = tuna_lib.tuna_matmul_workspace_bytes(4096, 16, 14336)
    assert need > 0
    buf = ctypes.create_string_buffer(256)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)
    assert tuna_lib.tuna_matmul(p, p, p, p, p, 4096, 16, 14336, None, 0, None) == -4
    assert tuna_lib.tuna_matmul(p, p, p, p, p, 4096, 16, 14336, p, 16, None) == -4


def test_bad_explicit_config_is_rejected(tuna_lib):
    buf = ctypes.create_string_buffer(256)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)
    big = 1 << 30

    def call(**kw):
        cfg = _lib.TunaConfig(**kw)
        return tuna_lib.tuna_matmul_cfg(p, p, p, p, p, 512, 16, 512, p, big, None, ctypes.byref(cfg))

    assert call(path=_lib.PATH_STREAM, tile_tok=16, rows_per_warp=3, warps_m=4, warps_k=4) == -5
    assert call(path=_lib.PATH_STREAM, tile_tok=16, rows_per_warp=2, warps_m=8, warps_k=4) == -5   # 32 warps
    assert call(path=_lib.PATH_STREAM, tile_tok=16, rows_per_warp=1, warps_m=3, warps_k=4) == -5   # not a power of 2
    assert call(path=_lib.PATH_STREAM, tile_tok=24) == -5
    assert call(path=_lib.PATH_STREAM, tile_tok=32, rows_per_warp=2) == -5                         # accumulators
    assert call(path=_lib.PATH_UMMA, tile_tok=48) == -5
    assert call(path=_lib.PATH_UMMA, tile_tok=256, row_blocks=2) == -5                             # TMEM columns
    assert call(path=_lib.PATH_UMMA, tile_tok=16, dequant_warps=6) == -5
    assert call(path=7) == -5
