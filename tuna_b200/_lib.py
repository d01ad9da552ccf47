"""ctypes binding of libtuna_b200.so (the C ABI in include/tuna_b200.h)."""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int32, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libtuna_b200.so"


class TunaConfig(ctypes.Structure):
    """Mirror of `struct tuna_config`."""

    _fields_ = [
        ("path", c_int32),
        ("tile_tok", c_int32),
        ("rows_per_warp", c_int32),
        ("warps_m", c_int32),
        ("warps_k", c_int32),
        ("k_steps", c_int32),
        ("ctas", c_int32),
        ("stages_w", c_int32),
        ("stages_x", c_int32),
        ("dequant_warps", c_int32),
        ("row_blocks", c_int32),
        ("stages_a", c_int32),
        ("k_accs", c_int32),
        ("reserved", c_int32 * 3),
    ]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_ if n != "reserved"}


class TunaGemmDesc(ctypes.Structure):
    """Mirror of `struct tuna_gemm_desc` (one GEMM of tuna_matmul_sequence)."""

    _fields_ = [("q", c_void_p), ("x", c_void_p), ("absmax", c_void_p), ("o", c_void_p),
                ("m", c_int32), ("n", c_int32), ("k", c_int32), ("flags", c_int32)]


PATH_AUTO, PATH_STREAM, PATH_UMMA, PATH_TSTREAM = 0, 1, 2, 3

# every symbol include/tuna_b200.h declares: name -> (restype, argtypes)
MAX_PEERS = 8
GEMM_PARTIAL = 1
IPC_HANDLE_BYTES = 64


class TunaExchange(ctypes.Structure):
    """`tuna_exchange` of include/tuna_b200.h: the exchange buffers of all ranks, in rank order."""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("buffer", c_void_p * MAX_PEERS), ("bytes", c_size_t)]


SYMBOLS = {
    "tuna_matmul": (c_int, [c_void_p] * 5 + [c_int] * 3 + [c_void_p, c_size_t, c_void_p]),
    "tuna_matmul_cfg": (c_int, [c_void_p] * 5 + [c_int] * 3 + [c_void_p, c_size_t, c_void_p, ctypes.POINTER(TunaConfig)]),
    "tuna_matmul_workspace_bytes": (c_size_t, [c_int] * 3),
    "tuna_matmul_batched": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_size_t] * 4 + [c_void_p, c_size_t, c_void_p]),
    "tuna_matmul_batched_workspace_bytes": (c_size_t, [c_int] * 4),
    "tuna_matmul_noalloc": (c_int, [c_void_p] * 5 + [c_int] * 3 + [c_void_p]),
    "tuna_matmul_sequence": (c_int, [ctypes.POINTER(TunaGemmDesc), c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tuna_matmul_sequence_workspace_bytes": (c_size_t, [ctypes.POINTER(TunaGemmDesc), c_int]),
    "tuna_matmul_sequence_reduce": (c_int, [ctypes.POINTER(TunaGemmDesc), c_int, c_void_p, c_void_p, c_size_t,
                                            ctypes.POINTER(TunaExchange), c_void_p]),
    "tuna_exchange_bytes": (c_size_t, [ctypes.POINTER(TunaGemmDesc), c_int, c_int]),
    "tuna_exchange_create": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "tuna_exchange_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "tuna_exchange_close": (c_int, [c_void_p]),
    "tuna_exchange_destroy": (c_int, [c_void_p]),
    "tuna_lookup_config": (c_int, [c_int] * 3 + [ctypes.POINTER(TunaConfig)]),
    "tuna_dequant": (c_int, [c_void_p] * 4 + [c_int] * 2 + [c_void_p]),
    "tuna_quantize": (c_int, [c_void_p] * 4 + [c_int] * 2 + [c_void_p]),
    "tuna_check_device_status": (c_int, [c_void_p]),
    "tuna_selftest_bounded_wait": (c_int, [c_void_p]),
    "tuna_status_string": (c_char_p, [c_int]),
    "tuna_abi_version": (c_int, []),
    "tuna_config_table_size": (c_int, []),
    "tuna_last_wrapper_status": (c_int, []),
    # the reference's own native symbols (C++ linkage, extension.cpp:22-24), Itanium-mangled
    "_Z7wrapperPvS_S_S_S_iiiP11CUstream_st": (None, [c_void_p] * 5 + [c_int] * 3 + [c_void_p]),
    "_Z18dequantize_wrapperPvS_S_S_iiP11CUstream_st": (None, [c_void_p] * 4 + [c_int] * 2 + [c_void_p]),
}

_lib = None


def load():
    """Load the shared library, failing loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m tuna_b200.build` "
                "(there is no fallback implementation)"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class TunaError(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        super().__init__(f"tuna_b200: {load().tuna_status_string(status).decode()} (status {status})")


def check(status: int) -> None:
    if status != 0:
        raise TunaError(status)
