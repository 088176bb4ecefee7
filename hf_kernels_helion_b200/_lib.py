"""ctypes binding of libb200fp8.so (C ABI: include/b200fp8.h).

There is deliberately no fallback: if the shared library is missing or a call
returns a non-zero status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200fp8.so"

OUT_BF16, OUT_FP32 = 0, 1
VARIANT_AUTO, VARIANT_TILE128, VARIANT_TILE256, VARIANT_STREAMK, VARIANT_TILE256_SK = 0, 1, 2, 3, 4
VARIANT_PAIR256, VARIANT_PAIR256_SPLIT = 5, 6
VARIANT_NAMES = {"auto": 0, "tile128": 1, "tile256": 2, "streamk": 3, "tile256_sk": 4, "pair256": 5, "pair256_split": 6,
                 "pair256_split_sk": 7}

# name -> (restype, argtypes); mirrors include/b200fp8.h one to one
SIGNATURES = {
    "b200fp8_version": (c_int, []),
    "b200fp8_strerror": (c_char_p, [c_int]),
    "b200fp8_quant_act": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "b200fp8_quant_weight": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                     c_void_p]),
    "b200fp8_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                             c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p,
                             c_void_p]),
    "b200fp8_gemm_rowscale": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p,
                                      c_void_p]),
    "b200fp8_gemm_rowscale_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "b200fp8_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200fp8_linear_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int]),
    "b200fp8_gemm_multicast": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                       c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t,
                                       c_void_p, c_void_p]),
    "b200fp8_gemm_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64,
                                     c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t,
                                     c_void_p, c_void_p]),
    "b200fp8_peer_barrier": (c_int, [c_void_p, c_int, c_int, ctypes.c_uint32, c_void_p, c_void_p]),
    "b200fp8_peer_barrier_limited": (c_int, [c_void_p, c_int, c_int, ctypes.c_uint32, c_int64, c_void_p, c_void_p]),
    "b200fp8_ipc_export": (c_int, [c_void_p, c_void_p, c_void_p]),
    "b200fp8_ipc_open": (c_int, [c_void_p, c_void_p]),
    "b200fp8_ipc_close": (c_int, [c_void_p]),
    "b200fp8_gemm_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int]),
    "b200fp8_gemm_pick_variant": (c_int, [c_int64, c_int64, c_int64]),
    "b200fp8_gemm_pair_clusters": (c_int, []),
    "b200fp8_gemm_decode_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b200fp8_streamk_first_unit": (c_int64, [c_int64, c_int64, c_int64]),
    "b200fp8_streamk_owner": (c_int64, [c_int64, c_int64, c_int64]),
    "b200fp8_streamk_grid": (c_int64, [c_int64, c_int64, c_int64]),
}

_lib = None


def load():
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m hf_kernels_helion_b200.build` "
                "(there is no non-CUDA fallback)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def strerror(status: int) -> str:
    return load().b200fp8_strerror(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed: b200fp8 status {status} ({strerror(status)})")
