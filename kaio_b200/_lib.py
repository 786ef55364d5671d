"""ctypes loader for ``libkaio_b200.so`` -- the only route from Python to the kernels.

There is no fallback: when the shared library is missing, loading raises; when the machine has
no sm_100 GPU, every op returns an error code that ``ops`` turns into ``KaioError``.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libkaio_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "kaio_b200.h")

_lib = None

_VP, _SZ, _U32, _I32, _F32 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_int32, C.c_float

# Argument types of every exported function, in header order.
SIGNATURES = {
    "kaio_b200_matmul_int8": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _F32, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int8_scaled": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int8_acc": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_tc": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_tc_async": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_tc_f16out": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_dequantize_int4": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int4": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int4_noalloc": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int4_allgather": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _U32,
                                        _U32, _VP],
    "kaio_b200_matmul_int4_allgather_multicast": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _U32, _U32, _U32,
                                                  _U32, _U32, _U32, _VP],
    "kaio_b200_allgather_cols": [_VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _VP, _VP],
    "kaio_b200_matmul_int4_f16out": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _VP],
    "kaio_b200_qkv_project_int8": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _F32, _F32, _F32,
                                   _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_qkv_project_int8_colscale": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _VP, _VP, _SZ,
                                            _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_qkv_project_w8a8": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _VP, _VP, _SZ,
                                   _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_qkv_project_int4": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ,
                                   _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _VP],
    "kaio_b200_attention_tc": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _I32, _VP],
    "kaio_b200_attention_mha_f16": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _U32,
                                    _U32, _I32, _VP],
    "kaio_b200_quantize_rows_int8": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _VP],
    "kaio_b200_quantize_pack_int4": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int4_peer_partials": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _I32, _U32, _U32,
                                            _U32, _U32, _VP],
    "kaio_b200_sum_partials_f32": [_VP, _SZ, _U32, _U32, _U32, _VP, _U32, _SZ, _U32, _U32, _VP],
    "kaio_b200_sum_partials_f32_multicast": [_VP, _SZ, _U32, _U32, _U32, _VP, _SZ, _U32, _U32, _VP],
    "kaio_b200_allreduce_multimem_f32": [_VP, _VP, _SZ, _U32, _U32, _U32, _U32, _VP],
    "kaio_b200_matmul_int4_silu_gate": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32,
                                        _VP],
    "kaio_b200_silu_gate_f32": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _VP],
    "kaio_b200_silu_gate_f16": [_VP, _SZ, _VP, _SZ, _VP, _SZ, _U32, _U32, _U32, _U32, _U32, _VP],
    "kaio_b200_device_status": [_VP, C.POINTER(_U32)],
    "kaio_b200_selftest_bounded_wait": [_U32, _VP],
    "kaio_b200_probe_int8_mma_rate": [_U32, C.POINTER(C.c_uint64), _VP],
}


def declared_symbols() -> list[str]:
    """Every function name ``include/kaio_b200.h`` declares."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(kaio_b200_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m kaio_b200.build` "
            "(there is no CPU or PyTorch fallback for these ops)")
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _I32
    lib.kaio_b200_last_error.restype = C.c_char_p
    lib.kaio_b200_last_error.argtypes = []
    lib.kaio_b200_last_variant.restype = C.c_char_p
    lib.kaio_b200_last_variant.argtypes = []
    lib.kaio_b200_shutdown.restype = None
    lib.kaio_b200_shutdown.argtypes = []
    lib.kaio_b200_version.restype = _I32
    lib.kaio_b200_version.argtypes = []
    _lib = lib
    return lib
