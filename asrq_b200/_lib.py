"""ctypes binding of ``libasrq_b200.so`` (the C ABI in ``include/asrq_b200.h``).

There is no fallback: if the library has not been built, or a call is made without
a CUDA device, this raises.  Build with ``python -m asrq_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libasrq_b200.so")

F16, BF16 = 0, 1
WS_A16_GEMV, WS_A16_GEMM, WS_W4A4_GEMM, WS_LINEARQ = 1, 2, 3, 4
STATUS_BYTES = 256
ACT_NONE, ACT_GELU = 0, 1


class AsrqError(RuntimeError):
    """A C-ABI call returned a non-zero status (same role as TORCH_CHECK failures in the
    reference binding, asrq/matmulq/csrc/bindings.cpp:164-176)."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with status {code}: {text}")
        self.code = code


class DeviceInfo(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 128),
        ("cc_major", c_int), ("cc_minor", c_int), ("sm_count", c_int),
        ("max_smem_per_block_optin", c_int), ("l2_bytes", c_int),
        ("clock_khz", c_int), ("mem_clock_khz", c_int), ("mem_bus_bits", c_int),
        ("total_mem", c_size_t),
    ]


_A16_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
             c_int, c_int, c_void_p, c_size_t, c_void_p]

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "asrq_version": (c_int, []),
    "asrq_last_error_string": (c_char_p, []),
    "asrq_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int64]),
    "asrq_w4a16_gemv": (c_int, _A16_ARGS),
    "asrq_w2a16_gemv": (c_int, _A16_ARGS),
    "asrq_w4a16_gemv_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int, c_int, c_void_p]),
    "asrq_w4a16_gemm": (c_int, _A16_ARGS),
    "asrq_w2a16_gemm": (c_int, _A16_ARGS),
    "asrq_linearq_a16": (c_int, [c_int] + _A16_ARGS),
    "asrq_linearq_a16_fused": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                       c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "asrq_add_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_float, c_void_p, c_void_p, c_int64,
                                   c_int64, c_int, c_void_p]),
    "asrq_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_float, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                 c_void_p]),
    "asrq_silu_mul": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "asrq_qk_norm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                  c_int64, c_int64, c_int, c_int, c_int, c_int64, ctypes.c_float, c_int, c_void_p]),
    "asrq_decode_self_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, ctypes.c_float,
                                           c_int, c_void_p]),
    "asrq_dense_head": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "asrq_rtn_pack": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                              c_void_p]),
    "asrq_hadamard_fold": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p]),
    "asrq_hadamard_quant_int4": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "asrq_w4a4_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "asrq_w4a4_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                 c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "asrq_w4a4_prepare_weight": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "asrq_w4a4_prepare_weight_f8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "asrq_hadamard_quant_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "asrq_w4a4_gemm_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "asrq_hadamard_quant_f8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "asrq_w4a4_gemm_f8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "asrq_set_option": (c_int, [c_char_p, c_int]),
    "asrq_get_option": (c_int, [c_char_p, ctypes.POINTER(c_int)]),
    "asrq_check_status": (c_int, [c_void_p, c_void_p]),
    "asrq_device_info_query": (c_int, [c_int, ctypes.POINTER(DeviceInfo)]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once and sets the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m asrq_b200.build` (needs nvcc). "
            "asrq_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().asrq_last_error_string().decode()


def check(fn_name: str, code: int) -> None:
    if code != 0:
        raise AsrqError(fn_name, code, last_error())


CALLS = 0  # C-ABI calls made through call() in this process (benchmarks count a step's launches with it)


def call(fn_name: str, *args) -> None:
    global CALLS
    CALLS += 1
    check(fn_name, getattr(load(), fn_name)(*args))


def set_option(name: str, value: int) -> None:
    """Sets a tuning / test switch of the library (see asrq_set_option in the header)."""
    call("asrq_set_option", name.encode(), int(value))


def get_option(name: str) -> int:
    v = c_int(0)
    call("asrq_get_option", name.encode(), ctypes.byref(v))
    return v.value


def workspace_bytes(kind: int, m: int, n: int, k: int) -> int:
    return int(load().asrq_workspace_bytes(kind, m, n, k))


def device_info(device: int = 0) -> dict:
    info = DeviceInfo()
    check("asrq_device_info_query", load().asrq_device_info_query(device, ctypes.byref(info)))
    out = {f: getattr(info, f) for f, _ in DeviceInfo._fields_}
    out["name"] = info.name.decode()
    return out
