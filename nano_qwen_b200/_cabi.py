"""ctypes binding of ``libnq_fp8.so`` (declarations: ``include/nq_fp8.h``).

There is no fallback: if the library is missing or a call is rejected, an
exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_uint64, c_void_p, POINTER

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libnq_fp8.so")

NQ_OK = 0
ALGO_AUTO, ALGO_TOKEN_LANE, ALGO_WEIGHT_LANE = 0, 1, 2
ALGO_TOKEN_LANE_128, ALGO_TOKEN_LANE_192, ALGO_TOKEN_LANE_256 = 3, 4, 5
ALGO_TOKEN_PAIR = 6
ALGO_WEIGHT_LANE_FUSED = 8
FUSED_MAX_TOKENS, FUSED_AUTO_TOKENS = 32, 0      # NQ_FUSED_MAX_TOKENS, NQ_FUSED_AUTO_TOKENS

# name -> (restype, argtypes); every symbol include/nq_fp8.h declares
SIGNATURES = {
    "nq_version": (c_int, []),
    "nq_source_hash": (c_char_p, []),
    "nq_status_string": (c_char_p, [c_int]),
    "nq_last_cuda_error": (c_char_p, []),
    "nq_init": (c_int, []),
    "nq_act_quant_e4m3_g128": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "nq_weight_quant_e4m3_b128": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "nq_silu_mul_quant_e4m3_g128": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "nq_rmsnorm_quant_e4m3_g128": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_float, c_int, c_int64, c_int64, c_int64,
                                           c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                           c_void_p]),
    "nq_fp8_gemm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "nq_fp8_gemm_bs128": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                  c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                  c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "nq_fp8_linear": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                              c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                              c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_void_p]),
    "nq_fp8_linear_noalloc": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                      c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                      c_int, c_int, c_void_p]),
    "nq_p2p_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "nq_p2p_free": (c_int, [c_void_p]),
    "nq_p2p_export": (c_int, [c_void_p, c_void_p]),
    "nq_p2p_import": (c_int, [c_void_p, POINTER(c_void_p)]),
    "nq_p2p_release": (c_int, [c_void_p]),
    "nq_row_reduce_p2p": (c_int, [c_void_p, c_void_p, c_int64, POINTER(c_void_p), c_int, c_int,
                                  c_int64, c_void_p, c_void_p]),
    "nq_row_reduce_pull": (c_int, [POINTER(c_void_p), c_void_p, c_int64, POINTER(c_void_p), c_int, c_int, c_void_p,
                                   c_int, c_void_p]),
    "nq_device_status": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int), c_int]),
    "nq_set_wait_limit_ns": (c_int, [c_uint64]),
    "nq_set_sm_reserve": (c_int, [c_int]),
    "nq_launch_count": (c_int64, []),
}


class NqError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__(f"{what}: status {status} ({detail})")


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nano_qwen_b200.build` "
                "(this package has no non-CUDA fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != NQ_OK:
        handle = lib()
        detail = handle.nq_status_string(status).decode()
        if status == -4:
            detail += ": " + handle.nq_last_cuda_error().decode()
        raise NqError(status, what, detail)


def device_status(reset: bool = False) -> dict:
    """The device-side status block (call after synchronising)."""
    code, where, block, aux = c_int(), c_int(), c_int(), c_int()
    check(lib().nq_device_status(code, where, block, aux, int(reset)), "nq_device_status")
    return {"code": code.value, "where": where.value, "block": block.value, "aux": aux.value}
